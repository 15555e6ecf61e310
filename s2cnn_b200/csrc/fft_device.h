// Shared-memory mixed-radix FFT used by every alpha/gamma transform on the path (replaces the
// torch.fft / cuFFT calls at s2cnn/soft/so3_fft.py:37,90,153,197 and s2cnn/soft/s2_fft.py:39,104).
//
// In-place decimation in frequency (Gentleman-Sande): natural-order input, digit-reversed
// output.  Consumers read frequency k at position pos[k] (host_math.h: fft_positions), so no
// reordering pass and no second buffer is needed.  Transforms are unnormalised in both
// directions, as on the reference path (its inverse multiplies torch's 1/n back).
//
// A batch of `count` transforms lives in shared memory; element i of transform t is at
// data[t * tstride + i * estride].  Work items are (transform, butterfly) pairs spread over the
// threads of the block; `t_fast` chooses which of the two varies fastest across threads
// (rows: butterfly fastest; columns: transform fastest) to keep bank conflicts low.
#pragma once

#include "backend.h"
#include "host_math.h"

namespace s2c {

S2C_D float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
S2C_D float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
S2C_D float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
S2C_D float2 cmul_conj(float2 a, float2 b) {  // a * conj(b)
  return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
// a * w^(DIR): DIR = +1 multiplies by w, DIR = -1 by conj(w)  (tw[k] = exp(+2 pi i k / n))
template <int DIR>
S2C_D float2 ctw(float2 a, float2 w) {
  return DIR > 0 ? cmul(a, w) : cmul_conj(a, w);
}
// multiply by (DIR * i)
template <int DIR>
S2C_D float2 cmul_i(float2 a) {
  return DIR > 0 ? make_float2(-a.y, a.x) : make_float2(a.y, -a.x);
}

template <int DIR, int R>
S2C_D void fft_butterfly(float2* v, const float2* tw, int n) {
  if (R == 2) {
    float2 a = v[0], b = v[1];
    v[0] = cadd(a, b);
    v[1] = csub(a, b);
  } else if (R == 4) {
    float2 t0 = cadd(v[0], v[2]), t1 = csub(v[0], v[2]);
    float2 t2 = cadd(v[1], v[3]), t3 = cmul_i<DIR>(csub(v[1], v[3]));
    v[0] = cadd(t0, t2);
    v[2] = csub(t0, t2);
    v[1] = cadd(t1, t3);
    v[3] = csub(t1, t3);
  } else {
    float2 u[R];
    const int step = n / R;
#pragma unroll
    for (int p = 0; p < R; ++p) {
      float2 acc = v[0];
#pragma unroll
      for (int k = 1; k < R; ++k) {
        const float2 w = tw[((p * k) % R) * step];
        const float2 t = ctw<DIR>(v[k], w);
        acc.x += t.x;
        acc.y += t.y;
      }
      u[p] = acc;
    }
#pragma unroll
    for (int p = 0; p < R; ++p) v[p] = u[p];
  }
}

template <int DIR, int R>
S2C_D void fft_stage(const Ctx& ctx, float2* data, int n, int len, int count, int tstride,
                     int estride, bool t_fast, const float2* tw) {
  const int m = len / R;          // butterfly span
  const int per = n / R;          // butterflies per transform
  const int twstep = n / len;
  const int items = count * per;
  for (int it = ctx.tid; it < items; it += ctx.nthr) {
    int t, q;
    if (t_fast) { q = it / count; t = it - q * count; }
    else        { t = it / per;   q = it - t * per; }
    const int blk = q / m, j = q - blk * m;
    float2* base = data + (size_t)t * tstride + (size_t)(blk * len + j) * estride;
    float2 v[R];
#pragma unroll
    for (int k = 0; k < R; ++k) v[k] = base[(size_t)k * m * estride];
    fft_butterfly<DIR, R>(v, tw, n);
    base[0] = v[0];
#pragma unroll
    for (int p = 1; p < R; ++p) {
      const float2 w = tw[j * p * twstep];
      base[(size_t)p * m * estride] = (m > 1) ? ctw<DIR>(v[p], w) : v[p];
    }
  }
}

// Generic radix (any prime up to kMaxRadix) - same arithmetic with run-time loop bounds.
template <int DIR>
S2C_D void fft_stage_generic(const Ctx& ctx, float2* data, int n, int len, int R, int count,
                             int tstride, int estride, bool t_fast, const float2* tw) {
  const int m = len / R, per = n / R, twstep = n / len, step = n / R;
  const int items = count * per;
  for (int it = ctx.tid; it < items; it += ctx.nthr) {
    int t, q;
    if (t_fast) { q = it / count; t = it - q * count; }
    else        { t = it / per;   q = it - t * per; }
    const int blk = q / m, j = q - blk * m;
    float2* base = data + (size_t)t * tstride + (size_t)(blk * len + j) * estride;
    float2 v[kMaxRadix], u[kMaxRadix];
    for (int k = 0; k < R; ++k) v[k] = base[(size_t)k * m * estride];
    for (int p = 0; p < R; ++p) {
      float2 acc = v[0];
      for (int k = 1; k < R; ++k) {
        const float2 t2 = ctw<DIR>(v[k], tw[((p * k) % R) * step]);
        acc.x += t2.x;
        acc.y += t2.y;
      }
      u[p] = acc;
    }
    base[0] = u[0];
    for (int p = 1; p < R; ++p)
      base[(size_t)p * m * estride] = ctw<DIR>(u[p], tw[j * p * twstep]);
  }
}

// All stages; every stage ends with a block barrier (so the result is visible on return).
template <int DIR>
S2C_D void fft_dif_inplace(const Ctx& ctx, float2* data, const FftDesc& d, int count,
                           int tstride, int estride, bool t_fast, const float2* tw) {
  int len = d.n;
  for (int s = 0; s < d.nstage; ++s) {
    const int r = d.radix[s];
    switch (r) {
      case 2: fft_stage<DIR, 2>(ctx, data, d.n, len, count, tstride, estride, t_fast, tw); break;
      case 3: fft_stage<DIR, 3>(ctx, data, d.n, len, count, tstride, estride, t_fast, tw); break;
      case 4: fft_stage<DIR, 4>(ctx, data, d.n, len, count, tstride, estride, t_fast, tw); break;
      case 5: fft_stage<DIR, 5>(ctx, data, d.n, len, count, tstride, estride, t_fast, tw); break;
      default:
        fft_stage_generic<DIR>(ctx, data, d.n, len, r, count, tstride, estride, t_fast, tw);
    }
    ctx.sync();
    len /= r;
  }
}

}  // namespace s2c
