// SO(3) and S2 generalised FFT kernels (general path: any bandwidth, three passes per
// direction with two scratch arrays in global memory, processed in batch chunks).
//
// Replaces the reference's NVRTC kernels so3fft.cu / so3ifft.cu (s2cnn/soft/so3_fft.py:246-443)
// and s2fft.cu / s2ifft.cu (s2cnn/soft/s2_fft.py:151-223) together with the torch.fft calls
// around them.  Notation: N = 2b samples per angle; K = number of kept frequencies
// (|m|, n < K); z = flattened batch index.
//
//   analysis :  x[z][beta][alpha][gamma]
//     fwd_gamma   real rows -> FFT over gamma (two rows per complex transform)
//                 -> U[z][n][beta][alpha]           (n = 0..K-1, the Hermitian half)
//     fwd_alpha   rows of U -> FFT over alpha -> V[n][m][z][beta]   (|m| < K)
//     fwd_wigner  per (m, n):  X[l][z] = sum_beta W[l][beta] V[z][beta], plus the mirrored row
//                 X[l,-m,-n] = (-1)^(m-n) conj X[l,m,n]  (real input)
//   synthesis:  the same three passes in reverse (inv_wigner, inv_alpha, inv_gamma).  The
//     spectrum is first symmetrised, Xs = (X[l,m,n] + (-1)^(m-n) conj X[l,-m,-n]) / 2, which makes
//     the real-output transform equal to the real part of the full complex transform for ANY
//     spectrum - the behaviour of the reference's CPU branch (so3_fft.py:184-199).
//
// The S2 transforms are the n = 0 special case of the same kernels (mode flags).
#pragma once

#include "backend.h"
#include "fft_device.h"
#include "fft_twostep.h"
#include "tables.h"

namespace s2c {

constexpr int kThreads = 256;

S2C_HD size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Shared-memory prologue common to the FFT kernels: twiddles and digit map.
struct FftSmem {
  float2* tw;
  unsigned short* pos;
  float2* data;
  float2* tmp;   // second buffer of the two-step FFT (lengths 64 / 128 / 256), else unused
};
S2C_HD size_t fft_smem_head_bytes(int n) { return align_up((size_t)n * (sizeof(float2) + 2), 16); }
S2C_D FftSmem fft_smem_carve(unsigned char* smem, int n, int rows) {
  FftSmem s;
  s.tw = reinterpret_cast<float2*>(smem);
  s.pos = reinterpret_cast<unsigned short*>(smem + (size_t)n * sizeof(float2));
  s.data = reinterpret_cast<float2*>(smem + fft_smem_head_bytes(n));
  s.tmp = s.data + (size_t)rows * (n + 1);
  return s;
}
inline size_t fft_smem_bytes(int n, int rows) {
  size_t b = fft_smem_head_bytes(n) + (size_t)rows * (n + 1) * sizeof(float2);
  if (fft_twostep_supported(n)) b += (size_t)rows * fft_twostep_ld2(n) * sizeof(float2);
  return b;
}
// Twiddles and the frequency -> position map.  The two-step FFT leaves its output in natural
// order, so its map is the identity.
S2C_D void fft_smem_load_tables(const Ctx& ctx, const FftSmem& s, const FftDev& f) {
  const bool natural = fft_twostep_supported(f.desc.n);
  for (int i = ctx.tid; i < f.desc.n; i += ctx.nthr) {
    s.tw[i] = f.tw[i];
    s.pos[i] = natural ? (unsigned short)i : f.pos[i];
  }
}
// In-place FFT of `cnt` rows (stride ld) held in s.data; ends with a block barrier.
template <int DIR>
S2C_D void fft_rows(const Ctx& ctx, const FftSmem& s, const FftDesc& d, int cnt, int ld) {
  if (fft_twostep_supported(d.n)) fft_twostep<DIR>(ctx, s.data, s.tmp, d.n, cnt, ld, s.tw);
  else fft_dif_inplace<DIR>(ctx, s.data, d, cnt, ld, 1, false, s.tw);
}

// ---------------------------------------------------------------------------------------------
// analysis, pass 1: FFT over gamma of real rows
// ---------------------------------------------------------------------------------------------
struct FwdGammaParams {
  const float* x;     // real signal, element e at x[e * in_stride + in_off]
  long in_stride, in_off;
  float2* u;          // [z][n < K][beta][alpha]
  int N, b, K, G;
  long npairs;        // nbatch * N * b row pairs; pair id = (z * N + beta) * b + p
  FftDev fft;
};

// G divides b: all row pairs of a block belong to one (z, beta) plane.
S2C_KERNEL(so3_fwd_gamma, FwdGammaParams) {
  const int N = p.N, ld = N + 1;
  FftSmem s = fft_smem_carve(smem, N, p.G);
  fft_smem_load_tables(ctx, s, p.fft);
  const int warp = ctx.tid >> 5, lane = ctx.tid & 31, nwarps = ctx.nthr >> 5;
  const long pair0 = (long)ctx.bid * p.G;
  const int cnt = (int)((p.npairs - pair0) < p.G ? (p.npairs - pair0) : p.G);
  if (p.in_stride == 1 && N % 4 == 0) {
    // the block's 2 * cnt rows are one contiguous run: 16-byte loads, four in flight per thread
    const float4* src = reinterpret_cast<const float4*>(p.x + pair0 * 2 * N);
    const int n4 = N / 4, total4 = cnt * 2 * n4;
    float* sdata = reinterpret_cast<float*>(s.data);
    for (int base = ctx.tid; base < total4; base += 4 * ctx.nthr) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        if (idx < total4) v[u] = src[idx];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        if (idx < total4) {
          const int row = idx / n4, c4 = idx - row * n4;     // row = 2 g + part
          float* d = sdata + ((row >> 1) * ld + 4 * c4) * 2 + (row & 1);
          d[0] = v[u].x;
          d[2] = v[u].y;
          d[4] = v[u].z;
          d[6] = v[u].w;
        }
      }
    }
  } else {
    for (int g = warp; g < cnt; g += nwarps) {
      const long e0 = (pair0 + g) * 2 * N;  // rows 2p and 2p+1 are adjacent in memory
      for (int gam = lane; gam < N; gam += 32) {
        const float a = p.x[(e0 + gam) * p.in_stride + p.in_off];
        const float b = p.x[(e0 + N + gam) * p.in_stride + p.in_off];
        s.data[g * ld + gam] = make_float2(a, b);
      }
    }
  }
  ctx.sync();
  fft_rows<-1>(ctx, s, p.fft.desc, cnt, ld);
  // separate the two real rows packed in one complex transform; keep n < K
  const long zb = pair0 / p.b;
  const int pp0 = (int)(pair0 - zb * p.b);
  const int beta = (int)(zb % N);
  const long z = zb / N;
  float2* ubase = p.u + ((z * p.K) * N + beta) * (long)N + 2 * pp0;
  for (int n = warp; n < p.K; n += nwarps) {
    const int pk = s.pos[n], pc = s.pos[n == 0 ? 0 : N - n];
    float2* dst = ubase + (long)n * N * N;
    for (int g = lane; g < cnt; g += 32) {
      const float2 zk = s.data[g * ld + pk];
      const float2 zc = s.data[g * ld + pc];
      float4 o;
      o.x = 0.5f * (zk.x + zc.x);
      o.y = 0.5f * (zk.y - zc.y);
      o.z = 0.5f * (zk.y + zc.y);
      o.w = -0.5f * (zk.x - zc.x);
      *reinterpret_cast<float4*>(dst + 2 * g) = o;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// analysis, pass 2: FFT over alpha of complex rows, keep |m| < K, transposed store
// ---------------------------------------------------------------------------------------------
struct FwdAlphaParams {
  const float* in;   // rows of N complex (or N real when in_real)
  int in_real;
  float2* v;         // [n < Kn][mi < 2K-1][z][beta]
  int nbatch, N, K, Kn, G;
  long nrows;        // nbatch * Kn * N; row id = (z * Kn + n) * N + beta
  FftDev fft;
};

// G divides N: all rows of a block share (z, n) and cover consecutive betas.
S2C_KERNEL(so3_fwd_alpha, FwdAlphaParams) {
  const int N = p.N, ld = N + 1;
  FftSmem s = fft_smem_carve(smem, N, p.G);
  fft_smem_load_tables(ctx, s, p.fft);
  const int warp = ctx.tid >> 5, lane = ctx.tid & 31, nwarps = ctx.nthr >> 5;
  const long row0 = (long)ctx.bid * p.G;
  const int cnt = (int)((p.nrows - row0) < p.G ? (p.nrows - row0) : p.G);
  if (p.in_real) {
    for (int g = warp; g < cnt; g += nwarps)
      for (int a = lane; a < N; a += 32)
        s.data[g * ld + a] = make_float2(p.in[(row0 + g) * N + a], 0.f);
  } else {
    // contiguous run of cnt rows: 16-byte loads (two complex numbers), four in flight per thread
    const float4* src = reinterpret_cast<const float4*>(p.in + (row0 * N) * 2);
    const int n2 = N / 2, total = cnt * n2;  // N is even
    for (int base = ctx.tid; base < total; base += 4 * ctx.nthr) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        if (idx < total) v[u] = src[idx];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        if (idx < total) {
          const int g = idx / n2, a2 = idx - g * n2;
          s.data[g * ld + 2 * a2] = make_float2(v[u].x, v[u].y);
          s.data[g * ld + 2 * a2 + 1] = make_float2(v[u].z, v[u].w);
        }
      }
    }
  }
  ctx.sync();
  fft_rows<-1>(ctx, s, p.fft.desc, cnt, ld);
  const int nm = 2 * p.K - 1;
  const long zn = row0 / N;
  const int beta0 = (int)(row0 - zn * N);
  const int n = (int)(zn % p.Kn);
  const long z = zn / p.Kn;
  float2* vbase = p.v + (((long)n * nm) * p.nbatch + z) * N + beta0;
  for (int mi = warp; mi < nm; mi += nwarps) {
    const int m = mi - (p.K - 1);
    const int pm = s.pos[m < 0 ? m + N : m];
    float2* dst = vbase + (long)mi * p.nbatch * N;
    for (int g = lane; g < cnt; g += 32) dst[g] = s.data[g * ld + pm];
  }
}

// ---------------------------------------------------------------------------------------------
// analysis, pass 3: Wigner-d contraction over beta
// ---------------------------------------------------------------------------------------------
enum WignerMode : int {
  kSo3Real = 0,      // write X and its Hermitian mirror
  kSo3AccumI = 1,    // X += i * result (imaginary part of a complex input), mirror likewise
  kS2 = 2,           // S2 transform: rows l^2 + l + m, no mirror
  kSo3RotI = 3,      // synthesis only: spectrum multiplied by -i first (imaginary output part)
  kS2Product = 4,    // fused synthesis only: spectrum = s2_mm(xs, ys) computed on the fly
};

struct FwdWignerParams {
  const float2* v;   // [n][mi][z][beta]
  float2* out;       // spectrum rows of `out_zstride` complex, already offset to the chunk's z0
  long out_zstride;
  PanelsDev pan;
  int nbatch, N, K, nl, ZT, nzt, mode;
};

S2C_KERNEL(so3_fwd_wigner, FwdWignerParams) {
  const int N = p.N, ldw = N + 1, ldv = N + 1;
  const int pair = ctx.bid / p.nzt, zt = ctx.bid - pair * p.nzt;
  int m, n;
  if (p.mode == kS2) { m = pair - (p.K - 1); n = 0; } else so3_pair_decode(pair, p.K, m, n);
  const int am = m < 0 ? -m : m;
  const int lmin = am > n ? am : n;
  const int L = p.nl - lmin;
  if (L <= 0) return;
  const int z0 = zt * p.ZT;
  const int zc = (p.nbatch - z0) < p.ZT ? (p.nbatch - z0) : p.ZT;
  float* Ws = reinterpret_cast<float*>(smem);
  float2* Vs = reinterpret_cast<float2*>(smem + align_up((size_t)p.nl * ldw * sizeof(float), 16));
  const float* panel = p.pan.data + p.pan.off[pair];
  for (int it = ctx.tid; it < L * N; it += ctx.nthr) {
    const int l = it / N, bt = it - l * N;
    Ws[l * ldw + bt] = panel[it];
  }
  const int nm = 2 * p.K - 1, mi = m + p.K - 1;
  const float2* vsrc = p.v + (((long)n * nm + mi) * p.nbatch + z0) * N;
  for (int it = ctx.tid; it < zc * N; it += ctx.nthr) {
    const int zz = it / N, bt = it - zz * N;
    Vs[zz * ldv + bt] = vsrc[it];
  }
  ctx.sync();
  const float fudge = ((m - n) & 1) ? -1.f : 1.f;
  for (int it = ctx.tid; it < L * zc; it += ctx.nthr) {
    const int li = it / zc, zz = it - li * zc;
    const float* w = Ws + li * ldw;
    const float2* vv = Vs + zz * ldv;
    float ar = 0.f, ai = 0.f;
    for (int bt = 0; bt < N; ++bt) {
      const float wv = w[bt];
      const float2 x = vv[bt];
      ar = fmaf(wv, x.x, ar);
      ai = fmaf(wv, x.y, ai);
    }
    const int l = lmin + li;
    if (p.mode == kS2) {
      p.out[((long)l * l + l + m) * p.out_zstride + z0 + zz] = make_float2(ar, ai);
    } else {
      float2* o1 = p.out + so3_row(l, m, n) * p.out_zstride + z0 + zz;
      float2* o2 = p.out + so3_row(l, -m, -n) * p.out_zstride + z0 + zz;
      const bool self = (m == 0 && n == 0);
      if (p.mode == kSo3Real) {
        *o1 = make_float2(ar, ai);
        if (!self) *o2 = make_float2(fudge * ar, -fudge * ai);
      } else {  // += i * (ar + i ai); mirror += i * fudge * conj
        float2 c = *o1;
        *o1 = make_float2(c.x - ai, c.y + ar);
        if (!self) {
          c = *o2;
          *o2 = make_float2(c.x + fudge * ai, c.y + fudge * ar);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// synthesis, pass 1: Wigner-d contraction over l
// ---------------------------------------------------------------------------------------------
struct InvWignerParams {
  const float2* x;   // spectrum rows of x_zstride complex, offset to the chunk's z0
  long x_zstride;
  float2* s;         // [n][mi][z][beta]
  PanelsDev pan;
  int nbatch, N, K, ZT, nzt, mode;
};

S2C_KERNEL(so3_inv_wigner, InvWignerParams) {
  const int N = p.N;
  const int pair = ctx.bid / p.nzt, zt = ctx.bid - pair * p.nzt;
  int m, n;
  if (p.mode == kS2) { m = pair - (p.K - 1); n = 0; } else so3_pair_decode(pair, p.K, m, n);
  const int am = m < 0 ? -m : m;
  const int lmin = am > n ? am : n;
  const int L = p.pan.nl - lmin;
  if (L <= 0) return;
  const int z0 = zt * p.ZT;
  const int zc = (p.nbatch - z0) < p.ZT ? (p.nbatch - z0) : p.ZT;
  float* Ws = reinterpret_cast<float*>(smem);
  float2* Xs = reinterpret_cast<float2*>(smem + align_up((size_t)p.pan.nl * N * sizeof(float), 16));
  const float* panel = p.pan.data + p.pan.off[pair];
  for (int it = ctx.tid; it < L * N; it += ctx.nthr) Ws[it] = panel[it];
  const float fudge = ((m - n) & 1) ? -1.f : 1.f;
  for (int it = ctx.tid; it < L * zc; it += ctx.nthr) {
    const int li = it / zc, zz = it - li * zc;
    const int l = lmin + li;
    float2 v;
    if (p.mode == kS2) {
      v = p.x[((long)l * l + l + m) * p.x_zstride + z0 + zz];
    } else {
      float2 a = p.x[so3_row(l, m, n) * p.x_zstride + z0 + zz];
      float2 b = p.x[so3_row(l, -m, -n) * p.x_zstride + z0 + zz];
      if (p.mode == kSo3RotI) {  // multiply the spectrum by -i
        a = make_float2(a.y, -a.x);
        b = make_float2(b.y, -b.x);
      }
      v = make_float2(0.5f * (a.x + fudge * b.x), 0.5f * (a.y - fudge * b.y));
    }
    Xs[li * p.ZT + zz] = v;
  }
  ctx.sync();
  const int nm = 2 * p.K - 1, mi = m + p.K - 1;
  float2* dst = p.s + (((long)n * nm + mi) * p.nbatch + z0) * N;
  for (int it = ctx.tid; it < zc * N; it += ctx.nthr) {
    const int zz = it / N, bt = it - zz * N;
    float ar = 0.f, ai = 0.f;
    for (int li = 0; li < L; ++li) {
      const float wv = Ws[li * N + bt];
      const float2 x = Xs[li * p.ZT + zz];
      ar = fmaf(wv, x.x, ar);
      ai = fmaf(wv, x.y, ai);
    }
    dst[it] = make_float2(ar, ai);
  }
}

// ---------------------------------------------------------------------------------------------
// synthesis, pass 2: inverse FFT over m -> alpha
// ---------------------------------------------------------------------------------------------
struct InvAlphaParams {
  const float2* s;   // [n < Kn][mi][z][beta]
  float* out;        // rows of N complex (or N real when out_real); row id = (z * Kn + n) * N + beta
  int out_real;
  int herm_n0;       // SO(3): for n = 0 only m >= 0 is stored; m < 0 is the conjugate
  int nbatch, N, K, Kn, G;
  long nrows;
  FftDev fft;
};

// G divides N: all rows of a block share (z, n) and cover consecutive betas.
S2C_KERNEL(so3_inv_alpha, InvAlphaParams) {
  const int N = p.N, ld = N + 1;
  FftSmem s = fft_smem_carve(smem, N, p.G);
  fft_smem_load_tables(ctx, s, p.fft);
  const int warp = ctx.tid >> 5, lane = ctx.tid & 31, nwarps = ctx.nthr >> 5;
  const long row0 = (long)ctx.bid * p.G;
  const int cnt = (int)((p.nrows - row0) < p.G ? (p.nrows - row0) : p.G);
  for (int it = ctx.tid; it < cnt * ld; it += ctx.nthr) s.data[it] = make_float2(0.f, 0.f);
  ctx.sync();
  const int nm = 2 * p.K - 1;
  const long zn = row0 / N;
  const int beta0 = (int)(row0 - zn * N);
  const int n = (int)(zn % p.Kn);
  const long z = zn / p.Kn;
  const bool herm = p.herm_n0 && n == 0;  // only m >= 0 is stored; m < 0 is the conjugate
  const float2* sbase = p.s + (((long)n * nm) * p.nbatch + z) * N + beta0;
  for (int mi0 = warp; mi0 < nm; mi0 += 4 * nwarps) {   // four independent loads per lane in flight
    for (int g = lane; g < cnt; g += 32) {
      float2 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int mi = mi0 + u * nwarps;
        const int m = mi - (p.K - 1);
        if (mi < nm && !(herm && m < 0)) v[u] = sbase[(long)mi * p.nbatch * N + g];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int mi = mi0 + u * nwarps;
        const int m = mi - (p.K - 1);
        if (mi < nm && !(herm && m < 0)) {
          s.data[g * ld + (m < 0 ? m + N : m)] = v[u];
          if (herm && m > 0) s.data[g * ld + N - m] = make_float2(v[u].x, -v[u].y);
        }
      }
    }
  }
  ctx.sync();
  fft_rows<+1>(ctx, s, p.fft.desc, cnt, ld);
  if (p.out_real) {
    for (int g = warp; g < cnt; g += nwarps)
      for (int a = lane; a < N; a += 32) p.out[(row0 + g) * N + a] = s.data[g * ld + s.pos[a]].x;
  } else {
    float2* out2 = reinterpret_cast<float2*>(p.out);
    for (int g = warp; g < cnt; g += nwarps)
      for (int a = lane; a < N; a += 32) out2[(row0 + g) * N + a] = s.data[g * ld + s.pos[a]];
  }
}

// ---------------------------------------------------------------------------------------------
// synthesis, pass 3: Hermitian inverse FFT over n -> gamma, two real rows per transform
// ---------------------------------------------------------------------------------------------
struct InvGammaParams {
  const float2* t;   // [z][n < K][beta][alpha]
  float* out;        // real signal, element e at out[e * out_stride + out_off]
  long out_stride, out_off;
  const float* bias; // optional [nfeat]; feature of row z is (z0 + z) % nfeat
  int nfeat;
  long z0;
  int N, b, K, G;
  long npairs;
  FftDev fft;
};

// G divides b: all row pairs of a block belong to one (z, beta) plane.
S2C_KERNEL(so3_inv_gamma, InvGammaParams) {
  const int N = p.N, ld = N + 1;
  FftSmem s = fft_smem_carve(smem, N, p.G);
  fft_smem_load_tables(ctx, s, p.fft);
  const int warp = ctx.tid >> 5, lane = ctx.tid & 31, nwarps = ctx.nthr >> 5;
  const long pair0 = (long)ctx.bid * p.G;
  const int cnt = (int)((p.npairs - pair0) < p.G ? (p.npairs - pair0) : p.G);
  for (int it = ctx.tid; it < cnt * ld; it += ctx.nthr) s.data[it] = make_float2(0.f, 0.f);
  ctx.sync();
  const long zb = pair0 / p.b;
  const int pp0 = (int)(pair0 - zb * p.b);
  const int beta = (int)(zb % N);
  const long z = zb / N;
  const float2* tbase = p.t + ((z * p.K) * N + beta) * (long)N + 2 * pp0;
  for (int n0 = warp; n0 < p.K; n0 += 4 * nwarps) {   // four independent loads per lane in flight
    for (int g = lane; g < cnt; g += 32) {
      float4 tv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int n = n0 + u * nwarps;
        if (n < p.K) tv[u] = *reinterpret_cast<const float4*>(tbase + (long)n * N * N + 2 * g);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int n = n0 + u * nwarps;
        if (n >= p.K) continue;
        const float4 t4 = tv[u];
        if (n == 0) {
          // T[alpha][0] is real for a Hermitian spectrum; its rounding-level imaginary part is dropped
          s.data[g * ld] = make_float2(t4.x, t4.z);
        } else {
          s.data[g * ld + n] = make_float2(t4.x - t4.w, t4.y + t4.z);       // T1 + i T2
          s.data[g * ld + N - n] = make_float2(t4.x + t4.w, t4.z - t4.y);   // conj(T1) + i conj(T2)
        }
      }
    }
  }
  ctx.sync();
  fft_rows<+1>(ctx, s, p.fft.desc, cnt, ld);
  float add = 0.f;
  if (p.bias) add = p.bias[(p.z0 + z) % p.nfeat];
  for (int g = warp; g < cnt; g += nwarps) {
    const long e0 = (pair0 + g) * 2 * N;
    for (int gam = lane; gam < N; gam += 32) {
      const float2 v = s.data[g * ld + s.pos[gam]];
      p.out[(e0 + gam) * p.out_stride + p.out_off] = v.x + add;
      p.out[(e0 + N + gam) * p.out_stride + p.out_off] = v.y + add;
    }
  }
}

}  // namespace s2c
