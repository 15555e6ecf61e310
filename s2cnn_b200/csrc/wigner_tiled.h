// Register-tiled Wigner-d contractions for the general (large bandwidth) SO(3) path.
//
// Same inputs, outputs and arithmetic as so3_fwd_wigner / so3_inv_wigner (so3_kernels.h), i.e. the
// beta / l contraction of the reference's so3fft.cu / so3ifft.cu tile loops
// (s2cnn/soft/so3_fft.py:296-336 and :391-431), but organised as a small GEMM per frequency pair:
// a block stages the whole Wigner panel and a tile of up to 64 batch elements in shared memory and
// every thread owns 4 x 2 complex outputs, so that one pair of 16-byte shared-memory loads feeds
// 16 fused multiply-adds.
#pragma once

#include "backend.h"
#include "so3_kernels.h"

namespace s2c {

constexpr int kWigZT = 64;  // batch elements per block tile (even)
constexpr int kWigHalves = 1;  // pieces of the beta range in the forward contraction

inline size_t fwd_wigner_t_smem(int N, int nl) {
  return (size_t)((nl + 3) / 4 * 4) * (N / kWigHalves + 4) * sizeof(float) +
         (size_t)kWigZT * (N / kWigHalves + 2) * sizeof(float2);
}

// X[l][z] = sum_beta W[l][beta] V[z][beta]   (+ Hermitian mirror row)
//
// The beta range can be processed in kWigHalves pieces with the accumulators kept in registers
// (less shared memory per block, more blocks per SM); one piece is the faster setting.  Panel rows
// and batch rows are staged exactly as they lie in memory (16-byte copies, no transposition): the
// beta loop runs four samples at a time, a thread reads W[l][beta..beta+3] for its four degrees
// (the whole warp shares the address: broadcast) and V[z][beta..beta+3] for its two batch elements
// z = tz and tz + ceil(zc/2) (row stride N + 2 complex numbers, so the 8 lanes of a 16-byte access phase
// hit 8 different bank groups).
S2C_KERNEL(so3_fwd_wigner_t, FwdWignerParams) {
  const int N = p.N, NH = N / kWigHalves;
  const int pair = ctx.bid / p.nzt, zt = ctx.bid - pair * p.nzt;
  int m, n;
  so3_pair_decode(pair, p.K, m, n);
  const int am = m < 0 ? -m : m;
  const int lmin = am > n ? am : n;
  const int L = p.nl - lmin;
  if (L <= 0) return;
  const int z0 = zt * kWigZT;
  const int zc = (p.nbatch - z0) < kWigZT ? (p.nbatch - z0) : kWigZT;
  const int LDW = NH + 4, LDV = NH + 2, ZH = (zc + 1) / 2;   // a thread's batch elements: tz, tz + ZH
  float* Ws = reinterpret_cast<float*>(smem);                                        // [nl up to 4][LDW]
  float2* Vs = reinterpret_cast<float2*>(Ws + (size_t)((p.nl + 3) / 4 * 4) * LDW);    // [kWigZT][LDV]
  const int LT = (L + 3) / 4;
  const float* panel = p.pan.data + p.pan.off[pair];
  const int nm = 2 * p.K - 1, mi = m + p.K - 1;
  const float2* vsrc = p.v + (((long)n * nm + mi) * p.nbatch + z0) * N;
  // 4 x 2 tiles (degrees x batch elements), or 4 x 1 when the pair has few degrees so that more
  // threads share the beta loop; at most two tiles per thread either way (LT <= 16, 256 threads)
  const bool narrow = LT * ZH < ctx.nthr;
  const int ntiles = narrow ? LT * zc : LT * ZH;
  float ar[2][4][2], ai[2][4][2];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) { ar[t][i][0] = ar[t][i][1] = ai[t][i][0] = ai[t][i][1] = 0.f; }

  for (int half = 0; half < kWigHalves; ++half) {
    if (half) ctx.sync();
    {
      const int n4 = NH / 4, total = LT * 4 * n4;                    // rows past L are zero
      for (int base = ctx.tid; base < total; base += 4 * ctx.nthr) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * ctx.nthr;
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (idx < total && idx / n4 < L) {
            const int l = idx / n4, c4 = idx - l * n4;
            v[u] = *reinterpret_cast<const float4*>(panel + (long)l * N + half * NH + 4 * c4);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * ctx.nthr;
          if (idx < total) {
            const int l = idx / n4, c4 = idx - l * n4;
            *reinterpret_cast<float4*>(Ws + l * LDW + 4 * c4) = v[u];
          }
        }
      }
    }
    {
      const int n2 = NH / 2, total = 2 * ZH * n2;                     // a row past zc is zero
      for (int base = ctx.tid; base < total; base += 4 * ctx.nthr) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * ctx.nthr;
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (idx < total && idx / n2 < zc) {
            const int zz = idx / n2, c2 = idx - zz * n2;
            v[u] = *reinterpret_cast<const float4*>(vsrc + (long)zz * N + half * NH + 2 * c2);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * ctx.nthr;
          if (idx < total) {
            const int zz = idx / n2, c2 = idx - zz * n2;
            *reinterpret_cast<float4*>(Vs + zz * LDV + 2 * c2) = v[u];
          }
        }
      }
    }
    ctx.sync();
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int tile = ctx.tid + t * ctx.nthr;
      if (tile >= ntiles) continue;
      if (narrow) {
        const int tl = tile / zc, zz = tile - tl * zc;
        const float* wp = Ws + 4 * tl * LDW;
        const float2* vp = Vs + zz * LDV;
        for (int bt = 0; bt < NH; bt += 4) {
          const float4 va = *reinterpret_cast<const float4*>(vp + bt);
          const float4 vb = *reinterpret_cast<const float4*>(vp + bt + 2);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 w4 = *reinterpret_cast<const float4*>(wp + i * LDW + bt);
            ar[t][i][0] = fmaf(w4.x, va.x, ar[t][i][0]); ai[t][i][0] = fmaf(w4.x, va.y, ai[t][i][0]);
            ar[t][i][0] = fmaf(w4.y, va.z, ar[t][i][0]); ai[t][i][0] = fmaf(w4.y, va.w, ai[t][i][0]);
            ar[t][i][0] = fmaf(w4.z, vb.x, ar[t][i][0]); ai[t][i][0] = fmaf(w4.z, vb.y, ai[t][i][0]);
            ar[t][i][0] = fmaf(w4.w, vb.z, ar[t][i][0]); ai[t][i][0] = fmaf(w4.w, vb.w, ai[t][i][0]);
          }
        }
      } else {
        const int tl = tile / ZH, tz = tile - tl * ZH;
        const float* wp = Ws + 4 * tl * LDW;
        const float2* v0 = Vs + tz * LDV;
        const float2* v1 = Vs + (tz + ZH) * LDV;
        for (int bt = 0; bt < NH; bt += 4) {
          float4 w4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) w4[i] = *reinterpret_cast<const float4*>(wp + i * LDW + bt);
          const float4 a0 = *reinterpret_cast<const float4*>(v0 + bt);       // beta, beta+1 of z = tz
          const float4 b0 = *reinterpret_cast<const float4*>(v0 + bt + 2);   // beta+2, beta+3
          const float4 a1 = *reinterpret_cast<const float4*>(v1 + bt);       // z = tz + ZH
          const float4 b1 = *reinterpret_cast<const float4*>(v1 + bt + 2);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ar[t][i][0] = fmaf(w4[i].x, a0.x, ar[t][i][0]); ai[t][i][0] = fmaf(w4[i].x, a0.y, ai[t][i][0]);
            ar[t][i][0] = fmaf(w4[i].y, a0.z, ar[t][i][0]); ai[t][i][0] = fmaf(w4[i].y, a0.w, ai[t][i][0]);
            ar[t][i][0] = fmaf(w4[i].z, b0.x, ar[t][i][0]); ai[t][i][0] = fmaf(w4[i].z, b0.y, ai[t][i][0]);
            ar[t][i][0] = fmaf(w4[i].w, b0.z, ar[t][i][0]); ai[t][i][0] = fmaf(w4[i].w, b0.w, ai[t][i][0]);
            ar[t][i][1] = fmaf(w4[i].x, a1.x, ar[t][i][1]); ai[t][i][1] = fmaf(w4[i].x, a1.y, ai[t][i][1]);
            ar[t][i][1] = fmaf(w4[i].y, a1.z, ar[t][i][1]); ai[t][i][1] = fmaf(w4[i].y, a1.w, ai[t][i][1]);
            ar[t][i][1] = fmaf(w4[i].z, b1.x, ar[t][i][1]); ai[t][i][1] = fmaf(w4[i].z, b1.y, ai[t][i][1]);
            ar[t][i][1] = fmaf(w4[i].w, b1.z, ar[t][i][1]); ai[t][i][1] = fmaf(w4[i].w, b1.w, ai[t][i][1]);
          }
        }
      }
    }
  }

  const float fudge = ((m - n) & 1) ? -1.f : 1.f;
  const bool self = (m == 0 && n == 0);
  auto emit = [&](int li, int zz, float re, float im) {
    if (li >= L || zz >= zc) return;
    const int l = lmin + li;
    float2* o1 = p.out + so3_row(l, m, n) * p.out_zstride + z0 + zz;
    float2* o2 = p.out + so3_row(l, -m, -n) * p.out_zstride + z0 + zz;
    if (p.mode == kSo3Real) {
      *o1 = make_float2(re, im);
      if (!self) *o2 = make_float2(fudge * re, -fudge * im);
    } else {  // += i * (re + i im); mirror += i * fudge * conj
      float2 c = *o1;
      *o1 = make_float2(c.x - im, c.y + re);
      if (!self) {
        c = *o2;
        *o2 = make_float2(c.x + fudge * im, c.y + fudge * re);
      }
    }
  };
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int tile = ctx.tid + t * ctx.nthr;
    if (tile >= ntiles) continue;
    if (narrow) {
      const int tl = tile / zc, zz = tile - tl * zc;
#pragma unroll
      for (int i = 0; i < 4; ++i) emit(4 * tl + i, zz, ar[t][i][0], ai[t][i][0]);
    } else {
      const int tl = tile / ZH, tz = tile - tl * ZH;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        emit(4 * tl + i, tz, ar[t][i][0], ai[t][i][0]);
        emit(4 * tl + i, tz + ZH, ar[t][i][1], ai[t][i][1]);
      }
    }
  }
}

inline size_t inv_wigner_t_smem(int N, int K) {
  return (size_t)K * N * sizeof(float) + (size_t)K * (kWigZT + 2) * sizeof(float2);
}

// S[z][beta] = sum_l W[l][beta] Xs[l][z],  Xs = symmetrised spectrum
S2C_KERNEL(so3_inv_wigner_t, InvWignerParams) {
  const int N = p.N;
  const int pair = ctx.bid / p.nzt, zt = ctx.bid - pair * p.nzt;
  int m, n;
  so3_pair_decode(pair, p.K, m, n);
  const int am = m < 0 ? -m : m;
  const int lmin = am > n ? am : n;
  const int L = p.pan.nl - lmin;
  if (L <= 0) return;
  const int z0 = zt * kWigZT;
  const int zc = (p.nbatch - z0) < kWigZT ? (p.nbatch - z0) : kWigZT;
  const int ZP = kWigZT + 2;
  float* Ws = reinterpret_cast<float*>(smem);                            // [L][N]
  float2* Xs = reinterpret_cast<float2*>(Ws + (size_t)p.pan.nl * N);      // [L][ZP]
  const int Z2 = (zc + 1) / 2;
  const float* panel = p.pan.data + p.pan.off[pair];
  {
    const float4* src = reinterpret_cast<const float4*>(panel);
    float4* dst4 = reinterpret_cast<float4*>(Ws);
    const int total = L * N / 4;
    for (int base = ctx.tid; base < total; base += 4 * ctx.nthr) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (base + u * ctx.nthr < total) v[u] = src[base + u * ctx.nthr];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (base + u * ctx.nthr < total) dst4[base + u * ctx.nthr] = v[u];
    }
  }
  const float fudge = ((m - n) & 1) ? -1.f : 1.f;
  for (int it = ctx.tid; it < L * Z2 * 2; it += ctx.nthr) {
    const int li = it / (Z2 * 2), zz = it - li * (Z2 * 2);
    float2 v = make_float2(0.f, 0.f);
    if (zz < zc) {
      const int l = lmin + li;
      float2 a = p.x[so3_row(l, m, n) * p.x_zstride + z0 + zz];
      float2 b = p.x[so3_row(l, -m, -n) * p.x_zstride + z0 + zz];
      if (p.mode == kSo3RotI) {  // multiply the spectrum by -i
        a = make_float2(a.y, -a.x);
        b = make_float2(b.y, -b.x);
      }
      v = make_float2(0.5f * (a.x + fudge * b.x), 0.5f * (a.y - fudge * b.y));
    }
    Xs[li * ZP + zz] = v;
  }
  ctx.sync();
  const int nm = 2 * p.K - 1, mi = m + p.K - 1;
  float2* dst = p.s + (((long)n * nm + mi) * p.nbatch + z0) * N;
  const int B4 = N / 4;
  for (int tile = ctx.tid; tile < B4 * Z2; tile += ctx.nthr) {
    const int tz = tile / B4, tb = tile - tz * B4;  // consecutive threads -> consecutive beta
    float ar[2][4], ai[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) { ar[j][i] = 0.f; ai[j][i] = 0.f; }
    const float* wp = Ws + 4 * tb;
    const float2* xp = Xs + 2 * tz;
    for (int li = 0; li < L; ++li) {
      const float4 w4 = *reinterpret_cast<const float4*>(wp + li * N);
      const float4 x4 = *reinterpret_cast<const float4*>(xp + li * ZP);  // (re0, im0, re1, im1)
      const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ar[0][i] = fmaf(w[i], x4.x, ar[0][i]);
        ai[0][i] = fmaf(w[i], x4.y, ai[0][i]);
        ar[1][i] = fmaf(w[i], x4.z, ar[1][i]);
        ai[1][i] = fmaf(w[i], x4.w, ai[1][i]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int zz = 2 * tz + j;
      if (zz >= zc) continue;
      float4* o = reinterpret_cast<float4*>(dst + (long)zz * N + 4 * tb);
      o[0] = make_float4(ar[j][0], ai[j][0], ar[j][1], ai[j][1]);
      o[1] = make_float4(ar[j][2], ai[j][2], ar[j][3], ai[j][3]);
    }
  }
}

}  // namespace s2c
