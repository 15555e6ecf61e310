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

inline size_t fwd_wigner_t_smem(int N, int nl) {
  const int LW = (nl + 3) / 4 * 4 + 4;
  return (size_t)N * LW * sizeof(float) + (size_t)N * (kWigZT + 2) * sizeof(float2);
}

// X[l][z] = sum_beta W[l][beta] V[z][beta]   (+ Hermitian mirror row)
S2C_KERNEL(so3_fwd_wigner_t, FwdWignerParams) {
  const int N = p.N;
  const int pair = ctx.bid / p.nzt, zt = ctx.bid - pair * p.nzt;
  int m, n;
  so3_pair_decode(pair, p.K, m, n);
  const int am = m < 0 ? -m : m;
  const int lmin = am > n ? am : n;
  const int L = p.nl - lmin;
  if (L <= 0) return;
  const int z0 = zt * kWigZT;
  const int zc = (p.nbatch - z0) < kWigZT ? (p.nbatch - z0) : kWigZT;
  const int LW = (p.nl + 3) / 4 * 4 + 4, ZP = kWigZT + 2;
  float* Ws = reinterpret_cast<float*>(smem);                  // [N][LW]   (transposed panel)
  float2* Vs = reinterpret_cast<float2*>(Ws + (size_t)N * LW);  // [N][ZP]   (transposed tile)
  const int LT = (L + 3) / 4, Z2 = (zc + 1) / 2;
  const float* panel = p.pan.data + p.pan.off[pair];
  // panel and batch tile, transposed into [beta][.]; 16-byte loads, four in flight per thread
  {
    const float4* src = reinterpret_cast<const float4*>(panel);   // panel offsets are multiples of N
    const int n4 = N / 4, total = LT * 4 * n4;
    for (int base = ctx.tid; base < total; base += 4 * ctx.nthr) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < total && idx / n4 < L) v[u] = src[idx];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        if (idx < total) {
          const int l = idx / n4, bt = 4 * (idx - l * n4);
          Ws[(bt + 0) * LW + l] = v[u].x;
          Ws[(bt + 1) * LW + l] = v[u].y;
          Ws[(bt + 2) * LW + l] = v[u].z;
          Ws[(bt + 3) * LW + l] = v[u].w;
        }
      }
    }
  }
  const int nm = 2 * p.K - 1, mi = m + p.K - 1;
  {
    const float4* src = reinterpret_cast<const float4*>(p.v + (((long)n * nm + mi) * p.nbatch + z0) * N);
    const int n2 = N / 2, total = Z2 * 2 * n2;
    for (int base = ctx.tid; base < total; base += 4 * ctx.nthr) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < total && idx / n2 < zc) v[u] = src[idx];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * ctx.nthr;
        if (idx < total) {
          const int zz = idx / n2, bt = 2 * (idx - zz * n2);
          Vs[bt * ZP + zz] = make_float2(v[u].x, v[u].y);
          Vs[(bt + 1) * ZP + zz] = make_float2(v[u].z, v[u].w);
        }
      }
    }
  }
  ctx.sync();
  const float fudge = ((m - n) & 1) ? -1.f : 1.f;
  const bool self = (m == 0 && n == 0);
  if (LT * Z2 < ctx.nthr) {
    // few degrees for this pair: 4 x 1 tiles so that more threads share the beta loop
    for (int tile = ctx.tid; tile < LT * zc; tile += ctx.nthr) {
      const int tl = tile / zc, zz = tile - tl * zc;
      float ar[4] = {0.f, 0.f, 0.f, 0.f}, ai[4] = {0.f, 0.f, 0.f, 0.f};
      const float* wp = Ws + 4 * tl;
      const float2* vp = Vs + zz;
      for (int bt = 0; bt < N; ++bt) {
        const float4 w4 = *reinterpret_cast<const float4*>(wp + bt * LW);
        const float2 v2 = vp[bt * ZP];
        ar[0] = fmaf(w4.x, v2.x, ar[0]); ai[0] = fmaf(w4.x, v2.y, ai[0]);
        ar[1] = fmaf(w4.y, v2.x, ar[1]); ai[1] = fmaf(w4.y, v2.y, ai[1]);
        ar[2] = fmaf(w4.z, v2.x, ar[2]); ai[2] = fmaf(w4.z, v2.y, ai[2]);
        ar[3] = fmaf(w4.w, v2.x, ar[3]); ai[3] = fmaf(w4.w, v2.y, ai[3]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int li = 4 * tl + i;
        if (li >= L) continue;
        const int l = lmin + li;
        float2* o1 = p.out + so3_row(l, m, n) * p.out_zstride + z0 + zz;
        float2* o2 = p.out + so3_row(l, -m, -n) * p.out_zstride + z0 + zz;
        const float re = ar[i], im = ai[i];
        if (p.mode == kSo3Real) {
          *o1 = make_float2(re, im);
          if (!self) *o2 = make_float2(fudge * re, -fudge * im);
        } else {
          float2 c = *o1;
          *o1 = make_float2(c.x - im, c.y + re);
          if (!self) {
            c = *o2;
            *o2 = make_float2(c.x + fudge * im, c.y + fudge * re);
          }
        }
      }
    }
    return;
  }
  for (int tile = ctx.tid; tile < LT * Z2; tile += ctx.nthr) {
    const int tl = tile / Z2, tz = tile - tl * Z2;
    float ar[4][2], ai[4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) { ar[i][0] = ar[i][1] = ai[i][0] = ai[i][1] = 0.f; }
    const float* wp = Ws + 4 * tl;
    const float2* vp = Vs + 2 * tz;
    for (int bt = 0; bt < N; ++bt) {
      const float4 w4 = *reinterpret_cast<const float4*>(wp + bt * LW);
      const float4 v4 = *reinterpret_cast<const float4*>(vp + bt * ZP);  // (re0, im0, re1, im1)
      const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ar[i][0] = fmaf(w[i], v4.x, ar[i][0]);
        ai[i][0] = fmaf(w[i], v4.y, ai[i][0]);
        ar[i][1] = fmaf(w[i], v4.z, ar[i][1]);
        ai[i][1] = fmaf(w[i], v4.w, ai[i][1]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int li = 4 * tl + i;
      if (li >= L) continue;
      const int l = lmin + li;
      float2* o1 = p.out + so3_row(l, m, n) * p.out_zstride + z0;
      float2* o2 = p.out + so3_row(l, -m, -n) * p.out_zstride + z0;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int zz = 2 * tz + j;
        if (zz >= zc) continue;
        const float re = ar[i][j], im = ai[i][j];
        if (p.mode == kSo3Real) {
          o1[zz] = make_float2(re, im);
          if (!self) o2[zz] = make_float2(fudge * re, -fudge * im);
        } else {  // += i * (re + i im); mirror += i * fudge * conj
          float2 c = o1[zz];
          o1[zz] = make_float2(c.x - im, c.y + re);
          if (!self) {
            c = o2[zz];
            o2[zz] = make_float2(c.x + fudge * im, c.y + fudge * re);
          }
        }
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
