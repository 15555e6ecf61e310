// Small dense kernels on the path:
//   * kernel-grid -> spectrum transform  y[s, f, c] = sum_a x[f, a] F[a, s, c]  and its transpose
//     (the torch.einsum("ia,afc->fic") of s2cnn/s2_ft.py:22 and s2cnn/so3_ft.py:22 and its autograd)
//   * Haar integration over SO(3) and its transpose (s2cnn/soft/so3_integrate.py:7-29)
#pragma once

#include "backend.h"

namespace s2c {

// ---- rft forward: out[s][f][2] = sum_a x[f][a] * F[a][s][2] -----------------------------------
struct RftFwdParams {
  const float* x;    // [nf][ng]
  const float2* F;   // [ng][ns]
  float2* out;       // [ns][nf]
  int nf, ng, ns;
  int tiles_f;
};
constexpr int kRftTF = 32, kRftTS = 32, kRftTA = 32;

S2C_KERNEL(rft_forward, RftFwdParams) {
  // block: 32 f x 32 s outputs, 256 threads, each thread 1 f x 4 s
  float* xs = reinterpret_cast<float*>(smem);                                  // [TF][TA+1]
  float2* fs = reinterpret_cast<float2*>(smem + kRftTF * (kRftTA + 1) * 4);    // [TA][TS]
  const int tf = ctx.bid % p.tiles_f, ts = ctx.bid / p.tiles_f;
  const int f0 = tf * kRftTF, s0 = ts * kRftTS;
  const int fi = ctx.tid & 31, sg = ctx.tid >> 5;  // sg in 0..7, s = sg + 8*q
  float2 acc[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) acc[q] = make_float2(0.f, 0.f);
  for (int a0 = 0; a0 < p.ng; a0 += kRftTA) {
    for (int e = ctx.tid; e < kRftTF * kRftTA; e += ctx.nthr) {
      const int f = e / kRftTA, a = e - f * kRftTA;
      xs[f * (kRftTA + 1) + a] =
          (f0 + f < p.nf && a0 + a < p.ng) ? p.x[(long)(f0 + f) * p.ng + a0 + a] : 0.f;
    }
    for (int e = ctx.tid; e < kRftTA * kRftTS; e += ctx.nthr) {
      const int a = e / kRftTS, s = e - a * kRftTS;
      fs[e] = (a0 + a < p.ng && s0 + s < p.ns) ? p.F[(long)(a0 + a) * p.ns + s0 + s]
                                               : make_float2(0.f, 0.f);
    }
    ctx.sync();
#pragma unroll 8
    for (int a = 0; a < kRftTA; ++a) {
      const float xv = xs[fi * (kRftTA + 1) + a];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fv = fs[a * kRftTS + sg + 8 * q];
        acc[q].x = fmaf(xv, fv.x, acc[q].x);
        acc[q].y = fmaf(xv, fv.y, acc[q].y);
      }
    }
    ctx.sync();
  }
  if (f0 + fi < p.nf) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int s = s0 + sg + 8 * q;
      if (s < p.ns) p.out[(long)s * p.nf + f0 + fi] = acc[q];
    }
  }
}

// ---- rft backward: gx[f][a] = sum_s  g[s][f] . F[a][s]   (real dot of complex pairs) ---------
struct RftBwdParams {
  const float2* g;   // [ns][nf]
  const float2* F;   // [ng][ns]
  float* gx;         // [nf][ng]
  int nf, ng, ns;
  int tiles_f;
};

S2C_KERNEL(rft_backward, RftBwdParams) {
  // block: 32 f x 32 a outputs, 256 threads, each thread 1 f x 4 a
  float2* gs = reinterpret_cast<float2*>(smem);                       // [TS][TF]
  float2* fs = gs + kRftTS * kRftTF;                                  // [TA][TS+1]
  const int tf = ctx.bid % p.tiles_f, ta = ctx.bid / p.tiles_f;
  const int f0 = tf * kRftTF, a0 = ta * kRftTA;
  const int fi = ctx.tid & 31, ag = ctx.tid >> 5;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s0 = 0; s0 < p.ns; s0 += kRftTS) {
    for (int e = ctx.tid; e < kRftTS * kRftTF; e += ctx.nthr) {
      const int s = e / kRftTF, f = e - s * kRftTF;
      gs[e] = (s0 + s < p.ns && f0 + f < p.nf) ? p.g[(long)(s0 + s) * p.nf + f0 + f]
                                               : make_float2(0.f, 0.f);
    }
    for (int e = ctx.tid; e < kRftTA * kRftTS; e += ctx.nthr) {
      const int a = e / kRftTS, s = e - a * kRftTS;
      fs[a * (kRftTS + 1) + s] = (a0 + a < p.ng && s0 + s < p.ns)
                                     ? p.F[(long)(a0 + a) * p.ns + s0 + s]
                                     : make_float2(0.f, 0.f);
    }
    ctx.sync();
#pragma unroll 8
    for (int s = 0; s < kRftTS; ++s) {
      const float2 gv = gs[s * kRftTF + fi];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fv = fs[(ag + 8 * q) * (kRftTS + 1) + s];
        acc[q] = fmaf(gv.x, fv.x, acc[q]);
        acc[q] = fmaf(gv.y, fv.y, acc[q]);
      }
    }
    ctx.sync();
  }
  if (f0 + fi < p.nf) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int a = a0 + ag + 8 * q;
      if (a < p.ng) p.gx[(long)(f0 + fi) * p.ng + a] = acc[q];
    }
  }
}

// ---- so3_integrate ----------------------------------------------------------------------------
struct IntegrateParams {
  const float* x;    // [n][2b][2b*2b]
  const float* w;    // [2b]
  float* out;        // [n]
  long n;
  int N;             // 2b
  int relu;          // apply max(x, 0) before summing (fused activation, optional)
};

constexpr int kIntegrateWarps = 8;  // signals per block (one warp each)

S2C_KERNEL(so3_integrate_fwd, IntegrateParams) {
  // one warp per signal: 16-byte loads (a group of 4 samples never straddles a beta plane because
  // (2b)^2 is a multiple of 4), lane partials through shared memory, fixed summation order
  float* red = reinterpret_cast<float*>(smem);  // [kIntegrateWarps][32]
  const int warp = ctx.tid >> 5, lane = ctx.tid & 31;
  const long z = (long)ctx.bid * kIntegrateWarps + warp;
  const int plane4 = p.N * p.N / 4;
  const int total4 = p.N * plane4;
  float acc = 0.f;
  if (z < p.n) {
    const float4* src = reinterpret_cast<const float4*>(p.x + z * (long)total4 * 4);
    for (int e = lane; e < total4; e += 32) {
      float4 v = src[e];
      if (p.relu) {
        v.x = v.x > 0.f ? v.x : 0.f;
        v.y = v.y > 0.f ? v.y : 0.f;
        v.z = v.z > 0.f ? v.z : 0.f;
        v.w = v.w > 0.f ? v.w : 0.f;
      }
      acc = fmaf(p.w[e / plane4], (v.x + v.y) + (v.z + v.w), acc);
    }
  }
  red[ctx.tid] = acc;
  ctx.sync();
  if (lane == 0 && z < p.n) {
    float s = 0.f;
    for (int i = 0; i < 32; ++i) s += red[warp * 32 + i];
    p.out[z] = s;
  }
}

struct IntegrateBwdParams {
  const float* g;    // [n]
  const float* w;    // [2b]
  const float* x;    // forward input (only read when relu)
  float* gx;         // [n][2b][2b*2b]
  long total;        // n * (2b)^3
  int N;
  int relu;
};

S2C_KERNEL(so3_integrate_bwd, IntegrateBwdParams) {
  const int plane = p.N * p.N;
  const long per = (long)p.N * plane;
  for (long e = (long)ctx.bid * ctx.nthr + ctx.tid; e < p.total; e += (long)ctx.nblk * ctx.nthr) {
    const long z = e / per;
    const int beta = (int)((e - z * per) / plane);
    float v = p.g[z] * p.w[beta];
    if (p.relu && !(p.x[e] > 0.f)) v = 0.f;
    p.gx[e] = v;
  }
}

}  // namespace s2c
