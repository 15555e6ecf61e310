// Gradients of s2_mm for layers with few input features (f_in <= kThinFi = 8; the first layer of
// the reference's models has 1 to 6):
//   gx[l,m,i,k] = sum_{n,j} gz[l,m,n,i,j] y[l,n,k,j]            (s2cnn/s2_mm.py:38-46, kernel :222-262)
//   gy[l,n,k,j] = sum_{m,i} conj(gz[l,m,n,i,j]) x[l,m,i,k]      (s2cnn/s2_mm.py:48-58, kernel :265-312)
// With f_in that small both are reductions over the large tensor gz with a handful of outputs per
// row or column - matrix-vector shaped, so the 64 x 64 tiles of cgemm_grouped would sit almost
// empty.  Here gz is streamed exactly once; the small operand is broadcast from shared memory
// (grad x) or read at a warp-uniform address (grad y).
#pragma once

#include "backend.h"
#include "host_math.h"

namespace s2c {

constexpr int kThinFi = 8;           // largest f_in these kernels take
constexpr int kThinRows = 64;        // batch rows per block of the grad-x kernel
constexpr int kThinSlices = 4;       // slices of the n range per block of the grad-x kernel

struct S2ThinParams {
  const float2* gz;     // [nspec3(nl)][nb][fo]
  const float2* other;  // grad x: y [nl^2][fi][fo];  grad y: x [nl^2][nb][fi]
  float2* out;          // grad x: gx [nl^2][nb][fi]; grad y: gy [nl^2][fi][fo]
  int nl, nb, fi, fo;
};

S2C_D int thin_isqrt(int v) {   // floor(sqrt(v)) for the small row indices used here
  int r = (int)sqrtf((float)v);
  while (r * r > v) --r;
  while ((r + 1) * (r + 1) <= v) ++r;
  return r;
}

inline size_t s2_gradx_thin_smem(int nl, int fi, int fo) {
  const size_t ys = (size_t)(2 * nl - 1) * fi * fo * sizeof(float2);
  const size_t red = (size_t)kThinSlices * kThinRows * kThinFi * sizeof(float2);
  return ys + red;
}

// block = (l, m, tile of kThinRows batch rows); thread = (row, slice of n)
S2C_KERNEL(s2_mm_gradx_thin, S2ThinParams) {
  const int tiles_i = (p.nb + kThinRows - 1) / kThinRows;
  // largest degrees first: a block's work grows with 2l + 1, and the blocks that start last should
  // be the short ones
  const int rbid = ctx.nblk - 1 - ctx.bid;
  const int lm = rbid / tiles_i, itile = rbid - lm * tiles_i;
  const int l = thin_isqrt(lm), m = lm - l * l;
  const int L = 2 * l + 1;
  float2* ys = reinterpret_cast<float2*>(smem);                     // [L][fi][fo]
  float2* red = ys + (size_t)(2 * p.nl - 1) * p.fi * p.fo;          // [slices][rows][kThinFi]
  {
    const float2* ysrc = p.other + (size_t)l * l * p.fi * p.fo;     // rows l^2 .. l^2 + L - 1
    for (int e = ctx.tid; e < L * p.fi * p.fo; e += ctx.nthr) ys[e] = ysrc[e];
  }
  ctx.sync();
  const int r = ctx.tid % kThinRows, slice = ctx.tid / kThinRows;
  const int i = itile * kThinRows + r;
  float2 acc[kThinFi];
#pragma unroll
  for (int k = 0; k < kThinFi; ++k) acc[k] = make_float2(0.f, 0.f);
  if (i < p.nb) {
    const long row0 = (long)so3_offset(l) + (long)m * L;
    for (int n = slice; n < L; n += kThinSlices) {
      const float2* g = p.gz + ((row0 + n) * p.nb + i) * p.fo;
      const float2* yn = ys + (size_t)n * p.fi * p.fo;
      for (int j = 0; j < p.fo; ++j) {
        const float2 gv = g[j];
#pragma unroll
        for (int k = 0; k < kThinFi; ++k) {
          if (k < p.fi) {
            const float2 yv = yn[k * p.fo + j];
            acc[k].x = fmaf(gv.x, yv.x, acc[k].x);
            acc[k].x = fmaf(-gv.y, yv.y, acc[k].x);
            acc[k].y = fmaf(gv.x, yv.y, acc[k].y);
            acc[k].y = fmaf(gv.y, yv.x, acc[k].y);
          }
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kThinFi; ++k) red[(slice * kThinRows + r) * kThinFi + k] = acc[k];
  ctx.sync();
  if (slice == 0 && i < p.nb) {
    float2* dst = p.out + ((long)(l * l + m) * p.nb + i) * p.fi;
#pragma unroll
    for (int k = 0; k < kThinFi; ++k) {
      if (k < p.fi) {
        float2 s = red[r * kThinFi + k];
        for (int sl = 1; sl < kThinSlices; ++sl) {
          const float2 t = red[(sl * kThinRows + r) * kThinFi + k];
          s.x += t.x;
          s.y += t.y;
        }
        dst[k] = s;
      }
    }
  }
}

inline int s2_grady_thin_threads(int fo) {
  int t = (1024 / fo) * fo;          // whole slices of fo threads
  return t < fo ? fo : t;
}
inline size_t s2_grady_thin_smem(int fo) {
  return (size_t)s2_grady_thin_threads(fo) * kThinFi * sizeof(float2);
}

// block = (l, n); thread = (slice of the batch rows, j); all of (m, i) is summed inside the block
S2C_KERNEL_BOUNDS(s2_mm_grady_thin, S2ThinParams, 1024, 1) {
  const int rbid = ctx.nblk - 1 - ctx.bid;     // largest degrees (the long blocks) first
  const int l = thin_isqrt(rbid), n = rbid - l * l;
  const int L = 2 * l + 1;
  const int nsl = ctx.nthr / p.fo;
  const int j = ctx.tid % p.fo, sl = ctx.tid / p.fo;
  float2* red = reinterpret_cast<float2*>(smem);   // [nthr][kThinFi]
  float2 acc[kThinFi];
#pragma unroll
  for (int k = 0; k < kThinFi; ++k) acc[k] = make_float2(0.f, 0.f);
  if (sl < nsl) {
    for (int m = 0; m < L; ++m) {
      const float2* g = p.gz + (((long)so3_offset(l) + (long)m * L + n) * p.nb) * p.fo + j;
      const float2* xr = p.other + ((long)(l * l + m) * p.nb) * p.fi;
#pragma unroll 4
      for (int i = sl; i < p.nb; i += nsl) {
        const float2 gv = g[(long)i * p.fo];
#pragma unroll
        for (int k = 0; k < kThinFi; ++k) {
          if (k < p.fi) {
            const float2 xv = xr[i * p.fi + k];   // conj(gv) * xv
            acc[k].x = fmaf(gv.x, xv.x, acc[k].x);
            acc[k].x = fmaf(gv.y, xv.y, acc[k].x);
            acc[k].y = fmaf(gv.x, xv.y, acc[k].y);
            acc[k].y = fmaf(-gv.y, xv.x, acc[k].y);
          }
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kThinFi; ++k) red[ctx.tid * kThinFi + k] = acc[k];
  ctx.sync();
  // fixed summation order over the slices
  for (int e = ctx.tid; e < p.fo * p.fi; e += ctx.nthr) {
    const int k = e / p.fo, jj = e - k * p.fo;
    float2 s = make_float2(0.f, 0.f);
    for (int s2 = 0; s2 < nsl; ++s2) {
      const float2 t = red[(s2 * p.fo + jj) * kThinFi + k];
      s.x += t.x;
      s.y += t.y;
    }
    p.out[((long)(l * l + n) * p.fi + k) * p.fo + jj] = s;
  }
}

inline bool s2_mm_thin_supported(int nl, int fi, int fo) {
  return fi <= kThinFi && fo <= 1024 && s2_gradx_thin_smem(nl, fi, fo) <= 200 * 1024;
}

}  // namespace s2c
