// Grouped complex GEMM over the degrees l of a block-diagonal spectral product.
//
// One kernel covers all six products on the path - the forward, grad-x and grad-y of
//   so3_mm:  z[l,m,n,i,j] = sum_{p,k} x[l,m,p,i,k] conj(y[l,n,p,k,j])     (s2cnn/so3_mm.py:8-122)
//   s2_mm :  z[l,m,n,i,j] = sum_k     x[l,m,i,k]   conj(y[l,n,k,j])       (s2cnn/s2_mm.py:10-101)
// which the reference implements as the NVRTC kernels so3_mm.cu (so3_mm.py:125-261) and
// s2mm*.cu (s2_mm.py:140-312).  Every operand index (row, column, contraction) is a pair
// (outer, inner) - e.g. row = (m, batch) - and every operand address is
//     base(l) + outer_1 * so1(l) + inner_1 * si1 + outer_2 * so2(l) + inner_2 * si2
// with strides that are constants or constants times L = 2l+1.  The kernel works directly on
// the reference's interleaved [spectral, batch, feature, 2] layouts; no operand is transposed
// or copied beforehand.
//
// Tiling: 64 x 64 complex outputs per block, K tiles of 16, 256 threads with a 4 x 4 complex
// register tile each; operands are staged in shared memory split into real and imaginary
// planes, conjugation applied while staging.  All degrees are scheduled in one launch, largest
// degree first.
#pragma once

#include "backend.h"

namespace s2c {

struct CgemmOperand {
  long base_unit;   // base(l) = (base_sq ? l*l : l(4l^2-1)/3) * base_unit       (complex units)
  int base_sq;
  long o1c, o1L;    // outer stride of the first index  = o1c + o1L * L
  long i1;          // inner stride of the first index
  long o2c, o2L;    // outer stride of the second index
  long i2;          // inner stride of the second index
};

struct CgemmParams {
  const float2* A;  // first index = row, second = contraction
  const float2* B;  // first index = contraction, second = column
  float2* C;        // first index = row, second = column
  CgemmOperand a, b, c;
  int nl;
  int R2, C2, K2;   // inner extents of row / column / contraction indices
  int rL, cL, kL;   // outer extent is L (1) or 1 (0)
  int conjA, conjB;
  int a_fast_k;     // A is contiguous along the contraction index (else along rows)
  int b_fast_k;     // B is contiguous along the contraction index (else along columns)
};

constexpr int kGemmBM = 64, kGemmBN = 64, kGemmBK = 16;

S2C_HD long cgemm_tiles_for(const CgemmParams& p, int l) {
  const int L = 2 * l + 1;
  const long M = (long)(p.rL ? L : 1) * p.R2, N = (long)(p.cL ? L : 1) * p.C2;
  return ((M + kGemmBM - 1) / kGemmBM) * ((N + kGemmBN - 1) / kGemmBN);
}

S2C_D long cgemm_base(const CgemmOperand& o, int l) {
  const long s = o.base_sq ? (long)l * l : (long)l * (4L * l * l - 1) / 3;
  return s * o.base_unit;
}

S2C_KERNEL_BOUNDS(cgemm_grouped, CgemmParams, 256, 2) {
  // locate (l, tile_m, tile_n): degrees are laid out from the largest down
  int l = p.nl - 1;
  long t = ctx.bid;
  for (;; --l) {
    const long c = cgemm_tiles_for(p, l);
    if (t < c) break;
    t -= c;
  }
  const int L = 2 * l + 1;
  const int M = (p.rL ? L : 1) * p.R2, N = (p.cL ? L : 1) * p.C2, K = (p.kL ? L : 1) * p.K2;
  const int tiles_n = (N + kGemmBN - 1) / kGemmBN;
  const int tm = (int)(t / tiles_n), tn = (int)(t - (long)tm * tiles_n);
  const int row0 = tm * kGemmBM, col0 = tn * kGemmBN;

  const float2* A = p.A + cgemm_base(p.a, l);
  const float2* B = p.B + cgemm_base(p.b, l);
  float2* C = p.C + cgemm_base(p.c, l);
  const long a_o1 = p.a.o1c + p.a.o1L * L, a_o2 = p.a.o2c + p.a.o2L * L;
  const long b_o1 = p.b.o1c + p.b.o1L * L, b_o2 = p.b.o2c + p.b.o2L * L;
  const long c_o1 = p.c.o1c + p.c.o1L * L, c_o2 = p.c.o2c + p.c.o2L * L;

  float* Ar = reinterpret_cast<float*>(smem);
  float* Ai = Ar + kGemmBK * kGemmBM;
  float* Br = Ai + kGemmBK * kGemmBM;
  float* Bi = Br + kGemmBK * kGemmBN;

  const int tid = ctx.tid;
  const int tx = tid & 15, ty = tid >> 4;
  float cr[4][4], ci[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { cr[i][j] = 0.f; ci[i][j] = 0.f; }

  // each thread stages 4 elements of A and 4 of B per K tile
  // A tile element e = tid + 256 * q  ->  (row, kk)
  const float sa = p.conjA ? -1.f : 1.f, sb = p.conjB ? -1.f : 1.f;

  for (int k0 = 0; k0 < K; k0 += kGemmBK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = tid + 256 * q;
      int r, kk;
      if (p.a_fast_k) { r = e / kGemmBK; kk = e - r * kGemmBK; }
      else            { kk = e / kGemmBM; r = e - kk * kGemmBM; }
      const int gr = row0 + r, gk = k0 + kk;
      float2 v = make_float2(0.f, 0.f);
      if (gr < M && gk < K) {
        const int ro = gr / p.R2, ri = gr - ro * p.R2;
        const int ko = gk / p.K2, ki = gk - ko * p.K2;
        v = A[ro * a_o1 + ri * p.a.i1 + ko * a_o2 + ki * p.a.i2];
      }
      Ar[kk * kGemmBM + r] = v.x;
      Ai[kk * kGemmBM + r] = sa * v.y;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = tid + 256 * q;
      int cidx, kk;
      if (p.b_fast_k) { cidx = e / kGemmBK; kk = e - cidx * kGemmBK; }
      else            { kk = e / kGemmBN; cidx = e - kk * kGemmBN; }
      const int gc = col0 + cidx, gk = k0 + kk;
      float2 v = make_float2(0.f, 0.f);
      if (gc < N && gk < K) {
        const int co = gc / p.C2, cin = gc - co * p.C2;
        const int ko = gk / p.K2, ki = gk - ko * p.K2;
        v = B[ko * b_o1 + ki * p.b.i1 + co * b_o2 + cin * p.b.i2];
      }
      Br[kk * kGemmBN + cidx] = v.x;
      Bi[kk * kGemmBN + cidx] = sb * v.y;
    }
    ctx.sync();
#pragma unroll
    for (int kk = 0; kk < kGemmBK; ++kk) {
      float ar[4], ai[4], br[4], bi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ar[i] = Ar[kk * kGemmBM + ty + 16 * i];
        ai[i] = Ai[kk * kGemmBM + ty + 16 * i];
        br[i] = Br[kk * kGemmBN + tx + 16 * i];
        bi[i] = Bi[kk * kGemmBN + tx + 16 * i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          cr[i][j] = fmaf(ar[i], br[j], cr[i][j]);
          cr[i][j] = fmaf(-ai[i], bi[j], cr[i][j]);
          ci[i][j] = fmaf(ar[i], bi[j], ci[i][j]);
          ci[i][j] = fmaf(ai[i], br[j], ci[i][j]);
        }
    }
    ctx.sync();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty + 16 * i;
    if (gr >= M) continue;
    const int ro = gr / p.R2, ri = gr - ro * p.R2;
    const long rbase = ro * c_o1 + ri * p.c.i1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tx + 16 * j;
      if (gc >= N) continue;
      const int co = gc / p.C2, cin = gc - co * p.C2;
      C[rbase + co * c_o2 + cin * p.c.i2] = make_float2(cr[i][j], ci[i][j]);
    }
  }
}

inline size_t cgemm_smem_bytes() {
  return (size_t)(2 * kGemmBK * kGemmBM + 2 * kGemmBK * kGemmBN) * sizeof(float);
}
inline long cgemm_total_tiles(const CgemmParams& p) {
  long t = 0;
  for (int l = 0; l < p.nl; ++l) t += cgemm_tiles_for(p, l);
  return t;
}

// ---- operand descriptions of the six products ------------------------------------------------
enum MmOp : int { kMmFwd = 0, kMmGradX = 1, kMmGradY = 2 };

// so3 = true: x [nspec3, nb, fi], y [nspec3, fi, fo], z [nspec3, nb, fo]
// so3 = false: x [nl^2, nb, fi], y [nl^2, fi, fo], z [nspec3, nb, fo]
inline CgemmParams mm_params(bool so3, int op, int nl, int nb, int fi, int fo) {
  CgemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.nl = nl;
  const long NB = nb, FI = fi, FO = fo;
  // operand "shapes" in complex units
  CgemmOperand X, Y, Z;
  std::memset(&X, 0, sizeof(X));
  std::memset(&Y, 0, sizeof(Y));
  std::memset(&Z, 0, sizeof(Z));
  X.base_unit = NB * FI; X.base_sq = so3 ? 0 : 1;
  Y.base_unit = FI * FO; Y.base_sq = so3 ? 0 : 1;
  Z.base_unit = NB * FO; Z.base_sq = 0;
  if (op == kMmFwd) {
    // rows (m,i)  cols (n,j)  contraction (p,k) [so3] or k [s2]
    p.rL = 1; p.R2 = nb; p.cL = 1; p.C2 = fo; p.kL = so3 ? 1 : 0; p.K2 = fi;
    p.a = X;  // A[(m,i),(p,k)] = x[l,m,p,i,k]   |  x[l,m,i,k]
    if (so3) { p.a.o1L = NB * FI; p.a.i1 = FI; p.a.o2c = NB * FI; p.a.i2 = 1; }
    else     { p.a.o1c = NB * FI; p.a.i1 = FI; p.a.o2c = 0;       p.a.i2 = 1; }
    p.b = Y;  // B[(p,k),(n,j)] = y[l,n,p,k,j]   |  y[l,n,k,j]
    if (so3) { p.b.o1c = FI * FO; p.b.i1 = FO; p.b.o2L = FI * FO; p.b.i2 = 1; }
    else     { p.b.o1c = 0;       p.b.i1 = FO; p.b.o2c = FI * FO; p.b.i2 = 1; }
    p.c = Z;  // z[l,m,n,i,j]
    p.c.o1L = NB * FO; p.c.i1 = FO; p.c.o2c = NB * FO; p.c.i2 = 1;
    p.conjA = 0; p.conjB = 1; p.a_fast_k = 1; p.b_fast_k = 0;
  } else if (op == kMmGradX) {
    // gx[l,m,p,i,k] = sum_{n,j} gz[l,m,n,i,j] y[l,n,p,k,j]: rows (m,i) cols (p,k)|k contraction (n,j)
    p.rL = 1; p.R2 = nb; p.cL = so3 ? 1 : 0; p.C2 = fi; p.kL = 1; p.K2 = fo;
    p.a = Z;  // A[(m,i),(n,j)] = gz
    p.a.o1L = NB * FO; p.a.i1 = FO; p.a.o2c = NB * FO; p.a.i2 = 1;
    p.b = Y;  // B[(n,j),(p,k)] = y[l,n,p,k,j]  |  y[l,n,k,j]
    if (so3) { p.b.o1L = FI * FO; p.b.i1 = 1; p.b.o2c = FI * FO; p.b.i2 = FO; }
    else     { p.b.o1c = FI * FO; p.b.i1 = 1; p.b.o2c = 0;       p.b.i2 = FO; }
    p.c = X;  // gx
    if (so3) { p.c.o1L = NB * FI; p.c.i1 = FI; p.c.o2c = NB * FI; p.c.i2 = 1; }
    else     { p.c.o1c = NB * FI; p.c.i1 = FI; p.c.o2c = 0;       p.c.i2 = 1; }
    p.conjA = 0; p.conjB = 0; p.a_fast_k = 1; p.b_fast_k = 1;
  } else {
    // gy[l,n,p,k,j] = sum_{m,i} conj(gz[l,m,n,i,j]) x[l,m,p,i,k]: rows (p,k)|k cols (n,j)
    p.rL = so3 ? 1 : 0; p.R2 = fi; p.cL = 1; p.C2 = fo; p.kL = 1; p.K2 = nb;
    p.a = X;  // A[(p,k),(m,i)] = x[l,m,p,i,k]  |  x[l,m,i,k]
    if (so3) { p.a.o1c = NB * FI; p.a.i1 = 1; p.a.o2L = NB * FI; p.a.i2 = FI; }
    else     { p.a.o1c = 0;       p.a.i1 = 1; p.a.o2c = NB * FI; p.a.i2 = FI; }
    p.b = Z;  // B[(m,i),(n,j)] = conj gz
    p.b.o1L = NB * FO; p.b.i1 = FO; p.b.o2c = NB * FO; p.b.i2 = 1;
    p.c = Y;  // gy[l,n,p,k,j]  |  gy[l,n,k,j]
    if (so3) { p.c.o1c = FI * FO; p.c.i1 = FO; p.c.o2L = FI * FO; p.c.i2 = 1; }
    else     { p.c.o1c = 0;       p.c.i1 = FO; p.c.o2c = FI * FO; p.c.i2 = 1; }
    p.conjA = 0; p.conjB = 1; p.a_fast_k = 0; p.b_fast_k = 0;
  }
  return p;
}

// Rotation of an SO(3) spectrum by block-diagonal Wigner-D matrices (s2cnn/soft/so3_rotation.py:22-41):
//   adjoint = 0:  z[l,m,n,b]  = sum_k conj(U^l[m,k]) x[l,k,n,b]
//   adjoint = 1:  gx[l,k,n,b] = sum_m      U^l[m,k]  gz[l,m,n,b]      (transpose of the above)
// U is the concatenation over l of the (2l+1) x (2l+1) matrices, x / z are [nspec3, nbatch].
inline CgemmParams rotation_params(int nl, long nbatch, int adjoint) {
  CgemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.nl = nl;
  p.rL = 1; p.R2 = 1; p.cL = 1; p.C2 = (int)nbatch; p.kL = 1; p.K2 = 1;
  p.a.base_unit = 1;
  if (!adjoint) { p.a.o1L = 1; p.a.o2c = 1; p.a_fast_k = 1; p.conjA = 1; }
  else          { p.a.o1c = 1; p.a.o2L = 1; p.a_fast_k = 0; p.conjA = 0; }
  p.b.base_unit = nbatch; p.b.o1L = nbatch; p.b.o2c = nbatch; p.b.i2 = 1;
  p.c = p.b;
  p.conjB = 0; p.b_fast_k = 0;
  return p;
}

}  // namespace s2c
