// Plane kernels of the general SO(3) path for N = 2b in {64, 128}: BOTH row transforms of one
// (z, beta) plane in one kernel, so that the [z][n][beta][alpha] scratch array of the three-pass
// organisation (so3_kernels.h) and its write + read of 8 K N^2 bytes per signal disappear.
//
//   analysis  (so3_fwd_plane): real plane x[alpha][gamma] -> FFT over gamma of N/2 packed row
//       pairs (alpha, alpha + N/2) -> shared plane C[t][f] -> FFT over alpha of the kept columns
//       n < K, the Hermitian split of the packed pairs applied while loading -> V[n][m][z][beta]
//   synthesis (so3_inv_plane): the same steps reversed, ending with + bias and the store of the
//       real plane.
//
// Every 1-D transform is a two-step register FFT (N = R1 * R2: R1-point transforms, twiddle,
// transpose through a small buffer, R2-point transforms, natural order out) run by ONE WARP on four
// rows (or columns) at a time with a warp-private transpose buffer, so the steps are separated by
// warp barriers only; a block of 8 warps needs one block barrier per plane (between the two
// transforms).  The first step of the first transform reads global memory directly and the
// second step of the last one writes it directly, so a sample crosses shared memory three times
// instead of global memory twice.  Strides are chosen so that every shared-memory access pattern
// is conflict free: the plane C[t][f] has an odd row stride and a warp works on rows
// {t, t+8, t+1, t+9} and columns {n, n+8, n+16, n+24}; transpose rows have a stride = 8 mod 16.
//
// Same arithmetic as so3_fwd_gamma + so3_fwd_alpha and so3_inv_alpha + so3_inv_gamma, i.e. the
// torch.fft calls around the reference's Wigner kernels (s2cnn/soft/so3_fft.py:40-42, 89-92,
// 181-199).
//
// V is beta-innermost (the Wigner contraction runs over beta), so a block that owns one plane
// touches V in isolated 8-byte pieces - measured on a B200 at b = 64 that alone makes the kernel
// slower than the two passes it replaces.  The CL = true variants therefore run as thread-block
// clusters of 4 consecutive beta planes of one signal and exchange through distributed shared
// memory: each warp parks its columns of V in its own transpose buffer, and after a cluster
// barrier block r moves the r-th quarter of the entries for all 4 planes - 32 contiguous bytes per
// entry, neighbouring lanes on neighbouring 16-byte pieces - between the blocks' shared memories
// and global memory.  (Measured at b = 64, batch 64: 8 B pieces 1.2 ms, clusters of 4 0.52 ms,
// clusters of 8 0.58 ms; of the 0.52 ms about 0.20 is arithmetic and shared-memory traffic, 0.14
// the stores of V, 0.11 the remote shared-memory reads, 0.07 the input loads, 0.05 the barriers.)
// The CL = false variants touch V directly; the host-emulation build and the tests use them as a
// second implementation.
#pragma once

#include "backend.h"
#include "fft_device.h"
#include "fft_reg.h"

#ifndef S2C_EMUL
#include <cooperative_groups.h>
#endif

namespace s2c {

constexpr int kPlaneCluster = 4;   // blocks (beta planes) per cluster of the CL variants (8 measured slower)
constexpr int kPlaneRW = 4;        // rows (or columns) a warp transforms at a time: 4 (8 warps) or 2 (16 warps, measured slower)

#ifndef S2C_EMUL
__device__ __forceinline__ unsigned plane_cluster_rank() {
  return cooperative_groups::this_cluster().block_rank();
}
__device__ __forceinline__ void plane_cluster_sync() { cooperative_groups::this_cluster().sync(); }
// the same shared-memory location in block `rank` of the cluster
__device__ __forceinline__ float2* plane_cluster_ptr(float2* local, unsigned rank) {
  return cooperative_groups::this_cluster().map_shared_rank(local, rank);
}
#else
// never instantiated with CL = true in the emulation build
inline unsigned plane_cluster_rank() { return 0; }
inline void plane_cluster_sync() {}
inline float2* plane_cluster_ptr(float2* local, unsigned) { return local; }
#endif

struct FwdPlaneParams {
  const float* x;     // real signal, element e at x[e * in_stride + in_off]
  long in_stride, in_off;
  float2* v;          // [n < K][mi < 2K-1][z][beta]
  const float2* tw;   // exp(+2 pi i k / N), k < N
  int nbatch, K;
};

struct InvPlaneParams {
  const float2* s;    // [n < K][mi < 2K-1][z][beta]; for n = 0 only m >= 0 is stored
  float* out;         // real signal, element e at out[e * out_stride + out_off]
  long out_stride, out_off;
  const float* bias;  // optional [nfeat]; feature of signal z is (z0 + z) % nfeat
  int nfeat;
  long z0;
  const float2* tw;
  int nbatch, K;
};

S2C_HD constexpr bool plane_supported(int N) { return N == 64 || N == 128; }
S2C_HD constexpr int plane_rb(int N) { return N / 8; }              // N = 8 * RB, RB = 8 or 16
S2C_HD constexpr int plane_ldb(int N) { return N + 1; }             // odd row stride of the plane
// row stride of a transpose buffer whose first step has radix R1: >= N + R1 - 1 and = 8 mod 16
S2C_HD constexpr int plane_ldt(int N, int R1) { return (N + R1 - 1 + 7) / 16 * 16 + 8; }
// RW rows per warp at a time: 32 / RW warps per block cover 32 columns (or row pairs) per pass
S2C_HD constexpr int plane_warps(int RW) { return 32 / RW; }
S2C_HD constexpr int plane_threads(int RW) { return 32 * plane_warps(RW); }
// complex numbers per warp-private buffer (RW rows)
S2C_HD constexpr int plane_wt(int N, int RW) { return RW * plane_ldt(N, 8); }
inline size_t plane_smem_bytes(int N, int RW) {
  return ((size_t)N + (size_t)(N / 2) * plane_ldb(N) + (size_t)plane_warps(RW) * plane_wt(N, RW)) *
         sizeof(float2);
}
// row tl of row group g: rows of one group differ by 8 (and 1), e.g. {t, t+8, t+1, t+9} for RW = 4
S2C_HD constexpr int plane_row(int RW, int g, int tl) {
  return RW == 4 ? 16 * (g / 4) + 2 * (g % 4) + (tl & 1) * 8 + (tl >> 1)
                 : 16 * (g / 8) + (g % 8) + 8 * tl;
}
// column chunk of 32: warp w owns columns first + 8 i, i < RW
S2C_HD constexpr int plane_col0(int RW, int warp) { return (warp % 8) + 8 * RW * (warp / 8); }
// ... and column nl of the chunk lives in this warp / this row of the warp's buffer
S2C_HD constexpr int plane_col_warp(int RW, int nl) { return (nl % 8) + 8 * (nl / (8 * RW)); }
S2C_HD constexpr int plane_col_row(int RW, int nl) { return (nl / 8) % RW; }

// step 1 output: frequency pc of the R1-point transform, times W_N^(j pc), to dst[pc * (R2 + 1)]
template <int R1, int R2, int DIR>
S2C_D void plane_put_step1(float2 (&v)[R1], float2* dst, int j, const float2* tw) {
  static_for<0, R1>([&](auto pc_) {
    constexpr int pc = decltype(pc_)::value;
    constexpr int pp = fft_reg_pos<R1>(pc);
    if constexpr (pc == 0) dst[0] = v[pp];
    else dst[pc * (R2 + 1)] = ctw<DIR>(v[pp], tw[j * pc]);
  });
}

template <int N, bool CL, int RW>
struct so3_fwd_plane_impl {
  static S2C_D void run(const Ctx& ctx, const FwdPlaneParams& p, unsigned char* smem) {
    constexpr int RB = plane_rb(N);                 // both transforms: radix 8 first, then RB
    constexpr int LDB = plane_ldb(N), LDT = plane_ldt(N, 8), WT = plane_wt(N, RW);
    constexpr int NW = plane_warps(RW);
    constexpr int NG = (N / 2) / 32;                 // row groups per warp
    float2* tw = reinterpret_cast<float2*>(smem);
    float2* B = tw + N;                               // packed plane C[t][f], [N/2][LDB]
    float2* tmp = B + (size_t)(N / 2) * LDB;          // [warps][WT]
    const int warp = ctx.tid >> 5, lane = ctx.tid & 31;
    float2* wtmp = tmp + warp * WT;
    const int K = p.K, nm = 2 * K - 1;
    const long z = ctx.bid / N;
    const int beta = (int)(ctx.bid - z * N);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    ctx.sync();

    // ---- FFT over gamma of the packed row pairs (t, t + N/2) -----------------------------------
    const long plane0 = ((z * N + beta) * N) * (long)N;
    for (int gi = 0; gi < NG; ++gi) {
      const int g = gi * NW + warp;
#pragma unroll
      for (int it0 = 0; it0 < RW * RB; it0 += 32) {
        const int it = it0 + lane, tl = it / RB, j = it % RB;
        if (RW * RB < 32 && it >= RW * RB) continue;
        const long e1 = plane0 + (long)plane_row(RW, g, tl) * N + j;
        const long e2 = e1 + (long)(N / 2) * N;
        float2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[k].x = p.x[(e1 + RB * k) * p.in_stride + p.in_off];
          v[k].y = p.x[(e2 + RB * k) * p.in_stride + p.in_off];
        }
        fft_reg<8, -1>(v, tw);
        plane_put_step1<8, RB, -1>(v, wtmp + tl * LDT + j, j, tw);
      }
      ctx.sync_warp();
      if (lane < RW * 8) {
        const int tl = lane / 8, pq = lane % 8;
        const float2* src = wtmp + tl * LDT + pq * (RB + 1);
        float2 u[RB];
#pragma unroll
        for (int j = 0; j < RB; ++j) u[j] = src[j];
        fft_reg<RB, -1>(u, tw);
        float2* dst = B + plane_row(RW, g, tl) * LDB + pq;
        static_for<0, RB>([&](auto q_) {
          constexpr int q = decltype(q_)::value;
          dst[8 * q] = u[fft_reg_pos<RB>(q)];
        });
      }
      ctx.sync_warp();
    }
    ctx.sync();

    // ---- FFT over alpha of the kept columns, Hermitian split on load ----------------------------
    const int nchunks = (K + 31) / 32;
    for (int c = 0; c < nchunks; ++c) {
      const int n0 = c * 32 + plane_col0(RW, warp);   // this warp's columns: n0 + 8 i, i < RW
#pragma unroll
      for (int it0 = 0; it0 < RW * RB; it0 += 32) {
        const int it = it0 + lane, i = it / RB, j = it % RB;
        const int n = (RW * RB < 32 && it >= RW * RB) ? K : n0 + 8 * i;
        if (n < K) {
          const int nc = n == 0 ? 0 : N - n;
          float2 v[8];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const int t = j + RB * kk;
            const float2 a = B[t * LDB + n], cc = B[t * LDB + nc];
            v[kk] = make_float2(0.5f * (a.x + cc.x), 0.5f * (a.y - cc.y));          // row t
            v[kk + 4] = make_float2(0.5f * (a.y + cc.y), -0.5f * (a.x - cc.x));     // row t + N/2
          }
          fft_reg<8, -1>(v, tw);
          plane_put_step1<8, RB, -1>(v, wtmp + i * LDT + j, j, tw);
        }
      }
      ctx.sync_warp();
      const int i = lane / 8, pq = lane % 8;
      const int n = lane < RW * 8 ? n0 + 8 * i : K;
      float2 u[RB];
      if (n < K) {
        const float2* src = wtmp + i * LDT + pq * (RB + 1);
#pragma unroll
        for (int j = 0; j < RB; ++j) u[j] = src[j];
        fft_reg<RB, -1>(u, tw);
      }
      if constexpr (CL) {
        // the transpose rows become the exchange rows xb[i][mi] of this warp's columns
        ctx.sync_warp();
        if (n < K) {
          static_for<0, RB>([&](auto q_) {
            constexpr int q = decltype(q_)::value;
            const int f = pq + 8 * q;
            const int m = f < N / 2 ? f : f - N;       // f = N/2 gives |m| = N/2 >= K: dropped
            if (m > -K && m < K) wtmp[i * LDT + m + K - 1] = u[fft_reg_pos<RB>(q)];
          });
        }
        plane_cluster_sync();
        {
          const unsigned rank = plane_cluster_rank();
          const int ncols = (K - c * 32) < 32 ? (K - c * 32) : 32;
          // item = (entry, pair of planes): neighbouring lanes write neighbouring 16-byte pieces, so a
          // warp's store covers whole 32-byte sectors
          constexpr int HP = kPlaneCluster / 2;
          const int entries = ncols * nm;
          const int per = (entries + kPlaneCluster - 1) / kPlaneCluster;   // entries per block
          const int e_lo = (int)rank * per;
          const int e_cnt = (entries - e_lo) < per ? (entries - e_lo) : per;
          for (int it = ctx.tid; it < e_cnt * HP; it += ctx.nthr) {
            const int e = e_lo + it / HP, h = it % HP;
            const int nl = e / nm, mi = e - nl * nm;
            float2* cell = tmp + plane_col_warp(RW, nl) * WT + plane_col_row(RW, nl) * LDT + mi;
            const float2 v0 = *plane_cluster_ptr(cell, 2 * h);
            const float2 v1 = *plane_cluster_ptr(cell, 2 * h + 1);
            float4* dst = reinterpret_cast<float4*>(
                p.v + ((((long)(c * 32 + nl)) * nm + mi) * p.nbatch + z) * N + (beta - (int)rank));
            dst[h] = make_float4(v0.x, v0.y, v1.x, v1.y);
          }
        }
        plane_cluster_sync();   // peers are done with this block's exchange rows
      } else {
        if (n < K) {
          float2* vcol = p.v + (((long)n * nm) * p.nbatch + z) * N + beta;
          static_for<0, RB>([&](auto q_) {
            constexpr int q = decltype(q_)::value;
            const int f = pq + 8 * q;
            const int m = f < N / 2 ? f : f - N;
            if (m > -K && m < K) vcol[(long)(m + K - 1) * p.nbatch * N] = u[fft_reg_pos<RB>(q)];
          });
        }
        ctx.sync_warp();
      }
    }
  }
};

template <int N, bool CL, int RW>
struct so3_inv_plane_impl {
  static S2C_D void run(const Ctx& ctx, const InvPlaneParams& p, unsigned char* smem) {
    constexpr int RB = plane_rb(N);                 // both transforms: radix 8 first, then RB
    constexpr int LDB = plane_ldb(N), LDA = plane_ldt(N, 8), LDG = plane_ldt(N, 8);
    constexpr int WT = plane_wt(N, RW);
    constexpr int NW = plane_warps(RW);
    constexpr int NG = (N / 2) / 32;
    float2* tw = reinterpret_cast<float2*>(smem);
    float2* B = tw + N;
    float2* tmp = B + (size_t)(N / 2) * LDB;
    const int warp = ctx.tid >> 5, lane = ctx.tid & 31;
    float2* wtmp = tmp + warp * WT;
    const int K = p.K, nm = 2 * K - 1;
    const long z = ctx.bid / N;
    const int beta = (int)(ctx.bid - z * N);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    {  // frequencies K .. N-K of every packed row are zero
      const int cnt = N - 2 * K + 1;
      for (int it = ctx.tid; it < (N / 2) * cnt; it += ctx.nthr) {
        const int row = it / cnt, col = K + (it - row * cnt);
        B[row * LDB + col] = make_float2(0.f, 0.f);
      }
    }
    ctx.sync();

    // ---- inverse FFT over m -> alpha of the kept columns, packed into row pairs on store --------
    const int nchunks = (K + 31) / 32;
    for (int c = 0; c < nchunks; ++c) {
      const int n0 = c * 32 + plane_col0(RW, warp);   // this warp's columns: n0 + 8 i, i < RW
      if constexpr (CL) {
        // bring the chunk's slice of V for the cluster's planes in, 8 contiguous bytes per plane and entry,
        // and deal it out to the exchange rows xb[i][mi] of the warps that own the columns
        plane_cluster_sync();   // every block runs, and is done with its buffers of the previous chunk
        const unsigned rank = plane_cluster_rank();
        const int ncols = (K - c * 32) < 32 ? (K - c * 32) : 32;
        const int total = ncols * nm;
        const int per = (total + kPlaneCluster - 1) / kPlaneCluster;
        for (int e0 = ctx.tid; e0 < per; e0 += ctx.nthr) {
          const int e = (int)rank * per + e0;
          if (e >= total) continue;
          const int nl = e / nm, mi = e - nl * nm;
          float2* cell = tmp + plane_col_warp(RW, nl) * WT + plane_col_row(RW, nl) * LDA + mi;
          const float4* src = reinterpret_cast<const float4*>(
              p.s + ((((long)(c * 32 + nl)) * nm + mi) * p.nbatch + z) * N + (beta - (int)rank));
          float4 val[kPlaneCluster / 2];
#pragma unroll
          for (int r = 0; r < kPlaneCluster / 2; ++r) val[r] = src[r];
#pragma unroll
          for (int r = 0; r < kPlaneCluster / 2; ++r) {
            *plane_cluster_ptr(cell, 2 * r) = make_float2(val[r].x, val[r].y);
            *plane_cluster_ptr(cell, 2 * r + 1) = make_float2(val[r].z, val[r].w);
          }
        }
        plane_cluster_sync();
      }
#pragma unroll
      for (int it0 = 0; it0 < RW * RB; it0 += 32) {
        const int it = it0 + lane, i = it / RB, j = it % RB;
        const int n = (RW * RB < 32 && it >= RW * RB) ? K : n0 + 8 * i;
        float2 v[8];
        if (n < K) {
          const float2* scol = p.s + (((long)n * nm) * p.nbatch + z) * N + beta;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int f = j + RB * k;
            const int m = f < N / 2 ? f : f - N;
            const bool keep = m > -K && m < K;
            const bool cj = n == 0 && m < 0;            // stored as the conjugate of (0, -m)
            const int mi = (cj ? -m : m) + K - 1;
            float2 a = make_float2(0.f, 0.f);
            if (keep) a = CL ? wtmp[i * LDA + mi] : scol[(long)mi * p.nbatch * N];
            if (cj) a.y = -a.y;
            v[k] = a;
          }
        }
        if constexpr (CL) ctx.sync_warp();   // the exchange rows of this pass are consumed
        if (n < K) {
          fft_reg<8, +1>(v, tw);
          plane_put_step1<8, RB, +1>(v, wtmp + i * LDA + j, j, tw);
        }
      }
      ctx.sync_warp();
      {
        const int i = lane / 8, pq = lane % 8;
        const int n = lane < RW * 8 ? n0 + 8 * i : K;
        if (n < K) {
          const float2* src = wtmp + i * LDA + pq * (RB + 1);
          float2 u[RB];
#pragma unroll
          for (int j = 0; j < RB; ++j) u[j] = src[j];
          fft_reg<RB, +1>(u, tw);
          static_for<0, RB / 2>([&](auto q_) {
            constexpr int q = decltype(q_)::value;
            const float2 t1 = u[fft_reg_pos<RB>(q)];            // alpha = pq + 8 q          (row t)
            const float2 t2 = u[fft_reg_pos<RB>(q + RB / 2)];   // alpha + N/2               (row t + N/2)
            float2* row = B + (pq + 8 * q) * LDB;
            if (n == 0) {
              // T[alpha][0] is real for a Hermitian spectrum; its rounding-level imaginary part is dropped
              row[0] = make_float2(t1.x, t2.x);
            } else {
              row[n] = make_float2(t1.x - t2.y, t1.y + t2.x);       // T1 + i T2
              row[N - n] = make_float2(t1.x + t2.y, t2.x - t1.y);   // conj(T1) + i conj(T2)
            }
          });
        }
      }
      ctx.sync_warp();
    }
    ctx.sync();

    // ---- inverse FFT over n -> gamma of the packed rows, + bias, store --------------------------
    float add = 0.f;
    if (p.bias) add = p.bias[(p.z0 + z) % p.nfeat];
    const long plane0 = ((z * N + beta) * N) * (long)N;
    for (int gi = 0; gi < NG; ++gi) {
      const int g = gi * NW + warp;
#pragma unroll
      for (int it0 = 0; it0 < RW * RB; it0 += 32) {
        const int it = it0 + lane, tl = it / RB, j = it % RB;
        if (RW * RB < 32 && it >= RW * RB) continue;
        const float2* src = B + plane_row(RW, g, tl) * LDB + j;
        float2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = src[RB * k];
        fft_reg<8, +1>(v, tw);
        plane_put_step1<8, RB, +1>(v, wtmp + tl * LDG + j, j, tw);
      }
      ctx.sync_warp();
      if (lane < RW * 8) {
        const int tl = lane / 8, pq = lane % 8;
        const float2* src = wtmp + tl * LDG + pq * (RB + 1);
        float2 u[RB];
#pragma unroll
        for (int j = 0; j < RB; ++j) u[j] = src[j];
        fft_reg<RB, +1>(u, tw);
        const long e1 = plane0 + (long)plane_row(RW, g, tl) * N + pq;
        const long e2 = e1 + (long)(N / 2) * N;
        static_for<0, RB>([&](auto q_) {
          constexpr int q = decltype(q_)::value;
          const float2 val = u[fft_reg_pos<RB>(q)];
          p.out[(e1 + 8 * q) * p.out_stride + p.out_off] = val.x + add;
          p.out[(e2 + 8 * q) * p.out_stride + p.out_off] = val.y + add;
        });
      }
      ctx.sync_warp();
    }
  }
};

#ifndef S2C_EMUL
template <int N>
__global__ void __launch_bounds__(plane_threads(kPlaneRW), 2) so3_fwd_plane(const FwdPlaneParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_fwd_plane_impl<N, false, kPlaneRW>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
template <int N>
__global__ void __launch_bounds__(plane_threads(kPlaneRW), 2) so3_inv_plane(const InvPlaneParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_inv_plane_impl<N, false, kPlaneRW>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
// cluster variants: consecutive blocks = consecutive beta planes of one signal (N % cluster == 0)
template <int N>
__global__ void __cluster_dims__(kPlaneCluster, 1, 1) __launch_bounds__(plane_threads(kPlaneRW), 2)
so3_fwd_plane_cl(const FwdPlaneParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_fwd_plane_impl<N, true, kPlaneRW>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
template <int N>
__global__ void __cluster_dims__(kPlaneCluster, 1, 1) __launch_bounds__(plane_threads(kPlaneRW), 2)
so3_inv_plane_cl(const InvPlaneParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_inv_plane_impl<N, true, kPlaneRW>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
#define S2C_LAUNCH_PLANE(name, N, grid, stream, params)                                       \
  s2c::launch_impl(name<N>, #name, (long)(grid), s2c::plane_threads(s2c::kPlaneRW),           \
                   s2c::plane_smem_bytes(N, s2c::kPlaneRW), stream, params)
#define S2C_LAUNCH_PLANE_CL(name, N, grid, stream, params)                                    \
  s2c::launch_impl(name##_cl<N>, #name "_cl", (long)(grid), s2c::plane_threads(s2c::kPlaneRW),\
                   s2c::plane_smem_bytes(N, s2c::kPlaneRW), stream, params)
#else
#define S2C_LAUNCH_PLANE(name, N, grid, stream, params)                                       \
  s2c::emu_launch<name##_impl<N, false, s2c::kPlaneRW>>(                                      \
      #name, (long)(grid), s2c::plane_threads(s2c::kPlaneRW),                                 \
      s2c::plane_smem_bytes(N, s2c::kPlaneRW), params)
#define S2C_LAUNCH_PLANE_CL(name, N, grid, stream, params)                                    \
  S2C_LAUNCH_PLANE(name, N, grid, stream, params)
#endif

}  // namespace s2c
