// Plane kernels of the large-bandwidth SO(3) path for N = 2b in {64, 128}: BOTH row transforms of
// one (z, beta) plane in one kernel, so that the [z][n][beta][alpha] scratch array of the three-pass
// organisation (so3_kernels.h) and its write + read of 8 K N^2 bytes per signal disappear.
//
//   analysis  (so3_fwd_plane): real plane x[alpha][gamma] -> FFT over gamma of N/2 packed row
//       pairs (alpha, alpha + N/2) -> shared plane C[t][f] -> FFT over alpha of the kept columns
//       n < K, the Hermitian split of the packed pairs applied while loading -> V
//   synthesis (so3_inv_plane): the same steps reversed, ending with + bias and the store of the
//       real plane.
//
// Scratch layout, chosen for THESE kernels:  V[n < K][z < zc][beta < N][f < N]  (complex), f the
// raw FFT bin of the alpha transform (frequency m at f = m mod N).  A block that owns one plane
// therefore reads / writes, for every kept n, one contiguous row of N complex numbers (1 KB at
// b = 64), 64 aligned bytes per 8 lanes.  The Wigner kernels (wigner_rows.h) do the transposition to
// "beta innermost" on their side, through shared memory, 32 bytes (one sector) at a time.  The batch
// is processed in chunks of zc signals sized so that V (8 K N^2 bytes per signal) stays in L2
// between the two kernels; the signal itself is read / written with streaming (evict-first) hints.
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
#pragma once

#include "backend.h"
#include "fft_device.h"
#include "fft_reg.h"

namespace s2c {

constexpr int kPlaneRW = 4;        // rows (or columns) a warp transforms at a time: 8 warps per block

// streaming accesses: the signal is touched once, keep it from displacing V and the tables in L2
#ifndef S2C_EMUL
__device__ __forceinline__ float plane_ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ void plane_st_stream(float* p, float v) { __stcs(p, v); }
#else
inline float plane_ld_stream(const float* p) { return *p; }
inline void plane_st_stream(float* p, float v) { *p = v; }
#endif

struct FwdPlaneParams {
  const float* x;     // real signal, element e at x[e * in_stride + in_off]
  long in_stride, in_off;
  float2* v;          // [n < K][z < nbatch][beta][f < N]
  const float2* tw;   // exp(+2 pi i k / N), k < N
  int nbatch, K;      // nbatch = signals of this chunk
};

struct InvPlaneParams {
  const float2* s;    // [n < K][z < nbatch][beta][f < N]
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

template <int N, int RW>
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
    const int K = p.K;
    const long z = ctx.bid / N;
    const int beta = (int)(ctx.bid - z * N);
    // ---- FFT over gamma of the packed row pairs (t, t + N/2) -----------------------------------
    // The loads of batch k + 1 are issued before batch k is transformed, so a global-memory
    // latency is exposed once per plane instead of once per batch.
    const long plane0 = ((z * N + beta) * N) * (long)N;
    constexpr int IT = (RW * RB + 31) / 32;          // batches of 32 (row, j) items per row group
    auto load_batch = [&](int bi, float2 (&v)[8]) {
      const int g = (bi / IT) * NW + warp;
      const int it = (bi % IT) * 32 + lane, tl = it / RB, j = it % RB;
      if (RW * RB < 32 && it >= RW * RB) return;
      const long e1 = plane0 + (long)plane_row(RW, g, tl) * N + j;
      const long e2 = e1 + (long)(N / 2) * N;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[k].x = plane_ld_stream(p.x + (e1 + RB * k) * p.in_stride + p.in_off);
        v[k].y = plane_ld_stream(p.x + (e2 + RB * k) * p.in_stride + p.in_off);
      }
    };
    float2 vnext[8];
    load_batch(0, vnext);
#ifndef S2C_EMUL
    // Ask L2 for the plane that a block starting about one wave later will read (blocks are
    // dispatched in index order, two per SM): its first rows then arrive with the latency of L2
    // instead of HBM.  The register prefetch above reaches only one batch of rows ahead.
    if (p.in_stride == 1) {
      const long ahead = ctx.bid + 2L * 148;
      if (ahead < ctx.nblk) {
        const float* nx = p.x + p.in_off + ahead * (long)N * N;
        for (int i = ctx.tid * 32; i < N * N; i += ctx.nthr * 32)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + i));
      }
    }
#endif
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    ctx.sync();
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      const int g = gi * NW + warp;
#pragma unroll
      for (int ii = 0; ii < IT; ++ii) {
        const int it = ii * 32 + lane, tl = it / RB, j = it % RB;
        float2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = vnext[k];
        if (gi * IT + ii + 1 < NG * IT) load_batch(gi * IT + ii + 1, vnext);
        if (RW * RB < 32 && it >= RW * RB) continue;
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
      if (n < K) {
        const float2* src = wtmp + i * LDT + pq * (RB + 1);
        float2 u[RB];
#pragma unroll
        for (int j = 0; j < RB; ++j) u[j] = src[j];
        fft_reg<RB, -1>(u, tw);
        // row of this (n, z, beta): bins pq + 8 q; eight neighbouring lanes write 64 aligned bytes
        float2* vrow = p.v + (((long)n * p.nbatch + z) * N + beta) * N + pq;
        static_for<0, RB>([&](auto q_) {
          constexpr int q = decltype(q_)::value;
          const int f = pq + 8 * q;
          const int m = f < N / 2 ? f : f - N;       // f = N/2 is |m| = N/2 >= K: never read
          if (m > -K && m < K) vrow[8 * q] = u[fft_reg_pos<RB>(q)];
        });
      }
      ctx.sync_warp();
    }
  }
};

template <int N, int RW>
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
    const int K = p.K;
    const long z = ctx.bid / N;
    const int beta = (int)(ctx.bid - z * N);
    // ---- inverse FFT over m -> alpha of the kept columns, packed into row pairs on store --------
    // The rows of batch k + 1 are requested before batch k is transformed (see so3_fwd_plane).
    const int nchunks = (K + 31) / 32;
    constexpr int IT = (RW * RB + 31) / 32;
    auto load_batch = [&](int bi, float2 (&v)[8]) {
      const int c = bi / IT;
      const int n0 = c * 32 + plane_col0(RW, warp);   // this warp's columns: n0 + 8 i, i < RW
      const int it = (bi % IT) * 32 + lane, i = it / RB, j = it % RB;
      const int n = (RW * RB < 32 && it >= RW * RB) ? K : n0 + 8 * i;
      if (n < K) {
        // bins j + RB k of the row of this (n, z, beta): RB neighbouring lanes read RB * 8
        // contiguous bytes per k
        const float2* srow = p.s + (((long)n * p.nbatch + z) * N + beta) * N + j;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int f = j + RB * k;
          const int m = f < N / 2 ? f : f - N;
          v[k] = (m > -K && m < K) ? srow[RB * k] : make_float2(0.f, 0.f);
        }
      }
    };
    float2 vnext[8];
    load_batch(0, vnext);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    {  // frequencies K .. N-K of every packed row are zero
      const int cnt = N - 2 * K + 1;
      for (int it = ctx.tid; it < (N / 2) * cnt; it += ctx.nthr) {
        const int row = it / cnt, col = K + (it - row * cnt);
        B[row * LDB + col] = make_float2(0.f, 0.f);
      }
    }
    ctx.sync();
    for (int c = 0; c < nchunks; ++c) {
      const int n0 = c * 32 + plane_col0(RW, warp);
#pragma unroll
      for (int ii = 0; ii < IT; ++ii) {
        const int it = ii * 32 + lane, i = it / RB, j = it % RB;
        const int n = (RW * RB < 32 && it >= RW * RB) ? K : n0 + 8 * i;
        float2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = vnext[k];
        if (c * IT + ii + 1 < nchunks * IT) load_batch(c * IT + ii + 1, vnext);
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
          plane_st_stream(p.out + (e1 + 8 * q) * p.out_stride + p.out_off, val.x + add);
          plane_st_stream(p.out + (e2 + 8 * q) * p.out_stride + p.out_off, val.y + add);
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
  so3_fwd_plane_impl<N, kPlaneRW>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
template <int N>
__global__ void __launch_bounds__(plane_threads(kPlaneRW), 2) so3_inv_plane(const InvPlaneParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_inv_plane_impl<N, kPlaneRW>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
#define S2C_LAUNCH_PLANE(name, N, grid, stream, params)                                       \
  s2c::launch_impl(name<N>, #name, (long)(grid), s2c::plane_threads(s2c::kPlaneRW),           \
                   s2c::plane_smem_bytes(N, s2c::kPlaneRW), stream, params)
#else
#define S2C_LAUNCH_PLANE(name, N, grid, stream, params)                                       \
  s2c::emu_launch<name##_impl<N, s2c::kPlaneRW>>(                                             \
      #name, (long)(grid), s2c::plane_threads(s2c::kPlaneRW),                                 \
      s2c::plane_smem_bytes(N, s2c::kPlaneRW), params)
#endif

}  // namespace s2c
