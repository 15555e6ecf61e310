// so3_mm and its two gradients on the 5th-generation tensor cores (tcgen05.mma, accumulator in
// TMEM), 3xTF32.
//
//   z[l,m,n,i,j] = sum_{p,k} x[l,m,p,i,k] conj(y[l,n,p,k,j])            (s2cnn/so3_mm.py:8-93)
//
// is, for every degree l, ONE real GEMM on the reference's interleaved layouts:
//   C'[(m,i), (n,j,c)] = sum_{(p,k,c')} A'[(m,i),(p,k,c')] * B'[(p,k,c'),(n,j,c)]
// where A' is the x tensor read as plain floats (re, im interleaved along K - no transformation),
// C' is the z tensor written as plain floats, and B' is built from y while staging:
//   B'[(k,0),(j,0)] =  yr   B'[(k,1),(j,0)] = yi      (real part of x * conj(y))
//   B'[(k,0),(j,1)] = -yi   B'[(k,1),(j,1)] = yr      (imaginary part)
// so the complex product costs 8 real flops per complex MAC, the algorithmic count.  The two
// gradient products (s2cnn/so3_mm.py:95-122 and the backward kernels :125-261) have the same
// shape with other row / column / contraction roles; the kernel is instantiated per product.
//
// Precision: TF32 has 10 mantissa bits, not enough for the 1e-4 bar.  Every operand is split in
// float32 into hi = v truncated to TF32 and lo = v - hi and three MMAs (hi*hi, lo*hi, hi*lo)
// accumulate into the same float32 TMEM accumulator.  The tensor core's own accumulation
// truncates - a bias of up to one unit in the last place per MMA, always in the same direction,
// which adds up along the K loop.  The MMAs therefore alternate between two accumulators: every
// kTcFlushBlocks K blocks the issuer switches to the other one, and while the tensor core fills
// it the threads add the finished partial sum, rounding properly, into a third TMEM region.
//
// Tiling: one CTA per (l, 128-row tile, 128-column tile); the K loop walks the blocks (outer
// contraction index, slice of its run of floats).  Operands are staged by all 512 threads into
// shared memory in the canonical K-major, no-swizzle UMMA layout (8 rows x 16 bytes core matrices),
// double buffered; one elected thread issues tcgen05.mma and commits to an mbarrier that releases
// the stage.  The epilogue reads the accumulator with tcgen05.ld (32 lanes x 32 columns per warp
// and instruction) and stores the result directly in its interleaved layout.  Every mbarrier wait
// is bounded; on a time-out the kernel raises an error flag, frees its TMEM columns and returns.
#pragma once

#ifndef S2C_EMUL

#include <cuda_runtime.h>
#include <stdint.h>

#include "backend.h"

namespace s2c {

// The same kernel runs the forward product and its two gradients; they differ in how the rows
// of the two operands are addressed and in the sign pattern that turns complex into real
// arithmetic (the op code selects both):
//   kTcFwd    z[l,m,n,i,j]  = sum_{p,k} x[l,m,p,i,k] conj(y[l,n,p,k,j])     a = x,  b = y,  c = z
//   kTcGradX  gx[l,m,p,i,k] = sum_{n,j} gz[l,m,n,i,j] y[l,n,p,k,j]          a = gz, b = y,  c = gx
//   kTcGradY  gy[l,n,p,k,j] = sum_{m,i} conj(gz[l,m,n,i,j]) x[l,m,p,i,k]    a = x,  b = gz, c = gy
// (s2cnn/so3_mm.py:8-122).  An output row is (outer, inner) = (m, i) - or (p, k) for kTcGradY - and
// an output column (outer, 2 * inner + re/im).  The contraction index is (outer, run of `run`
// floats): a "contiguous" operand holds the run of a row as consecutive floats (16-byte loads), a
// "strided" one holds it as complex pairs `stride` floats apart (two 8-byte loads per chunk).
enum TcOp : int { kTcFwd = 0, kTcGradX = 1, kTcGradY = 2 };

struct MmTcParams {
  const float* a;   // operand read along the output rows
  const float* b;   // operand read along the output columns
  float* c;         // output
  int nl, nb, fi, fo;
  int run;          // floats per outer contraction index: 2 fi (fwd), 2 fo (grad x), 2 nb (grad y)
  int kblk;         // floats per K block (multiple of 8, <= kTcKMax)
  int nblk;         // K blocks per run
  int ksplit;       // CTAs sharing one output tile (each takes a slice of the outer contraction
                    // index and adds its partial result atomically into the zeroed output); 1 = none
  int* err;         // device flag, set to 1 on a wait time-out
};

// row / column geometry of one degree
struct TcGeom {
  int RI;           // inner extent of a row index
  int CW;           // floats per outer column index (2 * inner extent)
};
__host__ __device__ __forceinline__ TcGeom tc_geom(int op, int nb, int fi, int fo) {
  TcGeom g;
  g.RI = op == kTcGradY ? fi : nb;
  g.CW = op == kTcGradX ? 2 * fi : 2 * fo;
  return g;
}

constexpr int kTcBM = 128, kTcBN = 128;
constexpr int kTcKMax = 48;                       // floats per K block
constexpr int kTcLBO = kTcBM * 16 + 16;           // bytes between K-adjacent core matrices (padded)
constexpr int kTcSBO = 128;                       // bytes between row-adjacent core matrices
constexpr int kTcBufBytes = (kTcKMax / 4) * kTcLBO;   // one operand buffer (hi or lo)
constexpr int kTcStageBytes = 4 * kTcBufBytes;        // A hi, A lo, B hi, B lo
constexpr int kTcSmemBytes = 2 * kTcStageBytes + 64;
constexpr int kTcThreads = 512;
// K blocks accumulated by the tensor core before the partial sum is added, in FP32 with rounding,
// into the sum region (bounds the length of the tensor core's own accumulation chain, whose
// additions truncate): 4 blocks = 72 MMAs per chain.
constexpr int kTcFlushBlocks = 4;
// tensor-memory columns: two alternating accumulators and the FP32 sum region (power of two)
constexpr int kTcTmemCols = 512;
constexpr int kTcSumCol = 2 * kTcBN;

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
  // K-major, no swizzle: start >> 4 | LBO >> 4 << 16 | SBO >> 4 << 32 | version 1 << 46
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(kTcLBO >> 4) << 16;
  d |= (uint64_t)(kTcSBO >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

__device__ __forceinline__ float tc_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

__device__ __forceinline__ void tc_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc_smem_u32(bar)), "r"(count));
}

// Bounded wait on an mbarrier phase; returns false on time-out.
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = tc_smem_u32(bar);
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin > 64) __nanosleep(64);
  }
  return false;
}

__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   tc_smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_st16(uint32_t taddr, const float (&v)[16]) {
  uint32_t r[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(v[i]);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__host__ __device__ __forceinline__ long tc_tiles_for(int op, int nb, int fi, int fo, int l) {
  const TcGeom g = tc_geom(op, nb, fi, fo);
  const long L = 2 * l + 1;
  const long M = L * g.RI, N = L * g.CW;
  return ((M + kTcBM - 1) / kTcBM) * ((N + kTcBN - 1) / kTcBN);
}

// FLUSH = false drops the partial-sum code (fewer registers); valid while no degree needs more than
// kTcFlushBlocks K blocks.
// VEC = true: 16-byte loads and stores (feature counts - for grad y the batch - even); VEC = false:
// 8-byte accesses, any sizes.
template <int OP, bool FLUSH, bool VEC>
__global__ void __launch_bounds__(kTcThreads, 1) so3_mm_tc_kernel(const MmTcParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(s2c_dyn_smem);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(smem + 2 * kTcStageBytes);      // [2] stages
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 2 * kTcStageBytes + 16);
  uint64_t* flushbar = reinterpret_cast<uint64_t*>(smem + 2 * kTcStageBytes + 32);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- which tile ---------------------------------------------------------------------------
  int l = p.nl - 1;
  long t = blockIdx.x;
  for (;; --l) {
    const int sl = p.ksplit < 2 * l + 1 ? p.ksplit : 2 * l + 1;
    const long c = tc_tiles_for(OP, p.nb, p.fi, p.fo, l) * sl;
    if (t < c) break;
    t -= c;
  }
  const int L = 2 * l + 1;
  // slice of the outer contraction index handled by this CTA
  const int nsplit = p.ksplit < L ? p.ksplit : L;
  const int split = (int)(t % nsplit);
  t /= nsplit;
  const int o_lo = (int)((long)split * L / nsplit), o_hi = (int)((long)(split + 1) * L / nsplit);
  const TcGeom geo = tc_geom(OP, p.nb, p.fi, p.fo);
  const int RI = geo.RI, CW = geo.CW;
  const int M = L * RI, Np = L * CW;
  const int tiles_n = (Np + kTcBN - 1) / kTcBN;
  const int row0 = (int)(t / tiles_n) * kTcBM, col0 = (int)(t % tiles_n) * kTcBN;
  const long spec0 = (long)l * (4L * l * l - 1) / 3;
  const int fi2 = 2 * p.fi, fo2 = 2 * p.fo;
  // operand addressing (floats): offset of outer contraction index `o`, element `kf` of its run =
  //   contiguous:  o * ko + kf          strided:  o * ko + (kf / 2) * st + (kf % 2)
  constexpr bool a_str = OP == kTcGradY, b_str = OP != kTcGradX;
  long a_ko, b_ko, a_st = 0, b_st = 0;
  if (OP == kTcFwd)        { a_ko = (long)p.nb * fi2;      b_ko = (long)p.fi * fo2;      b_st = fo2; }
  else if (OP == kTcGradX) { a_ko = (long)p.nb * fo2;      b_ko = (long)L * p.fi * fo2; }
  else                       { a_ko = (long)L * p.nb * fi2;  b_ko = (long)L * p.nb * fo2;  a_st = fi2; b_st = fo2; }

  // ---- set-up: barriers, tensor memory ------------------------------------------------------
  if (tid == 0) {
    tc_mbar_init(&mbar[0], 1);
    tc_mbar_init(&mbar[1], 1);
    tc_mbar_init(flushbar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     tc_smem_u32(tmem_slot)),
                 "r"(kTcTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // instruction descriptor: D = F32, A = B = TF32, both K-major, N = 128, M = 128
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTcBN >> 3) << 17) |
                         ((uint32_t)(kTcBM >> 4) << 24);

  const int nit = (o_hi - o_lo) * p.nblk;
  bool ok = true;

  // Per-thread staging slots.  The (row, 16-byte chunk) handled by a slot and the part of its
  // global offset that does not change along K are computed once; the K loop only adds the offset
  // of block (outer index, slice of the run).  Slots are laid out for the full block width kblk;
  // chunks past the end of a shorter last slice are staged as zeros.  A contiguous operand maps
  // consecutive threads to consecutive chunks of one row (coalesced 16-byte loads), a strided one
  // to consecutive rows (neighbouring 8-byte loads).
  constexpr int kSlots = kTcBM * (kTcKMax / 4) / kTcThreads;  // 6 for A and 6 for B
  const int nchf = p.kblk / 4;                                 // chunks per full block
  long offA[kSlots], offB[kSlots];
  int soA[kSlots], soB[kSlots], chA[kSlots], chB[kSlots];
  unsigned oddB = 0;                                           // bit q: slot q stages an "imaginary" column
  float4 ra[kSlots], rb[kSlots];
#pragma unroll
  for (int q = 0; q < kSlots; ++q) {
    const int e = tid + kTcThreads * q;
    {
      int r, ch;
      if (a_str) { r = e % kTcBM; ch = e / kTcBM; } else { r = e / nchf; ch = e - r * nchf; }
      const int gr = row0 + r;
      chA[q] = (r < kTcBM && ch < nchf && gr < M) ? ch : -1;
      const int ro = gr / RI, ri = gr - ro * RI;
      long base;
      if (OP == kTcFwd)        base = ((spec0 + (long)ro * L) * p.nb + ri) * fi2;
      else if (OP == kTcGradX) base = ((spec0 + (long)ro * L) * p.nb + ri) * fo2;
      else                       base = (spec0 + ro) * p.nb * fi2 + 2 * ri;
      offA[q] = base + (a_str ? (long)(2 * ch) * a_st : 4 * ch);
      soA[q] = ch * kTcLBO + r * 16;
    }
    {
      int rr, ch;
      if (b_str) { rr = e % kTcBN; ch = e / kTcBN; } else { rr = e / nchf; ch = e - rr * nchf; }
      const int gcol = col0 + rr;
      chB[q] = (rr < kTcBN && ch < nchf && gcol < Np) ? ch : -1;
      const int co = gcol / CW, rem = gcol - co * CW;
      const int in = rem >> 1;
      if (rem & 1) oddB |= 1u << q;
      long base;
      if (OP == kTcFwd)        base = ((spec0 + (long)co * L) * p.fi * p.fo + in) * 2;
      else if (OP == kTcGradX) base = ((spec0 + co) * p.fi + in) * fo2;
      else                       base = (spec0 + co) * p.nb * fo2 + 2 * in;
      offB[q] = base + (b_str ? (long)(2 * ch) * b_st : 4 * ch);
      soB[q] = ch * kTcLBO + rr * 16;
    }
  }

  auto block_geom = [&](int it, int& oidx, int& k0, int& kvalid) {
    const int oi = it / p.nblk;
    const int kb = it - oi * p.nblk;
    oidx = o_lo + oi;
    k0 = kb * p.kblk;
    kvalid = (p.run - k0) < p.kblk ? (p.run - k0) : p.kblk;   // floats with data (even; VEC: multiple of 4)
  };
  // four consecutive K floats of one row: (re, im) of two complex numbers; `nvalid` (2 or 4) of them
  // lie inside the run
  auto load4 = [&](const float* src, bool strided, long st, int nvalid) {
    if (VEC && !strided) return __ldg(reinterpret_cast<const float4*>(src));
    const float2 u = __ldg(reinterpret_cast<const float2*>(src));
    float2 w = make_float2(0.f, 0.f);
    if (VEC || nvalid > 2) w = __ldg(reinterpret_cast<const float2*>(src + (strided ? st : 2)));
    return make_float4(u.x, u.y, w.x, w.y);
  };
  auto prefetch = [&](int it) {
    int oidx, k0, kvalid;
    block_geom(it, oidx, k0, kvalid);
    const long pa = (long)oidx * a_ko + (a_str ? (long)(k0 >> 1) * a_st : k0);
    const long pb = (long)oidx * b_ko + (b_str ? (long)(k0 >> 1) * b_st : k0);
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
      ra[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (chA[q] >= 0 && 4 * chA[q] < kvalid)
        ra[q] = load4(p.a + offA[q] + pa, a_str, a_st, kvalid - 4 * chA[q]);
      rb[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (chB[q] >= 0 && 4 * chB[q] < kvalid)
        rb[q] = load4(p.b + offB[q] + pb, b_str, b_st, kvalid - 4 * chB[q]);
    }
  };
  // v = hi + lo with hi carrying the 10 explicit TF32 mantissa bits (the tensor core ignores the
  // lower 13 bits of its inputs, so lo = v - hi needs no further rounding)
  auto split_store = [&](unsigned char* hi_buf, unsigned char* lo_buf, int so, float4 v) {
    float4 hi, lo;
    hi.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
    hi.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
    hi.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
    hi.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
    lo.x = v.x - hi.x;
    lo.y = v.y - hi.y;
    lo.z = v.z - hi.z;
    lo.w = v.w - hi.w;
    *reinterpret_cast<float4*>(hi_buf + so) = hi;
    *reinterpret_cast<float4*>(lo_buf + so) = lo;
  };
  // Real rows of the column operand, per complex number (a, b) of the run:
  //   fwd, grad y (conjugated operand):  even column (a, b)    odd column (-b, a)
  //   grad x (plain product):            even column (a, -b)   odd column ( b, a)
  constexpr bool conj_b = OP != kTcGradX;
  auto column_rows = [&](float4 v, bool odd) {
    if (conj_b) return odd ? make_float4(-v.y, v.x, -v.w, v.z) : v;
    return odd ? make_float4(v.y, v.x, v.w, v.z) : make_float4(v.x, -v.y, v.z, -v.w);
  };

  // This thread's share of an accumulator (TMEM lanes 32 (warp % 4) + lane, 32 columns).  The
  // accumulator of K-block group g is columns (g & 1) * kTcBN ...; the finished partial sum of a
  // group is added in FP32 by the threads into the sum region (columns kTcSumCol ...) while the
  // tensor core works on the next group in the other accumulator.
  constexpr int kColGroups = kTcThreads / 128;
  constexpr int kColsPerWarp = kTcBN / kColGroups;
  static_assert(kColsPerWarp == 32, "one tcgen05.ld of 32 columns per warp");
  const uint32_t tmem_mine = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) +
                             (uint32_t)(kColsPerWarp * (warp >> 2));
  bool have_sum = false, pending_flush = false;
  uint32_t flush_parity = 0;
  bool fresh = true;   // the next MMA starts a new accumulation in tensor memory

  prefetch(0);
  for (int it = 0; it < nit; ++it) {
    const int s = it & 1;
    int oidx, k0, kvalid;
    block_geom(it, oidx, k0, kvalid);
    const int ksteps = (kvalid + 7) / 8;
    unsigned char* stage = smem + (size_t)s * kTcStageBytes;
    unsigned char* Ahi = stage;
    unsigned char* Alo = stage + kTcBufBytes;
    unsigned char* Bhi = stage + 2 * kTcBufBytes;
    unsigned char* Blo = stage + 3 * kTcBufBytes;

    if (it >= 2) {  // the MMAs that read this stage two iterations ago must have finished
      if (!tc_mbar_wait(&mbar[s], (uint32_t)((it / 2 - 1) & 1))) ok = false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
      const int e = tid + kTcThreads * q;
      if (e < kTcBM * nchf) {
        split_store(Ahi, Alo, soA[q], ra[q]);
        split_store(Bhi, Blo, soB[q], column_rows(rb[q], (oddB >> q) & 1u));
      }
    }
    if (FLUSH && pending_flush) {
      if (!tc_mbar_wait(flushbar, flush_parity)) ok = false;
      flush_parity ^= 1u;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      // the group that just ended: iteration it - 1, accumulator ((it - 1) / kTcFlushBlocks) & 1
      const uint32_t done_acc = (uint32_t)((((it - 1) / kTcFlushBlocks) & 1) * kTcBN);
      for (int h = 0; h < 2; ++h) {       // 16 columns at a time keeps the transient registers low
        float v[16];
        tc_ld16(tmem_mine + done_acc + 16 * h, v);
        if (have_sum) {
          float w[16];
          tc_ld16(tmem_mine + kTcSumCol + 16 * h, w);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += w[i];
        }
        tc_st16(tmem_mine + kTcSumCol + 16 * h, v);
      }
      have_sum = true;
      // that accumulator is written again kTcFlushBlocks iterations from now, after block barriers
      // that every thread reaches only once these reads are done
    }
    if (it + 1 < nit) prefetch(it + 1);
    // make the generic-proxy writes visible to the tensor core (async proxy), then hand over
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_hi = tc_smem_u32(Ahi), a_lo = tc_smem_u32(Alo);
      const uint32_t b_hi = tc_smem_u32(Bhi), b_lo = tc_smem_u32(Blo);
      const uint32_t acc = tmem_base + (FLUSH ? (uint32_t)(((it / kTcFlushBlocks) & 1) * kTcBN) : 0u);
      for (int ks = 0; ks < ksteps; ++ks) {
        const uint32_t koff = (uint32_t)ks * 2u * kTcLBO;
        const uint64_t dah = tc_smem_desc(a_hi + koff), dal = tc_smem_desc(a_lo + koff);
        const uint64_t dbh = tc_smem_desc(b_hi + koff), dbl = tc_smem_desc(b_lo + koff);
        tc_mma_tf32(acc, dah, dbh, idesc, (fresh && ks == 0) ? 0u : 1u);
        tc_mma_tf32(acc, dal, dbh, idesc, 1u);
        tc_mma_tf32(acc, dah, dbl, idesc, 1u);
      }
      tc_commit(&mbar[s]);
    }
    // every kTcFlushBlocks blocks the issuer moves on to the other accumulator; the finished
    // partial sum is collected at the top of the next iteration, where the staging registers are free
    pending_flush = FLUSH && ((it + 1) % kTcFlushBlocks == 0) && (it + 1 < nit);
    fresh = pending_flush;
    if (pending_flush && tid == 0) tc_commit(flushbar);   // arrives when every MMA so far has finished
  }

  // ---- wait for the last commit (it covers every earlier MMA of the issuing thread) ----------
  {
    const int last = nit - 1;
    if (!tc_mbar_wait(&mbar[last & 1], (uint32_t)((last / 2) & 1))) ok = false;
    if (nit >= 2) {  // drain the other stage's barrier too so no arrival is pending at exit
      const int prev = nit - 2;
      if (!tc_mbar_wait(&mbar[prev & 1], (uint32_t)((prev / 2) & 1))) ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  ok = __syncthreads_and(ok) != 0;  // block-uniform from here on

  // ---- epilogue: TMEM -> registers -> z -----------------------------------------------------
  if (ok) {
    // warp w may only touch TMEM lanes 32 (w % 4) .. +31; the warps sharing a lane quarter split
    // the 128 accumulator columns between them
    const int q = warp & 3, cg = warp >> 2;
    const int r = row0 + 32 * q + lane;
    const int ro = r / RI, ri = r - ro * RI;
    // c[((spec0 + ro * sro + co * sco) * RI + ri) * CW + rem]
    const int sro = OP == kTcGradY ? 1 : L, sco = OP == kTcGradY ? L : 1;
#pragma unroll 1
    const uint32_t last_acc = FLUSH ? (uint32_t)((((nit - 1) / kTcFlushBlocks) & 1) * kTcBN) : 0u;
    for (int g = 0; g < kColsPerWarp / 32; ++g) {
      const int cbase = kColsPerWarp * cg + 32 * g;
      float v[32];
      tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + last_acc + (uint32_t)cbase, v);
      if (FLUSH && have_sum) {
        float w[32];
        tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(kTcSumCol + cbase), w);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += w[i];
      }
      if (r < M) {
        if constexpr (VEC) {
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            const int gcol = col0 + cbase + 4 * c4;
            if (gcol < Np) {  // CW is a multiple of 4, so a group of 4 is all in or all out
              const int co = gcol / CW, rem = gcol - co * CW;
              float* dst = p.c + ((spec0 + (long)ro * sro + (long)co * sco) * RI + ri) * CW + rem;
              if (nsplit > 1) {
#pragma unroll
                for (int u = 0; u < 4; ++u) atomicAdd(dst + u, v[4 * c4 + u]);
              } else {
                *reinterpret_cast<float4*>(dst) =
                    make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
              }
            }
          }
        } else {
#pragma unroll
          for (int c2 = 0; c2 < 16; ++c2) {
            const int gcol = col0 + cbase + 2 * c2;
            if (gcol < Np) {  // one complex number: never straddles an outer column index
              const int co = gcol / CW, rem = gcol - co * CW;
              float* dst = p.c + ((spec0 + (long)ro * sro + (long)co * sco) * RI + ri) * CW + rem;
              if (nsplit > 1) {
                atomicAdd(dst, v[2 * c2]);
                atomicAdd(dst + 1, v[2 * c2 + 1]);
              } else {
                *reinterpret_cast<float2*>(dst) = make_float2(v[2 * c2], v[2 * c2 + 1]);
              }
            }
          }
        }
      }
    }
  } else if (tid == 0) {
    atomicExch(p.err, 1);
  }

  // ---- release tensor memory ------------------------------------------------------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTcTmemCols)
                 : "memory");
  }
}

// 16-byte accesses need the run of the contraction index and the column width to be multiples of 4
// floats: fwd and grad x: f_in and f_out even; grad y: batch and f_out even.  Other sizes take the
// 8-byte variant.
inline bool so3_mm_tc_vec16(int op, int nb, int fi, int fo) {
  if (op == kTcGradY) return (nb % 2 == 0) && (fo % 2 == 0);
  return (fi % 2 == 0) && (fo % 2 == 0);
}

inline long so3_mm_tc_tiles(int op, int nl, int nb, int fi, int fo, int ksplit = 1) {
  long t = 0;
  for (int l = 0; l < nl; ++l)
    t += tc_tiles_for(op, nb, fi, fo, l) * (ksplit < 2 * l + 1 ? ksplit : 2 * l + 1);
  return t;
}

}  // namespace s2c

#endif  // S2C_EMUL
