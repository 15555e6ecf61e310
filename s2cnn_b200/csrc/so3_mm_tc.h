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
// Tiling: one CTA per (l, 128-row tile, 128-column tile); the K loop walks blocks of at most
// kTcKMax floats (outer contraction index, slice of its run of floats).  The CTA is warp
// specialised (17 warps):
//   * 12 producer warps read the two operands from global memory (register prefetch one block
//     ahead), split them into hi / lo TF32 parts and stage them in shared memory in the canonical
//     K-major, no-swizzle UMMA layout (8 rows x 16 bytes core matrices), kTcStages stages deep; a
//     warp arrives on the stage's "full" mbarrier once its lanes have written their share;
//   * one issuer warp waits for "full", issues the nine tcgen05.mma of the block (hi*hi, lo*hi,
//     hi*lo for each k-step of 8) from one elected lane and commits them to the stage's "empty"
//     mbarrier, which lets the producers overwrite the stage; it alternates between two accumulators
//     in tensor memory every kTcFlushBlocks blocks and commits to an "accumulator done" mbarrier;
//   * 4 collector warps (one per TMEM lane quarter) add each finished accumulator, with proper
//     rounding, into a third tensor-memory region and hand the accumulator back ("accumulator
//     free") - all of it while the tensor core fills the other one.
// The epilogue (all 16 non-issuer warps) reads the last accumulator and the sum region with
// tcgen05.ld (32 lanes x 32 columns per warp and instruction) and stores the result directly in
// its interleaved layout.  Every mbarrier wait is bounded; on a time-out the waiting thread raises a
// block-wide abort flag, every role leaves its loop, the kernel raises the error flag, frees its
// TMEM columns and returns.
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
//   kTcPlainCC / kTcPlainSC: a plain real product C[r][c] = sum_k A[r][k] B[c][k] on the same
//   pipeline, with explicit strides (rows, pairs of consecutive k, pairs of consecutive c) instead
//   of the spectral geometry: the kernel-grid -> spectrum transforms s2_rft / so3_rft and their
//   transposes (s2cnn/s2_ft.py:22, s2cnn/so3_ft.py:22).  CC: both operands hold k contiguously;
//   SC: the row operand holds k as pairs `a_ps` floats apart.
enum TcOp : int { kTcFwd = 0, kTcGradX = 1, kTcGradY = 2, kTcPlainCC = 3, kTcPlainSC = 4 };

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
  // plain products only (floats): element (row r, k) of a at r * a_rs + (k / 2) * a_ps + k % 2,
  // element (column c, k) of b likewise, element (r, c) of the result at r * c_rs + (c / 2) * c_ps + c % 2;
  // nb = rows, fi = K / 2, fo = columns / 2, nl = 1
  long a_rs, a_ps, b_rs, b_ps, c_rs, c_ps;
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
constexpr int kTcKMax = 24;                       // floats per K block
constexpr int kTcStages = 4;
constexpr int kTcLBO = kTcBM * 16 + 64;           // bytes between K-adjacent core matrices (padded)
constexpr int kTcSBO = 128;                       // bytes between row-adjacent core matrices
constexpr int kTcBufBytes = (kTcKMax / 4) * kTcLBO;   // one operand buffer (hi or lo)
constexpr int kTcStageBytes = 4 * kTcBufBytes;        // A hi, A lo, B hi, B lo
constexpr int kTcSmemBytes = kTcStages * kTcStageBytes + 256;   // + mbarriers, TMEM slot, abort flag
constexpr int kTcProducerWarps = 12, kTcCollectorWarps = 4;
constexpr int kTcProducers = 32 * kTcProducerWarps;
constexpr int kTcFirstProducer = 32 * (1 + kTcCollectorWarps);  // thread index of the first producer
constexpr int kTcThreads = 32 * (1 + kTcCollectorWarps + kTcProducerWarps);
// K blocks accumulated by the tensor core before the partial sum is added, in FP32 with rounding,
// into the sum region (bounds the length of the tensor core's own accumulation chain, whose
// additions truncate): 8 blocks = 72 MMAs per chain.
constexpr int kTcFlushBlocks = 8;
// longest chain (in MMAs) left to the tensor core's own accumulation without partial sums: its
// truncation bias stays below about 1e-5 relative
constexpr int kTcChainMax = 200;
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

// Staging slot e of a contiguous operand -> (row, 16-byte chunk of the K block): groups of 8 slots
// cover 4 rows x 2 adjacent chunks, consecutive groups the chunk pairs of the same 4 rows (nchf,
// the chunks per block, is even).
__device__ __forceinline__ void tc_slot_contiguous(int e, int nchf, int& r, int& ch) {
  const int g = e >> 3, u = e & 7, npair = nchf >> 1;
  const int rq = g / npair, cp = g - rq * npair;
  r = 4 * rq + (u >> 1);
  ch = 2 * cp + (u & 1);
}

__host__ __device__ __forceinline__ long tc_tiles_for(int op, int nb, int fi, int fo, int l) {
  const TcGeom g = tc_geom(op, nb, fi, fo);
  const long L = 2 * l + 1;
  const long M = L * g.RI, N = L * g.CW;
  return ((M + kTcBM - 1) / kTcBM) * ((N + kTcBN - 1) / kTcBN);
}

// FLUSH = false keeps the whole chain in one tensor-memory accumulator and drops the partial-sum
// code; the host selects it while no CTA issues more than kTcChainMax MMAs.
// VEC = true: 16-byte loads and stores (feature counts - for grad y the batch - even); VEC = false:
// 8-byte accesses, any sizes.
template <int OP, bool FLUSH, bool VEC>
__global__ void __launch_bounds__(kTcThreads, 1) so3_mm_tc_kernel(const MmTcParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(s2c_dyn_smem);
  unsigned char* ctl = smem + kTcStages * kTcStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctl);                 // [stages] producers -> issuer
  uint64_t* empty = full + kTcStages;                                // [stages] tensor core -> producers
  uint64_t* accdone = empty + kTcStages;                             // [2] tensor core -> collectors
  uint64_t* accfree = accdone + 2;                                   // [2] collectors -> issuer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfree + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
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
  const int nit = (o_hi - o_lo) * p.nblk;                 // K blocks of this CTA
  // accumulator groups (one when the whole chain stays in the tensor core's accumulator)
  const int ngroups = FLUSH ? (nit + kTcFlushBlocks - 1) / kTcFlushBlocks : 1;

  // ---- set-up: barriers, tensor memory ------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < kTcStages; ++i) {
      tc_mbar_init(&full[i], kTcProducerWarps);
      tc_mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc_mbar_init(&accdone[i], 1);
      tc_mbar_init(&accfree[i], kTcCollectorWarps);
    }
    *abort_flag = 0;
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

  bool ok = true;
  // a wait that gives up tells every role to leave its loop
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (tc_mbar_wait(bar, parity)) return true;
    *abort_flag = 1;
    ok = false;
    return false;
  };

  if (warp == 0) {
    // ================================ issuer ====================================================
    // instruction descriptor: D = F32, A = B = TF32, both K-major, N = 128, M = 128
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTcBN >> 3) << 17) |
                           ((uint32_t)(kTcBM >> 4) << 24);
    // The operand descriptors of every (stage, buffer, k-step) differ from the one of stage 0,
    // A hi, k-step 0 only in the 14-bit start-address field (bytes >> 4), so they are obtained by
    // adding constants (the whole staging area is below 256 KB, the field cannot overflow).
    const uint64_t d0 = tc_smem_desc(tc_smem_u32(smem));
    constexpr uint64_t kDBuf = kTcBufBytes >> 4, kDStage = kTcStageBytes >> 4, kDStep = (2u * kTcLBO) >> 4;
    constexpr int kStepsMax = kTcKMax / 8;
    const int steps_full = (p.kblk + 7) / 8;
    const int steps_tail = (p.run - (p.nblk - 1) * p.kblk + 7) / 8;
    int kb = 0, s = 0, g = 0, ing = 0;           // block within its run, stage, group, block within its group
    uint32_t full_par = 0;                        // parity of the `full` phase of the current round of stages
    for (int it = 0; it < nit && !*abort_flag; ++it) {
      if (FLUSH && ing == 0 && g >= 2)            // the collectors are done with this accumulator
        if (!wait(&accfree[g & 1], (uint32_t)((g / 2 - 1) & 1))) break;
      if (!wait(&full[s], full_par)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const int ksteps = kb + 1 == p.nblk ? steps_tail : steps_full;
        const uint64_t da = d0 + (uint64_t)s * kDStage;
        const uint32_t acc = tmem_base + (FLUSH ? (uint32_t)((g & 1) * kTcBN) : 0u);
#pragma unroll
        for (int ks = 0; ks < kStepsMax; ++ks) {
          if (ks < ksteps) {
            const uint64_t dah = da + ks * kDStep, dal = dah + kDBuf;
            const uint64_t dbh = dah + 2 * kDBuf, dbl = dah + 3 * kDBuf;
            tc_mma_tf32(acc, dah, dbh, idesc, ((FLUSH ? ing == 0 : it == 0) && ks == 0) ? 0u : 1u);
            tc_mma_tf32(acc, dal, dbh, idesc, 1u);
            tc_mma_tf32(acc, dah, dbl, idesc, 1u);
          }
        }
        tc_commit(&empty[s]);     // arrives when these MMAs have read the stage
        if ((FLUSH && ing + 1 == kTcFlushBlocks) || it + 1 == nit) tc_commit(&accdone[g & 1]);
      }
      __syncwarp();
      if (++kb == p.nblk) kb = 0;
      if (++s == kTcStages) { s = 0; full_par ^= 1u; }
      if (FLUSH && ++ing == kTcFlushBlocks) { ing = 0; ++g; }
    }
  } else if (warp <= kTcCollectorWarps) {
    // ================================ collectors ================================================
    // This warp's TMEM lane quarter, all 128 columns: every finished accumulator but the last is
    // added into the sum region while the tensor core fills the other accumulator.
    if (FLUSH) {
      const uint32_t lanes = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
      for (int g = 0; g + 1 < ngroups && !*abort_flag; ++g) {
        if (!wait(&accdone[g & 1], (uint32_t)((g / 2) & 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int h = 0; h < kTcBN / 16; ++h) {   // 16 columns at a time keeps the registers low
          float v[16];
          tc_ld16(lanes + (uint32_t)((g & 1) * kTcBN + 16 * h), v);
          if (g > 0) {
            float w[16];
            tc_ld16(lanes + (uint32_t)(kTcSumCol + 16 * h), w);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] += w[i];
          }
          tc_st16(lanes + (uint32_t)(kTcSumCol + 16 * h), v);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(&accfree[g & 1]))
                       : "memory");
      }
    }
  } else {
    // ================================ producers =================================================
    const int pt = tid - kTcFirstProducer;
    // operand addressing (floats): offset of outer contraction index `o`, element `kf` of its run =
    //   contiguous:  o * ko + kf          strided:  o * ko + (kf / 2) * st + (kf % 2)
    constexpr bool plain = OP == kTcPlainCC || OP == kTcPlainSC;
    constexpr bool a_str = OP == kTcGradY || OP == kTcPlainSC, b_str = OP == kTcFwd || OP == kTcGradY;
    long a_ko, b_ko, a_st = 0, b_st = 0;
    if (OP == kTcFwd)        { a_ko = (long)p.nb * fi2;      b_ko = (long)p.fi * fo2;      b_st = fo2; }
    else if (OP == kTcGradX) { a_ko = (long)p.nb * fo2;      b_ko = (long)L * p.fi * fo2; }
    else if (OP == kTcGradY) { a_ko = (long)L * p.nb * fi2;  b_ko = (long)L * p.nb * fo2;  a_st = fi2; b_st = fo2; }
    else                       { a_ko = 0; b_ko = 0; a_st = p.a_ps; b_st = p.b_ps; }   // one outer index

    // Per-thread staging slots.  Everything that does not change along K is computed once per
    // slot: the global address of its 16-byte chunk in K block 0 (null for a row, column or chunk
    // outside the problem), its place in a stage buffer, whether it lies inside the shorter last
    // block of a run, and for the column operand whether it builds an "imaginary" column.  The K
    // loop then only adds one running offset per operand (advanced by a constant per block and by
    // another per outer index - no division, no per-slot geometry).  A strided operand maps
    // consecutive threads to consecutive rows of one chunk (neighbouring 8-byte loads; 32 lanes store
    // 512 contiguous bytes).  A contiguous operand maps every 8 consecutive threads to 4 rows x 2
    // adjacent chunks: each row's two chunks are one 32-byte sector of global memory, consecutive
    // groups of 8 walk along the same rows, and with chunk columns 128 * 16 + 64 bytes apart the 8
    // 16-byte stores of a quarter warp fall into 8 different bank groups.
    constexpr int kSlots = kTcBM * (kTcKMax / 4) / kTcProducers;  // 2 for A and 2 for B
    static_assert(kSlots * kTcProducers == kTcBM * (kTcKMax / 4), "slots per producer");
    float4 ra0[kSlots], rb0[kSlots], ra1[kSlots], rb1[kSlots];   // two K blocks in flight
    const int nchf = p.kblk / 4;                                 // chunks per full block
    const int tail = p.run - (p.nblk - 1) * p.kblk;              // floats of a run's last block (even; VEC: multiple of 4)
    const float* gA[kSlots];
    const float* gB[kSlots];
    int soA[kSlots], soB[kSlots];
    unsigned tailA = 0, tailB = 0;        // bit q: slot q has data in the last block of a run ...
    unsigned tailA2 = 0, tailB2 = 0;      // ... but only its first complex number (8-byte variant)
    unsigned oddB = 0;                    // bit q: slot q stages an "imaginary" column
    unsigned live = 0;                    // bit q: slot q is written at all (zeros if its pointer is null)
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
      const int e = pt + kTcProducers * q;
      if (e < kTcBM * nchf) live |= 1u << q;
      {
        int r, ch;
        if (a_str) { r = e % kTcBM; ch = e / kTcBM; } else { tc_slot_contiguous(e, nchf, r, ch); }
        const int gr = row0 + r;
        const bool okA = r < kTcBM && ch < nchf && gr < M;
        const int ro = gr / RI, ri = gr - ro * RI;
        long base;
        if (OP == kTcFwd)        base = ((spec0 + (long)ro * L) * p.nb + ri) * fi2;
        else if (OP == kTcGradX) base = ((spec0 + (long)ro * L) * p.nb + ri) * fo2;
        else if (OP == kTcGradY) base = (spec0 + ro) * p.nb * fi2 + 2 * ri;
        else                       base = (long)gr * p.a_rs;
        base += (long)o_lo * a_ko + (a_str ? (long)(2 * ch) * a_st : 4 * ch);
        gA[q] = okA ? p.a + base : nullptr;
        soA[q] = ch * kTcLBO + r * 16;
        if (4 * ch < tail) tailA |= 1u << q;
        if (tail - 4 * ch == 2) tailA2 |= 1u << q;
      }
      {
        int rr, ch;
        if (b_str) { rr = e % kTcBN; ch = e / kTcBN; } else { tc_slot_contiguous(e, nchf, rr, ch); }
        const int gcol = col0 + rr;
        const bool okB = rr < kTcBN && ch < nchf && gcol < Np;
        const int co = gcol / CW, rem = gcol - co * CW;
        const int in = rem >> 1;
        if (rem & 1) oddB |= 1u << q;
        long base;
        if (OP == kTcFwd)        base = ((spec0 + (long)co * L) * p.fi * p.fo + in) * 2;
        else if (OP == kTcGradX) base = ((spec0 + co) * p.fi + in) * fo2;
        else if (OP == kTcGradY) base = (spec0 + co) * p.nb * fo2 + 2 * in;
        else                       base = (long)gcol * p.b_rs;
        base += (long)o_lo * b_ko + (b_str ? (long)(2 * ch) * b_st : 4 * ch);
        gB[q] = okB ? p.b + base : nullptr;
        soB[q] = ch * kTcLBO + rr * 16;
        if (4 * ch < tail) tailB |= 1u << q;
        if (tail - 4 * ch == 2) tailB2 |= 1u << q;
      }
    }
    // offsets (floats) from K block 0 to the next block of a run / to block 0 of the next outer index
    const long a_stepk = a_str ? (long)(p.kblk >> 1) * a_st : p.kblk;
    const long b_stepk = b_str ? (long)(p.kblk >> 1) * b_st : p.kblk;
    const long a_stepo = a_ko - (long)(p.nblk - 1) * a_stepk;
    const long b_stepo = b_ko - (long)(p.nblk - 1) * b_stepk;

    // four consecutive K floats of one row: (re, im) of two complex numbers
    auto load4 = [&](const float* src, bool strided, long st, bool only_first) {
      if (VEC && !strided) return __ldg(reinterpret_cast<const float4*>(src));
      const float2 u = __ldg(reinterpret_cast<const float2*>(src));
      float2 w = make_float2(0.f, 0.f);
      if (VEC || !only_first) w = __ldg(reinterpret_cast<const float2*>(src + (strided ? st : 2)));
      return make_float4(u.x, u.y, w.x, w.y);
    };
    // the cursor of the loads runs two K blocks ahead of the one being staged
    long cur_a = 0, cur_b = 0;
    int cur_kb = 0;
    unsigned validA = 0, validB = 0;      // bit q: slot q has a source address at all
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
      if (gA[q]) validA |= 1u << q;
      if (gB[q]) validB |= 1u << q;
    }
    auto prefetch = [&](float4 (&ra)[kSlots], float4 (&rb)[kSlots]) {
      const bool last = cur_kb + 1 == p.nblk;
      if (!last) {
        // a full block: every slot that has a source is loaded; the others hold the zeros they were
        // given before the loop (or by the last block of the previous run)
#pragma unroll
        for (int q = 0; q < kSlots; ++q) {
          if ((validA >> q) & 1u) ra[q] = load4(gA[q] + cur_a, a_str, a_st, false);
          if ((validB >> q) & 1u) rb[q] = load4(gB[q] + cur_b, b_str, b_st, false);
        }
        ++cur_kb; cur_a += a_stepk; cur_b += b_stepk;
        return;
      }
#pragma unroll
      for (int q = 0; q < kSlots; ++q) {
        ra[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (((validA & tailA) >> q) & 1u)
          ra[q] = load4(gA[q] + cur_a, a_str, a_st, (tailA2 >> q) & 1u);
        rb[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (((validB & tailB) >> q) & 1u)
          rb[q] = load4(gB[q] + cur_b, b_str, b_st, (tailB2 >> q) & 1u);
      }
      cur_kb = 0; cur_a += a_stepo; cur_b += b_stepo;
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
      if (plain) return v;
      if (conj_b) return odd ? make_float4(-v.y, v.x, -v.w, v.z) : v;
      return odd ? make_float4(v.y, v.x, v.w, v.z) : make_float4(v.x, -v.y, v.z, -v.w);
    };

    // stage K block `it` from the registers that hold it, then refill them with block it + 2
    auto stage_block = [&](int it, float4 (&ra)[kSlots], float4 (&rb)[kSlots]) {
      const int s = it % kTcStages;
      unsigned char* stage = smem + (size_t)s * kTcStageBytes;
      if (it >= kTcStages) {  // the MMAs that read this stage kTcStages blocks ago must have finished
        if (!wait(&empty[s], (uint32_t)((it / kTcStages - 1) & 1))) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
#pragma unroll
      for (int q = 0; q < kSlots; ++q) {
        if ((live >> q) & 1u) {
          split_store(stage, stage + kTcBufBytes, soA[q], ra[q]);
          split_store(stage + 2 * kTcBufBytes, stage + 3 * kTcBufBytes, soB[q],
                      column_rows(rb[q], (oddB >> q) & 1u));
        }
      }
      if (it + 2 < nit) prefetch(ra, rb);
      // make the generic-proxy writes visible to the tensor core (async proxy), then hand over:
      // one arrival per producer warp
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(&full[s])) : "memory");
      return true;
    };
#pragma unroll
    for (int q = 0; q < kSlots; ++q)
      ra0[q] = rb0[q] = ra1[q] = rb1[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    prefetch(ra0, rb0);
    if (nit > 1) prefetch(ra1, rb1);
    for (int it = 0; it < nit && !*abort_flag; it += 2) {
      if (!stage_block(it, ra0, rb0)) break;
      if (it + 1 < nit && !stage_block(it + 1, ra1, rb1)) break;
    }
  }

  // ---- every MMA of this CTA has finished once the last accumulator group has been committed ----
  // (waited for by the collectors, which have followed every earlier phase of these barriers; the
  // block barrier below passes the fact on to the other warps)
  __syncwarp();
  if (warp >= 1 && warp <= kTcCollectorWarps && !*abort_flag) {
    const int glast = ngroups - 1;
    wait(&accdone[glast & 1], (uint32_t)((glast / 2) & 1));
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  ok = __syncthreads_and(ok && !*abort_flag) != 0;  // block-uniform from here on
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // ---- epilogue: TMEM -> registers -> z -----------------------------------------------------
  if (ok && warp != 0) {
    // warp w may only touch TMEM lanes 32 (w % 4) .. +31; the four warps sharing a lane quarter
    // split the 128 accumulator columns between them
    constexpr int kColsPerWarp = kTcBN / 4;
    static_assert(kColsPerWarp == 32, "one tcgen05.ld of 32 columns per warp");
    const int q = warp & 3, cg = (warp - 1) >> 2;
    const int r = row0 + 32 * q + lane;
    const int ro = r / RI, ri = r - ro * RI;
    // c[((spec0 + ro * sro + co * sco) * RI + ri) * CW + rem]
    const int sro = OP == kTcGradY ? 1 : L, sco = OP == kTcGradY ? L : 1;
    const uint32_t last_acc = FLUSH ? (uint32_t)(((ngroups - 1) & 1) * kTcBN) : 0u;
    const int cbase = kColsPerWarp * cg;
    float v[32];
    tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + last_acc + (uint32_t)cbase, v);
    if (FLUSH && ngroups > 1) {
      float w[32];
      tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(kTcSumCol + cbase), w);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += w[i];
    }
    if (r < M && (OP == kTcPlainCC || OP == kTcPlainSC)) {
#pragma unroll
      for (int c2 = 0; c2 < 16; ++c2) {
        const int gcol = col0 + cbase + 2 * c2;
        if (gcol < Np)
          *reinterpret_cast<float2*>(p.c + (long)r * p.c_rs + (long)(gcol >> 1) * p.c_ps) =
              make_float2(v[2 * c2], v[2 * c2 + 1]);
      }
    } else if (r < M) {
      if (VEC && nsplit == 1 && CW % 8 == 0 && reinterpret_cast<unsigned long long>(p.c) % 32 == 0) {
        // a lane owns a row: 32-byte stores write whole sectors (16-byte ones would send every
        // sector to L2 in two halves); CW % 8 == 0 keeps a group of 8 inside one outer column index
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          const int gcol = col0 + cbase + 8 * c8;
          if (gcol < Np) {
            const int co = gcol / CW, rem = gcol - co * CW;
            float* dst = p.c + ((spec0 + (long)ro * sro + (long)co * sco) * RI + ri) * CW + rem;
            float8 o;
            o.lo = make_float4(v[8 * c8], v[8 * c8 + 1], v[8 * c8 + 2], v[8 * c8 + 3]);
            o.hi = make_float4(v[8 * c8 + 4], v[8 * c8 + 5], v[8 * c8 + 6], v[8 * c8 + 7]);
            st_global_256(dst, o);
          }
        }
      } else if constexpr (VEC) {
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
  } else if (!ok && tid == 0) {
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
