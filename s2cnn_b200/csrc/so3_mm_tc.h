// so3_mm forward on the 5th-generation tensor cores (tcgen05.mma, accumulator in TMEM), 3xTF32.
//
//   z[l,m,n,i,j] = sum_{p,k} x[l,m,p,i,k] conj(y[l,n,p,k,j])            (s2cnn/so3_mm.py:8-93)
//
// is, for every degree l, ONE real GEMM on the reference's interleaved layouts:
//   C'[(m,i), (n,j,c)] = sum_{(p,k,c')} A'[(m,i),(p,k,c')] * B'[(p,k,c'),(n,j,c)]
// where A' is the x tensor read as plain floats (re, im interleaved along K - no transformation),
// C' is the z tensor written as plain floats, and B' is built from y while staging:
//   B'[(k,0),(j,0)] =  yr   B'[(k,1),(j,0)] = yi      (real part of x * conj(y))
//   B'[(k,0),(j,1)] = -yi   B'[(k,1),(j,1)] = yr      (imaginary part)
// so the complex product costs 8 real flops per complex MAC, the algorithmic count.
//
// Precision: TF32 has 10 mantissa bits, not enough for the 1e-4 bar.  Every operand is split in
// float32 into hi = v truncated to TF32 and lo = v - hi and three MMAs (hi*hi, lo*hi, hi*lo) accumulate into
// the same float32 TMEM accumulator, which restores float32-level accuracy.
//
// Tiling: one CTA per (l, 128-row tile, 128-column tile); the K loop walks the blocks (p, slice of
// the 2*f_in floats).  Operands are staged by all 256 threads into shared memory in the canonical
// K-major, no-swizzle UMMA layout (8 rows x 16 bytes core matrices), double buffered; one elected
// thread issues tcgen05.mma and commits to an mbarrier that releases the stage.  The epilogue reads
// the accumulator with tcgen05.ld (32 lanes x 32 columns per warp and instruction) and stores z
// directly in its interleaved layout.  Every mbarrier wait is bounded; on a time-out the kernel
// raises an error flag, frees its TMEM columns and returns.
#pragma once

#ifndef S2C_EMUL

#include <cuda_runtime.h>
#include <stdint.h>

#include "backend.h"

namespace s2c {

struct MmTcParams {
  const float* x;   // [nspec, nb, fi, 2]
  const float* y;   // [nspec, fi, fo, 2]
  float* z;         // [nspec, nb, fo, 2]
  int nl, nb, fi, fo;
  int kblk;         // floats per K block (multiple of 8, <= kTcKMax)
  int nblk;         // K blocks per p
  int* err;         // device flag, set to 1 on a wait time-out
};

constexpr int kTcBM = 128, kTcBN = 128;
constexpr int kTcKMax = 48;                       // floats per K block
constexpr int kTcLBO = kTcBM * 16 + 16;           // bytes between K-adjacent core matrices (padded)
constexpr int kTcSBO = 128;                       // bytes between row-adjacent core matrices
constexpr int kTcBufBytes = (kTcKMax / 4) * kTcLBO;   // one operand buffer (hi or lo)
constexpr int kTcStageBytes = 4 * kTcBufBytes;        // A hi, A lo, B hi, B lo
constexpr int kTcSmemBytes = 2 * kTcStageBytes + 64;
constexpr int kTcThreads = 512;

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

__device__ __forceinline__ long tc_tiles_for(const MmTcParams& p, int l) {
  const long L = 2 * l + 1;
  const long M = L * p.nb, N = L * p.fo * 2;
  return ((M + kTcBM - 1) / kTcBM) * ((N + kTcBN - 1) / kTcBN);
}

__global__ void __launch_bounds__(kTcThreads, 1) so3_mm_tc_kernel(const MmTcParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(s2c_dyn_smem);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(smem + 2 * kTcStageBytes);      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 2 * kTcStageBytes + 16);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- which tile ---------------------------------------------------------------------------
  int l = p.nl - 1;
  long t = blockIdx.x;
  for (;; --l) {
    const long c = tc_tiles_for(p, l);
    if (t < c) break;
    t -= c;
  }
  const int L = 2 * l + 1;
  const int M = L * p.nb, Np = L * p.fo * 2;
  const int tiles_n = (Np + kTcBN - 1) / kTcBN;
  const int row0 = (int)(t / tiles_n) * kTcBM, col0 = (int)(t % tiles_n) * kTcBN;
  const long spec0 = (long)l * (4L * l * l - 1) / 3;
  const int fi2 = 2 * p.fi, fo2 = 2 * p.fo;

  // ---- set-up: barriers, tensor memory ------------------------------------------------------
  if (tid == 0) {
    tc_mbar_init(&mbar[0], 1);
    tc_mbar_init(&mbar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     tc_smem_u32(tmem_slot)),
                 "r"(kTcBN)
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

  const int nit = L * p.nblk;
  bool ok = true;

  // Per-thread staging slots.  The (row, 16-byte chunk) handled by a slot and the part of its
  // global offset that does not change along K are computed once; the K loop only adds the offset
  // of block (p, slice).  Slots are laid out for the full block width kblk; chunks past the end of
  // a shorter last slice are staged as zeros.
  constexpr int kSlots = kTcBM * (kTcKMax / 4) / kTcThreads;  // 6 for A and 6 for B
  const int nchf = p.kblk / 4;                                 // chunks per full block
  long offA[kSlots], offB[kSlots];
  int soA[kSlots], soB[kSlots], chA[kSlots], kqB[kSlots];
  float4 ra[kSlots];
  float2 rb0[kSlots], rb1[kSlots];
#pragma unroll
  for (int q = 0; q < kSlots; ++q) {
    const int e = tid + kTcThreads * q;
    {  // A: consecutive threads -> consecutive chunks of one row (coalesced 16-byte loads)
      const int r = e / nchf, ch = e - r * nchf;
      const int gr = row0 + r;
      chA[q] = (r < kTcBM && gr < M) ? ch : -1;
      const int m = gr / p.nb, i = gr - m * p.nb;
      offA[q] = (((spec0 + (long)m * L) * p.nb + i) * fi2) + 4 * ch;
      soA[q] = ch * kTcLBO + r * 16;
    }
    {  // B': consecutive threads -> consecutive rows (n, j, c); each stages one 16-byte chunk
      const int rr = e % kTcBN, kq = e / kTcBN;
      const int gcol = col0 + rr;
      kqB[q] = (kq < nchf && gcol < Np) ? kq : -1;
      const int n = gcol / fo2, j = (gcol - n * fo2) >> 1;
      offB[q] = ((spec0 + (long)n * L) * p.fi * p.fo + j) * 2;
      soB[q] = kq * kTcLBO + rr * 16;
    }
  }
  const bool imag_row = (tid & 1) != 0;  // rr and tid have the same parity (kTcThreads, kTcBN even)

  auto block_geom = [&](int it, int& pidx, int& k0, int& kvalid) {
    pidx = it / p.nblk;
    const int kb = it - pidx * p.nblk;
    k0 = kb * p.kblk;
    kvalid = (fi2 - k0) < p.kblk ? (fi2 - k0) : p.kblk;   // floats with data (multiple of 4)
  };
  auto prefetch = [&](int it) {
    int pidx, k0, kvalid;
    block_geom(it, pidx, k0, kvalid);
    const long pa = (long)pidx * p.nb * fi2 + k0;
    const long pb = ((long)pidx * p.fi + (k0 >> 1)) * p.fo * 2;
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
      ra[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (chA[q] >= 0 && 4 * chA[q] < kvalid)
        ra[q] = __ldg(reinterpret_cast<const float4*>(p.x + offA[q] + pa));
      rb0[q] = make_float2(0.f, 0.f);
      rb1[q] = make_float2(0.f, 0.f);
      if (kqB[q] >= 0 && 4 * kqB[q] < kvalid) {  // complex k = 2 kq and 2 kq + 1 of this block
        const float* src = p.y + offB[q] + pb + (long)(2 * kqB[q]) * p.fo * 2;
        rb0[q] = __ldg(reinterpret_cast<const float2*>(src));
        rb1[q] = __ldg(reinterpret_cast<const float2*>(src + p.fo * 2));
      }
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

  prefetch(0);
  for (int it = 0; it < nit; ++it) {
    const int s = it & 1;
    int pidx, k0, kvalid;
    block_geom(it, pidx, k0, kvalid);
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
      if (e < kTcBM * nchf) split_store(Ahi, Alo, soA[q], ra[q]);
      if (e < kTcBN * nchf) {
        // row (j,0) = (yr, yi) per complex k;  row (j,1) = (-yi, yr)   [x * conj(y)]
        const float2 a = rb0[q], b = rb1[q];
        const float4 v = imag_row ? make_float4(-a.y, a.x, -b.y, b.x)
                                  : make_float4(a.x, a.y, b.x, b.y);
        split_store(Bhi, Blo, soB[q], v);
      }
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
      for (int ks = 0; ks < ksteps; ++ks) {
        const uint32_t koff = (uint32_t)ks * 2u * kTcLBO;
        const uint64_t dah = tc_smem_desc(a_hi + koff), dal = tc_smem_desc(a_lo + koff);
        const uint64_t dbh = tc_smem_desc(b_hi + koff), dbl = tc_smem_desc(b_lo + koff);
        tc_mma_tf32(tmem_base, dah, dbh, idesc, (it > 0 || ks > 0) ? 1u : 0u);
        tc_mma_tf32(tmem_base, dal, dbh, idesc, 1u);
        tc_mma_tf32(tmem_base, dah, dbl, idesc, 1u);
      }
      tc_commit(&mbar[s]);
    }
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
    constexpr int kColGroups = kTcThreads / 128;
    constexpr int kColsPerWarp = kTcBN / kColGroups;
    const int q = warp & 3, cg = warp >> 2;
    const int r = row0 + 32 * q + lane;
    const int m = r / p.nb, i = r - m * p.nb;
#pragma unroll 1
    for (int g = 0; g < kColsPerWarp / 32; ++g) {
      const int cbase = kColsPerWarp * cg + 32 * g;
      float v[32];
      tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)cbase, v);
      if (r < M) {
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const int gcol = col0 + cbase + 4 * c4;
          if (gcol < Np) {  // Np is a multiple of 4, so a group of 4 is all in or all out
            const int n = gcol / fo2, rem = gcol - n * fo2;
            float* dst = p.z + ((spec0 + (long)m * L + n) * p.nb + i) * fo2 + rem;
            *reinterpret_cast<float4*>(dst) =
                make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
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
                 "r"(kTcBN)
                 : "memory");
  }
}

inline bool so3_mm_tc_supported(int nl, int nb, int fi, int fo) {
  (void)nl;
  (void)nb;
  return (fi % 2 == 0) && (fo % 2 == 0);
}

inline long so3_mm_tc_tiles(int nl, int nb, int fo) {
  long t = 0;
  for (int l = 0; l < nl; ++l) {
    const long L = 2 * l + 1;
    t += ((L * nb + kTcBM - 1) / kTcBM) * ((L * fo * 2 + kTcBN - 1) / kTcBN);
  }
  return t;
}

}  // namespace s2c

#endif  // S2C_EMUL
