// Backend layer: one kernel source, two ways to run it.
//
//  * default (nvcc, sm_100a): kernels are __global__ functions launched on a CUDA stream.
//  * -DS2C_EMUL (g++, test-only): every CUDA thread of a block becomes a user-level fiber on
//    the host and __syncthreads() becomes a fiber barrier, so the same kernel bodies, index
//    arithmetic, dispatch code and table builders can be checked on a machine without a GPU.
//    The emulation library is built and loaded by the test-suite only; the shipped Python
//    package never loads it.
//
// A kernel is written once as
//
//     S2C_KERNEL(my_kernel, MyParams) { ... ctx.tid / ctx.nthr / ctx.bid / ctx.sync() ... }
//
// and launched with S2C_LAUNCH(my_kernel, grid, block, smem_bytes, stream, params).
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <mutex>
#include <string>
#include <vector>

namespace s2c {

// Thread-local last error text, returned by s2c_last_error().
inline std::string& last_error_ref() {
  static thread_local std::string e;
  return e;
}
inline int fail(int code, const std::string& msg) {
  last_error_ref() = msg;
  return code;
}

enum Status : int {
  S2C_OK = 0,
  S2C_ERR_BAD_ARG = 1,
  S2C_ERR_CUDA = 2,
  S2C_ERR_WORKSPACE = 3,
  S2C_ERR_UNSUPPORTED = 4,
};

}  // namespace s2c

#ifndef S2C_EMUL
// ------------------------------------------------------------------------------------------
// CUDA backend
// ------------------------------------------------------------------------------------------
#include <cuda_runtime.h>

#define S2C_D __device__ __forceinline__
#define S2C_HD __host__ __device__ __forceinline__

namespace s2c {

typedef cudaStream_t stream_t;

struct Ctx {
  int tid, nthr, bid, nblk;
  __device__ __forceinline__ void sync() const { __syncthreads(); }
  // barrier among the 32 threads of a warp (every warp of the block must call it equally often:
  // the emulation build implements it as a block barrier)
  __device__ __forceinline__ void sync_warp() const { __syncwarp(); }
};

inline int cuda_check(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return S2C_OK;
  return fail(S2C_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

inline void* dev_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) return nullptr;
  return p;
}
inline void dev_free(void* p) { cudaFree(p); }
inline int dev_upload(void* dst, const void* src, size_t bytes) {
  return cuda_check(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice), "table upload");
}
inline int dev_current() {
  int d = 0;
  cudaGetDevice(&d);
  return d;
}
inline int dev_memset_async(void* p, int v, size_t bytes, stream_t s) {
  return cuda_check(cudaMemsetAsync(p, v, bytes, s), "memset");
}
inline int dev_smem_limit() {
  int dev = dev_current(), v = 0;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  return v;
}

}  // namespace s2c

#define S2C_KERNEL(name, P)                                                                  \
  struct name##_impl {                                                                       \
    static __device__ __forceinline__ void run(const s2c::Ctx& ctx, const P& p,              \
                                               unsigned char* smem);                         \
  };                                                                                         \
  __global__ void name(const P p) {                                                          \
    extern __shared__ float4 s2c_dyn_smem[];                                                 \
    s2c::Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};        \
    name##_impl::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));                \
  }                                                                                          \
  __device__ __forceinline__ void name##_impl::run(const s2c::Ctx& ctx, const P& p,          \
                                                   unsigned char* smem)

#define S2C_KERNEL_BOUNDS(name, P, MAXT, MINB)                                               \
  struct name##_impl {                                                                       \
    static __device__ __forceinline__ void run(const s2c::Ctx& ctx, const P& p,              \
                                               unsigned char* smem);                         \
  };                                                                                         \
  __global__ void __launch_bounds__(MAXT, MINB) name(const P p) {                            \
    extern __shared__ float4 s2c_dyn_smem[];                                                 \
    s2c::Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};        \
    name##_impl::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));                \
  }                                                                                          \
  __device__ __forceinline__ void name##_impl::run(const s2c::Ctx& ctx, const P& p,          \
                                                   unsigned char* smem)

namespace s2c {
extern thread_local long g_launch_count;  // kernels launched by this thread (bench counter)

// Optional per-kernel timing (s2c_timing_begin / s2c_timing_end): one CUDA event pair per launch,
// recorded on the launching stream.
struct TimingRec {
  const char* name;
  cudaEvent_t a, b;
};
inline std::atomic<bool>& timing_on() {
  static std::atomic<bool> on{false};
  return on;
}
inline std::mutex& timing_mutex() {
  static std::mutex m;
  return m;
}
inline std::vector<TimingRec>& timing_recs() {   // guarded by timing_mutex()
  static std::vector<TimingRec> r;
  return r;
}

template <class K, class P>
inline int launch_impl(K kernel, const char* kname, long grid, int block, size_t smem,
                       stream_t stream, const P& p) {
  if (grid <= 0) return S2C_OK;
  if (grid > 2147483647L) return fail(S2C_ERR_UNSUPPORTED, std::string(kname) + ": grid too large");
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return cuda_check(e, kname);
  }
  TimingRec rec{kname, nullptr, nullptr};
  const bool timed = timing_on();
  if (timed) {
    cudaEventCreate(&rec.a);
    cudaEventCreate(&rec.b);
    cudaEventRecord(rec.a, stream);
  }
  kernel<<<(unsigned)grid, block, smem, stream>>>(p);
  if (timed) {
    cudaEventRecord(rec.b, stream);
    std::lock_guard<std::mutex> lock(timing_mutex());
    timing_recs().push_back(rec);
  }
  ++g_launch_count;
  return cuda_check(cudaGetLastError(), kname);
}
}  // namespace s2c

#define S2C_LAUNCH(name, grid, block, smem, stream, params) \
  s2c::launch_impl(name, #name, (long)(grid), (int)(block), (size_t)(smem), stream, params)

namespace s2c {
// ---- asynchronous bulk copy global -> shared (TMA, 1-D) completing on an mbarrier -------------
// dst, src and bytes must be multiples of 16.  One thread initialises the barrier and issues the
// copies; every thread waits with bulk_wait (bounded: returns false if the copy never lands, in
// which case the caller reads the data from global memory instead).
__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void bulk_barrier_init(unsigned long long* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bulk_load_issue(void* dst, const void* src, unsigned bytes,
                                                unsigned long long* bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// 32-byte global accesses (one full sector per lane and instruction); p must be 32-byte aligned
struct float8 {
  float4 lo, hi;
};
__device__ __forceinline__ float8 ld_global_256(const float* p) {
  float8 r;
  asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(r.lo.x), "=f"(r.lo.y), "=f"(r.lo.z), "=f"(r.lo.w), "=f"(r.hi.x), "=f"(r.hi.y),
                 "=f"(r.hi.z), "=f"(r.hi.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void st_global_256(float* p, const float8& v) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v.lo.x), "f"(v.lo.y),
               "f"(v.lo.z), "f"(v.lo.w), "f"(v.hi.x), "f"(v.hi.y), "f"(v.hi.z), "f"(v.hi.w)
               : "memory");
}

__device__ __forceinline__ bool bulk_wait(const Ctx&, unsigned long long* bar, unsigned parity) {
  const unsigned addr = smem_u32(bar);
  for (int spin = 0; spin < (1 << 20); ++spin) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin > 32) __nanosleep(32);
  }
  return false;
}
}  // namespace s2c

#else
// ------------------------------------------------------------------------------------------
// Host emulation backend (test-only)
// ------------------------------------------------------------------------------------------
#include <ucontext.h>

#define S2C_D inline
#define S2C_HD inline

struct float2 {
  float x, y;
};
struct float4 {
  float x, y, z, w;
};
struct int4 {
  int x, y, z, w;
};
inline int4 make_int4(int x, int y, int z, int w) { return int4{x, y, z, w}; }
inline float2 make_float2(float x, float y) { return float2{x, y}; }
inline float4 make_float4(float x, float y, float z, float w) { return float4{x, y, z, w}; }
inline float __ldg(const float* p) { return *p; }
inline float2 __ldg(const float2* p) { return *p; }
inline int __ldg(const int* p) { return *p; }
inline long long __ldg(const long long* p) { return *p; }
inline unsigned short __ldg(const unsigned short* p) { return *p; }

namespace s2c {

typedef void* stream_t;

struct EmuBlock {
  int nthr = 0;
  std::vector<ucontext_t> th;
  ucontext_t sched;
  std::vector<unsigned char> stacks;
  std::vector<char> done;
  void (*entry)(int tid, void* arg) = nullptr;
  void* arg = nullptr;
  int cur = 0;
};
inline EmuBlock*& emu_cur() {
  static thread_local EmuBlock* b = nullptr;
  return b;
}

struct Ctx {
  int tid, nthr, bid, nblk;
  void sync() const {
    EmuBlock* b = emu_cur();
    if (b->nthr > 1) swapcontext(&b->th[tid], &b->sched);
  }
  void sync_warp() const { sync(); }
};

inline void emu_trampoline() {
  EmuBlock* b = emu_cur();
  int t = b->cur;
  b->entry(t, b->arg);
  b->done[t] = 1;
  swapcontext(&b->th[t], &b->sched);
}

// Run one block: every thread is a fiber; a barrier is "yield to the scheduler"; the scheduler
// resumes the fibers round-robin, which executes the block phase by phase.
inline void emu_run_block(int nthr, void (*entry)(int, void*), void* arg) {
  static thread_local EmuBlock blk;
  const size_t kStack = 128 * 1024;
  blk.nthr = nthr;
  blk.entry = entry;
  blk.arg = arg;
  emu_cur() = &blk;
  if (nthr == 1) {
    entry(0, arg);
    return;
  }
  blk.th.resize(nthr);
  blk.done.assign(nthr, 0);
  if (blk.stacks.size() < kStack * nthr) blk.stacks.resize(kStack * nthr);
  for (int t = 0; t < nthr; ++t) {
    getcontext(&blk.th[t]);
    blk.th[t].uc_stack.ss_sp = blk.stacks.data() + kStack * t;
    blk.th[t].uc_stack.ss_size = kStack;
    blk.th[t].uc_link = &blk.sched;
    makecontext(&blk.th[t], (void (*)())emu_trampoline, 0);
  }
  int remaining = nthr;
  while (remaining > 0) {
    for (int t = 0; t < nthr; ++t) {
      if (blk.done[t]) continue;
      blk.cur = t;
      swapcontext(&blk.sched, &blk.th[t]);
      if (blk.done[t]) --remaining;
    }
  }
}

inline void* dev_alloc(size_t bytes) { return std::malloc(bytes ? bytes : 1); }
inline void dev_free(void* p) { std::free(p); }
inline int dev_upload(void* dst, const void* src, size_t bytes) {
  std::memcpy(dst, src, bytes);
  return S2C_OK;
}
inline int dev_current() { return 0; }
inline int dev_memset_async(void* p, int v, size_t bytes, stream_t) {
  std::memset(p, v, bytes);
  return S2C_OK;
}
inline int dev_smem_limit() { return 227 * 1024; }

extern thread_local long g_launch_count;

template <class Impl, class P>
struct EmuLaunch {
  const P* p;
  int bid, nblk, nthr;
  unsigned char* smem;
  static void entry(int tid, void* a) {
    EmuLaunch* self = (EmuLaunch*)a;
    Ctx ctx{tid, self->nthr, self->bid, self->nblk};
    Impl::run(ctx, *self->p, self->smem);
  }
};

template <class Impl, class P>
inline int emu_launch(const char* kname, long grid, int block, size_t smem, const P& p) {
  if (grid <= 0) return S2C_OK;
  if (smem > (size_t)dev_smem_limit())
    return fail(S2C_ERR_UNSUPPORTED, std::string(kname) + ": shared memory over the limit");
  if (block > 1024) return fail(S2C_ERR_UNSUPPORTED, std::string(kname) + ": block > 1024");
  std::vector<unsigned char> sm(smem + 64);
  EmuLaunch<Impl, P> L;
  L.p = &p;
  L.nblk = (int)grid;
  L.nthr = block;
  L.smem = sm.data() + ((64 - (uintptr_t)sm.data() % 64) % 64);
  for (long b = 0; b < grid; ++b) {
    L.bid = (int)b;
    emu_run_block(block, &EmuLaunch<Impl, P>::entry, &L);
  }
  ++g_launch_count;
  return S2C_OK;
}

}  // namespace s2c

#define S2C_KERNEL(name, P)                                                                  \
  struct name##_impl {                                                                       \
    static inline void run(const s2c::Ctx& ctx, const P& p, unsigned char* smem);            \
  };                                                                                         \
  inline void name##_impl::run(const s2c::Ctx& ctx, const P& p, unsigned char* smem)

#define S2C_KERNEL_BOUNDS(name, P, MAXT, MINB) S2C_KERNEL(name, P)

namespace s2c {
// Host stand-ins of the bulk-copy helpers: the copy happens at issue time, the wait is a block
// barrier (every thread of the block calls it at the same point).
inline void bulk_barrier_init(unsigned long long*) {}
inline void bulk_load_issue(void* dst, const void* src, unsigned bytes, unsigned long long*) {
  std::memcpy(dst, src, bytes);
}
struct float8 {
  float4 lo, hi;
};
inline float8 ld_global_256(const float* p) {
  float8 r;
  r.lo = *reinterpret_cast<const float4*>(p);
  r.hi = *reinterpret_cast<const float4*>(p + 4);
  return r;
}
inline void st_global_256(float* p, const float8& v) {
  *reinterpret_cast<float4*>(p) = v.lo;
  *reinterpret_cast<float4*>(p + 4) = v.hi;
}
inline bool bulk_wait(const Ctx& ctx, unsigned long long*, unsigned) {
  ctx.sync();
  return true;
}
}  // namespace s2c

#define S2C_LAUNCH(name, grid, block, smem, stream, params)                                  \
  s2c::emu_launch<name##_impl>(#name, (long)(grid), (int)(block), (size_t)(smem), params)

#endif  // S2C_EMUL
