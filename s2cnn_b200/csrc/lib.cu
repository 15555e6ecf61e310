// C-ABI entry points of s2cnn_b200 (see include/s2cnn_b200.h) and the host-side dispatch that
// sequences the kernels.  Single translation unit: nvcc -gencode arch=compute_100a,code=sm_100a
// for the product; g++ -x c++ -DS2C_EMUL for the host-emulation build used by the CPU tests.
#include "../../include/s2cnn_b200.h"

#include <algorithm>
#include <atomic>
#include <complex>

#include "backend.h"
#include "host_math.h"
#include "tables.h"
#include "fft_device.h"
#include "so3_kernels.h"
#include "so3_plane_kernels.h"
#include "s2_fused_kernels.h"
#include "so3_fused_kernels.h"
#include "so3_relay_kernels.h"
#include "wigner_tiled.h"
#include "wigner_rows.h"
#include "cgemm_kernels.h"
#include "s2_mm_thin.h"
#include "so3_mm_tc.h"
#include "misc_kernels.h"
#include "project_kernels.h"

namespace s2c {
thread_local long g_launch_count = 0;
// test switches (process-wide, race-free; see the "test hooks" section of the header)
static std::atomic<int> g_force_general{0};   // 1 = no single-kernel path, 2 = also no plane kernels
static std::atomic<int> g_plane_chunk{0};     // plane path: signals per chunk (0 = default)

#define S2C_TRY(expr)            \
  do {                           \
    int rc__ = (expr);           \
    if (rc__ != S2C_OK) return rc__; \
  } while (0)

static inline stream_t as_stream(void* s) { return (stream_t)s; }

// Rows (or row pairs) per block of the FFT passes: about 4096 complex numbers of shared memory,
// and a divisor of `period` so that a block never straddles two planes / two (z, n) slabs.
static inline int fft_group(int N, int period) {
  const int cap = std::max(1, std::min(256, 4096 / N));
  int g = 1;
  for (int d = 1; d <= period && d <= cap; ++d)
    if (period % d == 0) g = d;
  return g;
}

static size_t so3_ws_per_z(int N, int K) {
  // two scratch arrays of complex numbers: [z][K][N][N] and [K][2K-1][z][N]
  return ((size_t)K * N * N + (size_t)K * (2 * K - 1) * N) * sizeof(float2);
}
static size_t s2_ws_per_z(int N, int K) { return (size_t)(2 * K - 1) * N * sizeof(float2); }

// Large-bandwidth path for N = 64 and 128: a plane kernel (both row transforms of a (z, beta)
// plane) and a Wigner kernel per direction, through the scratch array V[n][z][beta][f] of
// 8 K N^2 bytes per signal, in chunks of at most kRowsZC signals so that V stays in L2 between the
// two kernels (b = 64: 8.4 MB per signal, 67 MB per chunk of the 126 MB).
static size_t so3_v_per_z(int N, int K) { return (size_t)K * N * N * sizeof(float2); }
static bool use_plane_kernels(int N) { return plane_supported(N) && g_force_general < 2; }
static int launch_fwd_plane(int N, long zc, stream_t st, const FwdPlaneParams& f) {
  const long grid = zc * N;
  if (N == 128) return S2C_LAUNCH_PLANE(so3_fwd_plane, 128, grid, st, f);
  return S2C_LAUNCH_PLANE(so3_fwd_plane, 64, grid, st, f);
}
static int launch_inv_plane(int N, long zc, stream_t st, const InvPlaneParams& f) {
  const long grid = zc * N;
  if (N == 128) return S2C_LAUNCH_PLANE(so3_inv_plane, 128, grid, st, f);
  return S2C_LAUNCH_PLANE(so3_inv_plane, 64, grid, st, f);
}
static int launch_fwd_rows(int N, stream_t st, const FwdRowsParams& f) {
  if (N == 128) return S2C_LAUNCH_ROWS(so3_fwd_wigner_r, 128, rows_grid(f.K, f.zc), st, f);
  return S2C_LAUNCH_ROWS(so3_fwd_wigner_r, 64, rows_grid(f.K, f.zc), st, f);
}
static int launch_inv_rows(int N, stream_t st, const InvRowsParams& f) {
  if (N == 128) return S2C_LAUNCH_ROWS(so3_inv_wigner_r, 128, rows_grid(f.K, f.zc), st, f);
  return S2C_LAUNCH_ROWS(so3_inv_wigner_r, 64, rows_grid(f.K, f.zc), st, f);
}

// Runs `first(z0, zc, buffer, stream)` then `second(z0, zc, buffer, stream)` for every chunk of the
// batch, in order on the caller's stream, through one scratch buffer.  (Running the two kernel
// kinds of neighbouring chunks concurrently on two streams through two half-size buffers was
// measured slower: both kinds are limited by the same shared-memory / L1 data path.)
template <class F1, class F2>
static int plane_pipeline(long nbatch, int N, int K, void* ws, size_t ws_bytes, stream_t st,
                          F1 first, F2 second) {
  const size_t vz = so3_v_per_z(N, K);
  const int want = g_plane_chunk.load();
  const long fit = (long)(ws_bytes / vz);
  if (fit < 1 || ws == nullptr)
    return fail(S2C_ERR_WORKSPACE, "workspace smaller than one batch element (" + std::to_string(vz) +
                                       " bytes needed)");
  long chunk = (want >= 1 && want <= kRowsZC) ? want : kRowsZC;
  chunk = std::min(std::min(chunk, fit), nbatch);
  for (long z0 = 0; z0 < nbatch; z0 += chunk) {
    const long zc = std::min(chunk, nbatch - z0);
    S2C_TRY(first(z0, zc, (float2*)ws, st));
    S2C_TRY(second(z0, zc, (float2*)ws, st));
  }
  return S2C_OK;
}

static int check_b(int b_in, int b_out) {
  if (b_in < 1 || b_out < 1) return fail(S2C_ERR_BAD_ARG, "bandwidths must be >= 1");
  return S2C_OK;
}

// ---------------------------------------------------------------------------------------------
// SO(3) analysis:  real signal (strided) -> spectrum rows [nspec(b_out)][nbatch]
// ---------------------------------------------------------------------------------------------
static int so3_analysis(const float* x, long in_stride, long in_off, float2* out, long nbatch,
                        int b_in, int b_out, bool weighted, int mode, void* ws, size_t ws_bytes,
                        stream_t st, bool relu = false, float* sums = nullptr) {
  const int N = 2 * b_in, K = std::min(b_in, b_out);
  FftDev fft;
  PanelsDev pan;
  S2C_TRY(TableCache::get().fft(N, fft));
  S2C_TRY(TableCache::get().panels(b_in, b_out, K, weighted, false, pan));
  if (b_out > b_in && mode == kSo3Real)  // rows with |m| or |n| >= b_in stay zero (so3_fft.py:44-48)
    S2C_TRY(dev_memset_async(out, 0, (size_t)so3_nspec(b_out) * nbatch * sizeof(float2), st));
  if (!g_force_general && N <= kFusedMaxN &&
      fwd_fused_smem_bytes(N, pan.nrows) <= (size_t)dev_smem_limit() - 1024) {
    FwdFusedParams f;
    f.x = x; f.in_stride = in_stride; f.in_off = in_off;
    f.out = out; f.out_zstride = nbatch;
    f.pan = pan; f.tw = fft.tw;
    f.nbatch = (int)nbatch; f.K = K; f.BG = fused_bg(N); f.KP = fused_kp(N); f.PS = fused_plane_stride(N, K);
    f.nrows = pan.nrows; f.mode = mode; f.relu = relu;
    f.wide = in_stride == 1 && in_off == 0 && N % 4 == 0 && (uintptr_t)x % 32 == 0;
    f.sums = sums;
    int rc = S2C_OK;
    const long grid = (nbatch + kFusedZG - 1) / kFusedZG;
    const size_t sm = fwd_fused_smem_bytes(N, pan.nrows);
    S2C_DISPATCH_N(N, rc = S2C_LAUNCH_N(so3_fwd_fused, kN, grid,
                                        fused_threads(sm, (size_t)dev_smem_limit()), sm, st, f));
    return rc;
  }
  if (relu) return fail(S2C_ERR_UNSUPPORTED, "fused ReLU input needs the small-bandwidth path");
  if (sums) return fail(S2C_ERR_UNSUPPORTED, "per-signal sums need the small-bandwidth path");
  if (use_plane_kernels(N)) {
    HalfPanelsDev hp;
    hp.nbeta = N; hp.nl = b_out; hp.K = K; hp.npairs = pan.npairs;
    S2C_TRY(TableCache::get().half_panels(b_in, b_out, K, weighted, &hp.data, &hp.off));
    auto planes = [&](long z0, long zc, float2* v, stream_t s) {
      FwdPlaneParams f;
      f.x = x + (size_t)z0 * N * N * N * in_stride;
      f.in_stride = in_stride; f.in_off = in_off;
      f.v = v; f.tw = fft.tw; f.nbatch = (int)zc; f.K = K;
      return launch_fwd_plane(N, zc, s, f);
    };
    auto wigner = [&](long z0, long zc, float2* v, stream_t s) {
      FwdRowsParams r;
      r.v = v; r.out = out + z0; r.out_zstride = nbatch; r.pan = hp;
      r.zc = (int)zc; r.K = K; r.nl = b_out; r.mode = mode;
      return launch_fwd_rows(N, s, r);
    };
    return plane_pipeline(nbatch, N, K, ws, ws_bytes, st, planes, wigner);
  }
  const size_t per_z = so3_ws_per_z(N, K);
  long chunk = (long)std::min<size_t>((size_t)nbatch, ws_bytes / per_z);
  if (chunk < 1 || ws == nullptr)
    return fail(S2C_ERR_WORKSPACE, "workspace smaller than one batch element (" +
                                       std::to_string(per_z) + " bytes needed)");
  const int G = fft_group(N, N), Gg = fft_group(N, N / 2);  // alpha passes, gamma passes
  const size_t fft_smem = fft_smem_bytes(N, G);
  for (long z0 = 0; z0 < nbatch; z0 += chunk) {
    const long zc = std::min(chunk, nbatch - z0);
    float2* u = (float2*)ws;
    float2* v = u + (size_t)zc * K * N * N;
    {
    FwdGammaParams g;
    g.x = x + (size_t)z0 * N * N * N * in_stride;
    g.in_stride = in_stride;
    g.in_off = in_off;
    g.u = u;
    g.N = N; g.b = b_in; g.K = K; g.G = Gg;
    g.npairs = zc * N * b_in;
    g.fft = fft;
    S2C_TRY(S2C_LAUNCH(so3_fwd_gamma, (g.npairs + Gg - 1) / Gg, kThreads, fft_smem_bytes(N, Gg), st, g));
    FwdAlphaParams a;
    a.in = (const float*)u;
    a.in_real = 0;
    a.v = v;
    a.nbatch = (int)zc; a.N = N; a.K = K; a.Kn = K; a.G = G;
    a.nrows = zc * K * N;
    a.fft = fft;
    S2C_TRY(S2C_LAUNCH(so3_fwd_alpha, (a.nrows + G - 1) / G, kThreads, fft_smem, st, a));
    }
    FwdWignerParams w;
    w.v = v;
    w.out = out + z0;
    w.out_zstride = nbatch;
    w.pan = pan;
    w.nbatch = (int)zc; w.N = N; w.K = K; w.nl = b_out;
    w.ZT = (int)std::min<long>(32, zc);
    w.nzt = (int)((zc + w.ZT - 1) / w.ZT);
    w.mode = mode;
    if (N % (4 * kWigHalves) == 0 && fwd_wigner_t_smem(N, b_out) <= (size_t)dev_smem_limit() - 1024) {
      w.ZT = kWigZT;
      w.nzt = (int)((zc + kWigZT - 1) / kWigZT);
      S2C_TRY(S2C_LAUNCH(so3_fwd_wigner_t, (long)pan.npairs * w.nzt, kThreads,
                         fwd_wigner_t_smem(N, b_out), st, w));
      continue;
    }
    const size_t wsm = align_up((size_t)b_out * (N + 1) * sizeof(float), 16) +
                       (size_t)w.ZT * (N + 1) * sizeof(float2);
    S2C_TRY(S2C_LAUNCH(so3_fwd_wigner, (long)pan.npairs * w.nzt, kThreads, wsm, st, w));
  }
  return S2C_OK;
}

// ---------------------------------------------------------------------------------------------
// SO(3) synthesis:  spectrum rows [nspec(b_in)][nbatch] -> real signal (strided)
// ---------------------------------------------------------------------------------------------
struct S2ProductArgs {
  const float2* xs = nullptr;
  const float2* ys = nullptr;
  int nb = 0, fin = 0, fout = 0;
};

static bool so3_synthesis_is_fused(int b_in, int b_out) {
  const int N = 2 * b_out, K = std::min(b_in, b_out);
  if (g_force_general || N > kFusedMaxN) return false;
  const int nrows = (so3_nspec(K) - K) / 2 + K;  // half-plane rows: the (0,0) pair is its own mirror
  return fused_smem_bytes(N, nrows) <= (size_t)dev_smem_limit() - 1024;
}

static int so3_synthesis(const float2* x, float* out, long out_stride, long out_off, long nbatch,
                         int b_in, int b_out, bool weighted, int mode, const float* bias,
                         int nfeat, void* ws, size_t ws_bytes, stream_t st,
                         const S2ProductArgs* prod = nullptr, float* integral = nullptr,
                         const float* mask = nullptr) {
  const int N = 2 * b_out, K = std::min(b_in, b_out);
  FftDev fft;
  PanelsDev pan;
  S2C_TRY(TableCache::get().fft(N, fft));
  S2C_TRY(TableCache::get().panels(b_out, K, K, weighted, false, pan));
  if (!g_force_general && N <= kFusedMaxN &&
      fused_smem_bytes(N, pan.nrows) <= (size_t)dev_smem_limit() - 1024) {
    InvFusedParams f;
    f.x = x; f.x_zstride = nbatch;
    f.out = out; f.out_stride = out_stride; f.out_off = out_off;
    f.bias = bias; f.nfeat = nfeat > 0 ? nfeat : 1;
    f.pan = pan; f.tw = fft.tw;
    f.nbatch = (int)nbatch; f.K = K; f.BG = fused_bg(N); f.KP = fused_kp(N); f.PS = fused_plane_stride(N, K);
    f.nrows = pan.nrows; f.mode = mode;
    f.xs = nullptr; f.ys = nullptr; f.s2_nb = f.s2_fin = f.s2_fout = 0;
    f.iw = nullptr; f.isum = nullptr;
    f.mask = mask;
    if (mask && (out_stride != 1 || out_off != 0))
      return fail(S2C_ERR_UNSUPPORTED, "masked synthesis: real output only");
    f.wide = out_stride == 1 && out_off == 0 && N % 4 == 0 && out && (uintptr_t)out % 32 == 0 &&
             (uintptr_t)mask % 32 == 0;
    if (integral) {
      if (N % f.BG != 0 || kFusedZG * f.BG * (N / 2) > 256)
        return fail(S2C_ERR_UNSUPPORTED, "fused integration: unsupported grouping");
      S2C_TRY(TableCache::get().quad_weights(b_out, &f.iw));
      f.isum = integral;
    }
    if (prod) {
      f.mode = kS2Product;
      f.xs = prod->xs; f.ys = prod->ys;
      f.s2_nb = prod->nb; f.s2_fin = prod->fin; f.s2_fout = prod->fout;
    }
    int rc = S2C_OK;
    const long grid = (nbatch + kFusedZG - 1) / kFusedZG;
    const size_t sm = fused_smem_bytes(N, pan.nrows);
    S2C_DISPATCH_N(N, rc = S2C_LAUNCH_N(so3_inv_fused, kN, grid,
                                        fused_threads(sm, (size_t)dev_smem_limit()), sm, st, f));
    return rc;
  }
  if (integral)
    return fail(S2C_ERR_UNSUPPORTED, "fused ReLU + integration needs the small-bandwidth path");
  if (mask) return fail(S2C_ERR_UNSUPPORTED, "masked synthesis needs the small-bandwidth path");
  if (use_plane_kernels(N)) {
    HalfPanelsDev hp;
    hp.nbeta = N; hp.nl = K; hp.K = K; hp.npairs = pan.npairs;
    S2C_TRY(TableCache::get().half_panels(b_out, K, K, weighted, &hp.data, &hp.off));
    auto wigner = [&](long z0, long zc, float2* s, stream_t sm) {
      InvRowsParams r;
      r.x = x + z0; r.x_zstride = nbatch; r.s = s; r.pan = hp;
      r.zc = (int)zc; r.K = K; r.mode = mode;
      return launch_inv_rows(N, sm, r);
    };
    auto planes = [&](long z0, long zc, float2* s, stream_t sm) {
      InvPlaneParams f;
      f.s = s;
      f.out = out + (size_t)z0 * N * N * N * out_stride;
      f.out_stride = out_stride; f.out_off = out_off;
      f.bias = bias; f.nfeat = nfeat > 0 ? nfeat : 1; f.z0 = z0;
      f.tw = fft.tw; f.nbatch = (int)zc; f.K = K;
      return launch_inv_plane(N, zc, sm, f);
    };
    return plane_pipeline(nbatch, N, K, ws, ws_bytes, st, wigner, planes);
  }
  const size_t per_z = so3_ws_per_z(N, K);
  long chunk = (long)std::min<size_t>((size_t)nbatch, ws_bytes / per_z);
  if (chunk < 1 || ws == nullptr)
    return fail(S2C_ERR_WORKSPACE, "workspace smaller than one batch element (" +
                                       std::to_string(per_z) + " bytes needed)");
  const int G = fft_group(N, N), Gg = fft_group(N, N / 2);  // alpha passes, gamma passes
  const size_t fft_smem = fft_smem_bytes(N, G);
  for (long z0 = 0; z0 < nbatch; z0 += chunk) {
    const long zc = std::min(chunk, nbatch - z0);
    float2* t = (float2*)ws;                                   // [z][K][N][N]
    float2* s = t + (size_t)zc * K * N * N;                    // [K][2K-1][z][N]
    InvWignerParams w;
    w.x = x + z0;
    w.x_zstride = nbatch;
    w.s = s;
    w.pan = pan;
    w.nbatch = (int)zc; w.N = N; w.K = K;
    w.ZT = (int)std::min<long>(32, zc);
    w.nzt = (int)((zc + w.ZT - 1) / w.ZT);
    w.mode = mode;
    if (N % 4 == 0 && inv_wigner_t_smem(N, K) <= (size_t)dev_smem_limit() - 1024) {
      w.ZT = kWigZT;
      w.nzt = (int)((zc + kWigZT - 1) / kWigZT);
      S2C_TRY(S2C_LAUNCH(so3_inv_wigner_t, (long)pan.npairs * w.nzt, kThreads,
                         inv_wigner_t_smem(N, K), st, w));
    } else {
      const size_t wsm = align_up((size_t)K * N * sizeof(float), 16) + (size_t)K * w.ZT * sizeof(float2);
      S2C_TRY(S2C_LAUNCH(so3_inv_wigner, (long)pan.npairs * w.nzt, kThreads, wsm, st, w));
    }
    InvAlphaParams a;
    a.s = s;
    a.out = (float*)t;
    a.out_real = 0;
    a.herm_n0 = 1;
    a.nbatch = (int)zc; a.N = N; a.K = K; a.Kn = K; a.G = G;
    a.nrows = zc * K * N;
    a.fft = fft;
    S2C_TRY(S2C_LAUNCH(so3_inv_alpha, (a.nrows + G - 1) / G, kThreads, fft_smem, st, a));
    InvGammaParams g;
    g.t = t;
    g.out = out + (size_t)z0 * N * N * N * out_stride;
    g.out_stride = out_stride;
    g.out_off = out_off;
    g.bias = bias;
    g.nfeat = nfeat > 0 ? nfeat : 1;
    g.z0 = z0;
    g.N = N; g.b = b_out; g.K = K; g.G = Gg;
    g.npairs = zc * N * b_out;
    g.fft = fft;
    S2C_TRY(S2C_LAUNCH(so3_inv_gamma, (g.npairs + Gg - 1) / Gg, kThreads, fft_smem_bytes(N, Gg), st, g));
  }
  return S2C_OK;
}

static int mm_dispatch(bool so3, int op, const float* a, const float* b, float* c, int nl, int nb,
                       int fi, int fo, stream_t st) {
  if (nl < 1 || nb < 1 || fi < 1 || fo < 1) return fail(S2C_ERR_BAD_ARG, "sizes must be >= 1");
  CgemmParams p = mm_params(so3, op, nl, nb, fi, fo);
  p.A = (const float2*)a;
  p.B = (const float2*)b;
  p.C = (float2*)c;
  return S2C_LAUNCH(cgemm_grouped, cgemm_total_tiles(p), 256, cgemm_smem_bytes(), st, p);
}

}  // namespace s2c

using namespace s2c;

extern "C" {

const char* s2c_last_error(void) { return last_error_ref().c_str(); }
int s2c_version(void) { return 100; }
long s2c_launch_count(void) { return g_launch_count; }
void s2c_clear_tables(void) { TableCache::get().clear(); }
void s2c_set_table_cache_dir(const char* dir) { TableDiskCache::get().set_dir(dir); }
long s2c_table_cache_hits(void) { return TableDiskCache::get().hits(); }
long s2c_table_cache_stores(void) { return TableDiskCache::get().stores(); }
long s2c_tables_computed(void) { return TableCache::computed_count().load(); }
int s2c_is_cuda_build(void) {
#ifdef S2C_EMUL
  return 0;
#else
  return 1;
#endif
}

void s2c_timing_begin(void) {
#ifndef S2C_EMUL
  {
    std::lock_guard<std::mutex> lock(timing_mutex());
    timing_recs().clear();
  }
  timing_on() = true;
#endif
}

int s2c_timing_end(char* buf, size_t buf_bytes) {
  if (!buf || buf_bytes == 0) return fail(S2C_ERR_BAD_ARG, "s2c_timing_end: no buffer");
  buf[0] = 0;
#ifndef S2C_EMUL
  timing_on() = false;
  std::lock_guard<std::mutex> lock(timing_mutex());
  struct Acc { long n = 0; double ms = 0; };
  std::vector<std::pair<std::string, Acc>> acc;
  for (auto& r : timing_recs()) {
    float ms = 0.f;
    cudaEventSynchronize(r.b);
    cudaEventElapsedTime(&ms, r.a, r.b);
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
    size_t i = 0;
    for (; i < acc.size(); ++i) if (acc[i].first == r.name) break;
    if (i == acc.size()) acc.push_back({r.name, Acc()});
    acc[i].second.n += 1;
    acc[i].second.ms += ms;
  }
  timing_recs().clear();
  std::string out;
  for (auto& kv : acc) {
    char line[256];
    std::snprintf(line, sizeof(line), "%s %ld %.6f\n", kv.first.c_str(), kv.second.n, kv.second.ms);
    out += line;
  }
  if (out.size() + 1 > buf_bytes) return fail(S2C_ERR_BAD_ARG, "s2c_timing_end: buffer too small");
  std::memcpy(buf, out.c_str(), out.size() + 1);
#endif
  return S2C_OK;
}

// ---- host generators ---------------------------------------------------------------------------
int s2c_wigner_d(int l, double beta, double* out) {
  if (l < 0 || !out) return fail(S2C_ERR_BAD_ARG, "s2c_wigner_d: bad argument");
  const int L = 2 * l + 1;
  std::vector<double> col(l + 2);
  for (int m = -l; m <= l; ++m)
    for (int n = -l; n <= l; ++n) {
      const int l0 = wigner_d_degrees(m, n, beta, l + 1, col.data());
      out[(m + l) * L + (n + l)] = col[l - l0];
    }
  return S2C_OK;
}

int s2c_quadrature_weights(int b, double* out) {
  if (b < 1 || !out) return fail(S2C_ERR_BAD_ARG, "s2c_quadrature_weights: bad argument");
  std::vector<double> w;
  quadrature_weights(b, w);
  std::copy(w.begin(), w.end(), out);
  return S2C_OK;
}

int s2c_so3_wigner_table(int b, int nl, int weighted, float* out) {
  if (b < 1 || nl < 1 || !out) return fail(S2C_ERR_BAD_ARG, "s2c_so3_wigner_table: bad argument");
  std::vector<double> beta, w, col(nl + 1);
  soft_betas(b, beta);
  quadrature_weights(b, w);
  const long ns = so3_nspec(nl);
  for (int j = 0; j < 2 * b; ++j)
    for (int m = -(nl - 1); m < nl; ++m)
      for (int n = -(nl - 1); n < nl; ++n) {
        const int l0 = wigner_d_degrees(m, n, beta[j], nl, col.data());
        for (int l = l0; l < nl; ++l)
          out[j * ns + so3_row(l, m, n)] =
              (float)(col[l - l0] * (weighted ? w[j] : (2.0 * l + 1.0)));
      }
  return S2C_OK;
}

int s2c_s2_wigner_table(int b, int nl, int weighted, float* out) {
  if (b < 1 || nl < 1 || !out) return fail(S2C_ERR_BAD_ARG, "s2c_s2_wigner_table: bad argument");
  std::vector<double> beta, w, col(nl + 1);
  soft_betas(b, beta);
  quadrature_weights(b, w);
  for (int j = 0; j < 2 * b; ++j)
    for (int m = -(nl - 1); m < nl; ++m) {
      const int l0 = wigner_d_degrees(m, 0, beta[j], nl, col.data());
      for (int l = l0; l < nl; ++l)
        out[(long)j * nl * nl + l * l + l + m] =
            (float)(col[l - l0] * (weighted ? w[j] * 2.0 * b : (2.0 * l + 1.0)));
    }
  return S2C_OK;
}

// F = conj(D^l_mn(alpha, beta, gamma)) = exp(-i m alpha) d^l_mn(beta) exp(-i n gamma)
int s2c_so3_ft_matrix(int b, const double* grid, int n_grid, float* F) {
  if (b < 1 || n_grid < 1 || !grid || !F) return fail(S2C_ERR_BAD_ARG, "s2c_so3_ft_matrix: bad argument");
  const long ns = so3_nspec(b);
  std::vector<double> col(b + 1);
  for (int i = 0; i < n_grid; ++i) {
    const double beta = grid[3 * i], alpha = grid[3 * i + 1], gamma = grid[3 * i + 2];
    for (int m = -(b - 1); m < b; ++m)
      for (int n = -(b - 1); n < b; ++n) {
        const int l0 = wigner_d_degrees(m, n, beta, b, col.data());
        const std::complex<double> ph = std::exp(std::complex<double>(0.0, -(m * alpha + n * gamma)));
        for (int l = l0; l < b; ++l) {
          const std::complex<double> v = ph * col[l - l0];
          float* dst = F + ((long)i * ns + so3_row(l, m, n)) * 2;
          dst[0] = (float)v.real();
          dst[1] = (float)v.imag();
        }
      }
  }
  return S2C_OK;
}

// F = 2b conj(D^l_m0(alpha, beta, 0))
int s2c_s2_ft_matrix(int b, const double* grid, int n_grid, float* F) {
  if (b < 1 || n_grid < 1 || !grid || !F) return fail(S2C_ERR_BAD_ARG, "s2c_s2_ft_matrix: bad argument");
  std::vector<double> col(b + 1);
  for (int i = 0; i < n_grid; ++i) {
    const double beta = grid[2 * i], alpha = grid[2 * i + 1];
    for (int m = -(b - 1); m < b; ++m) {
      const int l0 = wigner_d_degrees(m, 0, beta, b, col.data());
      const std::complex<double> ph = std::exp(std::complex<double>(0.0, -m * alpha));
      for (int l = l0; l < b; ++l) {
        const std::complex<double> v = (2.0 * b) * ph * col[l - l0];
        float* dst = F + ((long)i * b * b + l * l + l + m) * 2;
        dst[0] = (float)v.real();
        dst[1] = (float)v.imag();
      }
    }
  }
  return S2C_OK;
}

// ---- SO(3) transforms ----------------------------------------------------------------------------
size_t s2c_so3_fft_workspace_min(int b_in, int b_out) {
  // the beta grid is b_in's for analysis and b_out's for synthesis; take the larger of the two
  const int K = std::min(b_in, b_out);
  return std::max(so3_ws_per_z(2 * b_in, K), so3_ws_per_z(2 * b_out, K));
}

size_t s2c_so3_fft_workspace(long nbatch, int b_in, int b_out) {
  const size_t per_z = s2c_so3_fft_workspace_min(b_in, b_out);
  if (plane_supported(2 * b_in) && plane_supported(2 * b_out)) {
    // large-bandwidth path: one chunk of the scratch array V (sized to stay in L2); never less than
    // one signal of the three-pass organisation, which the test switches can select instead
    const int K = std::min(b_in, b_out);
    const size_t v = std::max(so3_v_per_z(2 * b_in, K), so3_v_per_z(2 * b_out, K));
    return std::max(per_z, v * (size_t)std::min<long>(kRowsZC, std::max(1L, nbatch)));
  }
  const size_t target = (size_t)256 << 20;
  long chunk = (long)std::max<size_t>(32, target / per_z);
  chunk = std::min(chunk, std::max(1L, nbatch));
  return per_z * (size_t)chunk;
}

int s2c_so3_rfft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                 void* ws, size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rfft: bad argument");
  return so3_analysis(x, 1, 0, (float2*)out, nbatch, b_in, b_out, !for_grad, kSo3Real, ws,
                      ws_bytes, as_stream(stream));
}

int s2c_so3_rfft_relu(const float* x, float* out, long nbatch, int b_in, int b_out, void* ws,
                      size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rfft_relu: bad argument");
  return so3_analysis(x, 1, 0, (float2*)out, nbatch, b_in, b_out, true, kSo3Real, ws, ws_bytes,
                      as_stream(stream), true);
}

int s2c_so3_rfft_sums(const float* x, float* out, float* sums, long nbatch, int b_in, int b_out,
                      int for_grad, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || !sums || nbatch < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rfft_sums: bad argument");
  return so3_analysis(x, 1, 0, (float2*)out, nbatch, b_in, b_out, !for_grad, kSo3Real, nullptr, 0,
                      as_stream(stream), false, sums);
}

void s2c_debug_force_general_path(int level) { g_force_general = level < 0 ? 0 : level; }
void s2c_debug_plane_chunk(int signals) { g_plane_chunk = signals < 0 ? 0 : signals; }

int s2c_so3_fft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                void* ws, size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_fft: bad argument");
  // linearity: FT(re + i im) = FT(re) + i FT(im), each a real-input transform
  S2C_TRY(so3_analysis(x, 2, 0, (float2*)out, nbatch, b_in, b_out, !for_grad, kSo3Real, ws,
                       ws_bytes, as_stream(stream)));
  return so3_analysis(x, 2, 1, (float2*)out, nbatch, b_in, b_out, !for_grad, kSo3AccumI, ws,
                      ws_bytes, as_stream(stream));
}

int s2c_so3_rifft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                  const float* bias, int nfeature, void* ws, size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft: bad argument");
  if (bias && nfeature < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft: nfeature must be >= 1 with a bias");
  return so3_synthesis((const float2*)x, out, 1, 0, nbatch, b_in, b_out, for_grad != 0, kSo3Real,
                       bias, nfeature, ws, ws_bytes, as_stream(stream));
}

int s2c_so3_rifft_relu_grad(const float* x, const float* act, float* out, long nbatch, int b_in,
                            int b_out, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !act || !out || nbatch < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_relu_grad: bad argument");
  return so3_synthesis((const float2*)x, out, 1, 0, nbatch, b_in, b_out, true, kSo3Real, nullptr, 0,
                       nullptr, 0, as_stream(stream), nullptr, nullptr, act);
}

int s2c_so3_rifft_relu_integrate(const float* x, float* out, long nbatch, int b_in, int b_out,
                                 const float* bias, int nfeature, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_relu_integrate: bad argument");
  if (bias && nfeature < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_relu_integrate: nfeature must be >= 1 with a bias");
  if (!so3_synthesis_is_fused(b_in, b_out))
    return fail(S2C_ERR_UNSUPPORTED, "s2c_so3_rifft_relu_integrate: needs 2 b_out <= 32");
  return so3_synthesis((const float2*)x, nullptr, 1, 0, nbatch, b_in, b_out, false, kSo3Real, bias,
                       nfeature, nullptr, 0, as_stream(stream), nullptr, out);
}

// Largest beta group (a divisor of N whose row stage fits one pass of the block) that keeps three
// blocks of the relay kernel on an SM; failing that, the largest that fits at all (0: none).
static int relay_bg(int N, int Kin, int nrows_in, int nrows_out) {
  int best3 = 0, best = 0;
  for (int d = 1; d <= N && d <= kMaxBG; ++d) {
    if (N % d != 0 || kFusedZG * d * (N / 2) > 256) continue;
    const size_t sm = relay_smem_bytes(N, Kin, nrows_in, nrows_out, d);
    if (sm <= (size_t)dev_smem_limit() - 1024) best = d;
    if (3 * (sm + 1024) <= (size_t)227 * 1024) best3 = d;
  }
  return best3 ? best3 : best;
}

// relay kernel: synthesis at bandwidth b_mid of a spectrum of bandwidth b_in (plain, or the s2_mm
// product of xs and ys when xs is set), + bias, ReLU, analysis to bandwidth b_next
static int relay_launch(const float2* x, const float2* xs, const float2* ys, int s2_nb, int s2_fin,
                        float* out, long nz, int nfeat, int b_in, int b_mid, int b_next,
                        const float* bias, stream_t st, const char* who) {
  const int N = 2 * b_mid;
  if (N > kFusedMaxN || b_next > b_mid || b_in > b_mid)
    return fail(S2C_ERR_UNSUPPORTED,
                std::string(who) + ": needs 2 b <= 32, b_in <= b and b_next <= b");
  FftDev fft;
  RelayParams f;
  S2C_TRY(TableCache::get().fft(N, fft));
  S2C_TRY(TableCache::get().panels(b_mid, b_in, b_in, false, false, f.pin));
  S2C_TRY(TableCache::get().panels(b_mid, b_next, b_next, true, false, f.pout));
  f.BG = relay_bg(N, b_in, f.pin.nrows, f.pout.nrows);
  if (f.BG < 1) return fail(S2C_ERR_UNSUPPORTED, std::string(who) + ": shared memory");
  S2C_TRY(TableCache::get().grouped(b_mid, b_in, b_in, false, f.BG, &f.win_g, &f.win_stride));
  S2C_TRY(TableCache::get().grouped(b_mid, b_next, b_next, true, f.BG, &f.wout_g, &f.wout_stride));
  f.x = x; f.x_zstride = nz;
  f.xs = xs; f.ys = ys;
  f.s2_nb = s2_nb; f.s2_fin = s2_fin; f.s2_fout = nfeat;
  f.bias = bias; f.nfeat = nfeat > 0 ? nfeat : 1;
  f.out = (float2*)out; f.out_zstride = nz;
  f.tw = fft.tw;
  f.nbatch = (int)nz; f.Kin = b_in; f.Kout = b_next;
  f.KP = fused_kp(N); f.PS = fused_plane_stride(N, b_in);
  int rc = S2C_OK;
  const long grid = (nz + kFusedZG - 1) / kFusedZG;
  const size_t sm = relay_smem_bytes(N, b_in, f.pin.nrows, f.pout.nrows, f.BG);
  S2C_DISPATCH_N(N, rc = S2C_LAUNCH_N(so3_relay_fused, kN, grid, 256, sm, st, f));
  return rc;
}

int s2c_s2_conv_relu_so3_rfft(const float* xs, const float* ys, float* out, int nbatch, int f_in,
                              int f_out, int b, int b_next, const float* bias, void* stream) {
  S2C_TRY(check_b(b, b_next));
  if (!xs || !ys || !out || nbatch < 1 || f_in < 1 || f_out < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_s2_conv_relu_so3_rfft: bad argument");
  return relay_launch(nullptr, (const float2*)xs, (const float2*)ys, nbatch, f_in, out,
                      (long)nbatch * f_out, f_out, b, b, b_next, bias, as_stream(stream),
                      "s2c_s2_conv_relu_so3_rfft");
}

int s2c_so3_rifft_relu_rfft(const float* x, float* out, long nbatch, int b_in, int b_mid, int b_next,
                            const float* bias, int nfeature, void* stream) {
  S2C_TRY(check_b(b_in, b_mid));
  S2C_TRY(check_b(b_mid, b_next));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_relu_rfft: bad argument");
  if (bias && nfeature < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_relu_rfft: nfeature must be >= 1 with a bias");
  return relay_launch((const float2*)x, nullptr, nullptr, 0, 0, out, nbatch, bias ? nfeature : 0,
                      b_in, b_mid, b_next, bias, as_stream(stream), "s2c_so3_rifft_relu_rfft");
}

size_t s2c_s2_conv_synthesis_workspace(int nbatch, int f_out, int b) {
  if (so3_synthesis_is_fused(b, b)) return 16;
  const size_t z_bytes = (size_t)so3_nspec(b) * nbatch * f_out * sizeof(float2);
  return z_bytes + s2c_so3_fft_workspace((long)nbatch * f_out, b, b);
}

int s2c_s2_conv_synthesis(const float* xs, const float* ys, float* out, int nbatch, int f_in,
                          int f_out, int b, const float* bias, void* ws, size_t ws_bytes,
                          void* stream) {
  S2C_TRY(check_b(b, b));
  if (!xs || !ys || !out || nbatch < 1 || f_in < 1 || f_out < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_s2_conv_synthesis: bad argument");
  const long nz = (long)nbatch * f_out;
  if (so3_synthesis_is_fused(b, b)) {
    S2ProductArgs pr;
    pr.xs = (const float2*)xs; pr.ys = (const float2*)ys;
    pr.nb = nbatch; pr.fin = f_in; pr.fout = f_out;
    return so3_synthesis(nullptr, out, 1, 0, nz, b, b, false, kSo3Real, bias, f_out, ws, ws_bytes,
                         as_stream(stream), &pr);
  }
  // larger bandwidths: product into the head of the workspace, then the general synthesis
  const size_t z_bytes = (size_t)so3_nspec(b) * nz * sizeof(float2);
  if (!ws || ws_bytes <= z_bytes)
    return fail(S2C_ERR_WORKSPACE, "s2c_s2_conv_synthesis: workspace too small");
  S2C_TRY(mm_dispatch(false, kMmFwd, xs, ys, (float*)ws, b, nbatch, f_in, f_out, as_stream(stream)));
  return so3_synthesis((const float2*)ws, out, 1, 0, nz, b, b, false, kSo3Real, bias, f_out,
                       (unsigned char*)ws + z_bytes, ws_bytes - z_bytes, as_stream(stream));
}

int s2c_so3_ifft(const float* x, float* out, long nbatch, int b_in, int b_out, int for_grad,
                 void* ws, size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_ifft: bad argument");
  // Re(A X) and Im(A X) = Re(A (-i X)) for the complex-linear synthesis A
  S2C_TRY(so3_synthesis((const float2*)x, out, 2, 0, nbatch, b_in, b_out, for_grad != 0, kSo3Real,
                        nullptr, 1, ws, ws_bytes, as_stream(stream)));
  return so3_synthesis((const float2*)x, out, 2, 1, nbatch, b_in, b_out, for_grad != 0, kSo3RotI,
                       nullptr, 1, ws, ws_bytes, as_stream(stream));
}

// ---- S2 transforms -------------------------------------------------------------------------------
size_t s2c_s2_fft_workspace(long nbatch, int b_in, int b_out) {
  const int K = std::min(b_in, b_out), N = 2 * std::max(b_in, b_out);
  return s2_ws_per_z(N, K) * (size_t)std::max(1L, nbatch);
}

int s2c_s2_fft(const float* x, int x_is_real, float* out, long nbatch, int b_in, int b_out,
               int for_grad, void* ws, size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_s2_fft: bad argument");
  if (b_out > b_in) return fail(S2C_ERR_BAD_ARG, "s2c_s2_fft: requires b_out <= b_in");
  stream_t st = as_stream(stream);
  const int N = 2 * b_in, K = b_out;
  FftDev fft;
  PanelsDev pan;
  S2C_TRY(TableCache::get().fft(N, fft));
  S2C_TRY(TableCache::get().panels(b_in, b_out, K, !for_grad, true, pan));
  if (!g_force_general && x_is_real && N % 2 == 0 && s2_fwd_fused_smem(N) <= 96 * 1024) {
    // real signal whose packed half plane fits in shared memory: one kernel, no scratch
    S2FwdFusedParams f;
    f.x = x; f.out = (float2*)out; f.out_zstride = nbatch;
    f.pan = pan; f.fft = fft; f.N = N; f.K = K;
    return S2C_LAUNCH(s2_fwd_fused, nbatch, kThreads, s2_fwd_fused_smem(N), st, f);
  }
  const size_t per_z = s2_ws_per_z(N, K);
  long chunk = (long)std::min<size_t>((size_t)nbatch, ws_bytes / per_z);
  if (chunk < 1 || !ws) return fail(S2C_ERR_WORKSPACE, "s2c_s2_fft: workspace too small");
  const int G = fft_group(N, N), Gg = fft_group(N, N / 2);  // alpha passes, gamma passes
  for (long z0 = 0; z0 < nbatch; z0 += chunk) {
    const long zc = std::min(chunk, nbatch - z0);
    FwdAlphaParams a;
    a.in = x + (size_t)z0 * N * N * (x_is_real ? 1 : 2);
    a.in_real = x_is_real ? 1 : 0;
    a.v = (float2*)ws;
    a.nbatch = (int)zc; a.N = N; a.K = K; a.Kn = 1; a.G = G;
    a.nrows = zc * N;
    a.fft = fft;
    S2C_TRY(S2C_LAUNCH(so3_fwd_alpha, (a.nrows + G - 1) / G, kThreads, fft_smem_bytes(N, G), st, a));
    FwdWignerParams w;
    w.v = (const float2*)ws;
    w.out = (float2*)out + z0;
    w.out_zstride = nbatch;
    w.pan = pan;
    w.nbatch = (int)zc; w.N = N; w.K = K; w.nl = b_out;
    w.ZT = (int)std::min<long>(32, zc);
    w.nzt = (int)((zc + w.ZT - 1) / w.ZT);
    w.mode = kS2;
    const size_t wsm = align_up((size_t)b_out * (N + 1) * sizeof(float), 16) +
                       (size_t)w.ZT * (N + 1) * sizeof(float2);
    S2C_TRY(S2C_LAUNCH(so3_fwd_wigner, (long)pan.npairs * w.nzt, kThreads, wsm, st, w));
  }
  return S2C_OK;
}

int s2c_s2_ifft(const float* x, float* out, int out_is_real, long nbatch, int b_in, int b_out,
                int for_grad, void* ws, size_t ws_bytes, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_s2_ifft: bad argument");
  if (b_out < b_in) return fail(S2C_ERR_BAD_ARG, "s2c_s2_ifft: requires b_out >= b_in");
  stream_t st = as_stream(stream);
  const int N = 2 * b_out, K = b_in;
  FftDev fft;
  PanelsDev pan;
  S2C_TRY(TableCache::get().fft(N, fft));
  S2C_TRY(TableCache::get().panels(b_out, b_in, K, for_grad != 0, true, pan));
  const size_t per_z = s2_ws_per_z(N, K);
  long chunk = (long)std::min<size_t>((size_t)nbatch, ws_bytes / per_z);
  if (chunk < 1 || !ws) return fail(S2C_ERR_WORKSPACE, "s2c_s2_ifft: workspace too small");
  const int G = fft_group(N, N), Gg = fft_group(N, N / 2);  // alpha passes, gamma passes
  for (long z0 = 0; z0 < nbatch; z0 += chunk) {
    const long zc = std::min(chunk, nbatch - z0);
    InvWignerParams w;
    w.x = (const float2*)x + z0;
    w.x_zstride = nbatch;
    w.s = (float2*)ws;
    w.pan = pan;
    w.nbatch = (int)zc; w.N = N; w.K = K;
    w.ZT = (int)std::min<long>(32, zc);
    w.nzt = (int)((zc + w.ZT - 1) / w.ZT);
    w.mode = kS2;
    const size_t wsm = align_up((size_t)K * N * sizeof(float), 16) + (size_t)K * w.ZT * sizeof(float2);
    S2C_TRY(S2C_LAUNCH(so3_inv_wigner, (long)pan.npairs * w.nzt, kThreads, wsm, st, w));
    InvAlphaParams a;
    a.s = (const float2*)ws;
    a.out = out + (size_t)z0 * N * N * (out_is_real ? 1 : 2);
    a.out_real = out_is_real ? 1 : 0;
    a.herm_n0 = 0;
    a.nbatch = (int)zc; a.N = N; a.K = K; a.Kn = 1; a.G = G;
    a.nrows = zc * N;
    a.fft = fft;
    S2C_TRY(S2C_LAUNCH(so3_inv_alpha, (a.nrows + G - 1) / G, kThreads, fft_smem_bytes(N, G), st, a));
  }
  return S2C_OK;
}

// ---- spectral products ---------------------------------------------------------------------------
#ifndef S2C_EMUL
static __device__ int g_tc_err_flag;
#endif

#ifndef S2C_EMUL
// so3_mm or one of its gradients on the tensor cores; `handled` tells whether the shape qualified.
static int so3_mm_tc_launch(int op, const float* a, const float* b, float* c, int nl, int nb, int fi,
                            int fo, stream_t st, bool* handled) {
  *handled = !g_force_general;
  if (!*handled) return S2C_OK;
  MmTcParams p;
  p.a = a; p.b = b; p.c = c;
  p.nl = nl; p.nb = nb; p.fi = fi; p.fo = fo;
  p.run = 2 * (op == kTcFwd ? fi : op == kTcGradX ? fo : nb);
  if (p.run <= kTcKMax) { p.kblk = (p.run + 7) / 8 * 8; p.nblk = 1; }
  else { p.kblk = kTcKMax; p.nblk = (p.run + kTcKMax - 1) / kTcKMax; }
  void* flag = nullptr;
  S2C_TRY(cuda_check(cudaGetSymbolAddress(&flag, g_tc_err_flag), "tensor-core status flag"));
  p.err = (int*)flag;
  // Few output tiles (the grad-y product: its rows are only (p, k)) leave most SMs idle: several
  // CTAs then share a tile, each contracting a slice of the outer index and adding its partial
  // result atomically into the zeroed output (float additions in arrival order).
  p.ksplit = 1;
  {
    const long plain = so3_mm_tc_tiles(op, nl, nb, fi, fo);
    if (op == kTcGradY && plain < 100 && nl > 1) p.ksplit = (int)std::min<long>(8, (148 + plain - 1) / plain);
  }
  if (p.ksplit > 1) {
    const size_t out_bytes = (size_t)so3_nspec(nl) * fi * fo * sizeof(float2);
    S2C_TRY(cuda_check(cudaMemsetAsync(c, 0, out_bytes, st), "so3_mm split-K output clear"));
  }
  const long tiles = so3_mm_tc_tiles(op, nl, nb, fi, fo, p.ksplit);
  // longest K loop of any CTA
  const long lmax = 2 * nl - 1;
  const long chain_mmas = ((lmax + p.ksplit - 1) / p.ksplit) * (long)((p.run + 7) / 8) * 3;
  const bool flush = chain_mmas > kTcChainMax;
  const bool vec = so3_mm_tc_vec16(op, nb, fi, fo);
#define S2C_TC_LAUNCH2(OP, FL, NAME)                                                               \
  (vec ? launch_impl(so3_mm_tc_kernel<OP, FL, true>, NAME, tiles, kTcThreads, kTcSmemBytes, st, p)  \
       : launch_impl(so3_mm_tc_kernel<OP, FL, false>, NAME, tiles, kTcThreads, kTcSmemBytes, st, p))
#define S2C_TC_LAUNCH(OP, NAME) (flush ? S2C_TC_LAUNCH2(OP, true, NAME) : S2C_TC_LAUNCH2(OP, false, NAME))
  if (op == kTcFwd) return S2C_TC_LAUNCH(kTcFwd, "so3_mm_tc_kernel");
  if (op == kTcGradX) return S2C_TC_LAUNCH(kTcGradX, "so3_mm_tc_gradx");
  return S2C_TC_LAUNCH(kTcGradY, "so3_mm_tc_grady");
}

// A plain real product C[r][c] = sum_k A[r][k] B[c][k] (M rows, N columns, K terms; N and K even)
// on the tensor-core pipeline: the kernel-grid -> spectrum transforms and their transposes.
static int plain_tc_launch(bool a_strided, const float* a, const float* b, float* c, long M, long N,
                           long K, long a_rs, long a_ps, long b_rs, long b_ps, long c_rs, long c_ps,
                           stream_t st) {
  MmTcParams p;
  p.a = a; p.b = b; p.c = c;
  p.nl = 1; p.nb = (int)M; p.fi = (int)(K / 2); p.fo = (int)(N / 2);
  p.run = (int)K;
  if (p.run <= kTcKMax) { p.kblk = (p.run + 7) / 8 * 8; p.nblk = 1; }
  else { p.kblk = kTcKMax; p.nblk = (p.run + kTcKMax - 1) / kTcKMax; }
  p.ksplit = 1;
  p.a_rs = a_rs; p.a_ps = a_ps; p.b_rs = b_rs; p.b_ps = b_ps; p.c_rs = c_rs; p.c_ps = c_ps;
  void* flag = nullptr;
  S2C_TRY(cuda_check(cudaGetSymbolAddress(&flag, g_tc_err_flag), "tensor-core status flag"));
  p.err = (int*)flag;
  const long tiles = ((M + kTcBM - 1) / kTcBM) * ((N + kTcBN - 1) / kTcBN);
  const bool flush = (long)((p.run + 7) / 8) * 3 > kTcChainMax;
  // 16-byte loads need K a multiple of 4 and 16-byte aligned rows of every contiguous operand
  const bool vec = K % 4 == 0 && b_rs % 4 == 0 && (a_strided || a_rs % 4 == 0);
  if (a_strided) return S2C_TC_LAUNCH(kTcPlainSC, "rft_tc_backward");
  return S2C_TC_LAUNCH(kTcPlainCC, "rft_tc_forward");
#undef S2C_TC_LAUNCH2
#undef S2C_TC_LAUNCH
}
#endif

int s2c_so3_mm(const float* x, const float* y, float* z, int nl, int nb, int fi, int fo, void* st) {
  if (!x || !y || !z) return fail(S2C_ERR_BAD_ARG, "s2c_so3_mm: null pointer");
  if (nl < 1 || nb < 1 || fi < 1 || fo < 1) return fail(S2C_ERR_BAD_ARG, "sizes must be >= 1");
#ifndef S2C_EMUL
  bool handled = false;
  S2C_TRY(so3_mm_tc_launch(kTcFwd, x, y, z, nl, nb, fi, fo, as_stream(st), &handled));
  if (handled) return S2C_OK;
#endif
  return mm_dispatch(true, kMmFwd, x, y, z, nl, nb, fi, fo, as_stream(st));
}

int s2c_so3_mm_tc_status(void) {
#ifndef S2C_EMUL
  // wait for every stream of the device (the products run on the caller's streams, which a plain
  // copy from the symbol would not be ordered after), then read the flag
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_err_flag, sizeof(int)) != cudaSuccess) return -1;
  return v;
#else
  return 0;
#endif
}
int s2c_so3_mm_gradx(const float* gz, const float* y, float* gx, int nl, int nb, int fi, int fo,
                     void* st) {
  if (!gz || !y || !gx) return fail(S2C_ERR_BAD_ARG, "s2c_so3_mm_gradx: null pointer");
  if (nl < 1 || nb < 1 || fi < 1 || fo < 1) return fail(S2C_ERR_BAD_ARG, "sizes must be >= 1");
#ifndef S2C_EMUL
  bool handled = false;
  S2C_TRY(so3_mm_tc_launch(kTcGradX, gz, y, gx, nl, nb, fi, fo, as_stream(st), &handled));
  if (handled) return S2C_OK;
#endif
  return mm_dispatch(true, kMmGradX, gz, y, gx, nl, nb, fi, fo, as_stream(st));
}
int s2c_so3_mm_grady(const float* gz, const float* x, float* gy, int nl, int nb, int fi, int fo,
                     void* st) {
  if (!gz || !x || !gy) return fail(S2C_ERR_BAD_ARG, "s2c_so3_mm_grady: null pointer");
  if (nl < 1 || nb < 1 || fi < 1 || fo < 1) return fail(S2C_ERR_BAD_ARG, "sizes must be >= 1");
#ifndef S2C_EMUL
  bool handled = false;
  S2C_TRY(so3_mm_tc_launch(kTcGradY, x, gz, gy, nl, nb, fi, fo, as_stream(st), &handled));
  if (handled) return S2C_OK;
#endif
  return mm_dispatch(true, kMmGradY, x, gz, gy, nl, nb, fi, fo, as_stream(st));
}
int s2c_s2_mm(const float* x, const float* y, float* z, int nl, int nb, int fi, int fo, void* st) {
  if (!x || !y || !z) return fail(S2C_ERR_BAD_ARG, "s2c_s2_mm: null pointer");
  return mm_dispatch(false, kMmFwd, x, y, z, nl, nb, fi, fo, as_stream(st));
}
int s2c_s2_mm_gradx(const float* gz, const float* y, float* gx, int nl, int nb, int fi, int fo,
                    void* st) {
  if (!gz || !y || !gx) return fail(S2C_ERR_BAD_ARG, "s2c_s2_mm_gradx: null pointer");
  if (nl < 1 || nb < 1 || fi < 1 || fo < 1) return fail(S2C_ERR_BAD_ARG, "sizes must be >= 1");
  if (!g_force_general && s2_mm_thin_supported(nl, fi, fo)) {
    S2ThinParams p;
    p.gz = (const float2*)gz; p.other = (const float2*)y; p.out = (float2*)gx;
    p.nl = nl; p.nb = nb; p.fi = fi; p.fo = fo;
    const long blocks = (long)nl * nl * ((nb + kThinRows - 1) / kThinRows);
    return S2C_LAUNCH(s2_mm_gradx_thin, blocks, kThinRows * kThinSlices,
                      s2_gradx_thin_smem(nl, fi, fo), as_stream(st), p);
  }
  return mm_dispatch(false, kMmGradX, gz, y, gx, nl, nb, fi, fo, as_stream(st));
}
int s2c_s2_mm_grady(const float* gz, const float* x, float* gy, int nl, int nb, int fi, int fo,
                    void* st) {
  if (!gz || !x || !gy) return fail(S2C_ERR_BAD_ARG, "s2c_s2_mm_grady: null pointer");
  if (nl < 1 || nb < 1 || fi < 1 || fo < 1) return fail(S2C_ERR_BAD_ARG, "sizes must be >= 1");
  if (!g_force_general && s2_mm_thin_supported(nl, fi, fo)) {
    S2ThinParams p;
    p.gz = (const float2*)gz; p.other = (const float2*)x; p.out = (float2*)gy;
    p.nl = nl; p.nb = nb; p.fi = fi; p.fo = fo;
    return S2C_LAUNCH(s2_mm_grady_thin, (long)nl * nl, s2_grady_thin_threads(fo),
                      s2_grady_thin_smem(fo), as_stream(st), p);
  }
  return mm_dispatch(false, kMmGradY, x, gz, gy, nl, nb, fi, fo, as_stream(st));
}

// ---- kernel-grid -> spectrum -----------------------------------------------------------------------
int s2c_rft_forward(const float* x, const float* F, float* out, int nf, int ng, int ns, void* st) {
  if (!x || !F || !out || nf < 1 || ng < 1 || ns < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_rft_forward: bad argument");
  RftFwdParams p;
  p.x = x; p.F = (const float2*)F; p.out = (float2*)out;
  p.nf = nf; p.ng = ng; p.ns = ns;
  p.tiles_f = (nf + kRftTF - 1) / kRftTF;
  const long tiles_s = (ns + kRftTS - 1) / kRftTS;
  const size_t sm = kRftTF * (kRftTA + 1) * 4 + kRftTA * kRftTS * 8;
  return S2C_LAUNCH(rft_forward, p.tiles_f * tiles_s, 256, sm, as_stream(st), p);
}

int s2c_rft_forward_t(const float* x, const float* Ft, float* out, int nf, int ng, int ns, void* st) {
  if (!x || !Ft || !out || nf < 1 || ng < 1 || ns < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_rft_forward_t: bad argument");
#ifndef S2C_EMUL
  if (ng % 2 == 0) {
    // C[f][(s, c)] = sum_a x[f][a] Ft[(s, c)][a], written to out[s][f][c]
    return plain_tc_launch(false, x, Ft, out, nf, 2L * ns, ng, ng, 2, ng, 2, 2, 2L * nf, as_stream(st));
  }
#endif
  return fail(S2C_ERR_UNSUPPORTED, "s2c_rft_forward_t: needs the CUDA build and an even n_grid");
}

int s2c_rft_backward(const float* g, const float* F, float* gx, int nf, int ng, int ns, void* st) {
  if (!g || !F || !gx || nf < 1 || ng < 1 || ns < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_rft_backward: bad argument");
#ifndef S2C_EMUL
  if (!g_force_general && ng % 2 == 0) {
    // gx[f][a] = sum_{(s, c)} g[s][f][c] F[a][(s, c)]: the row operand holds k = (s, c) as pairs
    // 2 nf floats apart
    return plain_tc_launch(true, g, F, gx, nf, ng, 2L * ns, 2, 2L * nf, 2L * ns, 2, ng, 2, as_stream(st));
  }
#endif
  RftBwdParams p;
  p.g = (const float2*)g; p.F = (const float2*)F; p.gx = gx;
  p.nf = nf; p.ng = ng; p.ns = ns;
  p.tiles_f = (nf + kRftTF - 1) / kRftTF;
  const long tiles_a = (ng + kRftTA - 1) / kRftTA;
  const size_t sm = kRftTS * kRftTF * 8 + kRftTA * (kRftTS + 1) * 8;
  return S2C_LAUNCH(rft_backward, p.tiles_f * tiles_a, 256, sm, as_stream(st), p);
}

// ---- integration ---------------------------------------------------------------------------------
int s2c_so3_integrate(const float* x, float* out, long n, int b, int relu, void* st) {
  if (!x || !out || n < 1 || b < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_integrate: bad argument");
  IntegrateParams p;
  p.x = x; p.out = out; p.n = n; p.N = 2 * b; p.relu = relu;
  S2C_TRY(TableCache::get().quad_weights(b, &p.w));
  return S2C_LAUNCH(so3_integrate_fwd, (n + kIntegrateWarps - 1) / kIntegrateWarps,
                    32 * kIntegrateWarps, 32 * kIntegrateWarps * sizeof(float), as_stream(st), p);
}

int s2c_so3_integrate_backward(const float* g, const float* x, float* gx, long n, int b, int relu,
                               void* st) {
  if (!g || !gx || n < 1 || b < 1 || (relu && !x))
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_integrate_backward: bad argument");
  IntegrateBwdParams p;
  p.g = g; p.x = x; p.gx = gx; p.N = 2 * b; p.relu = relu;
  p.total = n * (long)p.N * p.N * p.N;
  S2C_TRY(TableCache::get().quad_weights(b, &p.w));
  const long blocks = std::min<long>((p.total + 255) / 256, 148L * 16);
  return S2C_LAUNCH(so3_integrate_bwd, blocks, 256, 0, as_stream(st), p);
}

int s2c_project_on_sphere(const float* verts, int nv, const int* faces, int nf, const float* grid,
                          int nr, float* out, void* st) {
  if (!verts || !faces || !grid || !out || nv < 1 || nf < 1 || nr < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_project_on_sphere: bad argument");
  ProjectParams p;
  p.verts = verts; p.faces = faces; p.grid = grid; p.out = out;
  p.nv = nv; p.nf = nf; p.nr = nr;
  return S2C_LAUNCH(project_on_sphere, (nr + kProjThreads - 1) / kProjThreads, kProjThreads,
                    kProjTile * 12 * sizeof(float), as_stream(st), p);
}

int s2c_so3_rotation_matrices(int b, double alpha, double beta, double gamma, float* out) {
  if (b < 1 || !out) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rotation_matrices: bad argument");
  std::vector<double> col(b + 1);
  for (int m = -(b - 1); m <= b - 1; ++m)
    for (int n = -(b - 1); n <= b - 1; ++n) {
      const int l0 = wigner_d_degrees(m, n, beta, b, col.data());
      const double ph = m * alpha + n * gamma;
      const double cr = std::cos(ph), ci = std::sin(ph);
      for (int l = l0; l < b; ++l) {
        const long idx = so3_offset(l) + (long)(m + l) * (2 * l + 1) + (n + l);
        out[2 * idx] = (float)(cr * col[l - l0]);
        out[2 * idx + 1] = (float)(ci * col[l - l0]);
      }
    }
  return S2C_OK;
}

int s2c_so3_rotate_spectrum(const float* U, const float* x, float* z, int b, long nbatch,
                            int adjoint, void* st) {
  if (!U || !x || !z || b < 1 || nbatch < 1 || nbatch > 0x7fffffffL / (2 * b))
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rotate_spectrum: bad argument");
  CgemmParams p = rotation_params(b, nbatch, adjoint ? 1 : 0);
  p.A = (const float2*)U;
  p.B = (const float2*)x;
  p.C = (float2*)z;
  return S2C_LAUNCH(cgemm_grouped, cgemm_total_tiles(p), 256, cgemm_smem_bytes(), as_stream(st), p);
}


}  // extern "C"

// ================================================================================================
// s2c_so3_rifft_static: the SO(3) synthesis without any device allocation.
//
// Some callers of this library cannot obtain device memory at call time: a serving process whose
// whole GPU is pre-reserved by another allocator at start-up (a later cudaMalloc simply fails), or
// a control loop that must not take the device-wide synchronisation a cudaMalloc/cudaFree implies.
// For them the scratch arrays of the synthesis and the constant tables it reads live in the two
// file-scope device arrays below, which every GPU that loads this library holds until the process
// exits (kStaticScratchBytes + kStaticTableBytes = 36 MiB per GPU).
//
// In host code the array names are host-side stand-ins, not device addresses; the device address
// is fetched once per device with cudaGetSymbolAddress (with that device current) and handed to
// the kernels.  That set-up, and the (synchronous) upload of the tables for the requested
// bandwidths, happen on the first call on a device and again whenever a call asks for different
// bandwidths / weighting than the tables currently held - make such a call before any stream
// capture.  All calls on a device share the arrays: the scratch keeps the previous call's
// contents (every element a pass reads has been written by the pass before it in the same call,
// so nothing needs clearing), and two calls that overlap on the GPU - different streams or host
// threads - race on it.
// ================================================================================================
namespace s2c {

constexpr size_t kStaticScratchBytes = (size_t)32 << 20;
constexpr size_t kStaticTableBytes = (size_t)4 << 20;

#ifndef S2C_EMUL
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) unsigned char g_static_tables[kStaticTableBytes];
#else
alignas(256) static unsigned char g_static_scratch[kStaticScratchBytes];
alignas(256) static unsigned char g_static_tables[kStaticTableBytes];
#endif

struct StaticDeviceState {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device addresses of the two arrays on this device
  unsigned char* tables = nullptr;
  int b_beta = -1, K = -1, weighted = -1;  // configuration the table array currently holds
  FftDev fft;
  PanelsDev pan;
};

static std::mutex g_static_mu;
static std::map<int, StaticDeviceState> g_static_state;

static int static_setup(StaticDeviceState& st) {
  if (st.ready) return S2C_OK;
#ifndef S2C_EMUL
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
  if (e != cudaSuccess) return cuda_check(e, "cudaGetSymbolAddress(scratch)");
  st.scratch = (unsigned char*)p;
  e = cudaGetSymbolAddress(&p, g_static_tables);
  if (e != cudaSuccess) return cuda_check(e, "cudaGetSymbolAddress(tables)");
  st.tables = (unsigned char*)p;
#else
  st.scratch = g_static_scratch;
  st.tables = g_static_tables;
#endif
  st.ready = true;
  return S2C_OK;
}

// Builds the FFT and Wigner tables for (b_beta, K, weighted) on the host and copies them into the
// static table array (no allocation; cudaMemcpy waits for the copy).
static int static_load_tables(StaticDeviceState& st, int b_beta, int K, bool weighted,
                              stream_t stream) {
  if (st.b_beta == b_beta && st.K == K && st.weighted == (int)weighted) return S2C_OK;
  const int N = 2 * b_beta;
  FftDev f;
  if (!fft_plan(N, f.desc))
    return fail(S2C_ERR_UNSUPPORTED, "s2c_so3_rifft_static: unsupported FFT length");
  std::vector<float> tw;
  std::vector<unsigned short> pos;
  fft_twiddles(N, tw);
  fft_positions(f.desc, pos);
  std::vector<float> pdata;
  std::vector<long long> poff;
  TableCache::build_panels(b_beta, K, K, weighted, false, pdata, poff);
  const size_t o_tw = 0;
  const size_t o_pos = align_up(o_tw + tw.size() * sizeof(float), 256);
  const size_t o_off = align_up(o_pos + pos.size() * sizeof(unsigned short), 256);
  const size_t o_dat = align_up(o_off + poff.size() * sizeof(long long), 256);
  const size_t total = o_dat + pdata.size() * sizeof(float);
  if (total > kStaticTableBytes)
    return fail(S2C_ERR_UNSUPPORTED,
                "s2c_so3_rifft_static: tables for these bandwidths need " + std::to_string(total) +
                    " bytes, the static table array holds " + std::to_string(kStaticTableBytes));
#ifndef S2C_EMUL
  // Kernels of an earlier call on this stream may still be reading the old tables.  Only the
  // caller's stream is waited for: calls on other streams must not overlap this one anyway (they
  // would race on the shared arrays, as the header says).
  S2C_TRY(cuda_check(cudaStreamSynchronize(stream), "stream sync before table reload"));
#endif
  (void)stream;
  // From here on the array no longer holds a complete table set: forget the old key first, so that
  // a failed upload cannot leave a later call with the old bandwidths reading a half-written array.
  st.b_beta = st.K = st.weighted = -1;
  S2C_TRY(dev_upload(st.tables + o_tw, tw.data(), tw.size() * sizeof(float)));
  S2C_TRY(dev_upload(st.tables + o_pos, pos.data(), pos.size() * sizeof(unsigned short)));
  S2C_TRY(dev_upload(st.tables + o_off, poff.data(), poff.size() * sizeof(long long)));
  S2C_TRY(dev_upload(st.tables + o_dat, pdata.data(), pdata.size() * sizeof(float)));
  f.tw = (const float2*)(st.tables + o_tw);
  f.pos = (const unsigned short*)(st.tables + o_pos);
  st.fft = f;
  st.pan.nbeta = N;
  st.pan.nl = K;
  st.pan.K = K;
  st.pan.npairs = (int)poff.size() - 1;
  st.pan.s2 = 0;
  st.pan.nrows = (int)(poff.back() / N);
  st.pan.rowmap = nullptr;
  st.pan.data_g = nullptr;
  st.pan.g_bg = 0;
  st.pan.g_stride = 0;
  st.pan.order = nullptr;
  st.pan.off = (const long long*)(st.tables + o_off);
  st.pan.data = (const float*)(st.tables + o_dat);
  st.b_beta = b_beta;
  st.K = K;
  st.weighted = (int)weighted;
  return S2C_OK;
}

}  // namespace s2c

extern "C" {

size_t s2c_so3_rifft_static_max_bytes(void) { return kStaticScratchBytes; }

int s2c_so3_rifft_static(const float* x, float* out, long nbatch, int b_in, int b_out,
                         int for_grad, const float* bias, int nfeature, void* stream) {
  S2C_TRY(check_b(b_in, b_out));
  if (!x || !out || nbatch < 1) return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_static: bad argument");
  if (bias && nfeature < 1)
    return fail(S2C_ERR_BAD_ARG, "s2c_so3_rifft_static: nfeature must be >= 1 with a bias");
  const int N = 2 * b_out, K = std::min(b_in, b_out);
  // scratch of the synthesis: both arrays are laid out on the OUTPUT grid (2 b_out samples per axis)
  const size_t need = so3_ws_per_z(N, K) * (size_t)nbatch;
  if (need > kStaticScratchBytes)
    return fail(S2C_ERR_WORKSPACE,
                "s2c_so3_rifft_static: this call needs " + std::to_string(need) +
                    " bytes of scratch, the static array holds " +
                    std::to_string(kStaticScratchBytes) + " (use s2c_so3_rifft with a workspace)");
  stream_t st = as_stream(stream);
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticDeviceState& dev = g_static_state[dev_current()];
  S2C_TRY(static_setup(dev));
  S2C_TRY(static_load_tables(dev, b_out, K, for_grad != 0, st));

  const int G = fft_group(N, N), Gg = fft_group(N, N / 2);  // alpha passes, gamma passes
  const size_t fft_smem = fft_smem_bytes(N, G);
  float2* t = (float2*)dev.scratch;                   // [z][K][N][N]
  float2* s = t + (size_t)nbatch * K * N * N;         // [K][2K-1][z][N]
  InvWignerParams w;
  w.x = (const float2*)x;
  w.x_zstride = nbatch;
  w.s = s;
  w.pan = dev.pan;
  w.nbatch = (int)nbatch; w.N = N; w.K = K;
  w.ZT = (int)std::min<long>(32, nbatch);
  w.nzt = (int)((nbatch + w.ZT - 1) / w.ZT);
  w.mode = kSo3Real;
  const size_t wsm = align_up((size_t)K * N * sizeof(float), 16) + (size_t)K * w.ZT * sizeof(float2);
  S2C_TRY(S2C_LAUNCH(so3_inv_wigner, (long)dev.pan.npairs * w.nzt, kThreads, wsm, st, w));
  InvAlphaParams a;
  a.s = s;
  a.out = (float*)t;
  a.out_real = 0;
  a.herm_n0 = 1;
  a.nbatch = (int)nbatch; a.N = N; a.K = K; a.Kn = K; a.G = G;
  a.nrows = nbatch * K * N;
  a.fft = dev.fft;
  S2C_TRY(S2C_LAUNCH(so3_inv_alpha, (a.nrows + G - 1) / G, kThreads, fft_smem, st, a));
  InvGammaParams g;
  g.t = t;
  g.out = out;
  g.out_stride = 1;
  g.out_off = 0;
  g.bias = bias;
  g.nfeat = nfeature > 0 ? nfeature : 1;
  g.z0 = 0;
  g.N = N; g.b = b_out; g.K = K; g.G = Gg;
  g.npairs = nbatch * N * b_out;
  g.fft = dev.fft;
  return S2C_LAUNCH(so3_inv_gamma, (g.npairs + Gg - 1) / Gg, kThreads, fft_smem_bytes(N, Gg), st, g);
}

}  // extern "C"
