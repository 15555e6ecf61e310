// Per-device cache of the constant tables the kernels read: FFT twiddles / digit maps, Wigner-d
// panels and quadrature weights.  Plays the role of the reference's `_setup_wigner` lru_cache
// (s2cnn/soft/so3_fft.py:205-209, s2cnn/soft/s2_fft.py:109-113) and of the table builders
// `_setup_so3_fft` / `_setup_s2_fft` (so3_fft.py:212-243, s2_fft.py:116-147), with a layout chosen
// for the kernels rather than the reference's [beta, lmn]:
//
//   one contiguous panel per frequency pair (m, n):  panel[l - lmin][beta_j]
//       = d^l_mn(beta_j) * (w_j  if weighted  else  2l+1),     lmin = max(|m|, |n|)
//
// SO(3) panels exist only for the half plane  n > 0  or  (n = 0, m >= 0); the mirrored pair
// (-m, -n) is served by d^l_{-m,-n} = (-1)^(m-n) d^l_{mn}.  S2 panels (column n = 0, weight
// w_j * 2b) exist for every |m| < K.
//
// Tables are built in float64 on the host, rounded to float32 and uploaded on first use; the
// first call for a new (bandwidth, kind, device) therefore allocates and copies synchronously.
#pragma once

#include <algorithm>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <tuple>
#ifndef _WIN32
#include <unistd.h>
#endif

#include "backend.h"
#include "host_math.h"

namespace s2c {

struct FftDev {
  FftDesc desc;
  const float2* tw;            // device, n entries exp(+2 pi i k / n)
  const unsigned short* pos;   // device, n entries
};

struct PanelsDev {
  int nbeta;   // 2 * b of the beta grid
  int nl;      // degrees l < nl
  int K;       // frequencies |m|, n < K
  int npairs;
  int s2;      // 1: S2 panels (n = 0, all m), 0: SO(3) half plane
  int nrows;   // total panel rows = off[npairs] / nbeta
  const float* data;        // device
  const long long* off;     // device, npairs + 1 offsets (in floats)
  const int* rowmap;        // device, nrows entries: l | (m + 128) << 8 | n << 16 of each panel row
  // Copy for the single-kernel path (only when nbeta <= 32, else null): the same values regrouped
  // by beta group, data_g[g * g_stride + row * g_bg + bi] = data[row * nbeta + g * g_bg + bi], so
  // that the slice a block needs for one beta group is one contiguous, 16-byte aligned run.
  const float* data_g;
  int g_bg;                 // betas per group
  int g_stride;             // floats per group slice (multiple of 4)
  // Single-kernel path only (else null): the panel rows sorted by (l, n, m).  Threads that walk the
  // rows in this order find the same (l, n) in neighbouring lanes (same address of the second S2
  // spectrum when the product s2_mm is computed on the fly).
  const int* order;
};

// ---- configuration of the single-kernel path (shared by the table builder and the kernels) ----
constexpr int kFusedZG = 4;    // batch elements per block
constexpr int kMaxBG = 8;      // upper bound of the betas per group
constexpr int kFusedMaxN = 32;
constexpr int kFusedMaxThreads = 512;
// Betas per group: the largest divisor of N that keeps the per-group transform count
// (ZG * BG * N/2 threads, one transform each) within one pass of a 256-thread block.
inline int fused_bg(int N) {
  int best = 1;
  for (int d = 1; d <= N; ++d)
    if (N % d == 0 && d <= kMaxBG && kFusedZG * d * (N / 2) <= 256) best = d;
  return best;
}

S2C_HD int so3_npairs(int K) { return K + (K - 1) * (2 * K - 1); }
S2C_HD int so3_pair_index(int m, int n, int K) {
  return n == 0 ? m : K + (n - 1) * (2 * K - 1) + (m + K - 1);
}
S2C_HD void so3_pair_decode(int idx, int K, int& m, int& n) {
  if (idx < K) { m = idx; n = 0; }
  else { const int t = idx - K; n = t / (2 * K - 1) + 1; m = t % (2 * K - 1) - (K - 1); }
}

// ---- optional on-disk cache of the Wigner panel tables ------------------------------------------
// Plays the role of the reference's `cached_dirpklgz` decorator around its table builders
// (s2cnn/utils/decorator.py:54-104, used at s2cnn/soft/so3_fft.py:212 and s2_fft.py:116): the host
// build of a large table (seconds at b = 128) is paid once per machine instead of once per process.
// Unlike the reference's index.pkl read-modify-write it is safe with several processes: one file per
// key, written under a temporary name and moved into place with rename(); a reader checks magic,
// key, sizes and a checksum and rebuilds (and rewrites) the table on any mismatch.  Off unless a
// directory is given (s2c_set_table_cache_dir, or the environment variable S2CNN_B200_TABLE_CACHE).
class TableDiskCache {
 public:
  static TableDiskCache& get() {
    static TableDiskCache c;
    return c;
  }
  void set_dir(const char* dir) {
    std::lock_guard<std::mutex> g(mu_);
    dir_ = dir ? dir : "";
    env_checked_ = true;
  }
  std::string dir() {
    std::lock_guard<std::mutex> g(mu_);
    if (!env_checked_) {
      const char* e = std::getenv("S2CNN_B200_TABLE_CACHE");
      if (e) dir_ = e;
      env_checked_ = true;
    }
    return dir_;
  }
  long hits() const { return hits_; }
  long stores() const { return stores_; }

  struct Key {
    int b_beta, nl, K, weighted, s2;
  };
  bool load(const Key& k, std::vector<float>& data, std::vector<long long>& off) {
    const std::string d = dir();
    if (d.empty()) return false;
    FILE* f = std::fopen(path(d, k).c_str(), "rb");
    if (!f) return false;
    Header h;
    bool ok = std::fread(&h, sizeof(h), 1, f) == 1 && h.magic == kMagic && h.version == kVersion &&
              h.key[0] == k.b_beta && h.key[1] == k.nl && h.key[2] == k.K && h.key[3] == k.weighted &&
              h.key[4] == k.s2 && h.n_off < (1ull << 32) && h.n_data < (1ull << 34);
    if (ok) {
      off.resize((size_t)h.n_off);
      data.resize((size_t)h.n_data);
      ok = std::fread(off.data(), sizeof(long long), off.size(), f) == off.size() &&
           std::fread(data.data(), sizeof(float), data.size(), f) == data.size() &&
           checksum(data, off) == h.checksum;
    }
    std::fclose(f);
    if (ok) ++hits_;
    return ok;
  }
  void store(const Key& k, const std::vector<float>& data, const std::vector<long long>& off) {
    const std::string d = dir();
    if (d.empty()) return;
    const std::string final_path = path(d, k);
    char suffix[64];
    std::snprintf(suffix, sizeof(suffix), ".tmp.%ld.%p", (long)getpid(), (const void*)&data);
    const std::string tmp = final_path + suffix;
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) return;   // the cache is an optimisation: an unwritable directory is not an error
    Header h;
    h.magic = kMagic; h.version = kVersion;
    h.key[0] = k.b_beta; h.key[1] = k.nl; h.key[2] = k.K; h.key[3] = k.weighted; h.key[4] = k.s2;
    h.n_off = off.size(); h.n_data = data.size();
    h.checksum = checksum(data, off);
    bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1 &&
              std::fwrite(off.data(), sizeof(long long), off.size(), f) == off.size() &&
              std::fwrite(data.data(), sizeof(float), data.size(), f) == data.size();
    ok = (std::fclose(f) == 0) && ok;
    if (ok && std::rename(tmp.c_str(), final_path.c_str()) == 0) ++stores_;
    else std::remove(tmp.c_str());
  }

 private:
  struct Header {
    unsigned magic, version;
    int key[5];
    int pad;
    unsigned long long n_off, n_data, checksum;
  };
  static constexpr unsigned kMagic = 0x54433253u, kVersion = 1;   // "S2CT"
  static std::string path(const std::string& dir, const Key& k) {
    char name[160];
    std::snprintf(name, sizeof(name), "/wigner_%s_b%d_nl%d_K%d_%s.s2ct", k.s2 ? "s2" : "so3", k.b_beta,
                  k.nl, k.K, k.weighted ? "quadrature" : "degree");
    return dir + name;
  }
  static unsigned long long checksum(const std::vector<float>& data, const std::vector<long long>& off) {
    unsigned long long h = 1469598103934665603ull;   // FNV-1a over 64-bit words
    auto mix = [&](unsigned long long v) { h = (h ^ v) * 1099511628211ull; };
    for (long long o : off) mix((unsigned long long)o);
    const size_t n2 = data.size() / 2;
    const unsigned long long* w = reinterpret_cast<const unsigned long long*>(data.data());
    for (size_t i = 0; i < n2; ++i) mix(w[i]);
    if (data.size() & 1) { unsigned u; std::memcpy(&u, &data.back(), 4); mix(u); }
    return h;
  }
  std::mutex mu_;
  std::string dir_;
  bool env_checked_ = false;
  std::atomic<long> hits_{0}, stores_{0};
};

class TableCache {
 public:
  static TableCache& get() {
    static TableCache c;
    return c;
  }

  int fft(int n, FftDev& out) {
    std::lock_guard<std::mutex> g(mu_);
    const int dev = dev_current();
    auto key = std::make_pair(dev, n);
    auto it = fft_.find(key);
    if (it == fft_.end()) {
      FftDev f;
      if (!fft_plan(n, f.desc))
        return fail(S2C_ERR_UNSUPPORTED,
                    "FFT length " + std::to_string(n) + " has a prime factor above " +
                        std::to_string(kMaxRadix));
      if (n > 65535) return fail(S2C_ERR_UNSUPPORTED, "FFT length above 65535");
      std::vector<float> tw;
      std::vector<unsigned short> pos;
      fft_twiddles(n, tw);
      fft_positions(f.desc, pos);
      void* dtw = dev_alloc(tw.size() * sizeof(float));
      void* dpos = dev_alloc(pos.size() * sizeof(unsigned short));
      if (!dtw || !dpos) return fail(S2C_ERR_CUDA, "table allocation failed");
      int rc = dev_upload(dtw, tw.data(), tw.size() * sizeof(float));
      if (rc) return rc;
      rc = dev_upload(dpos, pos.data(), pos.size() * sizeof(unsigned short));
      if (rc) return rc;
      f.tw = (const float2*)dtw;
      f.pos = (const unsigned short*)dpos;
      it = fft_.emplace(key, f).first;
    }
    out = it->second;
    return S2C_OK;
  }

  // Host build of the panel table, through the on-disk cache when one is configured.
  static void build_panels(int b_beta, int nl, int K, bool weighted, bool s2,
                           std::vector<float>& data, std::vector<long long>& off) {
    const TableDiskCache::Key key{b_beta, nl, K, (int)weighted, (int)s2};
    if (TableDiskCache::get().load(key, data, off)) return;
    compute_panels(b_beta, nl, K, weighted, s2, data, off);
    ++computed_count();
    TableDiskCache::get().store(key, data, off);
  }

  // number of panel tables this process has computed from scratch (not read from the disk cache)
  static std::atomic<long>& computed_count() {
    static std::atomic<long> n{0};
    return n;
  }

  static void compute_panels(int b_beta, int nl, int K, bool weighted, bool s2,
                             std::vector<float>& data, std::vector<long long>& off) {
    const int nbeta = 2 * b_beta;
    std::vector<double> beta, w;
    soft_betas(b_beta, beta);
    quadrature_weights(b_beta, w);
    if (s2) for (auto& v : w) v *= 2.0 * b_beta;  // s2cnn/soft/s2_fft.py:124
    const int npairs = s2 ? 2 * K - 1 : so3_npairs(K);
    off.assign(npairs + 1, 0);
    for (int p = 0; p < npairs; ++p) {
      int m, n;
      if (s2) { m = p - (K - 1); n = 0; } else so3_pair_decode(p, K, m, n);
      const int lmin = std::max(std::abs(m), n);
      off[p + 1] = off[p] + (long long)std::max(nl - lmin, 0) * nbeta;
    }
    data.assign((size_t)off[npairs], 0.f);
    std::vector<double> col(nl + 1);
    for (int p = 0; p < npairs; ++p) {
      int m, n;
      if (s2) { m = p - (K - 1); n = 0; } else so3_pair_decode(p, K, m, n);
      const int lmin = std::max(std::abs(m), n);
      if (lmin >= nl) continue;
      float* panel = data.data() + off[p];
      for (int j = 0; j < nbeta; ++j) {
        wigner_d_degrees(m, n, beta[j], nl, col.data());
        for (int l = lmin; l < nl; ++l) {
          const double wt = weighted ? w[j] : (2.0 * l + 1.0);
          panel[(size_t)(l - lmin) * nbeta + j] = (float)(col[l - lmin] * wt);
        }
      }
    }
  }

  // (l, m, n) of every panel row, in panel order.
  static void build_rowmap(int nl, int K, bool s2, std::vector<int>& rowmap) {
    const int npairs = s2 ? 2 * K - 1 : so3_npairs(K);
    rowmap.clear();
    for (int p = 0; p < npairs; ++p) {
      int m, n;
      if (s2) { m = p - (K - 1); n = 0; } else so3_pair_decode(p, K, m, n);
      const int lmin = std::max(std::abs(m), n);
      for (int l = lmin; l < nl; ++l) rowmap.push_back(l | ((m + 128) << 8) | (n << 16));
    }
  }

  int panels(int b_beta, int nl, int K, bool weighted, bool s2, PanelsDev& out) {
    std::lock_guard<std::mutex> g(mu_);
    const int dev = dev_current();
    auto key = std::make_tuple(dev, b_beta, nl, K, (int)weighted, (int)s2);
    auto it = panels_.find(key);
    if (it == panels_.end()) {
      std::vector<float> data;
      std::vector<long long> off;
      build_panels(b_beta, nl, K, weighted, s2, data, off);
      std::vector<int> rowmap;
      build_rowmap(nl, K, s2, rowmap);
      void* dd = dev_alloc(data.size() * sizeof(float));
      void* doff = dev_alloc(off.size() * sizeof(long long));
      void* drm = dev_alloc(rowmap.size() * sizeof(int));
      if (!dd || !doff || !drm) return fail(S2C_ERR_CUDA, "table allocation failed");
      int rc = dev_upload(dd, data.data(), data.size() * sizeof(float));
      if (rc) return rc;
      rc = dev_upload(doff, off.data(), off.size() * sizeof(long long));
      if (rc) return rc;
      rc = dev_upload(drm, rowmap.data(), rowmap.size() * sizeof(int));
      if (rc) return rc;
      PanelsDev pd;
      pd.data_g = nullptr;
      pd.g_bg = 0;
      pd.g_stride = 0;
      pd.order = nullptr;
      if (!s2 && 2 * b_beta <= kFusedMaxN) {
        std::vector<int> order(rowmap.size());
        for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
        auto key_of = [&](int r) {   // l, then n, then m
          const int v = rowmap[(size_t)r];
          return ((v & 0xff) << 16) | (((v >> 16) & 0xff) << 8) | ((v >> 8) & 0xff);
        };
        std::sort(order.begin(), order.end(), [&](int a, int b) { return key_of(a) < key_of(b); });
        void* dord = dev_alloc(order.size() * sizeof(int));
        if (!dord) return fail(S2C_ERR_CUDA, "table allocation failed");
        rc = dev_upload(dord, order.data(), order.size() * sizeof(int));
        if (rc) return rc;
        pd.order = (const int*)dord;
        const int nbeta = 2 * b_beta, bg = fused_bg(nbeta), nrows = (int)rowmap.size();
        const int stride = (nrows * bg + 3) / 4 * 4;
        std::vector<float> grouped((size_t)stride * (nbeta / bg), 0.f);
        for (int g = 0; g < nbeta / bg; ++g)
          for (int r = 0; r < nrows; ++r)
            for (int bi = 0; bi < bg; ++bi)
              grouped[(size_t)g * stride + (size_t)r * bg + bi] = data[(size_t)r * nbeta + g * bg + bi];
        void* dg = dev_alloc(grouped.size() * sizeof(float));
        if (!dg) return fail(S2C_ERR_CUDA, "table allocation failed");
        rc = dev_upload(dg, grouped.data(), grouped.size() * sizeof(float));
        if (rc) return rc;
        pd.data_g = (const float*)dg;
        pd.g_bg = bg;
        pd.g_stride = stride;
      }
      pd.nrows = (int)rowmap.size();
      pd.rowmap = (const int*)drm;
      pd.nbeta = 2 * b_beta;
      pd.nl = nl;
      pd.K = K;
      pd.npairs = (int)off.size() - 1;
      pd.s2 = s2 ? 1 : 0;
      pd.data = (const float*)dd;
      pd.off = (const long long*)doff;
      it = panels_.emplace(key, pd).first;
    }
    out = it->second;
    return S2C_OK;
  }

  // SO(3) panel values regrouped for beta groups of `bg` (layout of PanelsDev::data_g), for kernels
  // that walk the beta axis in groups other than fused_bg(2 b_beta).  stride = floats per group.
  int grouped(int b_beta, int nl, int K, bool weighted, int bg, const float** data_g, int* stride) {
    std::lock_guard<std::mutex> g(mu_);
    const int dev = dev_current();
    auto key = std::make_tuple(dev, b_beta, nl, K, (int)weighted, bg);
    auto it = grouped_.find(key);
    if (it == grouped_.end()) {
      const int nbeta = 2 * b_beta;
      if (bg < 1 || nbeta % bg != 0) return fail(S2C_ERR_BAD_ARG, "grouped table: bad group size");
      std::vector<float> data;
      std::vector<long long> off;
      build_panels(b_beta, nl, K, weighted, false, data, off);
      const int nrows = (int)(off.back() / nbeta);
      const int st = (nrows * bg + 3) / 4 * 4;
      std::vector<float> grouped((size_t)st * (nbeta / bg), 0.f);
      for (int gidx = 0; gidx < nbeta / bg; ++gidx)
        for (int r = 0; r < nrows; ++r)
          for (int bi = 0; bi < bg; ++bi)
            grouped[(size_t)gidx * st + (size_t)r * bg + bi] = data[(size_t)r * nbeta + gidx * bg + bi];
      void* dg = dev_alloc(grouped.size() * sizeof(float));
      if (!dg) return fail(S2C_ERR_CUDA, "table allocation failed");
      const int rc = dev_upload(dg, grouped.data(), grouped.size() * sizeof(float));
      if (rc) return rc;
      it = grouped_.emplace(key, std::make_pair((const float*)dg, st)).first;
    }
    *data_g = it->second.first;
    *stride = it->second.second;
    return S2C_OK;
  }

  // First half of the beta range of every SO(3) panel (rows of nbeta / 2 floats), for kernels that
  // obtain the second half from d^l_{m,n}(pi - beta_j) = (-1)^(l+n) d^l_{-m,n}(beta_j) and the
  // symmetry of the SOFT grid and its quadrature weights under beta -> pi - beta.  `off` holds
  // npairs + 1 offsets in floats (pair order of so3_pair_index).
  int half_panels(int b_beta, int nl, int K, bool weighted, const float** data,
                  const long long** off) {
    std::lock_guard<std::mutex> g(mu_);
    const int dev = dev_current();
    auto key = std::make_tuple(dev, b_beta, nl, K, (int)weighted, 0);
    auto it = half_.find(key);
    if (it == half_.end()) {
      std::vector<float> full;
      std::vector<long long> foff;
      build_panels(b_beta, nl, K, weighted, false, full, foff);
      const int nbeta = 2 * b_beta, nh = nbeta / 2;
      std::vector<long long> hoff(foff.size());
      for (size_t i = 0; i < foff.size(); ++i) hoff[i] = foff[i] / 2;
      std::vector<float> half((size_t)hoff.back());
      const long long nrows = foff.back() / nbeta;
      for (long long r = 0; r < nrows; ++r)
        std::copy(full.begin() + r * nbeta, full.begin() + r * nbeta + nh, half.begin() + r * nh);
      void* dd = dev_alloc(half.size() * sizeof(float));
      void* doff = dev_alloc(hoff.size() * sizeof(long long));
      if (!dd || !doff) return fail(S2C_ERR_CUDA, "table allocation failed");
      int rc = dev_upload(dd, half.data(), half.size() * sizeof(float));
      if (rc) return rc;
      rc = dev_upload(doff, hoff.data(), hoff.size() * sizeof(long long));
      if (rc) return rc;
      it = half_.emplace(key, std::make_pair((const float*)dd, (const long long*)doff)).first;
    }
    *data = it->second.first;
    *off = it->second.second;
    return S2C_OK;
  }

  int quad_weights(int b, const float** out) {
    std::lock_guard<std::mutex> g(mu_);
    const int dev = dev_current();
    auto key = std::make_pair(dev, b);
    auto it = quad_.find(key);
    if (it == quad_.end()) {
      std::vector<double> w;
      quadrature_weights(b, w);
      std::vector<float> wf(w.begin(), w.end());
      void* d = dev_alloc(wf.size() * sizeof(float));
      if (!d) return fail(S2C_ERR_CUDA, "table allocation failed");
      int rc = dev_upload(d, wf.data(), wf.size() * sizeof(float));
      if (rc) return rc;
      it = quad_.emplace(key, (const float*)d).first;
    }
    *out = it->second;
    return S2C_OK;
  }

  void clear() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : fft_) { dev_free((void*)kv.second.tw); dev_free((void*)kv.second.pos); }
    for (auto& kv : panels_) {
      dev_free((void*)kv.second.data);
      dev_free((void*)kv.second.off);
      dev_free((void*)kv.second.rowmap);
      if (kv.second.order) dev_free((void*)kv.second.order);
      if (kv.second.data_g) dev_free((void*)kv.second.data_g);
    }
    for (auto& kv : quad_) dev_free((void*)kv.second);
    for (auto& kv : grouped_) dev_free((void*)kv.second.first);
    for (auto& kv : half_) { dev_free((void*)kv.second.first); dev_free((void*)kv.second.second); }
    half_.clear();
    grouped_.clear();
    fft_.clear();
    panels_.clear();
    quad_.clear();
  }

 private:
  std::mutex mu_;
  std::map<std::pair<int, int>, FftDev> fft_;
  std::map<std::tuple<int, int, int, int, int, int>, PanelsDev> panels_;
  std::map<std::pair<int, int>, const float*> quad_;
  std::map<std::tuple<int, int, int, int, int, int>, std::pair<const float*, int>> grouped_;
  std::map<std::tuple<int, int, int, int, int, int>, std::pair<const float*, const long long*>> half_;
};

}  // namespace s2c
