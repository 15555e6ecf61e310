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

#include <map>
#include <memory>
#include <mutex>
#include <tuple>

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
};

// ---- configuration of the single-kernel path (shared by the table builder and the kernels) ----
constexpr int kFusedZG = 4;    // batch elements per block
constexpr int kMaxBG = 8;      // upper bound of the betas per group
constexpr int kFusedMaxN = 32;
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

  // Host build of the panel table (also exported for tests).
  static void build_panels(int b_beta, int nl, int K, bool weighted, bool s2,
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
      if (!s2 && 2 * b_beta <= kFusedMaxN) {
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
