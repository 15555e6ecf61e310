// Host-side float64 generators for every constant table on the spectral path:
// Wigner-d functions, SOFT quadrature weights, FFT twiddles and digit-reversal maps.
//
// Replaces what the reference obtains from the third-party `lie_learn` package
// (s2cnn/soft/so3_fft.py:213-243, s2cnn/soft/s2_fft.py:117-147, s2cnn/s2_ft.py:27-50,
// s2cnn/so3_ft.py:27-52, s2cnn/soft/so3_integrate.py:32-37).  Written from the published
// mathematics:  d^l(beta) = exp(-i beta J_y) in the |l,m> basis (so d^1_{1,0} = -sin(beta)/sqrt2),
// evaluated by the closed form at l0 = max(|m|,|n|) and the three-term recurrence in l.
#pragma once

#include <cmath>
#include <vector>

#include "backend.h"

namespace s2c {

S2C_HD int so3_nspec(int b) { return b * (4 * b * b - 1) / 3; }
S2C_HD int so3_offset(int l) { return l * (4 * l * l - 1) / 3; }
S2C_HD long so3_row(int l, int m, int n) {
  return (long)so3_offset(l) + (long)(l + m) * (2 * l + 1) + (l + n);
}

// log sqrt( (2l)! / ((l+k)! (l-k)!) )
inline double log_seed_coef(int l, int k) {
  return 0.5 * (std::lgamma(2.0 * l + 1) - std::lgamma((double)l + k + 1) -
                std::lgamma((double)l - k + 1));
}

// coef * c^a * s^b evaluated in the log domain (no premature underflow), exact zeros handled.
inline double seed_value(double logcoef, double c, int a, double s, int b) {
  if ((c == 0.0 && a > 0) || (s == 0.0 && b > 0)) return 0.0;
  double lg = logcoef;
  if (a > 0) lg += a * std::log(std::fabs(c));
  if (b > 0) lg += b * std::log(std::fabs(s));
  double v = std::exp(lg);
  // c = cos(beta/2), s = sin(beta/2) are non-negative on [0, pi]; keep signs for generality
  if (c < 0 && (a & 1)) v = -v;
  if (s < 0 && (b & 1)) v = -v;
  return v;
}

// out[l - l0] = d^l_{mn}(beta) for l = l0 .. nl-1, l0 = max(|m|,|n|).  Returns l0.
inline int wigner_d_degrees(int m, int n, double beta, int nl, double* out) {
  const int am = m < 0 ? -m : m, an = n < 0 ? -n : n;
  const int l0 = am > an ? am : an;
  if (l0 >= nl) return l0;
  const double c = std::cos(0.5 * beta), s = std::sin(0.5 * beta);
  double seed;
  if (m == l0) {            // d^l_{l,n} = (-1)^(l-n) C(l,n) c^(l+n) s^(l-n)
    seed = seed_value(log_seed_coef(l0, n), c, l0 + n, s, l0 - n);
    if ((l0 - n) & 1) seed = -seed;
  } else if (n == l0) {     // d_{m,l} = (-1)^(m-l) d_{l,m}
    seed = seed_value(log_seed_coef(l0, m), c, l0 + m, s, l0 - m);
  } else if (m == -l0) {    // d_{-l,n} = d_{-n,l}
    seed = seed_value(log_seed_coef(l0, n), c, l0 - n, s, l0 + n);
  } else {                  // n == -l0: d_{m,-l} = d_{l,-m}
    seed = seed_value(log_seed_coef(l0, m), c, l0 - m, s, l0 + m);
    if ((l0 + m) & 1) seed = -seed;
  }
  out[0] = seed;
  if (l0 + 1 >= nl) return l0;
  const double cb = std::cos(beta);
  double prev = 0.0, cur = seed;
  int l = l0;
  if (l0 == 0) {  // m = n = 0: d^1_00 = cos(beta); the general step divides by l
    out[1] = cb;
    prev = 1.0;
    cur = cb;
    l = 1;
  }
  const double mn = (double)m * n, m2 = (double)m * m, n2 = (double)n * n;
  for (; l + 1 < nl; ++l) {
    const double l1 = l + 1.0;
    const double num = (2.0 * l + 1.0) * (l * l1 * cb - mn) * cur -
                       l1 * std::sqrt(((double)l * l - m2) * ((double)l * l - n2)) * prev;
    const double den = l * std::sqrt((l1 * l1 - m2) * (l1 * l1 - n2));
    const double next = num / den;
    out[l + 1 - l0] = next;
    prev = cur;
    cur = next;
  }
  return l0;
}

inline void soft_betas(int b, std::vector<double>& beta) {
  beta.resize(2 * b);
  for (int j = 0; j < 2 * b; ++j) beta[j] = M_PI * (2 * j + 1) / (4.0 * b);
}

// SOFT / Driscoll-Healy weights with sum_j w_j = 1/(2b)^2  (what lie_learn's
// S3.quadrature_weights must return for the reference's round-trip tests to hold).
inline void quadrature_weights(int b, std::vector<double>& w) {
  w.resize(2 * b);
  for (int j = 0; j < 2 * b; ++j) {
    const double th = M_PI * (2 * j + 1) / (4.0 * b);
    double s = 0.0;
    for (int k = 0; k < b; ++k) s += std::sin(th * (2 * k + 1)) / (2 * k + 1);
    w[j] = (2.0 / b) * std::sin(th) * s / (2.0 * (2.0 * b) * (2.0 * b));
  }
}

// ---- FFT planning -------------------------------------------------------------------------
constexpr int kMaxFftStages = 12;
constexpr int kMaxRadix = 32;

struct FftDesc {
  int n;
  int nstage;
  int radix[kMaxFftStages];
};

// Factor n into radices (4s first, then 2, 3, 5, then remaining primes).  Returns false when a
// prime factor exceeds kMaxRadix.
inline bool fft_plan(int n, FftDesc& d) {
  d.n = n;
  d.nstage = 0;
  int r = n;
  while (r % 4 == 0) { d.radix[d.nstage++] = 4; r /= 4; }
  while (r % 2 == 0) { d.radix[d.nstage++] = 2; r /= 2; }
  for (int p = 3; p <= r; p += 2) {
    while (r % p == 0) {
      if (p > kMaxRadix || d.nstage >= kMaxFftStages) return false;
      d.radix[d.nstage++] = p;
      r /= p;
    }
  }
  if (n == 1) { d.radix[0] = 1; d.nstage = 0; }
  return r == 1;
}

// Position of frequency k after the in-place decimation-in-frequency stages of fft_plan's
// radix order: k = p1 + r1 (p2 + r2 (p3 + ...)),  pos = p1 n/r1 + p2 n/(r1 r2) + ...
inline void fft_positions(const FftDesc& d, std::vector<unsigned short>& pos) {
  pos.resize(d.n);
  for (int k = 0; k < d.n; ++k) {
    int kk = k, len = d.n, p = 0;
    for (int s = 0; s < d.nstage; ++s) {
      const int r = d.radix[s];
      len /= r;
      p += (kk % r) * len;
      kk /= r;
    }
    pos[k] = (unsigned short)p;
  }
}

inline void fft_twiddles(int n, std::vector<float>& tw) {
  tw.resize(2 * (size_t)n);
  for (int k = 0; k < n; ++k) {
    const double a = 2.0 * M_PI * k / n;
    tw[2 * k] = (float)std::cos(a);
    tw[2 * k + 1] = (float)std::sin(a);
  }
}

}  // namespace s2c
