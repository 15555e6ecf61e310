// Register-resident FFT of compile-time length N (N <= 32): one thread transforms one whole
// row or column held in registers - no shared-memory exchange and no barrier inside a 1-D
// transform.  Same algorithm and radix order as fft_device.h (in-place decimation in frequency,
// radices 4, 2, then odd primes ascending; output digit-reversed).  Every loop index is a
// compile-time constant, so the array stays in registers, twiddle factors are immediates
// (evaluated in double precision by the compiler) and multiplications by 1, -1, +-i vanish.
#pragma once

#include <type_traits>

#include "fft_device.h"

namespace s2c {

template <int I, int E, class F>
S2C_D void static_for(F&& f) {
  if constexpr (I < E) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, E>(f);
  }
}

S2C_HD constexpr int fft_pick_radix(int len) {
  if (len % 4 == 0) return 4;
  if (len % 2 == 0) return 2;
  for (int p = 3; p <= len; p += 2)
    if (len % p == 0) return p;
  return len;
}

// position of frequency k in the digit-reversed output (matches host fft_positions)
template <int N>
S2C_HD constexpr int fft_reg_pos(int k) {
  int len = N, p = 0, kk = k;
  while (len > 1) {
    const int r = fft_pick_radix(len);
    len /= r;
    p += (kk % r) * len;
    kk /= r;
  }
  return p;
}

// ---- compile-time cos / sin of 2 pi k / n ----------------------------------------------------
S2C_HD constexpr double cx_sin_series(double x) {  // |x| <= pi/4
  double term = x, sum = x;
  for (int i = 1; i < 12; ++i) {
    term *= -x * x / ((2.0 * i) * (2.0 * i + 1.0));
    sum += term;
  }
  return sum;
}
S2C_HD constexpr double cx_cos_series(double x) {  // |x| <= pi/4
  double term = 1.0, sum = 1.0;
  for (int i = 1; i < 12; ++i) {
    term *= -x * x / ((2.0 * i - 1.0) * (2.0 * i));
    sum += term;
  }
  return sum;
}
// cos and sin of 2 pi num / den by octant reduction on the exact fraction (so multiples of pi/4
// come out to series rounding, ~1e-17)
S2C_HD constexpr double cx_cos_turn(long long num, long long den) {
  num %= den;
  if (num < 0) num += den;
  if (2 * num > den) num = den - num;                             // cos(2 pi - t) = cos t
  if (4 * num > den) return -cx_cos_turn(den - 2 * num, 2 * den);  // cos(t) = -cos(pi - t)
  const double two_pi = 6.28318530717958647692528676655900577;
  if (8 * num <= den) return cx_cos_series(two_pi * (double)num / (double)den);
  return cx_sin_series(two_pi * (double)(den - 4 * num) / (double)(4 * den));  // sin(pi/2 - t)
}
S2C_HD constexpr double cx_sin_turn(long long num, long long den) {
  return cx_cos_turn(4 * num - den, 4 * den);                      // sin t = cos(t - pi/2)
}

template <int K, int NN>
struct Twiddle {
  static constexpr int k = ((K % NN) + NN) % NN;
  static constexpr float re = (float)cx_cos_turn(k, NN);
  static constexpr float im = (float)cx_sin_turn(k, NN);
};

// v * exp(DIR * 2 pi i K / NN) with the trivial cases folded away at compile time
template <int DIR, int K, int NN>
S2C_D float2 tw_mul(float2 v) {
  constexpr int k = ((K % NN) + NN) % NN;
  if constexpr (k == 0) return v;
  else if constexpr (2 * k == NN) return make_float2(-v.x, -v.y);
  else if constexpr (4 * k == NN) return cmul_i<DIR>(v);
  else if constexpr (4 * k == 3 * NN) return cmul_i<-DIR>(v);
  else {
    constexpr float wr = Twiddle<k, NN>::re, wi = DIR * Twiddle<k, NN>::im;
    return make_float2(fmaf(v.x, wr, -v.y * wi), fmaf(v.x, wi, v.y * wr));
  }
}

// ---- small DFTs in registers -------------------------------------------------------------------
template <int DIR, int R>
S2C_D void reg_butterfly(float2 (&t)[R]) {
  if constexpr (R == 2) {
    const float2 a = t[0], b = t[1];
    t[0] = cadd(a, b);
    t[1] = csub(a, b);
  } else if constexpr (R == 3) {
    constexpr float h = 0.86602540378443864676f;  // sin(2 pi / 3)
    const float2 s = cadd(t[1], t[2]), d = csub(t[1], t[2]);
    const float2 a = make_float2(fmaf(-0.5f, s.x, t[0].x), fmaf(-0.5f, s.y, t[0].y));
    const float2 b = cmul_i<DIR>(make_float2(h * d.x, h * d.y));
    t[0] = cadd(t[0], s);
    t[1] = cadd(a, b);
    t[2] = csub(a, b);
  } else if constexpr (R == 4) {
    const float2 t0 = cadd(t[0], t[2]), t1 = csub(t[0], t[2]);
    const float2 t2 = cadd(t[1], t[3]), t3 = cmul_i<DIR>(csub(t[1], t[3]));
    t[0] = cadd(t0, t2);
    t[2] = csub(t0, t2);
    t[1] = cadd(t1, t3);
    t[3] = csub(t1, t3);
  } else if constexpr (R == 5) {
    constexpr float c1 = 0.30901699437494742410f, c2 = -0.80901699437494742410f;  // cos 2pi/5, 4pi/5
    constexpr float s1 = 0.95105651629515357212f, s2 = 0.58778525229247312917f;   // sin 2pi/5, 4pi/5
    const float2 t1 = cadd(t[1], t[4]), t2 = cadd(t[2], t[3]);
    const float2 t3 = csub(t[1], t[4]), t4 = csub(t[2], t[3]);
    const float2 a1 = make_float2(fmaf(c1, t1.x, fmaf(c2, t2.x, t[0].x)),
                                  fmaf(c1, t1.y, fmaf(c2, t2.y, t[0].y)));
    const float2 a2 = make_float2(fmaf(c2, t1.x, fmaf(c1, t2.x, t[0].x)),
                                  fmaf(c2, t1.y, fmaf(c1, t2.y, t[0].y)));
    const float2 b1 = cmul_i<DIR>(make_float2(fmaf(s1, t3.x, s2 * t4.x), fmaf(s1, t3.y, s2 * t4.y)));
    const float2 b2 = cmul_i<DIR>(make_float2(fmaf(s2, t3.x, -s1 * t4.x), fmaf(s2, t3.y, -s1 * t4.y)));
    t[0] = make_float2(t[0].x + t1.x + t2.x, t[0].y + t1.y + t2.y);
    t[1] = cadd(a1, b1);
    t[4] = csub(a1, b1);
    t[2] = cadd(a2, b2);
    t[3] = csub(a2, b2);
  } else {
    // any other prime: direct DFT with immediate twiddles
    float2 u[R];
    static_for<0, R>([&](auto pc) {
      constexpr int p = decltype(pc)::value;
      float2 acc = t[0];
      static_for<1, R>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        const float2 w = tw_mul<DIR, (p * k) % R, R>(t[k]);
        acc.x += w.x;
        acc.y += w.y;
      });
      u[p] = acc;
    });
    static_for<0, R>([&](auto pc) { t[decltype(pc)::value] = u[decltype(pc)::value]; });
  }
}

template <int N, int LEN, int DIR>
S2C_D void fft_reg_stages(float2 (&v)[N]) {
  constexpr int R = fft_pick_radix(LEN);
  constexpr int M = LEN / R;
  static_for<0, N / LEN>([&](auto bc) {
    constexpr int blk = decltype(bc)::value;
    static_for<0, M>([&](auto jc) {
      constexpr int j = decltype(jc)::value;
      float2 t[R];
      static_for<0, R>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        t[k] = v[blk * LEN + j + k * M];
      });
      reg_butterfly<DIR, R>(t);
      static_for<0, R>([&](auto pc) {
        constexpr int p = decltype(pc)::value;
        v[blk * LEN + j + p * M] = tw_mul<DIR, j * p, LEN>(t[p]);
      });
    });
  });
  if constexpr (M > 1) fft_reg_stages<N, M, DIR>(v);
}

// v: natural order in, digit-reversed out (frequency k at v[fft_reg_pos<N>(k)]).  `tw` is unused
// (twiddles are compile-time constants) and kept for signature compatibility.
template <int N, int DIR>
S2C_D void fft_reg(float2 (&v)[N], const float2* tw) {
  (void)tw;
  if constexpr (N > 1) fft_reg_stages<N, N, DIR>(v);
}

}  // namespace s2c
