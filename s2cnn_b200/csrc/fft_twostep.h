// Two-step ("four-step" without the final transpose) FFT for the row transforms of the general
// path: N = R1 * R2 with both factors small enough for a register FFT (fft_reg.h).
//
//   step 1  thread (t, j), j < R2:  v[k] = x[t][j + R2 k]  ->  R1-point FFT in registers,
//           y_p[j] = V[p] * W_N^(j p)  written to a second buffer as  tmp[t][p (R2+1) + j]
//   step 2  thread (t, p), p < R1:  u[j] = tmp[t][p (R2+1) + j]  ->  R2-point FFT in registers,
//           X[p + R1 q] = U[q]  written back to x[t] in NATURAL frequency order.
//
// Compared with the generic radix-by-radix shared-memory FFT (fft_device.h) an element crosses
// shared memory twice instead of once per radix stage, all butterflies run on registers with
// compile-time twiddles, and there are two block barriers per batch instead of one per stage.
// Supported lengths: 64 = 8 x 8, 128 = 8 x 16, 256 = 16 x 16 (SOFT grids of bandwidth 32, 64, 128).
#pragma once

#include "backend.h"
#include "fft_reg.h"

namespace s2c {

S2C_HD bool fft_twostep_supported(int n) { return n == 64 || n == 128 || n == 256; }
S2C_HD int fft_twostep_ld2(int n) {  // row stride of the second buffer, in complex numbers
  const int r1 = (n == 256) ? 16 : 8;
  return n + r1 + 1;
}

template <int R1, int R2, int DIR>
S2C_D void fft_twostep_impl(const Ctx& ctx, float2* data, float2* tmp, int count, int ld, int ld2,
                            const float2* tw) {
  constexpr int N = R1 * R2;
  // step 1: R1-point transforms over the stride-R2 subsequences, twiddle, transpose into tmp
  for (int it = ctx.tid; it < count * R2; it += ctx.nthr) {
    const int t = it / R2, j = it - t * R2;
    const float2* src = data + (size_t)t * ld + j;
    float2 v[R1];
#pragma unroll
    for (int k = 0; k < R1; ++k) v[k] = src[R2 * k];
    fft_reg<R1, DIR>(v, tw);
    float2* dst = tmp + (size_t)t * ld2 + j;
    static_for<0, R1>([&](auto pc) {
      constexpr int p = decltype(pc)::value;
      constexpr int pp = fft_reg_pos<R1>(p);
      if constexpr (p == 0) {
        dst[0] = v[pp];
      } else {
        const float2 w = tw[j * p];  // exp(+2 pi i j p / N), j p < N
        dst[p * (R2 + 1)] = ctw<DIR>(v[pp], w);
      }
    });
  }
  ctx.sync();
  // step 2: R2-point transforms, natural-order output
  for (int it = ctx.tid; it < count * R1; it += ctx.nthr) {
    const int t = it / R1, p = it - t * R1;
    const float2* src = tmp + (size_t)t * ld2 + p * (R2 + 1);
    float2 u[R2];
#pragma unroll
    for (int j = 0; j < R2; ++j) u[j] = src[j];
    fft_reg<R2, DIR>(u, tw);
    float2* dst = data + (size_t)t * ld + p;
    static_for<0, R2>([&](auto qc) {
      constexpr int q = decltype(qc)::value;
      constexpr int qq = fft_reg_pos<R2>(q);
      dst[R1 * q] = u[qq];
    });
  }
  ctx.sync();
  (void)N;
}

// Batch of `count` transforms of length n (must satisfy fft_twostep_supported), rows at stride ld
// in `data`, scratch rows at stride fft_twostep_ld2(n) in `tmp`.  Natural order in and out.
template <int DIR>
S2C_D void fft_twostep(const Ctx& ctx, float2* data, float2* tmp, int n, int count, int ld,
                       const float2* tw) {
  const int ld2 = fft_twostep_ld2(n);
  if (n == 64) fft_twostep_impl<8, 8, DIR>(ctx, data, tmp, count, ld, ld2, tw);
  else if (n == 128) fft_twostep_impl<8, 16, DIR>(ctx, data, tmp, count, ld, ld2, tw);
  else fft_twostep_impl<16, 16, DIR>(ctx, data, tmp, count, ld, ld2, tw);
}

}  // namespace s2c
