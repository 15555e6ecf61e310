// Register-resident FFT of compile-time length N (N <= 32): one thread transforms one whole
// row or column held in registers - no shared-memory exchange and no barrier inside a 1-D
// transform.  Same algorithm and radix order as fft_device.h (in-place decimation in frequency,
// radices 4, 2, then odd primes ascending; output digit-reversed), with every loop unrolled at
// compile time so that the array stays in registers and twiddle indices become constants.
#pragma once

#include "fft_device.h"

namespace s2c {

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

template <int N, int LEN, int DIR>
S2C_D void fft_reg_stages(float2 (&v)[N], const float2* tw) {
  constexpr int R = fft_pick_radix(LEN);
  constexpr int M = LEN / R;
  constexpr int TWSTEP = N / LEN;
#pragma unroll
  for (int blk = 0; blk < N / LEN; ++blk) {
#pragma unroll
    for (int j = 0; j < M; ++j) {
      float2 t[R];
#pragma unroll
      for (int k = 0; k < R; ++k) t[k] = v[blk * LEN + j + k * M];
      fft_butterfly<DIR, R>(t, tw, N);
      v[blk * LEN + j] = t[0];
#pragma unroll
      for (int p = 1; p < R; ++p)
        v[blk * LEN + j + p * M] = (j > 0) ? ctw<DIR>(t[p], tw[j * p * TWSTEP]) : t[p];
    }
  }
  if constexpr (M > 1) fft_reg_stages<N, M, DIR>(v, tw);
}

// v: natural order in, digit-reversed out (frequency k at v[fft_reg_pos<N>(k)]); tw[k] =
// exp(+2 pi i k / N) (shared memory or any readable pointer).
template <int N, int DIR>
S2C_D void fft_reg(float2 (&v)[N], const float2* tw) {
  if constexpr (N > 1) fft_reg_stages<N, N, DIR>(v, tw);
}

}  // namespace s2c
