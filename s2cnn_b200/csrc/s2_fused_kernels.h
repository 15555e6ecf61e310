// S2 analysis of a real signal in one kernel, for grids whose half plane fits in shared memory
// (the first layer of the reference's models: b = 30 ... 64).  One block per signal: the 2b rows
// are transformed over alpha two at a time (rows beta and beta + b packed into one complex FFT),
// the packed spectra stay in shared memory, and one thread per output coefficient (l, m) runs the
// Wigner-d contraction over beta, separating the packed rows while it reads them.
//
// Same values as so3_fwd_alpha (real input) followed by so3_fwd_wigner in S2 mode, i.e. the
// reference's s2_fft for a real signal (s2cnn/soft/s2_fft.py:13-50, kernel s2fft.cu :151-186).
#pragma once

#include "backend.h"
#include "so3_kernels.h"
#include "tables.h"

namespace s2c {

struct S2FwdFusedParams {
  const float* x;      // [nbatch][N][N] real
  float2* out;         // rows l*l + l + m of out_zstride complex
  long out_zstride;
  PanelsDev pan;       // S2 panels: pair = m + K - 1, rows l - |m|, columns beta
  FftDev fft;
  int N, K;            // K = b_out = number of degrees
};

inline size_t s2_fwd_fused_smem(int N) { return fft_smem_bytes(N, N / 2); }

S2C_KERNEL(s2_fwd_fused, S2FwdFusedParams) {
  const int N = p.N, ld = N + 1, H = N / 2;
  FftSmem s = fft_smem_carve(smem, N, H);
  fft_smem_load_tables(ctx, s, p.fft);
  const long z = ctx.bid;
  const float* src = p.x + z * (long)N * N;
  for (int e = ctx.tid; e < H * N; e += ctx.nthr) {
    const int t = e / N, a = e - t * N;
    s.data[t * ld + a] = make_float2(src[e], src[e + H * N]);   // rows t and t + H
  }
  ctx.sync();
  fft_rows<-1>(ctx, s, p.fft.desc, H, ld);
  for (int o = ctx.tid; o < p.K * p.K; o += ctx.nthr) {
    int l = (int)sqrtf((float)o);
    while (l * l > o) --l;
    while ((l + 1) * (l + 1) <= o) ++l;
    const int m = o - l * l - l;
    const int am = m < 0 ? -m : m;
    const float* w = p.pan.data + p.pan.off[m + p.K - 1] + (long)(l - am) * N;
    const int pk = s.pos[m < 0 ? m + N : m];
    const int pc = s.pos[m == 0 ? 0 : (m < 0 ? -m : N - m)];
    float ar = 0.f, ai = 0.f;
    for (int t = 0; t < H; ++t) {
      const float2 zk = s.data[t * ld + pk], zc = s.data[t * ld + pc];
      const float w1 = w[t], w2 = w[t + H];
      // row t:     (zk + conj zc) / 2        row t + H:  (zk - conj zc) / (2 i)
      ar = fmaf(w1, 0.5f * (zk.x + zc.x), ar);
      ai = fmaf(w1, 0.5f * (zk.y - zc.y), ai);
      ar = fmaf(w2, 0.5f * (zk.y + zc.y), ar);
      ai = fmaf(w2, -0.5f * (zk.x - zc.x), ai);
    }
    p.out[(long)o * p.out_zstride + z] = make_float2(ar, ai);
  }
}

}  // namespace s2c
