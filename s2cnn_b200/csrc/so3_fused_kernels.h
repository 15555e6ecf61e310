// Fused SO(3) transforms for small bandwidths (N = 2b <= 32): one kernel per direction, no
// scratch in global memory.  A block owns ZG consecutive batch elements (so that its accesses to
// the [spectrum][batch] layout are whole 32-byte sectors) and walks the beta axis in groups; all
// intermediates of a group live in shared memory, every 1-D FFT runs in the registers of one
// thread (fft_reg.h).
//
//   synthesis (so3_inv_fused):  symmetrised half spectrum -> shared memory once; per beta group:
//     Wigner contraction over l -> column FFTs (m -> alpha) -> Hermitian row FFTs (n -> gamma,
//     two real rows per complex transform) -> (+ bias) -> coalesced store of whole planes.
//   analysis (so3_fwd_fused):  per beta group: load planes (optional ReLU on load) -> row FFTs
//     (two real rows per transform) -> column FFTs -> accumulate the Wigner contraction over beta
//     into a shared-memory spectrum; written once at the end together with the Hermitian mirror.
//
// They replace the same reference code as the general path in so3_kernels.h
// (s2cnn/soft/so3_fft.py:64-112,158-202,246-443) and produce the same values.
#pragma once

#include <type_traits>

#include "backend.h"
#include "fft_reg.h"
#include "so3_kernels.h"
#include "tables.h"

namespace s2c {

constexpr int kFusedZG = 4;

template <int I, int E, class F>
S2C_D void static_for(F&& f) {
  if constexpr (I < E) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, E>(f);
  }
}

S2C_D void rowmap_unpack(int packed, int& l, int& m, int& n) {
  l = packed & 0xff;
  m = ((packed >> 8) & 0xff) - 128;
  n = (packed >> 16) & 0xff;
}

// ---------------------------------------------------------------------------------------------
struct InvFusedParams {
  const float2* x;     // spectrum rows of x_zstride complex
  long x_zstride;
  float* out;          // element e of the real signal at out[e * out_stride + out_off]
  long out_stride, out_off;
  const float* bias;
  int nfeat;
  PanelsDev pan;       // beta grid of b_out, nl = K
  const float2* tw;    // N twiddles
  int nbatch, K, BG, KP, nrows, mode;
  // mode == kS2Product: the spectrum is never materialised; row (l,m,n), batch z = (i, j) is
  //   sum_k xs[l,m,i,k] conj(ys[l,n,k,j])        (s2_mm fused into the synthesis prologue)
  const float2* xs;    // [K*K, s2_nb, s2_fin]
  const float2* ys;    // [K*K, s2_fin, s2_fout]
  int s2_nb, s2_fin, s2_fout;
};

S2C_D float2 s2_product_entry(const InvFusedParams& p, int l, int m, int n, int i, int j) {
  const float2* xr = p.xs + ((long)(l * l + l + m) * p.s2_nb + i) * p.s2_fin;
  const float2* yr = p.ys + (long)(l * l + l + n) * p.s2_fin * p.s2_fout + j;
  float re = 0.f, im = 0.f;
  for (int k = 0; k < p.s2_fin; ++k) {
    const float2 a = xr[k], b = yr[(long)k * p.s2_fout];
    re = fmaf(a.x, b.x, re);
    re = fmaf(a.y, b.y, re);
    im = fmaf(a.y, b.x, im);
    im = fmaf(-a.x, b.y, im);
  }
  return make_float2(re, im);
}

template <int N>
struct so3_inv_fused_impl {
  static S2C_D void run(const Ctx& ctx, const InvFusedParams& p, unsigned char* smem) {
    constexpr int ZG = kFusedZG;
    const int K = p.K, KP = p.KP;
    float2* tw = reinterpret_cast<float2*>(smem);
    float2* Xh = tw + N;                              // [nrows][ZG]
    float2* planes = Xh + (size_t)p.nrows * ZG;       // [ZG * BG][N][KP]
    const int plane_sz = N * KP;
    const long z0 = (long)ctx.bid * ZG;
    const int zc = (int)((p.nbatch - z0) < ZG ? (p.nbatch - z0) : ZG);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    // symmetrised half spectrum  Xs = (X[l,m,n] + (-1)^(m-n) conj X[l,-m,-n]) / 2
    for (int it = ctx.tid; it < p.nrows * ZG; it += ctx.nthr) {
      const int r = it / ZG, zz = it - r * ZG;
      float2 v = make_float2(0.f, 0.f);
      if (zz < zc) {
        int l, m, n;
        rowmap_unpack(p.pan.rowmap[r], l, m, n);
        float2 a, b;
        if (p.mode == kS2Product) {
          const int z = (int)(z0 + zz);
          const int i = z / p.s2_fout, j = z - i * p.s2_fout;
          a = s2_product_entry(p, l, m, n, i, j);
          b = s2_product_entry(p, l, -m, -n, i, j);
        } else {
          a = p.x[so3_row(l, m, n) * p.x_zstride + z0 + zz];
          b = p.x[so3_row(l, -m, -n) * p.x_zstride + z0 + zz];
        }
        if (p.mode == kSo3RotI) {
          a = make_float2(a.y, -a.x);
          b = make_float2(b.y, -b.x);
        }
        const float fudge = ((m - n) & 1) ? -1.f : 1.f;
        v = make_float2(0.5f * (a.x + fudge * b.x), 0.5f * (a.y - fudge * b.y));
      }
      Xh[it] = v;
    }
    ctx.sync();

    for (int bg0 = 0; bg0 < N; bg0 += p.BG) {
      const int bc = (N - bg0) < p.BG ? (N - bg0) : p.BG;
      // ---- Wigner contraction over l: one (pair, beta) per work item, ZG accumulators -------
      for (int it = ctx.tid; it < p.pan.npairs * bc; it += ctx.nthr) {
        const int pr = it / bc, bi = it - pr * bc;
        int m, n;
        so3_pair_decode(pr, K, m, n);
        const int am = m < 0 ? -m : m;
        const int lmin = am > n ? am : n;
        const int L = K - lmin;
        const long off = p.pan.off[pr];
        const float* w = p.pan.data + off + bg0 + bi;
        const float2* xs = Xh + (off / N) * ZG;
        float2 acc[ZG];
#pragma unroll
        for (int z = 0; z < ZG; ++z) acc[z] = make_float2(0.f, 0.f);
        for (int li = 0; li < L; ++li) {
          const float wv = w[li * N];
#pragma unroll
          for (int z = 0; z < ZG; ++z) {
            const float2 xv = xs[li * ZG + z];
            acc[z].x = fmaf(wv, xv.x, acc[z].x);
            acc[z].y = fmaf(wv, xv.y, acc[z].y);
          }
        }
        const int row = m < 0 ? m + N : m;
#pragma unroll
        for (int z = 0; z < ZG; ++z) {
          float2* pl = planes + (size_t)(z * p.BG + bi) * plane_sz;
          pl[row * KP + n] = acc[z];
          if (n == 0 && m > 0) pl[(N - m) * KP] = make_float2(acc[z].x, -acc[z].y);
        }
      }
      ctx.sync();
      // ---- column FFTs m -> alpha: one thread per (z, beta, n) ------------------------------
      for (int it = ctx.tid; it < ZG * bc * K; it += ctx.nthr) {
        const int n = it % K, zb = it / K;
        const int bi = zb % bc, z = zb / bc;
        float2* col = planes + (size_t)(z * p.BG + bi) * plane_sz + n;
        float2 v[N];
#pragma unroll
        for (int i = 0; i < N; ++i)
          v[i] = (i < K || i > N - K) ? col[i * KP] : make_float2(0.f, 0.f);
        fft_reg<N, +1>(v, tw);
        static_for<0, N>([&](auto ic) {
          constexpr int a = decltype(ic)::value;
          constexpr int pa = fft_reg_pos<N>(a);
          col[a * KP] = v[pa];
        });
      }
      ctx.sync();
      // ---- Hermitian row FFTs n -> gamma: one thread per (z, beta, alpha pair) ---------------
      for (int it = ctx.tid; it < ZG * bc * (N / 2); it += ctx.nthr) {
        const int ap = it % (N / 2), zb = it / (N / 2);
        const int bi = zb % bc, z = zb / bc;
        float2* r1 = planes + (size_t)(z * p.BG + bi) * plane_sz + (2 * ap) * KP;
        float2* r2 = r1 + KP;
        float2 v[N];
        {
          const float2 t1 = r1[0], t2 = r2[0];
          v[0] = make_float2(t1.x, t2.x);  // T[alpha][0] is real for a Hermitian spectrum
        }
        if constexpr (N > 1) v[N / 2] = make_float2(0.f, 0.f);
#pragma unroll
        for (int n = 1; n < N / 2; ++n) {
          if (n < K) {
            const float2 t1 = r1[n], t2 = r2[n];
            v[n] = make_float2(t1.x - t2.y, t1.y + t2.x);      // T1 + i T2
            v[N - n] = make_float2(t1.x + t2.y, t2.x - t1.y);  // conj(T1) + i conj(T2)
          } else {
            v[n] = make_float2(0.f, 0.f);
            v[N - n] = make_float2(0.f, 0.f);
          }
        }
        fft_reg<N, +1>(v, tw);
        float add = 0.f;
        if (p.bias) add = p.bias[(z0 + z) % p.nfeat];
        float* o1 = reinterpret_cast<float*>(r1);
        float* o2 = reinterpret_cast<float*>(r2);
        static_for<0, N>([&](auto ic) {
          constexpr int g = decltype(ic)::value;
          constexpr int pg = fft_reg_pos<N>(g);
          const float2 t = v[pg];
          o1[g] = t.x + add;
          o2[g] = t.y + add;
        });
      }
      ctx.sync();
      // ---- store whole planes ----------------------------------------------------------------
      if (p.out_stride == 1) {
        for (int it = ctx.tid; it < zc * bc * N * (N / 2); it += ctx.nthr) {
          const int g2 = it % (N / 2);
          int t = it / (N / 2);
          const int a = t % N;
          t /= N;
          const int bi = t % bc, z = t / bc;
          const float* src = reinterpret_cast<const float*>(
              planes + (size_t)(z * p.BG + bi) * plane_sz + a * KP);
          const float2 val = make_float2(src[2 * g2], src[2 * g2 + 1]);
          float* dst = p.out + (((z0 + z) * N + bg0 + bi) * N + a) * (long)N + 2 * g2;
          *reinterpret_cast<float2*>(dst) = val;
        }
      } else {
        for (int it = ctx.tid; it < zc * bc * N * N; it += ctx.nthr) {
          const int g = it % N;
          int t = it / N;
          const int a = t % N;
          t /= N;
          const int bi = t % bc, z = t / bc;
          const float* src = reinterpret_cast<const float*>(
              planes + (size_t)(z * p.BG + bi) * plane_sz + a * KP);
          const long e = (((z0 + z) * N + bg0 + bi) * N + a) * (long)N + g;
          p.out[e * p.out_stride + p.out_off] = src[g];
        }
      }
      ctx.sync();
    }
  }
};

// ---------------------------------------------------------------------------------------------
struct FwdFusedParams {
  const float* x;      // element e of the real signal at x[e * in_stride + in_off]
  long in_stride, in_off;
  float2* out;         // spectrum rows of out_zstride complex
  long out_zstride;
  PanelsDev pan;       // beta grid of b_in, nl = b_out, K
  const float2* tw;
  int nbatch, K, BG, KP, nrows, mode, relu;
};

template <int N>
struct so3_fwd_fused_impl {
  static S2C_D void run(const Ctx& ctx, const FwdFusedParams& p, unsigned char* smem) {
    constexpr int ZG = kFusedZG;
    const int K = p.K, KP = p.KP;
    float2* tw = reinterpret_cast<float2*>(smem);
    float2* acc = tw + N;                               // [nrows][ZG]
    float2* planes = acc + (size_t)p.nrows * ZG;        // [ZG * BG][N][KP]
    const int plane_sz = N * KP;
    const long z0 = (long)ctx.bid * ZG;
    const int zc = (int)((p.nbatch - z0) < ZG ? (p.nbatch - z0) : ZG);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    for (int it = ctx.tid; it < p.nrows * ZG; it += ctx.nthr) acc[it] = make_float2(0.f, 0.f);
    ctx.sync();

    for (int bg0 = 0; bg0 < N; bg0 += p.BG) {
      const int bc = (N - bg0) < p.BG ? (N - bg0) : p.BG;
      // ---- load planes (rows of N floats at a stride of 2 KP floats) -------------------------
      if (p.in_stride == 1) {
        for (int it = ctx.tid; it < ZG * bc * N * (N / 2); it += ctx.nthr) {
          const int g2 = it % (N / 2);
          int t = it / (N / 2);
          const int a = t % N;
          t /= N;
          const int bi = t % bc, z = t / bc;
          float2 val = make_float2(0.f, 0.f);
          if (z < zc) {
            const float* src = p.x + (((z0 + z) * N + bg0 + bi) * N + a) * (long)N + 2 * g2;
            val = *reinterpret_cast<const float2*>(src);
            if (p.relu) {
              val.x = val.x > 0.f ? val.x : 0.f;
              val.y = val.y > 0.f ? val.y : 0.f;
            }
          }
          float* dst = reinterpret_cast<float*>(planes + (size_t)(z * p.BG + bi) * plane_sz + a * KP);
          dst[2 * g2] = val.x;
          dst[2 * g2 + 1] = val.y;
        }
      } else {
        for (int it = ctx.tid; it < ZG * bc * N * N; it += ctx.nthr) {
          const int g = it % N;
          int t = it / N;
          const int a = t % N;
          t /= N;
          const int bi = t % bc, z = t / bc;
          float val = 0.f;
          if (z < zc) {
            const long e = (((z0 + z) * N + bg0 + bi) * N + a) * (long)N + g;
            val = p.x[e * p.in_stride + p.in_off];
            if (p.relu) val = val > 0.f ? val : 0.f;
          }
          reinterpret_cast<float*>(planes + (size_t)(z * p.BG + bi) * plane_sz + a * KP)[g] = val;
        }
      }
      ctx.sync();
      // ---- row FFTs gamma -> n, two real rows per complex transform --------------------------
      for (int it = ctx.tid; it < ZG * bc * (N / 2); it += ctx.nthr) {
        const int ap = it % (N / 2), zb = it / (N / 2);
        const int bi = zb % bc, z = zb / bc;
        float2* r1 = planes + (size_t)(z * p.BG + bi) * plane_sz + (2 * ap) * KP;
        float2* r2 = r1 + KP;
        const float* f1 = reinterpret_cast<const float*>(r1);
        const float* f2 = reinterpret_cast<const float*>(r2);
        float2 v[N];
#pragma unroll
        for (int g = 0; g < N; ++g) v[g] = make_float2(f1[g], f2[g]);
        fft_reg<N, -1>(v, tw);
        static_for<0, N / 2>([&](auto ic) {
          constexpr int n = decltype(ic)::value;
          constexpr int pn = fft_reg_pos<N>(n), pq = fft_reg_pos<N>(n == 0 ? 0 : N - n);
          if (n < K) {
            const float2 zk = v[pn];
            const float2 zq = v[pq];
            r1[n] = make_float2(0.5f * (zk.x + zq.x), 0.5f * (zk.y - zq.y));
            r2[n] = make_float2(0.5f * (zk.y + zq.y), -0.5f * (zk.x - zq.x));
          }
        });
      }
      ctx.sync();
      // ---- column FFTs alpha -> m: one thread per (z, beta, n) --------------------------------
      for (int it = ctx.tid; it < ZG * bc * K; it += ctx.nthr) {
        const int n = it % K, zb = it / K;
        const int bi = zb % bc, z = zb / bc;
        float2* col = planes + (size_t)(z * p.BG + bi) * plane_sz + n;
        float2 v[N];
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = col[i * KP];
        fft_reg<N, -1>(v, tw);
        static_for<0, N>([&](auto ic) {
          constexpr int f = decltype(ic)::value;
          constexpr int pf = fft_reg_pos<N>(f);
          if (f < K || f > N - K) col[f * KP] = v[pf];
        });
      }
      ctx.sync();
      // ---- accumulate the Wigner contraction over the betas of this group ---------------------
      for (int it = ctx.tid; it < p.nrows * ZG; it += ctx.nthr) {
        const int r = it / ZG, z = it - r * ZG;
        int l, m, n;
        rowmap_unpack(p.pan.rowmap[r], l, m, n);
        const float* w = p.pan.data + (long)r * N + bg0;
        const float2* src = planes + (size_t)(z * p.BG) * plane_sz + (m < 0 ? m + N : m) * KP + n;
        float ar = 0.f, ai = 0.f;
        for (int bi = 0; bi < bc; ++bi) {
          const float wv = w[bi];
          const float2 xv = src[(size_t)bi * plane_sz];
          ar = fmaf(wv, xv.x, ar);
          ai = fmaf(wv, xv.y, ai);
        }
        float2 c = acc[it];
        acc[it] = make_float2(c.x + ar, c.y + ai);
      }
      ctx.sync();
    }
    // ---- write the spectrum and its Hermitian mirror ----------------------------------------
    for (int it = ctx.tid; it < p.nrows * ZG; it += ctx.nthr) {
      const int r = it / ZG, z = it - r * ZG;
      if (z >= zc) continue;
      int l, m, n;
      rowmap_unpack(p.pan.rowmap[r], l, m, n);
      const float2 a = acc[it];
      const float fudge = ((m - n) & 1) ? -1.f : 1.f;
      float2* o1 = p.out + so3_row(l, m, n) * p.out_zstride + z0 + z;
      float2* o2 = p.out + so3_row(l, -m, -n) * p.out_zstride + z0 + z;
      const bool self = (m == 0 && n == 0);
      if (p.mode == kSo3Real) {
        *o1 = a;
        if (!self) *o2 = make_float2(fudge * a.x, -fudge * a.y);
      } else {  // += i * a ; mirror += i * fudge * conj(a)
        float2 c = *o1;
        *o1 = make_float2(c.x - a.y, c.y + a.x);
        if (!self) {
          c = *o2;
          *o2 = make_float2(c.x + fudge * a.y, c.y + fudge * a.x);
        }
      }
    }
  }
};

#ifndef S2C_EMUL
template <int N>
__global__ void __launch_bounds__(256) so3_inv_fused(const InvFusedParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_inv_fused_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
template <int N>
__global__ void __launch_bounds__(256) so3_fwd_fused(const FwdFusedParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_fwd_fused_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
#define S2C_LAUNCH_N(name, N, grid, block, smem, stream, params) \
  s2c::launch_impl(name<N>, #name, (long)(grid), (int)(block), (size_t)(smem), stream, params)
#else
#define S2C_LAUNCH_N(name, N, grid, block, smem, stream, params) \
  s2c::emu_launch<name##_impl<N>>(#name, (long)(grid), (int)(block), (size_t)(smem), params)
#endif

// run-time N -> compile-time N
#define S2C_DISPATCH_N(N, CALL)                                                              \
  switch (N) {                                                                               \
    case 2: { constexpr int kN = 2; CALL; } break;                                           \
    case 4: { constexpr int kN = 4; CALL; } break;                                           \
    case 6: { constexpr int kN = 6; CALL; } break;                                           \
    case 8: { constexpr int kN = 8; CALL; } break;                                           \
    case 10: { constexpr int kN = 10; CALL; } break;                                         \
    case 12: { constexpr int kN = 12; CALL; } break;                                         \
    case 14: { constexpr int kN = 14; CALL; } break;                                         \
    case 16: { constexpr int kN = 16; CALL; } break;                                         \
    case 18: { constexpr int kN = 18; CALL; } break;                                         \
    case 20: { constexpr int kN = 20; CALL; } break;                                         \
    case 22: { constexpr int kN = 22; CALL; } break;                                         \
    case 24: { constexpr int kN = 24; CALL; } break;                                         \
    case 26: { constexpr int kN = 26; CALL; } break;                                         \
    case 28: { constexpr int kN = 28; CALL; } break;                                         \
    case 30: { constexpr int kN = 30; CALL; } break;                                         \
    case 32: { constexpr int kN = 32; CALL; } break;                                         \
    default: rc = s2c::fail(s2c::S2C_ERR_UNSUPPORTED, "no fused kernel for this length");    \
  }

constexpr int kFusedMaxN = 32;

inline int fused_kp(int N) { return N / 2 + 1; }
inline int fused_bg(int N) {
  const int per_beta = kFusedZG * N * fused_kp(N) * (int)sizeof(float2);
  int bg = (32 * 1024) / per_beta;
  if (bg < 1) bg = 1;
  if (bg > N) bg = N;
  return bg;
}
inline size_t fused_smem_bytes(int N, int nrows) {
  return (size_t)N * sizeof(float2) + (size_t)nrows * kFusedZG * sizeof(float2) +
         (size_t)kFusedZG * fused_bg(N) * N * fused_kp(N) * sizeof(float2);
}

}  // namespace s2c
