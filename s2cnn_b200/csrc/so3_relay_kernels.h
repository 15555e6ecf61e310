// Two layers' worth of transforms in one kernel, for small bandwidths (N = 2b <= 32):
//
//   S2Convolution tail      z = so3_rifft(s2_mm(xs, ys)) + bias        (s2cnn/soft/s2_conv.py:42-45)
//     or SO3Convolution tail  z = so3_rifft(x) + bias                  (s2cnn/soft/so3_conv.py:55-56)
//   activation              relu(z)
//   SO3Convolution head     so3_rfft(relu(z), b_out = b_next)          (s2cnn/soft/so3_conv.py:50)
//
// The signal z (the largest tensor of such a network) never exists in memory: a block owns ZG
// batch elements and walks the beta axis in groups as the single-direction kernels do
// (so3_fused_kernels.h); the thread that finishes two rows of the synthesis (alpha, alpha + N/2 as
// the real and imaginary part of one inverse transform) adds the bias, applies the ReLU and runs
// the forward transform of the same two rows in its registers; the analysis then continues in the
// same shared-memory planes and accumulates the Wigner contraction of the next layer's bandwidth.
#pragma once

#include "backend.h"
#include "fft_reg.h"
#include "so3_fused_kernels.h"
#include "tables.h"

namespace s2c {

struct RelayParams {
  // synthesis side: either a plain SO(3) spectrum x (rows of x_zstride complex) ...
  const float2* x;
  long x_zstride;
  // ... or, when xs is set, spectrum = s2_mm(xs, ys) computed on the fly
  const float2* xs;    // [Kin^2, s2_nb, s2_fin]
  const float2* ys;    // [Kin^2, s2_fin, s2_fout]
  int s2_nb, s2_fin, s2_fout;
  const float* bias;   // optional [nfeat]
  int nfeat;
  PanelsDev pin;       // beta grid of b, nl = Kin (unweighted)
  const float* win_g;  // pin's values regrouped for groups of BG betas
  int win_stride;
  // analysis side
  PanelsDev pout;      // beta grid of b, nl = b_next, K = Kout (weighted)
  const float* wout_g; // pout's values regrouped for groups of BG betas
  int wout_stride;
  float2* out;         // spectrum rows of out_zstride complex
  long out_zstride;
  const float2* tw;
  int nbatch, Kin, Kout, BG, KP, PS;
};

inline size_t relay_smem_bytes(int N, int Kin, int nrows_in, int nrows_out, int BG) {
  const int K = N / 2;
  (void)Kin;
  return (size_t)N * sizeof(float2) + (size_t)nrows_in * kFusedZG * sizeof(float2) +
         (size_t)so3_npairs(K) * sizeof(int4) + ((size_t)nrows_in * BG + 4) * sizeof(float) + 16 +
         (size_t)nrows_out * kFusedZG * sizeof(float2) +
         (size_t)kFusedZG * BG * (N * fused_kp(N) + 16) * sizeof(float2);
}

template <int N>
struct so3_relay_fused_impl {
  static S2C_D void run(const Ctx& ctx, const RelayParams& p, unsigned char* smem) {
    constexpr int ZG = kFusedZG;
    const int Kin = p.Kin, Kout = p.Kout, KP = p.KP;
    const int nrows_in = p.pin.nrows, nrows_out = p.pout.nrows;
    float2* tw = reinterpret_cast<float2*>(smem);
    // half spectrum, split in two arrays of 16-byte rows: [nrows_in][z 0,1] then [nrows_in][z 2,3]
    // (rows of consecutive frequency pairs then start 16 L instead of 32 L bytes apart, which
    // halves the bank conflicts of the per-pair 16-byte loads)
    float2* Xh = tw + N;
    auto xh_at = [&](int r, int z) -> float2& { return Xh[((z >> 1) * nrows_in + r) * 2 + (z & 1)]; };
    int4* pinfo = reinterpret_cast<int4*>(Xh + (size_t)nrows_in * ZG);      // [npairs_in]
    float* Wg = reinterpret_cast<float*>(pinfo + p.pin.npairs);             // [nrows_in][BG]
    unsigned long long* wbar = reinterpret_cast<unsigned long long*>(Wg + p.win_stride);
    // accumulated spectrum of the analysis, split like Xh: [nrows_out][z 0, 1] then [nrows_out][z 2, 3]
    float2* acc = reinterpret_cast<float2*>(wbar + 2);
    auto acc_at = [&](int r, int z) -> float2& { return acc[((z >> 1) * nrows_out + r) * 2 + (z & 1)]; };
    float4* acc4 = reinterpret_cast<float4*>(acc);
    float2* planes = acc + (size_t)nrows_out * ZG;                          // [ZG * BG][N][KP]
    const unsigned wbytes = (unsigned)p.win_stride * sizeof(float);
    if (ctx.tid == 0) {
      bulk_barrier_init(wbar);
      bulk_load_issue(Wg, p.win_g, wbytes, wbar);   // Wigner slice of the first beta group
    }
    const int plane_sz = p.PS;
    const long z0 = (long)ctx.bid * ZG;
    const int zc = (int)((p.nbatch - z0) < ZG ? (p.nbatch - z0) : ZG);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    for (int it = ctx.tid; it < nrows_out * ZG; it += ctx.nthr) acc[it] = make_float2(0.f, 0.f);
    for (int pr = ctx.tid; pr < p.pin.npairs; pr += ctx.nthr) {
      int m, n;
      so3_pair_decode(pr, Kin, m, n);
      const int am = m < 0 ? -m : m;
      const int lmin = am > n ? am : n;
      pinfo[pr] = make_int4((int)(p.pin.off[pr] / N), Kin - lmin, m < 0 ? m + N : m, n);
    }
    // symmetrised half spectrum of the product, Xs = (X[l,m,n] + (-1)^(m-n) conj X[l,-m,-n]) / 2,
    // X[l,m,n](i,j) = sum_k xs[l,m,i,k] conj(ys[l,n,k,j]).  The block's batch elements are
    // (i, j .. j+3) when f_out is a multiple of 4: one work item per panel row then serves all four
    // (xs loaded once, ys with 16-byte loads); otherwise one item per (row, batch element).
    if (!p.xs) {
      // plain spectrum: the block's batch elements are 32 contiguous bytes of every row
      const bool vec = zc == ZG && ZG == 4 && p.x_zstride % 2 == 0;
      for (int r = ctx.tid; r < nrows_in; r += ctx.nthr) {
        int l, m, n;
        rowmap_unpack(p.pin.rowmap[r], l, m, n);
        const float2* pa = p.x + so3_row(l, m, n) * p.x_zstride + z0;
        const float2* pb = p.x + so3_row(l, -m, -n) * p.x_zstride + z0;
        float2 av[ZG], bv[ZG];
        if (vec) {
          const float4 a01 = reinterpret_cast<const float4*>(pa)[0], a23 = reinterpret_cast<const float4*>(pa)[1];
          const float4 b01 = reinterpret_cast<const float4*>(pb)[0], b23 = reinterpret_cast<const float4*>(pb)[1];
          av[0] = make_float2(a01.x, a01.y); av[1] = make_float2(a01.z, a01.w);
          av[2] = make_float2(a23.x, a23.y); av[3] = make_float2(a23.z, a23.w);
          bv[0] = make_float2(b01.x, b01.y); bv[1] = make_float2(b01.z, b01.w);
          bv[2] = make_float2(b23.x, b23.y); bv[3] = make_float2(b23.z, b23.w);
        } else {
#pragma unroll
          for (int z = 0; z < ZG; ++z) {
            av[z] = z < zc ? pa[z] : make_float2(0.f, 0.f);
            bv[z] = z < zc ? pb[z] : make_float2(0.f, 0.f);
          }
        }
        const float fudge = ((m - n) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int z = 0; z < ZG; ++z)
          xh_at(r, z) = make_float2(0.5f * (av[z].x + fudge * bv[z].x), 0.5f * (av[z].y - fudge * bv[z].y));
      }
    } else if (zc == ZG && ZG == 4 && p.s2_fout % ZG == 0) {
      const int pi = (int)(z0 / p.s2_fout), pj = (int)(z0 - (long)pi * p.s2_fout);
      for (int r = ctx.tid; r < nrows_in; r += ctx.nthr) {
        int l, m, n;
        rowmap_unpack(p.pin.rowmap[r], l, m, n);
        const float2* xa = p.xs + ((long)(l * l + l + m) * p.s2_nb + pi) * p.s2_fin;
        const float2* xb = p.xs + ((long)(l * l + l - m) * p.s2_nb + pi) * p.s2_fin;
        const float2* ya = p.ys + (long)(l * l + l + n) * p.s2_fin * p.s2_fout + pj;
        const float2* yb = p.ys + (long)(l * l + l - n) * p.s2_fin * p.s2_fout + pj;
        float2 av[ZG], bv[ZG];
#pragma unroll
        for (int z = 0; z < ZG; ++z) { av[z] = make_float2(0.f, 0.f); bv[z] = make_float2(0.f, 0.f); }
        for (int k = 0; k < p.s2_fin; ++k) {
          const float2 xk = xa[k], xm = xb[k];
          const float4 y01 = *reinterpret_cast<const float4*>(ya + (long)k * p.s2_fout);
          const float4 y23 = *reinterpret_cast<const float4*>(ya + (long)k * p.s2_fout + 2);
          const float4 w01 = *reinterpret_cast<const float4*>(yb + (long)k * p.s2_fout);
          const float4 w23 = *reinterpret_cast<const float4*>(yb + (long)k * p.s2_fout + 2);
          const float2 yv[ZG] = {make_float2(y01.x, y01.y), make_float2(y01.z, y01.w),
                                 make_float2(y23.x, y23.y), make_float2(y23.z, y23.w)};
          const float2 wv[ZG] = {make_float2(w01.x, w01.y), make_float2(w01.z, w01.w),
                                 make_float2(w23.x, w23.y), make_float2(w23.z, w23.w)};
#pragma unroll
          for (int z = 0; z < ZG; ++z) {   // x * conj(y)
            av[z].x = fmaf(xk.x, yv[z].x, av[z].x);
            av[z].x = fmaf(xk.y, yv[z].y, av[z].x);
            av[z].y = fmaf(xk.y, yv[z].x, av[z].y);
            av[z].y = fmaf(-xk.x, yv[z].y, av[z].y);
            bv[z].x = fmaf(xm.x, wv[z].x, bv[z].x);
            bv[z].x = fmaf(xm.y, wv[z].y, bv[z].x);
            bv[z].y = fmaf(xm.y, wv[z].x, bv[z].y);
            bv[z].y = fmaf(-xm.x, wv[z].y, bv[z].y);
          }
        }
        const float fudge = ((m - n) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int z = 0; z < ZG; ++z)
          xh_at(r, z) = make_float2(0.5f * (av[z].x + fudge * bv[z].x), 0.5f * (av[z].y - fudge * bv[z].y));
      }
    } else {
    for (int it = ctx.tid; it < nrows_in * ZG; it += ctx.nthr) {
      const int r = it / ZG, zz = it - r * ZG;
      int l, m, n;
      rowmap_unpack(p.pin.rowmap[r], l, m, n);
      float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
      if (zz < zc) {
        const int z = (int)(z0 + zz);
        const int i = z / p.s2_fout, j = z - i * p.s2_fout;
        const float2* xa = p.xs + ((long)(l * l + l + m) * p.s2_nb + i) * p.s2_fin;
        const float2* xb = p.xs + ((long)(l * l + l - m) * p.s2_nb + i) * p.s2_fin;
        const float2* ya = p.ys + (long)(l * l + l + n) * p.s2_fin * p.s2_fout + j;
        const float2* yb = p.ys + (long)(l * l + l - n) * p.s2_fin * p.s2_fout + j;
        for (int k = 0; k < p.s2_fin; ++k) {
          const float2 xk = xa[k], xm = xb[k];
          const float2 yk = ya[(long)k * p.s2_fout], ym = yb[(long)k * p.s2_fout];
          a.x = fmaf(xk.x, yk.x, a.x); a.x = fmaf(xk.y, yk.y, a.x);
          a.y = fmaf(xk.y, yk.x, a.y); a.y = fmaf(-xk.x, yk.y, a.y);
          b.x = fmaf(xm.x, ym.x, b.x); b.x = fmaf(xm.y, ym.y, b.x);
          b.y = fmaf(xm.y, ym.x, b.y); b.y = fmaf(-xm.x, ym.y, b.y);
        }
      }
      const float fudge = ((m - n) & 1) ? -1.f : 1.f;
      xh_at(r, zz) = make_float2(0.5f * (a.x + fudge * b.x), 0.5f * (a.y - fudge * b.y));
    }
    }
    ctx.sync();

    for (int bg0 = 0; bg0 < N; bg0 += p.BG) {
      const int bc = p.BG;   // BG divides N
      // ---- synthesis: Wigner contraction over l, one (pair, beta) per work item ----------------
      const int grp = bg0 / p.BG;
      const bool landed = bulk_wait(ctx, wbar, (unsigned)(grp & 1));
      const float* wslice = landed ? Wg : p.win_g + (size_t)grp * p.win_stride;
      if (p.BG == 4 && ZG == 4) {
        // groups of four betas: one frequency pair per work item with all 4 x 4 (beta, batch
        // element) accumulators in registers - three 16-byte loads feed 32 multiply-adds
        for (int pr = ctx.tid; pr < p.pin.npairs; pr += ctx.nthr) {
          const int4 info = pinfo[pr];  // {first panel row, L, FFT row of m, n}
          const float4* w4 = reinterpret_cast<const float4*>(wslice + info.x * 4);
          const float4* xa4 = reinterpret_cast<const float4*>(Xh) + info.x;
          const float4* xb4 = xa4 + nrows_in;
          float2 s[4][ZG];
#pragma unroll
          for (int bi = 0; bi < 4; ++bi)
#pragma unroll
            for (int z = 0; z < ZG; ++z) s[bi][z] = make_float2(0.f, 0.f);
          for (int li = 0; li < info.y; ++li) {
            const float4 w = w4[li], xa = xa4[li], xb = xb4[li];
            const float wv[4] = {w.x, w.y, w.z, w.w};
            const float2 xv[ZG] = {make_float2(xa.x, xa.y), make_float2(xa.z, xa.w),
                                   make_float2(xb.x, xb.y), make_float2(xb.z, xb.w)};
#pragma unroll
            for (int bi = 0; bi < 4; ++bi)
#pragma unroll
              for (int z = 0; z < ZG; ++z) {
                s[bi][z].x = fmaf(wv[bi], xv[z].x, s[bi][z].x);
                s[bi][z].y = fmaf(wv[bi], xv[z].y, s[bi][z].y);
              }
          }
          float2* pl = planes + info.z * KP + info.w;
          const bool mirror = (info.w == 0 && info.z > 0);  // n = 0, m > 0: row N - m holds the conjugate
#pragma unroll
          for (int bi = 0; bi < 4; ++bi)
#pragma unroll
            for (int z = 0; z < ZG; ++z) {
              float2* dst = pl + (size_t)(z * 4 + bi) * plane_sz;
              dst[0] = s[bi][z];
              if (mirror) dst[(N - 2 * info.z) * KP] = make_float2(s[bi][z].x, -s[bi][z].y);
            }
        }
      } else
      for (int it = ctx.tid; it < p.pin.npairs * bc; it += ctx.nthr) {
        const int pr = it / bc, bi = it - pr * bc;
        const int4 info = pinfo[pr];  // {first panel row, L, FFT row of m, n}
        const float* w = wslice + info.x * p.BG + bi;
        const int xrow = info.x;
        float2 s[ZG];
#pragma unroll
        for (int z = 0; z < ZG; ++z) s[z] = make_float2(0.f, 0.f);
        for (int li = 0; li < info.y; ++li) {
          const float wv = w[li * p.BG];
#pragma unroll
          for (int z = 0; z < ZG; ++z) {
            const float2 xv = xh_at(xrow + li, z);
            s[z].x = fmaf(wv, xv.x, s[z].x);
            s[z].y = fmaf(wv, xv.y, s[z].y);
          }
        }
        float2* pl = planes + (size_t)bi * plane_sz + info.z * KP + info.w;
        const bool mirror = (info.w == 0 && info.z > 0);  // n = 0, m > 0: row N - m holds the conjugate
#pragma unroll
        for (int z = 0; z < ZG; ++z) {
          pl[(size_t)z * p.BG * plane_sz] = s[z];
          if (mirror)
            pl[(size_t)z * p.BG * plane_sz + (N - 2 * info.z) * KP] = make_float2(s[z].x, -s[z].y);
        }
      }
      ctx.sync();
      if (ctx.tid == 0 && bg0 + p.BG < N)   // every thread is done with this slice: fetch the next
        bulk_load_issue(Wg, p.win_g + (size_t)(grp + 1) * p.win_stride, wbytes, wbar);
      // ---- synthesis: column FFTs m -> alpha, one thread per (z, beta, n) ----------------------
      for (int it = ctx.tid; it < ZG * bc * Kin; it += ctx.nthr) {
        const int n = it % Kin, zb = it / Kin;
        const int bi = zb % bc, z = zb / bc;
        float2* col = planes + (size_t)(z * p.BG + bi) * plane_sz + n;
        float2 v[N];
#pragma unroll
        for (int i = 0; i < N; ++i)
          v[i] = (i < Kin || i > N - Kin) ? col[i * KP] : make_float2(0.f, 0.f);
        fft_reg<N, +1>(v, tw);
        static_for<0, N>([&](auto ic) {
          constexpr int a = decltype(ic)::value;
          col[a * KP] = v[fft_reg_pos<N>(a)];
        });
      }
      ctx.sync();
      // ---- rows: Hermitian inverse transform n -> gamma of rows (alpha, alpha + N/2), + bias,
      //      ReLU, forward transform gamma -> n of the same two rows; one thread per
      //      (z, beta, alpha pair), one pass of the block -----------------------------------------
      {
        const int it = ctx.tid;
        const bool act = it < ZG * bc * (N / 2);
        const int ap = it % (N / 2), zb = it / (N / 2);
        const int bi = zb % bc, z = zb / bc;
        float2* r1 = planes + (size_t)(z * p.BG + bi) * plane_sz + ap * KP;
        float2* r2 = r1 + (N / 2) * KP;
        float2 v[N];
        if (act) {
          {
            const float2 t1 = r1[0], t2 = r2[0];
            v[0] = make_float2(t1.x, t2.x);  // T[alpha][0] is real for a Hermitian spectrum
          }
          if constexpr (N > 1) v[N / 2] = make_float2(0.f, 0.f);
#pragma unroll
          for (int n = 1; n < N / 2; ++n) {
            if (n < Kin) {
              const float2 t1 = r1[n], t2 = r2[n];
              v[n] = make_float2(t1.x - t2.y, t1.y + t2.x);      // T1 + i T2
              v[N - n] = make_float2(t1.x + t2.y, t2.x - t1.y);  // conj(T1) + i conj(T2)
            } else {
              v[n] = make_float2(0.f, 0.f);
              v[N - n] = make_float2(0.f, 0.f);
            }
          }
        }
        ctx.sync();   // every synthesis row is in registers: the planes can take the analysis
        if (act) {
          fft_reg<N, +1>(v, tw);
          float add = 0.f;
          if (p.bias) add = p.bias[(z0 + z) % p.nfeat];
          float2 u[N];
          static_for<0, N>([&](auto gc) {
            constexpr int g = decltype(gc)::value;
            constexpr int pg = fft_reg_pos<N>(g);
            const float a1 = v[pg].x + add, a2 = v[pg].y + add;   // samples gamma = g of both rows
            u[g] = make_float2(a1 > 0.f ? a1 : 0.f, a2 > 0.f ? a2 : 0.f);
          });
          if (z >= zc) {
#pragma unroll
            for (int g = 0; g < N; ++g) u[g] = make_float2(0.f, 0.f);
          }
          fft_reg<N, -1>(u, tw);
          static_for<0, N / 2>([&](auto ic) {
            constexpr int n = decltype(ic)::value;
            constexpr int pn = fft_reg_pos<N>(n), pq = fft_reg_pos<N>(n == 0 ? 0 : N - n);
            if (n < Kout) {
              const float2 zk = u[pn];
              const float2 zq = u[pq];
              r1[n] = make_float2(0.5f * (zk.x + zq.x), 0.5f * (zk.y - zq.y));
              r2[n] = make_float2(0.5f * (zk.y + zq.y), -0.5f * (zk.x - zq.x));
            }
          });
        }
      }
      ctx.sync();
      // ---- analysis: column FFTs alpha -> m, one thread per (z, beta, n) -----------------------
      for (int it = ctx.tid; it < ZG * bc * Kout; it += ctx.nthr) {
        const int n = it % Kout, zb = it / Kout;
        const int bi = zb % bc, z = zb / bc;
        float2* col = planes + (size_t)(z * p.BG + bi) * plane_sz + n;
        float2 v[N];
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = col[i * KP];
        fft_reg<N, -1>(v, tw);
        static_for<0, N>([&](auto ic) {
          constexpr int f = decltype(ic)::value;
          if (f < Kout || f > N - Kout) col[f * KP] = v[fft_reg_pos<N>(f)];
        });
      }
      ctx.sync();
      // ---- analysis: accumulate the Wigner contraction over the betas of this group ------------
      for (int r = ctx.tid; r < nrows_out; r += ctx.nthr) {
        int l, m, n;
        rowmap_unpack(p.pout.rowmap[r], l, m, n);
        // the group's table values of neighbouring rows are neighbouring pieces of the regrouped copy
        const float* w = p.wout_g + (size_t)grp * p.wout_stride + (size_t)r * p.BG;
        const float2* src = planes + (m < 0 ? m + N : m) * KP + n;
        const float4 a01 = acc4[r], a23 = acc4[nrows_out + r];
        float2 a[ZG] = {make_float2(a01.x, a01.y), make_float2(a01.z, a01.w),
                        make_float2(a23.x, a23.y), make_float2(a23.z, a23.w)};
        for (int bi = 0; bi < bc; ++bi) {
          const float wv = w[bi];
#pragma unroll
          for (int z = 0; z < ZG; ++z) {
            const float2 xv = src[(size_t)(z * p.BG + bi) * plane_sz];
            a[z].x = fmaf(wv, xv.x, a[z].x);
            a[z].y = fmaf(wv, xv.y, a[z].y);
          }
        }
        acc4[r] = make_float4(a[0].x, a[0].y, a[1].x, a[1].y);
        acc4[nrows_out + r] = make_float4(a[2].x, a[2].y, a[3].x, a[3].y);
      }
      ctx.sync();
    }
    // ---- write the next layer's spectrum and its Hermitian mirror -----------------------------
    for (int it = ctx.tid; it < nrows_out * ZG; it += ctx.nthr) {
      const int r = it / ZG, z = it - r * ZG;
      if (z >= zc) continue;
      int l, m, n;
      rowmap_unpack(p.pout.rowmap[r], l, m, n);
      const float2 a = acc_at(r, z);
      const float fudge = ((m - n) & 1) ? -1.f : 1.f;
      p.out[so3_row(l, m, n) * p.out_zstride + z0 + z] = a;
      if (!(m == 0 && n == 0))
        p.out[so3_row(l, -m, -n) * p.out_zstride + z0 + z] = make_float2(fudge * a.x, -fudge * a.y);
    }
  }
};

#ifndef S2C_EMUL
template <int N>
__global__ void __launch_bounds__(256, 3) so3_relay_fused(const RelayParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_relay_fused_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
#endif

}  // namespace s2c
