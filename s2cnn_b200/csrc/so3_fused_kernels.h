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

#include <map>
#include <mutex>
#include <string>
#include <type_traits>

#include "backend.h"
#include "fft_reg.h"
#include "so3_kernels.h"
#include "tables.h"

namespace s2c {


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
  int nbatch, K, BG, KP, PS, nrows, mode;
  // mode == kS2Product: the spectrum is never materialised; row (l,m,n), batch z = (i, j) is
  //   sum_k xs[l,m,i,k] conj(ys[l,n,k,j])        (s2_mm fused into the synthesis prologue)
  const float2* xs;    // [K*K, s2_nb, s2_fin]
  const float2* ys;    // [K*K, s2_fin, s2_fout]
  int s2_nb, s2_fin, s2_fout;
  // optional tail of a network: instead of writing the signal, integrate max(signal, 0) over SO(3)
  // (so3_integrate(relu(.)), s2cnn/soft/so3_integrate.py:7-29) and write one number per batch element
  const float* iw;     // quadrature weights [N] (null: write the signal)
  float* isum;         // [nbatch]
  // optional: a signal of the output's shape (unit stride); output samples where it is <= 0 are
  // written as 0 - the gradient of a ReLU that was applied while this signal was read
  const float* mask;
  int wide;            // out (and mask) are 32-byte aligned and N % 4 == 0: 32-byte stores
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
    // half spectrum, split in two arrays of 16-byte rows: [nrows][z 0, 1] then [nrows][z 2, 3] (the
    // rows of consecutive frequency pairs then start 16 L instead of 32 L bytes apart, which halves
    // the bank conflicts of the per-pair 16-byte loads)
    float2* Xh = tw + N;
    static_assert(kFusedZG == 4, "split spectrum layout");
    auto xh_at = [&](int r, int z) -> float2& { return Xh[((z >> 1) * p.nrows + r) * 2 + (z & 1)]; };
    int4* pinfo = reinterpret_cast<int4*>(Xh + (size_t)p.nrows * ZG);    // [npairs]
    float* Wg = reinterpret_cast<float*>(pinfo + p.pan.npairs);           // [nrows][BG] of one group
    unsigned long long* wbar = reinterpret_cast<unsigned long long*>(Wg + p.pan.g_stride);
    float2* planes = reinterpret_cast<float2*>(wbar + 2);                 // [ZG * BG][N][KP]
    const unsigned wbytes = (unsigned)p.pan.g_stride * sizeof(float);
    if (ctx.tid == 0) {
      bulk_barrier_init(wbar);
      bulk_load_issue(Wg, p.pan.data_g, wbytes, wbar);   // Wigner slice of the first beta group
    }
    const int plane_sz = p.PS;
    const long z0 = (long)ctx.bid * ZG;
    const int zc = (int)((p.nbatch - z0) < ZG ? (p.nbatch - z0) : ZG);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    for (int pr = ctx.tid; pr < p.pan.npairs; pr += ctx.nthr) {
      int m, n;
      so3_pair_decode(pr, K, m, n);
      const int am = m < 0 ? -m : m;
      const int lmin = am > n ? am : n;
      pinfo[pr] = make_int4((int)(p.pan.off[pr] / N), K - lmin, m < 0 ? m + N : m, n);
    }
    // symmetrised half spectrum  Xs = (X[l,m,n] + (-1)^(m-n) conj X[l,-m,-n]) / 2
    //
    // Fast path: one panel row per work item for all ZG batch elements at once.  The block's batch
    // elements are consecutive, so their spectrum entries are 32 contiguous bytes (two 16-byte
    // loads); with s2_mm fused they share the batch index i of xs and take consecutive output
    // features j of ys.  Index arithmetic and the xs loads are then paid once per row, not once
    // per (row, batch element).
    const bool prod = p.mode == kS2Product;
    bool fast = zc == ZG && ZG == 4;
    if (prod) fast = fast && (p.s2_fout % ZG == 0);
    else fast = fast && (p.x_zstride % 2 == 0);
    if (fast) {
      const int pi = prod ? (int)(z0 / p.s2_fout) : 0, pj = prod ? (int)(z0 - (long)pi * p.s2_fout) : 0;
      // With the product fused, the loads of the two S2 spectra are the cost of this loop.  The
      // first one is the same small slice (its batch index is fixed) for every row: it is staged in
      // the shared memory that the planes use later.  For the second one the threads walk the rows
      // sorted by (l, n, m), so that the lanes of a warp mostly read the same address.
      float2* xs_s = planes;
      const int nlm = K * K;
      const bool stage_xs = prod && (size_t)nlm * p.s2_fin <= (size_t)ZG * p.BG * plane_sz;
      if (stage_xs) {
        for (int e = ctx.tid; e < nlm * p.s2_fin; e += ctx.nthr) {
          const int lm = e / p.s2_fin, k = e - lm * p.s2_fin;
          xs_s[e] = p.xs[((long)lm * p.s2_nb + pi) * p.s2_fin + k];
        }
        ctx.sync();
      }
      const int* order = prod ? p.pan.order : nullptr;
      const bool wide_x = !prod && p.x_zstride % 4 == 0 && reinterpret_cast<unsigned long long>(p.x) % 32 == 0;
      for (int ri = ctx.tid; ri < p.nrows; ri += ctx.nthr) {
        const int r = order ? order[ri] : ri;
        int l, m, n;
        rowmap_unpack(p.pan.rowmap[r], l, m, n);
        float2 av[ZG], bv[ZG];
        if (prod) {
          const float2* xa = stage_xs ? xs_s + (l * l + l + m) * p.s2_fin
                                      : p.xs + ((long)(l * l + l + m) * p.s2_nb + pi) * p.s2_fin;
          const float2* xb = stage_xs ? xs_s + (l * l + l - m) * p.s2_fin
                                      : p.xs + ((long)(l * l + l - m) * p.s2_nb + pi) * p.s2_fin;
          const float2* ya = p.ys + (long)(l * l + l + n) * p.s2_fin * p.s2_fout + pj;
          const float2* yb = p.ys + (long)(l * l + l - n) * p.s2_fin * p.s2_fout + pj;
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
        } else {
          const float2* qa = p.x + so3_row(l, m, n) * p.x_zstride + z0;
          const float2* qb = p.x + so3_row(l, -m, -n) * p.x_zstride + z0;
          float4 a01, a23, b01, b23;
          if (wide_x) {   // the four batch elements of a row are one aligned 32-byte sector
            const float8 a = ld_global_256(reinterpret_cast<const float*>(qa));
            const float8 b = ld_global_256(reinterpret_cast<const float*>(qb));
            a01 = a.lo; a23 = a.hi; b01 = b.lo; b23 = b.hi;
          } else {
            const float4* pa = reinterpret_cast<const float4*>(qa);
            const float4* pb = reinterpret_cast<const float4*>(qb);
            a01 = pa[0]; a23 = pa[1]; b01 = pb[0]; b23 = pb[1];
          }
          av[0] = make_float2(a01.x, a01.y); av[1] = make_float2(a01.z, a01.w);
          av[2] = make_float2(a23.x, a23.y); av[3] = make_float2(a23.z, a23.w);
          bv[0] = make_float2(b01.x, b01.y); bv[1] = make_float2(b01.z, b01.w);
          bv[2] = make_float2(b23.x, b23.y); bv[3] = make_float2(b23.z, b23.w);
        }
        const float fudge = ((m - n) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int z = 0; z < ZG; ++z) {
          float2 a = av[z], b = bv[z];
          if (p.mode == kSo3RotI) {
            a = make_float2(a.y, -a.x);
            b = make_float2(b.y, -b.x);
          }
          xh_at(r, z) = make_float2(0.5f * (a.x + fudge * b.x), 0.5f * (a.y - fudge * b.y));
        }
      }
    } else {
    // general path: one (row, batch element) per work item, four at a time so that eight
    // independent row loads are in flight
    for (int base = ctx.tid; base < p.nrows * ZG; base += 4 * ctx.nthr) {
      int packed[4];
      float2 a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int it = base + u * ctx.nthr;
        packed[u] = it < p.nrows * ZG ? p.pan.rowmap[it / ZG] : 0;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int it = base + u * ctx.nthr;
        const int zz = it % ZG;
        a[u] = make_float2(0.f, 0.f);
        b[u] = make_float2(0.f, 0.f);
        if (it < p.nrows * ZG && zz < zc) {
          int l, m, n;
          rowmap_unpack(packed[u], l, m, n);
          if (p.mode == kS2Product) {
            const int z = (int)(z0 + zz);
            const int i = z / p.s2_fout, j = z - i * p.s2_fout;
            a[u] = s2_product_entry(p, l, m, n, i, j);
            b[u] = s2_product_entry(p, l, -m, -n, i, j);
          } else {
            a[u] = p.x[so3_row(l, m, n) * p.x_zstride + z0 + zz];
            b[u] = p.x[so3_row(l, -m, -n) * p.x_zstride + z0 + zz];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int it = base + u * ctx.nthr;
        if (it >= p.nrows * ZG) continue;
        int l, m, n;
        rowmap_unpack(packed[u], l, m, n);
        float2 av = a[u], bv = b[u];
        if (p.mode == kSo3RotI) {
          av = make_float2(av.y, -av.x);
          bv = make_float2(bv.y, -bv.x);
        }
        const float fudge = ((m - n) & 1) ? -1.f : 1.f;
        xh_at(it / ZG, it % ZG) = make_float2(0.5f * (av.x + fudge * bv.x), 0.5f * (av.y - fudge * bv.y));
      }
    }
    }
    ctx.sync();

    float ipart = 0.f;   // this thread's share of the integral (its rows of every beta group)
    for (int bg0 = 0; bg0 < N; bg0 += p.BG) {
      const int bc = (N - bg0) < p.BG ? (N - bg0) : p.BG;
      // ---- Wigner contraction over l: one (pair, beta) per work item, ZG accumulators.  The
      //      group's slice of the table was brought into shared memory by an asynchronous bulk
      //      copy issued one group earlier; if it did not land in time, read global memory. ----
      const int grp = bg0 / p.BG;
      const bool landed = bulk_wait(ctx, wbar, (unsigned)(grp & 1));
      const float* wslice = landed ? Wg : p.pan.data_g + (size_t)grp * p.pan.g_stride;
      if (p.BG == 4 && ZG == 4) {
        // groups of four betas: one frequency pair per work item with all 4 x 4 (beta, batch
        // element) accumulators in registers - three 16-byte loads feed 32 multiply-adds
        for (int pr = ctx.tid; pr < p.pan.npairs; pr += ctx.nthr) {
          const int4 info = pinfo[pr];  // {first panel row, L, FFT row of m, n}
          const float4* w4 = reinterpret_cast<const float4*>(wslice + info.x * 4);
          const float4* xa4 = reinterpret_cast<const float4*>(Xh) + info.x;
          const float4* xb4 = xa4 + p.nrows;
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
      for (int it = ctx.tid; it < p.pan.npairs * bc; it += ctx.nthr) {
        const int pr = it / bc, bi = it - pr * bc;
        const int4 info = pinfo[pr];  // {first panel row, L, FFT row of m, n}
        const float* w = wslice + info.x * p.BG + bi;
        const int xrow = info.x;
        float2 acc[ZG];
#pragma unroll
        for (int z = 0; z < ZG; ++z) acc[z] = make_float2(0.f, 0.f);
        for (int li = 0; li < info.y; ++li) {
          const float wv = w[li * p.BG];
#pragma unroll
          for (int z = 0; z < ZG; ++z) {
            const float2 xv = xh_at(xrow + li, z);
            acc[z].x = fmaf(wv, xv.x, acc[z].x);
            acc[z].y = fmaf(wv, xv.y, acc[z].y);
          }
        }
        float2* pl = planes + (size_t)bi * plane_sz + info.z * KP + info.w;
        const bool mirror = (info.w == 0 && info.z > 0);  // n = 0, m > 0: row N - m holds the conjugate
#pragma unroll
        for (int z = 0; z < ZG; ++z) {
          pl[(size_t)z * p.BG * plane_sz] = acc[z];
          if (mirror)
            pl[(size_t)z * p.BG * plane_sz + (N - 2 * info.z) * KP] = make_float2(acc[z].x, -acc[z].y);
        }
      }
      ctx.sync();
      if (ctx.tid == 0 && bg0 + p.BG < N)   // every thread is done with this slice: fetch the next
        bulk_load_issue(Wg, p.pan.data_g + (size_t)(grp + 1) * p.pan.g_stride, wbytes, wbar);
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
        // rows alpha = ap and ap + N/2 share one complex transform (row stride KP is odd, so
        // consecutive threads hit distinct banks)
        float2* r1 = planes + (size_t)(z * p.BG + bi) * plane_sz + ap * KP;
        float2* r2 = r1 + (N / 2) * KP;
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
        if (p.iw) {
          // the signal is not written: max(x, 0) of both rows, summed over gamma, times w_beta
          float rs = 0.f;
#pragma unroll
          for (int g = 0; g < N; ++g) {
            const float a1 = v[g].x + add, a2 = v[g].y + add;
            rs += (a1 > 0.f ? a1 : 0.f) + (a2 > 0.f ? a2 : 0.f);
          }
          ipart = fmaf(p.iw[bg0 + bi], rs, ipart);
        } else
        // store the two finished rows straight from registers (the plane is contiguous in memory)
        if (z < zc) {
          const long row1 = (((z0 + z) * N + bg0 + bi) * (long)N + ap) * N;   // first float of row ap
          const long row2 = row1 + (long)(N / 2) * N;
          if (N % 4 == 0 && p.wide) {
            // 32-byte stores, one whole sector per lane and instruction (with 16-byte stores every
            // sector would reach L2 in two halves).  Rows of N % 8 == 4 floats start on a sector
            // boundary only every other row (the planes themselves do, 4 N^2 bytes apart): even
            // rows end, odd rows begin with a 16-byte piece.
            auto keep = [](float4 val, float4 k) {
              return make_float4(k.x > 0.f ? val.x : 0.f, k.y > 0.f ? val.y : 0.f,
                                 k.z > 0.f ? val.z : 0.f, k.w > 0.f ? val.w : 0.f);
            };
            auto quad = [&](auto gc, float4& o1, float4& o2) {
              constexpr int g = decltype(gc)::value;
              constexpr int p0 = fft_reg_pos<N>(g), p1 = fft_reg_pos<N>(g + 1);
              constexpr int p2 = fft_reg_pos<N>(g + 2), p3 = fft_reg_pos<N>(g + 3);
              o1 = make_float4(v[p0].x + add, v[p1].x + add, v[p2].x + add, v[p3].x + add);
              o2 = make_float4(v[p0].y + add, v[p1].y + add, v[p2].y + add, v[p3].y + add);
            };
            auto st4 = [&](auto gc) {
              constexpr int g = decltype(gc)::value;
              float4 o1, o2;
              quad(gc, o1, o2);
              if (p.mask) {
                o1 = keep(o1, *reinterpret_cast<const float4*>(p.mask + row1 + g));
                o2 = keep(o2, *reinterpret_cast<const float4*>(p.mask + row2 + g));
              }
              *reinterpret_cast<float4*>(p.out + row1 + g) = o1;
              *reinterpret_cast<float4*>(p.out + row2 + g) = o2;
            };
            auto st8 = [&](auto gc) {
              constexpr int g = decltype(gc)::value;
              float8 o1, o2;
              quad(gc, o1.lo, o2.lo);
              quad(std::integral_constant<int, g + 4>{}, o1.hi, o2.hi);
              if (p.mask) {
                const float8 k1 = ld_global_256(p.mask + row1 + g), k2 = ld_global_256(p.mask + row2 + g);
                o1.lo = keep(o1.lo, k1.lo); o1.hi = keep(o1.hi, k1.hi);
                o2.lo = keep(o2.lo, k2.lo); o2.hi = keep(o2.hi, k2.hi);
              }
              st_global_256(p.out + row1 + g, o1);
              st_global_256(p.out + row2 + g, o2);
            };
            if constexpr (N % 8 == 0) {
              static_for<0, N / 8>([&](auto ic) { st8(std::integral_constant<int, 8 * decltype(ic)::value>{}); });
            } else if (ap & 1) {
              st4(std::integral_constant<int, 0>{});
              static_for<0, N / 8>([&](auto ic) { st8(std::integral_constant<int, 4 + 8 * decltype(ic)::value>{}); });
            } else {
              static_for<0, N / 8>([&](auto ic) { st8(std::integral_constant<int, 8 * decltype(ic)::value>{}); });
              st4(std::integral_constant<int, N - 4>{});
            }
          } else if (p.out_stride == 1) {
            constexpr int V = (N % 4 == 0) ? 4 : 2;
            static_for<0, N / V>([&](auto ic) {
              constexpr int g = V * decltype(ic)::value;
              constexpr int p0 = fft_reg_pos<N>(g), p1 = fft_reg_pos<N>(g + 1);
              if constexpr (V == 4) {
                constexpr int p2 = fft_reg_pos<N>(g + 2), p3 = fft_reg_pos<N>(g + 3);
                float4 o1 = make_float4(v[p0].x + add, v[p1].x + add, v[p2].x + add, v[p3].x + add);
                float4 o2 = make_float4(v[p0].y + add, v[p1].y + add, v[p2].y + add, v[p3].y + add);
                if (p.mask) {
                  const float4 k1 = *reinterpret_cast<const float4*>(p.mask + row1 + g);
                  const float4 k2 = *reinterpret_cast<const float4*>(p.mask + row2 + g);
                  o1 = make_float4(k1.x > 0.f ? o1.x : 0.f, k1.y > 0.f ? o1.y : 0.f,
                                   k1.z > 0.f ? o1.z : 0.f, k1.w > 0.f ? o1.w : 0.f);
                  o2 = make_float4(k2.x > 0.f ? o2.x : 0.f, k2.y > 0.f ? o2.y : 0.f,
                                   k2.z > 0.f ? o2.z : 0.f, k2.w > 0.f ? o2.w : 0.f);
                }
                *reinterpret_cast<float4*>(p.out + row1 + g) = o1;
                *reinterpret_cast<float4*>(p.out + row2 + g) = o2;
              } else {
                float2 o1 = make_float2(v[p0].x + add, v[p1].x + add);
                float2 o2 = make_float2(v[p0].y + add, v[p1].y + add);
                if (p.mask) {
                  const float2 k1 = *reinterpret_cast<const float2*>(p.mask + row1 + g);
                  const float2 k2 = *reinterpret_cast<const float2*>(p.mask + row2 + g);
                  o1 = make_float2(k1.x > 0.f ? o1.x : 0.f, k1.y > 0.f ? o1.y : 0.f);
                  o2 = make_float2(k2.x > 0.f ? o2.x : 0.f, k2.y > 0.f ? o2.y : 0.f);
                }
                *reinterpret_cast<float2*>(p.out + row1 + g) = o1;
                *reinterpret_cast<float2*>(p.out + row2 + g) = o2;
              }
            });
          } else {
            static_for<0, N>([&](auto ic) {
              constexpr int g = decltype(ic)::value;
              constexpr int pg = fft_reg_pos<N>(g);
              p.out[(row1 + g) * p.out_stride + p.out_off] = v[pg].x + add;
              p.out[(row2 + g) * p.out_stride + p.out_off] = v[pg].y + add;
            });
          }
        }
      }
      ctx.sync();
    }
    if (p.iw) {
      // Every group has the same number of betas here (the host only asks for the integral when BG
      // divides N and one pass of the block covers a group), so thread t always served batch
      // element t / (BG * N/2): sum the threads of each element in a fixed order.
      float* red = reinterpret_cast<float*>(planes);
      red[ctx.tid] = ipart;
      ctx.sync();
      if (ctx.tid < zc) {
        const int per = p.BG * (N / 2);
        float sum = 0.f;
        for (int t = 0; t < per; ++t) sum += red[ctx.tid * per + t];
        p.isum[z0 + ctx.tid] = sum;
      }
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
  int nbatch, K, BG, KP, PS, nrows, mode, relu;
  int wide;            // x is 32-byte aligned, unit stride and N % 4 == 0: 32-byte loads
  // optional by-product [nbatch]: the plain sum of every signal over its (2b)^3 samples (the
  // (m, n) = (0, 0) bin of each beta plane, summed over beta) - what the gradient of a bias that
  // was added to the signal needs, without another pass over the signal
  float* sums;
};

template <int N>
struct so3_fwd_fused_impl {
  static S2C_D void run(const Ctx& ctx, const FwdFusedParams& p, unsigned char* smem) {
    constexpr int ZG = kFusedZG;
    const int K = p.K, KP = p.KP;
    float2* tw = reinterpret_cast<float2*>(smem);
    // accumulated spectrum, split in two arrays of 16-byte rows: [nrows][z 0, 1] then [nrows][z 2, 3]
    // (threads that own neighbouring rows then read and write neighbouring 16-byte pieces; with 32
    // contiguous bytes per row the 8-byte accesses of a warp fell four to a bank)
    float2* acc = tw + N;
    static_assert(kFusedZG == 4, "split accumulator layout");
    auto acc_at = [&](int r, int z) -> float2& { return acc[((z >> 1) * p.nrows + r) * 2 + (z & 1)]; };
    float4* acc4 = reinterpret_cast<float4*>(acc);       // acc4[r] = z 0, 1;  acc4[nrows + r] = z 2, 3
    float2* planes = acc + (size_t)p.nrows * ZG;        // [ZG * BG][N][KP]
    const int plane_sz = p.PS;
    const long z0 = (long)ctx.bid * ZG;
    const int zc = (int)((p.nbatch - z0) < ZG ? (p.nbatch - z0) : ZG);
    for (int i = ctx.tid; i < N; i += ctx.nthr) tw[i] = p.tw[i];
    for (int it = ctx.tid; it < p.nrows * ZG; it += ctx.nthr) acc[it] = make_float2(0.f, 0.f);
    ctx.sync();
    float zsum = 0.f;   // threads 0 .. ZG-1: running sum of their batch element's (0, 0) bins

    for (int bg0 = 0; bg0 < N; bg0 += p.BG) {
      const int bc = (N - bg0) < p.BG ? (N - bg0) : p.BG;
      // ---- row FFTs gamma -> n: each thread reads two real rows (alpha, alpha + N/2) straight
      //      from global memory into registers (optional ReLU), transforms them as one complex
      //      sequence and leaves the n < K half spectra of both rows in shared memory -----------
      for (int it = ctx.tid; it < ZG * bc * (N / 2); it += ctx.nthr) {
        const int ap = it % (N / 2), zb = it / (N / 2);
        const int bi = zb % bc, z = zb / bc;
        float2* r1 = planes + (size_t)(z * p.BG + bi) * plane_sz + ap * KP;
        float2* r2 = r1 + (N / 2) * KP;
        float2 v[N];
        if (z < zc) {
          const long row1 = (((z0 + z) * N + bg0 + bi) * (long)N + ap) * N;
          const long row2 = row1 + (long)(N / 2) * N;
          if (N % 4 == 0 && p.wide) {
            // 32-byte loads, one whole sector per lane and instruction; rows of N % 8 == 4 floats
            // start on a sector boundary only every other row (see the synthesis kernel)
            auto ld4 = [&](auto gc) {
              constexpr int g = decltype(gc)::value;
              const float4 a = *reinterpret_cast<const float4*>(p.x + row1 + g);
              const float4 b = *reinterpret_cast<const float4*>(p.x + row2 + g);
              v[g] = make_float2(a.x, b.x);
              v[g + 1] = make_float2(a.y, b.y);
              v[g + 2] = make_float2(a.z, b.z);
              v[g + 3] = make_float2(a.w, b.w);
            };
            auto ld8 = [&](auto gc) {
              constexpr int g = decltype(gc)::value;
              const float8 a = ld_global_256(p.x + row1 + g), b = ld_global_256(p.x + row2 + g);
              v[g] = make_float2(a.lo.x, b.lo.x);
              v[g + 1] = make_float2(a.lo.y, b.lo.y);
              v[g + 2] = make_float2(a.lo.z, b.lo.z);
              v[g + 3] = make_float2(a.lo.w, b.lo.w);
              v[g + 4] = make_float2(a.hi.x, b.hi.x);
              v[g + 5] = make_float2(a.hi.y, b.hi.y);
              v[g + 6] = make_float2(a.hi.z, b.hi.z);
              v[g + 7] = make_float2(a.hi.w, b.hi.w);
            };
            if constexpr (N % 8 == 0) {
              static_for<0, N / 8>([&](auto ic) { ld8(std::integral_constant<int, 8 * decltype(ic)::value>{}); });
            } else if (ap & 1) {
              ld4(std::integral_constant<int, 0>{});
              static_for<0, N / 8>([&](auto ic) { ld8(std::integral_constant<int, 4 + 8 * decltype(ic)::value>{}); });
            } else {
              static_for<0, N / 8>([&](auto ic) { ld8(std::integral_constant<int, 8 * decltype(ic)::value>{}); });
              ld4(std::integral_constant<int, N - 4>{});
            }
          } else if (p.in_stride == 1) {
            constexpr int V = (N % 4 == 0) ? 4 : 2;
            static_for<0, N / V>([&](auto ic) {
              constexpr int g = V * decltype(ic)::value;
              if constexpr (V == 4) {
                const float4 a = *reinterpret_cast<const float4*>(p.x + row1 + g);
                const float4 b = *reinterpret_cast<const float4*>(p.x + row2 + g);
                v[g] = make_float2(a.x, b.x);
                v[g + 1] = make_float2(a.y, b.y);
                v[g + 2] = make_float2(a.z, b.z);
                v[g + 3] = make_float2(a.w, b.w);
              } else {
                const float2 a = *reinterpret_cast<const float2*>(p.x + row1 + g);
                const float2 b = *reinterpret_cast<const float2*>(p.x + row2 + g);
                v[g] = make_float2(a.x, b.x);
                v[g + 1] = make_float2(a.y, b.y);
              }
            });
          } else {
#pragma unroll
            for (int g = 0; g < N; ++g)
              v[g] = make_float2(p.x[(row1 + g) * p.in_stride + p.in_off],
                                 p.x[(row2 + g) * p.in_stride + p.in_off]);
          }
          if (p.relu) {
#pragma unroll
            for (int g = 0; g < N; ++g) {
              v[g].x = v[g].x > 0.f ? v[g].x : 0.f;
              v[g].y = v[g].y > 0.f ? v[g].y : 0.f;
            }
          }
        } else {
#pragma unroll
          for (int g = 0; g < N; ++g) v[g] = make_float2(0.f, 0.f);
        }
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
      if (p.sums && ctx.tid < ZG)
        for (int bi = 0; bi < bc; ++bi) zsum += planes[(size_t)(ctx.tid * p.BG + bi) * plane_sz].x;
      // ---- accumulate the Wigner contraction over the betas of this group: one panel row
      //      (l, m, n) per thread, all ZG batch elements -----------------------------------------
      if (p.BG == 4 && N % 4 == 0) {
        // four betas per group: the row's four table values are one 16-byte load, fetched (with the
        // row's indices) one pass ahead of their use so that the latency of global memory overlaps
        // the multiply-adds of the pass before
        // (from the copy of the table regrouped by beta group when there is one: neighbouring rows
        // are then neighbouring 16-byte pieces, whole sectors per warp)
        const bool grouped = p.pan.data_g != nullptr && p.pan.g_bg == 4;
        const float* wbase = grouped ? p.pan.data_g + (size_t)(bg0 / 4) * p.pan.g_stride : p.pan.data + bg0;
        const int wstep = grouped ? 4 : N;
        int r = ctx.tid;
        int packed = 0;
        float4 w4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < p.nrows) {
          packed = p.pan.rowmap[r];
          w4 = *reinterpret_cast<const float4*>(wbase + (long)r * wstep);
        }
        while (r < p.nrows) {
          const int rn = r + ctx.nthr;
          int packed_n = 0;
          float4 w4n = make_float4(0.f, 0.f, 0.f, 0.f);
          if (rn < p.nrows) {
            packed_n = p.pan.rowmap[rn];
            w4n = *reinterpret_cast<const float4*>(wbase + (long)rn * wstep);
          }
          int l, m, n;
          rowmap_unpack(packed, l, m, n);
          const float2* src = planes + (m < 0 ? m + N : m) * KP + n;
          const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
          const float4 a01 = acc4[r], a23 = acc4[p.nrows + r];
          float2 a[ZG] = {make_float2(a01.x, a01.y), make_float2(a01.z, a01.w),
                          make_float2(a23.x, a23.y), make_float2(a23.z, a23.w)};
#pragma unroll
          for (int bi = 0; bi < 4; ++bi)
#pragma unroll
            for (int z = 0; z < ZG; ++z) {
              const float2 xv = src[(size_t)(z * 4 + bi) * plane_sz];
              a[z].x = fmaf(wv[bi], xv.x, a[z].x);
              a[z].y = fmaf(wv[bi], xv.y, a[z].y);
            }
          acc4[r] = make_float4(a[0].x, a[0].y, a[1].x, a[1].y);
          acc4[p.nrows + r] = make_float4(a[2].x, a[2].y, a[3].x, a[3].y);
          r = rn;
          packed = packed_n;
          w4 = w4n;
        }
      } else
      for (int r = ctx.tid; r < p.nrows; r += ctx.nthr) {
        int l, m, n;
        rowmap_unpack(p.pan.rowmap[r], l, m, n);
        const float* w = (p.pan.data_g != nullptr && p.pan.g_bg == p.BG)
                             ? p.pan.data_g + (size_t)(bg0 / p.BG) * p.pan.g_stride + (size_t)r * p.BG
                             : p.pan.data + (long)r * N + bg0;
        const float2* src = planes + (m < 0 ? m + N : m) * KP + n;
        const float4 a01 = acc4[r], a23 = acc4[p.nrows + r];
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
        acc4[p.nrows + r] = make_float4(a[2].x, a[2].y, a[3].x, a[3].y);
      }
      ctx.sync();
    }
    if (p.sums && ctx.tid < zc) p.sums[z0 + ctx.tid] = zsum;
    // ---- write the spectrum and its Hermitian mirror ----------------------------------------
    for (int it = ctx.tid; it < p.nrows * ZG; it += ctx.nthr) {
      const int r = it / ZG, z = it - r * ZG;
      if (z >= zc) continue;
      int l, m, n;
      rowmap_unpack(p.pan.rowmap[r], l, m, n);
      const float2 a = acc_at(r, z);
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
__global__ void __launch_bounds__(kFusedMaxThreads) so3_inv_fused(const InvFusedParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_inv_fused_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
template <int N>
__global__ void __launch_bounds__(kFusedMaxThreads) so3_fwd_fused(const FwdFusedParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_fwd_fused_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
// name of an instantiation for the launch records, e.g. "so3_inv_fused<20>" (interned: the
// records keep the pointer)
inline const char* kernel_name_n(const char* base, int n) {
  static std::mutex mu;
  static std::map<std::pair<std::string, int>, std::string> names;
  std::lock_guard<std::mutex> g(mu);
  auto key = std::make_pair(std::string(base), n);
  auto it = names.find(key);
  if (it == names.end())
    it = names.emplace(key, std::string(base) + "<" + std::to_string(n) + ">").first;
  return it->second.c_str();
}
#define S2C_LAUNCH_N(name, N, grid, block, smem, stream, params)                              \
  s2c::launch_impl(name<N>, s2c::kernel_name_n(#name, N), (long)(grid), (int)(block),          \
                   (size_t)(smem), stream, params)
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


// Row stride of a plane in complex numbers: >= N/2 (a row must hold N floats) and odd, so that
// threads walking down a column of rows fall into distinct shared-memory banks.
inline int fused_kp(int N) { return (N / 2) % 2 == 0 ? N / 2 + 1 : N / 2 + 2; }
// Plane stride in complex numbers: padded so that plane p+1 starts K 8-byte banks after plane p
// (threads of consecutive planes reading the same row then continue the bank sequence).
inline int fused_plane_stride(int N, int K) {
  int ps = N * fused_kp(N);
  while (ps % 16 != K % 16) ++ps;
  return ps;
}
inline size_t fused_smem_bytes(int N, int nrows) {
  const int K = N / 2;  // upper bound of the pair count: so3_npairs(K)
  return (size_t)N * sizeof(float2) + (size_t)nrows * kFusedZG * sizeof(float2) +
         (size_t)so3_npairs(K) * sizeof(int4) + ((size_t)nrows * fused_bg(N) + 4) * sizeof(float) + 16 +
         (size_t)kFusedZG * fused_bg(N) * (N * fused_kp(N) + 16) * sizeof(float2);
}
// the analysis keeps no pair list and no table slice in shared memory
inline size_t fwd_fused_smem_bytes(int N, int nrows) {
  return (size_t)N * sizeof(float2) + (size_t)nrows * kFusedZG * sizeof(float2) +
         (size_t)kFusedZG * fused_bg(N) * (N * fused_kp(N) + 16) * sizeof(float2);
}
// Threads per block: 256 cover one transform per thread in every FFT phase; when the block's
// shared memory leaves room for only one block per SM anyway, 512 threads halve the passes of the
// Wigner phases and of the spectrum load / store loops.
inline int fused_threads(size_t smem_bytes, size_t smem_limit) {
  return 2 * (smem_bytes + 1024) > smem_limit ? kFusedMaxThreads : 256;
}

}  // namespace s2c
