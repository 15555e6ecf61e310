// Wigner-d contractions of the large-bandwidth SO(3) path (N = 2b in {64, 128}), written for SMALL
// batch chunks: the scratch array V between the plane kernels (so3_plane_kernels.h) and these
// kernels must stay in L2, so a launch sees only a handful of signals and a tile that reuses a
// staged Wigner panel over many batch elements (wigner_tiled.h) has nothing to reuse it over.
//
// Same arithmetic as so3_fwd_wigner / so3_inv_wigner (so3_kernels.h), i.e. the beta / l contraction
// of the reference's so3fft.cu / so3ifft.cu tile loops (s2cnn/soft/so3_fft.py:296-336, :391-431).
//
// Organisation: the 32 lanes of a warp split the BETA axis; a warp owns the frequency pair
// (+m, n) and (-m, n) for four batch elements, a block of 8 warps eight consecutive values of |m|.
//   * The table holds only the first half of the beta range (TableCache::half_panels): the
//     SOFT grid maps onto itself under beta -> pi - beta and
//         d^l_{m,n}(pi - beta_j) = (-1)^(l+n) d^l_{-m,n}(beta_j),
//     so the second half of panel (m, n) is the first half of panel (-m, n) up to that sign.  A warp
//     reads row l of both half panels once and uses each for both members of its pair.
//   * Panel rows reach a warp through a private ring in shared memory filled by 16-byte
//     asynchronous copies (cp.async), kRowsDepth - 1 steps ahead of their use: with one outstanding
//     row per warp the kernels ran at the latency, not the bandwidth, of L2 / HBM.  (Copies of 4 or
//     8 bytes per lane cost about six times the shared-memory wavefronts of 16-byte ones, so a lane
//     copies 16 bytes and reads the 4 or 8 bytes it needs after a warp barrier.)
//   * analysis: the warp keeps its slice of V in registers for the whole pair and streams the
//     panel rows; every two degrees end with a sum over the lanes (a 32-value transpose-reduce by
//     shuffles, after which lane i holds value i).
//   * synthesis: the accumulators (one beta slice of four signals per lane) stay in registers
//     while the rows stream; no cross-lane traffic at all.
//   * V is [n][z][beta][f] (f = alpha-frequency bin, see so3_plane_kernels.h): rows of one (z, beta)
//     are 8 N bytes apart, so the block moves its 16 columns (+-m) between global and shared memory
//     as 64-byte runs - four neighbouring lanes, 16 bytes each, per run - and the lanes read / write
//     the transposed tile [column][z][beta] without bank conflicts.
#pragma once

#include "backend.h"
#include "so3_kernels.h"

namespace s2c {

constexpr int kRowsMG = 8;      // values of |m| per block = warps per block
constexpr int kRowsZQ = 4;      // batch elements per block (and per warp)
constexpr int kRowsZC = 8;      // batch elements per chunk (what the host sizes V for)
constexpr int kRowsThreads = 32 * kRowsMG;
constexpr int kRowsDepth = 8;   // ring slots per warp

struct HalfPanelsDev {
  int nbeta;                // N = 2 b of the beta grid
  int nl, K, npairs;
  const float* data;        // per pair: rows l = lmin .. nl-1, N/2 floats each (beta_j, j < N/2)
  const long long* off;     // npairs + 1 offsets in floats
};

struct FwdRowsParams {
  const float2* v;      // [n < K][z < zc][beta][f]
  float2* out;          // spectrum rows of out_zstride complex, already offset to the chunk's z0
  long out_zstride;
  HalfPanelsDev pan;
  int zc, K, nl, mode;  // mode: kSo3Real or kSo3AccumI
};

struct InvRowsParams {
  const float2* x;      // spectrum rows of x_zstride complex, offset to the chunk's z0
  long x_zstride;
  float2* s;            // [n < K][z < zc][beta][f]
  HalfPanelsDev pan;
  int zc, K, mode;      // mode: kSo3Real or kSo3RotI
};

// Shared memory: the tile [16 columns][4 z][N beta] of complex numbers with a column stride of
// 4 N + 2 (so that four lanes storing to four columns hit four different bank groups).  The rings
// [warp][depth][rows per step][A, B][N / 2] live inside it: the analysis is done with the tile once
// every warp has its slice of V in registers (8 rings of depth 8 x 2 rows fill it), the synthesis
// keeps the symmetrised spectrum rows in the lower half until the tile is written and its rings
// (depth 8 x 1 row) in the upper half.  (+ in the host-emulation build a per-warp exchange buffer
// that stands in for the shuffles.)
template <int N>
S2C_HD constexpr int rows_cs() { return kRowsZQ * N + 2; }
template <int N>
S2C_HD constexpr int rows_tile_floats() { return 2 * kRowsMG * rows_cs<N>() * 2; }
template <int N>
S2C_HD constexpr int rows_ring_floats(int rows_per_step) { return kRowsDepth * rows_per_step * 2 * (N / 2); }
template <int N>
inline size_t rows_smem_bytes() {
  static_assert(kRowsMG * rows_ring_floats<N>(2) <= rows_tile_floats<N>(), "analysis rings");
  static_assert(kRowsMG * rows_ring_floats<N>(1) <= rows_tile_floats<N>() / 2, "synthesis rings");
  size_t b = (size_t)rows_tile_floats<N>() * sizeof(float);
#ifdef S2C_EMUL
  b += (size_t)kRowsMG * 32 * 33 * sizeof(float);
#endif
  return b;
}

// 16 bytes global -> shared, asynchronously; groups complete in issue order
#ifndef S2C_EMUL
S2C_D void rows_copy16_async(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
S2C_D void rows_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// kRowsDepth - 1 steps are in flight: wait until at most kRowsDepth - 2 of this thread's copy
// groups are pending, i.e. the oldest has landed.  (The step issued next goes into the slot that
// was read one iteration earlier, never into the one being read.)
S2C_D void rows_wait_oldest() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kRowsDepth - 2) : "memory");
}
#else
inline void rows_copy16_async(float* dst, const float* src) {
  for (int i = 0; i < 4; ++i) dst[i] = src[i];
}
inline void rows_commit() {}
inline void rows_wait_oldest() {}
#endif

// ---- sum over the lanes of a warp: v[i] of every lane -> lane i -------------------------------
#ifndef S2C_EMUL
S2C_D float rows_reduce32(const Ctx&, float (&v)[32], int lane, float*) {
#pragma unroll
  for (int step = 16; step >= 1; step >>= 1) {
    const bool upper = (lane & step) != 0;
#pragma unroll
    for (int k = 0; k < step; ++k) {
      const float send = upper ? v[k] : v[k + step];
      const float keep = upper ? v[k + step] : v[k];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, step);
    }
  }
  return v[0];
}
S2C_D float rows_partner(const Ctx&, float v, int, float*) {
  return __shfl_xor_sync(0xffffffffu, v, 1);
}
#else
// every warp of the block calls these equally often (a warp barrier is a block barrier here)
inline float rows_reduce32(const Ctx& ctx, float (&v)[32], int lane, float* xch) {
  for (int k = 0; k < 32; ++k) xch[lane * 33 + k] = v[k];
  ctx.sync_warp();
  float s = 0.f;
  for (int t = 0; t < 32; ++t) s += xch[t * 33 + lane];
  ctx.sync_warp();
  return s;
}
inline float rows_partner(const Ctx& ctx, float v, int lane, float* xch) {
  xch[lane] = v;
  ctx.sync_warp();
  const float r = xch[lane ^ 1];
  ctx.sync_warp();
  return r;
}
#endif

// which (n, |m| group, z quad) a block owns, and the columns of its tile:
//   c < 8:   frequency +(m0 + c)      at bin f = m0 + c
//   c >= 8:  frequency -(m0 + c - 8)  at bin f = N - (m0 + c - 8)      (not for m = 0)
struct RowsGeom {
  int n, m0, zq;
};
S2C_D RowsGeom rows_geom(int bid, int K, int zc) {
  const int ngroups = (K + kRowsMG - 1) / kRowsMG, nzq = (zc + kRowsZQ - 1) / kRowsZQ;
  RowsGeom g;
  g.zq = bid % nzq;
  const int t = bid / nzq;
  g.n = t / ngroups;
  g.m0 = (t - g.n * ngroups) * kRowsMG;
  return g;
}
inline long rows_grid(int K, int zc) {
  return (long)K * ((K + kRowsMG - 1) / kRowsMG) * ((zc + kRowsZQ - 1) / kRowsZQ);
}

// half-panel rows of the pair (+m, n) and (-m, n); for n = 0 only m >= 0 is stored and
// d_{-m,0} = (-1)^m d_{m,0}; for m = 0 the two coincide
struct RowsPanels {
  const float* a;      // half panel of (+m, n)
  const float* b;      // half panel of (-m, n) (or of (+m, n) with `bsign`)
  float bsign;
};
S2C_D RowsPanels rows_panels(const HalfPanelsDev& pan, int m, int n) {
  RowsPanels r;
  r.a = pan.data + pan.off[so3_pair_index(m, n, pan.K)];
  if (n == 0 || m == 0) {
    r.b = r.a;
    r.bsign = (n == 0 && (m & 1)) ? -1.f : 1.f;
  } else {
    r.b = pan.data + pan.off[so3_pair_index(-m, n, pan.K)];
    r.bsign = 1.f;
  }
  return r;
}

// One ring step = S rows of both half panels: [row][A, B][NH] floats, copied 16 bytes per lane.
template <int N, int S>
S2C_D void rows_issue(float* ring, int t, const float* pa, const float* pb, int L, int lane) {
  constexpr int NH = N / 2, P = NH / 4;      // 16-byte pieces per half-panel row
  float* slot = ring + (t % kRowsDepth) * (S * 2 * NH);
#pragma unroll
  for (int piece = lane; piece < S * 2 * P; piece += 32) {
    const int r = piece / (2 * P), rem = piece - r * 2 * P, ab = rem / P, q = rem - ab * P;
    const int row = S * t + r;
    if (row < L)
      rows_copy16_async(slot + (r * 2 + ab) * NH + 4 * q, (ab ? pb : pa) + (long)row * NH + 4 * q);
  }
  rows_commit();   // one group per step, empty or not, so that the wait counts steps
}

// The tile rows a thread moves: thread = (run piece q < 4, row r0 < 64), rows r0 + 64 k.
template <int N>
struct RowsTileMap {
  static constexpr int kPasses = kRowsZQ * N / 64;
  int q, r0;
  S2C_D explicit RowsTileMap(int tid) : q(tid & 3), r0(tid >> 2) {}
};

// ---------------------------------------------------------------------------------------------
// analysis:  X[l, +-m, n][z] = sum_beta W[l][beta] V[z][beta]   (+ Hermitian mirror rows)
// ---------------------------------------------------------------------------------------------
template <int N>
struct so3_fwd_wigner_r_impl {
  static S2C_D void run(const Ctx& ctx, const FwdRowsParams& p, unsigned char* smem) {
    constexpr int NH = N / 2, JL = NH / 32;           // betas of the half range per lane
    constexpr int ZS = N, CS = rows_cs<N>();          // tile strides (complex): z, column
    float2* tile = reinterpret_cast<float2*>(smem);   // [16][4][N] (column stride CS)
    const int warp = ctx.tid >> 5, lane = ctx.tid & 31;
    // ring step = two degrees: [depth][row 0 / 1][A / B][NH]; reuses the tile's memory (see below)
    float* ring = reinterpret_cast<float*>(smem) + warp * rows_ring_floats<N>(2);
    float* xch = reinterpret_cast<float*>(smem) + rows_tile_floats<N>() + warp * 32 * 33;
    const int K = p.K, zc = p.zc;
    const RowsGeom g = rows_geom(ctx.bid, K, zc);
    const int n = g.n, m0 = g.m0, zbase = g.zq * kRowsZQ;

    // ---- stage the block's columns of V: tile[c][z][beta] ----------------------------------------
    // Per (z, beta) row: bins m0 .. m0+7 (64 aligned bytes) and bins N-m0-7 .. N-m0, read as the
    // aligned run N-m0-8 .. N-m0-1 plus the single bin N-m0.  All loads of a thread are issued
    // before the first value is used.
    {
      const RowsTileMap<N> tm(ctx.tid);
      constexpr int kP = RowsTileMap<N>::kPasses;
      const float2* vn = p.v + ((long)n * zc + zbase) * N * N;
      float4 pos[kP], neg[kP];
      float2 one[kP];
#pragma unroll
      for (int k = 0; k < kP; ++k) {
        const int r = tm.r0 + 64 * k, z = r / N;
        pos[k] = neg[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        one[k] = make_float2(0.f, 0.f);
        if (zbase + z < zc) {
          const float2* row = vn + (long)r * N;           // r = z * N + beta
          pos[k] = *reinterpret_cast<const float4*>(row + m0 + 2 * tm.q);
          neg[k] = *reinterpret_cast<const float4*>(row + N - m0 - 8 + 2 * tm.q);
          if (tm.q == 0 && m0 > 0) one[k] = row[N - m0];
        }
      }
#pragma unroll
      for (int k = 0; k < kP; ++k) {
        const int r = tm.r0 + 64 * k, z = r / N, beta = r - z * N;
        float2* dst = tile + z * ZS + beta;
        dst[(2 * tm.q) * CS] = make_float2(pos[k].x, pos[k].y);
        dst[(2 * tm.q + 1) * CS] = make_float2(pos[k].z, pos[k].w);
        // bins N-m0-8+2q, N-m0-7+2q are the frequencies -(m0+8-2q), -(m0+7-2q)
        if (tm.q > 0) dst[(16 - 2 * tm.q) * CS] = make_float2(neg[k].x, neg[k].y);
        dst[(15 - 2 * tm.q) * CS] = make_float2(neg[k].z, neg[k].w);
        if (tm.q == 0) dst[8 * CS] = one[k];
      }
    }
    ctx.sync();

    const int m = m0 + warp;
    const int lmin = m > n ? m : n;
    const int L = (m < K) ? p.nl - lmin : 0;
#ifdef S2C_EMUL
    const int lmin_blk = m0 > n ? m0 : n;
    const int Lloop = p.nl - lmin_blk > 0 ? p.nl - lmin_blk : 0;   // uniform over the block
#else
    const int Lloop = L;
#endif

    // ---- this lane's slice of V: betas j (p) and N-1-j (q) of the columns +m and -m ----------------
    float2 vp[2][kRowsZQ][JL], vq[2][kRowsZQ][JL];
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int z = 0; z < kRowsZQ; ++z)
#pragma unroll
        for (int jj = 0; jj < JL; ++jj) {
          const int j = JL * lane + jj;
          const float2* col = tile + (s * kRowsMG + warp) * CS + z * ZS;
          vp[s][z][jj] = col[j];
          vq[s][z][jj] = col[N - 1 - j];
        }

    RowsPanels pn;
    pn.a = pn.b = p.pan.data;
    pn.bsign = 1.f;
    if (L > 0) pn = rows_panels(p.pan, m, n);
    const bool self = (m == 0);
    ctx.sync();   // every warp has its slice of V in registers: the tile's memory becomes the rings
#ifndef S2C_EMUL
    if (L <= 0) return;   // no block barrier below this point
#endif
    for (int t = 0; t < kRowsDepth - 1; ++t) rows_issue<N, 2>(ring, t, pn.a, pn.b, L, lane);

    // This lane's output in every step: value lane = r * 16 + s * 8 + z * 2 + c of the transpose-
    // reduce, i.e. degree lmin + li + r, frequency +-m, batch element z, real / imaginary part.
    // Its spectrum row and the Hermitian mirror row advance by two degrees per step; with
    // row(l, m, n) = l (4 l^2 - 1) / 3 + (l + m)(2 l + 1) + l + n the step is a quadratic in l, kept
    // by differences (no multiplications or divisions in the loop).
    const int o_r = lane >> 4, o_s = (lane >> 3) & 1, o_z = (lane >> 1) & 3, o_c = lane & 1;
    const int o_mm = o_s ? -m : m;
    const bool o_ok = zbase + o_z < zc && !(self && o_s == 1);
    const float o_fudge = ((o_mm - n) & 1) ? -1.f : 1.f;
    float* const o_base = reinterpret_cast<float*>(p.out + zbase + o_z) + o_c;
    const long o_zs2 = 2 * p.out_zstride;
    int o_row1 = (int)so3_row(lmin + o_r, o_mm, n), o_row2 = (int)so3_row(lmin + o_r, -o_mm, -n);
    int o_d1 = 8 * (lmin + o_r) * (lmin + o_r) + 24 * (lmin + o_r) + 22 + 4 * o_mm;
    int o_d2 = o_d1 - 8 * o_mm, o_dd = 32 * (lmin + o_r) + 80;

    float va[2][JL], vb[2][JL];     // rows li, li + 1 of the two half panels
    for (int li = 0; li < Lloop; li += 2) {
      rows_wait_oldest();
      ctx.sync_warp();              // the other lanes' pieces of this step have landed, too
      {
        const float* slot = ring + ((li / 2) % kRowsDepth) * (4 * NH) + JL * lane;
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int jj = 0; jj < JL; ++jj) {
            const bool ok = li + r < L;
            va[r][jj] = ok ? slot[(2 * r) * NH + jj] : 0.f;
            vb[r][jj] = ok ? pn.bsign * slot[(2 * r + 1) * NH + jj] : 0.f;
          }
      }
      rows_issue<N, 2>(ring, li / 2 + kRowsDepth - 1, pn.a, pn.b, L, lane);
      float val[32];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int l = lmin + li + r;
        const float sl = ((l + n) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int z = 0; z < kRowsZQ; ++z) {
          float pr = 0.f, pi = 0.f, qr = 0.f, qi = 0.f;
#pragma unroll
          for (int jj = 0; jj < JL; ++jj) {
            const float a = va[r][jj], b = vb[r][jj], sa = sl * a, sb = sl * b;
            // X_{+m} = sum A Vp_{+m} + s B Vq_{+m};   X_{-m} = sum B Vp_{-m} + s A Vq_{-m}
            pr = fmaf(a, vp[0][z][jj].x, pr);  pi = fmaf(a, vp[0][z][jj].y, pi);
            pr = fmaf(sb, vq[0][z][jj].x, pr); pi = fmaf(sb, vq[0][z][jj].y, pi);
            qr = fmaf(b, vp[1][z][jj].x, qr);  qi = fmaf(b, vp[1][z][jj].y, qi);
            qr = fmaf(sa, vq[1][z][jj].x, qr); qi = fmaf(sa, vq[1][z][jj].y, qi);
          }
          val[r * 16 + 0 * 8 + z * 2 + 0] = pr;
          val[r * 16 + 0 * 8 + z * 2 + 1] = pi;
          val[r * 16 + 1 * 8 + z * 2 + 0] = qr;
          val[r * 16 + 1 * 8 + z * 2 + 1] = qi;
        }
      }
      const float mine = rows_reduce32(ctx, val, lane, xch);   // value `lane` summed over the warp
      const float other = rows_partner(ctx, mine, lane, xch);  // the other component of the number
      if (li + o_r < L && o_ok) {
        float* o1 = o_base + o_row1 * o_zs2;
        const bool mirror = n > 0;      // for n = 0 the mirror (-m, 0) is computed directly
        float* o2 = o_base + o_row2 * o_zs2;
        if (p.mode == kSo3Real) {
          *o1 = mine;
          if (mirror) *o2 = o_c ? -o_fudge * mine : o_fudge * mine;
        } else {   // += i * (re + i im):  re -= im, im += re;   mirror += i * fudge * conj
          *o1 += o_c ? other : -other;
          if (mirror) *o2 += o_fudge * other;
        }
      }
      o_row1 += o_d1;
      o_row2 += o_d2;
      o_d1 += o_dd;
      o_d2 += o_dd;
      o_dd += 64;
    }
  }
};

// ---------------------------------------------------------------------------------------------
// synthesis:  S[z][beta] = sum_l W[l][beta] Xs[l][z],  Xs = symmetrised spectrum
// ---------------------------------------------------------------------------------------------
template <int N>
struct so3_inv_wigner_r_impl {
  static S2C_D void run(const Ctx& ctx, const InvRowsParams& p, unsigned char* smem) {
    constexpr int NH = N / 2, JL = NH / 32;
    constexpr int ZS = N, CS = rows_cs<N>();
    float2* tile = reinterpret_cast<float2*>(smem);     // [16][4][N], written after the loop
    float2* xs = tile;                                    // before: [16][Lmax][4] symmetrised rows
    const int warp = ctx.tid >> 5, lane = ctx.tid & 31;
    // ring step = one degree: [depth][A / B][NH], in the upper half of the tile's memory
    float* ring = reinterpret_cast<float*>(smem) + rows_tile_floats<N>() / 2 + warp * rows_ring_floats<N>(1);
    const int K = p.K, zc = p.zc, nl = p.pan.nl;
    const RowsGeom g = rows_geom(ctx.bid, K, zc);
    const int n = g.n, m0 = g.m0, zbase = g.zq * kRowsZQ;
    const int lmin_blk = m0 > n ? m0 : n;
    const int Lmax = nl - lmin_blk;                      // rows of the block's longest pair (<= N/2)

    // ---- symmetrised spectrum rows of the block's 16 columns: xs[c][li][z], li from lmin_blk ------
    // thread = (z, li); the loads of all 16 columns are issued before any is used
    {
      const int z = ctx.tid % kRowsZQ;
      for (int li = ctx.tid / kRowsZQ; li < Lmax; li += kRowsThreads / kRowsZQ) {
        const int l = lmin_blk + li;
        float2 a[2 * kRowsMG], b[2 * kRowsMG];
#pragma unroll
        for (int c = 0; c < 2 * kRowsMG; ++c) {
          const int mabs = m0 + (c % kRowsMG);
          const int mm = c < kRowsMG ? mabs : -mabs;
          const bool ok = zbase + z < zc && mabs < K && l >= mabs && !(c >= kRowsMG && mabs == 0);
          a[c] = b[c] = make_float2(0.f, 0.f);
          if (ok) {
            a[c] = p.x[so3_row(l, mm, n) * p.x_zstride + zbase + z];
            b[c] = p.x[so3_row(l, -mm, -n) * p.x_zstride + zbase + z];
          }
        }
#pragma unroll
        for (int c = 0; c < 2 * kRowsMG; ++c) {
          const int mabs = m0 + (c % kRowsMG);
          const int mm = c < kRowsMG ? mabs : -mabs;
          float2 u = a[c], w = b[c];
          if (p.mode == kSo3RotI) {  // multiply the spectrum by -i
            u = make_float2(u.y, -u.x);
            w = make_float2(w.y, -w.x);
          }
          const float fudge = ((mm - n) & 1) ? -1.f : 1.f;
          xs[(c * Lmax + li) * kRowsZQ + z] =
              make_float2(0.5f * (u.x + fudge * w.x), 0.5f * (u.y - fudge * w.y));
        }
      }
    }
    ctx.sync();

    const int m = m0 + warp;
    const int lmin = m > n ? m : n;
    const int L = (m < K) ? nl - lmin : 0;
#ifdef S2C_EMUL
    const int Lloop = Lmax;        // uniform over the block: a warp barrier is a block barrier here
#else
    const int Lloop = L;
#endif

    // accumulators: betas j (p) and N-1-j (q) of the columns +m (0) and -m (1)
    float2 sp[2][kRowsZQ][JL], sq[2][kRowsZQ][JL];
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int z = 0; z < kRowsZQ; ++z)
#pragma unroll
        for (int jj = 0; jj < JL; ++jj) sp[s][z][jj] = sq[s][z][jj] = make_float2(0.f, 0.f);

    {
      RowsPanels pn;
      pn.a = pn.b = p.pan.data;
      pn.bsign = 1.f;
      if (L > 0) pn = rows_panels(p.pan, m, n);
      const int lrel = L > 0 ? lmin - lmin_blk : 0;
      const float2* x0 = xs + ((0 * kRowsMG + warp) * Lmax + lrel) * kRowsZQ;
      const float2* x1 = xs + ((1 * kRowsMG + warp) * Lmax + lrel) * kRowsZQ;
      if (Lloop > 0)
        for (int t = 0; t < kRowsDepth - 1; ++t) rows_issue<N, 1>(ring, t, pn.a, pn.b, L, lane);
      float a[JL], b[JL];
      for (int li = 0; li < Lloop; ++li) {
        rows_wait_oldest();
        ctx.sync_warp();            // the other lanes' pieces of this row have landed, too
        const bool act = li < L;
        {
          const float* slot = ring + (li % kRowsDepth) * (2 * NH) + JL * lane;
#pragma unroll
          for (int jj = 0; jj < JL; ++jj) {
            a[jj] = act ? slot[jj] : 0.f;
            b[jj] = act ? pn.bsign * slot[NH + jj] : 0.f;
          }
        }
        rows_issue<N, 1>(ring, li + kRowsDepth - 1, pn.a, pn.b, L, lane);
        if (!act) continue;
        const int l = lmin + li;
        const float sl = ((l + n) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int z = 0; z < kRowsZQ; ++z) {
          const float2 xp = x0[li * kRowsZQ + z], xm = x1[li * kRowsZQ + z];
#pragma unroll
          for (int jj = 0; jj < JL; ++jj) {
            const float sa = sl * a[jj], sb = sl * b[jj];
            // S_{+m}[j] += A X_{+m};  S_{+m}[N-1-j] += s B X_{+m};  S_{-m}[j] += B X_{-m};  S_{-m}[N-1-j] += s A X_{-m}
            sp[0][z][jj].x = fmaf(a[jj], xp.x, sp[0][z][jj].x); sp[0][z][jj].y = fmaf(a[jj], xp.y, sp[0][z][jj].y);
            sq[0][z][jj].x = fmaf(sb, xp.x, sq[0][z][jj].x);    sq[0][z][jj].y = fmaf(sb, xp.y, sq[0][z][jj].y);
            sp[1][z][jj].x = fmaf(b[jj], xm.x, sp[1][z][jj].x); sp[1][z][jj].y = fmaf(b[jj], xm.y, sp[1][z][jj].y);
            sq[1][z][jj].x = fmaf(sa, xm.x, sq[1][z][jj].x);    sq[1][z][jj].y = fmaf(sa, xm.y, sq[1][z][jj].y);
          }
        }
      }
    }
    ctx.sync();   // every warp is done with the spectrum rows and its ring; the memory becomes the tile

#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int z = 0; z < kRowsZQ; ++z)
#pragma unroll
        for (int jj = 0; jj < JL; ++jj) {
          const int j = JL * lane + jj;
          float2* col = tile + (s * kRowsMG + warp) * CS + z * ZS;
          col[j] = sp[s][z][jj];
          col[N - 1 - j] = sq[s][z][jj];
        }
    ctx.sync();

    // ---- tile -> V[n][z][beta][f], the transfer of the analysis reversed ----------------------------
    // Only bins of this block's own frequencies are written: m0 .. m0+7 (all of them: bins of
    // frequencies >= K are never read by anyone) and N - m for m0 <= m <= m0+7, 0 < m < K.
    {
      const RowsTileMap<N> tm(ctx.tid);
      constexpr int kP = RowsTileMap<N>::kPasses;
      float2* vn = p.s + ((long)n * zc + zbase) * N * N;
#pragma unroll
      for (int k = 0; k < kP; ++k) {
        const int r = tm.r0 + 64 * k, z = r / N, beta = r - z * N;
        if (zbase + z >= zc) continue;
        const float2* src = tile + z * ZS + beta;
        float2* row = vn + (long)r * N;
        const float2 c0 = src[(2 * tm.q) * CS], c1 = src[(2 * tm.q + 1) * CS];
        *reinterpret_cast<float4*>(row + m0 + 2 * tm.q) = make_float4(c0.x, c0.y, c1.x, c1.y);
        const int m_hi = m0 + 8 - 2 * tm.q, m_lo = m0 + 7 - 2 * tm.q;   // bins N-m0-8+2q and the next
        const float2 d_lo = src[(15 - 2 * tm.q) * CS];
        if (tm.q > 0 && m_hi < K) {
          const float2 d_hi = src[(16 - 2 * tm.q) * CS];
          *reinterpret_cast<float4*>(row + N - m_hi) = make_float4(d_hi.x, d_hi.y, d_lo.x, d_lo.y);
        } else if (m_lo < K) {
          row[N - m_lo] = d_lo;
        }
        if (tm.q == 0 && m0 > 0 && m0 < K) row[N - m0] = src[8 * CS];
      }
    }
  }
};

#ifndef S2C_EMUL
template <int N>
__global__ void __launch_bounds__(kRowsThreads, 2) so3_fwd_wigner_r(const FwdRowsParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_fwd_wigner_r_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
template <int N>
__global__ void __launch_bounds__(kRowsThreads, 2) so3_inv_wigner_r(const InvRowsParams p) {
  extern __shared__ float4 s2c_dyn_smem[];
  Ctx ctx{(int)threadIdx.x, (int)blockDim.x, (int)blockIdx.x, (int)gridDim.x};
  so3_inv_wigner_r_impl<N>::run(ctx, p, reinterpret_cast<unsigned char*>(s2c_dyn_smem));
}
#define S2C_LAUNCH_ROWS(name, N, grid, stream, params)                                         \
  s2c::launch_impl(name<N>, #name, (long)(grid), s2c::kRowsThreads, s2c::rows_smem_bytes<N>(), \
                   stream, params)
#else
#define S2C_LAUNCH_ROWS(name, N, grid, stream, params)                                         \
  s2c::emu_launch<name##_impl<N>>(#name, (long)(grid), s2c::kRowsThreads,                      \
                                  s2c::rows_smem_bytes<N>(), params)
#endif

}  // namespace s2c
