// tcgen05 tensor-core path of the ISSM scan: backward.
//
// Same decomposition as the forward (one CTA per (batch, head) stream, thread t = state column n,
// 64-point sub-blocks), walked in REVERSE scan order while carrying G[n, p] = dLoss/dS (fp32, TMEM).
// With Cd = C 2^a, Bd = B dt 2^-a (a: in-block cumsum of dt*A in log2 units, relative to the block
// start), dy the gradient of the pre-skip / pre-gate output rows, S the state entering the
// block (saved by the forward) and g' = 2^(a_last) G, every O(rows x rows x states)
// term of issm_triton/issm_combined.py:95-179 becomes a tensor-core contraction:
//   dM  = tril(dy x^T)                  64 x 64,  K = P      (issm_chunk_scan.py:828)
//   M   = tril(Cd Bd^T)                 64 x 64,  K = N      (recomputed, issm_combined.py:141)
//   BD^T[n,s] = sum_l Cd[l,n] dM[l,s] + sum_p g'[n,p] x[s,p]      128 x 64 per 128 states
//   CD^T[n,l] = sum_s Bd[s,n] dM[l,s] + sum_p S[n,p] dy[l,p]      128 x 64 per 128 states
//   dx[l,p]   = sum_n Bd[l,n] g'[n,p] + sum_t M[t,l] dy[t,p]       64 x 48
//   G[n,p]   <- 2^(a_last) G[n,p] + sum_l Cd[l,n] dy[l,p]          128 x 48
// and the per-(row, state) epilogue, done by the thread that owns the state column, is
//   dC_h = 2^a CD,  dB_h = dt 2^-a BD,  ddt_direct = B 2^-a BD,
//   dacs = Cd CD - Bd BD,  ddA[l] = sum_{t>=l} dacs[t] + <S_next[n,:], G[n,:]>,
//   ddt = (ddt_direct + ddA A) * [not clamped] * sigmoid(pre),  dA += ddA dt,  ddt_bias += ddt
// (replacing issm_combined.py:451, issm_cabt_bmm.py:539, issm_chunk_scan.py:573/948,
// issm_chunk_state.py:559/159 and the torch glue of issm_combined.py:159-175).
// Per-head dB / dC partials go to a workspace as packed bf16 pairs and are summed over heads by a second kernel.
#include "issm_tensor.cuh"

namespace issm {

template <int NT>
struct BwdSmem {
  static constexpr int kCd = 0;                         // [NT/64 atoms][64 l][128 B]
  static constexpr int kBd = kCd + NT * 128;
  static constexpr int kGop = kBd + NT * 128;           // [NT n][128 B]: g' rows, p contiguous (SW128) ...
  static constexpr int kSC = kGop;                      // ... time-shared with the staged C rows [64][NT] bf16
  static constexpr int kSop = kGop + NT * 128;          // [PP/8][NT n][16 B]: S rows (interleaved)
  static constexpr int kX = kSop + NT * (PP * 2);       // [64 l][128 B]
  static constexpr int kDy = kX + QB * 128;             // [64 l][128 B]
  static constexpr int kDMm = kDy + QB * 128;           // [64 l][128 B], s contiguous
  static constexpr int kMm = kDMm + QB * 128;           // [64 l][128 B]
  static constexpr int kSdt = kMm + QB * 128;           // staging [64][NT] bf16
  static constexpr int kSB = kSdt + QB * NT * 2;
  static constexpr int kXch = kSB + QB * NT * 2;        // [4][NT] float: per-half exchange (sum dt*A, <S,G>, sum dacs)
  static constexpr int kRed = kSdt;                     // dD reduction scratch (after the walk)
  static constexpr int kDxT = kXch + 4 * NT * 4;        // [64][DXS] bf16: dx accumulator rows on their way to global memory
  static constexpr int DXS = 40;                        // row stride of that tile (headdim <= 40 on this path)
  static constexpr int kBars = kDxT + QB * DXS * 2;
  static constexpr int kTotal = kBars + 128;             // 8 mbarriers, TMEM holder, window flag
};

// Thread layout (as in the forward): 2*NT column threads, one service warp, three tile-I/O warps.
// Column thread (n = tid % NT, half = tid / NT) owns rows [32 half, 32 half + 32) of state column n in
// the operand pass and in the (row, state) epilogue, and columns [24 half, 24 half + 24) of TMEM lane n
// of the state gradient G, which lives in TMEM for the whole walk.
//
// As in the forward there are two instantiations: kWin = false is the fast kernel, which only marks a stream
// holding a block outside the range of the single-reference factorisation in a.redo; kWin = true is launched
// right behind it, returns at once for unmarked streams and redoes marked ones from the start.  In that kernel a
// flagged block is cut into 2^k row windows (see window_need) that are processed last to first, each as a
// pass of the ordinary block code restricted to the window's rows, with its own reference, the state entering the
// window as the S operand and the rescaled G as g'.  The window-entry states come from a short forward walk over
// the block's windows (S += Bd^T x on the tensor cores, rescale, bf16 copy to a.wscr) run first.
// kMode fixes the row order of the staged tiles at compile time, so that their addresses need no multiply:
// 1 = dt / B / C tiles staged in scan order (forward scan of regular arrays), 2 = staged in memory order for a
// reversed scan (walked backwards), 0 = decided at run time (row-by-row copies, mixed layouts).
template <int NT, typename TDT, bool kWin, int kMode>
__global__ void __launch_bounds__(2 * NT + 128, 1) k_bwd_tensor(const __grid_constant__ TArgs a, const __grid_constant__ CUtensorMap dtmap) {
  using SM = BwdSmem<NT>;
  constexpr bool kStageDt = sizeof(TDT) == 2;
  constexpr int NTH = 2 * NT;
  constexpr int NIO = 96;
  constexpr int HP = PP / 2;
  constexpr int NCG = NT / 64;                          // column groups of the row epilogues
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte aligned base, kept as "shared array + offset" so that the compiler still knows the address space
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bar1 = (uint64_t*)(smem + SM::kBars);
  uint64_t* bar2 = bar1 + 1;
  uint64_t* barS = bar1 + 2;     // dt staging
  uint64_t* barT = bar1 + 3;     // B staging
  uint64_t* barU = bar1 + 4;     // S operand (saved block-entry state)
  uint64_t* barV = bar1 + 5;     // C staging
  uint64_t* barW = bar1 + 6;     // MMAs of the window-entry-state walk (windowed blocks only)
  uint64_t* barX = bar1 + 7;     // windowed kernel: last MMA of a block (bar2 completes once per window there)
  uint64_t* bar2b = bar1 + 8;    // second half of MMA phase 2 (G, dx); bar2 covers BD^T / CD^T, which the epilogue needs first
  uint32_t* tmem_holder = (uint32_t*)(bar1 + 9);
  uint32_t* sFlag = tmem_holder + 1;                     // (iteration + 1) * 8 + log2(windows) of a block that needs windows
  float* sXch = (float*)(smem + SM::kXch);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_col = tid < NTH;
  const bool is_svc = warp == NTH / 32;
  const bool is_io = tid >= NTH + 32;
  const int io_t = tid - NTH - 32;
  const int h = blockIdx.y, b = blockIdx.z, g = h / a.hpg;
  // more than 256 states: blockIdx.x is a slice of 256 states, an independent scan over the same x (see the forward
  // kernel); its dx rows are partial sums that k_combine_dx adds, everything per state is the slice's own
  const int n_off = blockIdx.x * NT;
  const int stream = (blockIdx.x * a.b + b) * a.H + h;
  if (kWin && !a.redo[stream]) return;                   // the fast kernel finished this stream
  const int n = tid % NT, half = (tid / NT) & 1;
  const int ng = n_off + n;                              // state index in the (nheads, dstate) / (..., dstate) arrays
  const TDT* __restrict__ dtp = (const TDT*)a.dt + b * a.dt_sb + h * a.dt_sh + n_off;
  const bf16* __restrict__ Bp = a.B + b * a.B_sb + g * a.B_sg + n_off;
  const bf16* __restrict__ Cp = a.C + b * a.C_sb + g * a.C_sg + n_off;
  const bf16* __restrict__ xp = a.x + b * a.x_sb + h * a.x_sh;
  const bf16* __restrict__ zp = a.has_z ? a.z + b * a.z_sb + h * a.z_sh : nullptr;
  const bf16* __restrict__ yp = a.has_z ? a.out_x + b * a.o_sb + h * a.o_sh : nullptr;
  const bf16* __restrict__ gp = a.dout + b * a.g_sb + h * a.g_sh;
  const float A2 = __ldg(a.A + h * a.N + ng) * LOG2E;
  const float Anat = __ldg(a.A + h * a.N + ng);
  const float bias = a.has_bias ? __ldg(a.bias + h * a.N + ng) : 0.f;
  // the same constants for the two adjacent states (2 pr, 2 pr + 1) of the fast instantiation's operand pass
  const int pr0 = n_off + 2 * (tid % (NT / 2));
  const float2 A2p = f2(__ldg(a.A + h * a.N + pr0) * LOG2E, __ldg(a.A + h * a.N + pr0 + 1) * LOG2E);
  const float bsc = a.softplus ? LOG2E : 1.f;
  const float2 biasL2 = a.has_bias ? f2(__ldg(a.bias + h * a.N + pr0) * bsc, __ldg(a.bias + h * a.N + pr0 + 1) * bsc) : f2(0.f);
  const int nblk = (a.L + QB - 1) / QB;
  const size_t bh = (size_t)b * a.H + h;

  for (int i = tid; i < (SM::kSdt - SM::kGop) / 16; i += blockDim.x) ((uint4*)(smem + SM::kGop))[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    mbar_init(bar1, 1); mbar_init(bar2, 1); mbar_init(barS, 1); mbar_init(barT, 1); mbar_init(barU, 1); mbar_init(barV, 1);
    mbar_init(barW, 1); mbar_init(barX, 1); mbar_init(bar2b, 1);
    mbar_fence_init();
    *sFlag = 0;
  }
  if (warp == 0) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const int slab = n >> 7;
  const uint32_t t_dM = tmem, t_M = tmem + 64, t_dx = tmem;
  const uint32_t t_BD = tmem + lane_base + 128 + slab * 64 + half * 32;   // this thread's 32 rows of BD^T[n, :]
  const uint32_t t_CD = tmem + lane_base + 256 + slab * 64 + half * 32;
  const uint32_t t_G = tmem + lane_base + 384 + slab * PP + half * HP;    // this thread's part of G[n, :]
  const int kcol = n & 63;
  const bool flipB = kMode ? kMode == 2 : (a.bc_contig && a.rev);   // staged B rows are in memory order

  // ---- service warp: bulk prefetches ------------------------------------------------------------------
  auto prefetch_dt = [&](int blk) {
    if (!kStageDt) return;
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    if (a.dt_tma) {                                        // one tiled TMA load; the tile is staged in memory order
      if (lane == 0) {
        mbar_expect_tx(barS, (uint32_t)QB * NT * 2);
        tma_load_2d(smem + SM::kSdt, &dtmap, h * (int)a.dt_sh + n_off, b * a.L + (a.rev ? a.L - row0 - rows : row0), barS);
      }
      return;
    }
    if (lane == 0) mbar_expect_tx(barS, (uint32_t)rows * NT * 2);
    __syncwarp();
    for (int l = lane; l < rows; l += 32)
      bulk_g2s(smem + SM::kSdt + l * NT * 2, (const bf16*)dtp + (int64_t)trow(a, row0 + l) * a.dt_sl, NT * 2, barS);
  };
  auto prefetch_B = [&](int blk) {
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    if (lane == 0) mbar_expect_tx(barT, (uint32_t)rows * NT * 2);
    __syncwarp();
    if (a.bc_contig) {
      const int64_t m0 = a.rev ? a.L - row0 - rows : row0;
      if (lane == 0) bulk_g2s(smem + SM::kSB, Bp + m0 * a.B_sl, (uint32_t)rows * NT * 2, barT);
    } else {
      for (int l = lane; l < rows; l += 32)
        bulk_g2s(smem + SM::kSB + l * NT * 2, Bp + (int64_t)trow(a, row0 + l) * a.B_sl, NT * 2, barT);
    }
  };
  // C rows share their buffer with the g' operand: valid from here until the operand pass of the block ends
  auto prefetch_C = [&](int blk) {
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    if (lane == 0) mbar_expect_tx(barV, (uint32_t)rows * NT * 2);
    __syncwarp();
    if (a.bc_contig) {
      const int64_t m0 = a.rev ? a.L - row0 - rows : row0;
      if (lane == 0) bulk_g2s(smem + SM::kSC, Cp + m0 * a.C_sl, (uint32_t)rows * NT * 2, barV);
    } else {
      for (int l = lane; l < rows; l += 32)
        bulk_g2s(smem + SM::kSC + l * NT * 2, Cp + (int64_t)trow(a, row0 + l) * a.C_sl, NT * 2, barV);
    }
  };
  // state entering block `blk` (or the final state, blk = nblk): one copy, already in operand layout
  auto prefetch_S = [&](int blk) {
    if (lane == 0) {
      mbar_expect_tx(barU, (uint32_t)NT * PP * 2);
      const bf16* src = a.saved + (bh * (nblk + 1) + blk) * (size_t)a.N * PP;
      if (a.N == NT) {
        bulk_g2s(smem + SM::kSop, src, (uint32_t)NT * PP * 2, barU);
      } else {                                             // a slice of the states: its part of each of the PP / 8 head-dim chunks
#pragma unroll
        for (int c = 0; c < PP / 8; ++c)
          bulk_g2s(smem + SM::kSop + c * (NT * 16), src + ((size_t)c * a.N + n_off) * 8, (uint32_t)NT * 16, barU);
      }
    }
  };
  if (is_svc) { prefetch_dt(nblk - 1); prefetch_B(nblk - 1); prefetch_C(nblk - 1); prefetch_S(nblk); }

  // ---- column threads: G <- dfinal ---------------------------------------------------------------------
  if (is_col) {
    float gc[HP];
    const float* __restrict__ df = a.dfinal ? a.dfinal + (bh * a.P) * a.N + ng : nullptr;
#pragma unroll
    for (int j = 0; j < HP; ++j) gc[j] = (df && half * HP + j < a.P) ? df[(size_t)(half * HP + j) * a.N] : 0.f;
    tmem_st16(t_G, gc);
    tmem_st8(t_G + 16, gc + 16);
    tmem_st_wait();
  }

  // ---- I/O threads: groups of 4 consecutive head-dim elements, 8-byte accesses (see the forward kernel) -----
  constexpr int XG = (QB * (PP / 4) + NIO - 1) / NIO;    // groups per I/O thread (8)
  const int ngrp = a.P / 4;
  const int io_l0 = io_t / ngrp, io_g0 = io_t % ngrp, io_dl = NIO / ngrp, io_dg = NIO % ngrp;
  auto io_next = [&](int& l, int& gq) {
    l += io_dl; gq += io_dg;
    if (gq >= ngrp) { gq -= ngrp; ++l; }
  };
  auto bf_lo = [](uint32_t w) { return __uint_as_float(w << 16); };
  auto bf_hi = [](uint32_t w) { return __uint_as_float(w & 0xffff0000u); };
  const float dscalar = (a.has_D && !a.D_has_hdim) ? __ldg(a.D + h) : 0.f;
  float dDacc = 0.f;                                     // sum of dy * x over this thread's elements
  // dy = dout * z sigmoid(z) as the MMAs see it (rounded to bf16), for one group of 4
  auto gate_dy = [&](uint2 gv, uint2 zv, float* dy) {
    dy[0] = bf_lo(gv.x); dy[1] = bf_hi(gv.x); dy[2] = bf_lo(gv.y); dy[3] = bf_hi(gv.y);
    if (zp) {
      const float zf[4] = {bf_lo(zv.x), bf_hi(zv.x), bf_lo(zv.y), bf_hi(zv.y)};
#pragma unroll
      for (int q = 0; q < 4; ++q) dy[q] *= __fdividef(zf[q], 1.f + ex2f(-zf[q] * LOG2E));
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) dy[q] = __bfloat162float(__float2bfloat16_rn(dy[q]));
  };
  // Rows of a finished block: dx = accumulator tile + D dy and dz = dout * y * sigmoid(z)(1 + z(1 - sigmoid(z)))
  // (issm_chunk_scan.py:351-360).  The [64][P / 4] groups of the tile are dealt out one per thread: groups 0..511 to
  // the column threads (which do them while the second MMA phase of the next block runs and they would otherwise
  // wait), the rest to the I/O threads.  `group_load` issues the loads of dout, z and the saved pre-gate output,
  // `group_store` combines them with the dx row in shared memory and stores.
  struct RowGroup { uint2 gv, zv, yv; int l, gq; };
  auto group_load = [&](int t_row0, int t_rows, int gi) {
    RowGroup g;
    g.l = gi / ngrp;
    g.gq = gi - g.l * ngrp;
    const int64_t mr = trow(a, t_row0 + min(g.l, t_rows - 1));
    g.gv = *(const uint2*)(gp + mr * a.g_sl + g.gq * 4);
    g.zv = zp ? *(const uint2*)(zp + mr * a.z_sl + g.gq * 4) : make_uint2(0, 0);
    g.yv = zp ? *(const uint2*)(yp + mr * a.o_sl + g.gq * 4) : make_uint2(0, 0);
    return g;
  };
  auto group_store = [&](const RowGroup& g, int t_row0, int t_rows) {
    const int l = g.l, gq = g.gq;
    if (l >= t_rows) return;
    const uint2 tv = *(const uint2*)(smem + SM::kDxT + (l * SM::DXS + gq * 4) * 2);
    if (a.dxpart) {                                        // one slice of the states: D dy and dz come after the sum over the slices
      *(uint2*)(a.dxpart + ((((size_t)blockIdx.x * a.b + b) * a.L + trow(a, t_row0 + l)) * a.H + h) * a.P + gq * 4) = tv;
      return;
    }
    float v[4] = {bf_lo(tv.x), bf_hi(tv.x), bf_lo(tv.y), bf_hi(tv.y)};
    float dy[4] = {bf_lo(g.gv.x), bf_hi(g.gv.x), bf_lo(g.gv.y), bf_hi(g.gv.y)};
    const size_t o = (((size_t)b * a.L + trow(a, t_row0 + l)) * a.H + h) * a.P + gq * 4;
    if (zp) {
      const float zf[4] = {bf_lo(g.zv.x), bf_hi(g.zv.x), bf_lo(g.zv.y), bf_hi(g.zv.y)};
      const float yf[4] = {bf_lo(g.yv.x), bf_hi(g.yv.x), bf_lo(g.yv.y), bf_hi(g.yv.y)};
      float dzv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float sg = __fdividef(1.f, 1.f + ex2f(-zf[q] * LOG2E));
        dzv[q] = dy[q] * yf[q] * sg * (1.f + zf[q] * (1.f - sg));
        dy[q] *= zf[q] * sg;
      }
      *(uint2*)(a.dz + o) = make_uint2(pack_bf16(dzv[0], dzv[1]), pack_bf16(dzv[2], dzv[3]));
    }
    if (a.has_D) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        v[q] = fmaf(a.D_has_hdim ? __ldg(a.D + h * a.P + gq * 4 + q) : dscalar, __bfloat162float(__float2bfloat16_rn(dy[q])), v[q]);
    }
    *(uint2*)(a.dx + o) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  };
  constexpr int kColGroups = 512;                        // groups of a tile handled by the column threads
  constexpr int kColR = kColGroups / NTH;                // ... per column thread
  constexpr int kIoR = (QB * (PP / 4) - kColGroups + NIO - 1) / NIO;   // per I/O thread
  auto finish_rows_io = [&](int t_row0, int t_rows) {    // the I/O threads' share, loads first
    RowGroup g[kIoR];
#pragma unroll
    for (int r = 0; r < kIoR; ++r) g[r] = group_load(t_row0, t_rows, kColGroups + io_t + r * NIO);
#pragma unroll
    for (int r = 0; r < kIoR; ++r) group_store(g[r], t_row0, t_rows);
  };
  auto finish_rows = [&](int t_row0, int t_rows) {       // a whole tile at once (after the walk)
    if (is_col) {
#pragma unroll
      for (int r = 0; r < kColR; ++r) group_store(group_load(t_row0, t_rows, tid + r * NTH), t_row0, t_rows);
    } else if (is_io) {
      finish_rows_io(t_row0, t_rows);
    }
  };

  // descriptor bases
  const uint32_t sb = smem_u32(smem);
  const uint64_t dK = desc_sw128(sb);
  const uint64_t dMN = desc_sw128_mn(sb, QB * 128);
  const uint64_t dIL = desc_interleave(sb, NT * 16, 128);

  float dAacc = 0.f, dbacc = 0.f;
  bool failed = false;
  uint32_t unsafe = 0, windowed = 0;

  // The three roles run their own loop over the blocks (so that the registers of one role's state are not held
  // through the code of the others); they meet at the two block-wide barriers of every iteration.
  if (is_io) {
    // ================================================ tile-I/O warps ================================================
    for (int it = 0; it < nblk; ++it) {
      const int blk = nblk - 1 - it;
      const int row0 = blk * QB;
      const int rows = min(QB, a.L - row0);
      const uint32_t parity = it & 1;
      // ---- x / dy tiles and dD partials of this block; the tiles are free once the MMAs of the
      //      previous block have completed -------------------------------------------------------------------------
      if (it > 0 && !mbar_wait_warp(kWin ? barX : bar2b, parity ^ 1)) failed = true;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {                     // two passes of XG / 2 groups: 3 loads per group in flight
        uint2 xv[XG / 2], gv[XG / 2], zv[XG / 2];
        int l = io_l0, gq = io_g0;
        for (int k = 0; k < hf * (XG / 2); ++k) io_next(l, gq);
        int lc = l, gc = gq;
#pragma unroll
        for (int k = 0; k < XG / 2; ++k) {
          const int64_t mr = trow(a, row0 + min(lc, rows - 1));
          xv[k] = *(const uint2*)(xp + mr * a.x_sl + gc * 4);
          gv[k] = *(const uint2*)(gp + mr * a.g_sl + gc * 4);
          zv[k] = zp ? *(const uint2*)(zp + mr * a.z_sl + gc * 4) : make_uint2(0, 0);
          io_next(lc, gc);
        }
#pragma unroll
        for (int k = 0; k < XG / 2; ++k) {
          if (l < QB) {
            const bool valid = l < rows;
            float dy[4];
            gate_dy(gv[k], zv[k], dy);
            const uint2 xs = valid ? xv[k] : make_uint2(0, 0);
            const float xf[4] = {bf_lo(xs.x), bf_hi(xs.x), bf_lo(xs.y), bf_hi(xs.y)};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (!valid) dy[q] = 0.f;
              dDacc = fmaf(dy[q], xf[q], dDacc);
            }
            *(uint2*)(smem + SM::kX + sw128_off(l, gq * 4)) = xs;
            *(uint2*)(smem + SM::kDy + sw128_off(l, gq * 4)) = make_uint2(pack_bf16(dy[0], dy[1]), pack_bf16(dy[2], dy[3]));
          }
          io_next(l, gq);
        }
      }
      fence_async_smem();
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      // dx / dz rows of the previous block beyond the column threads' share; named barrier 9 keeps the dx tile
      // from being rewritten before every thread has read its part
      if (it > 0) finish_rows_io(row0 + QB, min(QB, a.L - row0 - QB));
      asm volatile("bar.arrive 9, %0;" ::"r"(NTH + NIO) : "memory");
      fence_before_sync();
    }
  } else if (is_svc) {
    // ================================================= service warp =================================================
    uint32_t c2 = 0;                                     // completions so far of bar2 / bar2b (windowed kernel)
    for (int it = 0; it < nblk; ++it) {
      const int blk = nblk - 1 - it;
      const int row0 = blk * QB;
      const int rows = min(QB, a.L - row0);
      const uint32_t parity = it & 1;
      // ---- service warp (one lane): MMA phase 1: dM = dy x^T, M = Cd Bd^T ---------------------------------------
      auto issue_phase1 = [&]() {
#pragma unroll
        for (int kk = 0; kk < PP / 16; ++kk)
          mma_bf16_off(t_dM, dK, SM::kDy + kk * 32, dK, SM::kX + kk * 32, idesc_bf16(64, 64), kk != 0);
#pragma unroll
        for (int at = 0; at < NT / 64; ++at)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_bf16_off(t_M, dK, SM::kCd + at * (QB * 128) + kk * 32, dK, SM::kBd + at * (QB * 128) + kk * 32,
                         idesc_bf16(64, 64), (at | kk) != 0);
        mma_commit(bar1);
      };
      // ---- service warp (one lane): MMA phase 2: BD^T, CD^T (what the (row, state) epilogue waits for), then G, dx ----
      auto issue_phase2 = [&](bool last) {
#pragma unroll
        for (int sl = 0; sl < NT / 128; ++sl) {
          const uint32_t dBD = tmem + 128 + sl * 64, dCD = tmem + 256 + sl * 64;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {                 // K = rows of the block
            const uint32_t oCd = SM::kCd + sl * (2 * QB * 128) + kk * 2048, oBd = SM::kBd + sl * (2 * QB * 128) + kk * 2048;
            mma_bf16_off(dBD, dMN, oCd, dMN, SM::kDMm + kk * 2048, idesc_bf16(128, 64, 1, 1), kk != 0);
            mma_bf16_off(dCD, dMN, oBd, dK, SM::kDMm + kk * 32, idesc_bf16(128, 64, 1, 0), kk != 0);
          }
#pragma unroll
          for (int kk = 0; kk < PP / 16; ++kk) {           // K = head dim
            mma_bf16_off(dBD, dK, SM::kGop + sl * (128 * 128) + kk * 32, dK, SM::kX + kk * 32, idesc_bf16(128, 64), 1);
            mma_bf16_off(dCD, dIL, SM::kSop + sl * (128 * 16) + kk * 2 * (NT * 16), dK, SM::kDy + kk * 32, idesc_bf16(128, 64), 1);
          }
        }
        mma_commit(bar2);
#pragma unroll
        for (int sl = 0; sl < NT / 128; ++sl)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)                   // G += Cd^T dy
            mma_bf16_off(tmem + 384 + sl * PP, dMN, SM::kCd + sl * (2 * QB * 128) + kk * 2048, dMN, SM::kDy + kk * 2048,
                         idesc_bf16(128, PP, 1, 1), 1);
#pragma unroll
        for (int at = 0; at < NT / 64; ++at)               // dx: K = states
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_bf16_off(t_dx, dK, SM::kBd + at * (QB * 128) + kk * 32, dMN, SM::kGop + (at * 4 + kk) * 2048,
                         idesc_bf16(64, PP, 0, 1), (at | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                     // dx: K = later rows
          mma_bf16_off(t_dx, dMN, SM::kMm + kk * 2048, dMN, SM::kDy + kk * 2048, idesc_bf16(64, PP, 1, 1), 1);
        mma_commit(bar2b);
        if (kWin && last) mma_commit(barX);
      };

      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      // windowed kernel: has some column asked for this block to be cut into 2^kw windows?
      int kw = 0;
      if (kWin) {
        const uint32_t flag = *sFlag;
        if ((flag >> 3) == (uint32_t)(it + 1)) kw = (int)(flag & 7);
      }
      const int ws = QB >> kw;
      const int npass = kw ? (rows + ws - 1) / ws : 1;
      if (kw == 0) {
        if (lane == 0) {
          fence_after_sync();
          issue_phase1();
        }
        __syncwarp();
        prefetch_S(blk);                                   // every column thread has read the previous content of the S tile
      }
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      if (kw == 0) {
        if (lane == 0) {
          fence_after_sync();
          if (!mbar_wait(barU, parity ^ 1)) { if (a.status) atomicOr(a.status, 1); }   // S tile of this block has landed
          issue_phase2(true);
        }
        __syncwarp();
        if (blk > 0) {                                     // B staging is free once every column thread has
          named_barrier(10, NTH + 32);                     // finished its (row, state) epilogue; the C rows take the
          prefetch_B(blk - 1);                             // place of the g' tile, which the dx MMAs read
          prefetch_dt(blk - 1);
          if (lane == 0 && !mbar_wait(bar2b, kWin ? (c2 & 1) : parity)) { if (a.status) atomicOr(a.status, 1); }
          __syncwarp();
          prefetch_C(blk - 1);
        }
      } else if (kWin) {
        // windowed block: MMAs of the window-entry-state walk, then of every pass (named barriers 11 / 12 / 13)
        for (int w = 0; w + 1 < npass; ++w) {              // walk producing the window-entry states
          named_barrier(11, NTH + 32);
          if (lane == 0) {
            fence_after_sync();
#pragma unroll
            for (int sl = 0; sl < NT / 128; ++sl)
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                mma_bf16_off(tmem + 128 + sl * 64, dMN, SM::kBd + sl * (2 * QB * 128) + kk * 2048, dMN, SM::kX + kk * 2048,
                             idesc_bf16(128, PP, 1, 1), 1);
            mma_commit(barW);
          }
          __syncwarp();
          named_barrier(12, NTH + 32);
        }
        for (int w = npass - 1; w >= 0; --w) {
          named_barrier(11, NTH + 32);
          if (lane == 0) { fence_after_sync(); issue_phase1(); }
          __syncwarp();
          named_barrier(12, NTH + 32);
          if (lane == 0) { fence_after_sync(); issue_phase2(w == 0); }
          __syncwarp();
          named_barrier(13, NTH + 32);
        }
        prefetch_S(blk);                                   // leaves the S tile as the next iteration expects it
        if (blk > 0) {
          named_barrier(10, NTH + 32);
          prefetch_B(blk - 1);
          prefetch_C(blk - 1);
          prefetch_dt(blk - 1);
        }
      }
      if (kWin) c2 += npass;
      fence_before_sync();
    }
  } else {
    // ================================================ column threads ================================================
    uint32_t c1 = 0, c2 = 0, cw = 0;                     // completions so far of bar1 / bar2 / barW (windowed kernel)
    for (int it = 0; it < nblk; ++it) {
      const int blk = nblk - 1 - it;
      const int row0 = blk * QB;
      const int rows = min(QB, a.L - row0);
      const uint32_t parity = it & 1;
      float a0 = 0.f, alast = 0.f, cst = 0.f, cpart_own = 0.f;

      // ---- column threads: operand pass restricted to rows [w0, w1) of the block.  `first` is the ordinary pass over
      //      the whole block (staged C, range check, waits for the staged tiles); later passes (windowed kernel only)
      //      rebuild the operands for one window: C comes from global memory because the g' operand has taken the place
      //      of the staged C rows, and the exponent is kept within +-100 (this only binds for single-row windows).
      //      Sets a0 (sum of dt*A over the first half's rows), alast (over all rows) and cst (sum of both cpart). -------
      auto phaseAB = [&](int w0, int w1, bool first, float cpart) {
        // Staged tiles are addressed as base + l * step in units of rows: a tile that was copied in memory
        // order for a reversed scan is walked backwards.  Full blocks run a guard-free instantiation.
        const bool flipT = kMode ? kMode == 2 : (a.dt_tma && a.rev);
        const bf16* sdt = (const bf16*)(smem + SM::kSdt) + n + (flipT ? (rows - 1) * NT : 0);
        const int dstep = flipT ? -NT : NT;
        const bf16* sB = (const bf16*)(smem + SM::kSB) + n + (flipB ? (rows - 1) * NT : 0);
        const bf16* sC = (const bf16*)(smem + SM::kSC) + n + (flipB ? (rows - 1) * NT : 0);
        const int bstep = flipB ? -NT : NT;

        // ---- phase A: dt of this thread's 32 rows and their summed log2-decay.  The loops over the rows run as
        //      4 iterations of 8 unrolled rows (a quarter of the instruction footprint of full unrolling, which
        //      measurably stalled instruction fetch); the dt values wait for phase B in this thread's own 32
        //      columns of the CD^T accumulator, which is not live before the second MMA phase ---------------------
        float asum = 0.f;
        auto phaseA = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            float dv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int l = half * 32 + ch * 8 + j;
              float raw;
              if (kStageDt) raw = __bfloat162float(sdt[(kFull ? l : min(l, rows - 1)) * dstep]);
              else raw = ldf(dtp + (int64_t)trow(a, row0 + (kFull ? l : min(l, rows - 1))) * a.dt_sl + n);
              bool clamped = false;
              float v = dt_transform(a, raw, bias, clamped);
              if (!kFull && (l < w0 || l >= w1)) v = 0.f;
              dv[j] = v;
              asum = fmaf(v, A2, asum);
            }
            tmem_st8(t_CD + ch * 8, dv);
          }
        };
        if (first && rows == QB) phaseA(std::true_type{}); else phaseA(std::false_type{});
        sXch[half * NT + n] = asum;
        sXch[(2 + half) * NT + n] = cpart;
        named_barrier(1 + (warp & (NT / 32 - 1)), 64);
        a0 = sXch[n];
        alast = a0 + sXch[NT + n];
        cst = sXch[2 * NT + n] + sXch[3 * NT + n];
        if (first) {
          // range of the factorisation: 2^(+-a) must stay finite in bf16 (see the forward kernel)
          if (!(fabsf(a0) <= 120.f && fabsf(alast) <= 120.f)) {
            if (kWin) atomicMax(sFlag, (uint32_t)(it + 1) * 8 + window_need<TDT>(a, sdt, dstep, dtp, row0, rows, half, n, A2, bias));
            else unsafe = 1;
          }
          if (!mbar_wait_warp(barT, parity)) failed = true;
          if (!mbar_wait_warp(barV, parity)) failed = true;
        }
        // ---- phase B: this thread's rows of Cd = C 2^a and Bd = B dt 2^-a ------------------------------------
        auto phaseB = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
          uint8_t* cd_col = smem + SM::kCd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
          uint8_t* bd_col = smem + SM::kBd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
          const int kc = kcol >> 3;
          float acc = half ? a0 : 0.f;
          tmem_st_wait();
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            float dv[8];
            tmem_ld8(t_CD + ch * 8, dv);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int l = half * 32 + ch * 8 + j;
              const int sl = kFull ? l : min(l, rows - 1);
              acc = fmaf(dv[j], A2, acc);
              const float e = (kWin && !first) ? fminf(fmaxf(acc, -100.f), 100.f) : acc;
              float cv;
              if (kWin && !first) cv = __bfloat162float(Cp[(int64_t)trow(a, row0 + sl) * a.C_sl + n]);
              else cv = __bfloat162float(sC[sl * bstep]);
              float cd = cv * ex2f(e);
              float bd = __bfloat162float(sB[sl * bstep]) * dv[j] * ex2f(-e);
              if (!kFull && (l < w0 || l >= w1)) { cd = 0.f; bd = 0.f; }
              const uint32_t off = (uint32_t)((ch * 8 + j) * 128 + ((kc ^ j) << 4));
              *(bf16*)(cd_col + off) = __float2bfloat16_rn(cd);
              *(bf16*)(bd_col + off) = __float2bfloat16_rn(bd);
            }
          }
        };
        if (first && rows == QB) phaseB(std::true_type{}); else phaseB(std::false_type{});
        fence_async_smem();
      };

      // ---- fast instantiation: the operand pass with two adjacent states (2 pr, 2 pr + 1) and the 16 rows of quarter
      //      qr per thread: every shared-memory access moves a bf16 pair and the fp32 arithmetic runs as packed pairs.
      //      The quarter sums of dt*A go through sXch ([4][NT]); a0 / alast of the thread's own column n are read from
      //      there after the next block-wide barrier (column n belongs to another group of warps than the pair). -------
      auto phaseAB_pairs = [&]() {
        constexpr int NPR = NT / 2;
        const int pr = tid % NPR, qr = tid / NPR;
        const bool flipT = kMode ? kMode == 2 : (a.dt_tma && a.rev);
        const uint32_t* sdt2 = (const uint32_t*)(smem + SM::kSdt) + pr + (flipT ? (rows - 1) * NPR : 0);
        const int dstep2 = flipT ? -NPR : NPR;
        const uint32_t* sB2 = (const uint32_t*)(smem + SM::kSB) + pr + (flipB ? (rows - 1) * NPR : 0);
        const uint32_t* sC2 = (const uint32_t*)(smem + SM::kSC) + pr + (flipB ? (rows - 1) * NPR : 0);
        const int bstep2 = flipB ? -NPR : NPR;
        float2 dtv[16];
        float2 asum2 = f2(0.f);
        auto phaseA2 = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int l = qr * 16 + j;
            const int sl = kFull ? l : min(l, rows - 1);
            float2 raw;
            if constexpr (kStageDt) raw = unpack_bf16(sdt2[sl * dstep2]);
            else raw = *(const float2*)((const float*)dtp + (int64_t)trow(a, row0 + sl) * a.dt_sl + 2 * pr);
            float2 v = dt_transform2(a, raw, biasL2);
            if (!kFull && l >= rows) v = f2(0.f);
            dtv[j] = v;
            asum2 = __ffma2_rn(v, A2p, asum2);
          }
        };
        if (rows == QB) phaseA2(std::true_type{}); else phaseA2(std::false_type{});
        *(float2*)(sXch + qr * NT + 2 * pr) = asum2;
        named_barrier(1 + (warp % (NPR / 32)), 128);       // the four warps that share these 64 columns
        const float2 q0 = *(const float2*)(sXch + 2 * pr), q1 = *(const float2*)(sXch + NT + 2 * pr),
                     q2 = *(const float2*)(sXch + 2 * NT + 2 * pr), q3 = *(const float2*)(sXch + 3 * NT + 2 * pr);
        const float2 c1 = q0, c2 = __fadd2_rn(c1, q1), c3 = __fadd2_rn(c2, q2), c4 = __fadd2_rn(c3, q3);
        // range of the factorisation: 2^(+-a) must stay finite in bf16 (see the forward kernel)
        const float worst = fmaxf(fmaxf(fmaxf(fabsf(c1.x), fabsf(c1.y)), fmaxf(fabsf(c2.x), fabsf(c2.y))),
                                  fmaxf(fmaxf(fabsf(c3.x), fabsf(c3.y)), fmaxf(fabsf(c4.x), fabsf(c4.y))));
        if (!(worst <= 120.f)) unsafe = 1;
        if (!mbar_wait_warp(barT, parity)) failed = true;
        if (!mbar_wait_warp(barV, parity)) failed = true;
        auto phaseB2 = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
          const int at = pr >> 5, kc = (pr & 31) >> 2;     // 64-state atom, 16-byte chunk inside its 128-byte rows
          uint8_t* cd_col = smem + SM::kCd + at * (QB * 128) + qr * (16 * 128) + ((pr & 3) << 2);
          uint8_t* bd_col = smem + SM::kBd + at * (QB * 128) + qr * (16 * 128) + ((pr & 3) << 2);
          float2 acc = qr == 0 ? f2(0.f) : (qr == 1 ? c1 : (qr == 2 ? c2 : c3));
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int l = qr * 16 + j;
            const int sl = kFull ? l : min(l, rows - 1);
            acc = __ffma2_rn(dtv[j], A2p, acc);
            float2 cd = __fmul2_rn(unpack_bf16(sC2[sl * bstep2]), ex2f2(acc));
            float2 bd = __fmul2_rn(__fmul2_rn(unpack_bf16(sB2[sl * bstep2]), dtv[j]), ex2f2_neg(acc));
            if (!kFull && l >= rows) { cd = f2(0.f); bd = f2(0.f); }
            const uint32_t off = (uint32_t)(j * 128 + ((kc ^ (j & 7)) << 4));
            *(uint32_t*)(cd_col + off) = pack_bf16(cd);
            *(uint32_t*)(bd_col + off) = pack_bf16(bd);
          }
        };
        if (rows == QB) phaseB2(std::true_type{}); else phaseB2(std::false_type{});
        fence_async_smem();
      };

      // ---- column threads: g' = 2^(a_last) G: back into TMEM for the accumulate MMA, bf16 copy as operand row -------
      auto gprime = [&]() {
        float gc[HP];
        tmem_ld16(t_G, gc);
        tmem_ld8(t_G + 16, gc + 16);
        tmem_ld_wait();
        const float eg = ex2f(alast);
#pragma unroll
        for (int j = 0; j < HP; ++j) gc[j] *= eg;
        tmem_st16(t_G, gc);
        tmem_st8(t_G + 16, gc + 16);
#pragma unroll
        for (int c = 0; c < HP / 8; ++c)
          *(uint4*)(smem + SM::kGop + sw128_chunk(n, half * (HP / 8) + c)) =
              make_uint4(pack_bf16(gc[c * 8], gc[c * 8 + 1]), pack_bf16(gc[c * 8 + 2], gc[c * 8 + 3]),
                         pack_bf16(gc[c * 8 + 4], gc[c * 8 + 5]), pack_bf16(gc[c * 8 + 6], gc[c * 8 + 7]));
        tmem_st_wait();
      };

      // ---- column threads, epilogue 1: causal masks, bf16 operands dMm[l][s] (first half of the warps) and Mm[l][s] ----
      auto epilogue1 = [&]() {
        const int l = (warp & 3) * 16 + lane;
        const uint32_t t0 = (half ? t_M : t_dM) + lane_base;
        uint8_t* dst = smem + (half ? SM::kMm : SM::kDMm);
        for (int c16 = (warp >> 2) % (NCG / 2 > 0 ? NCG / 2 : 1); c16 < 4; c16 += (NCG / 2 > 0 ? NCG / 2 : 1)) {
          float mv[16];
          tmem_ld16(t0 + c16 * 16, mv);
          tmem_ld_wait();
          if (lane < 16) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              uint32_t pk[4];
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const int s = c16 * 16 + c * 8 + j;
                pk[j >> 1] = pack_bf16(s <= l ? mv[c * 8 + j] : 0.f, s + 1 <= l ? mv[c * 8 + j + 1] : 0.f);
              }
              *(uint4*)(dst + sw128_chunk(l, c16 * 2 + c)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
      };

      // ---- column threads, epilogue (a): the owner of (rows 32 half.., state n): dB_h, dC_h, ddt and the reverse
      //      cumsum of dacs, for the rows [w0, w1) of the block ------------------------------------------------------
      auto epilogue_a = [&](int w0, int w1, bool first) {
        const bool flipT = kMode ? kMode == 2 : (a.dt_tma && a.rev);
        const bf16* sdt = (const bf16*)(smem + SM::kSdt) + n + (flipT ? (rows - 1) * NT : 0);
        const int dstep = flipT ? -NT : NT;
        const bf16* sB = (const bf16*)(smem + SM::kSB) + n + (flipB ? (rows - 1) * NT : 0);
        const int bstep = flipB ? -NT : NT;
        const uint8_t* cd_col = smem + SM::kCd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
        const uint8_t* bd_col = smem + SM::kBd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
        const int kc = kcol >> 3;
        float part = 0.f;                                  // sum over this thread's rows of dacs = Cd CD - Bd BD
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          float bdv[8], cdv[8];
          tmem_ld8(t_BD + ch * 8, bdv);
          tmem_ld8(t_CD + ch * 8, cdv);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t off = (uint32_t)((ch * 8 + j) * 128 + ((kc ^ j) << 4));
            part = fmaf(__bfloat162float(*(const bf16*)(cd_col + off)), cdv[j], part);
            part = fmaf(-__bfloat162float(*(const bf16*)(bd_col + off)), bdv[j], part);
          }
        }
        sXch[half * NT + n] = part;
        if constexpr (!kWin) sXch[(2 + half) * NT + n] = cpart_own;
        named_barrier(1 + (warp & (NT / 32 - 1)), 64);
        const float p0 = sXch[n];
        const float total = p0 + sXch[NT + n];
        if constexpr (!kWin) cst = sXch[2 * NT + n] + sXch[3 * NT + n];   // <S leaving the block, G> of column n
        // output element of row l: index o0 + l * ostep (rows of a reversed scan go down in memory)
        const int ostep = (a.rev ? -1 : 1) * a.H * a.N;
        const int64_t o0 = (((int64_t)b * a.L + trow(a, row0)) * a.H + h) * a.N + ng;
        TDT* const p_ddt = (TDT*)a.ddt + o0;
        uint32_t* const p_dBC = a.dBCh + o0;
        auto epi = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
          float prefix = half ? p0 : 0.f;
          float ac = half ? a0 : 0.f;
#pragma unroll 2
          for (int ch = 0; ch < 4; ++ch) {
            float bdv[8], cdv[8];
            tmem_ld8(t_BD + ch * 8, bdv);
            tmem_ld8(t_CD + ch * 8, cdv);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int l = half * 32 + ch * 8 + j;
              const int sl = kFull ? l : min(l, rows - 1);
              const bool in = kFull || (l >= w0 && l < w1);
              float raw;
              if (kStageDt) raw = __bfloat162float(sdt[sl * dstep]);
              else raw = ldf(dtp + (int64_t)trow(a, row0 + sl) * a.dt_sl + n);
              bool clamped = false;
              float dtl = dt_transform(a, raw, bias, clamped);
              if (!in) dtl = 0.f;
              ac = fmaf(dtl, A2, ac);
              const float e = (kWin && !first) ? fminf(fmaxf(ac, -100.f), 100.f) : ac;
              const float bd = ex2f(-e) * bdv[j], cd = ex2f(e) * cdv[j];
              const uint32_t off = (uint32_t)((ch * 8 + j) * 128 + ((kc ^ j) << 4));
              const float dacs = __bfloat162float(*(const bf16*)(cd_col + off)) * cdv[j] -
                                 __bfloat162float(*(const bf16*)(bd_col + off)) * bdv[j];
              const float ddA = cst + total - prefix;        // sum of dacs over rows >= l, plus <S_next, G>
              prefix += dacs;
              float gd = fmaf(ddA, Anat, __bfloat162float(sB[sl * bstep]) * bd);
              if (clamped) gd = 0.f;
              else if (a.softplus) gd *= 1.f - ex2f(-dtl * LOG2E);
              if (in) {
                dAacc = fmaf(ddA, dtl, dAacc);
                dbacc += gd;
                const int o = l * ostep;
                stf(p_ddt + o, gd);
                p_dBC[o] = pack_bf16(dtl * bd, cd);                 // one store for the pair {dB_h, dC_h}
              }
            }
          }
        };
        if (first && rows == QB) epi(std::true_type{}); else epi(std::false_type{});
      };

      // ---- fast instantiation: the same (row, state) epilogue over the whole block with the rows taken two at a time,
      //      so that the fp32 arithmetic runs as packed pairs (the running sums along the rows stay scalar) -------------
      auto epilogue_a_pairs = [&]() {
        const bool flipT = kMode ? kMode == 2 : (a.dt_tma && a.rev);
        const bf16* sdt = (const bf16*)(smem + SM::kSdt) + n + (flipT ? (rows - 1) * NT : 0);
        const int dstep = flipT ? -NT : NT;
        const bf16* sB = (const bf16*)(smem + SM::kSB) + n + (flipB ? (rows - 1) * NT : 0);
        const int bstep = flipB ? -NT : NT;
        const uint8_t* cd_col = smem + SM::kCd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
        const uint8_t* bd_col = smem + SM::kBd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
        const int kc = kcol >> 3;
        auto opnd = [&](const uint8_t* col, int r) {      // rows r, r + 1 of this thread's column of an operand tile
          return f2(__bfloat162float(*(const bf16*)(col + (uint32_t)(r * 128 + ((kc ^ (r & 7)) << 4)))),
                    __bfloat162float(*(const bf16*)(col + (uint32_t)((r + 1) * 128 + ((kc ^ ((r + 1) & 7)) << 4)))));
        };
        float2 part2 = f2(0.f);                            // sum over this thread's rows of dacs = Cd CD - Bd BD
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          float bdv[8], cdv[8];
          tmem_ld8(t_BD + ch * 8, bdv);
          tmem_ld8(t_CD + ch * 8, cdv);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            part2 = __ffma2_rn(opnd(cd_col, ch * 8 + j), f2(cdv[j], cdv[j + 1]), part2);
            part2 = __ffma2_rn(opnd(bd_col, ch * 8 + j), f2(-bdv[j], -bdv[j + 1]), part2);
          }
        }
        sXch[half * NT + n] = part2.x + part2.y;
        sXch[(2 + half) * NT + n] = cpart_own;
        named_barrier(1 + (warp & (NT / 32 - 1)), 64);
        const float p0 = sXch[n];
        const float total = p0 + sXch[NT + n];
        cst = sXch[2 * NT + n] + sXch[3 * NT + n];         // <S leaving the block, G> of column n
        const float base = cst + total;                    // ddA[l] = base - sum of dacs over the rows before l
        const int ostep = (a.rev ? -1 : 1) * a.H * a.N;
        const int64_t o0 = (((int64_t)b * a.L + trow(a, row0)) * a.H + h) * a.N + ng;
        TDT* const p_ddt = (TDT*)a.ddt + o0;
        uint32_t* const p_dBC = a.dBCh + o0;
        const float biasL = bias * (a.softplus ? LOG2E : 1.f);
        auto epi = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
          float prefix = half ? p0 : 0.f;
          float ac = half ? a0 : 0.f;
          float2 dA2 = f2(0.f), db2 = f2(0.f);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float bdv[8], cdv[8];
            tmem_ld8(t_BD + ch * 8, bdv);
            tmem_ld8(t_CD + ch * 8, cdv);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const int l = half * 32 + ch * 8 + j;
              const int s0 = kFull ? l : min(l, rows - 1), s1 = kFull ? l + 1 : min(l + 1, rows - 1);
              const bool in0 = kFull || l < rows, in1 = kFull || l + 1 < rows;
              float2 raw;
              if (kStageDt) raw = f2(__bfloat162float(sdt[s0 * dstep]), __bfloat162float(sdt[s1 * dstep]));
              else raw = f2(ldf(dtp + (int64_t)trow(a, row0 + s0) * a.dt_sl + n), ldf(dtp + (int64_t)trow(a, row0 + s1) * a.dt_sl + n));
              // dt transform (see dt_transform2) keeping the unclamped value: no gradient flows through a clamped dt
              float2 v;
              if (a.softplus) {
                const float2 t = __ffma2_rn(raw, f2(LOG2E), f2(biasL));
                float2 sp = lg2f2(__fadd2_rn(ex2f2(t), f2(1.f)));
                sp.x = t.x <= 20.f * LOG2E ? sp.x : t.x;
                sp.y = t.y <= 20.f * LOG2E ? sp.y : t.y;
                v = __fmul2_rn(sp, f2(LN2));
              } else {
                v = __fadd2_rn(raw, f2(biasL));
              }
              float2 dtl = f2(fminf(fmaxf(v.x, a.dtmin), a.dtmax), fminf(fmaxf(v.y, a.dtmin), a.dtmax));
              const bool cl0 = dtl.x != v.x, cl1 = dtl.y != v.y;
              if (!in0) dtl.x = 0.f;
              if (!in1) dtl.y = 0.f;
              const float ac0 = fmaf(dtl.x, A2, ac);
              ac = fmaf(dtl.y, A2, ac0);
              const float2 e = f2(ac0, ac);
              const float2 bdv2 = f2(bdv[j], bdv[j + 1]), cdv2 = f2(cdv[j], cdv[j + 1]);
              const float2 bd = __fmul2_rn(ex2f2_neg(e), bdv2), cd = __fmul2_rn(ex2f2(e), cdv2);
              const float2 tb = __fmul2_rn(opnd(bd_col, ch * 8 + j), bdv2);
              const float2 co = opnd(cd_col, ch * 8 + j);
              const float dacs0 = fmaf(co.x, cdv2.x, -tb.x), dacs1 = fmaf(co.y, cdv2.y, -tb.y);
              const float ddA0 = base - prefix;              // sum of dacs over rows >= l, plus <S_next, G>
              prefix += dacs0;
              const float ddA1 = base - prefix;
              prefix += dacs1;
              const float2 ddA = f2(ddA0, ddA1);
              const float2 Bv = f2(__bfloat162float(sB[s0 * bstep]), __bfloat162float(sB[s1 * bstep]));
              float2 gd = __ffma2_rn(ddA, f2(Anat), __fmul2_rn(Bv, bd));
              if (a.softplus) gd = __fmul2_rn(gd, __ffma2_rn(ex2f2(__fmul2_rn(dtl, f2(-LOG2E))), f2(-1.f), f2(1.f)));
              if (cl0) gd.x = 0.f;
              if (cl1) gd.y = 0.f;
              const float2 dBh = __fmul2_rn(dtl, bd);
              if (kFull) {
                dA2 = __ffma2_rn(ddA, dtl, dA2);
                db2 = __fadd2_rn(db2, gd);
              } else {
                if (in0) { dA2.x = fmaf(ddA0, dtl.x, dA2.x); db2.x += gd.x; }
                if (in1) { dA2.y = fmaf(ddA1, dtl.y, dA2.y); db2.y += gd.y; }
              }
              const int o = l * ostep;
              if (in0) { stf(p_ddt + o, gd.x); p_dBC[o] = pack_bf16(dBh.x, cd.x); }               // one store for the pair {dB_h, dC_h}
              if (in1) { stf(p_ddt + o + ostep, gd.y); p_dBC[o + ostep] = pack_bf16(dBh.y, cd.y); }
            }
          }
          dAacc += dA2.x + dA2.y;
          dbacc += db2.x + db2.y;
        };
        if (rows == QB) epi(std::true_type{}); else epi(std::false_type{});
      };

      // ---- column threads, epilogue (b): dx rows -> shared memory (every warp takes 16-column groups of its 16 rows) ----
      auto epilogue_b = [&](int w0, int w1, bool first) {
        const int l = (warp & 3) * 16 + lane;
        for (int c16 = (warp >> 2) % NCG; c16 < PP / 16; c16 += NCG) {
          float dv[16];
          tmem_ld16(t_dx + lane_base + c16 * 16, dv);
          tmem_ld_wait();
          if (lane < 16 && (first || (l >= w0 && l < w1))) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
              if (c16 * 16 + c * 4 < SM::DXS)
                *(uint2*)(smem + SM::kDxT + (l * SM::DXS + c16 * 16 + c * 4) * 2) =
                    make_uint2(pack_bf16(dv[c * 4], dv[c * 4 + 1]), pack_bf16(dv[c * 4 + 2], dv[c * 4 + 3]));
          }
        }
      };

      // ---- <S leaving the block, G> over this thread's state columns: the S operand tile still holds the
      //      state entering the block processed before this one, i.e. the state leaving this block ------------
      float cpart = 0.f;
      {
        float gc[HP];
        tmem_ld16(t_G, gc);
        tmem_ld8(t_G + 16, gc + 16);
        if (!mbar_wait_warp(barU, parity)) failed = true;
        uint4 snv[HP / 8];
#pragma unroll
        for (int c = 0; c < HP / 8; ++c) snv[c] = *(const uint4*)(smem + SM::kSop + (half * (HP / 8) + c) * (NT * 16) + n * 16);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < HP / 8; ++c) {
          const uint32_t w[4] = {snv[c].x, snv[c].y, snv[c].z, snv[c].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            cpart = fmaf(__uint_as_float(w[j] << 16), gc[c * 8 + 2 * j], cpart);
            cpart = fmaf(__uint_as_float(w[j] & 0xffff0000u), gc[c * 8 + 2 * j + 1], cpart);
          }
        }
      }
      if (kStageDt && !mbar_wait_warp(barS, parity)) failed = true;
      if constexpr (kWin) phaseAB(0, rows, true, cpart);
      else phaseAB_pairs();
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      if constexpr (!kWin) {                               // summed decay of this thread's own column n (see phaseAB_pairs)
        a0 = sXch[n] + sXch[NT + n];
        alast = (a0 + sXch[2 * NT + n]) + sXch[3 * NT + n];
        cpart_own = cpart;                                 // joins the other half's part in the epilogue's exchange
      }
      // windowed kernel: has some column asked for this block to be cut into 2^kw windows?
      int kw = 0;
      if (kWin) {
        const uint32_t flag = *sFlag;
        if ((flag >> 3) == (uint32_t)(it + 1)) kw = (int)(flag & 7);
      }
      const int ws = QB >> kw;
      const int npass = kw ? (rows + ws - 1) / ws : 1;
      if (kw == 0) {
        gprime();
        if (!mbar_wait_warp(bar1, kWin ? (c1 & 1) : parity)) failed = true;
        fence_after_sync();
        if (!failed) epilogue1();
        fence_async_smem();
      }
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      // dx / dz rows of the previous block, while the second MMA phase is issued
      if (it > 0) {
#pragma unroll
        for (int r = 0; r < kColR; ++r)
          group_store(group_load(row0 + QB, min(QB, a.L - row0 - QB), tid + r * NTH), row0 + QB, min(QB, a.L - row0 - QB));
      }
      if (kw == 0) {
        if (!mbar_wait_warp(bar2, kWin ? (c2 & 1) : parity)) failed = true;
        fence_after_sync();
        if (!failed) {
          if constexpr (kWin) epilogue_a(0, rows, true);
          else epilogue_a_pairs();
          asm volatile("bar.arrive 10, %0;" ::"r"(NTH + 32) : "memory");      // B staging reads are done
          named_barrier(9, NTH + NIO);                     // the previous block's dx rows have left the tile
          if (!mbar_wait_warp(bar2b, kWin ? (c2 & 1) : parity)) failed = true;
          fence_after_sync();
          epilogue_b(0, rows, true);
        } else {
          asm volatile("bar.arrive 10, %0;" ::"r"(NTH + 32) : "memory");
          named_barrier(9, NTH + NIO);
        }
      } else if (kWin) {
        // windowed block (named barriers 11 / 12 / 13 with the service warp)
      const size_t sblk = (size_t)a.N * PP;                // elements of one saved state
      windowed = 1;
      named_barrier(9, NTH + NIO);                       // the previous block's dx rows have left the tile
      const float cst_block = cst;
      const size_t mine = ((size_t)half * (HP / 8) * a.N + ng) * 8;          // this thread's chunks inside a state
      const bf16* sv0 = a.saved + (bh * (nblk + 1) + blk) * sblk + mine;    // state entering the block
      bf16* wsc = a.wscr + bh * 63 * sblk + mine;                           // slot j: state entering window j + 1
      const uint32_t t_W = tmem + lane_base + 128 + slab * 64 + half * HP;  // accumulator of the walk
      auto unpack = [&](const bf16* src, float* sc) {
#pragma unroll
        for (int c = 0; c < HP / 8; ++c) {
          const uint4 v = *(const uint4*)(src + (size_t)c * a.N * 8);
          const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sc[c * 8 + 2 * j] = __uint_as_float(wd[j] << 16);
            sc[c * 8 + 2 * j + 1] = __uint_as_float(wd[j] & 0xffff0000u);
          }
        }
      };
      {
        float sc[HP];
        unpack(sv0, sc);
        tmem_st16(t_W, sc);
        tmem_st8(t_W + 16, sc + 16);
        tmem_st_wait();
        for (int w = 0; w + 1 < npass; ++w) {
          phaseAB(w * ws, min(rows, w * ws + ws), false, 0.f);
          fence_before_sync();
          named_barrier(11, NTH + 32);
          if (!mbar_wait_warp(barW, cw & 1)) failed = true;
          ++cw;
          fence_after_sync();
          tmem_ld16(t_W, sc);
          tmem_ld8(t_W + 16, sc + 16);
          tmem_ld_wait();
          const float el = ex2f(fminf(fmaxf(alast, -100.f), 100.f));
#pragma unroll
          for (int j = 0; j < HP; ++j) sc[j] *= el;
          tmem_st16(t_W, sc);
          tmem_st8(t_W + 16, sc + 16);
          bf16* dst = wsc + (size_t)w * sblk;
#pragma unroll
          for (int c = 0; c < HP / 8; ++c)
            *(uint4*)(dst + (size_t)c * a.N * 8) = make_uint4(pack_bf16(sc[c * 8], sc[c * 8 + 1]), pack_bf16(sc[c * 8 + 2], sc[c * 8 + 3]),
                                pack_bf16(sc[c * 8 + 4], sc[c * 8 + 5]), pack_bf16(sc[c * 8 + 6], sc[c * 8 + 7]));
          tmem_st_wait();
          fence_before_sync();
          named_barrier(12, NTH + 32);
        }
      }
      for (int w = npass - 1, k = 0; w >= 0; --w, ++k) {
        const int w0 = w * ws, w1 = min(rows, w0 + ws);
        // <state leaving the window, G>: the last window leaves the block (computed above); the others read the walk's copy
        float cpart = half ? 0.f : cst_block;
        if (w < npass - 1) {
          float gc[HP], sn[HP];
          tmem_ld16(t_G, gc);
          tmem_ld8(t_G + 16, gc + 16);
          unpack(wsc + (size_t)w * sblk, sn);
          tmem_ld_wait();
          cpart = 0.f;
#pragma unroll
          for (int j = 0; j < HP; ++j) cpart = fmaf(sn[j], gc[j], cpart);
        }
        {                                                // S operand tile <- state entering the window
          const bf16* src = w ? wsc + (size_t)(w - 1) * sblk : sv0;
#pragma unroll
          for (int c = 0; c < HP / 8; ++c)
            *(uint4*)(smem + SM::kSop + (half * (HP / 8) + c) * (NT * 16) + n * 16) = *(const uint4*)(src + (size_t)c * a.N * 8);
        }
        phaseAB(w0, w1, false, cpart);
        alast = fminf(fmaxf(alast, -100.f), 100.f);
        gprime();
        fence_async_smem();
        fence_before_sync();
        named_barrier(11, NTH + 32);
        if (!mbar_wait_warp(bar1, (c1 + k) & 1)) failed = true;
        fence_after_sync();
        epilogue1();
        fence_async_smem();
        fence_before_sync();
        named_barrier(12, NTH + 32);
        if (!mbar_wait_warp(bar2, (c2 + k) & 1)) failed = true;
        fence_after_sync();
        epilogue_a(w0, w1, false);
        if (!mbar_wait_warp(bar2b, (c2 + k) & 1)) failed = true;
        fence_after_sync();
        epilogue_b(w0, w1, false);
        fence_before_sync();
        named_barrier(13, NTH + 32);
      }
      asm volatile("bar.arrive 10, %0;" ::"r"(NTH + 32) : "memory");
      }
      if (kWin) { c1 += npass; c2 += npass; }
      fence_before_sync();
    }
  }
  const int prev_row0 = 0, prev_rows = min(QB, a.L);     // the block processed last

  // the I/O warps store the dx rows of the last processed block
  // a wait of the last iteration can expire after that iteration's last block-wide vote: make the verdict
  // uniform over the block before the barriers below run under it
  const int votes = __syncthreads_or((int)unsafe | (failed ? 2 : 0));
  const int any_unsafe = votes & 1;
  failed = (votes & 2) != 0;
  if (!kWin && tid == 0) a.redo[stream] = any_unsafe;
  if (!failed && nblk > 0) finish_rows(prev_row0, prev_rows);
  __syncthreads();
  if (!failed) {
    if (is_col) {
      if (a.dinit) {
        float gc[HP];
        tmem_ld16(t_G, gc);
        tmem_ld8(t_G + 16, gc + 16);
        tmem_ld_wait();
        bf16* dp = a.dinit + (bh * a.P) * a.N + ng;
#pragma unroll
        for (int j = 0; j < HP; ++j)
          if (half * HP + j < a.P) dp[(size_t)(half * HP + j) * a.N] = __float2bfloat16_rn(gc[j]);
      }
      // dA / ddt_bias partials of the two row halves, summed in a fixed order
      sXch[half * NT + n] = dAacc;
      sXch[(2 + half) * NT + n] = dbacc;
    }
    float* red = (float*)(smem + SM::kRed);
    if (is_io) red[io_t] = dDacc;
    __syncthreads();
    if (is_col && half == 0) {
      a.dApart[bh * a.N + ng] = sXch[n] + sXch[NT + n];
      a.dbpart[bh * a.N + ng] = sXch[2 * NT + n] + sXch[3 * NT + n];
    }
    if (tid == 0) {                                       // scalar dD partial of this (batch, head)
      float sacc = 0.f;
      for (int i = 0; i < NIO; ++i) sacc += red[i];
      if (blockIdx.x == 0) a.dDpart[bh] = sacc;            // dy . x does not depend on the states: one slice reports it
    }
  }
  if (a.status) {
    if (failed && tid == 0) atomicOr(a.status, 1);
    if (windowed && tid == 0) atomicOr(a.status, 4);       // informational: some block ran windowed
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// dD[h, p] partials for a per-(head, head-dim) D: sum over the rows of one (batch, head) of dy * x, one
// warp per head-dim index (the scan kernel only accumulates the per-head scalar)
__global__ void k_dD_hdim(const TArgs a) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int p = warp; p < a.P; p += blockDim.x >> 5) {
    float acc = 0.f;
    for (int l = lane; l < a.L; l += 32) {
      float dy = __bfloat162float(a.dout[b * a.g_sb + (int64_t)l * a.g_sl + h * a.g_sh + p]);
      if (a.has_z) {
        const float z1 = __bfloat162float(a.z[b * a.z_sb + (int64_t)l * a.z_sl + h * a.z_sh + p]);
        dy *= z1 / (1.f + ex2f(-z1 * LOG2E));
      }
      acc = fmaf(__bfloat162float(__float2bfloat16_rn(dy)), __bfloat162float(a.x[b * a.x_sb + (int64_t)l * a.x_sl + h * a.x_sh + p]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) a.dDpart[((size_t)b * a.H + h) * PP + p] = acc;
  }
}

// State slices: dx = sum over the slices of the partial dx rows + D dy, and dz = dout y sigmoid(z)(1 + z(1 - sigmoid(z)))
// (what group_store of the scan kernel does for a single slice).  One thread per group of 4 head-dim elements.
__global__ void k_combine_dx(const TArgs a, int slices, size_t groups) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  const int ngrp = a.P / 4;
  const int gq = (int)(i % ngrp);
  size_t r = i / ngrp;
  const int h = (int)(r % a.H);
  r /= a.H;
  const int l = (int)(r % a.L);
  const int b = (int)(r / a.L);
  auto lo = [](uint32_t w) { return __uint_as_float(w << 16); };
  auto hi = [](uint32_t w) { return __uint_as_float(w & 0xffff0000u); };
  const size_t o = (((size_t)b * a.L + l) * a.H + h) * a.P + gq * 4;
  const size_t slice_stride = (size_t)a.b * a.L * a.H * a.P;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < slices; ++s) {
    const uint2 tv = *(const uint2*)(a.dxpart + s * slice_stride + o);
    v[0] += lo(tv.x); v[1] += hi(tv.x); v[2] += lo(tv.y); v[3] += hi(tv.y);
  }
  const uint2 gv = *(const uint2*)(a.dout + b * a.g_sb + (int64_t)l * a.g_sl + h * a.g_sh + gq * 4);
  float dy[4] = {lo(gv.x), hi(gv.x), lo(gv.y), hi(gv.y)};
  if (a.has_z) {
    const uint2 zv = *(const uint2*)(a.z + b * a.z_sb + (int64_t)l * a.z_sl + h * a.z_sh + gq * 4);
    const uint2 yv = *(const uint2*)(a.out_x + b * a.o_sb + (int64_t)l * a.o_sl + h * a.o_sh + gq * 4);
    const float zf[4] = {lo(zv.x), hi(zv.x), lo(zv.y), hi(zv.y)};
    const float yf[4] = {lo(yv.x), hi(yv.x), lo(yv.y), hi(yv.y)};
    float dzv[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float sg = __fdividef(1.f, 1.f + ex2f(-zf[q] * LOG2E));
      dzv[q] = dy[q] * yf[q] * sg * (1.f + zf[q] * (1.f - sg));
      dy[q] *= zf[q] * sg;
    }
    *(uint2*)(a.dz + o) = make_uint2(pack_bf16(dzv[0], dzv[1]), pack_bf16(dzv[2], dzv[3]));
  }
  if (a.has_D) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      v[q] = fmaf(a.D_has_hdim ? __ldg(a.D + h * a.P + gq * 4 + q) : __ldg(a.D + h), __bfloat162float(__float2bfloat16_rn(dy[q])), v[q]);
  }
  *(uint2*)(a.dx + o) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
}

// dB[b,l,g,n], dC[b,l,g,n] = sums over the heads of group g of the per-head partials, stored as packed bf16 pairs
// {dB_h, dC_h} per (b, l, h, n); fixed order, 8 states per thread
__global__ void k_reduce_heads_bf16(int hpg, int N, int H, size_t total, const uint32_t* __restrict__ part,
                                    bf16* __restrict__ outB, bf16* __restrict__ outC) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // over (b, l, g, n/8)
  if (i >= total) return;
  const int n8 = N / 8;
  const size_t blg = i / n8;
  const int c = i % n8;
  const int G = H / hpg;
  const size_t bl = blg / G;
  const int g = blg % G;
  float accB[8], accC[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { accB[j] = 0.f; accC[j] = 0.f; }
  for (int k = 0; k < hpg; ++k) {
    const uint4* src = (const uint4*)(part + ((bl * H + g * hpg + k) * N) + c * 8);
    const uint4 v0 = src[0], v1 = src[1];
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      accB[j] += __uint_as_float(w[j] << 16);
      accC[j] += __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  *(uint4*)(outB + blg * N + c * 8) = make_uint4(pack_bf16(accB[0], accB[1]), pack_bf16(accB[2], accB[3]),
                                                 pack_bf16(accB[4], accB[5]), pack_bf16(accB[6], accB[7]));
  *(uint4*)(outC + blg * N + c * 8) = make_uint4(pack_bf16(accC[0], accC[1]), pack_bf16(accC[2], accC[3]),
                                                 pack_bf16(accC[4], accC[5]), pack_bf16(accC[6], accC[7]));
}

// out[h, j] = sum_b part[b, h, j]   (fixed order)
__global__ void k_reduce_batch(const float* __restrict__ part, int batch, int stride, float* __restrict__ out) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= stride) return;
  float acc = 0.f;
  for (int i = 0; i < batch; ++i) acc += part[(size_t)i * stride + j];
  out[j] = acc;
}
// dD from (b, H, PP) partials: (H, P) or (H)
__global__ void k_reduce_dD(const float* __restrict__ part, int batch, int H, int P, int has_hdim, float* __restrict__ out) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (has_hdim) {
    if (j >= H * P) return;
    const int h = j / P, p = j % P;
    float acc = 0.f;
    for (int i = 0; i < batch; ++i) acc += part[((size_t)i * H + h) * PP + p];
    out[j] = acc;
  } else {
    if (j >= H) return;
    float acc = 0.f;
    for (int i = 0; i < batch; ++i)
      for (int p = 0; p < P; ++p) acc += part[((size_t)i * H + j) * PP + p];
    out[j] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
struct BwdWs {
  uint32_t* dBCh;
  bf16 *saved, *wscr, *dxpart;
  float *dApart, *dbpart, *dDpart;
  int *redo_fwd, *redo_bwd;
};

static BwdWs carve_bwd(const issm_params& p, size_t* total) {
  Carver c(p.workspace);
  BwdWs w{};
  const size_t b = p.batch, L = p.seqlen, H = p.nheads, N = p.dstate;
  const size_t nblk = (L + QB - 1) / QB;
  w.dBCh = c.take<uint32_t>(b * L * H * N);
  w.dApart = c.take<float>(b * H * N);
  w.dbpart = c.take<float>(b * H * N);
  w.dDpart = c.take<float>(b * H * PP);
  const size_t slices = (size_t)state_slices(p.dstate);
  w.redo_fwd = c.take<int>(slices * b * H);
  w.redo_bwd = c.take<int>(slices * b * H);
  w.dxpart = slices > 1 ? c.take<bf16>(slices * b * L * H * p.headdim) : nullptr;
  w.wscr = c.take<bf16>(b * H * 63 * N * PP);             // window-entry states of one block per stream (windowed kernel)
  w.saved = p.saved_states ? nullptr : c.take<bf16>(b * H * (nblk + 1) * N * PP);
  *total = c.off;
  return w;
}

size_t tensor_bwd_workspace_bytes(const issm_params& p) {
  issm_params q = p;
  q.workspace = nullptr;
  size_t total = 0;
  carve_bwd(q, &total);
  return total;
}

template <int NT, typename TDT, int kMode>
static int launch_bwd_mode(const TArgs& a, const CUtensorMap& dtmap, cudaStream_t s) {
  const size_t smem = BwdSmem<NT>::kTotal + 1024;
  struct FastTag {};
  struct WinTag {};
  if (SmemAttrOnce<FastTag>::set(k_bwd_tensor<NT, TDT, false, kMode>, smem) != ISSM_OK ||
      SmemAttrOnce<WinTag>::set(k_bwd_tensor<NT, TDT, true, 0>, smem) != ISSM_OK)
    return ISSM_ERR_CUDA;
  const int slices = a.N / NT;
  ISSM_LAUNCH((k_bwd_tensor<NT, TDT, false, kMode>), dim3(slices, a.H, a.b), 2 * NT + 128, smem, s, a, dtmap);
  ISSM_LAUNCH((k_bwd_tensor<NT, TDT, true, 0>), dim3(slices, a.H, a.b), 2 * NT + 128, smem, s, a, dtmap);   // marked streams only
  if (slices > 1) {
    const size_t groups = (size_t)a.b * a.L * a.H * (a.P / 4);
    ISSM_LAUNCH(k_combine_dx, (unsigned)cdiv64(groups, 256), 256, 0, s, a, slices, groups);
  }
  return ISSM_OK;
}

template <int NT, typename TDT>
static int launch_bwd(TArgs a, const issm_params& p, cudaStream_t s) {
  CUtensorMap dtmap;
  a.dt_tma = make_dt_tensor_map(p, &dtmap) ? 1 : 0;
  // whole-tile copies of dt (when it is staged at all) and of B / C: the row order of the staged tiles is known
  const bool tiles = a.bc_contig && (sizeof(TDT) != 2 || a.dt_tma);
  if (!tiles) return launch_bwd_mode<NT, TDT, 0>(a, dtmap, s);
  return a.rev ? launch_bwd_mode<NT, TDT, 2>(a, dtmap, s) : launch_bwd_mode<NT, TDT, 1>(a, dtmap, s);
}

int tensor_bwd(const issm_params& p, cudaStream_t s) {
  size_t total = 0;
  const BwdWs w = carve_bwd(p, &total);
  bf16* saved = (bf16*)p.saved_states;
  if (!saved) {                                           // recompute the block-entry states (reference: issm_combined.py:136-144)
    saved = w.saved;
    int rc = tensor_fwd_states_only(p, saved, w.redo_fwd, s);
    if (rc) return rc;
  }
  TArgs a = make_targs(p);
  a.saved = saved;
  a.out_x = p.has_z ? (bf16*)p.out_x : nullptr;
  a.dout = (const bf16*)p.dout; a.g_sb = p.dout_sb; a.g_sl = p.dout_sl; a.g_sh = p.dout_sh;
  a.dfinal = p.has_dfinal ? p.dfinal_states : nullptr;
  a.dx = (bf16*)p.dx; a.ddt = p.ddt; a.dz = (bf16*)p.dz; a.dinit = (bf16*)p.dinitial_states;
  a.dBCh = w.dBCh; a.dApart = w.dApart; a.dbpart = w.dbpart; a.dDpart = w.dDpart;
  a.redo = w.redo_bwd; a.wscr = w.wscr; a.dxpart = w.dxpart;
  int rc;
  if (p.dstate != 128) rc = p.dt_dtype == ISSM_BF16 ? launch_bwd<256, bf16>(a, p, s) : launch_bwd<256, float>(a, p, s);
  else rc = p.dt_dtype == ISSM_BF16 ? launch_bwd<128, bf16>(a, p, s) : launch_bwd<128, float>(a, p, s);
  if (rc) return rc;
  const int hpg = p.nheads / p.ngroups;
  const size_t tot = (size_t)p.batch * p.seqlen * p.ngroups * (p.dstate / 8);
  ISSM_LAUNCH(k_reduce_heads_bf16, (unsigned)cdiv64(tot, 256), 256, 0, s, hpg, p.dstate, p.nheads, tot, w.dBCh, (bf16*)p.dB, (bf16*)p.dC);
  const int HN = p.nheads * p.dstate;
  ISSM_LAUNCH(k_reduce_batch, (HN + 127) / 128, 128, 0, s, w.dApart, p.batch, HN, p.dA);
  if (p.has_dt_bias) ISSM_LAUNCH(k_reduce_batch, (HN + 127) / 128, 128, 0, s, w.dbpart, p.batch, HN, p.ddt_bias);
  if (p.has_D) {
    if (p.D_has_hdim) {
      ISSM_LAUNCH(k_dD_hdim, dim3(p.nheads, p.batch), 256, 0, s, a);
      ISSM_LAUNCH(k_reduce_dD, (p.nheads * p.headdim + 63) / 64, 64, 0, s, w.dDpart, p.batch, p.nheads, p.headdim, 1, p.dD);
    } else {
      ISSM_LAUNCH(k_reduce_batch, (p.nheads + 63) / 64, 64, 0, s, w.dDpart, p.batch, p.nheads, p.dD);
    }
  }
  return ISSM_OK;
}

}  // namespace issm
