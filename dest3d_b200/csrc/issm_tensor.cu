// tcgen05 tensor-core path of the ISSM scan (bf16 activations, fp32 accumulation in TMEM): forward.
//
// One CTA walks one (batch, head) stream along the sequence in sub-blocks of 64 points; thread t of
// the CTA owns state column n = t for the whole walk: it transforms dt, keeps the running
// cumulative decay of its column, builds its column of every MMA operand, and owns TMEM lane
// t % 128 of the running state S[n, p] (fp32).  Per sub-block (rows l, s; a = cumsum of dt*A
// inside the block in log2 units, relative to the block start; a_last = a at the block end):
//   Cd[l,n] = C[l,n] 2^(a[l,n])                 Bd[s,n] = B[s,n] dt[s,n] 2^(-a[s,n])
//   M[l,s]  = sum_n Cd[l,n] Bd[s,n]                                   tcgen05.mma  64 x 64, K = N
//   Y[l,p]  = sum_n Cd[l,n] S[p,n] + sum_{s<=l} M[l,s] x[s,p]         tcgen05.mma  64 x 48, K = N, then 64
//   S[n,p] <- 2^(a_last) ( S[n,p] + sum_l Bd[l,n] x[l,p] )            tcgen05.mma 128 x 48, K = 64
// This is the chunked algorithm of issm_triton/issm_combined.py:57-92 (dt transform + cumsum,
// chunk state, state passing, C.A.B^T, chunk scan with D skip and silu(z) gate) with a 64-row
// chunk and the state carried on chip instead of through HBM.  The decay inside the contraction is
// factored through the block-start reference, so every factor stays in range as long as the span of
// |a| over a 64-point block is below 120 (log2 units); a block that violates this for some column is
// redone in 2, 4, ... 64 row windows with one reference each (exact for any decay: with single-row
// windows only the decay itself is floored, at 2^-100), and bit 2 of the status word records that it happened.
// dt (bf16), B and C rows of the next block are prefetched into shared memory by bulk (TMA) copies
// while the current block computes.
// More than 256 states (dstate 512, 768, 1024): the scan is a sum over the states, so every slice of 256 states is
// an independent scan over the same x with its own columns of dt, A, B, C and of the state; blockIdx.x is the
// slice, each slice writes its pre-skip / pre-gate output rows as floats, and k_combine_slices adds the slices
// and applies the D skip and the silu(z) gate.
#include "issm_tensor.cuh"

#include <cstring>

namespace issm {

template <int NT>
struct FwdSmem {
  static constexpr int kCd = 0;                         // [NT/64 atoms][64 l][128 B]
  static constexpr int kAtomB = (QB + PP) * 128;        // per 64-state atom: 64 rows of Bd, then PP rows of the state operand,
  static constexpr int kBd = kCd + NT * 128;            //   so that M and the state term of Y come out of ONE 64 x 112 MMA
  static constexpr int kSop = kBd + QB * 128;
  static constexpr int kX = kBd + (NT / 64) * kAtomB;   // [64 l][128 B]   (p in the row)
  static constexpr int kMm = kX + QB * 128;             // [64 l][128 B]   (s in the row)
  static constexpr int kSdt = kMm + QB * 128;           // staging: [64][NT] bf16
  static constexpr int kSB = kSdt + QB * NT * 2;
  static constexpr int kSC = kSB + QB * NT * 2;
  static constexpr int kY = kSC + QB * NT * 2;          // [64][PP] float: pre-skip, pre-gate output rows
  static constexpr int kAsum = kY + QB * PP * 4;        // [4][NT] float: sums of dt*A over the four 16-row quarters of a block
  static constexpr int kBars = kAsum + 4 * NT * 4;      //   (the windowed instantiation keeps per-half sums in the first two rows)
  static constexpr int kTotal = kBars + 64;
};

// bf16 operand copy (row of the state operand tile) and saved copy of one thread's PP / 2 state values
__device__ __forceinline__ void publish_state_cols(const TArgs& a, const float* sc, uint8_t* sop_col, int kcol, int half,
                                                   bf16* savep, int blk_index, bool save) {
  constexpr int HP = PP / 2;
  if (!a.no_output) {
#pragma unroll
    for (int j = 0; j < HP; ++j) *(bf16*)(sop_col + sw128_off(half * HP + j, kcol)) = __float2bfloat16_rn(sc[j]);
  }
  if (savep && save) {
    bf16* dst = savep + (size_t)blk_index * a.N * PP;
#pragma unroll
    for (int c = 0; c < HP / 8; ++c)
      *(uint4*)(dst + (size_t)c * a.N * 8) = make_uint4(pack_bf16(sc[c * 8], sc[c * 8 + 1]), pack_bf16(sc[c * 8 + 2], sc[c * 8 + 3]),
                          pack_bf16(sc[c * 8 + 4], sc[c * 8 + 5]), pack_bf16(sc[c * 8 + 6], sc[c * 8 + 7]));
  }
}

template <typename TDT>
struct WinCtx {
  uint8_t* smem;
  uint64_t *barA, *barA2;
  const TDT* dtp;
  bf16* savep;
  uint8_t* sop_col;
  float* sAsum;
  float* final_col;            // this thread's column of final_states when this is the last block and they are wanted
  int n, half, rows, row0, blk, ws, npass;
  float A2, bias;
  uint32_t t_S, phA;
  bool failed;
};

// The windowed passes of one block as the column threads run them (the service warp issues the MMAs of
// every pass between named barriers 11 and 12): rebuild Cd / Bd for the window, wait for the MMAs, rescale the
// state by the window's decay and republish it.
template <int NT, typename TDT>
__device__ __noinline__ void fwd_windowed_passes(const TArgs& a, WinCtx<TDT>& c) {
  using SM = FwdSmem<NT>;
  constexpr bool kStageDt = sizeof(TDT) == 2;
  constexpr int NTH = 2 * NT, HP = PP / 2;
  uint8_t* smem = c.smem;
  const int n = c.n, half = c.half, rows = c.rows, kcol = n & 63;
  const bool flipT = a.dt_tma && a.rev, flipB = (a.bc_contig || a.bc_tma) && a.rev;
  const bf16* sdt = (const bf16*)(smem + SM::kSdt) + n + (flipT ? (rows - 1) * NT : 0);
  const int dstep = flipT ? -NT : NT;
  const bf16* sB = (const bf16*)(smem + SM::kSB) + n + (flipB ? (rows - 1) * NT : 0);
  const bf16* sC = (const bf16*)(smem + SM::kSC) + n + (flipB ? (rows - 1) * NT : 0);
  const int bstep = flipB ? -NT : NT;
  uint8_t* cd_col = smem + SM::kCd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
  uint8_t* bd_col = smem + SM::kBd + (n >> 6) * SM::kAtomB + half * (32 * 128) + ((kcol & 7) << 1);
  const int kc = kcol >> 3;
  for (int w = 0; w < c.npass; ++w) {
    const int w0 = w * c.ws;
    const bool mine = (w0 >> 5) == half;           // ws <= 32: a window lies inside one half
    float acc = 0.f;
#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
      const int l = half * 32 + j;
      float cd = 0.f, bd = 0.f;
      if (mine && l >= w0 && l < w0 + c.ws && l < rows) {
        float raw;
        if (kStageDt) raw = __bfloat162float(sdt[l * dstep]);
        else raw = ldf(c.dtp + (int64_t)trow(a, c.row0 + l) * a.dt_sl + n);
        bool clamped;
        const float v = dt_transform(a, raw, c.bias, clamped);
        acc = fmaf(v, c.A2, acc);
        const float ac = fminf(fmaxf(acc, -100.f), 100.f);   // only binds for single-row windows
        cd = __bfloat162float(sC[l * bstep]) * ex2f(ac);
        bd = __bfloat162float(sB[l * bstep]) * v * ex2f(-ac);
      }
      const uint32_t off = (uint32_t)(j * 128 + ((kc ^ (j & 7)) << 4));
      *(bf16*)(cd_col + off) = __float2bfloat16_rn(cd);
      *(bf16*)(bd_col + off) = __float2bfloat16_rn(bd);
    }
    if (mine) c.sAsum[n] = fminf(fmaxf(acc, -100.f), 100.f);
    fence_async_smem();
    fence_before_sync();
    named_barrier(11, NTH + 32);
    if (!mbar_wait_warp(c.barA, c.phA)) c.failed = true;
    if (!mbar_wait_warp(c.barA2, c.phA)) c.failed = true;
    c.phA ^= 1;
    fence_after_sync();
    {                                              // state after the window = 2^(window decay) * accumulator
      float sc[HP];
      tmem_ld16(c.t_S, sc);
      tmem_ld8(c.t_S + 16, sc + 16);
      tmem_ld_wait();
      const float el = ex2f(c.sAsum[n]);
#pragma unroll
      for (int j = 0; j < HP; ++j) sc[j] *= el;
      tmem_st16(c.t_S, sc);
      tmem_st8(c.t_S + 16, sc + 16);
      const bool last = w == c.npass - 1;
      publish_state_cols(a, sc, c.sop_col, kcol, half, c.savep, c.blk + 1, last);
      if (last && c.final_col) {
#pragma unroll
        for (int j = 0; j < HP; ++j)
          if (half * HP + j < a.P) c.final_col[(size_t)(half * HP + j) * a.N] = sc[j];
      }
      tmem_st_wait();
    }
    fence_async_smem();
    fence_before_sync();
    named_barrier(12, NTH + 32);
  }
}

// Thread layout: 2*NT column threads, one service warp, three tile-I/O warps (registers are allocated in
// groups of four warps, so the service warp brings three more along).  Column thread (n = tid % NT,
// half = tid / NT) owns rows [32 half, 32 half + 32) of state column n in the operand pass and columns
// [24 half, 24 half + 24) of TMEM lane n of the running state.  The service warp issues every MMA and
// every bulk prefetch.  The I/O warps load the x / z rows of the block, build the x operand tile and
// store the previous block's output rows (D skip and gate applied) with coalesced accesses.
//
// Two instantiations walk the streams.  kWin = false is the fast one: it only notices a block outside the range
// of the single-reference factorisation and marks its (batch, head) stream in a.redo.  kWin = true is launched
// right behind it, returns at once for unmarked streams and redoes the marked ones from the start with the
// windowed passes described at fwd_windowed_passes (keeping that code out of the fast kernel is worth 15 %).
// kMode fixes the row order of the staged tiles at compile time, so that their addresses need no multiply:
// 1 = dt / B / C tiles staged in scan order (forward scan of regular arrays), 2 = staged in memory order for a
// reversed scan (walked backwards), 0 = decided at run time (row-by-row copies, mixed layouts).
template <int NT, typename TDT, bool kWin, int kMode>
__global__ void __launch_bounds__(2 * NT + 128, 1) k_fwd_tensor(const __grid_constant__ TArgs a, const __grid_constant__ FwdMaps maps) {
  using SM = FwdSmem<NT>;
  constexpr bool kStageDt = sizeof(TDT) == 2;
  constexpr int NTH = 2 * NT;                           // column threads
  constexpr int NIO = 96;                               // tile-I/O threads
  constexpr int HP = PP / 2;                            // state columns per thread
  constexpr int NCG = NT / 64;                          // column groups of the row epilogues
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte aligned base, kept as "shared array + offset" so that the compiler still knows the address space
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* barA = (uint64_t*)(smem + SM::kBars);
  uint64_t* barB = barA + 1;
  uint64_t* barS = barA + 2;
  uint64_t* barA2 = barA + 3;                            // state-update MMAs (barA: the [M | Y] MMAs issued before them)
  uint32_t* tmem_holder = (uint32_t*)(barA + 4);
  uint32_t* sFlag = tmem_holder + 1;                     // (block index + 1) * 8 + log2(windows) of a block that needs windowed passes
  float* sAsum = (float*)(smem + SM::kAsum);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_col = tid < NTH;
  const bool is_svc = warp == NTH / 32;
  const bool is_io = tid >= NTH + 32;
  const int io_t = tid - NTH - 32;
  const int h = blockIdx.y, b = blockIdx.z, g = h / a.hpg;
  const int n_off = blockIdx.x * NT;                     // first state of this CTA's slice
  const int stream = (blockIdx.x * a.b + b) * a.H + h;
  if (kWin && !a.redo[stream]) return;                   // the fast kernel finished this stream
  const int n = tid % NT, half = (tid / NT) & 1;
  const TDT* __restrict__ dtp = (const TDT*)a.dt + b * a.dt_sb + h * a.dt_sh + n_off;
  const bf16* __restrict__ Bp = a.B + b * a.B_sb + g * a.B_sg + n_off;
  const bf16* __restrict__ Cp = a.C + b * a.C_sb + g * a.C_sg + n_off;
  const bf16* __restrict__ xp = a.x + b * a.x_sb + h * a.x_sh;
  const bf16* __restrict__ zp = a.has_z ? a.z + b * a.z_sb + h * a.z_sh : nullptr;
  const float A2 = __ldg(a.A + h * a.N + n_off + n) * LOG2E;
  const float bias = a.has_bias ? __ldg(a.bias + h * a.N + n_off + n) : 0.f;
  // the same constants for the two adjacent states (2 pr, 2 pr + 1) of the fast instantiation's operand pass
  const int pr0 = n_off + 2 * (tid % (NT / 2));
  const float2 A2p = f2(__ldg(a.A + h * a.N + pr0) * LOG2E, __ldg(a.A + h * a.N + pr0 + 1) * LOG2E);
  const float bsc = a.softplus ? LOG2E : 1.f;
  const float2 biasL2 = a.has_bias ? f2(__ldg(a.bias + h * a.N + pr0) * bsc, __ldg(a.bias + h * a.N + pr0 + 1) * bsc) : f2(0.f);
  const int nblk = (a.L + QB - 1) / QB;

  // one-time setup: zero the padded operand tiles, barriers, TMEM
  for (int i = tid; i < (SM::kSdt - SM::kBd) / 16; i += blockDim.x) ((uint4*)(smem + SM::kBd))[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) { mbar_init(barA, 1); mbar_init(barB, 1); mbar_init(barS, 1); mbar_init(barA2, 1); mbar_fence_init(); *sFlag = 0; }
  if (warp == 0) { tmem_alloc(tmem_holder, 256); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t t_M = tmem, t_Y = tmem + 64;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t t_S = tmem + lane_base + 128 + (n >> 7) * PP + half * HP;   // this thread's part of TMEM lane n

  // bulk prefetch of the dt / B / C rows of block `blk` (service warp, completion on barS).  When the
  // B / C rows are adjacent in memory a whole tile is ONE copy; a reversed scan then finds row l of
  // the block at staged row rows-1-l.
  auto prefetch = [&](int blk) {
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    const bool dt_tile = kStageDt && a.dt_tma;
    const int64_t m0 = a.rev ? a.L - row0 - rows : row0;            // lowest memory row of the tile
    // a tiled TMA load always delivers the whole 64-row box (rows past the array's end are filled with zeros)
    if (lane == 0) mbar_expect_tx(barS, (uint32_t)(a.bc_tma ? QB : rows) * NT * 2 * 2 + (kStageDt ? (uint32_t)(dt_tile ? QB : rows) * NT * 2 : 0u));
    __syncwarp();
    if (dt_tile && lane == 2) tma_load_2d(smem + SM::kSdt, &maps.dt, h * (int)a.dt_sh + n_off, b * a.L + (int)m0, barS);
    if (a.bc_tma) {
      if (lane == 0) tma_load_2d(smem + SM::kSB, &maps.B, g * (int)a.B_sg + n_off, b * a.L + (int)m0, barS);
      if (lane == 1) tma_load_2d(smem + SM::kSC, &maps.C, g * (int)a.C_sg + n_off, b * a.L + (int)m0, barS);
    } else if (a.bc_contig) {
      if (lane == 0) bulk_g2s(smem + SM::kSB, Bp + m0 * a.B_sl, (uint32_t)rows * NT * 2, barS);
      if (lane == 1) bulk_g2s(smem + SM::kSC, Cp + m0 * a.C_sl, (uint32_t)rows * NT * 2, barS);
    }
    for (int l = lane; l < rows; l += 32) {
      const int64_t mr = trow(a, row0 + l);
      if (kStageDt && !dt_tile) bulk_g2s(smem + SM::kSdt + l * NT * 2, (const bf16*)dtp + mr * a.dt_sl, NT * 2, barS);
      if (!a.bc_contig && !a.bc_tma) {
        bulk_g2s(smem + SM::kSB + l * NT * 2, Bp + mr * a.B_sl, NT * 2, barS);
        bulk_g2s(smem + SM::kSC + l * NT * 2, Cp + mr * a.C_sl, NT * 2, barS);
      }
    }
  };
  // the whole-tile copies of the block after the next one are announced to L2 at the same time
  auto prefetch_l2 = [&](int blk) {
    if (blk >= nblk) return;
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    const int64_t m0 = a.rev ? a.L - row0 - rows : row0;
    if (kStageDt && a.dt_tma && lane == 2) tma_prefetch_2d(&maps.dt, h * (int)a.dt_sh + n_off, b * a.L + (int)m0);
    if (a.bc_tma) {
      if (lane == 0) tma_prefetch_2d(&maps.B, g * (int)a.B_sg + n_off, b * a.L + (int)m0);
      if (lane == 1) tma_prefetch_2d(&maps.C, g * (int)a.C_sg + n_off, b * a.L + (int)m0);
    } else if (a.bc_contig) {
      if (lane == 0) bulk_prefetch_l2(Bp + m0 * a.B_sl, (uint32_t)rows * NT * 2);
      if (lane == 1) bulk_prefetch_l2(Cp + m0 * a.C_sl, (uint32_t)rows * NT * 2);
    }
  };
  if (is_svc) { prefetch(0); prefetch_l2(1); }

  uint8_t* sop_col = smem + SM::kSop + (n >> 6) * SM::kAtomB;
  const int kcol = n & 63;
  // saved block-entry states: (b, H, nblk + 1, PP / 8, N, 8) bf16, i.e. per block the interleaved
  // [head-dim chunk][state][8] layout the backward uses directly as an MMA operand
  bf16* savep = a.saved ? a.saved + (((size_t)b * a.H + h) * (nblk + 1)) * a.N * PP + ((size_t)half * (HP / 8) * a.N + n_off + n) * 8 : nullptr;
  auto publish_state = [&](const float* sc, int blk_index, bool save) {
    publish_state_cols(a, sc, sop_col, kcol, half, savep, blk_index, save);
  };
  if (is_col) {                                          // initial state -> TMEM, operand, saved[0]
    float sc[HP];
#pragma unroll
    for (int j = 0; j < HP; ++j) sc[j] = 0.f;
    if (a.has_init) {
      const bf16* __restrict__ ip = a.init + (((size_t)b * a.H + h) * a.P) * a.N + n_off + n;
#pragma unroll
      for (int j = 0; j < HP; ++j)
        if (half * HP + j < a.P) sc[j] = __bfloat162float(ip[(size_t)(half * HP + j) * a.N]);
    }
    tmem_st16(t_S, sc);
    tmem_st8(t_S + 16, sc + 16);
    publish_state(sc, 0, true);
    tmem_st_wait();
  }

  // I/O threads work on groups of 4 consecutive head-dim elements (8-byte accesses; headdim % 4 == 0):
  // group k of thread t is flat index t + k * NIO of the [64][P / 4] grid; (row, group) advance by
  // (NIO / (P/4), NIO % (P/4)), so there is no division in the loops.  All loads of a pass are
  // unconditional (row clamped into the block) and in flight together.
  const float dscalar = (a.has_D && !a.D_has_hdim) ? __ldg(a.D + h) : 0.f;
  constexpr int XG = (QB * (PP / 4) + NIO - 1) / NIO;    // groups per I/O thread (8)
  const int ngrp = a.P / 4;
  const int io_l0 = io_t / ngrp, io_g0 = io_t % ngrp, io_dl = NIO / ngrp, io_dg = NIO % ngrp;
  auto io_next = [&](int& l, int& gq) {
    l += io_dl; gq += io_dg;
    if (gq >= ngrp) { gq -= ngrp; ++l; }
  };
  auto bf_lo = [](uint32_t w) { return __uint_as_float(w << 16); };
  auto bf_hi = [](uint32_t w) { return __uint_as_float(w & 0xffff0000u); };
  // out = (y + D x) * silu(z) for the output rows of a finished block.  The [64][P / 4] groups of the tile are dealt
  // out one per thread: groups 0..511 to the column threads (which do them while the MMAs of the next block run and
  // they would otherwise wait), the rest to the I/O threads.  `group_load` issues the loads of x and z, `group_store`
  // combines them with the accumulator row in shared memory and stores.
  struct RowGroup { uint2 xv, zv; int l, gq; };
  auto group_load = [&](int t_row0, int t_rows, int gi) {
    RowGroup g;
    g.l = gi / ngrp;
    g.gq = gi - g.l * ngrp;
    const int64_t mr = trow(a, t_row0 + min(g.l, t_rows - 1));
    g.xv = *(const uint2*)(xp + mr * a.x_sl + g.gq * 4);
    g.zv = a.has_z ? *(const uint2*)(zp + mr * a.z_sl + g.gq * 4) : make_uint2(0, 0);
    return g;
  };
  auto group_store = [&](const RowGroup& g, int t_row0, int t_rows) {
    const int l = g.l, gq = g.gq;
    if (l >= t_rows) return;
    const float4 yv = *(const float4*)(smem + SM::kY + (l * PP + gq * 4) * 4);
    if (a.ypart) {                                         // one slice of the states: the skip and the gate come after the sum
      *(float4*)(a.ypart + ((((size_t)blockIdx.x * a.b + b) * a.L + trow(a, t_row0 + l)) * a.H + h) * a.P + gq * 4) = yv;
      return;
    }
    float y[4] = {yv.x, yv.y, yv.z, yv.w};
    const float xf[4] = {bf_lo(g.xv.x), bf_hi(g.xv.x), bf_lo(g.xv.y), bf_hi(g.xv.y)};
    const float zf[4] = {bf_lo(g.zv.x), bf_hi(g.zv.x), bf_lo(g.zv.y), bf_hi(g.zv.y)};
#pragma unroll
    for (int q = 0; q < 4; ++q)
      y[q] = fmaf(a.D_has_hdim ? __ldg(a.D + h * a.P + gq * 4 + q) : dscalar, xf[q], y[q]);
    const int64_t o = b * a.o_sb + (int64_t)trow(a, t_row0 + l) * a.o_sl + h * a.o_sh + gq * 4;
    if (a.has_z) {
      *(uint2*)(a.out_x + o) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
#pragma unroll
      for (int q = 0; q < 4; ++q) y[q] *= __fdividef(zf[q], 1.f + ex2f(-zf[q] * LOG2E));
    }
    *(uint2*)(a.out + o) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
  };
  constexpr int kColGroups = 512;                        // groups of a tile handled by the column threads
  constexpr int kColR = kColGroups / NTH;                // ... per column thread
  constexpr int kIoR = (QB * (PP / 4) - kColGroups + NIO - 1) / NIO;   // per I/O thread
  auto store_tile_io = [&](int t_row0, int t_rows) {     // the I/O threads' share, loads first
    RowGroup g[kIoR];
#pragma unroll
    for (int r = 0; r < kIoR; ++r) g[r] = group_load(t_row0, t_rows, kColGroups + io_t + r * NIO);
#pragma unroll
    for (int r = 0; r < kIoR; ++r) group_store(g[r], t_row0, t_rows);
  };
  auto store_tile = [&](int t_row0, int t_rows) {        // a whole tile at once (after the walk)
    if (is_col) {
#pragma unroll
      for (int r = 0; r < kColR; ++r) group_store(group_load(t_row0, t_rows, tid + r * NTH), t_row0, t_rows);
    } else if (is_io) {
      store_tile_io(t_row0, t_rows);
    }
  };

  // descriptor bases (start address = shared-memory base; per-MMA byte offsets are added at issue)
  const uint32_t sb = smem_u32(smem);
  const uint64_t dK = desc_sw128(sb);                          // K-major operands
  const uint64_t dMNb = desc_sw128_mn(sb, SM::kAtomB);         // Bd as [states x rows] operand: 64-state groups kAtomB apart
  const uint64_t dMNx = desc_sw128_mn(sb, QB * 128);           // x tile as [head-dim x rows] operand

  // every MMA of one pass over a block: [M | Y] = Cd [Bd ; S]^T (one 64 x 112 MMA per K step), S += Bd^T x
  auto issue_mmas = [&](bool accumulate) {
    if (!a.no_output) {
#pragma unroll
      for (int at = 0; at < NT / 64; ++at)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16_off(t_M, dK, SM::kCd + at * (QB * 128) + kk * 32, dK, SM::kBd + at * SM::kAtomB + kk * 32,
                       idesc_bf16(64, QB + PP), accumulate || (at | kk) != 0);
    }
    mma_commit(barA);
#pragma unroll
    for (int sl = 0; sl < NT / 128; ++sl)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        mma_bf16_off(tmem + 128 + sl * PP, dMNb, SM::kBd + sl * (2 * SM::kAtomB) + kk * 2048, dMNx, SM::kX + kk * 2048,
                     idesc_bf16(128, PP, 1, 1), 1);
    mma_commit(barA2);
  };

  bool failed = false;
  uint32_t windowed = 0, unsafe = 0;

  // The three roles run their own loop over the blocks (so that the registers of one role's state are not held
  // through the code of the others); they meet at the two block-wide barriers of every iteration.
  // Output rows of the block before: its accumulator tile was completed before the first barrier of an iteration
  // and is not rewritten until after the second one.
  if (is_io) {
    // ================================================ tile-I/O warps ================================================
    for (int blk = 0; blk < nblk; ++blk) {
      const int row0 = blk * QB;
      const int rows = min(QB, a.L - row0);
      const uint32_t parity = blk & 1;
      // ---- x rows of this block -> x operand tile [l][p] (swizzled rows); the tile is free once the last
      //      MMA of the previous block has completed ---------------------------------------------------------
      if (blk > 0 && !a.no_output && !mbar_wait_warp(barB, parity ^ 1)) failed = true;
      uint2 xv[XG];
      int l = io_l0, gq = io_g0;
#pragma unroll
      for (int k = 0; k < XG; ++k) {
        xv[k] = *(const uint2*)(xp + (int64_t)trow(a, row0 + min(l, rows - 1)) * a.x_sl + gq * 4);
        io_next(l, gq);
      }
      l = io_l0; gq = io_g0;
#pragma unroll
      for (int k = 0; k < XG; ++k) {
        if (l < QB) *(uint2*)(smem + SM::kX + sw128_off(l, gq * 4)) = l < rows ? xv[k] : make_uint2(0, 0);
        io_next(l, gq);
      }
      fence_async_smem();
      // the z rows of this block are first needed when its output rows are written, one block later: have them in L2
      if (a.has_z && !a.no_output)
        for (int r = io_t; r < rows; r += NIO) prefetch_l2_span(zp + (int64_t)trow(a, row0 + r) * a.z_sl, a.P * 2);
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      if (blk > 0 && !a.no_output) store_tile_io(row0 - QB, QB);
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
    }
  } else if (is_svc) {
    // ================================================= service warp =================================================
    for (int blk = 0; blk < nblk; ++blk) {
      const int row0 = blk * QB;
      const int rows = min(QB, a.L - row0);
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      // A block some column flagged is redone in windows of ws = 64 >> kw rows (the operands built above are
      // dropped): per window the column threads rebuild Cd / Bd relative to the window start with every row outside
      // the window zero, the MMAs accumulate [M | Y] over the windows (M becomes block diagonal, rows of later
      // windows see earlier ones through the state) and the state is rescaled by the window's decay.
      const uint32_t flag = kWin ? *sFlag : 0u;
      const int kw = (kWin && (flag >> 3) == (uint32_t)(blk + 1)) ? (int)(flag & 7) : 0;
      const int ws = QB >> kw;
      const int npass = kw ? (rows + ws - 1) / ws : 1;
      // ---- MMAs of the block (of every window of a flagged block) ---------------------------------------------
      if (!kWin || kw == 0) {
        if (lane == 0) {
          fence_after_sync();
          issue_mmas(false);
        }
        __syncwarp();
      } else {
        for (int w = 0; w < npass; ++w) {
          named_barrier(11, NTH + 32);                   // window operands are in place
          if (lane == 0) {
            fence_after_sync();
            issue_mmas(w != 0);
          }
          __syncwarp();
          named_barrier(12, NTH + 32);                   // state rescaled and republished
        }
      }
      if (blk + 1 < nblk) prefetch(blk + 1);             // every column thread is past its staging reads
      prefetch_l2(blk + 2);
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      if (a.no_output) continue;
      // ---- Y += tril(M) x ------------------------------------------------------------------------------
      if (lane == 0) {
        fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16_off(t_Y, dK, SM::kMm + kk * 32, dMNx, SM::kX + kk * 2048, idesc_bf16(64, PP, 0, 1), 1);
        mma_commit(barB);
      }
      fence_before_sync();
    }
  } else {
    // ================================================ column threads ================================================
    uint32_t phA = 0;
    for (int blk = 0; blk < nblk; ++blk) {
      const int row0 = blk * QB;
      const int rows = min(QB, a.L - row0);
      const uint32_t parity = blk & 1;
      float alast = 0.f;
      if (!mbar_wait_warp(barS, parity)) failed = true;  // staged dt / B / C of this block have landed

      // Staged tiles are addressed as base + l * step in units of rows: a tile that was copied in memory
      // order for a reversed scan is walked backwards.  Full blocks run a guard-free instantiation.
      const bool flipT = kMode ? kMode == 2 : (a.dt_tma && a.rev), flipB = kMode ? kMode == 2 : ((a.bc_contig || a.bc_tma) && a.rev);
      const bf16* sdt = (const bf16*)(smem + SM::kSdt) + n + (flipT ? (rows - 1) * NT : 0);
      const int dstep = flipT ? -NT : NT;
      const bf16* sB = (const bf16*)(smem + SM::kSB) + n + (flipB ? (rows - 1) * NT : 0);
      const bf16* sC = (const bf16*)(smem + SM::kSC) + n + (flipB ? (rows - 1) * NT : 0);
      const int bstep = flipB ? -NT : NT;

      if constexpr (kWin) {
        // the windowed instantiation keeps the one-state-per-thread pass (its window code addresses rows per half)
        // ---- phase A: dt of this thread's 32 rows and their summed log2-decay -----------------------
        float dtv[32];
        float asum = 0.f;
        auto phaseA = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
  #pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int l = half * 32 + j;
            const int sl = kFull ? l : min(l, rows - 1);
            float raw;
            if (kStageDt) raw = __bfloat162float(sdt[sl * dstep]);
            else raw = ldf(dtp + (int64_t)trow(a, row0 + sl) * a.dt_sl + n);
            bool clamped;
            float v = dt_transform(a, raw, bias, clamped);
            if (!kFull && l >= rows) v = 0.f;
            dtv[j] = v;
            asum = fmaf(v, A2, asum);
          }
        };
        if (rows == QB) phaseA(std::true_type{}); else phaseA(std::false_type{});
        sAsum[half * NT + n] = asum;
        named_barrier(1 + (warp & (NT / 32 - 1)), 64);     // the two warps that share these 32 columns
        const float a0 = sAsum[n];
        alast = a0 + sAsum[NT + n];
        // Range of the factorisation: 2^(+-a) must stay finite in bf16.  A column whose decay over the block
        // (or over its first half) exceeds 2^120 asks for the block to be redone in 2^k row windows, each with
        // its own reference: the smallest k for which this thread's windows stay within 2^100.
        if (!(fabsf(a0) <= 120.f && fabsf(alast) <= 120.f)) {
          if (kWin) atomicMax(sFlag, (uint32_t)(blk + 1) * 8 + window_need<TDT>(a, sdt, dstep, dtp, row0, rows, half, n, A2, bias));
          else unsafe = 1;
        }

        // ---- phase B: this thread's rows of column n of Cd = C 2^a and Bd = B dt 2^-a ------------------
        auto phaseB = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
          uint8_t* cd_col = smem + SM::kCd + (n >> 6) * (QB * 128) + half * (32 * 128) + ((kcol & 7) << 1);
          uint8_t* bd_col = smem + SM::kBd + (n >> 6) * SM::kAtomB + half * (32 * 128) + ((kcol & 7) << 1);
          const int kc = kcol >> 3;
          float acc = half ? a0 : 0.f;
  #pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int l = half * 32 + j;
            const int sl = kFull ? l : min(l, rows - 1);
            acc = fmaf(dtv[j], A2, acc);
            float cd = __bfloat162float(sC[sl * bstep]) * ex2f(acc);
            float bd = __bfloat162float(sB[sl * bstep]) * dtv[j] * ex2f(-acc);
            if (!kFull && l >= rows) { cd = 0.f; bd = 0.f; }
            const uint32_t off = (uint32_t)(j * 128 + ((kc ^ (j & 7)) << 4));
            *(bf16*)(cd_col + off) = __float2bfloat16_rn(cd);
            *(bf16*)(bd_col + off) = __float2bfloat16_rn(bd);
          }
        };
        if (rows == QB) phaseB(std::true_type{}); else phaseB(std::false_type{});
      } else {
        // ---- operand pass, two adjacent states (2 pr, 2 pr + 1) and the 16 rows of quarter qr per thread: every
        //      shared-memory access moves a bf16 pair (4 bytes) and the fp32 arithmetic runs as packed pairs --------
        constexpr int NPR = NT / 2;
        const int pr = tid % NPR, qr = tid / NPR;
        const bool flipB2 = kMode ? kMode == 2 : ((a.bc_contig || a.bc_tma) && a.rev);
        const uint32_t* sdt2 = (const uint32_t*)(smem + SM::kSdt) + pr + (flipT ? (rows - 1) * NPR : 0);
        const int dstep2 = flipT ? -NPR : NPR;
        const uint32_t* sB2 = (const uint32_t*)(smem + SM::kSB) + pr + (flipB2 ? (rows - 1) * NPR : 0);
        const uint32_t* sC2 = (const uint32_t*)(smem + SM::kSC) + pr + (flipB2 ? (rows - 1) * NPR : 0);
        const int bstep2 = flipB2 ? -NPR : NPR;
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
        *(float2*)(sAsum + qr * NT + 2 * pr) = asum2;
        named_barrier(1 + (warp % (NPR / 32)), 128);       // the four warps that share these 64 columns
        const float2 q0 = *(const float2*)(sAsum + 2 * pr), q1 = *(const float2*)(sAsum + NT + 2 * pr),
                     q2 = *(const float2*)(sAsum + 2 * NT + 2 * pr), q3 = *(const float2*)(sAsum + 3 * NT + 2 * pr);
        const float2 c1 = q0, c2 = __fadd2_rn(c1, q1), c3 = __fadd2_rn(c2, q2), c4 = __fadd2_rn(c3, q3);
        // range of the factorisation (see the windowed instantiation above): every running sum must stay within 2^120
        const float worst = fmaxf(fmaxf(fmaxf(fabsf(c1.x), fabsf(c1.y)), fmaxf(fabsf(c2.x), fabsf(c2.y))),
                                  fmaxf(fmaxf(fabsf(c3.x), fabsf(c3.y)), fmaxf(fabsf(c4.x), fabsf(c4.y))));
        if (!(worst <= 120.f)) unsafe = 1;
        auto phaseB2 = [&](auto full) {
          constexpr bool kFull = decltype(full)::value;
          const int at = pr >> 5, kc = (pr & 31) >> 2;     // 64-state atom, 16-byte chunk inside its 128-byte rows
          uint8_t* cd_col = smem + SM::kCd + at * (QB * 128) + qr * (16 * 128) + ((pr & 3) << 2);
          uint8_t* bd_col = smem + SM::kBd + at * SM::kAtomB + qr * (16 * 128) + ((pr & 3) << 2);
          float2 acc = qr == 0 ? f2(0.f) : (qr == 1 ? c1 : (qr == 2 ? c2 : c3));
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int l = qr * 16 + j;
            const int sl = kFull ? l : min(l, rows - 1);
            const float2 dtj = dtv[j];
            acc = __ffma2_rn(dtj, A2p, acc);
            float2 cd = __fmul2_rn(unpack_bf16(sC2[sl * bstep2]), ex2f2(acc));
            float2 bd = __fmul2_rn(__fmul2_rn(unpack_bf16(sB2[sl * bstep2]), dtj), ex2f2_neg(acc));
            if (!kFull && l >= rows) { cd = f2(0.f); bd = f2(0.f); }
            const uint32_t off = (uint32_t)(j * 128 + ((kc ^ (j & 7)) << 4));
            *(uint32_t*)(cd_col + off) = pack_bf16(cd);
            *(uint32_t*)(bd_col + off) = pack_bf16(bd);
          }
        };
        if (rows == QB) phaseB2(std::true_type{}); else phaseB2(std::false_type{});
      }
      fence_async_smem();
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      const uint32_t flag = kWin ? *sFlag : 0u;
      const int kw = (kWin && (flag >> 3) == (uint32_t)(blk + 1)) ? (int)(flag & 7) : 0;
      const int ws = QB >> kw;
      const int npass = kw ? (rows + ws - 1) / ws : 1;
      if constexpr (!kWin) alast = ((sAsum[n] + sAsum[NT + n]) + sAsum[2 * NT + n]) + sAsum[3 * NT + n];   // summed decay of column n
      // output rows of the previous block, while the MMAs of this one run and the column threads would wait anyway
      if (blk > 0 && !a.no_output) {
#pragma unroll
        for (int r = 0; r < kColR; ++r) group_store(group_load(row0 - QB, QB, tid + r * NTH), row0 - QB, QB);
      }
      if (!kWin || kw == 0) {
        if (!mbar_wait_warp(barA, phA)) failed = true;
        phA ^= 1;
        fence_after_sync();
      } else {
        windowed = 1;
        WinCtx<TDT> c;
        c.smem = smem; c.barA = barA; c.barA2 = barA2; c.dtp = dtp; c.savep = savep; c.sop_col = sop_col; c.sAsum = sAsum;
        c.final_col = (blk == nblk - 1 && a.want_final) ? a.final_states + (((size_t)b * a.H + h) * a.P) * a.N + n_off + n : nullptr;
        c.n = n; c.half = half; c.rows = rows; c.row0 = row0; c.blk = blk; c.ws = ws; c.npass = npass;
        c.A2 = A2; c.bias = bias; c.t_S = t_S; c.phA = phA; c.failed = failed;
        fwd_windowed_passes<NT, TDT>(a, c);
        phA = c.phA; failed = c.failed;
        fence_after_sync();
      }

      // ---- epilogue 1a: masked M -> bf16 operand (every warp takes 16-column groups of its 16 rows) ----
      if (!a.no_output && !failed) {
        const int l = (warp & 3) * 16 + lane;
        for (int c16 = (warp >> 2) % NCG; c16 < 4; c16 += NCG) {
          float mv[16];
          tmem_ld16(t_M + lane_base + c16 * 16, mv);
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
              *(uint4*)(smem + SM::kMm + sw128_chunk(l, c16 * 2 + c)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
      }
      // ---- epilogue 1b: new state = 2^(a_last) * accumulator; back to TMEM, operand and saved copies ----
      if (kw == 0) {
        if (!mbar_wait_warp(barA2, phA ^ 1)) failed = true; // phA was flipped after the barA wait of this block
        fence_after_sync();
      }
      if (!failed && kw == 0) {
        float sc[HP];
        tmem_ld16(t_S, sc);
        tmem_ld8(t_S + 16, sc + 16);
        tmem_ld_wait();
        const float el = ex2f(alast);
#pragma unroll
        for (int j = 0; j < HP; ++j) sc[j] *= el;
        tmem_st16(t_S, sc);
        tmem_st8(t_S + 16, sc + 16);
        publish_state(sc, blk + 1, true);
        if (blk == nblk - 1 && a.want_final) {
          float* fp = a.final_states + (((size_t)b * a.H + h) * a.P) * a.N + n_off + n;
#pragma unroll
          for (int j = 0; j < HP; ++j)
            if (half * HP + j < a.P) fp[(size_t)(half * HP + j) * a.N] = sc[j];
        }
        tmem_st_wait();
      }
      fence_async_smem();
      fence_before_sync();
      if (__syncthreads_or(failed)) { failed = true; break; }
      if (a.no_output) continue;
      if (!mbar_wait_warp(barB, parity)) failed = true;
      fence_after_sync();
      // ---- epilogue 2: accumulator rows -> shared memory (skip, gate and store happen coalesced) ----
      if (!failed) {
        const int l = (warp & 3) * 16 + lane;
        for (int c16 = (warp >> 2) % NCG; c16 < PP / 16; c16 += NCG) {
          float yv[16];
          tmem_ld16(t_Y + lane_base + c16 * 16, yv);
          tmem_ld_wait();
          if (lane < 16) {
            float4* dst = (float4*)(smem + SM::kY + (l * PP + c16 * 16) * 4);
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[c] = make_float4(yv[c * 4], yv[c * 4 + 1], yv[c * 4 + 2], yv[c * 4 + 3]);
          }
        }
      }
      fence_before_sync();
    }
  }
  const int prev_row0 = (nblk - 1) * QB, prev_rows = a.L - prev_row0;   // the block processed last

  // a wait of the last iteration can expire after that iteration's last block-wide vote: make the verdict
  // uniform over the block before anything below depends on it
  const int votes = __syncthreads_or((int)unsafe | (failed ? 2 : 0));
  const int any_unsafe = votes & 1;
  failed = (votes & 2) != 0;
  if (!failed && !a.no_output && nblk > 0) store_tile(prev_row0, prev_rows);   // last block's tile
  if (!kWin && tid == 0) a.redo[stream] = any_unsafe;
  if (a.status) {
    if (failed && tid == 0) atomicOr(a.status, 1);
    if (windowed && tid == 0) atomicOr(a.status, 4);       // informational: some block ran windowed
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------
static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// number of 256-state slices a call is cut into (1 for dstate 128 / 256; 0 = no tensor-core kernels for this dstate)
int state_slices(int dstate) {
  if (dstate == 128 || dstate == 256) return 1;
  if (dstate % 256 == 0 && dstate <= 1024) return dstate / 256;
  return 0;
}

bool tensor_path_supported(const issm_params& p, int pass) {
  if (p.io_dtype != ISSM_BF16) return false;
  // the tile-I/O warps move 4 head-dim elements (8 bytes) at a time; the backward's dx tile holds 40 columns
  if (p.headdim > 40 || (p.headdim & 3)) return false;
  // strides of dimensions of size 1 take no part in the rules (the entry points canonicalise them; direct callers of this
  // function get the same treatment here)
  const int64_t mb = p.batch > 1 ? -1 : 0, mh = p.nheads > 1 ? -1 : 0, mg = p.ngroups > 1 ? -1 : 0, ml = p.seqlen > 1 ? -1 : 0;
  if (((p.x_sb & mb) | (p.x_sl & ml) | (p.x_sh & mh) | (p.out_sb & mb) | (p.out_sl & ml) | (p.out_sh & mh) | (p.dout_sb & mb) |
       (p.dout_sl & ml) | (p.dout_sh & mh)) & 3) return false;
  if (p.has_z && (((p.z_sb & mb) | (p.z_sl & ml) | (p.z_sh & mh)) & 3)) return false;
  if (((uintptr_t)p.x | (uintptr_t)p.z | (uintptr_t)p.out | (uintptr_t)p.out_x | (uintptr_t)p.dout | (uintptr_t)p.dx | (uintptr_t)p.dz) & 7) return false;
  const int slices = state_slices(p.dstate);
  if (slices == 0) return false;
  // bulk (TMA) row copies need 16-byte aligned rows of B, C and (bf16) dt
  if (p.B && (!aligned16(p.B) || !aligned16(p.C))) return false;
  if (((p.B_sb & mb) | (p.B_sl & ml) | (p.B_sg & mg) | (p.C_sb & mb) | (p.C_sl & ml) | (p.C_sg & mg)) & 7) return false;
  if (p.dt_dtype == ISSM_BF16) {
    if (p.dt && !aligned16(p.dt)) return false;
    if (((p.dt_sb & mb) | (p.dt_sl & ml) | (p.dt_sh & mh)) & 7) return false;
  } else {
    // float dt is read from global memory two adjacent states (8 bytes) at a time
    if (((uintptr_t)p.dt & 7) || (((p.dt_sb & mb) | (p.dt_sl & ml) | (p.dt_sh & mh)) & 1)) return false;
  }
  return true;
}

size_t tensor_workspace_bytes(const issm_params& p, int pass) {
  if (pass != 0) return tensor_bwd_workspace_bytes(p);
  // forward: one mark per (slice, batch, head) stream; with more than one slice the float partial outputs
  const int slices = state_slices(p.dstate);
  size_t total = align_up((size_t)slices * p.batch * p.nheads * sizeof(int), 256);
  if (slices > 1) total += align_up((size_t)slices * p.batch * p.seqlen * p.nheads * p.headdim * sizeof(float), 256);
  return total;
}

// out = (sum over the slices of the partial outputs + D x) * silu(z); pre-gate rows to out_x when gated.
// One thread per group of 4 consecutive head-dim elements.
__global__ void k_combine_slices(const TArgs a, int slices, size_t groups) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  const int ngrp = a.P / 4;
  const int gq = (int)(i % ngrp);
  size_t r = i / ngrp;
  const int h = (int)(r % a.H);
  r /= a.H;
  const int l = (int)(r % a.L);
  const int b = (int)(r / a.L);
  const size_t slice_stride = (size_t)a.b * a.L * a.H * a.P;
  const float* yp = a.ypart + (((size_t)b * a.L + l) * a.H + h) * a.P + gq * 4;
  float4 acc = *(const float4*)yp;
  for (int s = 1; s < slices; ++s) {
    const float4 v = *(const float4*)(yp + s * slice_stride);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  float y[4] = {acc.x, acc.y, acc.z, acc.w};
  if (a.has_D) {
    const uint2 xv = *(const uint2*)(a.x + b * a.x_sb + (int64_t)l * a.x_sl + h * a.x_sh + gq * 4);
    const float xf[4] = {__uint_as_float(xv.x << 16), __uint_as_float(xv.x & 0xffff0000u), __uint_as_float(xv.y << 16), __uint_as_float(xv.y & 0xffff0000u)};
#pragma unroll
    for (int q = 0; q < 4; ++q) y[q] = fmaf(a.D_has_hdim ? __ldg(a.D + h * a.P + gq * 4 + q) : __ldg(a.D + h), xf[q], y[q]);
  }
  const int64_t o = b * a.o_sb + (int64_t)l * a.o_sl + h * a.o_sh + gq * 4;
  if (a.has_z) {
    *(uint2*)(a.out_x + o) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
    const uint2 zv = *(const uint2*)(a.z + b * a.z_sb + (int64_t)l * a.z_sl + h * a.z_sh + gq * 4);
    const float zf[4] = {__uint_as_float(zv.x << 16), __uint_as_float(zv.x & 0xffff0000u), __uint_as_float(zv.y << 16), __uint_as_float(zv.y & 0xffff0000u)};
#pragma unroll
    for (int q = 0; q < 4; ++q) y[q] *= __fdividef(zf[q], 1.f + ex2f(-zf[q] * LOG2E));
  }
  *(uint2*)(a.out + o) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
}

TArgs make_targs(const issm_params& p) {
  TArgs a{};
  a.b = p.batch; a.L = p.seqlen; a.H = p.nheads; a.P = p.headdim; a.N = p.dstate; a.G = p.ngroups;
  a.hpg = p.nheads / p.ngroups; a.rev = p.reverse;
  a.has_D = p.has_D; a.D_has_hdim = p.D_has_hdim; a.has_z = p.has_z; a.has_bias = p.has_dt_bias;
  a.softplus = p.dt_softplus; a.has_init = p.has_init; a.want_final = p.want_final;
  a.dtmin = p.dt_min; a.dtmax = p.dt_max;
  a.x = (const bf16*)p.x; a.x_sb = p.x_sb; a.x_sl = p.x_sl; a.x_sh = p.x_sh;
  a.dt = p.dt; a.dt_sb = p.dt_sb; a.dt_sl = p.dt_sl; a.dt_sh = p.dt_sh;
  a.B = (const bf16*)p.B; a.B_sb = p.B_sb; a.B_sl = p.B_sl; a.B_sg = p.B_sg;
  a.C = (const bf16*)p.C; a.C_sb = p.C_sb; a.C_sl = p.C_sl; a.C_sg = p.C_sg;
  a.z = (const bf16*)p.z; a.z_sb = p.z_sb; a.z_sl = p.z_sl; a.z_sh = p.z_sh;
  a.A = p.A; a.D = p.D; a.bias = p.dt_bias; a.init = (const bf16*)p.initial_states;
  a.out = (bf16*)p.out; a.o_sb = p.out_sb; a.o_sl = p.out_sl; a.o_sh = p.out_sh;
  a.out_x = p.has_z ? (bf16*)p.out_x : nullptr;
  a.final_states = p.final_states;
  a.status = p.status;
  a.saved = (bf16*)p.saved_states;
  // a whole 64-row tile of B / C is one contiguous copy only when a row IS the tile's row (not a 256-state slice of it)
  a.bc_contig = (p.B_sl == p.dstate && p.C_sl == p.dstate && p.dstate <= 256);
  a.dt_tma = 0;
  return a;
}

// ---- tensor map over dt ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) { (void)cudaGetLastError(); f = nullptr; }
    return (EncodeTiledFn)f;
  }();
  return fn;
}

bool make_rows_tensor_map(const void* base, int64_t sb, int64_t sl, int64_t width, int batch, int seqlen, int box_w, CUtensorMap* out) {
  memset(out, 0, sizeof(*out));
  // rows (b, l) must form one regular array: batch stride = seqlen * row stride; 16-byte aligned rows
  if (!base || sb != (int64_t)seqlen * sl || (sl & 7) || ((uintptr_t)base & 15)) return false;
  if (width > sl || width < box_w || (uint64_t)batch * seqlen > 0x7fffffffull) return false;
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t gdim[2] = {(cuuint64_t)width, (cuuint64_t)batch * seqlen};
  const cuuint64_t gstride[1] = {(cuuint64_t)sl * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_w, (cuuint32_t)QB};
  const cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_dt_tensor_map(const issm_params& p, CUtensorMap* out) {
  memset(out, 0, sizeof(*out));
  if (p.dt_dtype != ISSM_BF16 || (p.dt_sh & 7)) return false;
  // one tile = one 256-state slice (or all 128 / 256 states) of one head, 64 rows
  return make_rows_tensor_map(p.dt, p.dt_sb, p.dt_sl, (int64_t)(p.nheads - 1) * p.dt_sh + p.dstate, p.batch, p.seqlen,
                              p.dstate > 256 ? 256 : p.dstate, out);
}

template <int NT, typename TDT, int kMode>
static int launch_fwd_mode(const TArgs& a, const FwdMaps& maps, cudaStream_t s) {
  const size_t smem = FwdSmem<NT>::kTotal + 1024;
  struct FastTag {};
  struct WinTag {};
  if (SmemAttrOnce<FastTag>::set(k_fwd_tensor<NT, TDT, false, kMode>, smem) != ISSM_OK ||
      SmemAttrOnce<WinTag>::set(k_fwd_tensor<NT, TDT, true, 0>, smem) != ISSM_OK)
    return ISSM_ERR_CUDA;
  const int slices = a.N / NT;
  ISSM_LAUNCH((k_fwd_tensor<NT, TDT, false, kMode>), dim3(slices, a.H, a.b), 2 * NT + 128, smem, s, a, maps);
  ISSM_LAUNCH((k_fwd_tensor<NT, TDT, true, 0>), dim3(slices, a.H, a.b), 2 * NT + 128, smem, s, a, maps);   // marked streams only
  if (slices > 1 && !a.no_output) {
    const size_t groups = (size_t)a.b * a.L * a.H * (a.P / 4);
    ISSM_LAUNCH(k_combine_slices, (unsigned)cdiv64(groups, 256), 256, 0, s, a, slices, groups);
  }
  return ISSM_OK;
}

template <int NT, typename TDT>
static int launch_fwd(TArgs a, const issm_params& p, cudaStream_t s) {
  FwdMaps maps;
  a.dt_tma = make_dt_tensor_map(p, &maps.dt) ? 1 : 0;
  // B / C rows that are not adjacent in memory (a 256-state slice of a wider row, the two halves of one projection
  // output): a 64-row tile is one tiled TMA load each when the rows form a regular 2-D array
  const int box = p.dstate > 256 ? 256 : p.dstate;
  a.bc_tma = (!a.bc_contig && !((p.B_sg | p.C_sg) & 7) &&
              make_rows_tensor_map(p.B, p.B_sb, p.B_sl, (int64_t)(p.ngroups - 1) * p.B_sg + p.dstate, p.batch, p.seqlen, box, &maps.B) &&
              make_rows_tensor_map(p.C, p.C_sb, p.C_sl, (int64_t)(p.ngroups - 1) * p.C_sg + p.dstate, p.batch, p.seqlen, box, &maps.C)) ? 1 : 0;
  if (!a.bc_tma) { memset(&maps.B, 0, sizeof(maps.B)); memset(&maps.C, 0, sizeof(maps.C)); }
  // whole-tile copies of dt (when it is staged at all) and of B / C: the row order of the staged tiles is known
  const bool tiles = (a.bc_contig || a.bc_tma) && (sizeof(TDT) != 2 || a.dt_tma);
  if (!tiles) return launch_fwd_mode<NT, TDT, 0>(a, maps, s);
  return a.rev ? launch_fwd_mode<NT, TDT, 2>(a, maps, s) : launch_fwd_mode<NT, TDT, 1>(a, maps, s);
}

int tensor_fwd(const issm_params& p, cudaStream_t s) {
  TArgs a = make_targs(p);
  a.redo = (int*)p.workspace;
  const int slices = state_slices(p.dstate);
  if (slices > 1) {
    a.ypart = (float*)((char*)p.workspace + align_up((size_t)slices * p.batch * p.nheads * sizeof(int), 256));
  }
  if (p.dstate != 128) return p.dt_dtype == ISSM_BF16 ? launch_fwd<256, bf16>(a, p, s) : launch_fwd<256, float>(a, p, s);
  return p.dt_dtype == ISSM_BF16 ? launch_fwd<128, bf16>(a, p, s) : launch_fwd<128, float>(a, p, s);
}

// forward walk that only regenerates the block-entry states (for a backward without saved states)
int tensor_fwd_states_only(const issm_params& p, bf16* saved, int* redo, cudaStream_t s) {
  TArgs a = make_targs(p);
  a.saved = saved;
  a.redo = redo;
  a.no_output = 1;
  a.want_final = 0;
  if (p.dstate != 128) return p.dt_dtype == ISSM_BF16 ? launch_fwd<256, bf16>(a, p, s) : launch_fwd<256, float>(a, p, s);
  return p.dt_dtype == ISSM_BF16 ? launch_fwd<128, bf16>(a, p, s) : launch_fwd<128, float>(a, p, s);
}

}  // namespace issm
