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
// Per-head dB / dC partials go to a bf16 workspace and are summed over heads by a second kernel.
#include "issm_tensor.cuh"

namespace issm {

template <int NT>
struct BwdSmem {
  static constexpr int kCd = 0;                         // [NT/64 atoms][64 l][128 B]
  static constexpr int kBd = kCd + NT * 128;
  static constexpr int kGop = kBd + NT * 128;           // [NT n][128 B]: g' rows, p contiguous (SW128)
  static constexpr int kSop = kGop + NT * 128;          // [PP/8][NT n][16 B]: S' rows (interleaved)
  static constexpr int kX = kSop + NT * (PP * 2);       // [64 l][128 B]
  static constexpr int kDy = kX + QB * 128;             // [64 l][128 B]
  static constexpr int kDMm = kDy + QB * 128;           // [64 l][128 B], s contiguous
  static constexpr int kMm = kDMm + QB * 128;           // [64 l][128 B]
  static constexpr int kDxT = kDMm;                     // [64][PP] float, aliases dMm + Mm after the MMAs
  static constexpr int kSdt = kMm + QB * 128;           // staging [64][NT] bf16
  static constexpr int kSB = kSdt + QB * NT * 2;
  static constexpr int kRed = kSdt;                     // [XR * NT] float: dD partial reduction (after the walk)
  static constexpr int kBars = kSB + QB * NT * 2;
  static constexpr int kTotal = kBars + 64;
};

template <int NT, typename TDT>
__global__ void __launch_bounds__(NT, 1) k_bwd_tensor(const TArgs a) {
  using SM = BwdSmem<NT>;
  constexpr bool kStageDt = sizeof(TDT) == 2;
  constexpr int XR = (QB * PP + NT - 1) / NT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bar1 = (uint64_t*)(smem + SM::kBars);
  uint64_t* bar2 = bar1 + 1;
  uint64_t* barS = bar1 + 2;     // dt staging
  uint64_t* barT = bar1 + 3;     // B staging
  uint32_t* tmem_holder = (uint32_t*)(bar1 + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, b = blockIdx.z, g = h / a.hpg;
  const int n = tid;
  const TDT* __restrict__ dtp = (const TDT*)a.dt + b * a.dt_sb + h * a.dt_sh;
  const bf16* __restrict__ Bp = a.B + b * a.B_sb + g * a.B_sg;
  const bf16* __restrict__ Cp = a.C + b * a.C_sb + g * a.C_sg + n;
  const bf16* __restrict__ xp = a.x + b * a.x_sb + h * a.x_sh;
  const bf16* __restrict__ zp = a.has_z ? a.z + b * a.z_sb + h * a.z_sh : nullptr;
  const bf16* __restrict__ yp = a.has_z ? a.out_x + b * a.o_sb + h * a.o_sh : nullptr;
  const bf16* __restrict__ gp = a.dout + b * a.g_sb + h * a.g_sh;
  const float A2 = __ldg(a.A + h * a.N + n) * LOG2E;
  const float Anat = __ldg(a.A + h * a.N + n);
  const float bias = a.has_bias ? __ldg(a.bias + h * a.N + n) : 0.f;
  const int nblk = (a.L + QB - 1) / QB;
  const size_t bh = (size_t)b * a.H + h;

  for (int i = tid; i < (SM::kSdt - SM::kGop) / 16; i += NT) ((uint4*)(smem + SM::kGop))[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) { mbar_init(bar1, 1); mbar_init(bar2, 1); mbar_init(barS, 1); mbar_init(barT, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const int slab = tid >> 7;
  const uint32_t t_dM = tmem, t_M = tmem + 64, t_dx = tmem;
  const uint32_t t_BDrow = tmem + lane_base + 128 + slab * 64;
  const uint32_t t_CDrow = tmem + lane_base + 256 + slab * 64;
  const uint32_t t_Grow = tmem + lane_base + 384 + slab * PP;

  auto prefetch_dt = [&](int blk) {      // warp 1
    if (!kStageDt) return;
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    if (lane == 0) mbar_expect_tx(barS, (uint32_t)rows * NT * 2);
    __syncwarp();
    for (int l = lane; l < rows; l += 32)
      bulk_g2s(smem + SM::kSdt + l * NT * 2, (const bf16*)dtp + (int64_t)trow(a, row0 + l) * a.dt_sl, NT * 2, barS);
  };
  auto prefetch_B = [&](int blk) {       // warp 2
    const int row0 = blk * QB, rows = min(QB, a.L - row0);
    if (lane == 0) mbar_expect_tx(barT, (uint32_t)rows * NT * 2);
    __syncwarp();
    for (int l = lane; l < rows; l += 32)
      bulk_g2s(smem + SM::kSB + l * NT * 2, Bp + (int64_t)trow(a, row0 + l) * a.B_sl, NT * 2, barT);
  };
  if (warp == 1) prefetch_dt(nblk - 1);
  if (warp == 2) prefetch_B(nblk - 1);

  // gradient of the running state, and the state leaving the block (bf16 pairs)
  float G[PP];
  uint32_t Snext[PP / 2];
  {
    const float* __restrict__ df = a.dfinal ? a.dfinal + (bh * a.P) * a.N + n : nullptr;
#pragma unroll
    for (int p = 0; p < PP; ++p) G[p] = (df && p < a.P) ? df[(size_t)p * a.N] : 0.f;
    const uint4* src = (const uint4*)(a.saved + ((bh * (nblk + 1) + nblk) * a.N + n) * PP);
#pragma unroll
    for (int c = 0; c < PP / 8; ++c) {
      const uint4 v = src[c];
      Snext[c * 4] = v.x; Snext[c * 4 + 1] = v.y; Snext[c * 4 + 2] = v.z; Snext[c * 4 + 3] = v.w;
    }
  }
  const int kcol = tid & 63;
  const int npt = (QB * a.P + NT - 1) / NT;
  float dDacc[XR];
#pragma unroll
  for (int k = 0; k < XR; ++k) dDacc[k] = 0.f;
  float dAacc = 0.f, dbacc = 0.f;
  bool failed = false;
  uint32_t unsafe = 0;

  for (int it = 0; it < nblk; ++it) {
    const int blk = nblk - 1 - it;
    const int row0 = blk * QB;
    const int rows = min(QB, a.L - row0);
    const uint32_t parity = it & 1;

    // ---- issue the global loads of this block's small tiles and of the entering state -----------
    bf16 xr[XR], gr[XR], zr[XR], yr[XR];
#pragma unroll
    for (int k = 0; k < XR; ++k) {
      xr[k] = gr[k] = zr[k] = yr[k] = __float2bfloat16_rn(0.f);
      const int i = tid + k * NT;
      if (k < npt && i < rows * a.P) {
        const int l = i / a.P, p = i - l * a.P;
        const int64_t mr = trow(a, row0 + l);
        xr[k] = xp[mr * a.x_sl + p];
        gr[k] = gp[mr * a.g_sl + p];
        if (zp) { zr[k] = zp[mr * a.z_sl + p]; yr[k] = yp[mr * a.o_sl + p]; }
      }
    }
    uint32_t Scur[PP / 2];
    {
      const uint4* src = (const uint4*)(a.saved + ((bh * (nblk + 1) + blk) * a.N + n) * PP);
#pragma unroll
      for (int c = 0; c < PP / 8; ++c) {
        const uint4 v = src[c];
        Scur[c * 4] = v.x; Scur[c * 4 + 1] = v.y; Scur[c * 4 + 2] = v.z; Scur[c * 4 + 3] = v.w;
      }
    }

    // ---- state bookkeeping that needs no decay: <S leaving the block, G>, and the S operand ----------
    float cst = 0.f;
#pragma unroll
    for (int q = 0; q < PP / 2; ++q) {
      cst = fmaf(__uint_as_float(Snext[q] << 16), G[2 * q], cst);
      cst = fmaf(__uint_as_float(Snext[q] & 0xffff0000u), G[2 * q + 1], cst);
    }
#pragma unroll
    for (int c = 0; c < PP / 8; ++c)
      *(uint4*)(smem + SM::kSop + c * (NT * 16) + tid * 16) = make_uint4(Scur[c * 4], Scur[c * 4 + 1], Scur[c * 4 + 2], Scur[c * 4 + 3]);

    if (kStageDt && !mbar_wait(barS, parity)) failed = true;
    if (!mbar_wait(barT, parity)) failed = true;

    // ---- one pass over the rows: dt transform, cumulative decay, this column of Cd and Bd ----------
    // (C comes straight from global memory: L2-resident, shared by the heads of a sample)
    const float alast = build_operands<NT, TDT, kStageDt, false>(
        a, rows, row0, kcol, (const bf16*)(smem + SM::kSdt) + n, dtp + n, (const bf16*)(smem + SM::kSB) + n,
        nullptr, Cp, smem + SM::kCd + (tid >> 6) * (QB * 128), smem + SM::kBd + (tid >> 6) * (QB * 128), A2, bias);
    if (fabsf(alast) > 120.f) unsafe = 1;

    // ---- g' = 2^(a_last) G: fp32 copy parked in TMEM for the accumulate MMA, bf16 copy as operand ----
    {
      const float eg = ex2f(alast);
      float gs[PP];
#pragma unroll
      for (int p = 0; p < PP; ++p) gs[p] = G[p] * eg;
      tmem_st16(t_Grow, gs);
      tmem_st16(t_Grow + 16, gs + 16);
      tmem_st16(t_Grow + 32, gs + 32);
#pragma unroll
      for (int c = 0; c < PP / 8; ++c)
        *(uint4*)(smem + SM::kGop + sw128_chunk(tid, c)) =
            make_uint4(pack_bf16(gs[c * 8], gs[c * 8 + 1]), pack_bf16(gs[c * 8 + 2], gs[c * 8 + 3]),
                       pack_bf16(gs[c * 8 + 4], gs[c * 8 + 5]), pack_bf16(gs[c * 8 + 6], gs[c * 8 + 7]));
      tmem_st_wait();
    }

    // ---- x and dy tiles, dz, dD partials -------------------------------------------------------------
#pragma unroll
    for (int k = 0; k < XR; ++k) {
      const int i = tid + k * NT;
      if (k < npt && i < QB * a.P) {
        const int l = i / a.P, p = i - l * a.P;
        const float xv = __bfloat162float(xr[k]);
        float dy = __bfloat162float(gr[k]);
        if (zp) {
          const float zv = __bfloat162float(zr[k]);
          const float sg = 1.f / (1.f + ex2f(-zv * LOG2E));
          if (i < rows * a.P)
            a.dz[(((size_t)b * a.L + trow(a, row0 + l)) * a.H + h) * a.P + p] =
                __float2bfloat16_rn(dy * __bfloat162float(yr[k]) * sg * (1.f + zv * (1.f - sg)));
          dy *= zv * sg;
        }
        const bf16 dyb = __float2bfloat16_rn(dy);
        dDacc[k] = fmaf(__bfloat162float(dyb), xv, dDacc[k]);
        *(bf16*)(smem + SM::kX + sw128_off(l, p)) = xr[k];
        *(bf16*)(smem + SM::kDy + sw128_off(l, p)) = dyb;
      }
    }
    fence_async_smem();
    fence_before_sync();
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- MMA phase 1: dM = dy x^T, M = Cd Bd^T ---------------------------------------------------
    if (tid == 0) {
      fence_after_sync();
      const uint32_t sb = smem_u32(smem);
#pragma unroll
      for (int kk = 0; kk < PP / 16; ++kk)
        mma_bf16(t_dM, desc_sw128(sb + SM::kDy + kk * 32), desc_sw128(sb + SM::kX + kk * 32), idesc_bf16(64, 64), kk != 0);
#pragma unroll
      for (int at = 0; at < NT / 64; ++at)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t ko = at * (QB * 128) + kk * 32;
          mma_bf16(t_M, desc_sw128(sb + SM::kCd + ko), desc_sw128(sb + SM::kBd + ko), idesc_bf16(64, 64), (at | kk) != 0);
        }
      mma_commit(bar1);
    }
    if (!mbar_wait(bar1, parity)) failed = true;
    fence_after_sync();

    // ---- epilogue 1: causal masks, bf16 operands dMm[l][s], Mm[l][s] --------------------------------
    if (warp < 4 && !failed) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        float mv[64];
        const uint32_t t0 = (which ? t_M : t_dM) + lane_base;
        tmem_ld16(t0, mv);
        tmem_ld16(t0 + 16, mv + 16);
        tmem_ld16(t0 + 32, mv + 32);
        tmem_ld16(t0 + 48, mv + 48);
        tmem_ld_wait();
        if (lane < 16) {
          const int l = warp * 16 + lane;
          uint8_t* dst = smem + (which ? SM::kMm : SM::kDMm);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const int s = c * 8 + j;
              pk[j >> 1] = pack_bf16(s <= l ? mv[s] : 0.f, s + 1 <= l ? mv[s + 1] : 0.f);
            }
            *(uint4*)(dst + sw128_chunk(l, c)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
    }
    fence_async_smem();
    fence_before_sync();
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- MMA phase 2 ----------------------------------------------------------------------------------
    if (tid == 0) {
      fence_after_sync();
      const uint32_t sb = smem_u32(smem);
#pragma unroll
      for (int sl = 0; sl < NT / 128; ++sl) {
        const uint32_t dBD = tmem + 128 + sl * 64, dCD = tmem + 256 + sl * 64, dG = tmem + 384 + sl * PP;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {                 // K = rows of the block
          const uint64_t aCd = desc_sw128_mn(sb + SM::kCd + sl * (2 * QB * 128) + kk * 2048, QB * 128);
          const uint64_t aBd = desc_sw128_mn(sb + SM::kBd + sl * (2 * QB * 128) + kk * 2048, QB * 128);
          mma_bf16(dBD, aCd, desc_sw128_mn(sb + SM::kDMm + kk * 2048, QB * 128), idesc_bf16(128, 64, 1, 1), kk != 0);
          mma_bf16(dCD, aBd, desc_sw128(sb + SM::kDMm + kk * 32), idesc_bf16(128, 64, 1, 0), kk != 0);
          mma_bf16(dG, aCd, desc_sw128_mn(sb + SM::kDy + kk * 2048, QB * 128), idesc_bf16(128, PP, 1, 1), 1);
        }
#pragma unroll
        for (int kk = 0; kk < PP / 16; ++kk) {           // K = head dim
          mma_bf16(dBD, desc_sw128(sb + SM::kGop + sl * (128 * 128) + kk * 32), desc_sw128(sb + SM::kX + kk * 32),
                   idesc_bf16(128, 64), 1);
          mma_bf16(dCD, desc_interleave(sb + SM::kSop + sl * (128 * 16) + kk * 2 * (NT * 16), NT * 16, 128),
                   desc_sw128(sb + SM::kDy + kk * 32), idesc_bf16(128, 64), 1);
        }
      }
#pragma unroll
      for (int at = 0; at < NT / 64; ++at)               // dx: K = states
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(t_dx, desc_sw128(sb + SM::kBd + at * (QB * 128) + kk * 32),
                   desc_sw128_mn(sb + SM::kGop + (at * 4 + kk) * 2048, QB * 128), idesc_bf16(64, PP, 0, 1), (at | kk) != 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)                     // dx: K = later rows
        mma_bf16(t_dx, desc_sw128_mn(sb + SM::kMm + kk * 2048, QB * 128), desc_sw128_mn(sb + SM::kDy + kk * 2048, QB * 128),
                 idesc_bf16(64, PP, 1, 1), 1);
      mma_commit(bar2);
    }
    if (!mbar_wait(bar2, parity)) failed = true;
    fence_after_sync();

    // ---- epilogue 2 ------------------------------------------------------------------------------------
    if (!failed) {
      // (a) the owner of state column n: dB_h, dC_h, ddt, in-block reverse cumsum of dacs
      const bf16* sB = (const bf16*)(smem + SM::kSB) + n;
      const bf16* sdt = (const bf16*)(smem + SM::kSdt) + n;
      const uint8_t* cd_col = smem + SM::kCd + (tid >> 6) * (QB * 128);
      const uint8_t* bd_col = smem + SM::kBd + (tid >> 6) * (QB * 128);
      float total = 0.f;                                  // sum over the block of dacs = Cd CD - Bd BD
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        float bdv[16], cdv[16];
        tmem_ld16(t_BDrow + ch * 16, bdv);
        tmem_ld16(t_CDrow + ch * 16, cdv);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t off = (uint32_t)((ch * 16 + j) * 128 + ((((kcol >> 3) ^ (j & 7)) << 4) | ((kcol & 7) << 1)));
          total = fmaf(__bfloat162float(*(const bf16*)(cd_col + off)), cdv[j], total);
          total = fmaf(-__bfloat162float(*(const bf16*)(bd_col + off)), bdv[j], total);
        }
      }
      float prefix = 0.f, ac = 0.f;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        float bdv[16], cdv[16];
        tmem_ld16(t_BDrow + ch * 16, bdv);
        tmem_ld16(t_CDrow + ch * 16, cdv);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int l = ch * 16 + j;
          const bool valid = l < rows;
          const int64_t mr = trow(a, row0 + min(l, rows - 1));
          const float raw = kStageDt ? __bfloat162float(sdt[l * NT]) : ldf(dtp + mr * a.dt_sl + n);
          bool clamped = false;
          const float dtl = valid ? dt_transform(a, raw, bias, clamped) : 0.f;
          ac = fmaf(dtl, A2, ac);
          const float bd = ex2f(-ac) * bdv[j], cd = ex2f(ac) * cdv[j];
          const uint32_t off = (uint32_t)(l * 128 + ((((kcol >> 3) ^ (j & 7)) << 4) | ((kcol & 7) << 1)));
          const float dacs = __bfloat162float(*(const bf16*)(cd_col + off)) * cdv[j] -
                             __bfloat162float(*(const bf16*)(bd_col + off)) * bdv[j];
          const float ddA = cst + total - prefix;          // sum of dacs over rows >= l, plus <S_next, G>
          prefix += dacs;
          float gd = fmaf(ddA, Anat, __bfloat162float(sB[l * NT]) * bd);
          if (clamped) gd = 0.f;
          else if (a.softplus) gd *= 1.f - ex2f(-dtl * LOG2E);
          dAacc = fmaf(ddA, dtl, dAacc);
          if (valid) {
            dbacc += gd;
            const size_t o = (((size_t)b * a.L + mr) * a.H + h) * a.N + n;
            stf((TDT*)a.ddt + o, gd);
            a.dBh[o] = __float2bfloat16_rn(dtl * bd);
            a.dCh[o] = __float2bfloat16_rn(cd);
          }
        }
      }
      // (b) new state gradient
      {
        float gs[PP];
        tmem_ld16(t_Grow, gs);
        tmem_ld16(t_Grow + 16, gs + 16);
        tmem_ld16(t_Grow + 32, gs + 32);
        tmem_ld_wait();
#pragma unroll
        for (int p = 0; p < PP; ++p) G[p] = gs[p];
      }
#pragma unroll
      for (int q = 0; q < PP / 2; ++q) Snext[q] = Scur[q];
      // (c) dx rows -> shared memory
      if (warp < 4) {
        float dv[PP];
        tmem_ld16(t_dx + lane_base, dv);
        tmem_ld16(t_dx + lane_base + 16, dv + 16);
        tmem_ld16(t_dx + lane_base + 32, dv + 32);
        tmem_ld_wait();
        if (lane < 16) {
          float4* dst = (float4*)(smem + SM::kDxT + (warp * 16 + lane) * PP * 4);
#pragma unroll
          for (int c = 0; c < PP / 4; ++c) dst[c] = make_float4(dv[c * 4], dv[c * 4 + 1], dv[c * 4 + 2], dv[c * 4 + 3]);
        }
      }
    }
    fence_before_sync();
    if (__syncthreads_or(failed)) { failed = true; break; }
    if (warp == 1 && blk > 0) prefetch_dt(blk - 1);       // every thread is past its dt / B staging reads
    if (warp == 2 && blk > 0) prefetch_B(blk - 1);

    // ---- coalesced dx store: dx = tile + D dy --------------------------------------------------------
#pragma unroll
    for (int k = 0; k < XR; ++k) {
      const int i = tid + k * NT;
      if (k < npt && i < rows * a.P) {
        const int l = i / a.P, p = i - l * a.P;
        float v = *(const float*)(smem + SM::kDxT + (l * PP + p) * 4);
        if (a.has_D) v = fmaf(a.D_has_hdim ? __ldg(a.D + h * a.P + p) : __ldg(a.D + h),
                              __bfloat162float(*(const bf16*)(smem + SM::kDy + sw128_off(l, p))), v);
        a.dx[(((size_t)b * a.L + trow(a, row0 + l)) * a.H + h) * a.P + p] = __float2bfloat16_rn(v);
      }
    }
    // the tile buffers are rewritten only after the next block's first barrier, but the dx tile aliases
    // the masked-matrix operands that epilogue 1 of the next block writes: keep the readers ahead
    __syncthreads();
  }

  if (!failed) {
    if (a.dinit) {
      bf16* dp = a.dinit + (bh * a.P) * a.N + n;
#pragma unroll
      for (int p = 0; p < PP; ++p)
        if (p < a.P) dp[(size_t)p * a.N] = __float2bfloat16_rn(G[p]);
    }
    a.dApart[bh * a.N + n] = dAacc;
    a.dbpart[bh * a.N + n] = dbacc;
    // dD partials: element k of thread t always has p = (t + k NT) % P; fixed-order sum per p
    float* red = (float*)(smem + SM::kRed);
#pragma unroll
    for (int k = 0; k < XR; ++k) red[k * NT + tid] = (k < npt) ? dDacc[k] : 0.f;
    __syncthreads();
    if (tid < a.P) {
      float s = 0.f;
      for (int i = 0; i < npt * NT; ++i)
        if (i < QB * a.P && i % a.P == tid) s += red[(i / NT) * NT + (i % NT)];
      a.dDpart[bh * PP + tid] = s;
    }
  }
  if (a.status) {
    if (failed && tid == 0) atomicOr(a.status, 1);
    if (unsafe) atomicOr(a.status, 2);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// dB[b,l,g,n] = sum over the heads of group g of the bf16 per-head partials
__global__ void k_reduce_heads_bf16(int hpg, int N, int H, size_t total, const bf16* __restrict__ part, bf16* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // over (b, l, g, n/8)
  if (i >= total) return;
  const int n8 = N / 8;
  const size_t blg = i / n8;
  const int c = i % n8;
  const int G = H / hpg;
  const size_t bl = blg / G;
  const int g = blg % G;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int k = 0; k < hpg; ++k) {
    const uint4 v = *(const uint4*)(part + ((bl * H + g * hpg + k) * N) + c * 8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] += __uint_as_float(w[j] << 16);
      acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  *(uint4*)(out + blg * N + c * 8) = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]),
                                                pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
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
  bf16 *dBh, *dCh, *saved;
  float *dApart, *dbpart, *dDpart;
};

static BwdWs carve_bwd(const issm_params& p, size_t* total) {
  Carver c(p.workspace);
  BwdWs w{};
  const size_t b = p.batch, L = p.seqlen, H = p.nheads, N = p.dstate;
  const size_t nblk = (L + QB - 1) / QB;
  w.dBh = c.take<bf16>(b * L * H * N);
  w.dCh = c.take<bf16>(b * L * H * N);
  w.dApart = c.take<float>(b * H * N);
  w.dbpart = c.take<float>(b * H * N);
  w.dDpart = c.take<float>(b * H * PP);
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

template <int NT, typename TDT>
static int launch_bwd(const TArgs& a, cudaStream_t s) {
  const size_t smem = BwdSmem<NT>::kTotal + 1024;
  if (cudaFuncSetAttribute(k_bwd_tensor<NT, TDT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return ISSM_ERR_CUDA;
  }
  ISSM_LAUNCH((k_bwd_tensor<NT, TDT>), dim3(1, a.H, a.b), NT, smem, s, a);
  return ISSM_OK;
}

int tensor_bwd(const issm_params& p, cudaStream_t s) {
  size_t total = 0;
  const BwdWs w = carve_bwd(p, &total);
  bf16* saved = (bf16*)p.saved_states;
  if (!saved) {                                           // recompute the block-entry states (reference: issm_combined.py:136-144)
    saved = w.saved;
    int rc = tensor_fwd_states_only(p, saved, s);
    if (rc) return rc;
  }
  TArgs a = make_targs(p);
  a.saved = saved;
  a.out_x = p.has_z ? (bf16*)p.out_x : nullptr;
  a.dout = (const bf16*)p.dout; a.g_sb = p.dout_sb; a.g_sl = p.dout_sl; a.g_sh = p.dout_sh;
  a.dfinal = p.has_dfinal ? p.dfinal_states : nullptr;
  a.dx = (bf16*)p.dx; a.ddt = p.ddt; a.dz = (bf16*)p.dz; a.dinit = (bf16*)p.dinitial_states;
  a.dBh = w.dBh; a.dCh = w.dCh; a.dApart = w.dApart; a.dbpart = w.dbpart; a.dDpart = w.dDpart;
  int rc;
  if (p.dstate == 256) rc = p.dt_dtype == ISSM_BF16 ? launch_bwd<256, bf16>(a, s) : launch_bwd<256, float>(a, s);
  else rc = p.dt_dtype == ISSM_BF16 ? launch_bwd<128, bf16>(a, s) : launch_bwd<128, float>(a, s);
  if (rc) return rc;
  const int hpg = p.nheads / p.ngroups;
  const size_t tot = (size_t)p.batch * p.seqlen * p.ngroups * (p.dstate / 8);
  ISSM_LAUNCH(k_reduce_heads_bf16, (unsigned)cdiv64(tot, 256), 256, 0, s, hpg, p.dstate, p.nheads, tot, w.dBh, (bf16*)p.dB);
  ISSM_LAUNCH(k_reduce_heads_bf16, (unsigned)cdiv64(tot, 256), 256, 0, s, hpg, p.dstate, p.nheads, tot, w.dCh, (bf16*)p.dC);
  const int HN = p.nheads * p.dstate;
  ISSM_LAUNCH(k_reduce_batch, (HN + 127) / 128, 128, 0, s, w.dApart, p.batch, HN, p.dA);
  if (p.has_dt_bias) ISSM_LAUNCH(k_reduce_batch, (HN + 127) / 128, 128, 0, s, w.dbpart, p.batch, HN, p.ddt_bias);
  if (p.has_D) {
    const int cnt = p.D_has_hdim ? p.nheads * p.headdim : p.nheads;
    ISSM_LAUNCH(k_reduce_dD, (cnt + 63) / 64, 64, 0, s, w.dDpart, p.batch, p.nheads, p.headdim, p.D_has_hdim, p.dD);
  }
  return ISSM_OK;
}

}  // namespace issm
