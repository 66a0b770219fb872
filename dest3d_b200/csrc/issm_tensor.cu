// tcgen05 tensor-core path of the ISSM scan (bf16 activations, fp32 accumulation in TMEM).
//
// One CTA walks one (batch, head) stream along the sequence in sub-blocks of 64 points; thread t of
// the CTA owns state column n = t for the whole walk: it transforms dt, keeps the running
// cumulative decay of its column, builds its column of every MMA operand, and owns TMEM lane
// t % 128 of the running state S[n, p] (fp32).  Per sub-block (rows l, s of the block; a = cumsum
// of dt*A inside the block, r = a at mid-block, a_last = a at the end):
//   M[l,s]  = sum_n (C e^{a[l]-r})[l,n] (B dt e^{r-a[s]})[s,n]         tcgen05.mma  64 x 64, K = N
//   Y[l,p]  = sum_n (C e^{a[l]})[l,n] S[p,n] + sum_{s<=l} M[l,s] x[s,p]  tcgen05.mma  64 x 48, K = N, 64
//   S[n,p]  = e^{a_last[n]} S[n,p] + sum_l (B dt e^{a_last-a[l]})[l,n] x[l,p]   tcgen05.mma 128 x 48, K = 64
// which is the chunked algorithm of issm_triton/issm_combined.py:57-92 (chunk state, state passing,
// C.A.B^T, chunk scan) with a 64-row chunk, the state carried on chip instead of through HBM, and
// the decay inside the contraction factored through the mid-block reference so that both factors
// stay in range (half-span up to 120 in log2 units; beyond that the status word gets bit 2).
#include "issm_common.cuh"
#include "umma.cuh"

namespace issm {
using namespace umma;

constexpr int QB = 64;   // rows per sub-block
constexpr int PP = 48;   // head dim padded to an MMA-legal N
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct TArgs {
  int b, L, H, P, N, G, hpg, rev;
  int has_D, D_has_hdim, has_z, has_bias, softplus, has_init, want_final;
  float dtmin, dtmax;
  const bf16* x; int64_t x_sb, x_sl, x_sh;
  const void* dt; int64_t dt_sb, dt_sl, dt_sh;
  const bf16* B; int64_t B_sb, B_sl, B_sg;
  const bf16* C; int64_t C_sb, C_sl, C_sg;
  const bf16* z; int64_t z_sb, z_sl, z_sh;
  const float* A; const float* D; const float* bias;
  const bf16* init;
  bf16* out; int64_t o_sb, o_sl, o_sh;
  bf16* out_x;
  float* final_states;
  int* status;
};

template <int NT>
struct FwdSmem {
  static constexpr int kCs = 0;
  static constexpr int kCd = kCs + NT * 128;
  static constexpr int kBd = kCd + NT * 128;
  static constexpr int kBhT = kBd + NT * 128;
  static constexpr int kSop = kBhT + NT * 128;
  static constexpr int kXT = kSop + NT * (PP * 2);
  static constexpr int kMm = kXT + PP * 128;
  static constexpr int kBars = kMm + QB * 128;
  static constexpr int kTotal = kBars + 64;
};

__device__ __forceinline__ int trow(const TArgs& a, int t) { return a.rev ? a.L - 1 - t : t; }

__device__ __forceinline__ float softplus_fast(float v) {
  // softplus with the reference's threshold; log2-domain hardware approximations
  return v <= 20.f ? lg2f(1.f + ex2f(v * LOG2E)) * LN2 : v;
}

template <int NT, typename TDT>
__global__ void __launch_bounds__(NT, 1) k_fwd_tensor(const TArgs a) {
  using SM = FwdSmem<NT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* barA = (uint64_t*)(smem + SM::kBars);
  uint64_t* barB = barA + 1;
  uint32_t* tmem_holder = (uint32_t*)(barA + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, b = blockIdx.z, g = h / a.hpg;
  const int n = blockIdx.x * NT + tid;
  const TDT* dtp = (const TDT*)a.dt + b * a.dt_sb + h * a.dt_sh + n;
  const bf16* Bp = a.B + b * a.B_sb + g * a.B_sg + n;
  const bf16* Cp = a.C + b * a.C_sb + g * a.C_sg + n;
  const bf16* xp = a.x + b * a.x_sb + h * a.x_sh;
  const float A2 = a.A[h * a.N + n] * LOG2E;
  const float bias = a.has_bias ? a.bias[h * a.N + n] : 0.f;

  // one-time setup: zero the padded operand tiles, barriers, TMEM
  for (int i = tid; i < (SM::kBars - SM::kSop) / 16; i += NT) ((uint4*)(smem + SM::kSop))[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) { mbar_init(barA, 1); mbar_init(barB, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(tmem_holder, 256); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_holder;
  const uint32_t t_M = tmem, t_Y = tmem + 64;
  const uint32_t t_Srow = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 128 + (tid >> 7) * PP;   // this thread's lane
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

  float Srow[PP];
#pragma unroll
  for (int p = 0; p < PP; ++p) Srow[p] = 0.f;
  if (a.has_init) {
    const bf16* ip = a.init + (((size_t)b * a.H + h) * a.P) * a.N + n;
#pragma unroll
    for (int p = 0; p < PP; ++p)
      if (p < a.P) Srow[p] = __bfloat162float(ip[(size_t)p * a.N]);
  }
  uint8_t* sop_col = smem + SM::kSop + (tid >> 6) * (PP * 128);
#pragma unroll
  for (int p = 0; p < PP; ++p) *(bf16*)(sop_col + sw128_off(p, tid & 63)) = __float2bfloat16_rn(Srow[p]);

  const int nblk = (a.L + QB - 1) / QB;
  bool failed = false;
  uint32_t unsafe = 0;
  for (int blk = 0; blk < nblk; ++blk) {
    const int row0 = blk * QB;
    const int rows = min(QB, a.L - row0);
    const uint32_t parity = blk & 1;

    // ---- stage x^T (K-major over l) -------------------------------------------------------
    for (int i = tid; i < QB * a.P; i += NT) {
      const int l = i / a.P, p = i - l * a.P;
      bf16 v = __float2bfloat16_rn(0.f);
      if (l < rows) v = xp[(int64_t)trow(a, row0 + l) * a.x_sl + p];
      *(bf16*)(smem + SM::kXT + sw128_off(p, l)) = v;
    }

    // ---- pass 1: dt transform, cumulative log2-decay, references -----------------------------
    float dtv[QB];
    float acc = 0.f, r = 0.f;
#pragma unroll
    for (int l = 0; l < QB; ++l) {
      float v = 0.f;
      if (l < rows) {
        v = ldf(dtp + (int64_t)trow(a, row0 + l) * a.dt_sl) + bias;
        if (a.softplus) v = softplus_fast(v);
        v = fminf(fmaxf(v, a.dtmin), a.dtmax);
      }
      dtv[l] = v;
      acc = fmaf(v, A2, acc);
      if (l == QB / 2 - 1) r = acc;
    }
    const float alast = acc;
    if (fabsf(r) > 120.f || fabsf(alast - r) > 120.f) unsafe = 1;

    // ---- running state: S <- e^{a_last} S, parked in TMEM for the accumulate MMA -------------
    {
      const float decay = ex2f(alast);
#pragma unroll
      for (int p = 0; p < PP; ++p) Srow[p] *= decay;
      tmem_st16(t_Srow, Srow);
      tmem_st16(t_Srow + 16, Srow + 16);
      tmem_st16(t_Srow + 32, Srow + 32);
      tmem_st_wait();
    }

    // ---- pass 2: this column of every operand ------------------------------------------------
    {
      uint8_t* cs_col = smem + SM::kCs + (tid >> 6) * (QB * 128);
      uint8_t* cd_col = smem + SM::kCd + (tid >> 6) * (QB * 128);
      uint8_t* bd_col = smem + SM::kBd + (tid >> 6) * (QB * 128);
      uint8_t* bh_row = smem + SM::kBhT;
      const int k = tid & 63;
      acc = 0.f;
#pragma unroll
      for (int l0 = 0; l0 < QB; l0 += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int l = l0 + j;
          float cv = 0.f, bv = 0.f;
          if (l < rows) {
            const int64_t mr = trow(a, row0 + l);
            cv = __bfloat162float(Cp[mr * a.C_sl]);
            bv = __bfloat162float(Bp[mr * a.B_sl]);
          }
          acc = fmaf(dtv[l], A2, acc);
          const float bdt = bv * dtv[l];
          const float cs = cv * ex2f(acc);
          const float cd = cv * ex2f(acc - r);
          const float bh = bdt * ex2f(alast - acc);
          const float bd = bdt * ex2f(r - acc);
          const uint32_t off = sw128_off(l, k);
          *(bf16*)(cs_col + off) = __float2bfloat16_rn(cs);
          *(bf16*)(cd_col + off) = __float2bfloat16_rn(cd);
          *(bf16*)(bd_col + off) = __float2bfloat16_rn(bd);
          const uint32_t hb = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(bh));
          if (j & 1) packed[j >> 1] |= hb << 16; else packed[j >> 1] = hb;
        }
        *(uint4*)(bh_row + sw128_chunk(tid, l0 >> 3)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
    fence_async_smem();
    fence_before_sync();
    __syncthreads();

    // ---- MMAs: M = Cd Bd^T, Y = Cs S^T, S += BhT^T x^T ------------------------------------------
    if (tid == 0) {
      fence_after_sync();
      const uint32_t sb = smem_u32(smem);
#pragma unroll
      for (int at = 0; at < NT / 64; ++at)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t ko = at * (QB * 128) + kk * 32;
          mma_bf16(t_M, desc_sw128(sb + SM::kCd + ko), desc_sw128(sb + SM::kBd + ko), idesc_bf16(64, 64), (at | kk) != 0);
          mma_bf16(t_Y, desc_sw128(sb + SM::kCs + ko), desc_sw128(sb + SM::kSop + at * (PP * 128) + kk * 32),
                   idesc_bf16(64, PP), (at | kk) != 0);
        }
#pragma unroll
      for (int sl = 0; sl < NT / 128; ++sl)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(tmem + 128 + sl * PP, desc_sw128(sb + SM::kBhT + sl * (128 * 128) + kk * 32),
                   desc_sw128(sb + SM::kXT + kk * 32), idesc_bf16(128, PP), 1);
      mma_commit(barA);
    }
    if (!mbar_wait(barA, parity)) failed = true;
    if (__syncthreads_or(failed)) { failed = true; break; }
    fence_after_sync();

    // ---- epilogue 1: masked M -> bf16 operand; new state -> registers and bf16 operand --------
    if (warp < 4) {
      float mv[64];
      tmem_ld16(t_M + lane_base, mv);
      tmem_ld16(t_M + lane_base + 16, mv + 16);
      tmem_ld16(t_M + lane_base + 32, mv + 32);
      tmem_ld16(t_M + lane_base + 48, mv + 48);
      tmem_ld_wait();
      if (lane < 16) {
        const int l = warp * 16 + lane;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const int s = c * 8 + j;
            const float v0 = s <= l ? mv[s] : 0.f, v1 = s + 1 <= l ? mv[s + 1] : 0.f;
            pk[j >> 1] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v0)) |
                         ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v1)) << 16);
          }
          *(uint4*)(smem + SM::kMm + sw128_chunk(l, c)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
    }
    tmem_ld16(t_Srow, Srow);
    tmem_ld16(t_Srow + 16, Srow + 16);
    tmem_ld16(t_Srow + 32, Srow + 32);
    tmem_ld_wait();
#pragma unroll
    for (int p = 0; p < PP; ++p) *(bf16*)(sop_col + sw128_off(p, tid & 63)) = __float2bfloat16_rn(Srow[p]);
    fence_async_smem();
    fence_before_sync();
    __syncthreads();

    // ---- Y += tril(M) x ------------------------------------------------------------------------
    if (tid == 0) {
      fence_after_sync();
      const uint32_t sb = smem_u32(smem);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        mma_bf16(t_Y, desc_sw128(sb + SM::kMm + kk * 32), desc_sw128(sb + SM::kXT + kk * 32), idesc_bf16(64, PP), 1);
      mma_commit(barB);
    }
    if (!mbar_wait(barB, parity)) failed = true;
    if (__syncthreads_or(failed)) { failed = true; break; }
    fence_after_sync();

    // ---- epilogue 2: D skip, gate, store -----------------------------------------------------
    if (warp < 4) {
      float yv[PP];
      tmem_ld16(t_Y + lane_base, yv);
      tmem_ld16(t_Y + lane_base + 16, yv + 16);
      tmem_ld16(t_Y + lane_base + 32, yv + 32);
      tmem_ld_wait();
      const int l = warp * 16 + lane;
      if (lane < 16 && l < rows) {
        const int64_t mr = trow(a, row0 + l);
        const bf16* xr = xp + mr * a.x_sl;
        bf16* orow = a.out + b * a.o_sb + mr * a.o_sl + h * a.o_sh;
        bf16* oxr = a.out_x ? a.out_x + b * a.o_sb + mr * a.o_sl + h * a.o_sh : nullptr;
        const bf16* zr = a.has_z ? a.z + b * a.z_sb + mr * a.z_sl + h * a.z_sh : nullptr;
#pragma unroll
        for (int p = 0; p < PP; ++p) {
          if (p < a.P) {
            float y = yv[p];
            if (a.has_D) y = fmaf(a.D_has_hdim ? a.D[h * a.P + p] : a.D[h], __bfloat162float(xr[p]), y);
            if (zr) {
              oxr[p] = __float2bfloat16_rn(y);
              const float zv = __bfloat162float(zr[p]);
              y *= zv / (1.f + ex2f(-zv * LOG2E));
            }
            orow[p] = __float2bfloat16_rn(y);
          }
        }
      }
    }
    fence_before_sync();
  }

  if (!failed && a.want_final) {
    float* fp = a.final_states + (((size_t)b * a.H + h) * a.P) * a.N + n;
#pragma unroll
    for (int p = 0; p < PP; ++p)
      if (p < a.P) fp[(size_t)p * a.N] = Srow[p];
  }
  if (a.status) {
    if (failed && tid == 0) atomicOr(a.status, 1);
    if (unsafe) atomicOr(a.status, 2);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------
bool tensor_path_supported(const issm_params& p) {
  if (p.io_dtype != ISSM_BF16) return false;
  if (p.headdim > PP) return false;
  if (p.dstate != 128 && p.dstate != 256) return false;
  return true;
}

size_t tensor_workspace_bytes(const issm_params& p, int pass) {
  return pass == 0 ? 0 : simt_workspace_bytes(p, pass);
}

static TArgs make_targs(const issm_params& p) {
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
  return a;
}

template <int NT, typename TDT>
static int launch_fwd(const TArgs& a, cudaStream_t s) {
  const size_t smem = FwdSmem<NT>::kTotal + 1024;
  if (cudaFuncSetAttribute(k_fwd_tensor<NT, TDT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return ISSM_ERR_CUDA;
  }
  ISSM_LAUNCH((k_fwd_tensor<NT, TDT>), dim3(a.N / NT, a.H, a.b), NT, smem, s, a);
  return ISSM_OK;
}

int tensor_fwd(const issm_params& p, cudaStream_t s) {
  const TArgs a = make_targs(p);
  if (p.dstate == 256) return p.dt_dtype == ISSM_BF16 ? launch_fwd<256, bf16>(a, s) : launch_fwd<256, float>(a, s);
  return p.dt_dtype == ISSM_BF16 ? launch_fwd<128, bf16>(a, s) : launch_fwd<128, float>(a, s);
}

int tensor_bwd(const issm_params& p, cudaStream_t s) {
  // the backward still runs on the SIMT kernels (same workspace layout)
  return simt_bwd(p, s);
}

}  // namespace issm
