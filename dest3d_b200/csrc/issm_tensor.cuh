// Declarations shared by the forward and backward kernels of the tcgen05 ISSM path.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "issm_common.cuh"
#include "umma.cuh"

namespace issm {
using namespace umma;

constexpr int QB = 64;   // rows per sub-block
constexpr int PP = 48;   // head dim padded to an MMA-legal N
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// device-side view of one call (forward fields first, backward fields last)
struct TArgs {
  int b, L, H, P, N, G, hpg, rev;
  int has_D, D_has_hdim, has_z, has_bias, softplus, has_init, want_final, no_output;
  bf16* wscr;       // backward, windowed kernel: (batch, nheads, 63, state) bf16 window-entry states of the block in progress
  int* redo;        // (batch, nheads) marks: stream holds a block outside the fast kernel's range, redo it windowed
  bf16* dxpart;     // backward with state slices: (slice, b, L, H, P) bf16 partial dx rows (before the D skip)
  float* ypart;     // forward with the states cut into slices of 256 (dstate 512 ...): (slice, b, L, H, P) float partial outputs
  int dt_tma;       // dt is a regular 2-D array of rows: a 64-row tile is ONE tiled TMA load through a tensor map
  int bc_contig;    // B and C rows of one (batch, group) are adjacent in memory: a 64-row tile is one bulk copy
  int bc_tma;       // forward: B and C are regular 2-D arrays of rows (any row pitch): a 64-row tile is one tiled TMA load each
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
  bf16* saved;      // optional (b, H, nblk + 1, PP / 8, N, 8) bf16: state entering every 64-point block, and the final one
  int* status;
  // backward
  const bf16* dout; int64_t g_sb, g_sl, g_sh;
  const float* dfinal;
  bf16* dx; void* ddt; bf16* dz; bf16* dinit;
  uint32_t* dBCh;                       // per-head partials (b, L, H, N) of packed bf16 pairs {dB_h, dC_h}
  float* dApart; float* dbpart;         // (b, H, N)
  float* dDpart;                        // (b, H, PP)
};

__device__ __forceinline__ int trow(const TArgs& a, int t) { return a.rev ? a.L - 1 - t : t; }

__device__ __forceinline__ float softplus_fast(float v) {
  // softplus with the reference's threshold; log2-domain hardware approximations
  return v <= 20.f ? lg2f(1.f + ex2f(v * LOG2E)) * LN2 : v;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));   // one instruction: {hi, lo} -> packed pair
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float2 v) { return pack_bf16(v.x, v.y); }


// ---- two adjacent states per thread: packed fp32 pairs (one instruction per pair on sm_100) ---------------------
__device__ __forceinline__ float2 f2(float x, float y) { return make_float2(x, y); }
__device__ __forceinline__ float2 f2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 ex2f2(float2 v) { return make_float2(ex2f(v.x), ex2f(v.y)); }
__device__ __forceinline__ float2 ex2f2_neg(float2 v) { return make_float2(ex2f(-v.x), ex2f(-v.y)); }
__device__ __forceinline__ float2 lg2f2(float2 v) { return make_float2(lg2f(v.x), lg2f(v.y)); }
// a packed bf16 pair (low half = the lower address) -> two floats
__device__ __forceinline__ float2 unpack_bf16(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u)); }

// dt of one row, two adjacent states: bias, softplus (reference threshold 20, evaluated in the log2 domain: the
// pre-activation scaled by log2 e is `t`, softplus = ln 2 * lg2(1 + 2^t), and above the threshold t * ln 2), clamp.
// biasL = bias * log2 e when softplus is on, else the plain bias.
__device__ __forceinline__ float2 dt_transform2(const TArgs& a, float2 raw, float2 biasL) {
  float2 v;
  if (a.softplus) {
    const float2 t = __ffma2_rn(raw, f2(LOG2E), biasL);
    float2 s = lg2f2(__fadd2_rn(ex2f2(t), f2(1.f)));
    s.x = t.x <= 20.f * LOG2E ? s.x : t.x;
    s.y = t.y <= 20.f * LOG2E ? s.y : t.y;
    v = __fmul2_rn(s, f2(LN2));
  } else {
    v = __fadd2_rn(raw, biasL);
  }
  v.x = fminf(fmaxf(v.x, a.dtmin), a.dtmax);
  v.y = fminf(fmaxf(v.y, a.dtmin), a.dtmax);
  return v;
}

// dt of one row as the kernels use it: bias, softplus (reference threshold), clamp.
// `clamped` reports whether the clamp changed the value (no gradient flows then).
__device__ __forceinline__ float dt_transform(const TArgs& a, float raw, float bias, bool& clamped) {
  float v = raw + bias;
  if (a.softplus) v = softplus_fast(v);
  clamped = v < a.dtmin || v > a.dtmax;
  return fminf(fmaxf(v, a.dtmin), a.dtmax);
}

// ---- blocks outside the range of the single-reference factorisation (rare; kept out of line) -------------------
// Smallest k in 1..6 such that, with the block cut into 2^k windows of 64 >> k rows, the summed log2-decay
// of every window of this thread's 32 rows stays within 2^100 (k = 6, single rows, always qualifies: there
// the decay itself is floored).  sdt: this thread's column of the staged dt tile (unused for float dt).
template <typename TDT>
__device__ __noinline__ int window_need(const TArgs& a, const bf16* sdt, int dstep, const TDT* __restrict__ dtp, int row0,
                                        int rows, int half, int n, float A2, float bias) {
  int need = 6;
  for (int k = 5; k >= 1; --k) {
    const int wsz = QB >> k;
    float run = 0.f, mx = 0.f;
    for (int j = 0; j < 32; ++j) {
      const int l = half * 32 + j;
      if (l >= rows) break;
      float raw;
      if (sizeof(TDT) == 2) raw = __bfloat162float(sdt[l * dstep]);
      else raw = ldf(dtp + (int64_t)trow(a, row0 + l) * a.dt_sl + n);
      bool clamped;
      const float v = dt_transform(a, raw, bias, clamped);
      if (j % wsz == 0) run = 0.f;
      run = fmaf(v, A2, run);
      mx = fmaxf(mx, fabsf(run));
    }
    if (mx <= 100.f) need = k;
  }
  return need;
}

TArgs make_targs(const issm_params& p);
// Tensor map over bf16 dt viewed as (batch*seqlen rows) x (row pitch) with a (dstate x 64 rows) box; false if dt
// is not laid out as one regular 2-D array (then the kernels fall back to one bulk copy per row).
bool make_dt_tensor_map(const issm_params& p, CUtensorMap* out);
// Tensor map over a bf16 array viewed as (batch*seqlen rows) x (row pitch `sl` elements) with a (box_w x 64 rows) box;
// false if the rows do not form one regular 2-D array (batch stride != seqlen * row stride) or are not 16-byte aligned.
bool make_rows_tensor_map(const void* base, int64_t sb, int64_t sl, int64_t width, int batch, int seqlen, int box_w, CUtensorMap* out);
// the forward kernel's tensor maps (one kernel parameter)
struct FwdMaps { CUtensorMap dt, B, C; };
int state_slices(int dstate);
int tensor_fwd_states_only(const issm_params& p, bf16* saved, int* redo, cudaStream_t s);
size_t tensor_bwd_workspace_bytes(const issm_params& p);

}  // namespace issm
