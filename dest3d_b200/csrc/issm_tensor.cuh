// Declarations shared by the forward and backward kernels of the tcgen05 ISSM path.
#pragma once

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
  bf16* saved;      // optional (b, H, nblk + 1, N, PP) bf16: state entering every 64-point block, and the final one
  int* status;
  // backward
  const bf16* dout; int64_t g_sb, g_sl, g_sh;
  const float* dfinal;
  bf16* dx; void* ddt; bf16* dz; bf16* dinit;
  bf16* dBh; bf16* dCh;                 // per-head partials (b, L, H, N)
  float* dApart; float* dbpart;         // (b, H, N)
  float* dDpart;                        // (b, H, PP)
};

__device__ __forceinline__ int trow(const TArgs& a, int t) { return a.rev ? a.L - 1 - t : t; }

__device__ __forceinline__ float softplus_fast(float v) {
  // softplus with the reference's threshold; log2-domain hardware approximations
  return v <= 20.f ? lg2f(1.f + ex2f(v * LOG2E)) * LN2 : v;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
}


TArgs make_targs(const issm_params& p);
int tensor_fwd_states_only(const issm_params& p, bf16* saved, cudaStream_t s);
size_t tensor_bwd_workspace_bytes(const issm_params& p);

}  // namespace issm
