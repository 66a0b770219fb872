// Support for cutting one sequence into slices (over several GPUs, or as extra batch entries on one): the decay a
// slice applies to the state entering it is exp(A * sum of the transformed step sizes of the slice), the role the
// per-chunk `dA_cumsum[..., -1]` plays in the reference's state passing (issm_triton/issm_state_passing.py:92-107).
// This kernel produces the sums; one read of dt, coalesced over the states.
#include "issm_common.cuh"

namespace issm {

// part[seg, b, h, n] = sum over the rows of segment `seg` of clamp(softplus?(dt[b, l, h, n] + bias[h, n]))
template <typename T>
__global__ void __launch_bounds__(256) k_dt_sum(const T* __restrict__ dt, int64_t sb, int64_t sl, int64_t sh, const float* __restrict__ bias,
                                                 int softplus, float lo, float hi, int L, int rows, int N, float* __restrict__ part) {
  const int seg = blockIdx.x, h = blockIdx.y, b = blockIdx.z, H = gridDim.y, Bn = gridDim.z;
  const int l0 = seg * rows, l1 = min(L, l0 + rows);
  const T* p = dt + b * sb + h * sh;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    const float bv = bias ? bias[h * N + n] : 0.f;
    float acc = 0.f;
#pragma unroll 8
    for (int l = l0; l < l1; ++l) {
      float v = ldf(p + (int64_t)l * sl + n) + bv;
      if (softplus) v = softplus_thr(v);
      acc += fminf(fmaxf(v, lo), hi);
    }
    part[(((size_t)seg * Bn + b) * H + h) * N + n] = acc;
  }
}
}  // namespace issm

using namespace issm;

extern "C" int issm_b200_dt_sum(const void* dt, int32_t dt_dtype, int32_t batch, int32_t seqlen, int32_t nheads, int32_t dstate,
                                int64_t dt_sb, int64_t dt_sl, int64_t dt_sh, const float* dt_bias, int32_t dt_softplus, float dt_min,
                                float dt_max, int32_t rows_per_part, float* part, void* stream) {
  if (!dt || !part) return ISSM_ERR_NULL;
  if (batch <= 0 || batch > 65535 || seqlen <= 0 || nheads <= 0 || nheads > 65535 || dstate <= 0 || rows_per_part <= 0) return ISSM_ERR_SHAPE;
  if (dt_dtype != ISSM_F32 && dt_dtype != ISSM_BF16) return ISSM_ERR_DTYPE;
  const dim3 grid((seqlen + rows_per_part - 1) / rows_per_part, nheads, batch);
  const int threads = dstate >= 256 ? 256 : ((dstate + 31) / 32) * 32;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt_dtype == ISSM_F32)
    ISSM_LAUNCH(k_dt_sum<float>, grid, threads, 0, s, (const float*)dt, dt_sb, dt_sl, dt_sh, dt_bias, dt_softplus, dt_min, dt_max, seqlen, rows_per_part, dstate, part);
  else
    ISSM_LAUNCH(k_dt_sum<bf16>, grid, threads, 0, s, (const bf16*)dt, dt_sb, dt_sl, dt_sh, dt_bias, dt_softplus, dt_min, dt_max, seqlen, rows_per_part, dstate, part);
  return ISSM_OK;
}
