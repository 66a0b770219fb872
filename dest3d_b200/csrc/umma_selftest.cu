// Self-check of the tcgen05 building blocks (operand layouts, descriptors, TMEM row mapping):
// one CTA computes D = A * B^T for small bf16 matrices through exactly the helpers the ISSM
// tensor path uses.  The result is compared with a plain matmul by the test-suite.
#include "issm_common.cuh"
#include "umma.cuh"

namespace issm {
using namespace umma;

// layout kinds: 0 = SW128 K-major, 1 = INTERLEAVE K-major
__device__ uint32_t st_off(int kind, int rows, int row, int k) {
  if (kind == 0) return (uint32_t)((k >> 6) * rows * 128) + sw128_off(row, k & 63);
  return (uint32_t)((k >> 3) * rows * 16 + row * 16 + (k & 7) * 2);
}

__global__ void __launch_bounds__(128) k_umma_selftest(int M, int N, int K, int kindA, int kindB,
                                                       const bf16* __restrict__ A, const bf16* __restrict__ B,
                                                       float* __restrict__ D, float* __restrict__ Draw, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_holder;
  uint8_t* sA = smem;
  // a SW128 operand occupies whole 128-byte rows per 64-element atom, even when K is not a multiple of 64
  const size_t bytesA = kindA == 0 ? (size_t)M * ((K + 63) / 64) * 128 : (size_t)M * K * 2;
  uint8_t* sB = smem + ((bytesA + 1023) & ~(size_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < M * K; i += blockDim.x) *(bf16*)(sA + st_off(kindA, M, i / K, i % K)) = A[i];
  for (int i = tid; i < N * K; i += blockDim.x) *(bf16*)(sB + st_off(kindB, N, i / K, i % K)) = B[i];
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_holder, 256); tmem_relinquish(); }
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_holder;
  if (tid == 0) {
    const uint32_t idesc = idesc_bf16(M, N);
    for (int k0 = 0; k0 < K; k0 += 16) {
      uint64_t da, db;
      if (kindA == 0) da = desc_sw128(smem_u32(sA) + (k0 >> 6) * M * 128 + (k0 & 63) * 2);
      else da = desc_interleave(smem_u32(sA) + (k0 >> 3) * M * 16, M * 16, 128);
      if (kindB == 0) db = desc_sw128(smem_u32(sB) + (k0 >> 6) * N * 128 + (k0 & 63) * 2);
      else db = desc_interleave(smem_u32(sB) + (k0 >> 3) * N * 16, N * 16, 128);
      mma_bf16(tmem, da, db, idesc, k0 > 0);
    }
    mma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0, 1u << 22);
  if (!ok && status) atomicExch(status, 1);
  fence_after_sync();
  if (ok) {
    // raw dump: lane (32*warp + lane), all N columns (padded to 16)
    for (int c0 = 0; c0 < N; c0 += 16) {
      float v[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c0, v);
      tmem_ld_wait();
      for (int i = 0; i < 16; ++i)
        if (c0 + i < N) {
          const int tl = warp * 32 + lane;
          Draw[(size_t)tl * N + c0 + i] = v[i];
          int row = -1;
          if (M == 128) row = tl;
          else if (lane < 16) row = warp * 16 + lane;     // M = 64: rows 16w..16w+15 sit in lanes 32w..32w+15
          if (row >= 0) D[(size_t)row * N + c0 + i] = v[i];
        }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}
}  // namespace issm

using namespace issm;

extern "C" int issm_b200_selftest_umma(int M, int N, int K, int kindA, int kindB, const void* A, const void* B,
                                       float* D, float* Draw, int32_t* status, void* stream) {
  if ((M != 64 && M != 128) || N < 16 || N > 256 || N % 16 || K < 16 || K % 16 || !A || !B || !D || !Draw) return ISSM_ERR_SHAPE;
  const size_t bytesA = kindA == 0 ? (size_t)M * ((K + 63) / 64) * 128 : (size_t)M * K * 2;
  const size_t bytesB = kindB == 0 ? (size_t)N * ((K + 63) / 64) * 128 : (size_t)N * K * 2;
  const size_t smem = ((bytesA + 1023) & ~(size_t)1023) + bytesB + 2048;
  if (smem > 200 * 1024) return ISSM_ERR_SHAPE;
  if (cudaFuncSetAttribute(k_umma_selftest, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ISSM_ERR_CUDA;
  ISSM_LAUNCH(k_umma_selftest, 1, 128, smem, (cudaStream_t)stream, M, N, K, kindA, kindB, (const bf16*)A, (const bf16*)B, D, Draw, status);
  return ISSM_OK;
}
