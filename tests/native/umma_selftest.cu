// TEST-ONLY native code (built into tests/native/libissm_b200_selftest.so, never into the product library).
//
// 1. Self-check of the tcgen05 building blocks (operand layouts, descriptors, TMEM row mapping): one CTA
//    computes D = A * B^T for small bf16 matrices through exactly the helpers the ISSM tensor path uses
//    (dest3d_b200/csrc/umma.cuh).  The result is compared with a plain matmul by the test-suite.
//      M is 64 or 128; N and K multiples of 16; kind 0 = 128-byte swizzle K-major, 1 = interleaved core
//      matrices, 2 = 128-byte swizzle MN-major.  Draw (128 x N) receives the raw TMEM lanes.
// 2. The bounded wait: a kernel that waits, with a short poll limit, on an mbarrier nobody ever arrives on.
//    The wait runs out by construction (no fault, no trap, no endless loop); the kernel then records bit 0 in
//    the status word exactly as the ISSM kernels do and returns.
#include <cuda_runtime.h>

#include "../../dest3d_b200/csrc/umma.cuh"

typedef __nv_bfloat16 bf16;
enum { ST_OK = 0, ST_ERR_SHAPE = 2, ST_ERR_CUDA = 7 };

namespace issm {
using namespace umma;

// layout kinds: 0 = SW128 K-major, 1 = INTERLEAVE K-major, 2 = SW128 MN-major
__device__ uint32_t st_off(int kind, int rows, int K, int row, int k) {
  if (kind == 0) return (uint32_t)((k >> 6) * rows * 128) + sw128_off(row, k & 63);
  if (kind == 2) return (uint32_t)((row >> 6) * K * 128) + sw128_off(k, row & 63);
  return (uint32_t)((k >> 3) * rows * 16 + row * 16 + (k & 7) * 2);
}
__device__ size_t st_bytes(int kind, int rows, int K) {
  if (kind == 0) return (size_t)rows * ((K + 63) / 64) * 128;
  if (kind == 2) return (size_t)K * ((rows + 63) / 64) * 128;
  return (size_t)rows * K * 2;
}
__device__ uint64_t st_desc(int kind, uint32_t base, int rows, int K, int k0) {
  if (kind == 0) return desc_sw128(base + (k0 >> 6) * rows * 128 + (k0 & 63) * 2);
  if (kind == 2) return desc_sw128_mn(base + k0 * 128, K * 128);
  return desc_interleave(base + (k0 >> 3) * rows * 16, rows * 16, 128);
}

__global__ void __launch_bounds__(128) k_umma_selftest(int M, int N, int K, int kindA, int kindB,
                                                       const bf16* __restrict__ A, const bf16* __restrict__ B,
                                                       float* __restrict__ D, float* __restrict__ Draw, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_holder;
  uint8_t* sA = smem;
  // a SW128 operand occupies whole 128-byte rows per 64-element atom, even when K is not a multiple of 64
  const size_t bytesA = st_bytes(kindA, M, K);
  uint8_t* sB = smem + ((bytesA + 1023) & ~(size_t)1023);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < (int)((bytesA + 1023) / 1024 * 1024 + st_bytes(kindB, N, K)) / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0;
  __syncthreads();
  for (int i = tid; i < M * K; i += blockDim.x) *(bf16*)(sA + st_off(kindA, M, K, i / K, i % K)) = A[i];
  for (int i = tid; i < N * K; i += blockDim.x) *(bf16*)(sB + st_off(kindB, N, K, i / K, i % K)) = B[i];
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_holder, 256); tmem_relinquish(); }
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_holder;
  if (tid == 0) {
    const uint32_t idesc = idesc_bf16(M, N, kindA == 2, kindB == 2);
    for (int k0 = 0; k0 < K; k0 += 16)
      mma_bf16(tmem, st_desc(kindA, smem_u32(sA), M, K, k0), st_desc(kindB, smem_u32(sB), N, K, k0), idesc, k0 > 0);
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
  if ((M != 64 && M != 128) || N < 16 || N > 256 || N % 16 || K < 16 || K % 16 || !A || !B || !D || !Draw) return ST_ERR_SHAPE;
  auto bytes = [](int kind, int rows, int K) -> size_t {
    if (kind == 0) return (size_t)rows * ((K + 63) / 64) * 128;
    if (kind == 2) return (size_t)K * ((rows + 63) / 64) * 128;
    return (size_t)rows * K * 2;
  };
  if (kindA < 0 || kindA > 2 || kindB < 0 || kindB > 2) return ST_ERR_SHAPE;
  const size_t bytesA = bytes(kindA, M, K), bytesB = bytes(kindB, N, K);
  const size_t smem = ((bytesA + 1023) & ~(size_t)1023) + bytesB + 2048;
  if (smem > 200 * 1024) return ST_ERR_SHAPE;
  if (cudaFuncSetAttribute(k_umma_selftest, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return ST_ERR_CUDA;
  k_umma_selftest<<<1, 128, smem, (cudaStream_t)stream>>>(M, N, K, kindA, kindB, (const bf16*)A, (const bf16*)B, D, Draw, status);
  return cudaPeekAtLastError() == cudaSuccess ? ST_OK : ST_ERR_CUDA;
}

namespace issm {
// Every thread of the block polls an mbarrier that has one pending arrival which never comes, at most
// `limit` times; the expiry is reported like in the ISSM kernels (status bit 0) and the kernel returns.
__global__ void k_bounded_wait(uint32_t limit, int* status, int* polled_out) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  __syncthreads();
  const bool ok = mbar_wait_warp(&bar, 0, limit);
  if (!ok && threadIdx.x == 0) atomicOr(status, 1);
  if (threadIdx.x == 0) *polled_out = ok ? 0 : 1;
}
}  // namespace issm

extern "C" int issm_b200_selftest_bounded_wait(uint32_t limit, int32_t* status, int32_t* expired, void* stream) {
  if (!status || !expired || limit == 0 || limit > (1u << 16)) return ST_ERR_SHAPE;
  issm::k_bounded_wait<<<2, 64, 0, (cudaStream_t)stream>>>(limit, status, expired);
  return cudaPeekAtLastError() == cudaSuccess ? ST_OK : ST_ERR_CUDA;
}
