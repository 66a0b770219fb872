// Shared helpers for the ISSM kernels: typed loads/stores, launch accounting, size helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>
#include <mutex>

#include "../../include/issm_b200.h"

namespace issm {

typedef __nv_bfloat16 bf16;

extern std::atomic<uint64_t> g_launches;

// Launch + count + error check.  Evaluates to an ISSM_* code in `rc_` of the calling scope.
#define ISSM_LAUNCH(kernel, grid, block, smem, stream, ...)                         \
  do {                                                                              \
    kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);                     \
    issm::g_launches.fetch_add(1, std::memory_order_relaxed);                       \
    if (cudaPeekAtLastError() != cudaSuccess) {                                     \
      fprintf(stderr, "issm_b200: launch of %s failed: %s\n", #kernel, cudaGetErrorString(cudaGetLastError())); \
      return ISSM_ERR_CUDA;                                                         \
    }                                                                               \
  } while (0)

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

// softplus with the reference's threshold (issm_triton/softplus.py:9-11)
__device__ __forceinline__ float softplus_thr(float v) { return v <= 20.0f ? log1pf(expf(v)) : v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Raises the dynamic shared-memory limit of a kernel ONCE per device (the attribute is per device and per
// function): every distinct kernel gets its own table of once-flags through the tag type.  Returns ISSM_OK
// or ISSM_ERR_CUDA; a failure is remembered and reported by every later call on that device.
constexpr int kMaxDevices = 64;
template <typename Tag>
struct SmemAttrOnce {
  template <typename Kernel>
  static int set(Kernel kernel, size_t bytes) {
    static std::once_flag flags[kMaxDevices];
    static int result[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { (void)cudaGetLastError(); return ISSM_ERR_CUDA; }
    std::call_once(flags[dev], [&] {
      result[dev] = ISSM_OK;
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        result[dev] = ISSM_ERR_CUDA;
      }
    });
    return result[dev];
  }
};

// largest dynamic shared-memory size a block may opt into on the current device (0 on failure)
static inline size_t max_optin_smem() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return (size_t)v;
}

static inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Sequential carving of a workspace into 256-byte aligned pieces.
struct Carver {
  char* base;
  size_t off;
  explicit Carver(void* b) : base(static_cast<char*>(b)), off(0) {}
  template <typename T>
  T* take(size_t count) {
    T* r = reinterpret_cast<T*>(base + off);
    off = align_up(off + count * sizeof(T), 256);
    return r;
  }
};

// entry points implemented per path
size_t simt_workspace_bytes(const issm_params& p, int pass);
int simt_fwd(const issm_params& p, cudaStream_t s);
int simt_bwd(const issm_params& p, cudaStream_t s);

bool tensor_path_supported(const issm_params& p, int pass);
size_t tensor_workspace_bytes(const issm_params& p, int pass);
int tensor_fwd(const issm_params& p, cudaStream_t s);
int tensor_bwd(const issm_params& p, cudaStream_t s);

}  // namespace issm
