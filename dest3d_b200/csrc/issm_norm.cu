// Gated RMS / Layer norm, forward and backward (issm_triton/layernorm_gated.py:35-95, 145-258).
// Memory-bound: one warp per row, features strided over lanes, statistics by warp shuffles.
// Weight/bias gradients are accumulated per warp in shared memory without atomics and reduced
// over blocks in a fixed order, so results are bitwise reproducible.
#include "issm_common.cuh"

namespace issm {

__device__ __forceinline__ float siluf_(float v) { return v * sigmoidf_(v); }
__device__ __forceinline__ float dsiluf_(float v) {
  const float s = sigmoidf_(v);
  return s * (1.f + v * (1.f - s));
}

template <typename T>
__global__ void k_norm_fwd(issm_norm_params np) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= np.rows) return;
  const int gs = np.group_size, ng = np.hidden / gs;
  const T* x = (const T*)np.x + (int64_t)warp * np.x_sr;
  const T* z = np.has_z ? (const T*)np.z + (int64_t)warp * np.z_sr : nullptr;
  T* y = (T*)np.y + (int64_t)warp * np.y_sr;
  const bool pre_gate = z && !np.norm_before_gate, post_gate = z && np.norm_before_gate;
  for (int g = 0; g < ng; ++g) {
    float s1 = 0.f, s2 = 0.f;
    for (int f = g * gs + lane; f < (g + 1) * gs; f += 32) {
      float v = ldf(x + f);
      if (pre_gate) v *= siluf_(ldf(z + f));
      s1 += v;
      s2 = fmaf(v, v, s2);
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    float mean = 0.f, var;
    if (np.is_rms) {
      var = s2 / gs;
    } else {
      mean = s1 / gs;
      float sv = 0.f;
      for (int f = g * gs + lane; f < (g + 1) * gs; f += 32) {
        float v = ldf(x + f);
        if (pre_gate) v *= siluf_(ldf(z + f));
        sv = fmaf(v - mean, v - mean, sv);
      }
      var = warp_sum(sv) / gs;
    }
    const float rstd = rsqrtf(var + np.eps);
    if (lane == 0) {
      np.rstd[(size_t)warp * ng + g] = rstd;
      if (!np.is_rms && np.mean) np.mean[(size_t)warp * ng + g] = mean;
    }
    for (int f = g * gs + lane; f < (g + 1) * gs; f += 32) {
      float v = ldf(x + f);
      if (pre_gate) v *= siluf_(ldf(z + f));
      float o = (v - mean) * rstd * np.weight[f];
      if (np.has_bias) o += np.bias[f];
      if (post_gate) o *= siluf_(ldf(z + f));
      stf(y + f, o);
    }
  }
}

constexpr int NORM_BWD_WARPS = 4;

// grid = nblk blocks; block i handles rows [i*rpb, (i+1)*rpb); partial dw/db -> ws (nblk, hidden)
template <typename T>
__global__ void k_norm_bwd(issm_norm_params np, int rpb, float* __restrict__ dwpart, float* __restrict__ dbpart) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = np.hidden, gs = np.group_size, ng = H / gs;
  float* sdw = sm + (size_t)warp * H;
  float* sdb = sm + (size_t)NORM_BWD_WARPS * H + (size_t)warp * H;
  for (int f = lane; f < H; f += 32) { sdw[f] = 0.f; sdb[f] = 0.f; }
  __syncwarp();
  const bool pre_gate = np.has_z && !np.norm_before_gate, post_gate = np.has_z && np.norm_before_gate;
  const int r_end = min(np.rows, (int)(blockIdx.x + 1) * rpb);
  for (int row = blockIdx.x * rpb + warp; row < r_end; row += NORM_BWD_WARPS) {
    const T* x = (const T*)np.x + (int64_t)row * np.x_sr;
    const T* z = np.has_z ? (const T*)np.z + (int64_t)row * np.z_sr : nullptr;
    const T* dy = (const T*)np.dy + (int64_t)row * np.dy_sr;
    T* dx = (T*)np.dx + (int64_t)row * H;
    T* dz = np.has_z ? (T*)np.dz + (int64_t)row * H : nullptr;
    for (int g = 0; g < ng; ++g) {
      const float rstd = np.rstd[(size_t)row * ng + g];
      const float mean = np.is_rms ? 0.f : np.mean[(size_t)row * ng + g];
      float c1 = 0.f, c2 = 0.f;
      for (int f = g * gs + lane; f < (g + 1) * gs; f += 32) {
        float v = ldf(x + f);
        if (pre_gate) v *= siluf_(ldf(z + f));
        const float xh = (v - mean) * rstd;
        float g_out = ldf(dy + f);
        if (post_gate) g_out *= siluf_(ldf(z + f));
        const float wdy = g_out * np.weight[f];
        c1 = fmaf(xh, wdy, c1);
        c2 += wdy;
      }
      c1 = warp_sum(c1) / gs;
      c2 = np.is_rms ? 0.f : warp_sum(c2) / gs;
      for (int f = g * gs + lane; f < (g + 1) * gs; f += 32) {
        const float xr = ldf(x + f);
        const float zv = z ? ldf(z + f) : 0.f;
        const float v = pre_gate ? xr * siluf_(zv) : xr;
        const float xh = (v - mean) * rstd;
        const float go = ldf(dy + f);
        const float g_out = post_gate ? go * siluf_(zv) : go;
        const float wdy = g_out * np.weight[f];
        const float dv = (wdy - xh * c1 - c2) * rstd;
        sdw[f] = fmaf(g_out, xh, sdw[f]);
        sdb[f] += g_out;
        if (pre_gate) {
          stf(dx + f, dv * siluf_(zv));
          stf(dz + f, dv * xr * dsiluf_(zv));
        } else {
          stf(dx + f, dv);
          if (post_gate) {
            float yv = xh * np.weight[f];
            if (np.has_bias) yv += np.bias[f];
            stf(dz + f, go * yv * dsiluf_(zv));
          }
        }
      }
    }
  }
  __syncthreads();
  for (int f = threadIdx.x; f < H; f += blockDim.x) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < NORM_BWD_WARPS; ++w) {
      a += sm[(size_t)w * H + f];
      b += sm[(size_t)NORM_BWD_WARPS * H + (size_t)w * H + f];
    }
    dwpart[(size_t)blockIdx.x * H + f] = a;
    dbpart[(size_t)blockIdx.x * H + f] = b;
  }
}

__global__ void k_norm_reduce(const float* __restrict__ part, int count, int stride, float* __restrict__ out) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= stride) return;
  float acc = 0.f;
  for (int i = 0; i < count; ++i) acc += part[(size_t)i * stride + j];
  out[j] = acc;
}

static int norm_blocks(const issm_norm_params& p) {
  const int want = 148 * 4;
  return p.rows < want ? (p.rows > 0 ? p.rows : 1) : want;
}

static int norm_validate(const issm_norm_params* p, bool bwd) {
  if (!p) return ISSM_ERR_NULL;
  if (p->rows < 0 || p->hidden <= 0 || p->hidden > 4096 || p->group_size <= 0 || p->hidden % p->group_size) return ISSM_ERR_SHAPE;
  if (p->io_dtype != ISSM_F32 && p->io_dtype != ISSM_BF16) return ISSM_ERR_DTYPE;
  if (!p->x || !p->weight || !p->rstd || (p->has_z && !p->z) || (p->has_bias && !p->bias)) return ISSM_ERR_NULL;
  if (!p->is_rms && !p->mean) return ISSM_ERR_NULL;
  if (!bwd && !p->y) return ISSM_ERR_NULL;
  if (bwd && (!p->dy || !p->dx || !p->dweight || (p->has_z && !p->dz) || (p->has_bias && !p->dbias))) return ISSM_ERR_NULL;
  return ISSM_OK;
}

}  // namespace issm

using namespace issm;

extern "C" size_t issm_b200_norm_workspace_bytes(const issm_norm_params* p, int pass) {
  if (!p || pass == 0) return 0;
  return align_up((size_t)2 * norm_blocks(*p) * p->hidden * sizeof(float), 256);
}

extern "C" int issm_b200_norm_fwd(const issm_norm_params* p, void* stream) {
  int rc = norm_validate(p, false);
  if (rc) return rc;
  if (p->rows == 0) return ISSM_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int wpb = 8;
  const unsigned grid = (p->rows + wpb - 1) / wpb;
  if (p->io_dtype == ISSM_F32) ISSM_LAUNCH((k_norm_fwd<float>), grid, wpb * 32, 0, s, *p);
  else ISSM_LAUNCH((k_norm_fwd<bf16>), grid, wpb * 32, 0, s, *p);
  return ISSM_OK;
}

extern "C" int issm_b200_norm_bwd(const issm_norm_params* p, void* stream) {
  int rc = norm_validate(p, true);
  if (rc) return rc;
  if (p->rows == 0) return ISSM_OK;
  if (!p->workspace || p->workspace_bytes < issm_b200_norm_workspace_bytes(p, 1)) return ISSM_ERR_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  const int nblk = norm_blocks(*p);
  const int rpb = (p->rows + nblk - 1) / nblk;
  float* dwpart = (float*)p->workspace;
  float* dbpart = dwpart + (size_t)nblk * p->hidden;
  const size_t smem = (size_t)2 * NORM_BWD_WARPS * p->hidden * sizeof(float);
  struct F32Tag {};
  struct BF16Tag {};
  if (smem > 48 * 1024) {                                  // wide rows: opt in (once per device) to the device's limit
    const size_t lim = max_optin_smem();
    if (smem > lim) return ISSM_ERR_SHAPE;
    if ((p->io_dtype == ISSM_F32 ? SmemAttrOnce<F32Tag>::set(k_norm_bwd<float>, lim) : SmemAttrOnce<BF16Tag>::set(k_norm_bwd<bf16>, lim)) != ISSM_OK)
      return ISSM_ERR_CUDA;
  }
  if (p->io_dtype == ISSM_F32) ISSM_LAUNCH((k_norm_bwd<float>), nblk, NORM_BWD_WARPS * 32, smem, s, *p, rpb, dwpart, dbpart);
  else ISSM_LAUNCH((k_norm_bwd<bf16>), nblk, NORM_BWD_WARPS * 32, smem, s, *p, rpb, dwpart, dbpart);
  ISSM_LAUNCH(k_norm_reduce, (p->hidden + 127) / 128, 128, 0, s, dwpart, nblk, p->hidden, p->dweight);
  if (p->has_bias) ISSM_LAUNCH(k_norm_reduce, (p->hidden + 127) / 128, 128, 0, s, dbpart, nblk, p->hidden, p->dbias);
  return ISSM_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward of the gated norm for callers that must not allocate.
//
// Some hosts of this library cannot obtain device memory at call time: a plugin running inside an
// inference server whose memory pool is sealed after start-up, a real-time loop where a device
// allocation would stall every stream, or a binding in a language without a device allocator at
// hand.  For them the per-block weight / bias gradient partials of k_norm_bwd live in the fixed
// array below instead of a caller-provided workspace.  Every GPU that loads the library carries
// the array (4.6 MiB) until the process exits.
// ---------------------------------------------------------------------------------------------
namespace issm {
constexpr int kNoAllocMaxHidden = 1024;                 // widest row the built-in scratch covers
constexpr int kNoAllocMaxBlocks = 148 * 4;              // == the largest grid norm_blocks() returns
static __device__ __align__(256) float g_norm_scratch[2 * kNoAllocMaxBlocks * kNoAllocMaxHidden];

// The array's name is only a host-side handle; kernels need its device address, which differs per
// device.  Looked up once per device (with that device current) and cached.
static float* norm_scratch_address(int* rc) {
  static std::atomic<float*> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *rc = ISSM_ERR_CUDA; return nullptr; }
  float* ptr = cache[dev].load(std::memory_order_acquire);
  if (!ptr) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_norm_scratch) != cudaSuccess || !sym) {
      (void)cudaGetLastError();
      *rc = ISSM_ERR_CUDA;
      return nullptr;
    }
    ptr = static_cast<float*>(sym);
    cache[dev].store(ptr, std::memory_order_release);
  }
  *rc = ISSM_OK;
  return ptr;
}
}  // namespace issm

extern "C" int issm_b200_norm_bwd_noalloc(const issm_norm_params* p, void* stream) {
  int rc = norm_validate(p, true);
  if (rc) return rc;
  if (p->hidden > kNoAllocMaxHidden) return ISSM_ERR_LIMIT;
  if (p->rows == 0) return ISSM_OK;
  float* scratch = norm_scratch_address(&rc);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int nblk = norm_blocks(*p);                      // <= kNoAllocMaxBlocks
  const int rpb = (p->rows + nblk - 1) / nblk;
  float* dwpart = scratch;
  float* dbpart = scratch + (size_t)nblk * p->hidden;
  const size_t smem = (size_t)2 * NORM_BWD_WARPS * p->hidden * sizeof(float);   // <= 32 KiB here
  // every block writes its whole row of partials, so nothing in the scratch has to start at zero
  if (p->io_dtype == ISSM_F32) ISSM_LAUNCH((k_norm_bwd<float>), nblk, NORM_BWD_WARPS * 32, smem, s, *p, rpb, dwpart, dbpart);
  else ISSM_LAUNCH((k_norm_bwd<bf16>), nblk, NORM_BWD_WARPS * 32, smem, s, *p, rpb, dwpart, dbpart);
  ISSM_LAUNCH(k_norm_reduce, (p->hidden + 127) / 128, 128, 0, s, dwpart, nblk, p->hidden, p->dweight);
  if (p->has_bias) ISSM_LAUNCH(k_norm_reduce, (p->hidden + 127) / 128, 128, 0, s, dbpart, nblk, p->hidden, p->dbias);
  return ISSM_OK;
}
