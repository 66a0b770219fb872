// The parameter generation in front of the scan (models/dest_module.py:541-559), one read of the distance features:
//   dt[b, l, h, k] = softplus(dist[b, l, k, :] . Wdt[h, :] + tok[b, l, h]) * mask[b, l, k]
//   B [b, l, g, k] = dist[b, l, k, :] . Wb[g, :] + tok[b, l, H + g]          (C, and the second direction's B / C with
//                                                                             their own token terms, alike)
// where the reference runs dt_proj / bc_proj as two Linear layers over dist, transposes both results to the
// (b, l, h, k) layout the scan wants, adds the per-token terms, applies softplus and multiplies by the mask in
// separate elementwise passes.  Here a thread owns one state k of one point: it holds the M distance features in
// registers, forms every output row, and stores each row coalesced over k in the scan's layout.
// Backward: g = d(out) / d(pre) per output row; ddist = sum_r g[r] W[r, :]; the weight gradient sum_k g[r, k] dist[k, j]
// is formed per point from shared-memory tiles and accumulated per block; the token terms are g summed over k in a
// fixed order.
#include "issm_common.cuh"

namespace issm {

constexpr int GLUE_MAX_ROWS = 16;

struct GlueArgs {
  int L, K, H, G, back, RW, RO;                            // RW = H + 2G weight rows; RO = H + 2G (+ 2G) output rows
  const void* dist; int64_t d_sb, d_sl, d_sk;
  const float* w;                                          // (RW, M)
  const float* tok;                                        // (b, L, RO)
  const float* mask;                                       // (b, L, K) or null
  void* dt; void* bc;                                      // (b, L, H, K), (b, L, RO - H, K)
  const void* ddt; const void* dbc;                        // same shapes, either may be null
  void* ddist;                                             // (b, L, K, M)
  float* dwpart;                                           // (blocks, GLUE_MAX_ROWS * M) partial weight gradients
  float* dtok;                                             // (b, L, RO)
};

template <typename T, int M>
__device__ __forceinline__ void load_feats(const T* p, float (&d)[M]) {
  if constexpr (sizeof(T) == 2 && M % 8 == 0) {
#pragma unroll
    for (int c = 0; c < M / 8; ++c) {
      const uint4 u = ((const uint4*)p)[c];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        d[c * 8 + 2 * i] = __uint_as_float(w[i] << 16);
        d[c * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  } else if constexpr (sizeof(T) == 4 && M % 4 == 0) {
#pragma unroll
    for (int c = 0; c < M / 4; ++c) {
      const float4 u = ((const float4*)p)[c];
      d[c * 4] = u.x; d[c * 4 + 1] = u.y; d[c * 4 + 2] = u.z; d[c * 4 + 3] = u.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < M; ++j) d[j] = ldf(p + j);
  }
}

template <typename T, int M>
__device__ __forceinline__ void store_feats(T* p, const float (&d)[M]) {
  if constexpr (sizeof(T) == 2 && M % 8 == 0) {
#pragma unroll
    for (int c = 0; c < M / 8; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(d[c * 8 + 2 * i], d[c * 8 + 2 * i + 1]);
        w[i] = *(const uint32_t*)&h;
      }
      ((uint4*)p)[c] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else if constexpr (sizeof(T) == 4 && M % 4 == 0) {
#pragma unroll
    for (int c = 0; c < M / 4; ++c) ((float4*)p)[c] = make_float4(d[c * 4], d[c * 4 + 1], d[c * 4 + 2], d[c * 4 + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < M; ++j) stf(p + j, d[j]);
  }
}

__device__ __forceinline__ float glue_sigmoid(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }

// one block per point (b, l); threads over the states k
template <typename T, int M>
__global__ void __launch_bounds__(128) k_glue_fwd(GlueArgs a) {
  __shared__ float sw[GLUE_MAX_ROWS * M], stok[GLUE_MAX_ROWS + 4 * 2];
  const int l = blockIdx.x, b = blockIdx.y;
  for (int i = threadIdx.x; i < a.RW * M; i += blockDim.x) sw[i] = a.w[i];
  for (int i = threadIdx.x; i < a.RO; i += blockDim.x) stok[i] = a.tok[((int64_t)b * a.L + l) * a.RO + i];
  __syncthreads();
  const T* drow = (const T*)a.dist + b * a.d_sb + l * a.d_sl;
  const int64_t row = (int64_t)b * a.L + l;
  T* dt = (T*)a.dt + row * a.H * a.K;
  T* bc = (T*)a.bc + row * (a.RO - a.H) * a.K;
  for (int k = threadIdx.x; k < a.K; k += blockDim.x) {
    float d[M];
    load_feats<T, M>(drow + (int64_t)k * a.d_sk, d);
    const float mk = a.mask ? a.mask[row * a.K + k] : 1.f;
    for (int r = 0; r < a.RW; ++r) {
      float pre = 0.f;
#pragma unroll
      for (int j = 0; j < M; ++j) pre = fmaf(d[j], sw[r * M + j], pre);
      if (r < a.H) {
        const float v = pre + stok[r];
        stf(dt + (int64_t)r * a.K + k, (v <= 20.f ? log1pf(__expf(v)) : v) * mk);
      } else {
        stf(bc + (int64_t)(r - a.H) * a.K + k, pre + stok[r]);
        if (a.back) stf(bc + (int64_t)(r - a.H + 2 * a.G) * a.K + k, pre + stok[r + 2 * a.G]);
      }
    }
  }
}

constexpr int GLUE_KT = 256;                               // states per shared-memory tile of the weight-gradient product
constexpr int GLUE_BWD_BLOCKS = 148 * 8;

// A block walks points (b, l) with a grid stride.  Per point: (1) threads over the states form g, ddist and the token
// sums, and park g and the features in shared memory; (2) thread (r, j) adds sum_k g[r, k] dist[k, j] to its
// accumulator of the weight gradient.  The accumulators go out once per block and are summed in a fixed order.
template <typename T, int M>
__global__ void __launch_bounds__(128) k_glue_bwd(GlueArgs a, int npoints) {
  __shared__ float sw[GLUE_MAX_ROWS * M], stok[GLUE_MAX_ROWS + 8], sred[4][GLUE_MAX_ROWS + 8];
  __shared__ float sg[GLUE_MAX_ROWS][GLUE_KT + 1];
  __shared__ __align__(16) float sd[GLUE_KT][M + 4];         // rows 16 bytes apart from a power of two: 128-bit accesses without conflicts
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < a.RW * M; i += blockDim.x) sw[i] = a.w[i];
  // weight gradient: thread = (row r, four features 4 jq .. 4 jq + 3, one of NKG ranges of the tile's states)
  constexpr int JQ = M / 4;
  const int tiles = a.RW * JQ, NKG = 128 / tiles > 0 ? 128 / tiles : 1;
  const int tile = threadIdx.x % tiles, kg = threadIdx.x / tiles;
  const int wr = tile / JQ, wj = (tile % JQ) * 4;
  const int kspan = (GLUE_KT + NKG - 1) / NKG;
  float wacc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int pt = blockIdx.x; pt < npoints; pt += gridDim.x) {
    const int b = pt / a.L, l = pt - b * a.L;
    __syncthreads();                                       // the previous point's tiles and token terms are consumed
    for (int i = threadIdx.x; i < a.RO; i += blockDim.x) stok[i] = a.tok[(int64_t)pt * a.RO + i];
    __syncthreads();
    const T* drow = (const T*)a.dist + b * a.d_sb + l * a.d_sl;
    const int64_t row = pt;
    const T* ddt = a.ddt ? (const T*)a.ddt + row * a.H * a.K : nullptr;
    const T* dbc = a.dbc ? (const T*)a.dbc + row * (a.RO - a.H) * a.K : nullptr;
    T* ddist = (T*)a.ddist + row * a.K * M;
    float tsum[GLUE_MAX_ROWS + 8];                          // per output row: sum over this thread's states
#pragma unroll
    for (int r = 0; r < GLUE_MAX_ROWS + 8; ++r) tsum[r] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += GLUE_KT) {
      if (k0) __syncthreads();
      for (int kk = threadIdx.x; kk < GLUE_KT; kk += blockDim.x) {
        const int k = k0 + kk;
        const bool in = k < a.K;
        float d[M], dd[M];
        if (in) load_feats<T, M>(drow + (int64_t)k * a.d_sk, d);
        else {
#pragma unroll
          for (int j = 0; j < M; ++j) d[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < M; ++j) dd[j] = 0.f;
#pragma unroll
        for (int c = 0; c < M / 4; ++c) *(float4*)&sd[kk][c * 4] = make_float4(d[c * 4], d[c * 4 + 1], d[c * 4 + 2], d[c * 4 + 3]);
        const float mk = (in && a.mask) ? a.mask[row * a.K + k] : 1.f;
#pragma unroll
        for (int r = 0; r < GLUE_MAX_ROWS; ++r) {
          if (r < a.RW) {
            float g = 0.f;
            if (in) {
              if (r < a.H) {
                if (ddt) {
                  float pre = stok[r];
#pragma unroll
                  for (int j = 0; j < M; ++j) pre = fmaf(d[j], sw[r * M + j], pre);
                  g = ldf(ddt + (int64_t)r * a.K + k) * mk * (pre <= 20.f ? glue_sigmoid(pre) : 1.f);
                }
                tsum[r] += g;
              } else if (dbc) {
                g = ldf(dbc + (int64_t)(r - a.H) * a.K + k);
                if (a.back) g += ldf(dbc + (int64_t)(r - a.H + 2 * a.G) * a.K + k);   // both directions share the weight row
              }
            }
            sg[r][kk] = g;
#pragma unroll
            for (int j = 0; j < M; ++j) dd[j] = fmaf(g, sw[r * M + j], dd[j]);
          }
        }
        if (in) {
          store_feats<T, M>(ddist + (int64_t)k * M, dd);
          if (dbc) {                                       // token terms of the B / C rows (each output row has its own)
#pragma unroll
            for (int ro = 0; ro < GLUE_MAX_ROWS + 8; ++ro)
              if (ro >= a.H && ro < a.RO) tsum[ro] += ldf(dbc + (int64_t)(ro - a.H) * a.K + k);
          }
        }
      }
      __syncthreads();
      if (kg < NKG) {
        const int k1 = min(GLUE_KT, (kg + 1) * kspan);
#pragma unroll 4
        for (int kk = kg * kspan; kk < k1; ++kk) {
          const float g = sg[wr][kk];
          const float4 f = *(const float4*)&sd[kk][wj];
          wacc[0] = fmaf(g, f.x, wacc[0]); wacc[1] = fmaf(g, f.y, wacc[1]);
          wacc[2] = fmaf(g, f.z, wacc[2]); wacc[3] = fmaf(g, f.w, wacc[3]);
        }
      }
    }
    // token terms: sum over the states, warp shuffles then the four warps in a fixed order
#pragma unroll
    for (int r = 0; r < GLUE_MAX_ROWS + 8; ++r) {
      if (r < a.RO) {
        float v = tsum[r];
#pragma unroll
        for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) sred[warp][r] = v;
      }
    }
    __syncthreads();
    for (int r = threadIdx.x; r < a.RO; r += blockDim.x)
      a.dtok[row * a.RO + r] = ((sred[0][r] + sred[1][r]) + sred[2][r]) + sred[3][r];
  }
  // the NKG ranges of a tile are summed in a fixed order through shared memory, then one partial per block goes out
  __syncthreads();
  float* sacc = &sg[0][0];                                 // 128 x 4 floats fit
#pragma unroll
  for (int c = 0; c < 4; ++c) sacc[threadIdx.x * 4 + c] = wacc[c];
  __syncthreads();
  if (threadIdx.x < tiles) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float acc = 0.f;
      for (int q = 0; q < NKG; ++q) acc += sacc[(q * tiles + threadIdx.x) * 4 + c];
      a.dwpart[(size_t)blockIdx.x * GLUE_MAX_ROWS * M + wr * M + wj + c] = acc;
    }
  }
}

// dweight (RW, M) from the per-block partials: 32 outputs by 8 groups per block; a group sums its contiguous share of
// the partials, the groups are combined in a fixed order
__global__ void __launch_bounds__(256) k_glue_reduce(const float* __restrict__ part, int blocks, int stride, int n, float* __restrict__ dw) {
  __shared__ float red[8][32];
  const int o = blockIdx.x * 32 + threadIdx.x, grp = threadIdx.y;
  const int per = (blocks + 7) / 8;
  float acc = 0.f;
  if (o < n) {
    const int i1 = min(blocks, (grp + 1) * per);
#pragma unroll 4
    for (int i = grp * per; i < i1; ++i) acc += part[(size_t)i * stride + o];
  }
  red[grp][threadIdx.x] = acc;
  __syncthreads();
  if (grp == 0 && o < n) {
    float tot = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) tot += red[g][threadIdx.x];
    dw[o] = tot;
  }
}

static int glue_validate(const issm_glue_params* p, bool bwd) {
  if (!p) return ISSM_ERR_NULL;
  if (p->batch <= 0 || p->batch > 65535 || p->seqlen <= 0 || p->nstates <= 0 || p->nheads <= 0 || p->ngroups <= 0) return ISSM_ERR_SHAPE;
  if (p->nfeat != 4 && p->nfeat != 8 && p->nfeat != 16) return ISSM_ERR_SHAPE;
  if (p->nheads + 2 * p->ngroups > GLUE_MAX_ROWS || p->nheads + 4 * p->ngroups > GLUE_MAX_ROWS + 8) return ISSM_ERR_SHAPE;
  if (p->io_dtype != ISSM_F32 && p->io_dtype != ISSM_BF16) return ISSM_ERR_DTYPE;
  if (!p->dist || !p->weight || !p->tok) return ISSM_ERR_NULL;
  if (!bwd && (!p->dt || !p->bc)) return ISSM_ERR_NULL;
  if (bwd && (!p->ddist || !p->dweight || !p->dtok)) return ISSM_ERR_NULL;
  const size_t es = p->io_dtype == ISSM_F32 ? 4 : 2;
  if (((uintptr_t)p->dist % 16) || (p->dist_sb * es) % 16 || (p->dist_sl * es) % 16 || (p->dist_sk * es) % (p->nfeat * es >= 16 ? 16 : p->nfeat * es))
    return ISSM_ERR_ALIGN;
  return ISSM_OK;
}
static GlueArgs glue_args(const issm_glue_params& p) {
  GlueArgs a{};
  a.L = p.seqlen; a.K = p.nstates; a.H = p.nheads; a.G = p.ngroups; a.back = p.has_back;
  a.RW = p.nheads + 2 * p.ngroups; a.RO = a.RW + (p.has_back ? 2 * p.ngroups : 0);
  a.dist = p.dist; a.d_sb = p.dist_sb; a.d_sl = p.dist_sl; a.d_sk = p.dist_sk;
  a.w = p.weight; a.tok = p.tok; a.mask = p.mask; a.dt = p.dt; a.bc = p.bc;
  a.ddt = p.ddt; a.dbc = p.dbc; a.ddist = p.ddist; a.dwpart = (float*)p.workspace; a.dtok = p.dtok;
  return a;
}
}  // namespace issm

using namespace issm;

#define GLUE_DISPATCH(KERNEL)                                                                         \
  do {                                                                                                \
    const dim3 grid(p->seqlen, p->batch);                                                             \
    cudaStream_t s = (cudaStream_t)stream;                                                            \
    if (p->io_dtype == ISSM_F32) {                                                                    \
      if (p->nfeat == 16) ISSM_LAUNCH((KERNEL<float, 16>), grid, 128, 0, s, a);                       \
      else if (p->nfeat == 8) ISSM_LAUNCH((KERNEL<float, 8>), grid, 128, 0, s, a);                    \
      else ISSM_LAUNCH((KERNEL<float, 4>), grid, 128, 0, s, a);                                       \
    } else {                                                                                          \
      if (p->nfeat == 16) ISSM_LAUNCH((KERNEL<bf16, 16>), grid, 128, 0, s, a);                        \
      else if (p->nfeat == 8) ISSM_LAUNCH((KERNEL<bf16, 8>), grid, 128, 0, s, a);                     \
      else ISSM_LAUNCH((KERNEL<bf16, 4>), grid, 128, 0, s, a);                                        \
    }                                                                                                 \
  } while (0)

extern "C" size_t issm_b200_sizeof_glue_params(void) { return sizeof(issm_glue_params); }

extern "C" int issm_b200_glue_fwd(const issm_glue_params* p, void* stream) {
  int rc = glue_validate(p, false);
  if (rc) return rc;
  const GlueArgs a = glue_args(*p);
  GLUE_DISPATCH(k_glue_fwd);
  return ISSM_OK;
}

static int glue_bwd_blocks(const issm_glue_params* p) {
  const int64_t pts = (int64_t)p->batch * p->seqlen;
  return (int)(pts < GLUE_BWD_BLOCKS ? pts : GLUE_BWD_BLOCKS);
}

extern "C" size_t issm_b200_glue_workspace_bytes(const issm_glue_params* p) {
  if (!p || p->batch <= 0 || p->seqlen <= 0) return 0;
  return align_up((size_t)glue_bwd_blocks(p) * GLUE_MAX_ROWS * 16 * sizeof(float), 256);
}

extern "C" int issm_b200_glue_bwd(const issm_glue_params* p, void* stream) {
  int rc = glue_validate(p, true);
  if (rc) return rc;
  if (!p->workspace || p->workspace_bytes < issm_b200_glue_workspace_bytes(p)) return ISSM_ERR_WORKSPACE;
  if ((int64_t)p->batch * p->seqlen > 0x7fffffff) return ISSM_ERR_SHAPE;
  const GlueArgs a = glue_args(*p);
  const int blocks = glue_bwd_blocks(p), npoints = p->batch * p->seqlen;
  cudaStream_t s = (cudaStream_t)stream;
#define GLUE_BWD(TT, MM) ISSM_LAUNCH((k_glue_bwd<TT, MM>), blocks, 128, 0, s, a, npoints)
  if (p->io_dtype == ISSM_F32) {
    if (p->nfeat == 16) GLUE_BWD(float, 16); else if (p->nfeat == 8) GLUE_BWD(float, 8); else GLUE_BWD(float, 4);
  } else {
    if (p->nfeat == 16) GLUE_BWD(bf16, 16); else if (p->nfeat == 8) GLUE_BWD(bf16, 8); else GLUE_BWD(bf16, 4);
  }
#undef GLUE_BWD
  const int n = a.RW * p->nfeat;
  ISSM_LAUNCH(k_glue_reduce, (n + 31) / 32, dim3(32, 8), 0, s, a.dwpart, blocks, GLUE_MAX_ROWS * p->nfeat, n, p->dweight);
  return ISSM_OK;
}
