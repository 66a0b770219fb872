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

// softplus with threshold 20 in the log2 domain (hardware ex2 / lg2); below -4 the series of log1p in u = e^v, where
// lg2(1 + u) would lose the low bits of u
__device__ __forceinline__ float glue_softplus(float v) {
  float u, s;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(u) : "f"(v * 1.4426950408889634f));
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(1.f + u));
  const float series = u * fmaf(u, fmaf(u, 0.33333333f, -0.5f), 1.f);
  const float r = v < -4.f ? series : s * 0.6931471805599453f;
  return v <= 20.f ? r : v;
}

// one block per point (b, l); a thread owns two adjacent states and computes them with packed fp32 instructions,
// reading four weights per shared-memory access
// TD: element type of dist (and ddist), T: of dt / bc and their gradients (float dist with bfloat16 outputs is what
// autocast hands the block: the features stay float32, the activations are bfloat16)
template <typename TD, typename T, int M>
__global__ void __launch_bounds__(128) k_glue_fwd(GlueArgs a) {
  __shared__ __align__(16) float sw[GLUE_MAX_ROWS * M];
  __shared__ float stok[GLUE_MAX_ROWS + 8];
  const int l = blockIdx.x, b = blockIdx.y;
  for (int i = threadIdx.x; i < a.RW * M; i += blockDim.x) sw[i] = a.w[i];
  for (int i = threadIdx.x; i < a.RO; i += blockDim.x) stok[i] = a.tok[((int64_t)b * a.L + l) * a.RO + i];
  __syncthreads();
  const TD* drow = (const TD*)a.dist + b * a.d_sb + l * a.d_sl;
  const int64_t row = (int64_t)b * a.L + l;
  T* dt = (T*)a.dt + row * a.H * a.K;
  T* bc = (T*)a.bc + row * (a.RO - a.H) * a.K;
  const bool pair_store = !(a.K & 1);                      // rows of an even number of states keep pairs aligned
  for (int k = 2 * threadIdx.x; k < a.K; k += 2 * blockDim.x) {
    const bool two = k + 1 < a.K;
    float d0[M], d1[M];
    load_feats<TD, M>(drow + (int64_t)k * a.d_sk, d0);
    load_feats<TD, M>(drow + (int64_t)(two ? k + 1 : k) * a.d_sk, d1);
    float2 dp[M];
#pragma unroll
    for (int j = 0; j < M; ++j) dp[j] = make_float2(d0[j], d1[j]);
    float2 mk = make_float2(1.f, 1.f);
    if (a.mask) mk = make_float2(a.mask[row * a.K + k], a.mask[row * a.K + (two ? k + 1 : k)]);
    auto put = [&](T* p, float2 v) {
      if (pair_store) {
        if constexpr (sizeof(T) == 2) *(__nv_bfloat162*)p = __float22bfloat162_rn(v);
        else *(float2*)p = v;
      } else {
        stf(p, v.x);
        if (two) stf(p + 1, v.y);
      }
    };
    for (int r = 0; r < a.RW; ++r) {
      float2 pre = make_float2(stok[r], stok[r]);
#pragma unroll
      for (int c = 0; c < M / 4; ++c) {
        const float4 w4 = *(const float4*)&sw[r * M + c * 4];
        pre = __ffma2_rn(dp[c * 4], make_float2(w4.x, w4.x), pre);
        pre = __ffma2_rn(dp[c * 4 + 1], make_float2(w4.y, w4.y), pre);
        pre = __ffma2_rn(dp[c * 4 + 2], make_float2(w4.z, w4.z), pre);
        pre = __ffma2_rn(dp[c * 4 + 3], make_float2(w4.w, w4.w), pre);
      }
      if (r < a.H) {
        put(dt + (int64_t)r * a.K + k, __fmul2_rn(make_float2(glue_softplus(pre.x), glue_softplus(pre.y)), mk));
      } else {
        put(bc + (int64_t)(r - a.H) * a.K + k, pre);
        if (a.back) {
          const float dlt = stok[r + 2 * a.G] - stok[r];
          put(bc + (int64_t)(r - a.H + 2 * a.G) * a.K + k, __fadd2_rn(pre, make_float2(dlt, dlt)));
        }
      }
    }
  }
}

constexpr int GLUE_KT = 256;                               // states per shared-memory tile of the weight-gradient product
constexpr int GLUE_BWD_BLOCKS = 148 * 8;

__device__ __forceinline__ void cp_async(void* smem_dst, const void* gsrc, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if (bytes == 16) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
  else if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gsrc) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One stage of the backward's input pipeline: everything a (point, tile of 256 states) needs, as raw bytes.  The
// number of gradient rows is the call's (RO), so the layout is computed at run time.
template <typename TD, typename T, int M>
struct GlueStage {
  unsigned char* base;
  int ro;
  __host__ __device__ static size_t bytes(int ro) {
    return ((size_t)GLUE_KT * M * sizeof(TD) + (size_t)ro * GLUE_KT * sizeof(T) + GLUE_KT * 4 + (GLUE_MAX_ROWS + 8) * 4 + 15) / 16 * 16;
  }
  __device__ TD* dist(int kk) const { return (TD*)base + (size_t)kk * M; }                       // [GLUE_KT][M]
  __device__ T* grad(int r) const { return (T*)(base + (size_t)GLUE_KT * M * sizeof(TD)) + (size_t)r * GLUE_KT; }   // ddt rows, then the B / C rows
  __device__ float* mask() const { return (float*)(base + (size_t)GLUE_KT * (M * sizeof(TD) + ro * sizeof(T))); }
  __device__ float* tok() const { return mask() + GLUE_KT; }
};

// A block walks (point, tile of 256 states) items with a grid stride over the points, two items in flight: the
// inputs of the next item are copied into shared memory (cp.async) while the current one is computed.  Per item:
// (1) a thread takes two adjacent states: g, ddist, token sums; g and the features are parked in shared memory;
// (2) thread (row r, four features, a range of the tile's states) adds sum_k g[r, k] dist[k, j] to its accumulators of
// the weight gradient.  The accumulators go out once per block and are summed in a fixed order.
template <typename TD, typename T, int M>
__global__ void __launch_bounds__(128) k_glue_bwd(GlueArgs a, int npoints, int vec_ok) {
  extern __shared__ __align__(16) unsigned char glue_dyn[];
  const size_t stage_bytes = GlueStage<TD, T, M>::bytes(a.RO);
  auto stage_of = [&](int it) { return GlueStage<TD, T, M>{glue_dyn + (it & 1) * stage_bytes, a.RO}; };
  __shared__ __align__(16) float sw[GLUE_MAX_ROWS * M];
  __shared__ float sred[4][GLUE_MAX_ROWS + 8];
  __shared__ __align__(16) float sg[GLUE_MAX_ROWS][GLUE_KT + 4];   // g of the tile, read four states at a time
  // float copy of the tile's features for the weight gradient (rows 16 bytes apart from a power of two: 128-bit accesses
  // without conflicts); float features are read from the stage itself
  constexpr bool kCopy = sizeof(TD) != 4;
  __shared__ __align__(16) float sd[kCopy ? GLUE_KT : 1][M + 4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < a.RW * M; i += blockDim.x) sw[i] = a.w[i];
  // weight gradient: thread = (row r, four features 4 jq .. 4 jq + 3, one of NKG ranges of the tile's states)
  constexpr int JQ = M / 4;
  const int tiles = a.RW * JQ, NKG = 128 / tiles > 0 ? 128 / tiles : 1;
  const int tile = threadIdx.x % tiles, kg = threadIdx.x / tiles;
  const int wr = tile / JQ, wj = (tile % JQ) * 4;
  const int kspan = ((GLUE_KT + NKG - 1) / NKG + 3) & ~3;  // a multiple of four states
  float wacc[4] = {0.f, 0.f, 0.f, 0.f};
  const int ntile = (a.K + GLUE_KT - 1) / GLUE_KT;
  const int my_points = blockIdx.x < npoints ? (npoints - blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nitems = my_points * ntile;

  // copies of item `it` into stage `st`.  vec_ok: every row of states starts on a 16-byte boundary, so the gradient rows
  // and the mask go in 16-byte pieces; otherwise element by element through registers.
  auto issue = [&](int it, const GlueStage<TD, T, M>& st) {
    const int pt = blockIdx.x + (it / ntile) * gridDim.x, k0 = (it % ntile) * GLUE_KT;
    const int b = pt / a.L, l = pt - b * a.L;
    const int nk = min(GLUE_KT, a.K - k0);
    const TD* drow = (const TD*)a.dist + b * a.d_sb + l * a.d_sl + (int64_t)k0 * a.d_sk;
    constexpr int RB = M * (int)sizeof(TD), CS = RB >= 16 ? 16 : RB, CH = RB / CS;     // bytes per state, per piece, pieces per state
    for (int c = threadIdx.x; c < nk * CH; c += blockDim.x) {
      const int kk = c / CH, part = c % CH;
      cp_async((char*)st.dist(kk) + part * CS, (const char*)(drow + (int64_t)kk * a.d_sk) + part * CS, CS);
    }
    const int nrow = a.RO;
    const T* ddt = a.ddt ? (const T*)a.ddt + (int64_t)pt * a.H * a.K + k0 : nullptr;
    const T* dbc = a.dbc ? (const T*)a.dbc + (int64_t)pt * (a.RO - a.H) * a.K + k0 : nullptr;
    constexpr int EPC = 16 / (int)sizeof(T);               // elements per 16-byte piece
    if (vec_ok) {
      const int pieces = nk / EPC;                         // K is a multiple of EPC here
      for (int c = threadIdx.x; c < nrow * pieces; c += blockDim.x) {
        const int ro = c / pieces, q = c % pieces;
        const T* src = ro < a.H ? (ddt ? ddt + (int64_t)ro * a.K : nullptr) : (dbc ? dbc + (int64_t)(ro - a.H) * a.K : nullptr);
        if (src) cp_async(st.grad(ro) + q * EPC, src + q * EPC, 16);
      }
      if (a.mask)
        for (int c = threadIdx.x; c < nk / 4; c += blockDim.x) cp_async(st.mask() + c * 4, a.mask + (int64_t)pt * a.K + k0 + c * 4, 16);
    } else {
      for (int c = threadIdx.x; c < nrow * nk; c += blockDim.x) {
        const int ro = c / nk, kk = c % nk;
        const T* src = ro < a.H ? (ddt ? ddt + (int64_t)ro * a.K : nullptr) : (dbc ? dbc + (int64_t)(ro - a.H) * a.K : nullptr);
        if (src) st.grad(ro)[kk] = src[kk];
      }
      if (a.mask)
        for (int c = threadIdx.x; c < nk; c += blockDim.x) st.mask()[c] = a.mask[(int64_t)pt * a.K + k0 + c];
    }
    for (int i = threadIdx.x; i < a.RO; i += blockDim.x) cp_async(st.tok() + i, a.tok + (int64_t)pt * a.RO + i, 4);
    cp_async_commit();
  };

  float tsum[GLUE_MAX_ROWS + 8];                            // per output row: sum over this thread's states of the point
#pragma unroll
  for (int r = 0; r < GLUE_MAX_ROWS + 8; ++r) tsum[r] = 0.f;
  if (nitems > 0) issue(0, stage_of(0));
  for (int it = 0; it < nitems; ++it) {
    const GlueStage<TD, T, M> st = stage_of(it);
    if (it + 1 < nitems) { issue(it + 1, stage_of(it + 1)); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();                                       // this item's inputs are in shared memory
    const int pt = blockIdx.x + (it / ntile) * gridDim.x, k0 = (it % ntile) * GLUE_KT;
    const int64_t row = pt;
    TD* ddist = (TD*)a.ddist + row * a.K * M;
    {                                                      // two adjacent states per thread: 128 threads cover the tile
      const int kk = 2 * threadIdx.x, k = k0 + kk;
      const bool in0 = k < a.K, in1 = k + 1 < a.K;
      float d0[M], d1[M];
#pragma unroll
      for (int j = 0; j < M; ++j) { d0[j] = 0.f; d1[j] = 0.f; }
      if (in0) load_feats<TD, M>(st.dist(kk), d0);
      if (in1) load_feats<TD, M>(st.dist(kk + 1), d1);
      float2 dp[M], dd[M];
#pragma unroll
      for (int j = 0; j < M; ++j) { dp[j] = make_float2(d0[j], d1[j]); dd[j] = make_float2(0.f, 0.f); }
      if constexpr (kCopy) {
#pragma unroll
        for (int c = 0; c < M / 4; ++c) {
          *(float4*)&sd[kk][c * 4] = make_float4(d0[c * 4], d0[c * 4 + 1], d0[c * 4 + 2], d0[c * 4 + 3]);
          *(float4*)&sd[kk + 1][c * 4] = make_float4(d1[c * 4], d1[c * 4 + 1], d1[c * 4 + 2], d1[c * 4 + 3]);
        }
      } else {                                             // rows of the stage beyond the last state: zero, not stale
#pragma unroll
        for (int c = 0; c < M / 4; ++c) {
          if (!in0) *(float4*)((float*)st.dist(kk) + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
          if (!in1) *(float4*)((float*)st.dist(kk + 1) + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      const float2 inm = make_float2(in0 ? 1.f : 0.f, in1 ? 1.f : 0.f);
      float2 mk = inm;
      if (a.mask) mk = make_float2(in0 ? st.mask()[kk] : 0.f, in1 ? st.mask()[kk + 1] : 0.f);
      auto get = [&](int ro) {                             // the pair (k, k + 1) of one gradient row; zero outside the row
        float2 v;
        if constexpr (sizeof(T) == 2) v = __bfloat1622float2(*(const __nv_bfloat162*)(st.grad(ro) + kk));
        else v = *(const float2*)(st.grad(ro) + kk);
        return make_float2(in0 ? v.x : 0.f, in1 ? v.y : 0.f);
      };
#pragma unroll
      for (int r = 0; r < GLUE_MAX_ROWS; ++r) {
        if (r < a.RW) {
          float2 g = make_float2(0.f, 0.f);
          float4 wrow[M / 4];                              // the row's weights: read once, used for pre and for ddist
#pragma unroll
          for (int c = 0; c < M / 4; ++c) wrow[c] = *(const float4*)&sw[r * M + c * 4];
          if (r < a.H) {
            if (a.ddt) {
              float2 pre = make_float2(st.tok()[r], st.tok()[r]);
#pragma unroll
              for (int c = 0; c < M / 4; ++c) {
                pre = __ffma2_rn(dp[c * 4], make_float2(wrow[c].x, wrow[c].x), pre);
                pre = __ffma2_rn(dp[c * 4 + 1], make_float2(wrow[c].y, wrow[c].y), pre);
                pre = __ffma2_rn(dp[c * 4 + 2], make_float2(wrow[c].z, wrow[c].z), pre);
                pre = __ffma2_rn(dp[c * 4 + 3], make_float2(wrow[c].w, wrow[c].w), pre);
              }
              const float2 sg2 = make_float2(pre.x <= 20.f ? glue_sigmoid(pre.x) : 1.f, pre.y <= 20.f ? glue_sigmoid(pre.y) : 1.f);
              g = __fmul2_rn(__fmul2_rn(get(r), mk), sg2);
            }
            tsum[r] += g.x + g.y;
          } else if (a.dbc) {
            g = get(r);
            if (a.back) g = __fadd2_rn(g, get(r + 2 * a.G));   // both directions share the weight row
          }
          *(float2*)&sg[r][kk] = g;
#pragma unroll
          for (int c = 0; c < M / 4; ++c) {
            dd[c * 4] = __ffma2_rn(g, make_float2(wrow[c].x, wrow[c].x), dd[c * 4]);
            dd[c * 4 + 1] = __ffma2_rn(g, make_float2(wrow[c].y, wrow[c].y), dd[c * 4 + 1]);
            dd[c * 4 + 2] = __ffma2_rn(g, make_float2(wrow[c].z, wrow[c].z), dd[c * 4 + 2]);
            dd[c * 4 + 3] = __ffma2_rn(g, make_float2(wrow[c].w, wrow[c].w), dd[c * 4 + 3]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < M; ++j) { d0[j] = dd[j].x; d1[j] = dd[j].y; }
      if (in0) store_feats<TD, M>(ddist + (int64_t)k * M, d0);
      if (in1) store_feats<TD, M>(ddist + (int64_t)(k + 1) * M, d1);
      if (a.dbc) {                                         // token terms of the B / C rows (each output row has its own)
#pragma unroll
        for (int ro = 0; ro < GLUE_MAX_ROWS + 8; ++ro)
          if (ro >= a.H && ro < a.RO) {
            const float2 v = get(ro);
            tsum[ro] += v.x + v.y;
          }
      }
    }
    __syncthreads();
    if (kg < NKG) {
      const int k1 = min(GLUE_KT, (kg + 1) * kspan);       // rows beyond the last state hold g = 0 and zero features
#pragma unroll 2
      for (int kk = kg * kspan; kk < k1; kk += 4) {
        const float4 g4 = *(const float4*)&sg[wr][kk];
        const float gs[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float4 f;
          if constexpr (kCopy) f = *(const float4*)&sd[kk + i][wj];
          else f = *(const float4*)((const float*)st.dist(kk + i) + wj);
          wacc[0] = fmaf(gs[i], f.x, wacc[0]); wacc[1] = fmaf(gs[i], f.y, wacc[1]);
          wacc[2] = fmaf(gs[i], f.z, wacc[2]); wacc[3] = fmaf(gs[i], f.w, wacc[3]);
        }
      }
    }
    if (k0 + GLUE_KT >= a.K) {
      // last tile of the point: token terms, summed over the states by warp shuffles, then the four warps in a fixed order
#pragma unroll
      for (int r = 0; r < GLUE_MAX_ROWS + 8; ++r) {
        if (r < a.RO) {
          float v = tsum[r];
#pragma unroll
          for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) sred[warp][r] = v;
        }
        tsum[r] = 0.f;
      }
      __syncthreads();
      for (int r = threadIdx.x; r < a.RO; r += blockDim.x)
        a.dtok[row * a.RO + r] = ((sred[0][r] + sred[1][r]) + sred[2][r]) + sred[3][r];
    }
    __syncthreads();                                       // sg / sd / sred and this stage may be overwritten
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
  if (p->dist_dtype != p->io_dtype && !(p->dist_dtype == ISSM_F32 && p->io_dtype == ISSM_BF16)) return ISSM_ERR_DTYPE;
  if (!p->dist || !p->weight || !p->tok) return ISSM_ERR_NULL;
  if (!bwd && (!p->dt || !p->bc)) return ISSM_ERR_NULL;
  if (bwd && (!p->ddist || !p->dweight || !p->dtok)) return ISSM_ERR_NULL;
  const size_t es = p->dist_dtype == ISSM_F32 ? 4 : 2;
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

#define GLUE_DISPATCH_M(KERNEL, TD, T)                                                                \
  do {                                                                                                \
    if (p->nfeat == 16) ISSM_LAUNCH((KERNEL<TD, T, 16>), grid, 128, 0, s, a);                         \
    else if (p->nfeat == 8) ISSM_LAUNCH((KERNEL<TD, T, 8>), grid, 128, 0, s, a);                      \
    else ISSM_LAUNCH((KERNEL<TD, T, 4>), grid, 128, 0, s, a);                                         \
  } while (0)
#define GLUE_DISPATCH(KERNEL)                                                                         \
  do {                                                                                                \
    const dim3 grid(p->seqlen, p->batch);                                                             \
    cudaStream_t s = (cudaStream_t)stream;                                                            \
    if (p->io_dtype == ISSM_F32) GLUE_DISPATCH_M(KERNEL, float, float);                               \
    else if (p->dist_dtype == ISSM_F32) GLUE_DISPATCH_M(KERNEL, float, bf16);                         \
    else GLUE_DISPATCH_M(KERNEL, bf16, bf16);                                                         \
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
  const size_t es = p->io_dtype == ISSM_F32 ? 4 : 2;
  // 16-byte copies of the gradient rows and the mask need every row of states to start on a 16-byte boundary
  const int vec_ok = !((p->nstates * es) % 16) && !(p->nstates % 4) && !((uintptr_t)p->ddt % 16) && !((uintptr_t)p->dbc % 16) &&
                     !((uintptr_t)p->mask % 16);
#define GLUE_BWD(TD, TT, MM)                                                                          \
  do {                                                                                                \
    const size_t dyn = 2 * GlueStage<TD, TT, MM>::bytes(a.RO);                                        \
    struct Tag {};                                                                                    \
    if (int rc2 = SmemAttrOnce<Tag>::set(k_glue_bwd<TD, TT, MM>, 2 * GlueStage<TD, TT, MM>::bytes(GLUE_MAX_ROWS + 8))) return rc2; \
    ISSM_LAUNCH((k_glue_bwd<TD, TT, MM>), blocks, 128, dyn, s, a, npoints, vec_ok);                   \
  } while (0)
#define GLUE_BWD_M(TD, TT)                                                                            \
  do {                                                                                                \
    if (p->nfeat == 16) GLUE_BWD(TD, TT, 16); else if (p->nfeat == 8) GLUE_BWD(TD, TT, 8); else GLUE_BWD(TD, TT, 4); \
  } while (0)
  if (p->io_dtype == ISSM_F32) GLUE_BWD_M(float, float);
  else if (p->dist_dtype == ISSM_F32) GLUE_BWD_M(float, bf16);
  else GLUE_BWD_M(bf16, bf16);
#undef GLUE_BWD_M
#undef GLUE_BWD
  const int n = a.RW * p->nfeat;
  ISSM_LAUNCH(k_glue_reduce, (n + 31) / 32, dim3(32, 8), 0, s, a.dwpart, blocks, GLUE_MAX_ROWS * p->nfeat, n, p->dweight);
  return ISSM_OK;
}
