// The two point-wise steps on either side of the scan in the detector's ISSM block:
//  * serialization gather  dst[b, i, :] = src[b, index[b, i], :]   (models/dest_module.py:378-397, points.gather(dim=1, ...))
//  * PointLiteConv         y = silu(depthwise conv1d(k = 7, padding 3) over the point axis + bias), channels-last
//                          (models/dest_module.py:400-423; nn.Conv1d(groups = channels) applied to the transposed tensor)
// Both are memory-bound.  The convolution keeps a 7-row window per (thread, channel) in registers and walks a tile of
// rows, so every input row is read once per tile (plus a 6-row halo); threads of a warp own consecutive channels, so
// every access is coalesced.  Gradients of weight and bias are accumulated per block and reduced in a fixed order.
#include "issm_common.cuh"

namespace issm {

constexpr int CONV_K = 7, CONV_PAD = 3;


// ---- gather ----------------------------------------------------------------------------------------------
// one warp per destination row; VEC = bytes per lane access (16, 4 or 2)
template <int VEC>
__global__ void k_gather_rows(const char* __restrict__ src, const int64_t* __restrict__ index, char* __restrict__ dst,
                              int n_out, int n_src, int64_t row_bytes, int64_t src_batch_bytes, int64_t src_row_bytes, int* status) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y;
  if (warp >= n_out) return;
  int64_t j = index[(int64_t)b * n_out + warp];
  if (j < 0 || j >= n_src) {                               // an index outside the source: flag it, copy nothing
    if (lane == 0 && status) atomicOr(status, 2);
    return;
  }
  const char* s = src + b * src_batch_bytes + j * src_row_bytes;
  char* d = dst + ((int64_t)b * n_out + warp) * row_bytes;
  for (int64_t o = (int64_t)lane * VEC; o < row_bytes; o += 32 * VEC) {
    if (VEC == 16) *(uint4*)(d + o) = *(const uint4*)(s + o);
    else if (VEC == 4) *(uint32_t*)(d + o) = *(const uint32_t*)(s + o);
    else *(uint16_t*)(d + o) = *(const uint16_t*)(s + o);
  }
}

// ---- depthwise conv + silu ---------------------------------------------------------------------------------
// A block is 32 channel slots (x; a slot is V adjacent channels) by 8 row segments (y) of `tr` rows each; a warp reads
// 32 * V consecutive channels of one row per access.  V = 2 (one 4- or 8-byte access per thread) when the channel
// count, the strides and the pointers allow it, else 1.
struct ConvArgs {
  int B, N, C, tr;
  const void* x; int64_t x_sb, x_sl;
  const float* w; const float* bias;
  void* y;                                                 // forward output (B, N, C) contiguous
  const void* dy; int64_t dy_sb, dy_sl;
  void* dx;                                                // (B, N, C) contiguous
  float* part;                                             // (B * gridDim.y, C, 8): dw[0..6], dbias partials
};
constexpr int CONV_SEGS = 8;
constexpr int CONV_R = 8;                                 // rows loaded ahead of their use

// The value a thread carries per row: one channel (float) or two adjacent ones (float2, packed fp32 arithmetic).
template <int V> struct Val { using t = float; };
template <> struct Val<2> { using t = float2; };

__device__ __forceinline__ float ex2_ftz(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp_ftz(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ void vzero(float& v) { v = 0.f; }
__device__ __forceinline__ void vzero(float2& v) { v = make_float2(0.f, 0.f); }
__device__ __forceinline__ float vfma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ float2 vfma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float vmul(float a, float b) { return a * b; }
__device__ __forceinline__ float2 vmul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float vadd(float a, float b) { return a + b; }
__device__ __forceinline__ float2 vadd(float2 a, float2 b) { return __fadd2_rn(a, b); }
// 1 / (1 + 2^(-v log2 e)); exact 0 and 1 at the two ends of the range
__device__ __forceinline__ float vsigmoid(float v) { return rcp_ftz(1.f + ex2_ftz(-1.4426950408889634f * v)); }
__device__ __forceinline__ float2 vsigmoid(float2 v) {
  const float2 t = __fmul2_rn(v, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  const float2 e = __fadd2_rn(make_float2(ex2_ftz(t.x), ex2_ftz(t.y)), make_float2(1.f, 1.f));
  return make_float2(rcp_ftz(e.x), rcp_ftz(e.y));
}
// silu'(pre) = s (1 + pre (1 - s))
__device__ __forceinline__ float vdsilu(float pre, float s) { return s * fmaf(pre, 1.f - s, 1.f); }
__device__ __forceinline__ float2 vdsilu(float2 pre, float2 s) {
  const float2 one = make_float2(1.f, 1.f);
  return __fmul2_rn(s, __ffma2_rn(pre, make_float2(1.f - s.x, 1.f - s.y), one));
}
__device__ __forceinline__ float vlane(float v, int) { return v; }
__device__ __forceinline__ float vlane(float2 v, int i) { return i ? v.y : v.x; }

__device__ __forceinline__ void ldv(const float* p, float& v) { v = *p; }
__device__ __forceinline__ void ldv(const float* p, float2& v) { v = *(const float2*)p; }
__device__ __forceinline__ void ldv(const bf16* p, float& v) { v = __bfloat162float(*p); }
__device__ __forceinline__ void ldv(const bf16* p, float2& v) { v = __bfloat1622float2(*(const __nv_bfloat162*)p); }
__device__ __forceinline__ void stv(float* p, float v) { *p = v; }
__device__ __forceinline__ void stv(float* p, float2 v) { *(float2*)p = v; }
__device__ __forceinline__ void stv(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void stv(bf16* p, float2 v) { *(__nv_bfloat162*)p = __float22bfloat162_rn(v); }
__device__ __forceinline__ void ldw(const float* w, int C, int c, int stride, int k, float& v) { v = w[c * stride + k]; }
__device__ __forceinline__ void ldw(const float* w, int C, int c, int stride, int k, float2& v) {
  v = make_float2(w[c * stride + k], w[(c + 1) * stride + k]);
}

template <typename T, int V>
__global__ void __launch_bounds__(256) k_dwconv7_silu_fwd(ConvArgs a) {
  using F = typename Val<V>::t;
  constexpr int R = CONV_R;
  const int c = (blockIdx.x * 32 + threadIdx.x) * V;
  const int b = blockIdx.z;
  const int n0 = (blockIdx.y * CONV_SEGS + threadIdx.y) * a.tr, n1 = min(a.N, n0 + a.tr);
  if (c >= a.C || n0 >= a.N) return;
  const T* x = (const T*)a.x + b * a.x_sb + c;
  T* y = (T*)a.y + ((int64_t)b * a.N + n0) * a.C + c;
  F w[CONV_K], bias;
  vzero(bias);
  if (a.bias) ldw(a.bias, a.C, c, 1, 0, bias);
#pragma unroll
  for (int k = 0; k < CONV_K; ++k) ldw(a.w, a.C, c, CONV_K, k, w[k]);
  auto fetch = [&](int n, F& d) {
    if (n >= 0 && n < a.N) ldv(x + (int64_t)n * a.x_sl, d);
    else vzero(d);
  };
  // rows n - 3 .. n + R + 2 of a batch of R output rows; the R loads of a batch are issued before any is used
  F buf[CONV_K - 1 + R];
#pragma unroll
  for (int k = 0; k < CONV_K - 1; ++k) fetch(n0 - CONV_PAD + k, buf[k]);
  for (int n = n0; n < n1; n += R) {
    if (n + CONV_PAD + R <= a.N) {                         // the whole batch lies inside the sequence: no per-row test
      const T* px = x + (int64_t)(n + CONV_PAD) * a.x_sl;
#pragma unroll
      for (int r = 0; r < R; ++r) ldv(px + (int64_t)r * a.x_sl, buf[CONV_K - 1 + r]);
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) fetch(n + CONV_PAD + r, buf[CONV_K - 1 + r]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (n + r < n1) {
        F pre = bias;
#pragma unroll
        for (int k = 0; k < CONV_K; ++k) pre = vfma(w[k], buf[r + k], pre);
        stv(y + (int64_t)r * a.C, vmul(pre, vsigmoid(pre)));
      }
    }
    y += (int64_t)R * a.C;
#pragma unroll
    for (int k = 0; k < CONV_K - 1; ++k) buf[k] = buf[R + k];
  }
}

// Backward in one pass: g[m] = dy[m] * dsilu(pre[m]) is recomputed for the 3 halo rows on either side of the segment
// and kept in a 7-row register window, so dx[n] = sum_k w[k] g[n - k + 3] needs no intermediate in global memory.
template <typename T, int V>
__global__ void __launch_bounds__(256) k_dwconv7_silu_bwd(ConvArgs a) {
  using F = typename Val<V>::t;
  constexpr int R = CONV_R;
  __shared__ float red[CONV_SEGS][8][32 * V];
  const int c = (blockIdx.x * 32 + threadIdx.x) * V;
  const int b = blockIdx.z;
  const int n0 = (blockIdx.y * CONV_SEGS + threadIdx.y) * a.tr, n1 = min(a.N, n0 + a.tr);
  const bool live = c < a.C && n0 < a.N;
  F dw[CONV_K], db;
  vzero(db);
#pragma unroll
  for (int k = 0; k < CONV_K; ++k) vzero(dw[k]);
  if (live) {
    const T* x = (const T*)a.x + b * a.x_sb + c;
    const T* dy = (const T*)a.dy + b * a.dy_sb + c;
    T* dx = (T*)a.dx + (int64_t)b * a.N * a.C + c;
    F w[CONV_K], bias;
    vzero(bias);
    if (a.bias) ldw(a.bias, a.C, c, 1, 0, bias);
#pragma unroll
    for (int k = 0; k < CONV_K; ++k) ldw(a.w, a.C, c, CONV_K, k, w[k]);
    auto fetch = [&](const T* base, int64_t stride, int n, F& d) {
      if (n >= 0 && n < a.N) ldv(base + (int64_t)n * stride, d);
      else vzero(d);
    };
    F xb[CONV_K - 1 + R], gyb[R], gb[CONV_K - 1 + R];      // x[m - 3 .. m + R + 2]; dy[m .. m + R); g[m - 6 .. m + R)
    const int m0 = n0 - CONV_PAD, m1 = n1 + CONV_PAD;
#pragma unroll
    for (int k = 0; k < CONV_K - 1; ++k) fetch(x, a.x_sl, m0 - CONV_PAD + k, xb[k]);
#pragma unroll
    for (int k = 0; k < CONV_K - 1; ++k) vzero(gb[k]);
    for (int mb = m0; mb < m1; mb += R) {
      if (mb >= 0 && mb + CONV_PAD + R <= a.N) {           // whole batch inside the sequence
        const T* px = x + (int64_t)(mb + CONV_PAD) * a.x_sl;
        const T* pg = dy + (int64_t)mb * a.dy_sl;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          ldv(px + (int64_t)r * a.x_sl, xb[CONV_K - 1 + r]);
          ldv(pg + (int64_t)r * a.dy_sl, gyb[r]);
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          fetch(x, a.x_sl, mb + CONV_PAD + r, xb[CONV_K - 1 + r]);
          fetch(dy, a.dy_sl, mb + r, gyb[r]);              // zero outside the sequence, so g is zero there too
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int m = mb + r;
        if (m < m1) {
          F pre = bias;
#pragma unroll
          for (int k = 0; k < CONV_K; ++k) pre = vfma(w[k], xb[r + k], pre);
          const F g = vmul(gyb[r], vdsilu(pre, vsigmoid(pre)));
          gb[CONV_K - 1 + r] = g;
          if (m >= n0 && m < n1) {                         // rows of this segment; halo rows belong to a neighbour
            db = vadd(db, g);
#pragma unroll
            for (int k = 0; k < CONV_K; ++k) dw[k] = vfma(g, xb[r + k], dw[k]);
          }
          const int n = m - CONV_PAD;                      // gb[r .. r + 6] = g[n - 3 .. n + 3]
          if (n >= n0) {
            F acc;
            vzero(acc);
#pragma unroll
            for (int k = 0; k < CONV_K; ++k) acc = vfma(w[k], gb[r + CONV_K - 1 - k], acc);
            stv(dx + (int64_t)n * a.C, acc);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < CONV_K - 1; ++k) { xb[k] = xb[R + k]; gb[k] = gb[R + k]; }
    }
  }
  // the block's 8 segments, summed in a fixed order
#pragma unroll
  for (int v = 0; v < V; ++v) {
#pragma unroll
    for (int k = 0; k < CONV_K; ++k) red[threadIdx.y][k][threadIdx.x * V + v] = vlane(dw[k], v);
    red[threadIdx.y][7][threadIdx.x * V + v] = vlane(db, v);
  }
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;
  for (int i = t; i < 8 * 32 * V; i += 256) {
    const int k = i / (32 * V), cc = i % (32 * V);
    const int cg = blockIdx.x * 32 * V + cc;
    if (cg >= a.C) continue;
    float acc = 0.f;
#pragma unroll
    for (int sgm = 0; sgm < CONV_SEGS; ++sgm) acc += red[sgm][k][cc];
    a.part[(((size_t)b * gridDim.y + blockIdx.y) * a.C + cg) * 8 + k] = acc;
  }
}

// dweight (C, 7) and dbias (C) from the per-block partials: 32 (channel, tap) slots by 8 groups per block; a group sums
// its contiguous share of the partial rows, the groups are combined in a fixed order.
__global__ void __launch_bounds__(256) k_conv_reduce(const float* __restrict__ part, int blocks, int C, float* __restrict__ dw, float* __restrict__ db) {
  __shared__ float red[8][32];
  const int i = blockIdx.x * 32 + threadIdx.x;             // over (c, 8)
  const int grp = threadIdx.y;
  const int per = (blocks + 7) / 8;
  float acc = 0.f;
  if (i < C * 8) {
    const int j1 = min(blocks, (grp + 1) * per);
#pragma unroll 4
    for (int j = grp * per; j < j1; ++j) acc += part[(size_t)j * C * 8 + i];
  }
  red[grp][threadIdx.x] = acc;
  __syncthreads();
  if (grp == 0 && i < C * 8) {
    float tot = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < 8; ++g2) tot += red[g2][threadIdx.x];
    const int c = i >> 3, k = i & 7;
    if (k < CONV_K) dw[c * CONV_K + k] = tot;
    else if (db) db[c] = tot;
  }
}

struct ConvPlan { int V, tr; dim3 grid; };
static ConvPlan conv_plan(const issm_conv_params& p, bool bwd) {
  ConvPlan pl;
  const size_t es = p.io_dtype == ISSM_F32 ? 4 : 2;
  auto ok2 = [&](const void* q, int64_t sb, int64_t sl) { return !(((uintptr_t)q) % (2 * es)) && !(sb & 1) && !(sl & 1); };
  bool v2 = !(p.channels & 1) && ok2(p.x, p.x_sb, p.x_sl);
  if (!bwd) v2 = v2 && ok2(p.y, 0, 0);
  else v2 = v2 && ok2(p.dy, p.dy_sb, p.dy_sl) && ok2(p.dx, 0, 0);
  pl.V = v2 ? 2 : 1;
  const int slots = (p.channels + pl.V - 1) / pl.V;
  const int gx = (slots + 31) / 32;
  auto gy = [&](int tr) { return (p.seqlen + tr * CONV_SEGS - 1) / (tr * CONV_SEGS); };
  // long segments (fewer halo rows) when there are enough blocks to fill the GPU several times over
  pl.tr = ((int64_t)gx * gy(128) * p.batch >= 148 * 8) ? 128 : ((int64_t)gx * gy(64) * p.batch >= 148 * 4) ? 64 : 16;
  pl.grid = dim3(gx, gy(pl.tr), p.batch);
  return pl;
}

static int conv_validate(const issm_conv_params* p, bool bwd) {
  if (!p) return ISSM_ERR_NULL;
  if (p->batch <= 0 || p->seqlen <= 0 || p->channels <= 0 || p->batch > 65535) return ISSM_ERR_SHAPE;
  if (((int64_t)p->seqlen + 16 * CONV_SEGS - 1) / (16 * CONV_SEGS) > 65535) return ISSM_ERR_SHAPE;   // grid.y of the shortest segments
  if (p->io_dtype != ISSM_F32 && p->io_dtype != ISSM_BF16) return ISSM_ERR_DTYPE;
  if (!p->x || !p->weight) return ISSM_ERR_NULL;
  if (!bwd && !p->y) return ISSM_ERR_NULL;
  if (bwd && (!p->dy || !p->dx || !p->dweight)) return ISSM_ERR_NULL;
  return ISSM_OK;
}
static ConvArgs conv_args(const issm_conv_params& p) {
  ConvArgs a{};
  a.B = p.batch; a.N = p.seqlen; a.C = p.channels;
  a.x = p.x; a.x_sb = p.x_sb; a.x_sl = p.x_sl;
  a.w = p.weight; a.bias = p.bias; a.y = p.y;
  a.dy = p.dy; a.dy_sb = p.dy_sb; a.dy_sl = p.dy_sl; a.dx = p.dx;
  return a;
}
}  // namespace issm

using namespace issm;

extern "C" int issm_b200_gather_rows(const void* src, const int64_t* index, void* dst, int32_t batch, int32_t n_out, int32_t n_src,
                                     int64_t row_bytes, int64_t src_batch_bytes, int64_t src_row_bytes, int32_t* status, void* stream) {
  if (!src || !index || !dst) return ISSM_ERR_NULL;
  if (batch <= 0 || batch > 65535 || n_out <= 0 || n_src <= 0 || row_bytes <= 0 || (row_bytes & 1)) return ISSM_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((n_out + 7) / 8, batch);
  const bool a16 = !(((uintptr_t)src | (uintptr_t)dst | (uintptr_t)row_bytes | (uintptr_t)src_batch_bytes | (uintptr_t)src_row_bytes) & 15);
  const bool a4 = !(((uintptr_t)src | (uintptr_t)dst | (uintptr_t)row_bytes | (uintptr_t)src_batch_bytes | (uintptr_t)src_row_bytes) & 3);
  if (a16) ISSM_LAUNCH(k_gather_rows<16>, grid, 256, 0, s, (const char*)src, index, (char*)dst, n_out, n_src, row_bytes, src_batch_bytes, src_row_bytes, status);
  else if (a4) ISSM_LAUNCH(k_gather_rows<4>, grid, 256, 0, s, (const char*)src, index, (char*)dst, n_out, n_src, row_bytes, src_batch_bytes, src_row_bytes, status);
  else ISSM_LAUNCH(k_gather_rows<2>, grid, 256, 0, s, (const char*)src, index, (char*)dst, n_out, n_src, row_bytes, src_batch_bytes, src_row_bytes, status);
  return ISSM_OK;
}

extern "C" size_t issm_b200_sizeof_conv_params(void) { return sizeof(issm_conv_params); }

extern "C" size_t issm_b200_dwconv_workspace_bytes(const issm_conv_params* p) {
  if (!p || p->batch <= 0 || p->seqlen <= 0 || p->channels <= 0) return 0;
  // partial rows for the smallest segment length, so the size does not depend on pointer alignment
  const size_t rows = (size_t)((p->seqlen + 16 * CONV_SEGS - 1) / (16 * CONV_SEGS)) * p->batch;
  return align_up(rows * p->channels * 8 * sizeof(float), 256);
}

#define CONV_DISPATCH(KERNEL, pl, s, a)                                                               \
  do {                                                                                                \
    const dim3 blk(32, CONV_SEGS);                                                                    \
    if (p->io_dtype == ISSM_F32) {                                                                    \
      if (pl.V == 2) ISSM_LAUNCH((KERNEL<float, 2>), pl.grid, blk, 0, s, a);                          \
      else ISSM_LAUNCH((KERNEL<float, 1>), pl.grid, blk, 0, s, a);                                    \
    } else {                                                                                          \
      if (pl.V == 2) ISSM_LAUNCH((KERNEL<bf16, 2>), pl.grid, blk, 0, s, a);                           \
      else ISSM_LAUNCH((KERNEL<bf16, 1>), pl.grid, blk, 0, s, a);                                     \
    }                                                                                                 \
  } while (0)

extern "C" int issm_b200_dwconv7_silu_fwd(const issm_conv_params* p, void* stream) {
  int rc = conv_validate(p, false);
  if (rc) return rc;
  const ConvPlan pl = conv_plan(*p, false);
  ConvArgs a = conv_args(*p);
  a.tr = pl.tr;
  CONV_DISPATCH(k_dwconv7_silu_fwd, pl, (cudaStream_t)stream, a);
  return ISSM_OK;
}

extern "C" int issm_b200_dwconv7_silu_bwd(const issm_conv_params* p, void* stream) {
  int rc = conv_validate(p, true);
  if (rc) return rc;
  if (!p->workspace || p->workspace_bytes < issm_b200_dwconv_workspace_bytes(p)) return ISSM_ERR_WORKSPACE;
  if ((uintptr_t)p->workspace % 256) return ISSM_ERR_ALIGN;
  const ConvPlan pl = conv_plan(*p, true);
  ConvArgs a = conv_args(*p);
  a.tr = pl.tr;
  a.part = (float*)p->workspace;
  cudaStream_t s = (cudaStream_t)stream;
  CONV_DISPATCH(k_dwconv7_silu_bwd, pl, s, a);
  ISSM_LAUNCH(k_conv_reduce, (p->channels * 8 + 31) / 32, dim3(32, 8), 0, s, a.part, (int)(pl.grid.y * pl.grid.z), p->channels, p->dweight, p->dbias);
  return ISSM_OK;
}
