// Gated RMS / Layer norm, forward and backward (issm_triton/layernorm_gated.py:35-95, 145-258).
// Memory-bound: one warp per row, statistics by warp shuffles.  Two families of kernels:
//  * k_norm_fwd_vec / k_norm_bwd_vec: one statistics group per row (the detector's case), rows that fit the warp's
//    registers and 16-byte aligned rows: every tensor is read ONCE with 128-bit loads, the row lives in registers
//    between the statistics and the output, and the weight / bias gradients accumulate in registers over the rows
//    of a warp (a lane always owns the same features);
//  * k_norm_fwd / k_norm_bwd: any group size, width and alignment (features strided over lanes, per-warp
//    shared-memory accumulators).
// Weight/bias gradients are reduced over warps and blocks in a fixed order without atomics, so results are
// bitwise reproducible.
#include "issm_common.cuh"

namespace issm {

// sigmoid through the hardware exponential and reciprocal (about 2 ulp each; the exact expf and IEEE division cost
// ~40 instructions per element and made these kernels compute-bound)
__device__ __forceinline__ float fast_sigmoid(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }
__device__ __forceinline__ float siluf_(float v) { return v * fast_sigmoid(v); }
__device__ __forceinline__ float dsiluf_(float v) {
  const float s = fast_sigmoid(v);
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

// ---- vector kernels ------------------------------------------------------------------------------------
// 16 bytes of a row as floats: 8 bf16 or 4 float values
template <typename T> struct Vec16;
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float* v) { unpack(*(const uint4*)p, v); }
  static __device__ __forceinline__ void unpack(uint4 w, float* v) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(u[i] << 16); v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store(bf16* p, const float* v) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      u[i] = *(const uint32_t*)&h;
    }
    *(uint4*)p = make_uint4(u[0], u[1], u[2], u[3]);
  }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) { unpack(*(const uint4*)p, v); }
  static __device__ __forceinline__ void unpack(uint4 w, float* v) {
    v[0] = __uint_as_float(w.x); v[1] = __uint_as_float(w.y); v[2] = __uint_as_float(w.z); v[3] = __uint_as_float(w.w);
  }
  static __device__ __forceinline__ void store(float* p, const float* v) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
};

// 16 bytes of a row whose start is only known to be 4-byte aligned (the gate z of the detector is a column slice of a
// wider projection output: its rows start 4 bytes off a 16-byte boundary)
__device__ __forceinline__ uint4 ld16(const void* p, bool aligned16) {
  if (aligned16) return *(const uint4*)p;
  const uint32_t* q = (const uint32_t*)p;
  return make_uint4(q[0], q[1], q[2], q[3]);
}

// Chunk c of lane `lane` covers features [(c * 32 + lane) * V, +V); CH chunks per lane cover up to 32 * V * CH features.
// TL = 1: the row is CH full chunks plus 32 more features, one per lane (feature CH * 32 * V + lane) - the detector's
// 288 = 256 + 32 - instead of one more chunk in which 4 lanes of 32 would work.
template <typename T, int CH, int TL>
__global__ void __launch_bounds__(256, CH == 1 ? 4 : 2) k_norm_fwd_vec(issm_norm_params np) {
  constexpr int V = Vec16<T>::N, FT = CH * 32 * V;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int H = np.hidden;
  const bool has_z = np.has_z != 0;
  const bool z16 = !(((uintptr_t)np.z | (uintptr_t)(np.z_sr * (int64_t)sizeof(T))) & 15);
  const bool pre_gate = has_z && !np.norm_before_gate, post_gate = has_z && np.norm_before_gate;
  // a warp walks rows first, first + warps, ...; the 16-byte loads of the next row are issued (kept packed, 4 registers
  // per chunk) before the current row is worked on (two rows ahead measured slower: 121 registers, fewer resident warps)
  uint4 nx[CH], nz[CH];
  float nxt = 0.f, nzt = 0.f;
  auto issue = [&](int row) {
    const T* x = (const T*)np.x + (int64_t)row * np.x_sr;
    const T* z = has_z ? (const T*)np.z + (int64_t)row * np.z_sr : nullptr;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int f0 = (c * 32 + lane) * V;
      if (f0 < H) {
        nx[c] = *(const uint4*)(x + f0);
        if (has_z) nz[c] = ld16(z + f0, z16);
      }
    }
    if constexpr (TL) {
      nxt = ldf(x + FT + lane);
      if (has_z) nzt = ldf(z + FT + lane);
    }
  };
  int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row < np.rows) issue(row);
  for (; row < np.rows; row += warps) {
    T* y = (T*)np.y + (int64_t)row * np.y_sr;
    float v[CH][V], zg[CH][V];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if ((c * 32 + lane) * V < H) {
        Vec16<T>::unpack(nx[c], v[c]);
        if (has_z) Vec16<T>::unpack(nz[c], zg[c]);
      }
    }
    float vt = nxt, zgt = nzt;                             // the lane's tail feature (TL)
    if (row + warps < np.rows) issue(row + warps);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if ((c * 32 + lane) * V < H) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if (has_z) zg[c][i] = siluf_(zg[c][i]);
          if (pre_gate) v[c][i] *= zg[c][i];
          s1 += v[c][i];
          s2 = fmaf(v[c][i], v[c][i], s2);
        }
      }
    }
    if constexpr (TL) {
      if (has_z) zgt = siluf_(zgt);
      if (pre_gate) vt *= zgt;
      s1 += vt;
      s2 = fmaf(vt, vt, s2);
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    float mean = 0.f, var;
    if (np.is_rms) {
      var = s2 / H;
    } else {
      mean = s1 / H;
      float sv = 0.f;
#pragma unroll
      for (int c = 0; c < CH; ++c)
        if ((c * 32 + lane) * V < H) {
#pragma unroll
          for (int i = 0; i < V; ++i) sv = fmaf(v[c][i] - mean, v[c][i] - mean, sv);
        }
      if constexpr (TL) sv = fmaf(vt - mean, vt - mean, sv);
      var = warp_sum(sv) / H;
    }
    const float rstd = rsqrtf(var + np.eps);
    if (lane == 0) {
      np.rstd[row] = rstd;
      if (!np.is_rms && np.mean) np.mean[row] = mean;
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int f0 = (c * 32 + lane) * V;
      if (f0 < H) {
        float w[V], o[V];
        Vec16<float>::load(np.weight + f0, w);
        if (V == 8) Vec16<float>::load(np.weight + f0 + 4, w + 4);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          o[i] = (v[c][i] - mean) * rstd * w[i];
          if (np.has_bias) o[i] += np.bias[f0 + i];
          if (post_gate) o[i] *= zg[c][i];
        }
        Vec16<T>::store(y + f0, o);
      }
    }
    if constexpr (TL) {
      float o = (vt - mean) * rstd * np.weight[FT + lane];
      if (np.has_bias) o += np.bias[FT + lane];
      if (post_gate) o *= zgt;
      stf(y + FT + lane, o);
    }
  }
}

constexpr int NORM_BWD_WARPS = 4;

// grid = nblk blocks of NORM_BWD_WARPS warps; block i handles rows [i*rpb, (i+1)*rpb); partial dw/db -> (nblk, hidden)
// HB = 0: the call has no bias, so no bias-gradient accumulators are kept (a register per owned feature less).
template <typename T, int CH, int TL, int HB>
__global__ void __launch_bounds__(NORM_BWD_WARPS * 32, (CH == 1 && !HB) ? 5 : 0) k_norm_bwd_vec(issm_norm_params np, int rpb, float* __restrict__ dwpart,
                                                                        float* __restrict__ dbpart) {
  constexpr int V = Vec16<T>::N, FT = CH * 32 * V;       // TL: one more feature per lane behind the CH full chunks
  extern __shared__ float sm[];                          // [2][NORM_BWD_WARPS][hidden]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = np.hidden;
  const bool pre_gate = np.has_z && !np.norm_before_gate, post_gate = np.has_z && np.norm_before_gate;
  float dwacc[CH][V], dbacc[CH][V], w[CH][V];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int f0 = (c * 32 + lane) * V;
#pragma unroll
    for (int i = 0; i < V; ++i) { dwacc[c][i] = 0.f; dbacc[c][i] = 0.f; w[c][i] = f0 < H ? np.weight[f0 + i] : 0.f; }
  }
  float dwt = 0.f, dbt = 0.f;
  const float wt = TL ? np.weight[FT + lane] : 0.f;
  const int r_end = min(np.rows, (int)(blockIdx.x + 1) * rpb);
  const bool has_z = np.has_z != 0;
  const bool z16 = !(((uintptr_t)np.z | (uintptr_t)(np.z_sr * (int64_t)sizeof(T))) & 15);
  // the 16-byte loads of the warp's next row are issued (kept packed, 4 registers per chunk) before the current row is
  // worked on
  uint4 nx[CH], ng[CH], nz[CH];
  float nxt = 0.f, ngt = 0.f, nzt = 0.f;
  float nrstd = 0.f, nmean = 0.f;
  auto issue = [&](int row) {
    const T* x = (const T*)np.x + (int64_t)row * np.x_sr;
    const T* zp = has_z ? (const T*)np.z + (int64_t)row * np.z_sr : nullptr;
    const T* dy = (const T*)np.dy + (int64_t)row * np.dy_sr;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int f0 = (c * 32 + lane) * V;
      if (f0 < H) {
        nx[c] = *(const uint4*)(x + f0);
        ng[c] = *(const uint4*)(dy + f0);
        if (has_z) nz[c] = ld16(zp + f0, z16);
      }
    }
    if constexpr (TL) {
      nxt = ldf(x + FT + lane);
      ngt = ldf(dy + FT + lane);
      if (has_z) nzt = ldf(zp + FT + lane);
    }
    nrstd = np.rstd[row];
    nmean = np.is_rms ? 0.f : np.mean[row];
  };
  if ((int)(blockIdx.x * rpb + warp) < r_end) issue(blockIdx.x * rpb + warp);
  for (int row = blockIdx.x * rpb + warp; row < r_end; row += NORM_BWD_WARPS) {
    const bool z = has_z;
    T* dx = (T*)np.dx + (int64_t)row * H;
    T* dz = has_z ? (T*)np.dz + (int64_t)row * H : nullptr;
    const float rstd = nrstd;
    const float mean = nmean;
    float xr[CH][V], zv[CH][V], go[CH][V];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if ((c * 32 + lane) * V < H) {
        Vec16<T>::unpack(nx[c], xr[c]);
        Vec16<T>::unpack(ng[c], go[c]);
        if (has_z) Vec16<T>::unpack(nz[c], zv[c]);
      }
    }
    const float xrt = nxt, got = ngt, zvt = nzt;           // the lane's tail feature (TL)
    if (row + NORM_BWD_WARPS < r_end) issue(row + NORM_BWD_WARPS);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int f0 = (c * 32 + lane) * V;
      if (f0 < H) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float vv = pre_gate ? xr[c][i] * siluf_(zv[c][i]) : xr[c][i];
          const float xh = (vv - mean) * rstd;
          const float g_out = post_gate ? go[c][i] * siluf_(zv[c][i]) : go[c][i];
          const float wdy = g_out * w[c][i];
          c1 = fmaf(xh, wdy, c1);
          c2 += wdy;
        }
      }
    }
    if constexpr (TL) {
      const float vv = pre_gate ? xrt * siluf_(zvt) : xrt;
      const float g_out = post_gate ? got * siluf_(zvt) : got;
      c1 = fmaf((vv - mean) * rstd, g_out * wt, c1);
      c2 += g_out * wt;
    }
    c1 = warp_sum(c1) / H;
    c2 = np.is_rms ? 0.f : warp_sum(c2) / H;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int f0 = (c * 32 + lane) * V;
      if (f0 < H) {
        float odx[V], odz[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float zz = z ? zv[c][i] : 0.f;
          const float sgm = z ? fast_sigmoid(zz) : 1.f;
          const float sz = z ? zz * sgm : 1.f;
          const float dsz = sgm * (1.f + zz * (1.f - sgm));   // d silu / dz
          const float vv = pre_gate ? xr[c][i] * sz : xr[c][i];
          const float xh = (vv - mean) * rstd;
          const float g_out = post_gate ? go[c][i] * sz : go[c][i];
          const float wdy = g_out * w[c][i];
          const float dv = (wdy - xh * c1 - c2) * rstd;
          dwacc[c][i] = fmaf(g_out, xh, dwacc[c][i]);
          if constexpr (HB) dbacc[c][i] += g_out;
          if (pre_gate) {
            odx[i] = dv * sz;
            odz[i] = dv * xr[c][i] * dsz;
          } else {
            odx[i] = dv;
            float yv = xh * w[c][i];
            if (np.has_bias) yv += np.bias[f0 + i];
            odz[i] = post_gate ? go[c][i] * yv * dsz : 0.f;
          }
        }
        Vec16<T>::store(dx + f0, odx);
        if (z) Vec16<T>::store(dz + f0, odz);
      }
    }
    if constexpr (TL) {
      const float zz = z ? zvt : 0.f;
      const float sgm = z ? fast_sigmoid(zz) : 1.f;
      const float sz = z ? zz * sgm : 1.f;
      const float dsz = sgm * (1.f + zz * (1.f - sgm));
      const float vv = pre_gate ? xrt * sz : xrt;
      const float xh = (vv - mean) * rstd;
      const float g_out = post_gate ? got * sz : got;
      const float dv = (g_out * wt - xh * c1 - c2) * rstd;
      dwt = fmaf(g_out, xh, dwt);
      if constexpr (HB) dbt += g_out;
      if (pre_gate) {
        stf(dx + FT + lane, dv * sz);
        stf(dz + FT + lane, dv * xrt * dsz);
      } else {
        stf(dx + FT + lane, dv);
        if (z) {
          float yv = xh * wt;
          if (np.has_bias) yv += np.bias[FT + lane];
          stf(dz + FT + lane, post_gate ? got * yv * dsz : 0.f);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int f0 = (c * 32 + lane) * V;
    if (f0 < H) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        sm[(size_t)warp * H + f0 + i] = dwacc[c][i];
        sm[(size_t)NORM_BWD_WARPS * H + (size_t)warp * H + f0 + i] = HB ? dbacc[c][i] : 0.f;
      }
    }
  }
  if constexpr (TL) {
    sm[(size_t)warp * H + FT + lane] = dwt;
    sm[(size_t)NORM_BWD_WARPS * H + (size_t)warp * H + FT + lane] = HB ? dbt : 0.f;
  }
  __syncthreads();
  for (int f = threadIdx.x; f < H; f += blockDim.x) {
    float a = 0.f, b = 0.f;
    for (int wq = 0; wq < NORM_BWD_WARPS; ++wq) {
      a += sm[(size_t)wq * H + f];
      b += sm[(size_t)NORM_BWD_WARPS * H + (size_t)wq * H + f];
    }
    dwpart[(size_t)blockIdx.x * H + f] = a;
    dbpart[(size_t)blockIdx.x * H + f] = b;
  }
}

// chunks per lane the vector kernels need for this call, or 0 when it has to take the general kernels
static int norm_vec_chunks(const issm_norm_params& p, bool bwd) {
  const int V = p.io_dtype == ISSM_BF16 ? 8 : 4, esz = p.io_dtype == ISSM_BF16 ? 2 : 4;
  if (p.group_size != p.hidden || p.hidden % V) return 0;
  auto ok = [&](const void* ptr, int64_t stride) { return ((uintptr_t)ptr % 16 == 0) && ((stride * esz) % 16 == 0); };
  auto ok4 = [&](const void* ptr, int64_t stride) { return ((uintptr_t)ptr % 4 == 0) && ((stride * esz) % 4 == 0); };
  // the gate may start its rows on any 4-byte boundary (read as four 4-byte words then)
  if (!ok(p.x, p.x_sr) || (p.has_z && !ok4(p.z, p.z_sr)) || ((uintptr_t)p.weight % 16)) return 0;
  if (!bwd && !ok(p.y, p.y_sr)) return 0;
  if (bwd && (!ok(p.dy, p.dy_sr) || !ok(p.dx, p.hidden) || (p.has_z && !ok(p.dz, p.hidden)))) return 0;
  // full chunks plus exactly 32 more features: those go one per lane (returned as chunks + 16)
  if (p.hidden % (32 * V) == 32 && p.hidden / (32 * V) >= 1 && p.hidden / (32 * V) <= 2) return p.hidden / (32 * V) + 16;
  const int need = (p.hidden + 32 * V - 1) / (32 * V);
  return need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 0;
}



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

// out[j] = sum over the `count` partial rows of part[i][j], in a fixed order: 32 features x 8 row groups per block;
// group g adds rows g, g + 8, ... in order, then the eight group sums are added in order
__global__ void __launch_bounds__(256) k_norm_reduce(const float* __restrict__ part, int count, int stride, float* __restrict__ out) {
  __shared__ float sacc[8][33];
  const int fx = threadIdx.x & 31, gy = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + fx;
  float acc = 0.f;
  if (j < stride)
    for (int i = gy; i < count; i += 8) acc += part[(size_t)i * stride + j];
  sacc[gy][fx] = acc;
  __syncthreads();
  if (gy == 0 && j < stride) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) t += sacc[g][fx];
    out[j] = t;
  }
}

// blocks of the backward: one resident wave (five blocks of four warps per SM fit the bias-free vector kernel; the
// workspace-free entry point keeps to its built-in scratch of 148 * 4 partial rows)
static int norm_blocks(const issm_norm_params& p, int want = 148 * 5) {
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

// the backward main kernel of one call (vector kernels when the call qualifies, see norm_vec_chunks)
static int launch_norm_bwd_main(const issm_norm_params& p, int nblk, int rpb, float* dwpart, float* dbpart, size_t smem, cudaStream_t s) {
  const int ch = norm_vec_chunks(p, true);
#define ISSM_NORM_BWD_VEC2(T, HBV)                                                                                            \
  do {                                                                                                                      \
    if (ch == 17) ISSM_LAUNCH((k_norm_bwd_vec<T, 1, 1, HBV>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart);      \
    else if (ch == 18) ISSM_LAUNCH((k_norm_bwd_vec<T, 2, 1, HBV>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart); \
    else if (ch == 1) ISSM_LAUNCH((k_norm_bwd_vec<T, 1, 0, HBV>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart);  \
    else if (ch == 2) ISSM_LAUNCH((k_norm_bwd_vec<T, 2, 0, HBV>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart);  \
    else ISSM_LAUNCH((k_norm_bwd_vec<T, 4, 0, HBV>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart);               \
  } while (0)
#define ISSM_NORM_BWD_VEC(T)                                                                                          \
  do {                                                                                                                \
    /* the bias-free variant exists for one-chunk rows; wider rows keep the general one */                           \
    if (p.has_bias || (ch != 1 && ch != 17)) ISSM_NORM_BWD_VEC2(T, 1); else ISSM_NORM_BWD_VEC2(T, 0);                 \
  } while (0)
  if (ch) {                                               // rows of at most 1024 (bf16) / 512 (float) features: 32 KiB of shared memory at most
    if (p.io_dtype == ISSM_F32) ISSM_NORM_BWD_VEC(float); else ISSM_NORM_BWD_VEC(bf16);
    return ISSM_OK;
  }
  if (p.io_dtype == ISSM_F32) ISSM_LAUNCH((k_norm_bwd<float>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart);
  else ISSM_LAUNCH((k_norm_bwd<bf16>), nblk, NORM_BWD_WARPS * 32, smem, s, p, rpb, dwpart, dbpart);
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
  const int ch = norm_vec_chunks(*p, false);
  const unsigned vgrid = grid < 148u * 4u ? grid : 148u * 4u;   // the vector kernel walks the rows with a grid stride (one resident wave)
#define ISSM_NORM_FWD_VEC(T)                                                                                   \
  do {                                                                                                         \
    if (ch == 17) ISSM_LAUNCH((k_norm_fwd_vec<T, 1, 1>), vgrid, wpb * 32, 0, s, *p);                           \
    else if (ch == 18) ISSM_LAUNCH((k_norm_fwd_vec<T, 2, 1>), vgrid, wpb * 32, 0, s, *p);                      \
    else if (ch == 1) ISSM_LAUNCH((k_norm_fwd_vec<T, 1, 0>), vgrid, wpb * 32, 0, s, *p);                       \
    else if (ch == 2) ISSM_LAUNCH((k_norm_fwd_vec<T, 2, 0>), vgrid, wpb * 32, 0, s, *p);                       \
    else ISSM_LAUNCH((k_norm_fwd_vec<T, 4, 0>), vgrid, wpb * 32, 0, s, *p);                                    \
  } while (0)
  if (ch) {
    if (p->io_dtype == ISSM_F32) ISSM_NORM_FWD_VEC(float); else ISSM_NORM_FWD_VEC(bf16);
    return ISSM_OK;
  }
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
  // five resident blocks per SM only fit the kernel variant that was built for them (one chunk, no bias)
  const int vch = norm_vec_chunks(*p, true);
  const int nblk = norm_blocks(*p, ((vch == 1 || vch == 17) && !p->has_bias) ? 148 * 5 : 148 * 4);
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
  rc = launch_norm_bwd_main(*p, nblk, rpb, dwpart, dbpart, smem, s);
  if (rc) return rc;
  ISSM_LAUNCH(k_norm_reduce, (p->hidden + 31) / 32, 256, 0, s, dwpart, nblk, p->hidden, p->dweight);
  if (p->has_bias) ISSM_LAUNCH(k_norm_reduce, (p->hidden + 31) / 32, 256, 0, s, dbpart, nblk, p->hidden, p->dbias);
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
constexpr int kNoAllocMaxBlocks = 148 * 4;              // the grid limit handed to norm_blocks() below
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
  const int nblk = norm_blocks(*p, kNoAllocMaxBlocks);
  const int rpb = (p->rows + nblk - 1) / nblk;
  float* dwpart = scratch;
  float* dbpart = scratch + (size_t)nblk * p->hidden;
  const size_t smem = (size_t)2 * NORM_BWD_WARPS * p->hidden * sizeof(float);   // <= 32 KiB here
  // every block writes its whole row of partials, so nothing in the scratch has to start at zero
  rc = launch_norm_bwd_main(*p, nblk, rpb, dwpart, dbpart, smem, s);
  if (rc) return rc;
  ISSM_LAUNCH(k_norm_reduce, (p->hidden + 31) / 32, 256, 0, s, dwpart, nblk, p->hidden, p->dweight);
  if (p->has_bias) ISSM_LAUNCH(k_norm_reduce, (p->hidden + 31) / 32, 256, 0, s, dbpart, nblk, p->hidden, p->dbias);
  return ISSM_OK;
}
