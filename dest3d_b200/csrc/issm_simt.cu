// SIMT (fp32 arithmetic) kernels of the ISSM chunked scan: the float32 product path and the
// any-value-range path.  Every decay factor is evaluated as exp(a[l] - a[s]) of a non-positive
// difference, so no input range can overflow (the factored tensor-core path has range limits).
//
// Stage map (reference files are inside the reference project):
//   k_prep            issm_triton/issm_chunk_state.py:50-104   dt transform + in-chunk cumsum of dt*A
//   k_chunk_state     issm_triton/issm_chunk_state.py:282-356  per-chunk states      (MODE 0)
//                     issm_triton/issm_chunk_scan.py:423-512   dstates from dy       (MODE 1)
//   k_pass_fwd/bwd    issm_triton/issm_state_passing.py:48-107, 174-278
//   k_scan<false>     issm_triton/issm_cabt_bmm.py:78-153 + issm_chunk_scan.py:71-214
//   k_scan<true>      issm_triton/issm_combined.py:258-395     dx
//   k_dy              issm_triton/issm_chunk_scan.py:286-377   dz, dy
//   k_dM              issm_triton/issm_chunk_scan.py:828-900   dCABT
//   k_main            issm_combined.py:451-557, issm_cabt_bmm.py:539-672, issm_chunk_scan.py:573-657,
//                     :948-1031, issm_chunk_state.py:559-652, :159-231 (ddt, dB, dC, ddA, dt chain)
//   k_reduce_*        the torch sums / atomics of issm_combined.py:159,172-175 done in fixed order
//
// Index conventions: logical position t in [0, L) runs in scan order; with `reverse` it maps to
// memory row L-1-t.  Workspace tensors are indexed by (chunk, logical row in chunk).
#include "issm_common.cuh"

namespace issm {

struct SimtLayout {
  int nc;
  size_t n_dtv, n_states, n_dy, n_ddac, n_dM, n_part_hn, n_part_hp, n_headpart, n_grun;
};

static SimtLayout simt_layout(const issm_params& p) {
  SimtLayout l;
  l.nc = (p.seqlen + p.chunk_size - 1) / p.chunk_size;
  size_t b = p.batch, H = p.nheads, P = p.headdim, N = p.dstate, Q = p.chunk_size, L = p.seqlen, nc = l.nc;
  l.n_dtv = b * H * nc * Q * N;
  l.n_states = b * nc * H * P * N;
  l.n_dy = b * L * H * P;
  l.n_ddac = b * nc * H * N;
  l.n_dM = b * nc * H * Q * Q;
  l.n_part_hn = b * nc * H * N;
  l.n_part_hp = b * nc * H * P;
  l.n_headpart = (p.nheads / p.ngroups > 1) ? b * L * H * N : 0;
  l.n_grun = b * H * P * N;
  return l;
}

struct SimtWs {
  float *dtv, *acs, *states;
  float *dy, *dstates, *grun, *ddac, *dM, *dApart, *dbpart, *dDpart, *dBh, *dCh;
};

static SimtWs simt_carve(const issm_params& p, const SimtLayout& l, int pass, size_t* total) {
  Carver c(p.workspace);
  SimtWs w{};
  w.dtv = c.take<float>(l.n_dtv);
  w.acs = c.take<float>(l.n_dtv);
  w.states = c.take<float>(l.n_states);
  if (pass == 1) {
    w.dy = c.take<float>(l.n_dy);
    w.dstates = c.take<float>(l.n_states);
    w.grun = c.take<float>(l.n_grun);
    w.ddac = c.take<float>(l.n_ddac);
    w.dM = c.take<float>(l.n_dM);
    w.dApart = c.take<float>(l.n_part_hn);
    w.dbpart = c.take<float>(l.n_part_hn);
    w.dDpart = c.take<float>(l.n_part_hp);
    w.dBh = c.take<float>(l.n_headpart);
    w.dCh = c.take<float>(l.n_headpart);
  }
  *total = c.off;
  return w;
}

size_t simt_workspace_bytes(const issm_params& p, int pass) {
  issm_params q = p;
  q.workspace = nullptr;
  size_t total = 0;
  simt_carve(q, simt_layout(q), pass, &total);
  return total;
}

// ---------------------------------------------------------------------------------------------
// common device-side view of one call
// ---------------------------------------------------------------------------------------------
struct Dims {
  int b, L, H, P, N, G, Q, nc, hpg, rev;
};

__device__ __forceinline__ int mem_row(const Dims& d, int t) { return d.rev ? d.L - 1 - t : t; }

// ---------------------------------------------------------------------------------------------
// k_prep: dtv = clamp(softplus?(dt + bias)), acs = in-chunk inclusive cumsum of dtv * A
// grid (nc, H, b); threads stride over n.  Padded tail rows get dtv = 0 (cumsum stays flat).
// ---------------------------------------------------------------------------------------------
template <typename TDT>
__global__ void k_prep(Dims d, const TDT* __restrict__ dt, int64_t sb, int64_t sl, int64_t sh,
                       const float* __restrict__ A, const float* __restrict__ bias, int softplus,
                       float dtmin, float dtmax, float* __restrict__ dtv, float* __restrict__ acs) {
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  for (int n = threadIdx.x; n < d.N; n += blockDim.x) {
    const float a = A[h * d.N + n];
    const float bs = bias ? bias[h * d.N + n] : 0.f;
    float acc = 0.f;
    size_t idx = ((((size_t)b * d.H + h) * d.nc + c) * d.Q) * d.N + n;
    for (int r = 0; r < d.Q; ++r, idx += d.N) {
      const int t = c * d.Q + r;
      float v = 0.f;
      if (t < d.L) {
        v = ldf(dt + b * sb + (int64_t)mem_row(d, t) * sl + h * sh + n) + bs;
        if (softplus) v = softplus_thr(v);
        v = fminf(fmaxf(v, dtmin), dtmax);
      }
      acc += v * a;
      dtv[idx] = v;
      acs[idx] = acc;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// k_chunk_state: out[p, n] = sum_t src[t, p] * f[t, n]
//   MODE 0: src = x,  f = B * dtv * exp(a_last - a)        (chunk states)
//   MODE 1: src = dy, f = C * exp(a)                       (local state gradients)
// grid (nc, H, b); thread <-> n; 32 p-accumulators per pass.
// ---------------------------------------------------------------------------------------------
template <int MODE, typename TS, typename TBC>
__global__ void k_chunk_state(Dims d, const TS* __restrict__ src, int64_t s_sb, int64_t s_sl, int64_t s_sh,
                              const TBC* __restrict__ bc, int64_t bc_sb, int64_t bc_sl, int64_t bc_sg,
                              const float* __restrict__ dtv, const float* __restrict__ acs,
                              float* __restrict__ out) {
  __shared__ float xs[32][33];
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, g = h / d.hpg;
  const size_t base = ((((size_t)b * d.H + h) * d.nc + c) * d.Q) * d.N;
  const int rows = min(d.Q, d.L - c * d.Q);
  for (int n0 = 0; n0 < d.N; n0 += blockDim.x) {
    const int n = n0 + threadIdx.x;
    const bool act = n < d.N;
    const float alast = act ? acs[base + (size_t)(d.Q - 1) * d.N + n] : 0.f;
    for (int p0 = 0; p0 < d.P; p0 += 32) {
      float acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.f;
      for (int r0 = 0; r0 < rows; r0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * 32; i += blockDim.x) {
          const int r = i / 32, pp = i % 32;
          float v = 0.f;
          if (r0 + r < rows && p0 + pp < d.P)
            v = ldf(src + b * s_sb + (int64_t)mem_row(d, c * d.Q + r0 + r) * s_sl + h * s_sh + p0 + pp);
          xs[r][pp] = v;
        }
        __syncthreads();
        if (act) {
          const int rmax = min(32, rows - r0);
          for (int r = 0; r < rmax; ++r) {
            const size_t idx = base + (size_t)(r0 + r) * d.N + n;
            const float bcv = ldf(bc + b * bc_sb + (int64_t)mem_row(d, c * d.Q + r0 + r) * bc_sl + g * bc_sg + n);
            float f;
            if (MODE == 0) f = bcv * dtv[idx] * expf(alast - acs[idx]);
            else f = bcv * expf(acs[idx]);
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = fmaf(xs[r][i], f, acc[i]);
          }
        }
      }
      if (act) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (p0 + i < d.P) out[((((size_t)b * d.nc + c) * d.H + h) * d.P + p0 + i) * d.N + n] = acc[i];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// k_pass_fwd: states[c] <- state entering chunk c (in place); final <- state after the last chunk
// one thread per (b, h, p, n)
// ---------------------------------------------------------------------------------------------
template <typename TI>
__global__ void k_pass_fwd(Dims d, float* __restrict__ states, const float* __restrict__ acs,
                           const TI* __restrict__ init, float* __restrict__ final_states) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)d.b * d.H * d.P * d.N;
  if (i >= total) return;
  const int n = i % d.N;
  const int p = (i / d.N) % d.P;
  const int h = (i / ((size_t)d.N * d.P)) % d.H;
  const int b = i / ((size_t)d.N * d.P * d.H);
  float run = init ? ldf(init + i) : 0.f;
  for (int c = 0; c < d.nc; ++c) {
    const size_t si = ((((size_t)b * d.nc + c) * d.H + h) * d.P + p) * d.N + n;
    const float local = states[si];
    states[si] = run;
    const float alast = acs[((((size_t)b * d.H + h) * d.nc + c) * d.Q + d.Q - 1) * d.N + n];
    run = run * expf(alast) + local;
  }
  if (final_states) final_states[i] = run;
}

// k_pass_bwd: reverse recurrence over chunks, one thread per (b, h, n), looping p.
//   dstates[c] <- g_{c+1} (gradient w.r.t. the state leaving chunk c), in place
//   ddac[c, n]  = sum_p S_c[p, n] * g_{c+1}[p, n] * exp(a_last_c[n])
//   grun        = g_0 at the end (gradient w.r.t. the initial states)
__global__ void k_pass_bwd(Dims d, float* __restrict__ dstates, const float* __restrict__ states,
                           const float* __restrict__ acs, const float* __restrict__ dfinal,
                           float* __restrict__ grun, float* __restrict__ ddac) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)d.b * d.H * d.N;
  if (i >= total) return;
  const int n = i % d.N;
  const int h = (i / d.N) % d.H;
  const int b = i / ((size_t)d.N * d.H);
  const size_t gbase = (((size_t)b * d.H + h) * d.P) * d.N + n;
  for (int p = 0; p < d.P; ++p) grun[gbase + (size_t)p * d.N] = dfinal ? dfinal[gbase + (size_t)p * d.N] : 0.f;
  for (int c = d.nc - 1; c >= 0; --c) {
    const float decay = expf(acs[((((size_t)b * d.H + h) * d.nc + c) * d.Q + d.Q - 1) * d.N + n]);
    float acc = 0.f;
    const size_t sbase = ((((size_t)b * d.nc + c) * d.H + h) * d.P) * d.N + n;
    for (int p = 0; p < d.P; ++p) {
      const float g = grun[gbase + (size_t)p * d.N];
      const float local = dstates[sbase + (size_t)p * d.N];
      dstates[sbase + (size_t)p * d.N] = g;
      acc = fmaf(states[sbase + (size_t)p * d.N], g, acc);
      grun[gbase + (size_t)p * d.N] = fmaf(decay, g, local);
    }
    ddac[(((size_t)b * d.nc + c) * d.H + h) * d.N + n] = acc * decay;
  }
}

template <typename TI>
__global__ void k_cast_out(const float* __restrict__ src, TI* __restrict__ dst, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) stf(dst + i, src[i]);
}

// ---------------------------------------------------------------------------------------------
// k_scan: intra-chunk matrix rows on the fly + output rows.
//   m(t, s) = sum_n C[t,n] * B[s,n] * dtv[s,n] * exp(a[t,n] - a[s,n])          (s <= t)
//   BWD == false: y[t,p]  = sum_{s<=t} m(t,s) x[s,p] + sum_n C[t,n] e^{a[t,n]} S[p,n] + D x[t,p]
//                 out = y * z * sigmoid(z) when gated (out_x keeps y)
//   BWD == true : dx[s,p] = sum_{t>=s} m(t,s) dy[t,p] + sum_n B dtv e^{a_last - a[s,n]} g[p,n] + D dy[s,p]
// grid (nc * tiles, H, b), tiles = ceil(Q / TR); 8 warps; dynamic smem TR * (Q + 1) floats.
// ---------------------------------------------------------------------------------------------
constexpr int TR = 16;

template <bool BWD, typename TIO>
__global__ void k_scan(Dims d,
                       const TIO* __restrict__ x, int64_t x_sb, int64_t x_sl, int64_t x_sh,
                       const TIO* __restrict__ Bm, int64_t B_sb, int64_t B_sl, int64_t B_sg,
                       const TIO* __restrict__ Cm, int64_t C_sb, int64_t C_sl, int64_t C_sg,
                       const TIO* __restrict__ z, int64_t z_sb, int64_t z_sl, int64_t z_sh,
                       const float* __restrict__ Dv, int D_has_hdim,
                       const float* __restrict__ dtv, const float* __restrict__ acs,
                       const float* __restrict__ st,   // S entering (fwd) or g leaving (bwd): (b,nc,H,P,N)
                       const float* __restrict__ dy,   // bwd only: (b, L, H, P) fp32, memory rows
                       TIO* __restrict__ out, int64_t o_sb, int64_t o_sl, int64_t o_sh,
                       TIO* __restrict__ out_x) {
  extern __shared__ float sm[];
  const int tiles = (d.Q + TR - 1) / TR;
  const int c = blockIdx.x / tiles, tile = blockIdx.x % tiles;
  const int h = blockIdx.y, b = blockIdx.z, g = h / d.hpg;
  const int rows = min(d.Q, d.L - c * d.Q);
  const int r0 = tile * TR;
  if (r0 >= rows) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const size_t base = ((((size_t)b * d.H + h) * d.nc + c) * d.Q) * d.N;
  const int ldm = d.Q + 1;
  const int rt = min(TR, rows - r0);

  // phase 1: pair sums, one warp per (row, partner) pair, lanes over n
  for (int r = warp; r < rt; r += nwarp) {
    const int row = r0 + r;
    const int lo = BWD ? row : 0, hi = BWD ? rows - 1 : row;
    for (int q = lo; q <= hi; ++q) {
      const int t = BWD ? q : row, s = BWD ? row : q;
      const TIO* cp = Cm + b * C_sb + (int64_t)mem_row(d, c * d.Q + t) * C_sl + g * C_sg;
      const TIO* bp = Bm + b * B_sb + (int64_t)mem_row(d, c * d.Q + s) * B_sl + g * B_sg;
      const float* at = acs + base + (size_t)t * d.N;
      const float* as = acs + base + (size_t)s * d.N;
      const float* ds = dtv + base + (size_t)s * d.N;
      float acc = 0.f;
      for (int n = lane; n < d.N; n += 32)
        acc = fmaf(ldf(cp + n) * ldf(bp + n) * ds[n], expf(at[n] - as[n]), acc);
      acc = warp_sum(acc);
      if (lane == 0) sm[r * ldm + q] = acc;
    }
  }
  __syncthreads();

  // phase 2: one warp per output (row, p)
  const float* alastp = acs + base + (size_t)(d.Q - 1) * d.N;
  for (int o = warp; o < rt * d.P; o += nwarp) {
    const int r = o / d.P, p = o % d.P;
    const int row = r0 + r;
    const int lrow = mem_row(d, c * d.Q + row);
    float acc = 0.f;
    const int lo = BWD ? row : 0, hi = BWD ? rows - 1 : row;
    for (int q = lo + lane; q <= hi; q += 32) {
      const int lq = mem_row(d, c * d.Q + q);
      const float v = BWD ? dy[(((size_t)b * d.L + lq) * d.H + h) * d.P + p]
                          : ldf(x + b * x_sb + (int64_t)lq * x_sl + h * x_sh + p);
      acc = fmaf(sm[r * ldm + q], v, acc);
    }
    const float* sp = st + ((((size_t)b * d.nc + c) * d.H + h) * d.P + p) * d.N;
    const float* ar = acs + base + (size_t)row * d.N;
    if (!BWD) {
      const TIO* cp = Cm + b * C_sb + (int64_t)lrow * C_sl + g * C_sg;
      for (int n = lane; n < d.N; n += 32) acc = fmaf(ldf(cp + n) * expf(ar[n]), sp[n], acc);
    } else {
      const TIO* bp = Bm + b * B_sb + (int64_t)lrow * B_sl + g * B_sg;
      const float* dr = dtv + base + (size_t)row * d.N;
      for (int n = lane; n < d.N; n += 32)
        acc = fmaf(ldf(bp + n) * dr[n] * expf(alastp[n] - ar[n]), sp[n], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      const float dcoef = Dv ? (D_has_hdim ? Dv[h * d.P + p] : Dv[h]) : 0.f;
      if (!BWD) {
        float y = acc + dcoef * ldf(x + b * x_sb + (int64_t)lrow * x_sl + h * x_sh + p);
        const int64_t oi = b * o_sb + (int64_t)lrow * o_sl + h * o_sh + p;
        if (z) {
          stf(out_x + oi, y);
          const float zv = ldf(z + b * z_sb + (int64_t)lrow * z_sl + h * z_sh + p);
          y *= zv * sigmoidf_(zv);
        }
        stf(out + oi, y);
      } else {
        const float v = acc + dcoef * dy[(((size_t)b * d.L + lrow) * d.H + h) * d.P + p];
        stf(out + (((size_t)b * d.L + lrow) * d.H + h) * d.P + p, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// k_dy: dy = dout * z * sigmoid(z), dz = dout * y * sigmoid(z) (1 + z (1 - sigmoid(z)))
// (issm_chunk_scan.py:351-360); without z: dy = dout.  dy is fp32 (b, L, H, P) in memory order.
// ---------------------------------------------------------------------------------------------
template <typename TIO>
__global__ void k_dy(Dims d, const TIO* __restrict__ dout, int64_t g_sb, int64_t g_sl, int64_t g_sh,
                     const TIO* __restrict__ z, int64_t z_sb, int64_t z_sl, int64_t z_sh,
                     const TIO* __restrict__ y, int64_t y_sb, int64_t y_sl, int64_t y_sh,
                     float* __restrict__ dy, TIO* __restrict__ dz) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)d.b * d.L * d.H * d.P;
  if (i >= total) return;
  const int p = i % d.P;
  const int h = (i / d.P) % d.H;
  const int l = (i / ((size_t)d.P * d.H)) % d.L;
  const int b = i / ((size_t)d.P * d.H * d.L);
  const float go = ldf(dout + b * g_sb + (int64_t)l * g_sl + h * g_sh + p);
  if (z) {
    const float zv = ldf(z + b * z_sb + (int64_t)l * z_sl + h * z_sh + p);
    const float yv = ldf(y + b * y_sb + (int64_t)l * y_sl + h * y_sh + p);
    const float sg = sigmoidf_(zv);
    dy[i] = go * zv * sg;
    stf(dz + i, go * yv * sg * (1.f + zv * (1.f - sg)));
  } else {
    dy[i] = go;
  }
}

// k_dD: per (b, chunk) partial of dD[h, p] = sum_t dy[t,p] * x[t,p]; grid (nc, H, b), threads over p
template <typename TIO>
__global__ void k_dD(Dims d, const float* __restrict__ dy, const TIO* __restrict__ x, int64_t x_sb,
                     int64_t x_sl, int64_t x_sh, float* __restrict__ part) {
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int rows = min(d.Q, d.L - c * d.Q);
  for (int p = threadIdx.x; p < d.P; p += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < rows; ++r) {
      const int l = mem_row(d, c * d.Q + r);
      acc = fmaf(dy[(((size_t)b * d.L + l) * d.H + h) * d.P + p], ldf(x + b * x_sb + (int64_t)l * x_sl + h * x_sh + p), acc);
    }
    part[(((size_t)b * d.nc + c) * d.H + h) * d.P + p] = acc;
  }
}

// k_dM: dM[t, s] = sum_p dy[t,p] x[s,p] for s <= t (0 elsewhere); grid (nc, H, b)
template <typename TIO>
__global__ void k_dM(Dims d, const float* __restrict__ dy, const TIO* __restrict__ x, int64_t x_sb,
                     int64_t x_sl, int64_t x_sh, float* __restrict__ dM) {
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int rows = min(d.Q, d.L - c * d.Q);
  float* o = dM + ((((size_t)b * d.nc + c) * d.H + h) * d.Q) * d.Q;
  for (int i = threadIdx.x; i < d.Q * d.Q; i += blockDim.x) {
    const int t = i / d.Q, s = i % d.Q;
    float acc = 0.f;
    if (s <= t && t < rows) {
      const float* dyr = dy + (((size_t)b * d.L + mem_row(d, c * d.Q + t)) * d.H + h) * d.P;
      const TIO* xr = x + b * x_sb + (int64_t)mem_row(d, c * d.Q + s) * x_sl + h * x_sh;
      for (int p = 0; p < d.P; ++p) acc = fmaf(dyr[p], ldf(xr + p), acc);
    }
    o[i] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// k_main: everything of the backward that lives on the (row, state) grid of one (b, chunk, head):
//   G2[j,n] = sum_{s<=j} dM[j,s] B dtv[s,n] e^{a[j,n]-a[s,n]}     V[j,n] = e^{a[j,n]} sum_p dy[j,p] S[p,n]
//   G1[j,n] = sum_{t>=j} dM[t,j] C[t,n]   e^{a[t,n]-a[j,n]}       W[j,n] = e^{a_last-a[j,n]} sum_p x[j,p] g[p,n]
//   dB_h = dtv (G1 + W), dC_h = G2 + V, ddt_direct = B (G1 + W)
//   dacs = C (G2 + V) - B dtv (G1 + W);  ddA[j] = sum_{t>=j} dacs[t] + ddac_chunk + sum_s B dtv W
//   ddt = ddt_direct + ddA * A, chained through clamp and softplus; per-(b,chunk) partials of dA, ddt_bias
// grid (nc * ceil(N/32), H, b); 8 warps; lane <-> state n; dynamic smem 6 * Q * 32 floats.
// ---------------------------------------------------------------------------------------------
template <typename TIO, typename TDT>
__global__ void k_main(Dims d,
                       const TIO* __restrict__ x, int64_t x_sb, int64_t x_sl, int64_t x_sh,
                       const TIO* __restrict__ Bm, int64_t B_sb, int64_t B_sl, int64_t B_sg,
                       const TIO* __restrict__ Cm, int64_t C_sb, int64_t C_sl, int64_t C_sg,
                       const TDT* __restrict__ dt, int64_t dt_sb, int64_t dt_sl, int64_t dt_sh,
                       const float* __restrict__ A, const float* __restrict__ bias, int softplus,
                       float dtmin, float dtmax,
                       const float* __restrict__ dtv, const float* __restrict__ acs,
                       const float* __restrict__ S, const float* __restrict__ gout,
                       const float* __restrict__ dy, const float* __restrict__ dM,
                       const float* __restrict__ ddac,
                       TDT* __restrict__ ddt, TIO* __restrict__ dB, TIO* __restrict__ dC,
                       float* __restrict__ dBh, float* __restrict__ dCh,
                       float* __restrict__ dApart, float* __restrict__ dbpart) {
  extern __shared__ float sm[];
  const int ntile = (d.N + 31) / 32;
  const int c = blockIdx.x / ntile, n0 = (blockIdx.x % ntile) * 32;
  const int h = blockIdx.y, b = blockIdx.z, g = h / d.hpg;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int n = n0 + lane;
  const bool act = n < d.N;
  const int rows = min(d.Q, d.L - c * d.Q);
  float* sBdt = sm;
  float* sA = sBdt + d.Q * 32;
  float* sC = sA + d.Q * 32;
  float* sDacs = sC + d.Q * 32;
  float* sDdt = sDacs + d.Q * 32;
  float* sBW = sDdt + d.Q * 32;
  const size_t base = ((((size_t)b * d.H + h) * d.nc + c) * d.Q) * d.N;

  for (int r = warp; r < rows; r += nwarp) {
    float bv = 0.f, cv = 0.f, av = 0.f, dv = 0.f;
    if (act) {
      const int l = mem_row(d, c * d.Q + r);
      bv = ldf(Bm + b * B_sb + (int64_t)l * B_sl + g * B_sg + n);
      cv = ldf(Cm + b * C_sb + (int64_t)l * C_sl + g * C_sg + n);
      av = acs[base + (size_t)r * d.N + n];
      dv = dtv[base + (size_t)r * d.N + n];
    }
    sBdt[r * 32 + lane] = bv * dv;
    sA[r * 32 + lane] = av;
    sC[r * 32 + lane] = cv;
  }
  __syncthreads();

  const float alast = act ? acs[base + (size_t)(d.Q - 1) * d.N + n] : 0.f;
  const float* dMt = dM + ((((size_t)b * d.nc + c) * d.H + h) * d.Q) * d.Q;
  const size_t sbase = ((((size_t)b * d.nc + c) * d.H + h) * d.P) * d.N;
  for (int j = warp; j < rows; j += nwarp) {
    const float aj = sA[j * 32 + lane];
    float G2 = 0.f, G1 = 0.f;
    const float* dMrow = dMt + (size_t)j * d.Q;
    for (int s = 0; s <= j; ++s) G2 = fmaf(dMrow[s] * sBdt[s * 32 + lane], expf(aj - sA[s * 32 + lane]), G2);
    for (int t = j; t < rows; ++t) G1 = fmaf(dMt[(size_t)t * d.Q + j] * sC[t * 32 + lane], expf(sA[t * 32 + lane] - aj), G1);
    float W = 0.f, V = 0.f;
    const int l = mem_row(d, c * d.Q + j);
    if (act) {
      const TIO* xr = x + b * x_sb + (int64_t)l * x_sl + h * x_sh;
      const float* dyr = dy + (((size_t)b * d.L + l) * d.H + h) * d.P;
      for (int p = 0; p < d.P; ++p) {
        W = fmaf(ldf(xr + p), gout[sbase + (size_t)p * d.N + n], W);
        V = fmaf(dyr[p], S[sbase + (size_t)p * d.N + n], V);
      }
    }
    W *= expf(alast - aj);
    V *= expf(aj);
    const float bd = G1 + W, cd = G2 + V;
    const float bdt = sBdt[j * 32 + lane];
    float bv = 0.f, dv = 0.f;
    if (act) {
      bv = ldf(Bm + b * B_sb + (int64_t)l * B_sl + g * B_sg + n);
      dv = dtv[base + (size_t)j * d.N + n];
    }
    sDacs[j * 32 + lane] = sC[j * 32 + lane] * cd - bdt * bd;
    sDdt[j * 32 + lane] = bv * bd;
    sBW[j * 32 + lane] = bdt * W;
    if (act) {
      if (d.hpg == 1) {
        stf(dB + (((size_t)b * d.L + l) * d.G + g) * d.N + n, dv * bd);
        stf(dC + (((size_t)b * d.L + l) * d.G + g) * d.N + n, cd);
      } else {
        dBh[(((size_t)b * d.L + l) * d.H + h) * d.N + n] = dv * bd;
        dCh[(((size_t)b * d.L + l) * d.H + h) * d.N + n] = cd;
      }
    }
  }
  __syncthreads();

  if (warp == 0 && act) {
    float run = ddac[(((size_t)b * d.nc + c) * d.H + h) * d.N + n];
    for (int j = 0; j < rows; ++j) run += sBW[j * 32 + lane];
    const float an = A[h * d.N + n];
    const float bs = bias ? bias[h * d.N + n] : 0.f;
    float dAacc = 0.f, dbacc = 0.f;
    for (int j = rows - 1; j >= 0; --j) {
      run += sDacs[j * 32 + lane];
      const float dv = dtv[base + (size_t)j * d.N + n];
      dAacc = fmaf(run, dv, dAacc);
      float gd = fmaf(run, an, sDdt[j * 32 + lane]);
      const int l = mem_row(d, c * d.Q + j);
      const int64_t di = b * dt_sb + (int64_t)l * dt_sl + h * dt_sh + n;
      const float pre = ldf(dt + di) + bs;
      const float tv = softplus ? softplus_thr(pre) : pre;
      if (tv < dtmin || tv > dtmax) gd = 0.f;
      else if (softplus && pre <= 20.f) gd *= sigmoidf_(pre);
      stf(ddt + (((size_t)b * d.L + l) * d.H + h) * d.N + n, gd);
      dbacc += gd;
    }
    dApart[(((size_t)b * d.nc + c) * d.H + h) * d.N + n] = dAacc;
    dbpart[(((size_t)b * d.nc + c) * d.H + h) * d.N + n] = dbacc;
  }
}

// fixed-order reductions -------------------------------------------------------------------------
// out[j] = sum_{i < count} part[i * stride + j]
__global__ void k_reduce_rows(const float* __restrict__ part, int count, int stride, float* __restrict__ out) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= stride) return;
  float acc = 0.f;
  for (int i = 0; i < count; ++i) acc += part[(size_t)i * stride + j];
  out[j] = acc;
}

// dD (H) from partials (count, H, P): sum over count and p
__global__ void k_reduce_dD_head(const float* __restrict__ part, int count, int H, int P, float* __restrict__ out) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float acc = 0.f;
  for (int i = 0; i < count; ++i)
    for (int p = 0; p < P; ++p) acc += part[((size_t)i * H + h) * P + p];
  out[h] = acc;
}

// dB[b,l,g,n] = sum_{h in group g} part[b,l,h,n]
template <typename TIO>
__global__ void k_reduce_heads(Dims d, const float* __restrict__ part, TIO* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)d.b * d.L * d.G * d.N;
  if (i >= total) return;
  const int n = i % d.N;
  const int g = (i / d.N) % d.G;
  const size_t bl = i / ((size_t)d.N * d.G);
  float acc = 0.f;
  for (int k = 0; k < d.hpg; ++k) acc += part[(bl * d.H + g * d.hpg + k) * d.N + n];
  stf(out + i, acc);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static Dims make_dims(const issm_params& p, int nc) {
  Dims d;
  d.b = p.batch; d.L = p.seqlen; d.H = p.nheads; d.P = p.headdim; d.N = p.dstate; d.G = p.ngroups;
  d.Q = p.chunk_size; d.nc = nc; d.hpg = p.nheads / p.ngroups; d.rev = p.reverse;
  return d;
}

template <typename TIO, typename TDT>
static int simt_fwd_stages(const issm_params& p, const SimtWs& w, const Dims& d, cudaStream_t s, bool for_bwd) {
  const dim3 gchunk(d.nc, d.H, d.b);
  const int nthr = d.N >= 256 ? 256 : (d.N + 31) / 32 * 32;
  ISSM_LAUNCH((k_prep<TDT>), gchunk, nthr, 0, s, d, (const TDT*)p.dt, p.dt_sb, p.dt_sl, p.dt_sh, p.A,
              p.has_dt_bias ? p.dt_bias : nullptr, p.dt_softplus, p.dt_min, p.dt_max, w.dtv, w.acs);
  ISSM_LAUNCH((k_chunk_state<0, TIO, TIO>), gchunk, nthr, 0, s, d, (const TIO*)p.x, p.x_sb, p.x_sl, p.x_sh,
              (const TIO*)p.B, p.B_sb, p.B_sl, p.B_sg, w.dtv, w.acs, w.states);
  const size_t tot = (size_t)d.b * d.H * d.P * d.N;
  ISSM_LAUNCH((k_pass_fwd<TIO>), (unsigned)cdiv64(tot, 256), 256, 0, s, d, w.states, w.acs,
              p.has_init ? (const TIO*)p.initial_states : nullptr,
              (!for_bwd && p.want_final) ? p.final_states : nullptr);
  return ISSM_OK;
}

template <typename TIO, typename TDT>
static int simt_fwd_t(const issm_params& p, cudaStream_t s) {
  const SimtLayout l = simt_layout(p);
  size_t total = 0;
  const SimtWs w = simt_carve(p, l, 0, &total);
  const Dims d = make_dims(p, l.nc);
  int rc = simt_fwd_stages<TIO, TDT>(p, w, d, s, false);
  if (rc) return rc;
  const int tiles = (d.Q + TR - 1) / TR;
  const size_t smem = (size_t)TR * (d.Q + 1) * sizeof(float);
  ISSM_LAUNCH((k_scan<false, TIO>), dim3(d.nc * tiles, d.H, d.b), 256, smem, s, d,
              (const TIO*)p.x, p.x_sb, p.x_sl, p.x_sh, (const TIO*)p.B, p.B_sb, p.B_sl, p.B_sg,
              (const TIO*)p.C, p.C_sb, p.C_sl, p.C_sg,
              p.has_z ? (const TIO*)p.z : nullptr, p.z_sb, p.z_sl, p.z_sh,
              p.has_D ? p.D : nullptr, p.D_has_hdim, w.dtv, w.acs, w.states, (const float*)nullptr,
              (TIO*)p.out, p.out_sb, p.out_sl, p.out_sh, (TIO*)p.out_x);
  return ISSM_OK;
}

template <typename TIO, typename TDT>
static int simt_bwd_t(const issm_params& p, cudaStream_t s) {
  const SimtLayout l = simt_layout(p);
  size_t total = 0;
  const SimtWs w = simt_carve(p, l, 1, &total);
  const Dims d = make_dims(p, l.nc);
  int rc = simt_fwd_stages<TIO, TDT>(p, w, d, s, true);   // recompute dtv, acs, entering states
  if (rc) return rc;
  const dim3 gchunk(d.nc, d.H, d.b);
  const int nthr = d.N >= 256 ? 256 : (d.N + 31) / 32 * 32;
  const size_t n_act = (size_t)d.b * d.L * d.H * d.P;
  // out_x holds y when gated (saved by the forward); strides are those of out
  ISSM_LAUNCH((k_dy<TIO>), (unsigned)cdiv64(n_act, 256), 256, 0, s, d, (const TIO*)p.dout, p.dout_sb, p.dout_sl,
              p.dout_sh, p.has_z ? (const TIO*)p.z : nullptr, p.z_sb, p.z_sl, p.z_sh,
              (const TIO*)p.out_x, p.out_sb, p.out_sl, p.out_sh, w.dy, (TIO*)p.dz);
  if (p.has_D)
    ISSM_LAUNCH((k_dD<TIO>), gchunk, 64, 0, s, d, w.dy, (const TIO*)p.x, p.x_sb, p.x_sl, p.x_sh, w.dDpart);
  ISSM_LAUNCH((k_chunk_state<1, float, TIO>), gchunk, nthr, 0, s, d, (const float*)w.dy,
              (int64_t)d.L * d.H * d.P, (int64_t)d.H * d.P, (int64_t)d.P,
              (const TIO*)p.C, p.C_sb, p.C_sl, p.C_sg, w.dtv, w.acs, w.dstates);
  ISSM_LAUNCH(k_pass_bwd, (unsigned)cdiv64((size_t)d.b * d.H * d.N, 128), 128, 0, s, d, w.dstates, w.states, w.acs,
              p.has_dfinal ? p.dfinal_states : nullptr, w.grun, w.ddac);
  if (p.dinitial_states) {
    const size_t tot = (size_t)d.b * d.H * d.P * d.N;
    ISSM_LAUNCH((k_cast_out<TIO>), (unsigned)cdiv64(tot, 256), 256, 0, s, w.grun, (TIO*)p.dinitial_states, tot);
  }
  ISSM_LAUNCH((k_dM<TIO>), gchunk, 256, 0, s, d, w.dy, (const TIO*)p.x, p.x_sb, p.x_sl, p.x_sh, w.dM);
  {
    const int tiles = (d.Q + TR - 1) / TR;
    const size_t smem = (size_t)TR * (d.Q + 1) * sizeof(float);
    ISSM_LAUNCH((k_scan<true, TIO>), dim3(d.nc * tiles, d.H, d.b), 256, smem, s, d,
                (const TIO*)p.x, p.x_sb, p.x_sl, p.x_sh, (const TIO*)p.B, p.B_sb, p.B_sl, p.B_sg,
                (const TIO*)p.C, p.C_sb, p.C_sl, p.C_sg, (const TIO*)nullptr, (int64_t)0, (int64_t)0, (int64_t)0,
                p.has_D ? p.D : nullptr, p.D_has_hdim, w.dtv, w.acs, w.dstates, w.dy,
                (TIO*)p.dx, (int64_t)0, (int64_t)0, (int64_t)0, (TIO*)nullptr);
  }
  {
    const int ntile = (d.N + 31) / 32;
    const size_t smem = (size_t)6 * d.Q * 32 * sizeof(float);
    struct MainTag {};
    if (smem > 48 * 1024) {                                // opt in (once per device) to the device's limit
      const size_t lim = max_optin_smem();
      if (smem > lim) return ISSM_ERR_SHAPE;
      if (SmemAttrOnce<MainTag>::set(k_main<TIO, TDT>, lim) != ISSM_OK) return ISSM_ERR_CUDA;
    }
    ISSM_LAUNCH((k_main<TIO, TDT>), dim3(d.nc * ntile, d.H, d.b), 256, smem, s, d,
                (const TIO*)p.x, p.x_sb, p.x_sl, p.x_sh, (const TIO*)p.B, p.B_sb, p.B_sl, p.B_sg,
                (const TIO*)p.C, p.C_sb, p.C_sl, p.C_sg, (const TDT*)p.dt, p.dt_sb, p.dt_sl, p.dt_sh,
                p.A, p.has_dt_bias ? p.dt_bias : nullptr, p.dt_softplus, p.dt_min, p.dt_max,
                w.dtv, w.acs, w.states, w.dstates, w.dy, w.dM, w.ddac,
                (TDT*)p.ddt, (TIO*)p.dB, (TIO*)p.dC, w.dBh, w.dCh, w.dApart, w.dbpart);
  }
  const int HN = d.H * d.N;
  ISSM_LAUNCH(k_reduce_rows, (HN + 127) / 128, 128, 0, s, w.dApart, d.b * d.nc, HN, p.dA);
  if (p.has_dt_bias && p.ddt_bias)
    ISSM_LAUNCH(k_reduce_rows, (HN + 127) / 128, 128, 0, s, w.dbpart, d.b * d.nc, HN, p.ddt_bias);
  if (p.has_D) {
    if (p.D_has_hdim)
      ISSM_LAUNCH(k_reduce_rows, (d.H * d.P + 127) / 128, 128, 0, s, w.dDpart, d.b * d.nc, d.H * d.P, p.dD);
    else
      ISSM_LAUNCH(k_reduce_dD_head, (d.H + 31) / 32, 32, 0, s, w.dDpart, d.b * d.nc, d.H, d.P, p.dD);
  }
  if (d.hpg > 1) {
    const size_t tot = (size_t)d.b * d.L * d.G * d.N;
    ISSM_LAUNCH((k_reduce_heads<TIO>), (unsigned)cdiv64(tot, 256), 256, 0, s, d, w.dBh, (TIO*)p.dB);
    ISSM_LAUNCH((k_reduce_heads<TIO>), (unsigned)cdiv64(tot, 256), 256, 0, s, d, w.dCh, (TIO*)p.dC);
  }
  return ISSM_OK;
}

#define ISSM_DISPATCH(fn)                                                              \
  if (p.io_dtype == ISSM_F32 && p.dt_dtype == ISSM_F32) return fn<float, float>(p, s); \
  if (p.io_dtype == ISSM_BF16 && p.dt_dtype == ISSM_BF16) return fn<bf16, bf16>(p, s); \
  if (p.io_dtype == ISSM_BF16 && p.dt_dtype == ISSM_F32) return fn<bf16, float>(p, s); \
  if (p.io_dtype == ISSM_F32 && p.dt_dtype == ISSM_BF16) return fn<float, bf16>(p, s); \
  return ISSM_ERR_DTYPE;

int simt_fwd(const issm_params& p, cudaStream_t s) { ISSM_DISPATCH(simt_fwd_t) }
int simt_bwd(const issm_params& p, cudaStream_t s) { ISSM_DISPATCH(simt_bwd_t) }

}  // namespace issm
