/* issm_b200.h - C ABI of the B200-native ISSM chunked scan and gated norms.
 *
 * Every entry point takes plain device pointers, element strides and sizes; no torch types.
 * The library never allocates, frees or synchronises (except where an entry point says so):
 * the caller owns every buffer, including the workspace, and all work is enqueued on the
 * stream handed in.  Host-detectable problems (bad shapes, unsupported dtype, workspace too
 * small, null pointers) are reported through the int return code before anything is launched;
 * use issm_b200_strerror() for a message.  Device-side problems (a bounded wait that expired)
 * are written to the optional `status` word and never trap.
 *
 * Reference interfaces these entry points replace (paths inside the reference project):
 *   issm_triton/issm_combined.py:57-92    _issm_chunk_scan_combined_fwd   -> issm_b200_fwd
 *   issm_triton/issm_combined.py:95-179   _issm_chunk_scan_combined_bwd   -> issm_b200_bwd
 *   issm_triton/layernorm_gated.py:98-137 _layer_norm_fwd                 -> issm_b200_norm_fwd
 *   issm_triton/layernorm_gated.py:261-325 _layer_norm_bwd                -> issm_b200_norm_bwd
 */
#ifndef ISSM_B200_H_
#define ISSM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ISSM_B200_VERSION 1

/* element types of the activation tensors */
enum { ISSM_F32 = 0, ISSM_BF16 = 1 };

/* which kernels serve a call */
enum {
  ISSM_PATH_AUTO = 0,    /* bf16 activations + supported shape -> tensor-core path, else SIMT   */
  ISSM_PATH_SIMT = 1,    /* fp32-arithmetic SIMT kernels, any supported shape, any value range  */
  ISSM_PATH_TENSOR = 2   /* tcgen05 path; returns ISSM_ERR_UNSUPPORTED if the shape has none    */
};

/* return codes */
enum {
  ISSM_OK = 0,
  ISSM_ERR_NULL = 1,          /* a required pointer is null                     */
  ISSM_ERR_SHAPE = 2,         /* sizes out of the supported range               */
  ISSM_ERR_DTYPE = 3,         /* unknown dtype enum                             */
  ISSM_ERR_WORKSPACE = 4,     /* workspace missing or smaller than required     */
  ISSM_ERR_ALIGN = 5,         /* pointer or stride alignment not met            */
  ISSM_ERR_UNSUPPORTED = 6,   /* requested path does not cover this shape       */
  ISSM_ERR_CUDA = 7,          /* a CUDA runtime call failed (launch, attribute) */
  ISSM_ERR_DEVICE_STATUS = 8, /* reserved: device status word was non-zero      */
  ISSM_ERR_LIMIT = 9          /* size beyond the built-in scratch of a no-allocation entry point */
};

/* One ISSM scan call (forward, or forward-recompute + backward).
 *
 * Shapes (reference: issm_triton/issm_combined.py:16-35).  All strides are in ELEMENTS; the
 * innermost dimension of every tensor is contiguous.
 *   x, z, out, out_x, dout, dx, dz : (batch, seqlen, nheads, headdim)   dtype io_dtype
 *   dt, ddt                        : (batch, seqlen, nheads, dstate)    dtype dt_dtype
 *   B, C, dB, dC                   : (batch, seqlen, ngroups, dstate)   dtype io_dtype
 *   A, dt_bias, dA, ddt_bias       : (nheads, dstate) float, contiguous
 *   D, dD                          : (nheads) or (nheads, headdim) float, contiguous
 *   initial_states, dinitial_states: (batch, nheads, headdim, dstate)   dtype io_dtype, contiguous
 *   final_states, dfinal_states    : (batch, nheads, headdim, dstate)   float, contiguous
 * `reverse` scans from the last point to the first (equal to flipping x, dt, B, C, z along
 * seqlen, scanning, flipping out back: models/dest_module.py:567-573) without any copy.
 */
typedef struct issm_params {
  int32_t batch, seqlen, nheads, headdim, dstate, ngroups, chunk_size;
  int32_t io_dtype, dt_dtype;
  int32_t path;                 /* ISSM_PATH_* */
  int32_t has_D, D_has_hdim, has_z, has_dt_bias, dt_softplus;
  int32_t has_init, has_dfinal, reverse, want_final;
  float dt_min, dt_max;         /* clamp applied after bias/softplus (issm_chunk_state.py:97) */

  const void* x;   int64_t x_sb, x_sl, x_sh;
  const void* dt;  int64_t dt_sb, dt_sl, dt_sh;
  const void* B;   int64_t B_sb, B_sl, B_sg;
  const void* C;   int64_t C_sb, C_sl, C_sg;
  const void* z;   int64_t z_sb, z_sl, z_sh;
  const float* A;
  const float* D;
  const float* dt_bias;
  const void* initial_states;

  /* forward outputs */
  void* out;       int64_t out_sb, out_sl, out_sh;
  void* out_x;     /* pre-gate y, same strides as out; required when has_z (saved for bwd) */
  float* final_states;          /* required when want_final */

  /* backward inputs */
  const void* dout; int64_t dout_sb, dout_sl, dout_sh;
  const float* dfinal_states;
  /* backward outputs (contiguous, same shapes as the matching inputs) */
  void* dx; void* ddt; void* dB; void* dC; void* dz;
  float* dA; float* ddt_bias; float* dD;
  void* dinitial_states;        /* optional */

  void* workspace; size_t workspace_bytes;
  /* Optional device word the kernels OR bits into (never cleared by the library):
   *   bit 0 (1): a bounded device-side wait expired; the affected call's results are invalid.
   *   bit 2 (4): informational; some 64-point block of a (batch, head) stream exceeded the decay range of the
   *              tensor-core factorisation and that stream was redone by the windowed kernels (results exact). */
  int32_t* status;
  /* Optional, tensor path only: batch * nheads * (ceil(seqlen/64) + 1) * dstate * 48 bf16 elements, laid out
   * (batch, nheads, block, 6, dstate, 8): head-dim chunk, state, 8 head-dim values (padded to 48).  The
   * forward stores the state entering every 64-point block (and the final state) here; a backward given
   * the same buffer skips recomputing them (the reference recomputes: issm_combined.py:136-144). */
  void* saved_states;
} issm_params;

/* Gated RMS / Layer norm over the last dimension of a (rows, hidden) matrix
 * (issm_triton/layernorm_gated.py:35-95): y = norm(x) * silu(z) if norm_before_gate,
 * else norm(x * silu(z)); statistics per group of group_size features. */
typedef struct issm_norm_params {
  int32_t rows, hidden, group_size;   /* group_size divides hidden */
  int32_t io_dtype;                   /* x, z, y, dy, dx, dz */
  int32_t is_rms, norm_before_gate, has_z, has_bias;
  float eps;
  const void* x; int64_t x_sr;        /* row strides in elements */
  const void* z; int64_t z_sr;
  const float* weight; const float* bias;
  void* y; int64_t y_sr;
  float* rstd;                        /* (rows * hidden/group_size) */
  float* mean;                        /* same size; LayerNorm only */
  /* backward */
  const void* dy; int64_t dy_sr;
  void* dx; void* dz;                 /* contiguous (rows, hidden) */
  float* dweight; float* dbias;       /* (hidden) */
  void* workspace; size_t workspace_bytes;
} issm_norm_params;

int issm_b200_version(void);
const char* issm_b200_strerror(int code);
/* sizeof(issm_params) / sizeof(issm_norm_params) as compiled, so a foreign-language binding can
 * check its own struct declaration against the library's. */
size_t issm_b200_sizeof_params(void);
size_t issm_b200_sizeof_norm_params(void);

/* Bytes of workspace issm_b200_fwd (pass = 0) or issm_b200_bwd (pass = 1) needs for these
 * sizes, dtypes, flags and path.  Returns 0 on invalid sizes.  No pointer is dereferenced, but
 * two properties of the pointers select the kernels and with them the size, so they must be the
 * same in this query and in the call that follows: the alignment of x, z, out, out_x, dout, dx, dz
 * (8 bytes) and of B, C, bf16 dt (16 bytes) decides between the tensor-core and the SIMT kernels
 * under ISSM_PATH_AUTO (null pointers count as aligned), and a backward without `saved_states`
 * needs room to recompute them.  A query made with null pointers therefore sizes the workspace of
 * an aligned call that passes saved_states iff it is non-null in the query. */
size_t issm_b200_workspace_bytes(const issm_params* p, int pass);

/* Which path (ISSM_PATH_SIMT or ISSM_PATH_TENSOR) a forward call with these sizes would take; -1 when the
 * requested path does not cover them. */
int issm_b200_resolve_path(const issm_params* p);
/* The same per pass (0 = forward, 1 = backward); `saved_states` is only of use when the BACKWARD takes the
 * tensor path.  (dstate 512 / 768 / 1024 run on the tensor-core kernels in both passes: one 256-state slice per
 * CTA, the partial output rows / partial dx rows summed by a combine kernel.) */
int issm_b200_resolve_path_pass(const issm_params* p, int pass);

int issm_b200_fwd(const issm_params* p, void* cuda_stream);
int issm_b200_bwd(const issm_params* p, void* cuda_stream);

size_t issm_b200_norm_workspace_bytes(const issm_norm_params* p, int pass);
int issm_b200_norm_fwd(const issm_norm_params* p, void* cuda_stream);
int issm_b200_norm_bwd(const issm_norm_params* p, void* cuda_stream);

/* Backward of the gated norm WITHOUT any workspace (this entry point has no counterpart in the
 * reference).  For hosts that cannot allocate device memory when they call: a server plugin whose
 * memory pool is sealed after start-up, a latency-critical loop, or a language binding with no
 * device allocator.  Same arguments and results as issm_b200_norm_bwd; `workspace` /
 * `workspace_bytes` are ignored, and the per-block weight / bias gradient partials go to a fixed
 * device array inside the library (4.6 MiB per GPU, held until the process exits).
 *   - Limit: hidden <= 1024; a wider row returns ISSM_ERR_LIMIT and launches nothing.
 *   - Neither this call nor anything it uses allocates or frees device memory.
 *   - The first call on each device looks up the array's device address (the device of the call
 *     must be current) and, with lazy module loading, is also what makes the driver load the
 *     library's device code, array included: make that first (warm-up) call at start-up, outside
 *     any stream capture.  The address is cached for the life of the process; a cudaDeviceReset of
 *     that device invalidates it (do not reset a device and then call this entry point again).
 *   - All calls on a device share the one array, which keeps whatever the previous call left in
 *     it (each call overwrites all it reads).  Two calls whose kernels overlap in time on the same
 *     GPU - different streams, or different host threads - race on it: serialise them. */
int issm_b200_norm_bwd_noalloc(const issm_norm_params* p, void* cuda_stream);

/* ---- the point-wise steps on either side of the scan in the detector's ISSM block ----------------------- */

/* Serialization gather (models/dest_module.py:378-397, points.gather(dim = 1, index)): for every batch b and
 * output row i, dst[b, i, :] = src[b, index[b, i], :].  Rows are `row_bytes` contiguous bytes (even); dst is
 * (batch, n_out, row_bytes) contiguous, src rows are src_row_bytes apart and batches src_batch_bytes apart; index is
 * (batch, n_out) int64, contiguous.  An index outside [0, n_src) copies nothing for that row and ORs bit 1 (value 2)
 * into *status (optional). */
int issm_b200_gather_rows(const void* src, const int64_t* index, void* dst, int32_t batch, int32_t n_out, int32_t n_src,
                          int64_t row_bytes, int64_t src_batch_bytes, int64_t src_row_bytes, int32_t* status, void* cuda_stream);

/* PointLiteConv (models/dest_module.py:400-423): y = silu(conv + bias), conv a depthwise 1-D convolution with 7 taps
 * and zero padding 3 along the point axis of a channels-last (batch, seqlen, channels) tensor - what the reference
 * computes as nn.Conv1d(C, C, 7, padding = 3, groups = C) on the transposed tensor followed by nn.SiLU. */
typedef struct issm_conv_params {
  int32_t batch, seqlen, channels;
  int32_t io_dtype;                       /* x, y, dy, dx */
  const void* x; int64_t x_sb, x_sl;      /* element strides of batch and point; channel stride 1 */
  const float* weight;                    /* (channels, 7): Conv1d's (C, 1, 7) weight as float */
  const float* bias;                      /* (channels) or null */
  void* y;                                /* (batch, seqlen, channels) contiguous */
  /* backward */
  const void* dy; int64_t dy_sb, dy_sl;
  void* dx;                               /* contiguous */
  float* dweight;                         /* (channels, 7) */
  float* dbias;                           /* (channels) or null */
  void* workspace; size_t workspace_bytes;/* backward only; 256-byte aligned */
} issm_conv_params;

size_t issm_b200_sizeof_conv_params(void);
size_t issm_b200_dwconv_workspace_bytes(const issm_conv_params* p);
int issm_b200_dwconv7_silu_fwd(const issm_conv_params* p, void* cuda_stream);
int issm_b200_dwconv7_silu_bwd(const issm_conv_params* p, void* cuda_stream);

/* ---- the parameter generation in front of the scan (models/dest_module.py:541-559) ------------------------- */

/* dt, B, C (and the second direction's B, C) from the query-to-point distance features in ONE pass over them:
 *   pre[r]  = dist[b, l, k, :] . weight[r, :]            r = 0 .. nheads + 2 ngroups - 1   (dt_proj rows, then bc_proj rows)
 *   dt[b, l, h, k]  = softplus(pre[h] + tok[b, l, h]) * mask[b, l, k]                       (softplus threshold 20)
 *   bc[b, l, i, k]  = pre[nheads + i] + tok[b, l, nheads + i]                i < 2 ngroups: B rows then C rows
 *   bc[b, l, 2 ngroups + i, k] = pre[nheads + i] + tok[b, l, nheads + 2 ngroups + i]        only when has_back
 * tok holds the per-token terms the caller adds (key_proj's dt_bias split plus the dt_bias parameter; b_bias, c_bias;
 * their second-direction counterparts), float, (batch, seqlen, nheads + 2 ngroups [+ 2 ngroups]).
 * Backward: ddt / dbc (either may be null) -> ddist (batch, seqlen, nstates, nfeat), dweight (shape of weight; the
 * second direction's B / C rows add to the rows they share) and dtok (shape of tok); needs a workspace of
 * issm_b200_glue_workspace_bytes() for the per-block partial weight gradients, summed in a fixed order. */
typedef struct issm_glue_params {
  int32_t batch, seqlen, nstates, nfeat;  /* nfeat = 4, 8 or 16 */
  int32_t nheads, ngroups, has_back;
  int32_t io_dtype;                       /* dt, bc, ddt, dbc */
  int32_t dist_dtype;                     /* dist, ddist: io_dtype, or ISSM_F32 next to ISSM_BF16 outputs (float features, bfloat16 activations) */
  const void* dist; int64_t dist_sb, dist_sl, dist_sk;   /* element strides; feature stride 1; 16-byte aligned rows */
  const float* weight;                    /* (nheads + 2 ngroups, nfeat) */
  const float* tok;
  const float* mask;                      /* (batch, seqlen, nstates) multiplier or null */
  void* dt;                               /* (batch, seqlen, nheads, nstates) contiguous */
  void* bc;                               /* (batch, seqlen, 2 ngroups [+ 2 ngroups], nstates) contiguous */
  /* backward */
  const void* ddt; const void* dbc;
  void* ddist; float* dweight; float* dtok;
  void* workspace; size_t workspace_bytes;
} issm_glue_params;

size_t issm_b200_sizeof_glue_params(void);
size_t issm_b200_glue_workspace_bytes(const issm_glue_params* p);
int issm_b200_glue_fwd(const issm_glue_params* p, void* cuda_stream);
int issm_b200_glue_bwd(const issm_glue_params* p, void* cuda_stream);

/* ---- one sequence cut into slices (several GPUs, or extra batch entries on one GPU) ----------------------- */

/* Sums of the transformed step size over segments of `rows_per_part` points:
 *   part[seg, b, h, n] = sum_l clamp(softplus?(dt[b, l, h, n] + dt_bias[h, n]), dt_min, dt_max),
 * part is (ceil(seqlen / rows_per_part), batch, nheads, dstate) float, contiguous; dt has element strides dt_sb, dt_sl,
 * dt_sh and state stride 1; dt_bias is (nheads, dstate) float or null.  exp(A * sum over a slice) is the factor the
 * slice applies to the state entering it - what dA_cumsum[..., -1] of a chunk is to the reference's state passing
 * (issm_triton/issm_state_passing.py:92-107). */
int issm_b200_dt_sum(const void* dt, int32_t dt_dtype, int32_t batch, int32_t seqlen, int32_t nheads, int32_t dstate,
                     int64_t dt_sb, int64_t dt_sl, int64_t dt_sh, const float* dt_bias, int32_t dt_softplus, float dt_min,
                     float dt_max, int32_t rows_per_part, float* part, void* cuda_stream);

/* Number of kernel launches the library has enqueued since load (monotonic, process-wide);
 * used by the benchmark to report how many of its own kernels ran inside a timed region. */
uint64_t issm_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ISSM_B200_H_ */
