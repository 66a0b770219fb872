// C ABI of the ISSM scan: argument validation, path selection, dispatch.  See include/issm_b200.h.
#include "issm_common.cuh"

namespace issm {
std::atomic<uint64_t> g_launches{0};

static int validate(const issm_params* p, int pass) {
  if (!p) return ISSM_ERR_NULL;
  if (p->batch <= 0 || p->seqlen <= 0 || p->nheads <= 0 || p->headdim <= 0 || p->dstate <= 0 ||
      p->ngroups <= 0 || p->chunk_size <= 0)
    return ISSM_ERR_SHAPE;
  if (p->nheads % p->ngroups) return ISSM_ERR_SHAPE;
  if (p->chunk_size > 256) return ISSM_ERR_SHAPE;            // shared-memory tiles are sized for <= 256 rows
  if (p->batch > 65535 || p->nheads > 65535) return ISSM_ERR_SHAPE;
  if ((p->io_dtype != ISSM_F32 && p->io_dtype != ISSM_BF16) || (p->dt_dtype != ISSM_F32 && p->dt_dtype != ISSM_BF16))
    return ISSM_ERR_DTYPE;
  if (p->path < ISSM_PATH_AUTO || p->path > ISSM_PATH_TENSOR) return ISSM_ERR_UNSUPPORTED;
  if (!(p->dt_min <= p->dt_max)) return ISSM_ERR_SHAPE;
  return ISSM_OK;
}

static int validate_ptrs(const issm_params* p, int pass) {
  if (!p->x || !p->dt || !p->A || !p->B || !p->C) return ISSM_ERR_NULL;
  if (p->has_D && !p->D) return ISSM_ERR_NULL;
  if (p->has_z && (!p->z || !p->out_x)) return ISSM_ERR_NULL;
  if (p->has_dt_bias && !p->dt_bias) return ISSM_ERR_NULL;
  if (p->has_init && !p->initial_states) return ISSM_ERR_NULL;
  if (pass == 0) {
    if (!p->out) return ISSM_ERR_NULL;
    if (p->want_final && !p->final_states) return ISSM_ERR_NULL;
  } else {
    if (!p->dout || !p->dx || !p->ddt || !p->dB || !p->dC || !p->dA) return ISSM_ERR_NULL;
    if (p->has_z && !p->dz) return ISSM_ERR_NULL;
    if (p->has_D && !p->dD) return ISSM_ERR_NULL;
    if (p->has_dt_bias && !p->ddt_bias) return ISSM_ERR_NULL;
    if (p->has_dfinal && !p->dfinal_states) return ISSM_ERR_NULL;
  }
  return ISSM_OK;
}

// The stride of a dimension of size 1 is never used, and frameworks report arbitrary values there (a (b, L, 1, N) sum
// of broadcast views comes back with group stride 1): give such strides the value a contiguous tensor would have, so
// that they cannot fail an alignment rule or be taken for a gap between rows.
static issm_params canonical(const issm_params& in) {
  issm_params p = in;
  if (p.nheads == 1) { p.x_sh = p.z_sh = p.out_sh = p.dout_sh = p.headdim; p.dt_sh = p.dstate; }
  if (p.ngroups == 1) p.B_sg = p.C_sg = p.dstate;
  if (p.seqlen == 1) {
    p.x_sl = p.nheads * p.x_sh; p.z_sl = p.nheads * p.z_sh; p.out_sl = p.nheads * p.out_sh; p.dout_sl = p.nheads * p.dout_sh;
    p.dt_sl = p.nheads * p.dt_sh; p.B_sl = p.ngroups * p.B_sg; p.C_sl = p.ngroups * p.C_sg;
  }
  if (p.batch == 1) {
    p.x_sb = p.seqlen * p.x_sl; p.z_sb = p.seqlen * p.z_sl; p.out_sb = p.seqlen * p.out_sl; p.dout_sb = p.seqlen * p.dout_sl;
    p.dt_sb = p.seqlen * p.dt_sl; p.B_sb = p.seqlen * p.B_sl; p.C_sb = p.seqlen * p.C_sl;
  }
  return p;
}

static int resolve(const issm_params& p, int pass) {
  if (p.path == ISSM_PATH_SIMT) return ISSM_PATH_SIMT;
  const bool ok = tensor_path_supported(p, pass);
  if (p.path == ISSM_PATH_TENSOR) return ok ? ISSM_PATH_TENSOR : -1;
  return ok ? ISSM_PATH_TENSOR : ISSM_PATH_SIMT;
}
}  // namespace issm

using namespace issm;

extern "C" int issm_b200_version(void) { return ISSM_B200_VERSION; }

extern "C" const char* issm_b200_strerror(int code) {
  switch (code) {
    case ISSM_OK: return "ok";
    case ISSM_ERR_NULL: return "a required pointer is null";
    case ISSM_ERR_SHAPE: return "sizes out of the supported range (all > 0, nheads % ngroups == 0, chunk_size <= 256)";
    case ISSM_ERR_DTYPE: return "unknown dtype";
    case ISSM_ERR_WORKSPACE: return "workspace missing or too small (see issm_b200_workspace_bytes)";
    case ISSM_ERR_ALIGN: return "pointer or stride alignment not met";
    case ISSM_ERR_UNSUPPORTED: return "requested path does not cover this shape";
    case ISSM_ERR_CUDA: return "a CUDA runtime call failed";
    case ISSM_ERR_DEVICE_STATUS: return "device status word is non-zero";
    case ISSM_ERR_LIMIT: return "size exceeds the built-in scratch of the no-allocation entry point (hidden <= 1024)";
    default: return "unknown error code";
  }
}

extern "C" size_t issm_b200_sizeof_params(void) { return sizeof(issm_params); }
extern "C" size_t issm_b200_sizeof_norm_params(void) { return sizeof(issm_norm_params); }
extern "C" uint64_t issm_b200_launch_count(void) { return g_launches.load(); }

extern "C" int issm_b200_resolve_path(const issm_params* p) {
  if (validate(p, 0)) return -1;
  return resolve(canonical(*p), 0);
}
extern "C" int issm_b200_resolve_path_pass(const issm_params* p, int pass) {
  if (validate(p, pass) || (pass != 0 && pass != 1)) return -1;
  return resolve(canonical(*p), pass);
}

extern "C" size_t issm_b200_workspace_bytes(const issm_params* p, int pass) {
  if (validate(p, pass) || (pass != 0 && pass != 1)) return 0;
  const issm_params q = canonical(*p);
  const int path = resolve(q, pass);
  if (path < 0) return 0;
  return path == ISSM_PATH_TENSOR ? tensor_workspace_bytes(q, pass) : simt_workspace_bytes(q, pass);
}

static int run(const issm_params* in, void* stream, int pass) {
  int rc = validate(in, pass);
  if (rc) return rc;
  rc = validate_ptrs(in, pass);
  if (rc) return rc;
  const issm_params q = canonical(*in);
  const issm_params* p = &q;
  const int path = resolve(*p, pass);
  if (path < 0) return ISSM_ERR_UNSUPPORTED;
  const size_t need = path == ISSM_PATH_TENSOR ? tensor_workspace_bytes(*p, pass) : simt_workspace_bytes(*p, pass);
  if (need && (!p->workspace || p->workspace_bytes < need)) return ISSM_ERR_WORKSPACE;
  if ((uintptr_t)p->workspace % 256) return ISSM_ERR_ALIGN;
  if (path == ISSM_PATH_TENSOR) {
    // buffers the tensor-core kernels touch with 16-byte vector or bulk accesses and that the path selection
    // does not look at (a misaligned x / B / C / dt selects the SIMT kernels instead)
    if ((uintptr_t)p->saved_states % 16) return ISSM_ERR_ALIGN;
    if (pass == 1 && (((uintptr_t)p->dB | (uintptr_t)p->dC) % 16)) return ISSM_ERR_ALIGN;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (path == ISSM_PATH_TENSOR) return pass == 0 ? tensor_fwd(*p, s) : tensor_bwd(*p, s);
  return pass == 0 ? simt_fwd(*p, s) : simt_bwd(*p, s);
}

extern "C" int issm_b200_fwd(const issm_params* p, void* stream) { return run(p, stream, 0); }
extern "C" int issm_b200_bwd(const issm_params* p, void* stream) { return run(p, stream, 1); }
