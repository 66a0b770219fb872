// Torch C++ extension over the C ABI of include/issm_b200.h: TORCH_LIBRARY(issm_b200) ops `fwd`, `bwd`,
// `norm_fwd`, `norm_bwd`.  Each op validates its tensors the way the reference's Python wrappers do
// (issm_triton/issm_combined.py:58-82, issm_triton/layernorm_gated.py:98-137), makes them stride-compatible
// (unit stride in the last dimension), allocates outputs and workspace with torch's caching allocator, fills
// the parameter struct and calls the library on the current stream of the tensors' device.  No kernel lives
// here: this file is host-side C++ only and links against libissm_b200.so.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <cmath>
#include <tuple>
#include <vector>

#include "../../include/issm_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

int dtype_code(at::ScalarType t) {
  if (t == at::kFloat) return ISSM_F32;
  if (t == at::kBFloat16) return ISSM_BF16;
  TORCH_CHECK(false, "issm_b200: unsupported dtype ", t, " (the ISSM kernels take float32 or bfloat16)");
  return -1;
}

// activation tensor in the io dtype with a unit innermost stride; `keep` holds every temporary alive
Tensor act(const Tensor& t, at::ScalarType io, std::vector<Tensor>& keep) {
  Tensor r = t.scalar_type() == io ? t : t.to(io);
  if (r.stride(-1) != 1) r = r.contiguous();
  keep.push_back(r);
  return r;
}
Tensor par(const Tensor& t, std::vector<Tensor>& keep) {
  Tensor r = t.detach().to(at::kFloat).contiguous();
  keep.push_back(r);
  return r;
}
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, ": error ", rc, ": ", issm_b200_strerror(rc));
}
void* stream_of(const Tensor& t) { return (void*)c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }
Tensor none_like(const Tensor& t) { return at::empty({0}, t.options()); }

struct Common {
  issm_params p{};
  std::vector<Tensor> keep;
  Tensor x, dt, B, C;
};

// what issm_combined.py:58-82 checks, plus the struct fill shared by forward and backward
void fill_common(Common& c, const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C,
                 int64_t chunk_size, const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias,
                 const OptTensor& initial_states, bool dt_softplus, double dt_min, double dt_max, bool reverse,
                 int64_t path, const Tensor& status) {
  TORCH_CHECK(x.is_cuda(), "ISSM_chunk_scan_combined runs on CUDA tensors only; there is no CPU path");
  TORCH_CHECK(x.dim() == 4 && B.dim() == 4 && dt.dim() == 4 && A.dim() == 2, "issm_b200: x, dt, B, C must be 4-D and A 2-D");
  const int64_t batch = x.size(0), seqlen = x.size(1), nheads = x.size(2), headdim = x.size(3);
  const int64_t ngroups = B.size(2), dstate = B.size(3);
  TORCH_CHECK(nheads % ngroups == 0, "issm_b200: nheads must be divisible by ngroups");
  TORCH_CHECK(B.size(0) == batch && B.size(1) == seqlen, "issm_b200: B must be (batch, seqlen, ngroups, dstate)");
  TORCH_CHECK(dt.sizes() == at::IntArrayRef({batch, seqlen, nheads, dstate}), "issm_b200: dt must be (batch, seqlen, nheads, dstate)");
  TORCH_CHECK(A.sizes() == at::IntArrayRef({nheads, dstate}), "issm_b200: A must be (nheads, dstate)");
  TORCH_CHECK(C.sizes() == B.sizes(), "issm_b200: C must have the shape of B");
  if (z) TORCH_CHECK(z->sizes() == x.sizes(), "issm_b200: z must have the shape of x");
  if (D) TORCH_CHECK((D->dim() == 1 && D->size(0) == nheads) || (D->dim() == 2 && D->size(0) == nheads && D->size(1) == headdim),
                     "issm_b200: D must be (nheads,) or (nheads, headdim)");
  if (initial_states)
    TORCH_CHECK(initial_states->sizes() == at::IntArrayRef({batch, nheads, headdim, dstate}),
                "issm_b200: initial_states must be (batch, nheads, headdim, dstate)");
  const at::ScalarType io = x.scalar_type();
  issm_params& p = c.p;
  c.x = act(x, io, c.keep);
  c.B = act(B, io, c.keep);
  c.C = act(C, io, c.keep);
  Tensor dtk = (dt.scalar_type() == at::kFloat || dt.scalar_type() == at::kBFloat16) ? dt : dt.to(at::kFloat);
  if (dtk.stride(-1) != 1) dtk = dtk.contiguous();
  c.keep.push_back(dtk);
  c.dt = dtk;
  const Tensor Ak = par(A, c.keep);
  p.batch = (int32_t)batch; p.seqlen = (int32_t)seqlen; p.nheads = (int32_t)nheads; p.headdim = (int32_t)headdim;
  p.dstate = (int32_t)dstate; p.ngroups = (int32_t)ngroups; p.chunk_size = (int32_t)chunk_size;
  p.io_dtype = dtype_code(io);
  p.dt_dtype = dtype_code(dtk.scalar_type());
  p.path = (int32_t)path;
  p.has_D = D.has_value(); p.D_has_hdim = D.has_value() && D->dim() == 2;
  p.has_z = z.has_value(); p.has_dt_bias = dt_bias.has_value(); p.dt_softplus = dt_softplus;
  p.has_init = initial_states.has_value(); p.reverse = reverse;
  p.dt_min = (float)dt_min;
  p.dt_max = (float)std::fmin(dt_max, 3.0e38);
  p.x = c.x.data_ptr(); p.x_sb = c.x.stride(0); p.x_sl = c.x.stride(1); p.x_sh = c.x.stride(2);
  p.dt = dtk.data_ptr(); p.dt_sb = dtk.stride(0); p.dt_sl = dtk.stride(1); p.dt_sh = dtk.stride(2);
  p.B = c.B.data_ptr(); p.B_sb = c.B.stride(0); p.B_sl = c.B.stride(1); p.B_sg = c.B.stride(2);
  p.C = c.C.data_ptr(); p.C_sb = c.C.stride(0); p.C_sl = c.C.stride(1); p.C_sg = c.C.stride(2);
  if (z) {
    const Tensor zk = act(*z, io, c.keep);
    p.z = zk.data_ptr(); p.z_sb = zk.stride(0); p.z_sl = zk.stride(1); p.z_sh = zk.stride(2);
  }
  p.A = Ak.data_ptr<float>();
  if (D) p.D = par(*D, c.keep).data_ptr<float>();
  if (dt_bias) {
    // (nheads, dstate) as the reference asserts (issm_chunk_state.py:14-15); (nheads,) is broadcast
    Tensor bias = dt_bias->dim() == 2 ? *dt_bias : dt_bias->unsqueeze(1).expand({nheads, dstate});
    TORCH_CHECK(bias.sizes() == at::IntArrayRef({nheads, dstate}), "issm_b200: dt_bias must be (nheads, dstate) or (nheads,)");
    p.dt_bias = par(bias, c.keep).data_ptr<float>();
  }
  if (initial_states) {
    Tensor ik = initial_states->to(io).contiguous();
    c.keep.push_back(ik);
    p.initial_states = ik.data_ptr();
  }
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1, "issm_b200: status must be a CUDA int32 tensor");
  p.status = status.data_ptr<int32_t>();
}

void attach_workspace(Common& c, int pass) {
  const size_t need = issm_b200_workspace_bytes(&c.p, pass);
  Tensor ws = at::empty({(int64_t)std::max<size_t>(need, 256)}, c.x.options().dtype(at::kByte));
  c.keep.push_back(ws);
  c.p.workspace = ws.data_ptr();
  c.p.workspace_bytes = (size_t)ws.numel();
}

// Forward; counterpart of _issm_chunk_scan_combined_fwd (issm_combined.py:57-92).
// Returns (out, out_x, final_states, saved_states); absent ones are 0-element tensors.
std::tuple<Tensor, Tensor, Tensor, Tensor> fwd(const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C,
                                               int64_t chunk_size, const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias,
                                               const OptTensor& initial_states, bool dt_softplus, double dt_min, double dt_max,
                                               bool reverse, int64_t path, bool want_final, bool save_states, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(x.device());
  Common c;
  fill_common(c, x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_min, dt_max, reverse, path, status);
  issm_params& p = c.p;
  const auto opt = c.x.options();
  Tensor out = at::empty(c.x.sizes(), opt);
  Tensor out_x = z ? at::empty(c.x.sizes(), opt) : none_like(out);
  Tensor fin = want_final ? at::empty({p.batch, p.nheads, p.headdim, p.dstate}, opt.dtype(at::kFloat)) : none_like(out);
  Tensor saved = none_like(out);
  if (save_states && issm_b200_resolve_path_pass(&p, 1) == ISSM_PATH_TENSOR) {
    // the tensor-core backward reads the state entering every 64-point block instead of recomputing it
    saved = at::empty({p.batch, p.nheads, (p.seqlen + 63) / 64 + 1, p.dstate, 48}, opt.dtype(at::kBFloat16));
    p.saved_states = saved.data_ptr();
  }
  p.out = out.data_ptr(); p.out_sb = out.stride(0); p.out_sl = out.stride(1); p.out_sh = out.stride(2);
  p.out_x = z ? out_x.data_ptr() : nullptr;
  p.final_states = want_final ? fin.data_ptr<float>() : nullptr;
  p.want_final = want_final;
  attach_workspace(c, 0);
  check_rc(issm_b200_fwd(&p, stream_of(c.x)), "issm_b200_fwd");
  return {out, out_x, fin, saved};
}

// Backward; counterpart of _issm_chunk_scan_combined_bwd (issm_combined.py:95-179).
// Returns (dx, ddt, dA, dB, dC, dD, dz, ddt_bias, dinitial_states); absent ones are 0-element tensors;
// dA / dD / ddt_bias are float32.
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> bwd(
    const Tensor& dout, const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C, const OptTensor& out_x,
    int64_t chunk_size, const OptTensor& D, const OptTensor& z, const OptTensor& dt_bias, const OptTensor& initial_states,
    const OptTensor& dfinal_states, bool dt_softplus, double dt_min, double dt_max, bool reverse, int64_t path,
    const OptTensor& saved_states, const Tensor& status) {
  const c10::cuda::CUDAGuard guard(x.device());
  Common c;
  fill_common(c, x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_min, dt_max, reverse, path, status);
  issm_params& p = c.p;
  const at::ScalarType io = c.x.scalar_type();
  const auto opt = c.x.options();
  const Tensor doutk = act(dout, io, c.keep);
  TORCH_CHECK(doutk.sizes() == c.x.sizes(), "issm_b200: dout must have the shape of x");
  Tensor dx = at::empty(c.x.sizes(), opt);
  Tensor ddt = at::empty(c.dt.sizes(), opt.dtype(c.dt.scalar_type()));
  Tensor dB = at::empty(c.B.sizes(), opt);
  Tensor dC = at::empty(c.C.sizes(), opt);
  Tensor dz = z ? at::empty(c.x.sizes(), opt) : none_like(dx);
  Tensor dA = at::empty({p.nheads, p.dstate}, opt.dtype(at::kFloat));
  Tensor dbias = dt_bias ? at::empty({p.nheads, p.dstate}, opt.dtype(at::kFloat)) : none_like(dA);
  Tensor dD = D ? at::empty(D->sizes(), opt.dtype(at::kFloat)) : none_like(dA);
  Tensor dinit = initial_states ? at::empty(initial_states->sizes(), opt) : none_like(dx);
  if (z) {
    TORCH_CHECK(out_x.has_value() && out_x->is_contiguous() && out_x->sizes() == c.x.sizes(),
                "issm_b200: the pre-gate output saved by the forward is required when z is given");
    p.out_x = out_x->data_ptr();
    p.out_sb = out_x->stride(0); p.out_sl = out_x->stride(1); p.out_sh = out_x->stride(2);
  }
  p.dout = doutk.data_ptr(); p.dout_sb = doutk.stride(0); p.dout_sl = doutk.stride(1); p.dout_sh = doutk.stride(2);
  if (dfinal_states) {
    Tensor dfin = dfinal_states->to(at::kFloat).contiguous();
    c.keep.push_back(dfin);
    p.has_dfinal = 1;
    p.dfinal_states = dfin.data_ptr<float>();
  }
  p.dx = dx.data_ptr(); p.ddt = ddt.data_ptr(); p.dB = dB.data_ptr(); p.dC = dC.data_ptr();
  p.dz = z ? dz.data_ptr() : nullptr;
  p.dA = dA.data_ptr<float>();
  p.ddt_bias = dt_bias ? dbias.data_ptr<float>() : nullptr;
  p.dD = D ? dD.data_ptr<float>() : nullptr;
  p.dinitial_states = initial_states ? dinit.data_ptr() : nullptr;
  if (saved_states && saved_states->numel() > 0) p.saved_states = saved_states->data_ptr();
  attach_workspace(c, 1);
  check_rc(issm_b200_bwd(&p, stream_of(c.x)), "issm_b200_bwd");
  return {dx, ddt, dA, dB, dC, dD, dz, dbias, dinit};
}

// ---- gated norms ------------------------------------------------------------------------------------
void fill_norm(issm_norm_params& p, const Tensor& x2, const OptTensor& z2, const Tensor& weight, const OptTensor& bias,
               double eps, int64_t group_size, bool norm_before_gate, bool is_rms) {
  TORCH_CHECK(x2.is_cuda(), "the gated norm runs on CUDA tensors only; there is no CPU path");
  TORCH_CHECK(x2.dim() == 2 && x2.stride(1) == 1, "issm_b200: norm input must be (rows, hidden) with a unit inner stride");
  p.rows = (int32_t)x2.size(0); p.hidden = (int32_t)x2.size(1);
  p.group_size = (int32_t)(group_size > 0 ? group_size : x2.size(1));
  TORCH_CHECK(p.hidden % p.group_size == 0, "issm_b200: group_size must divide the hidden size");
  p.io_dtype = dtype_code(x2.scalar_type());
  p.is_rms = is_rms; p.norm_before_gate = norm_before_gate;
  p.has_z = z2.has_value(); p.has_bias = bias.has_value();
  p.eps = (float)eps;
  p.x = x2.data_ptr(); p.x_sr = x2.stride(0);
  if (z2) {
    TORCH_CHECK(z2->sizes() == x2.sizes() && z2->scalar_type() == x2.scalar_type() && z2->stride(1) == 1, "issm_b200: z must match x");
    p.z = z2->data_ptr(); p.z_sr = z2->stride(0);
  }
  TORCH_CHECK(weight.scalar_type() == at::kFloat && weight.is_contiguous() && weight.numel() == p.hidden, "issm_b200: weight must be float32 (hidden)");
  p.weight = weight.data_ptr<float>();
  if (bias) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous() && bias->numel() == p.hidden, "issm_b200: bias must be float32 (hidden)");
    p.bias = bias->data_ptr<float>();
  }
}

// (y, rstd, mean); mean is a 0-element tensor for RMS norm.  Counterpart of _layer_norm_fwd (layernorm_gated.py:98-137).
std::tuple<Tensor, Tensor, Tensor> norm_fwd(const Tensor& x2, const OptTensor& z2, const Tensor& weight, const OptTensor& bias, double eps,
                                            int64_t group_size, bool norm_before_gate, bool is_rms) {
  const c10::cuda::CUDAGuard guard(x2.device());
  issm_norm_params p{};
  fill_norm(p, x2, z2, weight, bias, eps, group_size, norm_before_gate, is_rms);
  const int64_t ng = p.hidden / p.group_size;
  Tensor y = at::empty(x2.sizes(), x2.options());
  Tensor rstd = at::empty({p.rows * ng}, x2.options().dtype(at::kFloat));
  Tensor mean = is_rms ? at::empty({0}, rstd.options()) : at::empty({p.rows * ng}, rstd.options());
  p.y = y.data_ptr(); p.y_sr = y.stride(0);
  p.rstd = rstd.data_ptr<float>();
  p.mean = is_rms ? nullptr : mean.data_ptr<float>();
  check_rc(issm_b200_norm_fwd(&p, stream_of(x2)), "issm_b200_norm_fwd");
  return {y, rstd, mean};
}

// (dx, dz, dweight, dbias); absent ones are 0-element tensors.  Counterpart of _layer_norm_bwd (layernorm_gated.py:261-325).
std::tuple<Tensor, Tensor, Tensor, Tensor> norm_bwd(const Tensor& dy2, const Tensor& x2, const OptTensor& z2, const Tensor& weight,
                                                    const OptTensor& bias, const Tensor& rstd, const OptTensor& mean, double eps,
                                                    int64_t group_size, bool norm_before_gate, bool is_rms) {
  const c10::cuda::CUDAGuard guard(x2.device());
  issm_norm_params p{};
  fill_norm(p, x2, z2, weight, bias, eps, group_size, norm_before_gate, is_rms);
  TORCH_CHECK(dy2.sizes() == x2.sizes() && dy2.scalar_type() == x2.scalar_type() && dy2.stride(1) == 1, "issm_b200: dy must match x");
  Tensor dx = at::empty(x2.sizes(), x2.options());
  Tensor dz = z2 ? at::empty(x2.sizes(), x2.options()) : at::empty({0}, x2.options());
  Tensor dw = at::empty({p.hidden}, x2.options().dtype(at::kFloat));
  Tensor db = bias ? at::empty({p.hidden}, dw.options()) : at::empty({0}, dw.options());
  p.rstd = rstd.data_ptr<float>();
  p.mean = (mean && mean->numel() > 0) ? mean->data_ptr<float>() : nullptr;
  p.dy = dy2.data_ptr(); p.dy_sr = dy2.stride(0);
  p.dx = dx.data_ptr(); p.dz = z2 ? dz.data_ptr() : nullptr;
  p.dweight = dw.data_ptr<float>(); p.dbias = bias ? db.data_ptr<float>() : nullptr;
  const size_t need = issm_b200_norm_workspace_bytes(&p, 1);
  Tensor ws = at::empty({(int64_t)std::max<size_t>(need, 256)}, x2.options().dtype(at::kByte));
  p.workspace = ws.data_ptr(); p.workspace_bytes = (size_t)ws.numel();
  check_rc(issm_b200_norm_bwd(&p, stream_of(x2)), "issm_b200_norm_bwd");
  return {dx, dz, dw, db};
}

}  // namespace

TORCH_LIBRARY(issm_b200, m) {
  m.def("fwd(Tensor x, Tensor dt, Tensor A, Tensor B, Tensor C, int chunk_size, Tensor? D, Tensor? z, Tensor? dt_bias, "
        "Tensor? initial_states, bool dt_softplus, float dt_min, float dt_max, bool reverse, int path, bool want_final, "
        "bool save_states, Tensor status) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("bwd(Tensor dout, Tensor x, Tensor dt, Tensor A, Tensor B, Tensor C, Tensor? out_x, int chunk_size, Tensor? D, Tensor? z, "
        "Tensor? dt_bias, Tensor? initial_states, Tensor? dfinal_states, bool dt_softplus, float dt_min, float dt_max, bool reverse, "
        "int path, Tensor? saved_states, Tensor status) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("norm_fwd(Tensor x, Tensor? z, Tensor weight, Tensor? bias, float eps, int group_size, bool norm_before_gate, bool is_rms) "
        "-> (Tensor, Tensor, Tensor)");
  m.def("norm_bwd(Tensor dy, Tensor x, Tensor? z, Tensor weight, Tensor? bias, Tensor rstd, Tensor? mean, float eps, int group_size, "
        "bool norm_before_gate, bool is_rms) -> (Tensor, Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(issm_b200, CUDA, m) {
  m.impl("fwd", &fwd);
  m.impl("bwd", &bwd);
  m.impl("norm_fwd", &norm_fwd);
  m.impl("norm_bwd", &norm_bwd);
}
