// tcgen05 tensor-core path of the ISSM scan (placeholder until the kernels land).
#include "issm_common.cuh"
namespace issm {
bool tensor_path_supported(const issm_params&) { return false; }
size_t tensor_workspace_bytes(const issm_params&, int) { return 0; }
int tensor_fwd(const issm_params&, cudaStream_t) { return ISSM_ERR_UNSUPPORTED; }
int tensor_bwd(const issm_params&, cudaStream_t) { return ISSM_ERR_UNSUPPORTED; }
}  // namespace issm
