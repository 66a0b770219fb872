"""`issm_triton.layernorm_gated` of the reference (issm_triton/layernorm_gated.py:328-427), served by dest3d_b200."""
from dest3d_b200.layernorm_gated import LayerNorm, LayerNormFn, RMSNorm, layernorm_fn, rmsnorm_fn  # noqa: F401
