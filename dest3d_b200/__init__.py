"""B200-native ISSM chunked scan (the hot path of the DEST 3D detector) behind the reference's
Python interface.  Importing the operators requires the built CUDA library; there is no fallback."""
from .issm_combined import (ISSM_chunk_scan_combined, ISSMChunkScanCombinedFn, issm_bidirectional_scan,  # noqa: F401
                            issm_bwd, issm_fwd, raise_on_device_error)
from .layernorm_gated import LayerNorm, LayerNormFn, RMSNorm, layernorm_fn, rmsnorm_fn  # noqa: F401
from .pointops import PointLiteConv, reorder_points  # noqa: F401
