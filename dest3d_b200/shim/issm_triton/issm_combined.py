"""`issm_triton.issm_combined` of the reference (issm_triton/issm_combined.py:16-54), served by dest3d_b200."""
from dest3d_b200.issm_combined import ISSM_chunk_scan_combined, ISSMChunkScanCombinedFn  # noqa: F401
