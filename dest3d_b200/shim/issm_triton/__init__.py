"""Import shim: a package named like the reference's `issm_triton` whose two modules forward to the B200
library.  Put the directory that holds this package (`dest3d_b200/shim`) on `sys.path` AHEAD of the reference
checkout and the reference's own call sites (`models/dest_module.py:12-13`) import the B200 operators without
any edit:

    from issm_triton.issm_combined import ISSM_chunk_scan_combined
    from issm_triton.layernorm_gated import RMSNorm as RMSNormGated
"""
