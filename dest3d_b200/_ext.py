"""Loader of the torch C++ extension (`libissm_b200_torch.so`, TORCH_LIBRARY namespace `issm_b200`): ops
`fwd`, `bwd`, `norm_fwd`, `norm_bwd` over the C ABI.  Like the C-ABI library itself it has to be built first;
there is no fallback."""
import os

import torch

from . import _lib

_EXT_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libissm_b200_torch.so")
_loaded = False


def ops():
    """torch.ops.issm_b200 (loads the extension on first use; raises when it has not been built)."""
    global _loaded
    if not _loaded:
        _lib.lib()                                            # same loud failure when the kernels are missing
        if not os.path.exists(_EXT_PATH):
            raise RuntimeError(f"{_EXT_PATH} is missing: the torch extension has not been built. "
                               "Run `python -m dest3d_b200.build`; there is no CPU or PyTorch fallback.")
        torch.ops.load_library(_EXT_PATH)
        _loaded = True
    return torch.ops.issm_b200


def opt(t):
    """0-element placeholder of an absent result -> None."""
    return t if t.numel() > 0 else None
