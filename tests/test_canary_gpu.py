"""Out-of-bounds evidence without a memory checker: every output, the saved block-entry states and the
workspace of a call are carved out of a larger buffer whose margins hold a known bit pattern, the payload is
pre-filled with NaN, and after the call the margins must be untouched and every output finite and equal to the
oracle's.  Run on the shapes where a predicated tail store or a vector store could overrun: L % 64 != 0,
L < 64, L = 1, head dim 36 padded to 48 inside the kernels, both scan directions, both kernel families."""
import pytest
import torch

from oracle import issm_oracle as O
from tests import parity

pytestmark = pytest.mark.gpu
OPTS = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1))
GUARD_BYTES = 4096
PATTERN = 0x5A


class GuardedAllocator:
    """Stand-in for dest3d_b200.issm_combined._empty: buffer = [guard | payload | guard]."""

    def __init__(self):
        self.raw = []

    def __call__(self, shape, dtype, device):
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        pay = (nbytes + 255) // 256 * 256                    # keeps the payload and the far guard 256-byte aligned
        raw = torch.full((GUARD_BYTES + pay + GUARD_BYTES,), PATTERN, dtype=torch.uint8, device=device)
        body = raw[GUARD_BYTES:GUARD_BYTES + nbytes]
        if dtype == torch.uint8:
            body.fill_(0xFF)
        else:
            body.view(dtype).fill_(float("nan"))
        self.raw.append((raw, nbytes, tuple(shape), dtype))
        return body.view(dtype).view(tuple(shape))

    def check(self):
        torch.cuda.synchronize()
        assert self.raw, "the allocator hook was never used"
        for raw, nbytes, shape, dtype in self.raw:
            lo = raw[:GUARD_BYTES]
            hi = raw[GUARD_BYTES + nbytes:]
            assert bool((lo == PATTERN).all()), f"write below a {dtype} buffer of shape {shape}"
            assert bool((hi == PATTERN).all()), f"write beyond a {dtype} buffer of shape {shape}"


CASES = [
    ("tail_37_of_64", (1, 165, 2, 36, 256, 1, 256)),
    ("short_L_lt_64", (2, 23, 2, 36, 256, 1, 64)),
    ("single_point", (1, 1, 2, 36, 128, 1, 64)),
    ("exact_blocks", (1, 128, 2, 36, 256, 1, 128)),
    ("headdim_40", (1, 70, 2, 40, 128, 1, 64)),
    ("two_state_slices", (1, 101, 2, 36, 512, 1, 64)),
]


@pytest.mark.parametrize("reverse", [False, True], ids=["forward_scan", "reversed_scan"])
@pytest.mark.parametrize("path", ["tensor", "simt"])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_guard_bands_survive(monkeypatch, case, path, reverse):
    from dest3d_b200 import issm_combined
    b, L, H, P, N, G, Q = case[1]
    inp = O.make_inputs(b, L, H, P, N, G=G, seed=3 + L, dtype=torch.bfloat16)
    opts = dict(OPTS, reverse=reverse)
    ref = parity.oracle_run(inp, Q, opts)
    alloc = GuardedAllocator()
    monkeypatch.setattr(issm_combined, "_empty", alloc)
    monkeypatch.setattr(issm_combined, "BINDING", "ctypes")    # the binding whose buffers come from _empty
    got = parity.cuda_run(inp, Q, opts, path=path)
    alloc.check()
    parity.compare(got, ref, torch.bfloat16)                   # also asserts that every output element was written (finite)
