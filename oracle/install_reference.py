"""Places an UNMODIFIED copy of a reference checkout under `baseline/_ref/` (git-ignored: it never enters this
repository's history, but it travels with the working tree to the machine that runs the GPU tests and the
benchmark, which has no other copy of the reference).  TEST / BENCHMARK INFRASTRUCTURE ONLY: the product
package never reads it.

    python oracle/install_reference.py <path-to-the-reference-checkout>

Used by: the drop-in test (the reference's own `MultiHeadISSMScan` driven through the import shim), the
`cpu_baseline` leg and the reference arm of `bench.py` (the reference's pure-PyTorch `ISSM_minimal_discrete`,
test_issm.py:18-67, timed on the host cores).  The reference has no installable Python package at its root
(no setup.py / pyproject.toml; only the PointNet++ CUDA extension has one), so "installing" it is a plain copy
of its Python sources; figures and the PointNet++ extension are left out.
"""
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref")
KEEP = ("issm_triton", "models", "utils", "test_issm.py", "LICENSE")


def install(src):
    src = os.path.abspath(src)
    if not os.path.isfile(os.path.join(src, "test_issm.py")):
        raise SystemExit(f"{src} does not look like a checkout of the reference (test_issm.py missing)")
    os.makedirs(DEST, exist_ok=True)
    for name in KEEP:
        s, d = os.path.join(src, name), os.path.join(DEST, name)
        if os.path.isdir(s):
            shutil.copytree(s, d, dirs_exist_ok=True, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
        elif os.path.isfile(s):
            shutil.copy2(s, d)
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(install(sys.argv[1]))
