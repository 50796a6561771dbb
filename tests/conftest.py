import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


# The suite asserts the library's defaults, among them that the default backward is bitwise
# repeatable: settings of the caller's shell that change a default (the opt-in one-pass backward, a
# forced tile shape) are not carried into the tests.
for _var in ("B200_ATTN_BWD_ONEPASS", "B200_GEMM_TILE", "B200_GEMM_PAIR_STAGES", "B200_GEMM_PLAIN"):
    os.environ.pop(_var, None)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    d = os.path.join(ROOT, "tests", "golden")
    out = {}
    for name in ("matmul", "fp8", "epilogue", "attn", "attn_old"):
        with np.load(os.path.join(d, name + ".npz")) as z:
            for k in z.files:
                out[k] = z[k]
    return out
