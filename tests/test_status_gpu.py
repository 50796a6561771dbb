"""A bounded device-side wait that runs out must be visible to the caller, not hand back garbage.

The kernels never wait without a limit: a wait that runs out records where it gave up in the
device status word, the kernel finishes normally, and the failure code is mirrored into pinned
host memory.  From then on the library refuses to launch (B200_ERR_KERNEL) until the word is
cleared.  The failure here is produced in the allowed way: `b200_selftest_wait_timeout` launches a
small kernel whose barrier nothing ever arrives on, with a limit of a few milliseconds.  Nothing
traps, faults or waits without a limit."""
import time

import numpy as np
import pytest
import torch

import triton_b200
from triton_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"
SITE_SELFTEST = 99


def test_a_wait_that_runs_out_is_reported_and_clears():
    g = torch.Generator().manual_seed(3)
    a = torch.randn(256, 320, generator=g).half().to(DEV)
    b = torch.randn(320, 192, generator=g).half().to(DEV)
    want = triton_b200.matmul(a, b)
    assert _lib.status() == 0
    L = _lib.lib()
    try:
        t0 = time.time()
        _lib.check(L.b200_selftest_wait_timeout(torch.cuda.current_stream().cuda_stream, 3000), "selftest")
        torch.cuda.synchronize()  # the kernel returns by itself: TMEM freed, context intact
        assert time.time() - t0 < 5.0
        # every launching entry point now refuses, with the failure site in the message, and launches nothing
        with pytest.raises(RuntimeError, match=r"code 5.*site 99"):
            triton_b200.matmul(a, b)
        q = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device=DEV)
        with pytest.raises(RuntimeError, match="code 5"):
            triton_b200.attention_forward(q, q, q, True, 0.5)
        v = _lib.status(clear=False)
        assert v & 0xFF == SITE_SELFTEST and (v >> 16) == 0, hex(v)
        assert _lib.status(clear=True) == v
    finally:
        _lib.status(clear=True)
    # cleared: the same call works again and gives the same bits; the CUDA context was never lost
    assert _lib.status() == 0
    got = triton_b200.matmul(a, b)
    assert torch.equal(got, want)
    np.testing.assert_allclose(got.float().cpu().numpy(), a.float().cpu().numpy() @ b.float().cpu().numpy(),
                               rtol=1e-2, atol=1e-2)
    q = (torch.randn(1, 2, 256, 64, generator=g) * 0.5).half().to(DEV)
    o, M = triton_b200.attention_forward(q, q, q, True, 0.5)
    assert torch.isfinite(o).all() and _lib.status() == 0


def test_selftest_argument_range():
    L = _lib.lib()
    assert L.b200_selftest_wait_timeout(None, 0) == _lib.ERR_ARG
    assert L.b200_selftest_wait_timeout(None, 10 ** 6) == _lib.ERR_ARG
    assert _lib.status() == 0
