"""The allocation-free backward entry point against the ordinary one.

Some programs that embed this library give all device memory to their own planner when they
start and may not allocate afterwards; b200_attention_bwd_noalloc lets them run the backward
with the `delta` scratch held in a fixed array inside the library instead of memory they would
have to allocate.  The test calls it through the C ABI twice in a row, with different inputs, and
requires the gradients to equal those of b200_attention_bwd (same kernels, deterministic, so the
comparison is exact) - the second call also shows that what the first call left in the shared
array does no harm.  It sits in a file that pytest collects last so that a failure here cannot
hide the other tests in a run that stops at the first failure.
"""
import pytest
import torch

from triton_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _inputs(seed, Z, H, N, D, dtype):
    g = torch.Generator().manual_seed(seed)
    mk = lambda std: (torch.randn(Z, H, N, D, generator=g) * std).to(dtype).cuda()
    return mk(0.5), mk(0.5), mk(0.5), mk(1.0)


def _noalloc_backward(q, k, v, o, M, do, causal, sm_scale):
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)  # the caller's outputs
    Z, H, N, D = q.shape
    s4 = _lib.strides4
    code = _lib.lib().b200_attention_bwd_noalloc(
        torch.cuda.current_stream().cuda_stream, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
        do.data_ptr(), M.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), Z, H, N, D,
        s4(q), s4(k), s4(v), s4(o), s4(do), s4(dq), s4(dk), s4(dv), float(sm_scale), 1 if causal else 0,
        ops._DT[q.dtype])
    _lib.check(code, "attention_bwd_noalloc")
    return dq, dk, dv


def test_noalloc_backward_matches_twice_in_a_row():
    for seed, shape, dtype, causal in ((1, (2, 3, 512, 64), torch.bfloat16, True),
                                       (2, (1, 2, 256, 128), torch.float16, False)):
        q, k, v, do = _inputs(seed, *shape, dtype)
        o, M = ops.attention_forward(q, k, v, causal, 0.5)
        want = ops.attention_backward(q, k, v, o, M, do, causal, 0.5)
        got = _noalloc_backward(q, k, v, o, M, do, causal, 0.5)
        torch.cuda.synchronize()
        for g, w, name in zip(got, want, ("dq", "dk", "dv")):
            assert torch.equal(g, w), f"{name} differs from the caller-scratch entry point (seed {seed})"
    assert _lib.status() == 0


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    cap = _lib.lib().b200_attention_bwd_noalloc_capacity()
    assert cap == 1 << 20
    # Z*H*N = 2^21 rows: refused before anything is launched or dereferenced
    s4 = (_lib._s4)(1, 1, 64, 1)
    code = _lib.lib().b200_attention_bwd_noalloc(None, *([256] * 9), 2, 8, 1 << 17, 64, *([s4] * 8), 0.5, 1, 0)
    assert code == 2
    assert "built-in scratch" in _lib.last_error()
