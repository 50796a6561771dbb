"""Parity of the CUDA flash attention (through the C ABI) with the CPU oracle and the
interpreter-generated golden fixtures; edge cases; full-size checks of configs 4 and 5 on
sampled heads.  Tolerance: rtol = atol = 1e-2 (python/tutorials/06-fused-attention.py:551-559
uses atol 1e-2); bf16 gradients get 2e-2 absolute because one bf16 ulp at |x| ~ 4 is 3e-2."""
import math

import numpy as np
import pytest
import torch

import cases
import triton_b200
from oracle import ref_ops as R
from triton_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def f32(t):
    return t.detach().float().cpu().numpy()


def status_ok():
    assert _lib.status() == 0, "a bounded device-side wait ran out"


def run_gpu(q, k, v, do, causal, sm_scale, bwd):
    qd, kd, vd = (t.to(DEV).requires_grad_(bwd) for t in (q, k, v))
    o, M = triton_b200.attention_forward(qd.detach(), kd.detach(), vd.detach(), causal, sm_scale)
    out = dict(o=f32(o), m=f32(M))
    if bwd:
        o2 = triton_b200.attention(qd, kd, vd, causal, sm_scale)
        o2.backward(do.to(DEV))
        assert torch.equal(o2.detach(), o)
        out.update(dq=f32(qd.grad), dk=f32(kd.grad), dv=f32(vd.grad))
    status_ok()
    return out


@pytest.mark.parametrize("name", list(cases.ATTN_CASES))
def test_attention_parity_with_oracle(golden, name):
    c = cases.ATTN_CASES[name]
    q, k, v, do = cases.attn_inputs(c)
    got = run_gpu(q, k, v, do, c["causal"], c["sm_scale"], c.get("bwd", False))
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), c["causal"], c["sm_scale"], c["dtype"])
    np.testing.assert_allclose(got["o"], o, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(got["m"], M, rtol=1e-4, atol=1e-3)
    if c["dtype"] == "fp16":
        np.testing.assert_allclose(got["o"], golden[f"attn.{name}.o"].astype(np.float32), rtol=1e-2, atol=1e-2)
        np.testing.assert_allclose(got["m"], golden[f"attn.{name}.m"], rtol=1e-4, atol=1e-3)
    if c.get("bwd"):
        dq, dk, dv = R.attention_bwd(f32(q), f32(k), f32(v), o, f32(do), M, c["sm_scale"], c["dtype"])
        tol = 1e-2 if c["dtype"] == "fp16" else 2e-2
        for key, want in (("dq", dq), ("dk", dk), ("dv", dv)):
            np.testing.assert_allclose(got[key], want, rtol=1e-2, atol=tol, err_msg=key)
            if c["dtype"] == "fp16":
                np.testing.assert_allclose(got[key], golden[f"attn.{name}.{key}"].astype(np.float32), rtol=1e-2,
                                           atol=1e-2, err_msg="golden " + key)


@pytest.mark.parametrize("name", [n for n, c in cases.ATTN_CASES.items() if c.get("old_style")])
def test_old_style_attention_against_its_interpreter_fixture(golden, name):
    """The reference's older flash attention, `attention(q, k, v, sm_scale)` (always causal;
    python/test/unit/hopper/test_flashattention.py:294-358): output and the three gradients against the
    fixture its own kernels produced under the interpreter, at that test's tolerance (atol 1e-2, :399-403),
    and the two statistics tensors it keeps - row sum L and row maximum M (:128-131)."""
    c = cases.ATTN_CASES[name]
    q, k, v, do = cases.attn_inputs(c)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    o = triton_b200.attention_old(qd, kd, vd, c["sm_scale"])
    o.backward(do.to(DEV))
    status_ok()
    np.testing.assert_allclose(f32(o), golden[f"attn_old.{name}.o"].astype(np.float32), atol=1e-2, rtol=0)
    for got, key in ((qd.grad, "dq"), (kd.grad, "dk"), (vd.grad, "dv")):
        np.testing.assert_allclose(f32(got), golden[f"attn_old.{name}.{key}"].astype(np.float32), atol=1e-2, rtol=0,
                                   err_msg=key)
    o2, L, M = triton_b200.attention_old_forward(qd.detach(), kd.detach(), vd.detach(), c["sm_scale"])
    assert torch.equal(o2, o.detach()) and L.shape == (c["Z"] * c["H"], c["N"]) and M.shape == L.shape
    np.testing.assert_allclose(f32(M), golden[f"attn_old.{name}.m"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(f32(L), golden[f"attn_old.{name}.l"], rtol=1e-3, atol=1e-4)
    with pytest.raises(AssertionError):
        big = torch.zeros(1, 1, 128, 256, dtype=torch.float16, device=DEV)
        triton_b200.attention_old(big, big, big, 0.5)  # the older wrapper's head dims end at 128 (:303)


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("N", [128, 200, 384, 1000])
@pytest.mark.parametrize("causal", [True, False])
def test_forward_ragged_lengths(dtype, D, N, causal):
    c = dict(Z=1, H=2, N=N, D=D, dtype=dtype, seed=N + D)
    q, k, v, _ = cases.attn_inputs(c)
    got = run_gpu(q, k, v, None, causal, D ** -0.5, False)
    # the oracle walks 128-row blocks like the reference; pad the ragged tail with masked keys
    pad = (-N) % 128
    if pad:
        qp, kp, vp = (torch.cat([t, torch.zeros(1, 2, pad, D, dtype=t.dtype)], 2) for t in (q, k, v))
        if causal:
            o, M = R.attention_fwd(f32(qp), f32(kp), f32(vp), True, D ** -0.5, dtype)
            o, M = o[:, :, :N], M[:, :, :N]
        else:  # full attention over exactly N keys: dense fp32 softmax with P rounded to the storage type
            s = (q.float() @ k.float().transpose(2, 3)) * D ** -0.5
            M = (torch.logsumexp(s, -1) / math.log(2.0)).numpy()
            p = torch.softmax(s, -1)
            o = (p @ v.float()).numpy()
    else:
        o, M = R.attention_fwd(f32(q), f32(k), f32(v), causal, D ** -0.5, dtype)
    np.testing.assert_allclose(got["o"], o, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(got["m"], M, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("where", ["first_half", "second_half", "growing", "one_row"])
def test_forward_scores_far_above_the_first_block(dtype, D, causal, where):
    """The 16-bit forward rescales its accumulator lazily: the running maximum of a row is followed
    exactly, but O and l are only multiplied through when it has grown by more than 2^8 since the
    last rescale.  These inputs make scores jump far above everything seen before - in the first
    half of a block, in the second half (after the P V MMAs on the first half were issued), in
    every block, and for a single row of a warp - so both the rescale and the no-rescale branch
    run with large factors."""
    N = 768
    c = dict(Z=1, H=2, N=N, D=D, dtype=dtype, seed=7 * D + len(where))
    q, k, v, _ = cases.attn_inputs(c)
    k = k.float()
    if where == "first_half":
        k[:, :, 256 + 5] *= 40.0
        k[:, :, 640 + 17] *= 90.0
    elif where == "second_half":
        k[:, :, 256 + 64 + 9] *= 40.0
        k[:, :, 512 + 127] *= 90.0
    elif where == "growing":
        k *= (1.0 + torch.arange(N).float() / 16.0)[None, None, :, None]
    else:
        q = q.float()
        q[:, :, 700] *= 30.0
        k[:, :, 300:] *= 4.0
        q = q.to(v.dtype)
    k = k.to(v.dtype)
    sm_scale = 0.5
    got = run_gpu(q, k, v, None, causal, sm_scale, False)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), causal, sm_scale, dtype)
    np.testing.assert_allclose(got["o"], o, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(got["m"], M, rtol=1e-4, atol=1e-3)
    assert np.isfinite(got["o"]).all() and np.isfinite(got["m"]).all()


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(1, 2, 256), (2, 3, 1024), (1, 1, 128)])
def test_one_pass_backward(dtype, causal, shape):
    """The head-dim-64 backward in one pass (partial dQ per K/V block added into an fp32 buffer, the
    layout of the reference's `sequence_parallel` mode, test_performance.py:174, 194) against the
    oracle at the backward's tolerances, and against the two-kernel path: dK and dV are the same
    arithmetic in the same order and must be the same bits; dQ is a sum of the same partial products
    in another order (fp32), so it may differ by a rounding of the storage type."""
    Z, H, N = shape
    c = dict(Z=Z, H=H, N=N, D=64, dtype=dtype, seed=6400 + N + causal)
    q, k, v, do = cases.attn_inputs(c)
    sm_scale = 0.5
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    o, M = triton_b200.attention_forward(qd, kd, vd, causal, sm_scale)
    two = triton_b200.attention_backward(qd, kd, vd, o, M, dod, causal, sm_scale, one_pass=False)
    one = triton_b200.attention_backward(qd, kd, vd, o, M, dod, causal, sm_scale, one_pass=True)
    status_ok()
    assert torch.equal(one[1], two[1]) and torch.equal(one[2], two[2]), "dK / dV differ from the two-kernel path"
    tol = 1e-2 if dtype == "fp16" else 2e-2
    np.testing.assert_allclose(f32(one[0]), f32(two[0]), rtol=1e-2, atol=tol)
    ro, rM = R.attention_fwd(f32(q), f32(k), f32(v), causal, sm_scale, dtype)
    if causal:
        want = R.attention_bwd(f32(q), f32(k), f32(v), ro, f32(do), rM, sm_scale, dtype)
    else:
        want = R.attention_bwd_full(f32(q), f32(k), f32(v), ro, f32(do), rM, sm_scale, False, dtype)
    for got, ref, name in zip(one, want, ("dq", "dk", "dv")):
        np.testing.assert_allclose(f32(got), ref, rtol=1e-2, atol=tol, err_msg=name)
    # through autograd with the reference's six-argument signature; twice, on a buffer that is not
    # cleared by the caller: the call clears its own accumulator
    qg, kg, vg = (t.clone().requires_grad_() for t in (qd, kd, vd))
    triton_b200.attention(qg, kg, vg, causal, sm_scale, True).backward(dod)
    assert torch.equal(kg.grad, two[1]) and torch.equal(vg.grad, two[2])
    np.testing.assert_allclose(f32(qg.grad), f32(two[0]), rtol=1e-2, atol=tol)


def test_one_pass_backward_head_dims_and_errors():
    """Other head dims take the two-kernel path whatever the flag says; the C entry point itself refuses them."""
    g = torch.Generator().manual_seed(9)
    q, k, v, do = ((torch.randn(1, 2, 256, 128, generator=g) * 0.5).half().to(DEV) for _ in range(4))
    o, M = triton_b200.attention_forward(q, k, v, True, 0.09)
    a = triton_b200.attention_backward(q, k, v, o, M, do, True, 0.09, one_pass=True)
    b = triton_b200.attention_backward(q, k, v, o, M, do, True, 0.09, one_pass=False)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    s4 = _lib.strides4
    code = _lib.lib().b200_attention_bwd_onepass(None, *([q.data_ptr()] * 5), M.data_ptr(), M.data_ptr(), M.data_ptr(),
                                                 *([q.data_ptr()] * 3), 1, 2, 256, 128, *([s4(q)] * 8), 0.09, 1, _lib.F16)
    assert code == _lib.ERR_UNSUPPORTED and "head dim 64" in _lib.last_error()
    assert _lib.lib().b200_attention_bwd_onepass_workspace(4, 48, 1024, 64) == 4 * 48 * 1024 * 64 * 4
    status_ok()


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
def test_backward_noncausal(dtype, D):
    c = dict(Z=2, H=2, N=384, D=D, dtype=dtype, seed=77 + D)
    q, k, v, do = cases.attn_inputs(c)
    got = run_gpu(q, k, v, do, False, 0.5, True)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), False, 0.5, dtype)
    dq, dk, dv = R.attention_bwd_full(f32(q), f32(k), f32(v), o, f32(do), M, 0.5, False, dtype)
    tol = 1e-2 if dtype == "fp16" else 2e-2
    for key, want in (("dq", dq), ("dk", dk), ("dv", dv)):
        np.testing.assert_allclose(got[key], want, rtol=1e-2, atol=tol, err_msg=key)


def test_strided_inputs_and_errors():
    # q, k, v as slices of one packed [Z, N, 3, H, D] buffer (strided, head dim contiguous)
    Z, H, N, D = 2, 3, 256, 64
    g = torch.Generator().manual_seed(3)
    packed = (torch.randn(Z, N, 3, H, D, generator=g) * 0.5).half().to(DEV)
    q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o, M = triton_b200.attention_forward(q, k, v, True, 0.125)
    oc, Mc = triton_b200.attention_forward(q.contiguous(), k.contiguous(), v.contiguous(), True, 0.125)
    assert torch.equal(o, oc) and torch.equal(M, Mc)
    with pytest.raises(RuntimeError, match="head dim 256"):  # the plain backward entry point names the one that takes scratch
        x = torch.zeros(1, 1, 128, 256, dtype=torch.float16, device=DEV)
        m = torch.zeros(1, 1, 128, dtype=torch.float32, device=DEV)
        s4 = _lib.strides4
        _lib.check(_lib.lib().b200_attention_bwd(
            None, *([x.data_ptr()] * 5), m.data_ptr(), m.data_ptr(), *([x.data_ptr()] * 3), 1, 1, 128, 256,
            *([s4(x)] * 8), 0.5, 1, _lib.F16), "attention_bwd")
    status_ok()


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("causal", [True, False])
def test_head_dim_256_forward_and_backward(dtype, causal):
    """Head dim 256, the largest of the reference's set (06-fused-attention.py:447): the forward runs one
    128-row tile per work item (the accumulator alone takes half of TMEM); the backward is laid out as
    matmuls with [N, N] scratch.  Both against the oracle, same tolerances as the other head dims."""
    c = dict(Z=2, H=2, N=384, D=256, dtype=dtype, seed=2560 + causal)
    q, k, v, do = cases.attn_inputs(c)
    sm_scale = 256 ** -0.5
    got = run_gpu(q, k, v, do, causal, sm_scale, True)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), causal, sm_scale, dtype)
    np.testing.assert_allclose(got["o"], o, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(got["m"], M, rtol=1e-4, atol=1e-3)
    if causal:
        dq, dk, dv = R.attention_bwd(f32(q), f32(k), f32(v), o, f32(do), M, sm_scale, dtype)
    else:
        dq, dk, dv = R.attention_bwd_full(f32(q), f32(k), f32(v), o, f32(do), M, sm_scale, False, dtype)
    tol = 1e-2 if dtype == "fp16" else 2e-2
    for key, want in (("dq", dq), ("dk", dk), ("dv", dv)):
        np.testing.assert_allclose(got[key], want, rtol=1e-2, atol=tol, err_msg=key)


@pytest.mark.parametrize("pad", [4, 8])
def test_outputs_tma_cannot_address(pad):
    """O, dQ, dK, dV whose row pitch is not a multiple of 16 bytes (pad = 4 elements) cannot be
    written by TMA stores: the kernels fall back to direct stores and give the same bits as the
    TMA path; pad = 8 keeps the TMA path on a padded layout."""
    from triton_b200.ops import _DT, _stream
    Z, H, N, D = 1, 2, 256, 64
    g = torch.Generator().manual_seed(11 + pad)
    q, k, v, do = ((torch.randn(Z, H, N, D, generator=g) * 0.5).to(torch.bfloat16).to(DEV) for _ in range(4))
    o_ref, M_ref = triton_b200.attention_forward(q, k, v, True, 0.125)
    dq_ref, dk_ref, dv_ref = triton_b200.attention_backward(q, k, v, o_ref, M_ref, do, True, 0.125)

    def padded():
        buf = torch.zeros(Z, H, N, D + pad, dtype=torch.bfloat16, device=DEV)
        return buf, buf[..., :D]
    (ob, o), (dqb, dq), (dkb, dk), (dvb, dv) = padded(), padded(), padded(), padded()
    M = torch.empty(Z, H, N, device=DEV, dtype=torch.float32)
    delta = torch.empty_like(M)
    L = _lib.lib()
    _lib.check(L.b200_attention_fwd(_stream(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), M.data_ptr(),
                                    Z, H, N, D, _lib.strides4(q), _lib.strides4(k), _lib.strides4(v), _lib.strides4(o),
                                    0.125, 1, _DT[q.dtype]), "fwd")
    assert torch.equal(o, o_ref) and torch.equal(M, M_ref)
    assert float(ob[..., D:].abs().max()) == 0.0, "the padding was written"
    _lib.check(L.b200_attention_bwd(_stream(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), o_ref.data_ptr(),
                                    do.data_ptr(), M.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                    dv.data_ptr(), Z, H, N, D, _lib.strides4(q), _lib.strides4(k), _lib.strides4(v),
                                    _lib.strides4(o_ref), _lib.strides4(do), _lib.strides4(dq), _lib.strides4(dk),
                                    _lib.strides4(dv), 0.125, 1, _DT[q.dtype]), "bwd")
    assert torch.equal(dq, dq_ref) and torch.equal(dk, dk_ref) and torch.equal(dv, dv_ref)
    for b in (dqb, dkb, dvb):
        assert float(b[..., D:].abs().max()) == 0.0, "the padding was written"
    status_ok()


def _check_heads(q, k, v, do, got, heads, causal, sm_scale, dtype, bwd):
    for (z, h) in heads:
        sl = (slice(z, z + 1), slice(h, h + 1))
        qq, kk, vv = (f32(t[sl]) for t in (q, k, v))
        o, M = R.attention_fwd(qq, kk, vv, causal, sm_scale, dtype)
        np.testing.assert_allclose(got["o"][sl], o, rtol=1e-2, atol=1e-2)
        np.testing.assert_allclose(got["m"][sl], M, rtol=1e-4, atol=1e-3)
        if bwd:
            dq, dk, dv = R.attention_bwd(qq, kk, vv, o, f32(do[sl]), M, sm_scale, dtype)
            for key, want in (("dq", dq), ("dk", dk), ("dv", dv)):
                np.testing.assert_allclose(got[key][sl], want, rtol=1e-2, atol=2e-2, err_msg=key)


def test_config4_full_size_forward():
    """Z4 H32 N4096 D128 fp16 causal: three sampled heads against the oracle, bitwise repeatability,
    and the row-stochastic property: with V = 1 every output element is 1."""
    c = dict(Z=4, H=32, N=4096, D=128, dtype="fp16", seed=20)
    q, k, v, _ = cases.attn_inputs(c)
    sm = 128 ** -0.5
    got = run_gpu(q, k, v, None, True, sm, False)
    _check_heads(q, k, v, None, got, [(0, 0), (2, 17), (3, 31)], True, sm, "fp16", False)
    qd, kd = q.to(DEV), k.to(DEV)
    o2, M2 = triton_b200.attention_forward(qd, kd, v.to(DEV), True, sm)
    assert np.array_equal(f32(o2), got["o"]) and np.array_equal(f32(M2), got["m"])
    ones, _ = triton_b200.attention_forward(qd, kd, torch.ones_like(qd), True, sm)
    np.testing.assert_allclose(f32(ones), 1.0, atol=2e-3)
    status_ok()


def test_config5_full_size_forward_backward():
    """Z4 H48 N1024 D64 bf16 causal forward + backward on sampled heads; dV of an all-ones dO
    equals the column sums of P (checked through sum over keys = number of queries)."""
    c = dict(Z=4, H=48, N=1024, D=64, dtype="bf16", seed=20)
    q, k, v, do = cases.attn_inputs(c)
    got = run_gpu(q, k, v, do, True, 0.5, True)
    _check_heads(q, k, v, do, got, [(0, 0), (1, 23), (3, 47)], True, 0.5, "bf16", True)
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    o, M = triton_b200.attention_forward(qd, kd, vd, True, 0.5)
    dq, dk, dv = triton_b200.attention_backward(qd, kd, vd, o, M, torch.ones_like(qd), True, 0.5)
    col = dv.float().sum(2)  # sum over keys of sum_q P[q, key] = N per (z, h, d)
    np.testing.assert_allclose(f32(col), 1024.0, rtol=2e-2)
    dq2, dk2, dv2 = triton_b200.attention_backward(qd, kd, vd, o, M, torch.ones_like(qd), True, 0.5)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    status_ok()


@pytest.mark.skipif(not hasattr(torch, "float8_e5m2"), reason="torch without float8_e5m2")
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("N,sm_scale,D", [(512, 0.0884, 128), (208, 0.0884, 128), (1024, 1.3, 128), (2048, 1.3, 128),
                                          (1024, 1.3, 64), (384, 0.125, 64), (208, 0.125, 64), (256, 0.18, 32)])
def test_forward_e5m2(causal, N, sm_scale, D):
    """The reference's 8-bit forward (06-fused-attention.py:66-69, 609-615): e5m2 q, k, v (v with
    the key dimension contiguous), P converted to e5m2, e5m2 output.  The reference has no test for
    it; the check is the oracle's restatement run with BLOCK_N = 128 (one of the reference's
    autotune choices; the 2-bit mantissa of P makes the result depend on the block-wise running
    maximum, i.e. on BLOCK_N): relative Frobenius error <= 2e-2, in fact all but a few elements in
    a million are bit-identical.  Both are also compared with exact fp64 attention.  Head dim 64 is
    the shape of the reference's own fp8 benchmark (:570) and has a kernel of its own (rows of 64
    bytes); head dim 32 runs on it with zero columns appended."""
    Z, H = 1, 2
    g = torch.Generator().manual_seed(N + int(causal) + D)
    q, k, v = ((torch.randn(Z, H, N, D, generator=g) * 0.5).to(torch.float8_e5m2) for _ in range(3))
    vd = v.to(DEV).permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)   # the reference's fp8 V layout
    o, M = triton_b200.attention_forward(q.to(DEV), k.to(DEV), vd, causal, sm_scale)
    status_ok()
    assert o.dtype == torch.float8_e5m2
    o2, M2 = triton_b200.attention_forward(q.to(DEV), k.to(DEV), v.to(DEV), causal, sm_scale)  # wrapper transposes
    assert torch.equal(o.view(torch.uint8), o2.view(torch.uint8)) and torch.equal(M, M2)
    qf, kf, vf = (f32(t) for t in (q, k, v))
    s = np.einsum("zhnd,zhmd->zhnm", qf.astype(np.float64), kf.astype(np.float64)) * sm_scale
    if causal:
        s = np.where(np.tril(np.ones((N, N), dtype=bool)), s, -np.inf)
    pr = np.exp(s - s.max(-1, keepdims=True))
    exact = np.einsum("zhnm,zhmd->zhnd", pr / pr.sum(-1, keepdims=True), vf.astype(np.float64))
    got = f32(o)
    assert not np.isnan(got).any()
    err = lambda x: np.linalg.norm(x - exact) / np.linalg.norm(exact)
    assert err(got) < 0.12  # e5m2 P and O: about 6 % is the format's own error
    pad = (-N) % 128
    if pad and not causal:
        return  # the block-walking oracle needs whole blocks; padded keys would take part without a causal mask
    if pad:
        qf, kf, vf = (np.concatenate([t, np.zeros((Z, H, pad, D), np.float32)], 2) for t in (qf, kf, vf))
    want, Mw = R.attention_fwd(qf, kf, vf, causal, sm_scale, "e5m2", BM=128, BN=128)
    want, Mw = want[:, :, :N], Mw[:, :, :N]
    np.testing.assert_allclose(f32(M), Mw, rtol=1e-4, atol=1e-3)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-2
    assert (got != want).mean() < 1e-3
    assert abs(err(got) - err(want)) < 1e-3


@pytest.mark.skipif(not hasattr(torch, "float8_e5m2"), reason="torch without float8_e5m2")
def test_forward_e5m2_errors():
    x = torch.zeros(1, 1, 128, 256, device=DEV).to(torch.float8_e5m2)
    with pytest.raises(AssertionError, match="head dims 64 and 128"):
        triton_b200.attention_forward(x, x, x, True, 0.5)
    s4 = _lib.strides4
    m = torch.zeros(1, 1, 128, device=DEV)
    code = _lib.lib().b200_attention_fwd(None, *([x.data_ptr()] * 4), m.data_ptr(), 1, 1, 128, 256, *([s4(x)] * 4),
                                         0.5, 1, _lib.E5M2)
    assert code == _lib.ERR_UNSUPPORTED and "head dims 64 and 128" in _lib.last_error()
    # the C entry point itself does not pad: head dim 32 is the wrapper's business
    x32 = torch.zeros(1, 1, 128, 32, device=DEV).to(torch.float8_e5m2)
    code = _lib.lib().b200_attention_fwd(None, *([x32.data_ptr()] * 4), m.data_ptr(), 1, 1, 128, 32, *([s4(x32)] * 4),
                                         0.5, 1, _lib.E5M2)
    assert code in (_lib.ERR_UNSUPPORTED, _lib.ERR_ARG)


def test_long_sequence_forward_sampled_rows():
    """N = 65536 (512 key blocks per row, 4.3e9 scores per head): sampled query rows against a
    dense fp32 softmax over all keys."""
    Z, H, N, D = 1, 2, 65536, 64
    g = torch.Generator(device=DEV).manual_seed(2)
    q, k, v = ((torch.randn(Z, H, N, D, generator=g, device=DEV) * 0.5).half() for _ in range(3))
    sm_scale = D ** -0.5
    for causal in (True, False):
        o, M = triton_b200.attention_forward(q, k, v, causal, sm_scale)
        status_ok()
        rows = torch.tensor([0, 1, 127, 128, 40000, N - 129, N - 1], device=DEV)
        s = (q[:, :, rows].float() @ k.float().transpose(2, 3)) * sm_scale          # [Z, H, R, N]
        if causal:
            s = s.masked_fill(torch.arange(N, device=DEV)[None, None, None, :] > rows[None, None, :, None], float("-inf"))
        want = torch.softmax(s, -1) @ v.float()
        np.testing.assert_allclose(f32(o[:, :, rows]), f32(want), rtol=1e-2, atol=1e-2)
        np.testing.assert_allclose(f32(M[:, :, rows]), f32(torch.logsumexp(s, -1) / math.log(2.0)), rtol=1e-4, atol=1e-3)


def test_ops_replay_from_a_cuda_graph():
    """The reference benchmarks attention with do_bench_cudagraph (test_performance.py:199): the ops
    must be capturable.  Forward, backward and a split-K matmul are captured once and replayed on
    new input values; results equal the eager ones bit for bit."""
    Z, H, N, D = 1, 2, 512, 64
    g = torch.Generator(device=DEV).manual_seed(4)
    q, k, v, do = ((torch.randn(Z, H, N, D, generator=g, device=DEV) * 0.5).to(torch.bfloat16) for _ in range(4))
    a = torch.randn(16, 4096, generator=g, device=DEV).half()
    b = torch.randn(4096, 256, generator=g, device=DEV).half()

    def step():
        o, M = triton_b200.attention_forward(q, k, v, True, 0.125)
        dq, dk, dv = triton_b200.attention_backward(q, k, v, o, M, do, True, 0.125)
        return o, dq, dk, dv, triton_b200.matmul(a, b)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # first calls outside capture (function attributes, context)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for trial in range(2):
        q.copy_((torch.randn(Z, H, N, D, generator=g, device=DEV) * 0.5).to(torch.bfloat16))
        a.copy_(torch.randn(16, 4096, generator=g, device=DEV).half())
        graph.replay()
        torch.cuda.synchronize()
        eager = step()
        for x, y in zip(outs, eager):
            assert torch.equal(x, y)
    status_ok()
    # the older six-argument signature
    o6 = triton_b200.attention(q, k, v, True, 0.125, True)
    assert torch.equal(o6, eager[0])


def test_graph_replay_beside_eager_launches_on_another_stream():
    """A captured launch keeps the work counter it was captured with.  Eager launches on another
    stream walk through the whole ring of eager counters several times while the graph is replayed:
    every replay and every eager result must stay bit-identical (captured launches draw their
    counters from a pool that eager launches never use)."""
    Z, H, N, D = 2, 4, 1024, 64
    g = torch.Generator(device=DEV).manual_seed(8)
    q, k, v, do = ((torch.randn(Z, H, N, D, generator=g, device=DEV) * 0.5).half() for _ in range(4))
    q2, k2, v2 = ((torch.randn(1, 8, 512, 128, generator=g, device=DEV) * 0.5).half() for _ in range(3))
    o_ref, M_ref = triton_b200.attention_forward(q, k, v, True, 0.125)
    grads_ref = triton_b200.attention_backward(q, k, v, o_ref, M_ref, do, True, 0.125)
    o2_ref, _ = triton_b200.attention_forward(q2, k2, v2, False, 0.09)
    torch.cuda.synchronize()
    cap, eager = torch.cuda.Stream(), torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=cap):
        o_g, M_g = triton_b200.attention_forward(q, k, v, True, 0.125)
        grads_g = triton_b200.attention_backward(q, k, v, o_g, M_g, do, True, 0.125)
    bad = 0
    for rnd in range(6):
        with torch.cuda.stream(eager):
            outs = [triton_b200.attention_forward(q2, k2, v2, False, 0.09)[0] for _ in range(120)]  # 720 in all: the ring has 256 slots
        with torch.cuda.stream(cap):
            for _ in range(10):
                o_g.zero_()
                graph.replay()
        torch.cuda.synchronize()
        bad += sum(0 if torch.equal(o, o2_ref) else 1 for o in outs)
        bad += 0 if torch.equal(o_g, o_ref) and all(torch.equal(x, y) for x, y in zip(grads_g, grads_ref)) else 1
    assert bad == 0
    status_ok()


def test_two_streams_and_two_host_threads():
    """Launches interleaved on two streams from two host threads (separate work counters per launch,
    per-thread error strings, one context per device): every result equals the single-stream one."""
    import threading
    Z, H, N, D = 2, 4, 1024, 64
    g = torch.Generator(device=DEV).manual_seed(6)
    q, k, v = ((torch.randn(Z, H, N, D, generator=g, device=DEV) * 0.5).half() for _ in range(3))
    a = torch.randn(1024, 512, generator=g, device=DEV).half()
    b = torch.randn(512, 768, generator=g, device=DEV).half()
    o_ref, M_ref = triton_b200.attention_forward(q, k, v, True, 0.125)
    c_ref = triton_b200.matmul(a, b)
    torch.cuda.synchronize()
    results, errors = {}, []

    def worker(name, fn):
        try:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                outs = [fn() for _ in range(40)]
            s.synchronize()
            results[name] = outs
        except Exception as e:  # surfaced below
            errors.append(repr(e))

    t1 = threading.Thread(target=worker, args=("attn", lambda: triton_b200.attention_forward(q, k, v, True, 0.125)[0]))
    t2 = threading.Thread(target=worker, args=("mm", lambda: triton_b200.matmul(a, b)))
    t1.start(); t2.start(); t1.join(); t2.join()
    assert not errors, errors
    assert all(torch.equal(o, o_ref) for o in results["attn"])
    assert all(torch.equal(c, c_ref) for c in results["mm"])
    status_ok()


def test_custom_ops_on_gpu():
    """torch.ops.triton_b200.*: same bits as the wrappers, autograd through `attention`, opcheck
    (schema, fake-tensor consistency, autograd registration)."""
    ns = torch.ops.triton_b200
    g = torch.Generator(device=DEV).manual_seed(8)
    a = torch.randn(256, 128, generator=g, device=DEV).half()
    b = torch.randn(128, 192, generator=g, device=DEV).half()
    assert torch.equal(ns.matmul(a, b), triton_b200.matmul(a, b))
    bias = torch.randn(1, 192, generator=g, device=DEV).half()
    assert torch.equal(ns.matmul(a, b, "leaky_relu", None, None, None, bias), triton_b200.matmul(a, b, "leaky_relu", bias=bias))
    q, k, v, do = ((torch.randn(1, 2, 256, 64, generator=g, device=DEV) * 0.5).to(torch.bfloat16) for _ in range(4))
    o_ref, M_ref = triton_b200.attention_forward(q, k, v, True, 0.125)
    dq_ref, dk_ref, dv_ref = triton_b200.attention_backward(q, k, v, o_ref, M_ref, do, True, 0.125)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o, M = ns.attention(qg, kg, vg, True, 0.125)
    o.backward(do)
    assert torch.equal(o, o_ref) and torch.equal(M, M_ref)
    assert torch.equal(qg.grad, dq_ref) and torch.equal(kg.grad, dk_ref) and torch.equal(vg.grad, dv_ref)
    torch.library.opcheck(ns.matmul.default, (a, b), test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(ns.attention_fwd.default, (q, k, v, True, 0.125), test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(ns.attention.default, (qg.detach().requires_grad_(), k, v, True, 0.125),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    status_ok()


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("D", [16, 32])
@pytest.mark.parametrize("causal", [True, False])
def test_small_head_dims_run_zero_padded(dtype, D, causal):
    """Head dims 16 and 32 of the reference's set (06-fused-attention.py:447) run on the head-dim-64
    kernels with zero columns appended; forward and backward against the oracle at the true D."""
    c = dict(Z=1, H=2, N=256, D=D, dtype=dtype, seed=900 + D)
    q, k, v, do = cases.attn_inputs(c)
    sm_scale = 0.5
    got = run_gpu(q, k, v, do, causal, sm_scale, True)
    assert got["o"].shape == (1, 2, 256, D) and got["dq"].shape == (1, 2, 256, D)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), causal, sm_scale, dtype)
    np.testing.assert_allclose(got["o"], o, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(got["m"], M, rtol=1e-4, atol=1e-3)
    if causal:
        dq, dk, dv = R.attention_bwd(f32(q), f32(k), f32(v), o, f32(do), M, sm_scale, dtype)
    else:
        dq, dk, dv = R.attention_bwd_full(f32(q), f32(k), f32(v), o, f32(do), M, sm_scale, False, dtype)
    tol = 1e-2 if dtype == "fp16" else 2e-2
    for key, want in (("dq", dq), ("dk", dk), ("dv", dv)):
        np.testing.assert_allclose(got[key], want, rtol=1e-2, atol=tol, err_msg=key)
