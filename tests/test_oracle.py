"""The numpy oracle against fixtures produced by the reference's kernels under the
Triton interpreter (tests/golden/make_golden.py), and against the reference tests'
own torch formulations (python/tutorials/06-fused-attention.py:533-559,
python/tutorials/03-matrix-multiplication.py:357-371)."""
import hashlib
import os

import numpy as np
import pytest
import torch

import cases
from oracle import ref_ops as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def f32(t):
    return t.detach().to(torch.float32).numpy()


@pytest.mark.parametrize("name", list(cases.MATMUL_CASES))
def test_matmul_matches_interpreter(golden, name):
    c = cases.MATMUL_CASES[name]
    a, b = cases.matmul_inputs(c)
    assert sha(a) == str(golden[f"matmul.{name}.sha_a"]) and sha(b) == str(golden[f"matmul.{name}.sha_b"])
    got = R.matmul(f32(a), f32(b), activation=c.get("activation", ""))
    want = golden[f"matmul.{name}.c"].astype(np.float32)
    # same tile order and fp32 accumulation: differences are BLAS summation order only
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-3)
    assert (got != want).mean() < 0.02


def test_interpreter_tile_program_matches_reference_fixture(golden, tmp_path):
    """oracle/interp_matmul.py restates the reference's matmul tile program in its own kernel language
    so that the Triton interpreter can be timed where no checkout of the reference exists.  Run under
    the same interpreter on the fixtures' inputs it must reproduce, bit for bit, what the reference's
    own kernel text produced (config 1 and the ragged case, whose edge tiles wrap and mask)."""
    import subprocess
    import sys
    script = tmp_path / "run.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path[:0] = [{ROOT!r}, {ROOT + '/tests/golden'!r}]\n"
        "from oracle import interp_matmul as im\n"
        "import cases\n"
        "out = {}\n"
        "for name in ('c1_512', 'ragged'):\n"
        "    a, b = cases.matmul_inputs(cases.MATMUL_CASES[name])\n"
        "    out[name] = im.matmul(a, b).numpy()\n"
        f"np.savez({str(tmp_path / 'out.npz')!r}, **out)\n")
    env = dict(os.environ, TRITON_INTERPRET="1")
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    with np.load(tmp_path / "out.npz") as z:
        for name in ("c1_512", "ragged"):
            assert np.array_equal(z[name], golden[f"matmul.{name}.c"]), name


def test_matmul_c1_reference_test_tolerance():
    # python/tutorials/03-matrix-multiplication.py:357-371 compares with torch.matmul at atol 1e-2;
    # an fp16 ulp is 0.03 at |c| > 32, so a one-ulp rounding difference needs the rtol term too
    a, b = cases.matmul_inputs(cases.MATMUL_CASES["c1_512"])
    got = R.matmul(f32(a), f32(b))
    want = torch.matmul(a.float(), b.float()).half().float().numpy()
    np.testing.assert_allclose(got, want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("name", list(cases.FP8_CASES))
def test_fp8_matches_interpreter(golden, name):
    c = cases.FP8_CASES[name]
    a8, b8, sa, sb = cases.fp8_inputs(c)
    assert sha(a8) == str(golden[f"fp8.{name}.sha_a"])
    acc = R.matmul_fp8(a8.view(torch.uint8).numpy(), b8.view(torch.uint8).numpy(), out="fp32")
    want = golden[f"fp8.{name}.acc"]
    # python/test/unit/language/test_core.py:5172-5173 tolerance for e4m3
    np.testing.assert_allclose(acc, want, rtol=1e-2, atol=1e-2)
    rel = np.linalg.norm(acc - want) / np.linalg.norm(want)
    assert rel < 1e-5
    # decode table agrees with torch's e4m3fn
    np.testing.assert_array_equal(R.decode_e4m3(a8.view(torch.uint8).numpy()), a8.float().numpy())


def test_bf16_rounding_matches_torch():
    x = torch.randn(100000, generator=torch.Generator().manual_seed(7)) * 100
    np.testing.assert_array_equal(R.round_bf16(x.numpy()), x.to(torch.bfloat16).float().numpy())


FP16_ATTN = [n for n, c in cases.ATTN_CASES.items() if c["dtype"] == "fp16"]


@pytest.mark.parametrize("name", FP16_ATTN)
def test_attention_fwd_matches_interpreter(golden, name):
    c = cases.ATTN_CASES[name]
    q, k, v, do = cases.attn_inputs(c)
    assert sha(q) == str(golden[f"attn.{name}.sha_q"])
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), c["causal"], c["sm_scale"], "fp16")
    np.testing.assert_allclose(o, golden[f"attn.{name}.o"].astype(np.float32), atol=2e-3, rtol=0)
    np.testing.assert_allclose(M, golden[f"attn.{name}.m"], atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("name", [n for n in FP16_ATTN if cases.ATTN_CASES[n].get("bwd")])
def test_attention_bwd_matches_interpreter(golden, name):
    c = cases.ATTN_CASES[name]
    q, k, v, do = cases.attn_inputs(c)
    o = golden[f"attn.{name}.o"].astype(np.float32)
    M = golden[f"attn.{name}.m"]
    dq, dk, dv = R.attention_bwd(f32(q), f32(k), f32(v), o, f32(do), M, c["sm_scale"], "fp16")
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        want = golden[f"attn.{name}.{key}"].astype(np.float32)
        np.testing.assert_allclose(got, want, atol=4e-3, rtol=1e-3)
    # dense restatement agrees with the blocked one
    dq2, dk2, dv2 = R.attention_bwd_full(f32(q), f32(k), f32(v), o, f32(do), M, c["sm_scale"], True, "fp16")
    for a_, b_ in ((dq, dq2), (dk, dk2), (dv, dv2)):
        np.testing.assert_allclose(a_, b_, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("name", [n for n, c in cases.ATTN_CASES.items() if c.get("old_style")])
def test_attention_old_style_second_opinion(golden, name):
    # python/test/unit/hopper/test_flashattention.py:361-403 (atol 1e-2)
    c = cases.ATTN_CASES[name]
    q, k, v, do = cases.attn_inputs(c)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), True, c["sm_scale"], "fp16")
    np.testing.assert_allclose(o, golden[f"attn_old.{name}.o"].astype(np.float32), atol=1e-2, rtol=0)
    dq, dk, dv = R.attention_bwd(f32(q), f32(k), f32(v), o, f32(do), M, c["sm_scale"], "fp16")
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        np.testing.assert_allclose(got, golden[f"attn_old.{name}.{key}"].astype(np.float32), atol=1e-2, rtol=0)
    # the older kernel's two statistics tensors (row sum L, row maximum M, natural base, :128-131)
    # against the newer kernel's one (base-2 log-sum-exp): lse2 = (M + ln L) / ln 2
    L, m = golden[f"attn_old.{name}.l"], golden[f"attn_old.{name}.m"]
    np.testing.assert_allclose((m + np.log(L)) / np.log(2.0), M.reshape(L.shape), rtol=1e-5, atol=1e-4)
    s = np.einsum("zhnd,zhmd->zhnm", f32(q), f32(k)) * c["sm_scale"]
    s = np.where(np.tril(np.ones(s.shape[-2:], dtype=bool)), s, -np.inf)
    np.testing.assert_allclose(m, s.max(-1).reshape(m.shape), rtol=1e-5, atol=1e-5)


def _torch_reference(q, k, v, do, causal, sm_scale):
    # the reference test's formulation: python/tutorials/06-fused-attention.py:533-549
    q, k, v = (t.detach().clone().float().requires_grad_(True) for t in (q, k, v))
    N = q.shape[2]
    p = torch.matmul(q, k.transpose(2, 3)) * sm_scale
    if causal:
        p = p.masked_fill(~torch.tril(torch.ones(N, N, dtype=torch.bool)), float("-inf"))
    p = torch.softmax(p, dim=-1)
    o = torch.matmul(p, v)
    o.backward(do.float())
    return o.detach().numpy(), q.grad.numpy(), k.grad.numpy(), v.grad.numpy()


@pytest.mark.parametrize("name", ["causal_d64", "causal_d64_bf16", "causal_d128"])
def test_attention_against_torch_formulation(name):
    c = cases.ATTN_CASES[name]
    q, k, v, do = cases.attn_inputs(c)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), c["causal"], c["sm_scale"], c["dtype"])
    dq, dk, dv = R.attention_bwd(f32(q), f32(k), f32(v), o, f32(do), M, c["sm_scale"], c["dtype"])
    ro, rdq, rdk, rdv = _torch_reference(q, k, v, do, c["causal"], c["sm_scale"])
    tol = 1e-2 if c["dtype"] == "fp16" else 3e-2
    for got, want in ((o, ro), (dq, rdq), (dk, rdk), (dv, rdv)):
        np.testing.assert_allclose(got, want, atol=tol, rtol=1e-2)
    # natural-log LSE = M * ln2
    s = torch.matmul(q.float(), k.float().transpose(2, 3)) * c["sm_scale"]
    s = s.masked_fill(~torch.tril(torch.ones(c["N"], c["N"], dtype=torch.bool)), float("-inf"))
    np.testing.assert_allclose(M * np.log(2.0), torch.logsumexp(s, -1).numpy(), atol=1e-3, rtol=1e-4)


def test_noncausal_bwd_full_against_torch():
    c = dict(cases.ATTN_CASES["full_d64"])
    q, k, v, do = cases.attn_inputs(c)
    o, M = R.attention_fwd(f32(q), f32(k), f32(v), False, c["sm_scale"], "fp16")
    dq, dk, dv = R.attention_bwd_full(f32(q), f32(k), f32(v), o, f32(do), M, c["sm_scale"], False, "fp16")
    ro, rdq, rdk, rdv = _torch_reference(q, k, v, do, False, c["sm_scale"])
    for got, want in ((o, ro), (dq, rdq), (dk, rdk), (dv, rdv)):
        np.testing.assert_allclose(got, want, atol=1e-2, rtol=1e-2)


def test_round_e4m3_matches_torch_and_saturates():
    """The oracle's fp32 -> e4m3 rounding is torch's float8_e4m3fn conversion below the largest
    finite value and saturates above it (the reference's cvt.rn.satfinite lowering)."""
    import torch
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 0.02, 1.0, 30.0, 200.0)] +
                       [np.array([0.0, -0.0, 448.0, -448.0, 447.9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9,
                                  2.5 * 2.0 ** -9, 0.0029296875], dtype=np.float32)])
    x = x[np.abs(x) <= 448]
    want = torch.tensor(x).to(torch.float8_e4m3fn).float().numpy()
    got = R.round_e4m3(x)
    assert np.array_equal(got, want)
    assert np.array_equal(np.signbit(got), np.signbit(want))
    np.testing.assert_array_equal(R.round_e4m3(np.array([500.0, -1e9, 460.0, 464.1], dtype=np.float32)),
                                  np.array([448.0, -448.0, 448.0, 448.0], dtype=np.float32))
    # every e4m3 value is a fixed point
    finite = R.E4M3[~np.isnan(R.E4M3)]
    assert np.array_equal(R.round_e4m3(finite), finite)


def test_bias_epilogue_rounds_twice_in_the_output_type():
    """`z = z.to(out_dtype); z += bias` (test_gemm.py:213-222): the oracle's add_bias rounds the
    product, adds, rounds again; checked against torch arithmetic in the output type."""
    import torch
    rng = np.random.default_rng(1)
    a = R.round_fp16(rng.standard_normal((64, 96)).astype(np.float32))
    b = R.round_fp16(rng.standard_normal((96, 80)).astype(np.float32))
    for shape in ((64, 80), (64, 1), (1, 80)):
        bias = R.round_fp16(rng.standard_normal(shape).astype(np.float32))
        got = R.matmul(a, b, out="fp16", bias=bias)
        z = torch.tensor(R.matmul(a, b, out="fp32")).half()  # the oracle's own fp32 accumulator
        z = z + torch.tensor(bias).half()
        np.testing.assert_array_equal(got, z.float().numpy())


def test_round_e5m2_matches_torch_and_saturates():
    import torch
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-5, 1e-3, 1.0, 300.0, 20000.0)] +
                       [np.array([0.0, -0.0, 57344.0, -57344.0, 2.0 ** -16, 2.0 ** -17, 1.5 * 2.0 ** -16, 2.5 * 2.0 ** -16],
                                 dtype=np.float32)])
    x = x[np.abs(x) <= 57344]
    want = torch.tensor(x).to(torch.float8_e5m2).float().numpy()
    got = R.round_e5m2(x)
    assert np.array_equal(got, want) and np.array_equal(np.signbit(got), np.signbit(want))
    np.testing.assert_array_equal(R.round_e5m2(np.array([6e4, -1e9], dtype=np.float32)),
                                  np.array([57344.0, -57344.0], dtype=np.float32))


@pytest.mark.parametrize("name", list(cases.EPILOGUE_CASES))
def test_epilogues_match_interpreter_fixture(golden, name):
    """Fixtures produced by the reference's matmul_kernel with epilogues
    (python/test/unit/hopper/test_gemm.py:143-247) under the interpreter: the bias epilogues are
    reproduced bit for bit (same tile loop, same two roundings), and so is chain-dot; the softmax epilogue within the
    reference test's own tolerance (rows normalised, rtol 1e-2, atol 1e-3; the interpreter sums the
    fp16 numerators in fp16, the oracle in fp32)."""
    c = cases.EPILOGUE_CASES[name]
    a, b, bias = cases.epilogue_inputs(c)
    for nm, t in (("a", a), ("b", b), ("bias", bias)):
        assert golden[f"epilogue.{name}.sha_{nm}"].item() == sha(t), "input generator drifted"
    want = golden[f"epilogue.{name}.z"].astype(np.float32)
    af, bf, biasf = a.float().numpy(), b.float().numpy(), bias.float().numpy()
    ep = c["epilogue"]
    if ep == "softmax":
        got = R.matmul(af, bf, activation="softmax", out=c["out"], BM=64, BN=c["N"], BK=32)
        nz = lambda x: x / np.linalg.norm(x, axis=1, keepdims=True)
        np.testing.assert_allclose(nz(got), nz(want), rtol=1e-2, atol=1e-3)
        np.testing.assert_allclose(got.sum(1), 1.0, atol=5e-3)
    elif ep == "chain-dot":  # same tile loop and the same three roundings: bit for bit
        w = cases.chain_weight(c).float().numpy()
        got = R.matmul_chain(af, bf, w, out=c["out"], storage="fp16", BM=64, BK=32)
        np.testing.assert_array_equal(got, want)
        exact = (af.astype(np.float64) @ bf.astype(np.float64)) @ w.astype(np.float64)
        np.testing.assert_allclose(got, exact, rtol=1e-2, atol=1e-2 * np.abs(exact).max())
    else:
        bsel = {"add-matrix": biasf, "add-rows": biasf[:, :1], "add-cols": biasf[:1, :]}[ep]
        got = R.matmul(af, bf, out=c["out"], BM=64, BN=64, BK=32, bias=bsel)
        np.testing.assert_array_equal(got, want)
