"""Parity of the CUDA matmul (through the C ABI) with the CPU oracle, the interpreter-generated
golden fixtures and, at the benchmark's full size, size-independent properties.

Tolerances: rtol = atol = 1e-2 for fp16 / bf16 (python/tutorials/03-matrix-multiplication.py:
367-368 uses atol 1e-2 against torch), relative Frobenius error <= 2e-2 for fp8 with scales
(python/test/unit/language/test_core.py:5172-5173 uses rtol = atol = 1e-2 on the accumulator)."""
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


@pytest.mark.parametrize("name", list(cases.MATMUL_CASES))
def test_matmul_parity_with_oracle_and_golden(golden, name):
    c = cases.MATMUL_CASES[name]
    a, b = cases.matmul_inputs(c)
    got = triton_b200.matmul(a.to(DEV), b.to(DEV), activation=c.get("activation", ""))
    status_ok()
    assert got.dtype == torch.float16 and got.shape == (c["M"], c["N"])
    want = R.matmul(f32(a), f32(b), activation=c.get("activation", ""))
    np.testing.assert_allclose(f32(got), want, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(f32(got), golden[f"matmul.{name}.c"].astype(np.float32), rtol=1e-2, atol=1e-2)
    # one fp32 accumulation and one rounding on both sides: almost all elements are bit-identical
    assert (f32(got) != want).mean() < 0.05


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 64, 64), (1, 8, 8), (129, 264, 72), (1000, 520, 200), (2048, 2048, 512),
                                   (8192, 8192, 1024)])
@pytest.mark.parametrize("b_layout", ["kn", "nk"])
def test_matmul_shapes_layouts(dtype, shape, b_layout):
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(K, N, generator=g).to(dtype)
    bd = b.to(DEV)
    if b_layout == "nk":
        bd = bd.t().contiguous().t()
    got = triton_b200.matmul(a.to(DEV), bd)
    status_ok()
    assert got.dtype == dtype
    if M * N * K <= 2048 * 2048 * 512:
        want = R.matmul(f32(a), f32(b), out="fp16" if dtype == torch.float16 else "bf16")
    else:  # the python tile loop is too slow here; same arithmetic through one fp32 matmul
        want = (a.float() @ b.float()).to(dtype).float().numpy()
    tol = 1e-2 if dtype == torch.float16 else 2e-2
    np.testing.assert_allclose(f32(got), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("tile", ["128064", "128128", "128192", "128256", "256192", "256256", "2256", "2512"])
def test_every_tile_shape(monkeypatch, tile):
    monkeypatch.setenv("B200_GEMM_TILE", tile)
    g = torch.Generator().manual_seed(11)
    a = torch.randn(600, 328, generator=g).half()
    b = torch.randn(328, 712, generator=g).half()
    want = R.matmul(f32(a), f32(b))
    got = triton_b200.matmul(a.to(DEV), b.to(DEV))
    status_ok()
    np.testing.assert_allclose(f32(got), want, rtol=1e-2, atol=1e-2)
    # the direct-store epilogue (used for fp32 outputs and for a C that TMA cannot address) gives the same bits
    monkeypatch.setenv("B200_GEMM_DIRECT_STORE", "1")
    direct = triton_b200.matmul(a.to(DEV), b.to(DEV))
    assert torch.equal(direct, got)
    # C as a column slice of a wider matrix (row stride 1424 bytes, still TMA-addressable) and fp32 output
    monkeypatch.delenv("B200_GEMM_DIRECT_STORE")
    wide = torch.zeros(600, 1424, dtype=torch.float16, device=DEV)
    triton_b200.matmul(a.to(DEV), b.to(DEV), out=wide[:, 8:720], out_dtype=torch.float16)
    assert torch.equal(wide[:, 8:720], got) and float(wide[:, :8].abs().sum()) == 0 and float(wide[:, 720:].abs().sum()) == 0
    acc = triton_b200.matmul(a.to(DEV), b.to(DEV), out_dtype=torch.float32)
    np.testing.assert_allclose(f32(acc), f32(a) @ f32(b), rtol=1e-3, atol=1e-3)
    status_ok()


def test_empty_and_degenerate():
    a = torch.zeros(0, 16, dtype=torch.float16, device=DEV)
    b = torch.zeros(16, 8, dtype=torch.float16, device=DEV)
    assert triton_b200.matmul(a, b).shape == (0, 8)
    a = torch.ones(5, 0, dtype=torch.float16, device=DEV)
    b = torch.ones(0, 8, dtype=torch.float16, device=DEV)
    c = triton_b200.matmul(a, b)
    assert c.shape == (5, 8) and float(c.abs().sum()) == 0.0  # empty sum
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("shape", [(8, 6, 12), (129, 257, 70), (300, 77, 513)])
def test_layouts_tma_cannot_address(dtype, shape):
    """Row strides that are not multiples of 16 bytes, and operands with no unit stride at all, are legal
    for the reference kernel (it takes arbitrary strides); they run on the plain CUDA-core kernel."""
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(K, N, generator=g).to(dtype)
    af, bf = a.float().numpy(), b.float().numpy()
    out = "fp16" if dtype == torch.float16 else "bf16"
    want = R.matmul(af, bf, out=out)
    got = triton_b200.matmul(a.to(DEV), b.to(DEV))
    np.testing.assert_allclose(f32(got), want, rtol=2e-2, atol=2e-2)
    # B with no unit stride: every second column of a wider matrix
    wide = torch.zeros(K, 2 * N, dtype=dtype, device=DEV)
    wide[:, ::2] = b.to(DEV)
    got2 = triton_b200.matmul(a.to(DEV), wide[:, ::2])
    assert torch.equal(got2, got)
    status_ok()


def test_plain_kernel_matches_tensor_core_kernel(monkeypatch):
    g = torch.Generator().manual_seed(99)
    a = torch.randn(320, 256, generator=g).half().to(DEV)
    b = torch.randn(256, 192, generator=g).half().to(DEV)
    fast = triton_b200.matmul(a, b, activation="leaky_relu")
    monkeypatch.setenv("B200_GEMM_PLAIN", "1")
    plain = triton_b200.matmul(a, b, activation="leaky_relu")
    np.testing.assert_allclose(f32(plain), f32(fast), rtol=2e-3, atol=2e-3)


def _raw_matmul_splitk(a, b, splits, out_dtype=None, activation="", scales=(None, None)):
    """Calls b200_matmul_splitk with an explicit split count (the wrapper only picks the planned one)."""
    from triton_b200.ops import _ACT, _DT, _stream
    M, K = a.shape
    N = b.shape[1]
    out_dtype = out_dtype or a.dtype
    c = torch.empty(M, N, device=a.device, dtype=out_dtype)
    ws = torch.empty(max(splits, 1) * M * N, device=a.device, dtype=torch.float32)
    sa, sb = scales
    code = _lib.lib().b200_matmul_splitk(
        _stream(a), a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), a.stride(1), b.stride(0),
        b.stride(1), c.stride(0), c.stride(1), _DT[a.dtype], _DT[out_dtype], _ACT[activation],
        sa.data_ptr() if sa is not None else None, sb.data_ptr() if sb is not None else None, splits,
        ws.data_ptr() if splits > 1 else None)
    _lib.check(code, "matmul_splitk")
    return c


@pytest.mark.parametrize("shape", [(16, 4096, 4096), (64, 4096, 4096), (8192, 64, 8192), (130, 72, 2120)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_skinny_shapes_take_split_k(shape, dtype):
    """Few tiles and a long K: the plan cuts K, the wrapper supplies the workspace, the result is the
    oracle's (fp32 partial sums, one rounding at the end)."""
    import ctypes
    M, N, K = shape
    splits, ws_bytes = ctypes.c_int(0), ctypes.c_size_t(0)
    _lib.check(_lib.lib().b200_matmul_plan(M, N, K, 0, ctypes.byref(splits), ctypes.byref(ws_bytes)), "plan")
    assert splits.value > 1 and ws_bytes.value == splits.value * M * N * 4
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(K, N, generator=g).to(dtype)
    got = triton_b200.matmul(a.to(DEV), b.to(DEV), activation="leaky_relu")
    status_ok()
    want = R.matmul(f32(a), f32(b), activation="leaky_relu", out="fp16" if dtype == torch.float16 else "bf16")
    np.testing.assert_allclose(f32(got), want, rtol=1e-2, atol=1e-2)
    # large problems are never split
    _lib.check(_lib.lib().b200_matmul_plan(4096, 4096, 4096, 0, ctypes.byref(splits), ctypes.byref(ws_bytes)), "plan")
    assert splits.value == 1 and ws_bytes.value == 0


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 16, 64])
def test_split_k_any_split_count(splits):
    """Any split count gives the unsplit result up to the fp32 summation order; more splits than
    K blocks are clipped; fp32 output, scales and fp8 operands take the same path."""
    M, N, K = 200, 136, 1544  # ragged in every dimension: 25 K blocks, the last one partial
    g = torch.Generator().manual_seed(splits)
    a = torch.randn(M, K, generator=g).half().to(DEV)
    b = torch.randn(K, N, generator=g).half().to(DEV)
    base = _raw_matmul_splitk(a, b, 1, out_dtype=torch.float32)
    got = _raw_matmul_splitk(a, b, splits, out_dtype=torch.float32)
    status_ok()
    want = f32(a).astype(np.float64) @ f32(b).astype(np.float64)
    np.testing.assert_allclose(f32(got), want, rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(f32(got), f32(base), rtol=1e-4, atol=1e-3)
    again = _raw_matmul_splitk(a, b, splits, out_dtype=torch.float32)
    assert torch.equal(got, again), "the reduction order is fixed: two runs are bit-identical"
    # fp8 with per-tensor scales and bf16 output
    a8, sa = triton_b200.quantize_e4m3(a.float())
    b8, sb = triton_b200.quantize_e4m3(b.float())
    c1 = _raw_matmul_splitk(a8, b8, 1, out_dtype=torch.bfloat16, scales=(sa, sb))
    cs = _raw_matmul_splitk(a8, b8, splits, out_dtype=torch.bfloat16, scales=(sa, sb))
    status_ok()
    np.testing.assert_allclose(f32(cs), f32(c1), rtol=1e-2, atol=1e-2)


def test_split_k_argument_errors():
    a = torch.zeros(16, 4096, device=DEV, dtype=torch.float16)
    b = torch.zeros(4096, 64, device=DEV, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="splits"):
        _raw_matmul_splitk(a, b, 65)
    from triton_b200.ops import _stream
    c = torch.empty(16, 64, device=DEV, dtype=torch.float16)
    code = _lib.lib().b200_matmul_splitk(_stream(a), a.data_ptr(), b.data_ptr(), c.data_ptr(), 16, 64, 4096, 4096, 1,
                                         64, 1, 64, 1, 0, 0, 0, None, None, 4, None)
    assert code == 1 and b"workspace" in _lib.lib().b200_last_error()


@pytest.mark.parametrize("name", list(cases.FP8_CASES))
def test_fp8_accumulator_matches_golden(golden, name):
    c = cases.FP8_CASES[name]
    a8, b8, sa, sb = cases.fp8_inputs(c)
    acc = triton_b200.matmul(a8.to(DEV), b8.to(DEV), out_dtype=torch.float32)
    status_ok()
    want = golden[f"fp8.{name}.acc"]
    np.testing.assert_allclose(f32(acc), want, rtol=1e-2, atol=1e-2)
    assert np.linalg.norm(f32(acc) - want) / np.linalg.norm(want) < 1e-5


@pytest.mark.parametrize("shape", [(256, 512, 512), (1024, 1024, 2048), (4096, 4096, 1024)])
def test_fp8_scaled_parity(shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(K, N, generator=g)
    a8, sa = cases.quantize_e4m3(a)
    b8, sb = cases.quantize_e4m3(b)
    got = triton_b200.matmul(a8.to(DEV), b8.to(DEV), scale_a=sa, scale_b=sb)
    status_ok()
    assert got.dtype == torch.bfloat16
    want = R.matmul_fp8(a8.view(torch.uint8).numpy(), b8.view(torch.uint8).numpy(), sa, sb, out="bf16")
    rel = np.linalg.norm(f32(got) - want) / np.linalg.norm(want)
    assert rel < 2e-2, rel
    # and against the unquantised product: quantisation noise only
    exact = (a @ b).numpy()
    assert np.linalg.norm(f32(got) - exact) / np.linalg.norm(exact) < 6e-2
    # device-side quantisation helper gives the same bits
    a8d, sad = triton_b200.quantize_e4m3(a.to(DEV))
    assert torch.equal(a8d.view(torch.uint8).cpu(), a8.view(torch.uint8))
    assert abs(float(sad) - sa) / sa < 1e-6


def _full_size_inputs(dtype):
    g = torch.Generator().manual_seed(2024)
    n = 8192
    a = (torch.randn(n, n, generator=g) / n ** 0.5)
    b = (torch.randn(n, n, generator=g) / n ** 0.5)
    return a, b


def test_full_size_fp16_properties():
    """Config 2 (8192^3 fp16): sampled entries against fp64 dot products, the checksum identity
    sum(C) = (1^T A)(B 1), and bitwise repeatability (catches shared-memory / TMEM races)."""
    a, b = _full_size_inputs(torch.float16)
    ah, bh = a.half(), b.half()
    ad, bd = ah.to(DEV), bh.to(DEV)
    c1 = triton_b200.matmul(ad, bd)
    c2 = triton_b200.matmul(ad, bd)
    status_ok()
    assert torch.equal(c1, c2)
    rs = np.random.RandomState(0)
    rows = rs.randint(0, 8192, 64)
    cols = rs.randint(0, 8192, 64)
    a64 = ah[rows].double().numpy()
    b64 = bh[:, cols].double().numpy()
    want = a64 @ b64
    got = c1[rows][:, cols].float().cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2)
    total = float(c1.double().sum())
    ident = float(ah.double().sum(0) @ bh.double().sum(1))
    assert abs(total - ident) < 1e-3 * max(1.0, abs(ident)) + 8192 * 8192 * 2e-5  # fp16 output rounding noise
    # linearity in A: (2A) B = 2 (A B) bit for bit wherever the fp16 result is a normal number
    # (a subnormal result rounds on a different grid once doubled)
    c3 = triton_b200.matmul(ad * 2, bd)
    normal = c1.abs() >= 2.0 ** -13
    assert torch.equal(c3[normal], (c1 * 2)[normal])
    assert float((c3.float() - 2 * c1.float()).abs().max()) <= 2.0 ** -23


def test_full_size_fp8_properties():
    a, b = _full_size_inputs(torch.float32)
    a8, sa = cases.quantize_e4m3(a * 8192 ** 0.5)
    b8, sb = cases.quantize_e4m3(b * 8192 ** 0.5)
    got = triton_b200.matmul(a8.to(DEV), b8.to(DEV), scale_a=sa, scale_b=sb)
    got2 = triton_b200.matmul(a8.to(DEV), b8.to(DEV), scale_a=sa, scale_b=sb)
    status_ok()
    assert torch.equal(got, got2)
    rs = np.random.RandomState(1)
    rows, cols = rs.randint(0, 8192, 48), rs.randint(0, 8192, 48)
    want = (a8[rows].double().numpy() @ b8[:, cols].double().numpy()) * (sa * sb)
    g = got[rows][:, cols].float().cpu().numpy()
    assert np.linalg.norm(g - want) / np.linalg.norm(want) < 2e-2


def test_full_size_configs_against_the_oracle_on_sampled_programs():
    """Configs 2 and 3 at full size against the ORACLE: the reference launches 64 x 32 programs of
    128 x 256 (python/tutorials/03-matrix-multiplication.py:169-170) over an 8192^3 problem; the
    oracle runs a handful of them (first, last, both edges of a rasterisation group, two interior)
    over the full K range and those tiles of the CUDA result must agree - rtol = atol = 1e-2
    for fp16, relative Frobenius error <= 2e-2 per tile for e4m3 with scales."""
    BM, BN = 128, 256
    n = 8192
    pids = [0, 7, 8 * 32 - 1, 8 * 32, 1000, 1337, 64 * 32 - 1]
    a, b = _full_size_inputs(torch.float16)
    ah, bh = a.half(), b.half()
    got = triton_b200.matmul(ah.to(DEV), bh.to(DEV))
    status_ok()
    want = R.matmul(ah.float().numpy(), bh.float().numpy(), pids=pids)
    seen = set()
    for pid in pids:
        m0, n0 = R.matmul_tile_origin(n, n, pid)
        seen.add((m0, n0))
        np.testing.assert_allclose(got[m0:m0 + BM, n0:n0 + BN].float().cpu().numpy(), want[m0:m0 + BM, n0:n0 + BN],
                                   rtol=1e-2, atol=1e-2, err_msg=f"program {pid}")
    assert len(seen) == len(pids) and (0, 0) in seen and (n - BM, n - BN) in seen
    del got
    # config 3: e4m3 with per-tensor scales, bf16 output; the fp8 kernel's programs run column-major
    a8, sa = cases.quantize_e4m3(a * n ** 0.5)
    b8, sb = cases.quantize_e4m3(b * n ** 0.5)
    got8 = triton_b200.matmul(a8.to(DEV), b8.to(DEV), scale_a=sa, scale_b=sb)
    status_ok()
    pids8 = [0, 63, 64, 1000, 64 * 32 - 1]
    want8 = R.matmul_fp8(a8.view(torch.uint8).numpy(), b8.view(torch.uint8).numpy(), float(sa), float(sb), pids=pids8)
    for pid in pids8:
        m0, n0 = (pid % 64) * BM, (pid // 64) * BN
        g, w = got8[m0:m0 + BM, n0:n0 + BN].float().cpu().numpy(), want8[m0:m0 + BM, n0:n0 + BN]
        assert np.linalg.norm(g - w) / np.linalg.norm(w) < 2e-2, f"program {pid}"
        np.testing.assert_allclose(g, w, rtol=2e-2, atol=2e-2, err_msg=f"program {pid}")


def test_host_matmul_pipeline_matches_device_matmul():
    """HostMatmul (pinned host operands, row blocks pipelined over two copy streams) gives the
    device-resident matmul's result, also for a row count that the blocks do not divide."""
    M, N, K = 1000, 520, 264
    g = torch.Generator().manual_seed(5)
    a_h = torch.randn(M, K, generator=g).half().pin_memory()
    b_h = torch.randn(K, N, generator=g).half().pin_memory()
    c_h = torch.empty(M, N, dtype=torch.float16).pin_memory()
    hm = triton_b200.HostMatmul(M, N, K, torch.float16, DEV, blocks=3)
    for _ in range(2):  # the second run reuses the device buffers while nothing of the first is pending
        hm.run(a_h, b_h, c_h, activation="leaky_relu")
        torch.cuda.synchronize()
        want = triton_b200.matmul(a_h.to(DEV), b_h.to(DEV), activation="leaky_relu")
        np.testing.assert_allclose(f32(c_h), f32(want), rtol=1e-2, atol=1e-2)
    # back-to-back calls without a synchronisation in between reuse the device buffers in stream
    # order: every call has its own host operands and result
    ins = [(torch.randn(M, K, generator=g).half().pin_memory(), torch.randn(K, N, generator=g).half().pin_memory())
           for _ in range(5)]
    outs = [torch.empty(M, N, dtype=torch.float16).pin_memory() for _ in range(5)]
    for (ah, bh), ch in zip(ins, outs):
        hm.run(ah, bh, ch)
    torch.cuda.synchronize()
    for (ah, bh), ch in zip(ins, outs):
        want = triton_b200.matmul(ah.to(DEV), bh.to(DEV))
        np.testing.assert_allclose(f32(ch), f32(want), rtol=1e-2, atol=1e-2)
    # an unchanged B is not sent again; one modified in place (same storage, new version) is
    ah, bh = ins[-1]
    hm.run(ah, bh, outs[0])
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[-1])
    bh.mul_(-1.0)
    hm.run(ah, bh, outs[1])
    torch.cuda.synchronize()
    np.testing.assert_allclose(f32(outs[1]), -f32(outs[-1]), rtol=0, atol=0)
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("mode", ["matrix", "rows", "cols"])
@pytest.mark.parametrize("shape", [(256, 512, 128), (200, 136, 72), (16, 4096, 4096)])
def test_bias_epilogues(dtype, mode, shape):
    """The reference's 'add-matrix' / 'add-rows' / 'add-cols' epilogues (test_gemm.py:213-222, 281)
    on the tensor-core path (TMA-store and direct-store epilogues) and on the split-K path."""
    M, N, K = shape
    g = torch.Generator().manual_seed(M + 3 * N + K)
    a = torch.randn(M, K, generator=g).half()
    b = torch.randn(K, N, generator=g).half()
    bshape = {"matrix": (M, N), "rows": (M, 1), "cols": (1, N)}[mode]
    bias = (torch.randn(bshape, generator=g) * 4).to(dtype)
    got = triton_b200.matmul(a.to(DEV), b.to(DEV), out_dtype=dtype, bias=bias.to(DEV))
    status_ok()
    out = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.float32: "fp32"}[dtype]
    want = R.matmul(f32(a), f32(b), out=out, bias=f32(bias))
    # the product is rounded to the output type before the addition: one ulp of the product (not
    # of the possibly much smaller sum) is the unit of disagreement
    prod = np.abs(R.matmul(f32(a), f32(b), out="fp32"))
    rel = 2e-2 if dtype == torch.bfloat16 else 1e-2  # two bf16 roundings: up to two ulps of 2^-8 .. 2^-7
    assert (np.abs(f32(got) - want) <= 1e-2 + rel * (prod + np.abs(f32(bias)))).all()
    if dtype != torch.float32 and K <= 128:
        assert (f32(got) != want).mean() < 0.05  # same two roundings: almost all elements bit-identical
    # a strided bias view (every second column of a wider buffer)
    if mode == "matrix":
        wide = torch.zeros(M, 2 * N, dtype=dtype)
        wide[:, ::2] = bias
        got2 = triton_b200.matmul(a.to(DEV), b.to(DEV), out_dtype=dtype, bias=wide.to(DEV)[:, ::2])
        assert torch.equal(got2, got)


def test_bias_on_the_plain_kernel_and_errors():
    a = torch.randn(70, 13).half().to(DEV)   # K pitch of 26 bytes: TMA cannot address it
    b = torch.randn(13, 9).half().to(DEV)
    bias = torch.randn(1, 9).half().to(DEV)
    got = triton_b200.matmul(a, b, bias=bias)
    want = R.matmul(f32(a), f32(b), out="fp16", bias=f32(bias))
    np.testing.assert_allclose(f32(got), want, rtol=1e-2, atol=2e-2)
    with pytest.raises(AssertionError, match="bias shape"):
        triton_b200.matmul(a, b, bias=torch.zeros(9, 1, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError, match="e4m3"):
        triton_b200.matmul(a, b, out_dtype=torch.float8_e4m3fn, bias=torch.zeros(1, 9, dtype=torch.float8_e4m3fn, device=DEV))
    status_ok()


@pytest.mark.parametrize("shape", [(256, 512, 256), (130, 200, 136), (64, 4096, 4096)])
@pytest.mark.parametrize("in_dtype", [torch.float16, torch.float8_e4m3fn])
def test_e4m3_output(shape, in_dtype):
    """8-bit output (python/tutorials/09-persistent-matmul.py:93-94): round to nearest even,
    saturating; checked against the oracle's rounding of the exact fp32 accumulator."""
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(K, N, generator=g)
    if in_dtype == torch.float8_e4m3fn:
        a8, sa = triton_b200.quantize_e4m3(a.to(DEV))
        b8, sb = triton_b200.quantize_e4m3(b.to(DEV))
        got = triton_b200.matmul(a8, b8, scale_a=sa, scale_b=sb, out_dtype=torch.float8_e4m3fn)
        acc = (a8.float() @ b8.float()) * (sa * sb)
    else:
        ah, bh = a.half().to(DEV), b.half().to(DEV)
        got = triton_b200.matmul(ah, bh, out_dtype=torch.float8_e4m3fn)
        acc = ah.float() @ bh.float()
    status_ok()
    assert got.dtype == torch.float8_e4m3fn
    want = R.round_e4m3(f32(acc))
    gotf = f32(got)
    assert not np.isnan(gotf).any(), "saturating conversion never produces NaN"
    assert np.abs(gotf).max() <= 448
    # fp32 summation order differs from torch's matmul: values next to a rounding boundary may land
    # on the neighbouring e4m3 value (1/8 relative step); everything else is identical
    close = np.abs(gotf - want) <= 0.13 * np.maximum(np.abs(want), 2.0 ** -6)
    assert close.all()
    assert (gotf != want).mean() < 0.02


def _grouped_inputs(shapes, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    A = [torch.rand(M, K, generator=g).to(dtype) for (M, N, K) in shapes]   # the reference uses torch.rand
    B = [torch.rand(K, N, generator=g).to(dtype) for (M, N, K) in shapes]
    return A, B


def test_grouped_matmul_reference_sizes():
    """python/tutorials/08-grouped-gemm.py:194-215: four square problems 1024 .. 128, fp16, compared
    per group with atol 1e-2 (the reference's check) against the oracle's tile loop."""
    shapes = [(s, s, s) for s in (1024, 512, 256, 128)]
    A, B = _grouped_inputs(shapes, torch.float16, 0)
    C = triton_b200.group_gemm_fn([t.to(DEV) for t in A], [t.to(DEV) for t in B])
    status_ok()
    assert len(C) == 4
    for a, b, c in zip(A, B, C):
        assert c.dtype == torch.float16 and c.shape == (a.shape[0], b.shape[1])
        want = R.matmul(f32(a), f32(b), out="fp16")
        # torch.rand inputs: |c| ~ K/4, one fp16 ulp at 256 is 0.125
        np.testing.assert_allclose(f32(c), want, rtol=1e-2, atol=1e-2)
        assert (f32(c) != want).mean() < 0.05


@pytest.mark.parametrize("dtype,out_dtype", [(torch.float16, None), (torch.bfloat16, torch.float32)])
def test_grouped_matmul_ragged_and_empty_groups(dtype, out_dtype):
    """Partial tiles in every dimension, one-row and one-tile problems, an empty group, a K = 0 group
    (an empty sum: zeros), more tiles than SMs; each group equals the single matmul's bits (up to the summation order
    where the single matmul splits K)."""
    shapes = [(130, 72, 200), (1, 8, 8), (300, 520, 64), (0, 64, 64), (64, 128, 0), (2000, 1544, 136), (128, 128, 4096)]
    A, B = _grouped_inputs(shapes, dtype, 1)
    Ad, Bd = [t.to(DEV) for t in A], [t.to(DEV) for t in B]
    C = triton_b200.group_gemm_fn(Ad, Bd, out_dtype=out_dtype)
    status_ok()
    od = out_dtype or dtype
    for (M, N, K), a, b, c in zip(shapes, Ad, Bd, C):
        assert c.shape == (M, N) and c.dtype == od
        if M == 0:
            continue
        if K == 0:
            assert float(c.abs().max()) == 0.0
            continue
        single = triton_b200.matmul(a, b, out_dtype=od)
        if K < 2048:  # longer K loops take split-K in the single matmul: another summation order
            assert torch.equal(c, single), (M, N, K)
        else:
            assert torch.allclose(c.float(), single.float(), rtol=4e-3, atol=1e-2), (M, N, K)
        out = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.float32: "fp32"}[od]
        if M * N * K <= 300 * 520 * 64:
            np.testing.assert_allclose(f32(c), R.matmul(f32(a), f32(b), out=out), rtol=1e-2, atol=1e-2)


def test_grouped_matmul_layout_errors_and_strided_operands():
    a = torch.rand(64, 72, dtype=torch.float16, device=DEV)
    b9 = torch.rand(72, 9, dtype=torch.float16, device=DEV)   # ldb = 9 elements: not addressable by TMA
    with pytest.raises(RuntimeError, match="16 bytes"):
        triton_b200.group_gemm_fn([a], [b9])
    # row-major views with padded leading dimensions are fine
    wide_a = torch.rand(64, 144, dtype=torch.float16, device=DEV)
    wide_b = torch.rand(72, 80, dtype=torch.float16, device=DEV)
    av, bv = wide_a[:, :72], wide_b[:, :40]
    (c,) = triton_b200.group_gemm_fn([av], [bv])
    assert torch.equal(c, triton_b200.matmul(av.contiguous(), bv.contiguous()))
    assert triton_b200.group_gemm_fn([], []) == []
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(64, 64, 64), (128, 128, 128), (16, 16, 64), (300, 200, 136), (1000, 256, 520)])
def test_softmax_epilogue(dtype, shape):
    """The reference's 'softmax' epilogue (test_gemm.py:223-228; its shapes at :268-272 plus ragged
    ones and more than one wave of row tiles): a softmax over every row of the product."""
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) / K ** 0.25).half()
    b = (torch.randn(K, N, generator=g) / K ** 0.25).half()
    got = triton_b200.matmul(a.to(DEV), b.to(DEV), activation="softmax", out_dtype=dtype)
    status_ok()
    out = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.float32: "fp32"}[dtype]
    want = R.matmul(f32(a), f32(b), activation="softmax", out=out)
    gotf = f32(got)
    np.testing.assert_allclose(gotf.sum(1), 1.0, atol=2e-2)
    # the reference's check: rows normalised to unit length, rtol 1e-2, atol 1e-3 (bf16: its coarser ulp)
    nz = lambda x: x / np.linalg.norm(x, axis=1, keepdims=True)
    np.testing.assert_allclose(nz(gotf), nz(want), rtol=2e-2 if dtype == torch.bfloat16 else 1e-2,
                               atol=4e-3 if dtype == torch.bfloat16 else 1e-3)
    exact = torch.softmax(a.float() @ b.float(), dim=1).numpy()
    np.testing.assert_allclose(gotf, exact, rtol=3e-2, atol=2e-3)


def test_softmax_epilogue_errors():
    a = torch.zeros(64, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="N <= 256"):
        triton_b200.matmul(a, torch.zeros(64, 512, dtype=torch.float16, device=DEV), activation="softmax")
    with pytest.raises(RuntimeError, match="no bias"):
        triton_b200.matmul(a, a, activation="softmax", bias=torch.zeros(1, 64, dtype=torch.float16, device=DEV))


def test_output_with_more_than_2_31_elements():
    """Index arithmetic past 32 bits: C has 46400^2 = 2.15e9 elements (4.3 GB); sampled entries are
    compared with fp64 dot products, through the TMA-store epilogue and the direct-store one."""
    M = N = 46400
    K = 64
    g = torch.Generator(device=DEV).manual_seed(1)
    a = torch.randn(M, K, generator=g, device=DEV).half()
    b = torch.randn(K, N, generator=g, device=DEV).half()
    rows = torch.tensor([0, 1, 12345, 46271, 46272, M - 1], device=DEV)
    cols = torch.tensor([0, 7, 33333, 46399], device=DEV)
    want = (a[rows].double() @ b[:, cols].double()).cpu().numpy()
    for out_dtype in (torch.float16, torch.float32):   # TMA stores / direct stores
        c = triton_b200.matmul(a, b, out_dtype=out_dtype)
        status_ok()
        got = c[rows][:, cols].double().cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2)
        # the far corner block is written and nothing else was clobbered: checksum of the last rows
        tail = c[-64:].float()
        np.testing.assert_allclose(tail.cpu().numpy(), (a[-64:].float() @ b.float()).cpu().numpy(), rtol=1e-2, atol=1e-2)
        del c, tail
        torch.cuda.empty_cache()


def test_grouped_matmul_prepared_plan_reruns():
    """GroupedMatmul: descriptors prepared once, launched repeatedly on changing operand values
    (what the reference times as triton_perf_fn, 08-grouped-gemm.py:218-229)."""
    shapes = [(256, 128, 64), (130, 72, 200), (512, 512, 512)]
    A, B = _grouped_inputs(shapes, torch.float16, 3)
    Ad, Bd = [t.to(DEV) for t in A], [t.to(DEV) for t in B]
    plan = triton_b200.GroupedMatmul(Ad, Bd)
    for trial in range(3):
        for t in Ad:
            t.uniform_(0, 1)
        out = plan.run()
        status_ok()
        for a, b, c in zip(Ad, Bd, out):
            assert torch.equal(c, triton_b200.matmul(a, b))


@pytest.mark.parametrize("name", list(cases.EPILOGUE_CASES))
def test_epilogues_against_interpreter_fixture(golden, name):
    """The CUDA epilogues against fixtures produced by the reference's own epilogue kernel
    (python/test/unit/hopper/test_gemm.py:143-247) under the interpreter."""
    c = cases.EPILOGUE_CASES[name]
    a, b, bias = cases.epilogue_inputs(c)
    want = golden[f"epilogue.{name}.z"].astype(np.float32)
    dt = torch.float16 if c["out"] == "fp16" else torch.float32
    ep = c["epilogue"]
    ad, bd, biasd = a.to(DEV), b.to(DEV), bias.to(DEV)
    if ep == "softmax":
        got = f32(triton_b200.matmul(ad, bd, activation="softmax", out_dtype=dt))
        nz = lambda x: x / np.linalg.norm(x, axis=1, keepdims=True)
        np.testing.assert_allclose(nz(got), nz(want), rtol=1e-2, atol=1e-3)  # the reference test's check
    elif ep == "chain-dot":
        w = cases.chain_weight(c)
        got = f32(triton_b200.matmul_chain(ad, bd, w.to(DEV), out_dtype=dt))
        np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2 * np.abs(want).max())
    else:
        bsel = {"add-matrix": biasd, "add-rows": biasd[:, :1], "add-cols": biasd[:1, :]}[ep]
        got = f32(triton_b200.matmul(ad, bd, out_dtype=dt, bias=bsel))
        np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2)
        if c["out"] == "fp16":  # same roundings: all but a few elements bit-identical (fp32 outputs
            assert (got != want).mean() < 0.02  # differ in the last bits with the summation order)
    status_ok()


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("out", ["same", "fp32"])
@pytest.mark.parametrize("M,N,K,N2", [(128, 128, 128, 128), (64, 64, 64, 64), (300, 96, 200, 128), (1000, 128, 512, 80),
                                      (5, 16, 8, 24), (4096, 128, 1024, 128)])
@pytest.mark.parametrize("layout", ["row", "transposed"])
def test_chain_dot(dtype, out, M, N, K, N2, layout):
    """out_type(in_type(out_type(A B)) W) in one launch against the oracle's restatement of the
    reference's chain-dot epilogue; ragged sizes, both operand layouts of B and W."""
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    odt = tdt if out == "same" else torch.float32
    oname = dtype if out == "same" else "fp32"
    g = torch.Generator().manual_seed(M + 3 * N + 5 * K + 7 * N2)
    a = (torch.randn(M, K, generator=g) / K ** 0.25).to(tdt)
    b = (torch.randn(K, N, generator=g) / K ** 0.25).to(tdt)
    w = (torch.randn(N, N2, generator=g) / N ** 0.5).to(tdt)
    ad = a.to(DEV)
    if layout == "row":
        bd, wd = b.to(DEV), w.to(DEV)
    else:  # [N, K] and [N2, N] storage, passed as transposed views
        bd, wd = b.t().contiguous().to(DEV).t(), w.t().contiguous().to(DEV).t()
    got = f32(triton_b200.matmul_chain(ad, bd, wd, out_dtype=odt))
    want = R.matmul_chain(f32(a), f32(b), f32(w), out=oname, storage=dtype)
    tol = 1e-2 if dtype == "fp16" else 2e-2
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol * max(1.0, np.abs(want).max()))
    # and against the same two products done by two launches of the plain matmul
    two = f32(triton_b200.matmul(triton_b200.matmul(ad, bd, out_dtype=odt).to(tdt), wd, out_dtype=odt))
    np.testing.assert_allclose(got, two, rtol=tol, atol=tol * max(1.0, np.abs(want).max()))
    status_ok()


def test_chain_dot_errors():
    a = torch.zeros(128, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="at most 128"):
        triton_b200.matmul_chain(a, torch.zeros(64, 256, dtype=torch.float16, device=DEV),
                                 torch.zeros(256, 64, dtype=torch.float16, device=DEV))
    with pytest.raises(AssertionError):
        triton_b200.matmul_chain(a, torch.zeros(64, 64, dtype=torch.float16, device=DEV),
                                 torch.zeros(32, 64, dtype=torch.float16, device=DEV))
    z = triton_b200.matmul_chain(torch.zeros(16, 0, dtype=torch.float16, device=DEV),
                                 torch.zeros(0, 32, dtype=torch.float16, device=DEV),
                                 torch.ones(32, 32, dtype=torch.float16, device=DEV))
    assert z.shape == (16, 32) and float(z.abs().max()) == 0.0
    status_ok()
