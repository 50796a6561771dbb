"""Seeded input generators shared by the golden-fixture generator and the tests.

Shapes and value distributions follow the reference's own tests for this path:
  python/tutorials/03-matrix-multiplication.py:357-359  (512x512 fp16, seed 0, randn)
  python/tutorials/06-fused-attention.py:526-531        (seed 20, N(0, 0.5) q/k/v, randn dO)
  python/test/unit/language/test_core.py:5143-5175      (fp8 e4m3 operands, fp32 result)
All tensors are produced on the CPU with torch's default generator so that the CPU
oracle and the GPU path see identical bits.
"""
import torch

MATMUL_CASES = {
    # name: shape (M, N, K), seed, optional scale / activation / b layout
    "c1_512": dict(M=512, N=512, K=512, seed=0),
    "ragged": dict(M=300, N=200, K=152, seed=1),
    "leaky": dict(M=256, N=256, K=128, seed=2, activation="leaky_relu"),
    "bT": dict(M=256, N=512, K=192, seed=3, b_transposed=True),
}

# Epilogue cases of python/test/unit/hopper/test_gemm.py (matmul_kernel with ADD_MATRIX / ADD_ROWS /
# ADD_COLS / DO_SOFTMAX).  `out`: the kernel's out_dtype.  Softmax needs BLOCK_N >= N.
EPILOGUE_CASES = {
    "add_matrix_f16": dict(M=128, N=128, K=64, seed=41, epilogue="add-matrix", out="fp16"),
    "add_rows_f16": dict(M=192, N=128, K=96, seed=42, epilogue="add-rows", out="fp16"),
    "add_cols_f32": dict(M=128, N=256, K=64, seed=43, epilogue="add-cols", out="fp32"),
    "softmax_f16": dict(M=128, N=128, K=128, seed=44, epilogue="softmax", out="fp16", scale=3.0),
    "softmax_f32": dict(M=64, N=64, K=64, seed=45, epilogue="softmax", out="fp32", scale=2.0),
    # chain-dot: BLOCK_N == N, W [N, N] (the reference's cases are M = N = K = BLOCK: test_gemm.py:269-284)
    "chain_dot_f16": dict(M=128, N=128, K=128, seed=46, epilogue="chain-dot", out="fp16", scale=4.0),
    "chain_dot_f32": dict(M=64, N=64, K=64, seed=47, epilogue="chain-dot", out="fp32", scale=4.0),
}


def epilogue_inputs(c):
    """A, B fp16 and the bias of the output type: full [M, N] matrix as in the reference test
    (add-rows reads its first column, add-cols its first row)."""
    g = torch.Generator().manual_seed(c["seed"])
    s = c.get("scale", 1.0)
    a = (torch.randn(c["M"], c["K"], generator=g) / s).half()
    b = (torch.randn(c["K"], c["N"], generator=g) / s).half()
    bias = torch.randn(c["M"], c["N"], generator=g).to(torch.float16 if c["out"] == "fp16" else torch.float32)
    return a, b, bias


def chain_weight(c):
    """W [N, N] fp16 of a chain-dot case, stored transposed as in the reference test
    (`torch.randn((N, N)).T`, test_gemm.py:386)."""
    g = torch.Generator().manual_seed(c["seed"] + 1000)
    return (torch.randn(c["N"], c["N"], generator=g) / c.get("scale", 1.0)).half().T


FP8_CASES = {
    "ref_shape": dict(M=128, N=256, K=256, seed=4),
    "k512": dict(M=256, N=512, K=512, seed=5),
}

ATTN_CASES = {
    "causal_d64": dict(Z=1, H=2, N=256, D=64, causal=True, sm_scale=0.5, dtype="fp16", bwd=True, seed=20,
                       old_style=True),
    "full_d64": dict(Z=1, H=2, N=256, D=64, causal=False, sm_scale=0.5, dtype="fp16", bwd=False, seed=21),
    "causal_d128": dict(Z=1, H=1, N=512, D=128, causal=True, sm_scale=128 ** -0.5, dtype="fp16", bwd=True,
                        seed=22, old_style=True),
    "full_d128": dict(Z=1, H=1, N=384, D=128, causal=False, sm_scale=128 ** -0.5, dtype="fp16", bwd=False,
                      seed=23),
    # bf16 has no interpreter fixture (its dot is invalid for bf16 tiles); the numpy oracle covers it
    "causal_d64_bf16": dict(Z=1, H=2, N=256, D=64, causal=True, sm_scale=0.5, dtype="bf16", bwd=True, seed=24),
}

_DT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def matmul_inputs(c, dtype=torch.float16):
    """A[M,K], B[K,N]; `scale` divides the normal samples (config 2 uses sqrt(K))."""
    g = torch.Generator().manual_seed(c["seed"])
    if c["seed"] == 0:
        # config 1 is the reference test verbatim: global seed 0, two randn calls
        torch.manual_seed(0)
        a = torch.randn((c["M"], c["K"]), dtype=torch.float32)
        b = torch.randn((c["K"], c["N"]), dtype=torch.float32)
    else:
        a = torch.randn((c["M"], c["K"]), generator=g)
        b = torch.randn((c["K"], c["N"]), generator=g)
    s = c.get("scale", 1.0)
    a = (a / s).to(dtype)
    b = (b / s).to(dtype)
    if c.get("b_transposed"):
        b = b.t().contiguous().t()  # same values, K-contiguous storage
    return a, b


def quantize_e4m3(x):
    """Per-tensor amax scaling to the e4m3 range: returns (x8, dequant scale as python float)."""
    s = 448.0 / float(x.abs().max())
    return (x * s).to(torch.float8_e4m3fn), 1.0 / s


def fp8_inputs(c):
    g = torch.Generator().manual_seed(c["seed"])
    a = torch.randn((c["M"], c["K"]), generator=g)
    b = torch.randn((c["K"], c["N"]), generator=g)
    a8, sa = quantize_e4m3(a)
    b8, sb = quantize_e4m3(b)
    return a8, b8, sa, sb


def attn_inputs(c):
    torch.manual_seed(c["seed"])
    dt = _DT[c["dtype"]]
    shape = (c["Z"], c["H"], c["N"], c["D"])
    q = torch.empty(shape, dtype=dt).normal_(mean=0.0, std=0.5)
    k = torch.empty(shape, dtype=dt).normal_(mean=0.0, std=0.5)
    v = torch.empty(shape, dtype=dt).normal_(mean=0.0, std=0.5)
    do = torch.randn(shape, dtype=torch.float32).to(dt)
    return q, k, v, do
