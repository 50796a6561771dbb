"""Generate the golden fixtures in this directory from the reference's own kernels.

The reference's hot-path kernels are Python source written in the `tl` DSL.  This
script loads their text at run time from a checkout of the reference (argument
--reference or the environment variable TRITON_REFERENCE), executes them on
the CPU through the Triton interpreter (TRITON_INTERPRET=1, the pip `triton` package
is the executor), and stores the outputs as small .npz fixtures.  Nothing of the
reference is copied into this repository: only numeric outputs are written.

Kernels used (paths inside the reference project):
  python/tutorials/03-matrix-multiplication.py   matmul_kernel, leaky_relu
  python/test/unit/language/test_core.py         matmul_kernel (fp8 in, fp32 out)
  python/test/unit/hopper/test_gemm.py           matmul_kernel (bias and softmax epilogues)
  python/tutorials/06-fused-attention.py         _attn_fwd*, _attn_bwd*, _attention
  python/test/unit/hopper/test_flashattention.py _fwd_kernel, _bwd_preprocess, _bwd_kernel

Module-level code of those files touches CUDA, so they are never imported: the
wanted FunctionDef / ClassDef nodes are extracted from the AST and executed in a
private namespace, and `triton.autotune` is replaced by a one-config shim because
the real autotuner times configs with CUDA events.

Inputs are not stored; they are regenerated from seeds by `cases.py` (shared with
the tests), and a SHA-256 of every input is stored so that drift of the generator is
detected instead of silently comparing different data.

Run:  python tests/golden/make_golden.py --reference /path/to/triton [--only name]
"""
import argparse
import ast
import hashlib
import os
import sys
import time

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import triton  # noqa: E402  (the interpreter executor)

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


class _OneConfig:
    """Stand-in for an autotuned kernel: always launches with one fixed config."""

    def __init__(self, fn, cfg):
        self.fn, self.cfg = fn, cfg

    def __getitem__(self, grid):
        def launch(*args, **kw):
            meta = dict(self.cfg.all_kwargs())
            meta.update(kw)
            g = grid(meta) if callable(grid) else grid
            return self.fn[g](*args, **meta)
        return launch


def _load(ref_root, rel, wanted, pick, first_lineno=None, extra_assign=()):
    path = os.path.join(ref_root, rel)
    tree = ast.parse(open(path).read())
    keep = []
    for n in tree.body:
        if isinstance(n, (ast.Import, ast.ImportFrom)):
            if isinstance(n, ast.ImportFrom) and n.module and "pytest" in n.module:
                continue
            keep.append(n)
        elif isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in wanted:
            if first_lineno and n.name in first_lineno and n.lineno != first_lineno[n.name]:
                continue
            keep.append(n)
        elif isinstance(n, ast.Assign) and len(n.targets) == 1 and isinstance(n.targets[0], ast.Name) \
                and n.targets[0].id in extra_assign:
            keep.append(n)
    keep.sort(key=lambda n: n.lineno)
    ns = {"is_hip": lambda: False, "is_cuda": lambda: True, "__file__": path, "__name__": "ref_kernels"}
    real_autotune = triton.autotune
    triton.autotune = lambda configs, key=None, **kw: (lambda fn: _OneConfig(fn, pick(list(configs))))
    try:
        exec(compile(ast.Module(keep, []), path, "exec"), ns)
    finally:
        triton.autotune = real_autotune
    return ns


def sha(t):
    if isinstance(t, torch.Tensor):
        t = t.contiguous().view(torch.uint8).numpy()
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()


def _find_lineno(ref_root, rel, name, nth_last=True):
    tree = ast.parse(open(os.path.join(ref_root, rel)).read())
    lines = [n.lineno for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name]
    return lines


def gen_matmul(ref_root, out):
    ns = _load(ref_root, "python/tutorials/03-matrix-multiplication.py", {"matmul_kernel", "leaky_relu",
               "get_autotune_config", "get_cuda_autotune_config", "get_hip_autotune_config"},
               pick=lambda cfgs: cfgs[0])
    kern = ns["matmul_kernel"]
    for name, c in cases.MATMUL_CASES.items():
        a, b = cases.matmul_inputs(c)
        M, K = a.shape
        N = b.shape[1]
        cc = torch.empty((M, N), dtype=torch.float16)
        t0 = time.time()
        grid = lambda META: (triton.cdiv(M, META["BLOCK_SIZE_M"]) * triton.cdiv(N, META["BLOCK_SIZE_N"]),)
        kern[grid](a, b, cc, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), cc.stride(0),
                   cc.stride(1), ACTIVATION=c.get("activation", ""))
        print(f"matmul {name}: {time.time()-t0:.2f}s")
        out[f"matmul.{name}.c"] = cc.numpy()
        out[f"matmul.{name}.sha_a"] = np.array(sha(a))
        out[f"matmul.{name}.sha_b"] = np.array(sha(b))


def gen_fp8(ref_root, out):
    rel = "python/test/unit/language/test_core.py"
    # several functions in that file are called matmul_kernel; the fp8 one is the last module-level one
    lines = _find_lineno(ref_root, rel, "matmul_kernel")
    ns = _load(ref_root, rel, {"matmul_kernel"}, pick=lambda c: c[0], first_lineno={"matmul_kernel": lines[-1]})
    kern = ns["matmul_kernel"]
    import triton.language as tl
    for name, c in cases.FP8_CASES.items():
        a8, b8, sa, sb = cases.fp8_inputs(c)
        M, K = a8.shape
        N = b8.shape[1]
        cc = torch.empty((M, N), dtype=torch.float32)
        BM, BN, BK = c.get("tile", (128, 256, 128))
        grid = (triton.cdiv(M, BM) * triton.cdiv(N, BN), 1)
        ta = triton.reinterpret(a8.view(torch.uint8), tl.float8e4nv)
        tb = triton.reinterpret(b8.view(torch.uint8), tl.float8e4nv)
        t0 = time.time()
        kern[grid](ta, tb, cc, M, N, K, a8.stride(0), a8.stride(1), b8.stride(0), b8.stride(1), cc.stride(0),
                   cc.stride(1), BM, BN, BK, 0)
        print(f"fp8 {name}: {time.time()-t0:.2f}s")
        # the fp32 accumulator is the kernel's output; the per-tensor scale epilogue is host arithmetic
        out[f"fp8.{name}.acc"] = cc.numpy()
        out[f"fp8.{name}.sha_a"] = np.array(sha(a8))
        out[f"fp8.{name}.sha_b"] = np.array(sha(b8))
        out[f"fp8.{name}.scales"] = np.array([float(sa), float(sb)], dtype=np.float32)


def gen_epilogue(ref_root, out):
    """matmul_kernel of python/test/unit/hopper/test_gemm.py:143-247 with its bias / softmax epilogues
    (block-pointer loads, plain masked store)."""
    import triton.language as tl
    ns = _load(ref_root, "python/test/unit/hopper/test_gemm.py", {"matmul_kernel"}, pick=lambda c: c[0])
    kern = ns["matmul_kernel"]
    for name, c in cases.EPILOGUE_CASES.items():
        a, b, bias = cases.epilogue_inputs(c)
        M, K = a.shape
        N = b.shape[1]
        odt = torch.float16 if c["out"] == "fp16" else torch.float32
        z = torch.full((M, N), 1.0, dtype=odt)
        ep = c["epilogue"]
        w = cases.chain_weight(c) if ep == "chain-dot" else torch.zeros((N, N), dtype=torch.float16)
        BM, BN, BK = 64, (N if ep in ("softmax", "chain-dot") else 64), 32
        grid = (triton.cdiv(M, BM) * triton.cdiv(N, BN),)
        t0 = time.time()
        kern[grid](a_ptr=a, b_ptr=b, w_ptr=w, bias_ptr=bias, z_ptr=z, M=M, N=N, K=K,
                   stride_am=a.stride(0), stride_ak=a.stride(1), stride_bk=b.stride(0), stride_bn=b.stride(1),
                   stride_wm=w.stride(0), stride_wn=w.stride(1), stride_zm=z.stride(0), stride_zn=z.stride(1),
                   BLOCK_M=BM, BLOCK_N=BN, BLOCK_K=BK, GROUP_SIZE_M=8,
                   out_dtype=tl.float16 if c["out"] == "fp16" else tl.float32, USE_TMA_STORE=False,
                   ADD_MATRIX=ep == "add-matrix", ADD_ROWS=ep == "add-rows", ADD_COLS=ep == "add-cols",
                   DO_SOFTMAX=ep == "softmax", CHAIN_DOT=ep == "chain-dot",
                   A_ORDER_0=1, A_ORDER_1=0, B_ORDER_0=1, B_ORDER_1=0, W_ORDER_0=0, W_ORDER_1=1,
                   Z_ORDER_0=1, Z_ORDER_1=0)
        print(f"epilogue {name}: {time.time()-t0:.2f}s")
        out[f"epilogue.{name}.z"] = z.numpy()
        for nm, t in (("a", a), ("b", b), ("bias", bias)):
            out[f"epilogue.{name}.sha_{nm}"] = np.array(sha(t))


def gen_attn(ref_root, out):
    wanted = {"_attn_fwd_inner", "_attn_fwd", "_attn_bwd_preprocess", "_attn_bwd_dkdv", "_attn_bwd_dq",
              "_attn_bwd", "_attention", "keep"}
    pick = lambda cfgs: [c for c in cfgs if c.kwargs["BLOCK_M"] == 128 and c.kwargs["BLOCK_N"] == 64][0]
    ns = _load(ref_root, "python/tutorials/06-fused-attention.py", wanted, pick, extra_assign=("configs",))
    attention = ns["_attention"].apply
    for name, c in cases.ATTN_CASES.items():
        if c["dtype"] != "fp16":
            continue  # the interpreter's dot is not valid for bf16 tiles
        q, k, v, do = cases.attn_inputs(c)
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        t0 = time.time()
        o = attention(q, k, v, c["causal"], c["sm_scale"])
        # the saved statistics tensor M (base-2 log-sum-exp of the scaled scores)
        M = o.grad_fn.saved_tensors[4]
        out[f"attn.{name}.o"] = o.detach().numpy()
        out[f"attn.{name}.m"] = M.detach().numpy()
        t1 = time.time()
        if c.get("bwd"):
            o.backward(do)
            out[f"attn.{name}.dq"] = q.grad.numpy()
            out[f"attn.{name}.dk"] = k.grad.numpy()
            out[f"attn.{name}.dv"] = v.grad.numpy()
        print(f"attn {name}: fwd {t1-t0:.2f}s bwd {time.time()-t1:.2f}s")
        for nm, t in (("q", q), ("k", k), ("v", v), ("do", do)):
            out[f"attn.{name}.sha_{nm}"] = np.array(sha(t.detach()))


def gen_attn_old(ref_root, out):
    wanted = {"_fwd_kernel", "_bwd_preprocess", "_bwd_kernel", "_attention"}
    ns = _load(ref_root, "python/test/unit/hopper/test_flashattention.py", wanted, pick=lambda c: c[0])
    attention = ns["_attention"].apply
    for name, c in cases.ATTN_CASES.items():
        if c["dtype"] != "fp16" or not c["causal"] or not c.get("old_style"):
            continue
        q, k, v, do = cases.attn_inputs(c)
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        t0 = time.time()
        o = attention(q, k, v, c["sm_scale"])
        # the wrapper saves (q, k, v, o, L, m) for its backward (test_flashattention.py:323): the two
        # statistics tensors of this kernel variant, row sum L and row maximum M, [Z*H, N] fp32
        saved = o.grad_fn.saved_tensors
        out[f"attn_old.{name}.l"] = saved[4].detach().numpy().copy()
        out[f"attn_old.{name}.m"] = saved[5].detach().numpy().copy()
        o.backward(do)
        print(f"attn-old {name}: {time.time()-t0:.2f}s")
        out[f"attn_old.{name}.o"] = o.detach().numpy()
        out[f"attn_old.{name}.dq"] = q.grad.numpy()   # fp32 in this variant
        out[f"attn_old.{name}.dk"] = k.grad.numpy()
        out[f"attn_old.{name}.dv"] = v.grad.numpy()


GENS = {"matmul": gen_matmul, "fp8": gen_fp8, "epilogue": gen_epilogue, "attn": gen_attn, "attn_old": gen_attn_old}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TRITON_REFERENCE"), required=not os.environ.get("TRITON_REFERENCE"),
                    help="checkout of the reference project (or set TRITON_REFERENCE)")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    for name, fn in GENS.items():
        if args.only and name != args.only:
            continue
        out = {}
        fn(args.reference, out)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print("wrote", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
