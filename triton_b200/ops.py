"""Host side of the hot path: the reference's op wrappers, same names and argument meaning.

  matmul(a, b, activation="")                python/tutorials/03-matrix-multiplication.py:330-348
                                             (stand-in for triton.ops.matmul(a, b),
                                              python/test/regression/test_performance.py:73)
  attention(q, k, v, causal, sm_scale)       python/tutorials/06-fused-attention.py:438-520
                                             (triton.ops.attention, test_performance.py:194)

Tensors are torch CUDA tensors (torch supplies device memory, streams and autograd
plumbing); the arithmetic is done by the library's sm_100a kernels through the C ABI.
"""
import ctypes
import os

import torch

from . import _lib

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}
if hasattr(torch, "float8_e4m3fn"):
    _DT[torch.float8_e4m3fn] = _lib.E4M3
if hasattr(torch, "float8_e5m2"):
    _DT[torch.float8_e5m2] = _lib.E5M2
_ACT = {"": _lib.ACT_NONE, None: _lib.ACT_NONE, "leaky_relu": _lib.ACT_LEAKY_RELU, "softmax": _lib.ACT_SOFTMAX}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t):
    """The current stream of the tensor's device, as the handle the C ABI takes."""
    if _raw_stream is not None:  # the call the reference's launcher uses too (driver.py:24-31); no Stream object is built
        return _raw_stream(t.device.index)
    return torch.cuda.current_stream(t.device).cuda_stream


class _on_device:
    """`with torch.cuda.device(dev)` that costs nothing when dev is already current."""

    __slots__ = ("ctx",)

    def __init__(self, dev):
        self.ctx = None if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


_plan_cache = {}  # (M, N, K, dtype, device, B200_GEMM_SPLITK) -> (splits, workspace bytes)


def _matmul_plan(M, N, K, dt):
    key = (M, N, K, dt, torch.cuda.current_device(), os.environ.get("B200_GEMM_SPLITK"))
    hit = _plan_cache.get(key)
    if hit is None:
        splits, ws_bytes = ctypes.c_int(1), ctypes.c_size_t(0)
        _lib.check(_lib.lib().b200_matmul_plan(M, N, K, dt, ctypes.byref(splits), ctypes.byref(ws_bytes)), "matmul_plan")
        hit = _plan_cache[key] = (splits.value, ws_bytes.value)
        if len(_plan_cache) > 4096:
            _plan_cache.clear()
    return hit


_scale_cache = {}  # (value, device) -> 1-element fp32 tensor: a python-float scale costs one H2D copy ever


def _scale_tensor(value, dev):
    key = (value, dev.index)
    t = _scale_cache.get(key)
    if t is None:
        if len(_scale_cache) > 1024:
            _scale_cache.clear()
        t = _scale_cache[key] = torch.tensor([value], dtype=torch.float32, device=dev)
    return t


def _check_out(c, M, N, out_dtype, dev):
    """The kernel writes M rows of N elements of `out_dtype` through `c`: anything else is an
    out-of-bounds device write, so the shape, type and device must hold whatever N is."""
    assert tuple(c.shape) == (M, N) and c.dtype == out_dtype and c.device == dev and (c.stride(1) == 1 or N == 1), \
        "out= must be an [M, N] tensor of the output type on the operands' device with unit column stride"


def _require_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("triton_b200 ops take CUDA tensors; there is no CPU fallback")
    dev = ts[0].device
    for t in ts:
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    return dev


def matmul(a, b, activation="", *, scale_a=None, scale_b=None, out_dtype=None, out=None, bias=None):
    """C = act(A @ B) with fp32 accumulation.

    Same contract as the reference wrapper: `a.shape[1] == b.shape[0]`, `a` contiguous, `b`
    any 2-D tensor with one unit stride; returns a new [M, N] tensor (fp16 for fp16 inputs,
    as the reference; bf16 for bf16 and fp8 inputs unless `out_dtype` says otherwise).
    fp8-e4m3 inputs take optional per-tensor dequantisation scales (`scale_a`, `scale_b`:
    python floats or 1-element fp32 CUDA tensors) that the epilogue multiplies in.
    `out_dtype=torch.float8_e4m3fn` stores an 8-bit C (round to nearest even, saturating).
    `activation="softmax"` is the reference's 'softmax' epilogue (test_gemm.py:223-228): a softmax
    over every row of the product (N <= 256).
    `bias` is the reference's epilogue addend (test_gemm.py 'add-matrix' / 'add-rows' /
    'add-cols'): a tensor of the output type and shape [M, N], [M, 1] (one value per row) or
    [1, N] (one per column), added after the conversion to the output type.
    """
    assert a.dim() == 2 and b.dim() == 2, "matmul takes 2-D tensors"
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.is_contiguous(), "Matrix A must be contiguous"
    assert a.dtype == b.dtype, "A and B must have the same dtype"
    assert a.dtype in _DT and a.dtype != torch.float32, f"unsupported input dtype {a.dtype}"
    assert activation in _ACT, f"unknown activation {activation!r}"
    dev = _require_cuda(a, b)
    M, K = a.shape
    _, N = b.shape
    if out_dtype is None:
        out_dtype = torch.float16 if a.dtype == torch.float16 else torch.bfloat16
    with _on_device(dev):
        c = out if out is not None else torch.empty((M, N), device=dev, dtype=out_dtype)
        _check_out(c, M, N, out_dtype, dev)

        def scale_ptr(s):
            if s is None:
                return None, None
            if not torch.is_tensor(s):
                s = _scale_tensor(float(s), dev)
            assert s.dtype == torch.float32 and s.numel() == 1 and s.device == dev
            return s.data_ptr(), s

        pa, keep_a = scale_ptr(scale_a)
        pb, keep_b = scale_ptr(scale_b)
        bias_mode, bias_ptr, bias_sm, bias_sn = _lib.BIAS_NONE, None, 0, 0
        if bias is not None:
            assert bias.dim() == 2 and bias.dtype == out_dtype and bias.device == dev, "bias: 2-D, output type, same device"
            if bias.shape == (M, N):
                bias_mode = _lib.BIAS_MATRIX
            elif bias.shape == (M, 1):
                bias_mode = _lib.BIAS_ROWS
            elif bias.shape == (1, N):
                bias_mode = _lib.BIAS_COLS
            else:
                raise AssertionError(f"bias shape {tuple(bias.shape)} is not [M, N], [M, 1] or [1, N]")
            bias_ptr, bias_sm, bias_sn = bias.data_ptr(), bias.stride(0), bias.stride(1)
        # skinny problems (few tiles, long K) are split along K; the fp32 partial tiles need scratch
        splits, ws_bytes = (1, 0) if activation == "softmax" else _matmul_plan(M, N, K, _DT[a.dtype])  # the row softmax needs the whole K range in one tile
        ws = torch.empty(ws_bytes // 4, device=dev, dtype=torch.float32) if splits > 1 else None
        code = _lib.lib().b200_matmul_bias(
            _stream(a), a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K,
            a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
            _DT[a.dtype], _DT[out_dtype], _ACT[activation], pa, pb, bias_ptr, bias_mode, bias_sm, bias_sn,
            splits, ws.data_ptr() if ws is not None else None)
        _lib.check(code, "matmul")
    return c


def matmul_chain(a, b, w, *, out_dtype=None):
    """out_type( in_type(out_type(A @ B)) @ W ): the reference's 'chain-dot' epilogue
    (python/test/unit/hopper/test_gemm.py:229-232) in one launch.  a [M, K], b [K, N], w [N, N2],
    fp16 or bf16, N and N2 at most 128 (a row of A @ B stays in one tile, as with the reference's
    BLOCK_N == N); `out_dtype` fp16 / bf16 / fp32 (default: the input type)."""
    assert a.dim() == 2 and b.dim() == 2 and w.dim() == 2, "matmul_chain takes 2-D tensors"
    assert a.shape[1] == b.shape[0] and b.shape[1] == w.shape[0], "Incompatible dimensions"
    assert a.dtype == b.dtype == w.dtype and a.dtype in (torch.float16, torch.bfloat16), "fp16 or bf16 operands"
    dev = _require_cuda(a, b, w)
    M, K = a.shape
    N, N2 = w.shape
    if out_dtype is None:
        out_dtype = a.dtype
    with _on_device(dev):
        c = torch.empty((M, N2), device=dev, dtype=out_dtype)
        code = _lib.lib().b200_matmul_chain(
            _stream(a), a.data_ptr(), b.data_ptr(), w.data_ptr(), c.data_ptr(), M, N, K, N2,
            a.stride(0), a.stride(1), b.stride(0), b.stride(1), w.stride(0), w.stride(1), c.stride(0), c.stride(1),
            _DT[a.dtype], _DT[out_dtype])
        _lib.check(code, "matmul_chain")
    return c


class GroupedMatmul:
    """A prepared grouped matmul: the groups' descriptors (pointers, sizes, tensor maps) are written
    to device memory once; `run()` is one persistent launch and can be repeated while the operand
    tensors stay where they are (their values may change).  This is what the reference times as
    `triton_perf_fn` (python/tutorials/08-grouped-gemm.py:218-229: launch only, tensors prepared
    before).  `out` is the list of result tensors, rewritten by every run."""

    def __init__(self, group_A, group_B, out_dtype=None):
        assert len(group_A) == len(group_B) and len(group_A) > 0
        G = len(group_A)
        self.dev = _require_cuda(*group_A, *group_B)
        dt = group_A[0].dtype
        assert dt in (torch.float16, torch.bfloat16), "grouped matmul takes fp16 or bf16"
        self.in_dt, self.out_dtype = dt, out_dtype or dt
        self.operands = (list(group_A), list(group_B))  # kept alive: the descriptors hold their addresses
        sizes, lds, self.out = [], [], []
        with torch.cuda.device(self.dev):
            for A, B in zip(group_A, group_B):
                assert A.dim() == 2 and B.dim() == 2 and A.shape[1] == B.shape[0]
                assert A.dtype == dt and B.dtype == dt
                assert (A.stride(1) == 1 or A.shape[1] == 1) and (B.stride(1) == 1 or B.shape[1] == 1), "row-major operands"
                M, K = A.shape
                N = B.shape[1]
                C = torch.empty((M, N), device=self.dev, dtype=self.out_dtype)
                self.out.append(C)
                sizes += [M, N, K]
                lds += [A.stride(0), B.stride(0), C.stride(0)]
            L = _lib.lib()
            PtrArr, IntArr = ctypes.c_void_p * G, ctypes.c_int * (3 * G)
            self.ws = torch.empty(L.b200_grouped_matmul_workspace(G) + 128, dtype=torch.uint8, device=self.dev)
            self.ws_ptr = (self.ws.data_ptr() + 127) & ~127
            tiles = ctypes.c_int(0)
            code = L.b200_grouped_matmul_prepare(
                _stream(group_A[0]), G, PtrArr(*[t.data_ptr() for t in group_A]),
                PtrArr(*[t.data_ptr() for t in group_B]), PtrArr(*[t.data_ptr() for t in self.out]), IntArr(*sizes),
                IntArr(*lds), _DT[dt], _DT[self.out_dtype], self.ws_ptr, ctypes.byref(tiles))
            _lib.check(code, "grouped_matmul_prepare")
            self.tiles = tiles.value

    def run(self):
        with torch.cuda.device(self.dev):
            code = _lib.lib().b200_grouped_matmul_run(torch.cuda.current_stream(self.dev).cuda_stream, self.ws_ptr,
                                                      self.tiles, _DT[self.in_dt], _DT[self.out_dtype])
            _lib.check(code, "grouped_matmul_run")
        return self.out


def group_gemm_fn(group_A, group_B, out_dtype=None):
    """[A_i @ B_i for every i] in one persistent launch: the reference's grouped GEMM
    (python/tutorials/08-grouped-gemm.py:144-191, same name and argument lists): every A_i is
    [M_i, K_i] and every B_i is [K_i, N_i], row-major 2-D CUDA tensors of one 16-bit dtype; returns
    the list of new C_i (dtype of A unless `out_dtype` says otherwise).  Unlike the reference,
    sizes need not be multiples of the tile shape.  (GroupedMatmul keeps the prepared descriptors
    for repeated launches.)"""
    if len(group_A) == 0:
        assert len(group_B) == 0
        return []
    plan = GroupedMatmul(group_A, group_B, out_dtype)
    out = plan.run()
    plan.ws.record_stream(torch.cuda.current_stream(plan.dev))  # the kernel reads the descriptors after this returns
    return out


class HostMatmul:
    """C = A @ B for operands that live in (pinned) host memory: the call a host-side user of the
    matmul makes.  A is sent in row blocks and every block's product is copied back while the next
    block is on its way, so the two directions of the link and the tensor cores overlap (the product
    of a block takes a fraction of its transfer time).  B goes to the device when it is new: a call
    that passes the same host tensor, unmodified since the previous call (same storage, same torch
    version counter - the weights of a layer, say), reuses the copy already on the device.
    Device buffers and the two copy streams are kept by the object; `run` returns after enqueueing,
    the caller's current stream waits for the last copy-out."""

    def __init__(self, M, N, K, dtype=torch.float16, device="cuda", blocks=8):
        self.M, self.N, self.K = M, N, K
        self.rows = max(1, -(-M // max(1, blocks)))
        self.dev = torch.device(device)
        with torch.cuda.device(self.dev):
            self.a = torch.empty(M, K, dtype=dtype, device=self.dev)
            self.b = torch.empty(K, N, dtype=dtype, device=self.dev)
            self.c = torch.empty(M, N, dtype=dtype, device=self.dev)
            self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self._b_key = None  # (data_ptr, version, strides) of the host B whose copy self.b holds

    def run(self, a_h, b_h, c_h, activation=""):
        assert a_h.shape == (self.M, self.K) and b_h.shape == (self.K, self.N) and c_h.shape == (self.M, self.N)
        cur = torch.cuda.current_stream(self.dev)
        self.s_in.wait_stream(cur)   # earlier work that still reads the device buffers
        self.s_out.wait_stream(cur)
        b_key = (b_h.data_ptr(), b_h._version, b_h.stride())
        if b_key != self._b_key:
            with torch.cuda.stream(self.s_in):
                self.b.copy_(b_h, non_blocking=True)
            self._b_key = b_key
        for r0 in range(0, self.M, self.rows):
            r1 = min(self.M, r0 + self.rows)
            with torch.cuda.stream(self.s_in):
                self.a[r0:r1].copy_(a_h[r0:r1], non_blocking=True)
                arrived = self.s_in.record_event()
            cur.wait_event(arrived)
            matmul(self.a[r0:r1], self.b, activation, out=self.c[r0:r1], out_dtype=self.c.dtype)
            done = cur.record_event()
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                c_h[r0:r1].copy_(self.c[r0:r1], non_blocking=True)
        cur.wait_stream(self.s_out)
        return c_h


def quantize_e4m3(x):
    """Per-tensor amax scaling to the e4m3 range; returns (x8, scale) with x ~= x8 * scale.
    `scale` is a 1-element fp32 tensor on x's device (no host synchronisation)."""
    amax = x.abs().amax().float().clamp_min(1e-12)
    s = 448.0 / amax
    return (x.float() * s).to(torch.float8_e4m3fn), (1.0 / s).reshape(1)


def attention_forward(q, k, v, causal, sm_scale, return_row_max=False):
    """Forward only: returns (O, M).  M[Z,H,N] is the reference's saved statistics tensor, the
    base-2 log-sum-exp of the scores scaled by sm_scale*log2(e) (06-fused-attention.py:183-184);
    the natural-log LSE is M * ln 2.  With return_row_max=True a third tensor follows: the base-2
    row maximum of the scaled scores (what the older kernels' separate L and M are made of, see
    attention_old_forward)."""
    HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
    assert q.dim() == 4 and k.shape == q.shape and v.shape == q.shape, "q, k, v must be [Z, H, N, D] of one shape"
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
    # the reference's set; kernels exist for 64 and 128, 16 and 32 run zero-padded to 64, 256 is rejected by the library
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    fp8 = hasattr(torch, "float8_e5m2") and q.dtype == torch.float8_e5m2
    assert (q.dtype in (torch.float16, torch.bfloat16) or fp8) and k.dtype == q.dtype and v.dtype == q.dtype
    dev = _require_cuda(q, k, v)
    Z, H, N, D = q.shape
    if D in (16, 32) and not fp8:
        # head dims below the kernels' 64: zero columns change neither q k^T nor the kept columns of O
        qp, kp, vp = (torch.nn.functional.pad(t, (0, 64 - D)) for t in (q, k, v))
        o, *stats = attention_forward(qp, kp, vp, causal, sm_scale, return_row_max)
        return (o[..., :D].contiguous(), *stats)
    if fp8 and D in (16, 32):
        # the 8-bit kernels are built for head dims 64 and 128 (rows of 64 / 128 bytes); smaller head dims
        # get zero columns appended, which leave q k^T, P and the kept columns of O bit for bit what they
        # are without them
        pad8 = lambda t: torch.nn.functional.pad(t.view(torch.uint8), (0, 64 - D)).view(torch.float8_e5m2)
        o, *stats = attention_forward(pad8(q), pad8(k), pad8(v), causal, sm_scale, return_row_max)
        return (o[..., :D].contiguous(), *stats)
    with _on_device(dev):
        if fp8:
            # the reference's fp8 forward (06-fused-attention.py:609-615) is given V with the key
            # dimension contiguous; any other V is brought into that layout first
            assert D in (64, 128), "the 8-bit forward has kernels for head dims 64 and 128 (smaller ones are padded above)"
            if v.stride(2) != 1:
                v = v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)
            o = torch.empty((Z, H, N, D), device=dev, dtype=q.dtype)
        else:
            o = torch.empty_like(q)
        M = torch.empty((Z, H, N), device=dev, dtype=torch.float32)
        row_max = torch.empty((Z, H, N), device=dev, dtype=torch.float32) if return_row_max else None
        code = _lib.lib().b200_attention_fwd_stats(
            _stream(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), M.data_ptr(),
            row_max.data_ptr() if return_row_max else None, Z, H, N, D,
            _lib.strides4(q), _lib.strides4(k), _lib.strides4(v), _lib.strides4(o),
            float(sm_scale), 1 if causal else 0, _DT[q.dtype])
        _lib.check(code, "attention_fwd")
    return (o, M, row_max) if return_row_max else (o, M)


def _one_pass_default():
    """B200_ATTN_BWD_ONEPASS=1 makes the one-pass backward the default wherever it applies."""
    return os.environ.get("B200_ATTN_BWD_ONEPASS", "0") not in ("", "0")


def attention_backward(q, k, v, o, M, do, causal, sm_scale, one_pass=None):
    """dq, dk, dv.  Same checks as the reference's backward (06-fused-attention.py:478-494).

    `one_pass` (head dim 64 only): a single kernel that computes the scores, exponentials and dS
    once per (K/V block, Q block) pair and adds the partial dQ of every K/V block into an fp32
    buffer - the layout of the reference's older `sequence_parallel` backward
    (python/test/regression/test_performance.py:174, 194) - instead of the two kernels of the
    reference's current layout, which each recompute them.  About 1.6x faster; dK and dV are the
    same bits, the last bit of dQ can vary from run to run because the partials are summed in no
    fixed order.  Default: off (bitwise repeatable), or what B200_ATTN_BWD_ONEPASS says."""
    assert do.is_contiguous()
    assert q.stride() == k.stride() == v.stride() == o.stride() == do.stride()
    Z, H, N, D = q.shape
    assert N % 128 == 0
    dev = _require_cuda(q, k, v, o, do, M)
    if one_pass is None:
        one_pass = _one_pass_default()
    if D in (16, 32):  # as in attention_forward: zero-padded to the kernels' head dim 64
        qp, kp, vp, op, dop = (torch.nn.functional.pad(t, (0, 64 - D)) for t in (q, k, v, o, do))
        return tuple(g[..., :D].contiguous() for g in attention_backward(qp, kp, vp, op, M, dop, causal, sm_scale, one_pass))
    with _on_device(dev):
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        delta = torch.empty_like(M)
        ptrs = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), M.data_ptr(), delta.data_ptr())
        tail = (dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), Z, H, N, D,
                _lib.strides4(q), _lib.strides4(k), _lib.strides4(v), _lib.strides4(o), _lib.strides4(do),
                _lib.strides4(dq), _lib.strides4(dk), _lib.strides4(dv), float(sm_scale), 1 if causal else 0, _DT[q.dtype])
        L = _lib.lib()
        if D == 256:
            # head dim 256: per-head matmuls with [N, N] intermediates in scratch (see the header)
            ws = torch.empty(L.b200_attention_bwd_wide_workspace(N) + 256, dtype=torch.uint8, device=dev)
            code = L.b200_attention_bwd_wide(_stream(q), *ptrs, *tail, (ws.data_ptr() + 255) & ~255)
        elif one_pass and D == 64:
            acc = torch.empty(L.b200_attention_bwd_onepass_workspace(Z, H, N, D) // 4, dtype=torch.float32, device=dev)
            code = L.b200_attention_bwd_onepass(_stream(q), *ptrs, acc.data_ptr(), *tail)
        else:
            code = L.b200_attention_bwd(_stream(q), *ptrs, *tail)
        _lib.check(code, "attention_bwd")
    return dq, dk, dv


class _attention(torch.autograd.Function):
    """Mirror of the reference's autograd wrapper (06-fused-attention.py:438-520)."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, sequence_parallel=False):
        o, M = attention_forward(q, k, v, causal, sm_scale)
        ctx.save_for_backward(q, k, v, o, M)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.sequence_parallel = sequence_parallel
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, M = ctx.saved_tensors
        one_pass = True if (ctx.sequence_parallel and q.shape[-1] == 64) else None
        dq, dk, dv = attention_backward(q, k, v, o, M, do.contiguous() if not do.is_contiguous() else do,
                                        ctx.causal, ctx.sm_scale, one_pass)
        return dq, dk, dv, None, None, None


def attention(q, k, v, causal, sm_scale, sequence_parallel=False):
    """O = softmax(Q K^T * sm_scale [causal]) V, differentiable: the reference's
    `attention = _attention.apply` (06-fused-attention.py:520).  The sixth argument is the older
    `triton.ops.attention(q, k, v, causal, sm_scale, sequence_parallel)` signature
    (python/test/regression/test_performance.py:194): with it the backward forms partial dQ per
    K/V block and sums them, which here is the one-pass backward kernel (head dim 64; other head
    dims run the two-kernel backward either way)."""
    return _attention.apply(q, k, v, causal, sm_scale, sequence_parallel)


# ---------------------------------------------------------------------------------------------
# The reference's older flash attention (python/test/unit/hopper/test_flashattention.py:294-358):
# `attention(q, k, v, sm_scale)`, always causal, statistics kept as two tensors L and M.
_LN2 = 0.6931471805599453


def attention_old_forward(q, k, v, sm_scale):
    """(O, L, M) of the older forward kernel (test_flashattention.py:36-131): M[Z*H, N] is the row
    maximum of q.k * sm_scale over the causal range and L[Z*H, N] the row sum of exp(score - M)
    (:128-131, natural base).  The same kernel as attention_forward computes them: it returns the
    base-2 log-sum-exp and the base-2 row maximum, and L = 2^(lse2 - max2), M = max2 * ln 2."""
    assert q.shape[-1] == k.shape[-1] == v.shape[-1] and q.shape[-1] in {16, 32, 64, 128}  # :301-303
    o, lse2, max2 = attention_forward(q, k, v, True, sm_scale, return_row_max=True)
    Z, H, N, _ = q.shape
    L = torch.exp2(lse2 - max2).reshape(Z * H, N)
    M = (max2 * _LN2).reshape(Z * H, N)
    return o, L, M


class _attention_old(torch.autograd.Function):
    """Mirror of the older autograd wrapper (test_flashattention.py:294-358): saves
    (q, k, v, o, L, m) as it does; the backward rebuilds the base-2 log-sum-exp from L and m."""

    @staticmethod
    def forward(ctx, q, k, v, sm_scale):
        o, L, m = attention_old_forward(q, k, v, sm_scale)
        ctx.save_for_backward(q, k, v, o, L, m)
        ctx.sm_scale = sm_scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, L, m = ctx.saved_tensors
        Z, H, N, _ = q.shape
        lse2 = ((m + torch.log(L)) * (1.0 / _LN2)).reshape(Z, H, N)
        dq, dk, dv = attention_backward(q, k, v, o, lse2, do.contiguous(), True, ctx.sm_scale)
        return dq, dk, dv, None


def attention_old(q, k, v, sm_scale):
    """The four-argument `attention = _attention.apply` of test_flashattention.py:358: causal
    attention, differentiable with respect to q, k and v."""
    return _attention_old.apply(q, k, v, sm_scale)
