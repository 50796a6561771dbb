"""CPU oracle: a numpy restatement of the reference's tiled matmul and flash attention.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this module; it
is used by tests/, by the smoke check and by the CPU-baseline leg of the benchmark.

Every function follows, block by block, the arithmetic of one reference kernel (the
kernel text is in the reference project; citations are file:line there), executed
the way the reference's CPU path (the Triton interpreter) executes it: each program
of the launch grid is one iteration of a Python loop, a `tl.dot` on a tile is a numpy
matmul with an fp32 accumulator (python/triton/runtime/interpreter.py:542-549), and
`.to(storage dtype)` is a rounding of fp32 values.

Parity pin: tests/test_oracle.py checks every function here against fixtures that
were produced by running the reference's unmodified kernel text under the interpreter
(tests/golden/make_golden.py).  Down-casts here round to nearest even for fp16 and
bf16, which is what the reference's GPU lowering does (cvt.rn, third_party/nvidia/lib/
TritonNVIDIAGPUToLLVM/ElementwiseOpToLLVM.cpp:346,368); the interpreter truncates
fp32->bf16 and cannot run bf16 dots at all, so the bf16 mode of this oracle is
pinned through its fp16 mode (same code, only the rounding function differs).
The bias, row-softmax and chain-dot epilogues (`add_bias`, `softmax_epilogue`, `matmul_chain`) are pinned the same
way: against tests/golden/epilogue.npz, produced by the reference's own epilogue kernel
(python/test/unit/hopper/test_gemm.py:143-247) under the interpreter; the two 8-bit
roundings (`round_e4m3`, `round_e5m2`) are pinned bit for bit against torch's float8
conversions, which implement the same IEEE-style round-to-nearest-even with saturation.
"""
import math

import numpy as np

# ----------------------------------------------------------------------------- dtypes


def round_fp16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_bf16(x):
    """fp32 -> bf16 (round to nearest even) -> fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


ROUND = {"fp16": round_fp16, "bf16": round_bf16}


def _e4m3_table():
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            v = float("nan")
        elif e == 0:
            v = m / 8.0 * 2.0 ** -6
        else:
            v = (1 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = s * v
    return t


E4M3 = _e4m3_table()


def decode_e4m3(bits_u8):
    """OCP e4m3fn bit patterns (uint8) -> fp32."""
    return E4M3[np.asarray(bits_u8, dtype=np.uint8)]


def round_e4m3(x):
    """fp32 -> e4m3fn (round to nearest even, saturating at +-448) -> fp32: what the reference's
    `accumulator.to(tl.float8e4nv)` (python/tutorials/09-persistent-matmul.py:93-94, 208-209) lowers to on NVIDIA GPUs (cvt.rn.satfinite.e4m3x2.f32,
    third_party/nvidia/lib/TritonNVIDIAGPUToLLVM/ElementwiseOpToLLVM.cpp:214-220).  Below 448 it is
    the conversion torch implements for float8_e4m3fn, which pins it (tests/test_oracle.py)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)            # subnormals share the quantum of the smallest binade
    q = np.exp2(e - 3.0)               # 3 mantissa bits
    r = np.rint(a / q) * q             # rint: ties to even; a carry into the next binade is exact
    out = np.copysign(r, x).astype(np.float32)
    return np.where(np.isnan(x), np.float32(np.nan), out)


ROUND["e4m3"] = round_e4m3


def round_e5m2(x):
    """fp32 -> e5m2 (round to nearest even, saturating at +-57344) -> fp32: the reference's
    `p.to(tl.float8e5)` (python/tutorials/06-fused-attention.py:66-67) and its e5m2 stores,
    cvt.rn.satfinite.e5m2x2.f32 on NVIDIA GPUs; below the largest finite value it is torch's
    float8_e5m2 conversion, which pins it (tests/test_oracle.py)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), 57344.0)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -14.0)           # subnormals share the quantum of the smallest binade
    q = np.exp2(e - 2.0)               # 2 mantissa bits
    r = np.rint(a / q) * q
    out = np.copysign(r, x).astype(np.float32)
    return np.where(np.isnan(x), np.float32(np.nan), out)


ROUND["e5m2"] = round_e5m2


def add_bias(c, bias, out):
    """The reference's bias epilogues, python/test/unit/hopper/test_gemm.py:213-222: the tile is
    already converted to the output type (`z = z.to(out_dtype)`) and `z += bias` rounds again in
    that type.  `bias` broadcasts: [M, N] ('add-matrix'), [M, 1] ('add-rows'), [1, N] ('add-cols')."""
    rnd = ROUND.get(out, lambda v: v)
    return rnd(rnd(c) + np.asarray(bias, dtype=np.float32))


# ----------------------------------------------------------------------------- matmul


def matmul_tile_origin(M, N, pid, BM=128, BN=256, GROUP_M=8):
    """(row, column) of the first element of program `pid`'s tile: the grouped ordering of
    python/tutorials/03-matrix-multiplication.py:265-273."""
    num_pid_m, num_pid_n = -(-M // BM), -(-N // BN)
    num_pid_in_group = GROUP_M * num_pid_n
    group_id = pid // num_pid_in_group
    first_pid_m = group_id * GROUP_M
    group_size_m = min(num_pid_m - first_pid_m, GROUP_M)
    pid_m = first_pid_m + ((pid % num_pid_in_group) % group_size_m)
    pid_n = (pid % num_pid_in_group) // group_size_m
    return pid_m * BM, pid_n * BN


def matmul(a, b, activation="", out="fp16", BM=128, BN=256, BK=64, GROUP_M=8, bias=None, pids=None):
    """C = A @ B, tile by tile.

    Follows matmul_kernel, python/tutorials/03-matrix-multiplication.py:241-316:
    grouped program-id ordering (:265-273), row/column offsets wrapped modulo M / N
    (:282-283), K loop with zero fill past K and an fp32 accumulator (:293-303),
    optional leaky_relu (:306-307, 320-322), one rounding to the output type (:308),
    store masked to M x N (:312-316).  `a`, `b` are fp32 arrays holding values that are
    exact in the storage type.  `pids`: run only these programs of the launch grid (the other
    tiles of the result stay zero; matmul_tile_origin says where a program's tile lies).
    """
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2, "Incompatible dimensions"
    c = np.zeros((M, N), dtype=np.float32)
    num_pid_m, num_pid_n = -(-M // BM), -(-N // BN)
    num_pid_in_group = GROUP_M * num_pid_n
    for pid in (range(num_pid_m * num_pid_n) if pids is None else pids):
        group_id = pid // num_pid_in_group
        first_pid_m = group_id * GROUP_M
        group_size_m = min(num_pid_m - first_pid_m, GROUP_M)
        pid_m = first_pid_m + ((pid % num_pid_in_group) % group_size_m)
        pid_n = (pid % num_pid_in_group) // group_size_m
        offs_am = (pid_m * BM + np.arange(BM)) % M
        offs_bn = (pid_n * BN + np.arange(BN)) % N
        full = pid_m * BM + BM <= M and pid_n * BN + BN <= N
        arows = a[pid_m * BM:pid_m * BM + BM] if full else a[offs_am]
        bcols = b[:, pid_n * BN:pid_n * BN + BN] if full else b[:, offs_bn]
        acc = np.zeros((BM, BN), dtype=np.float32)
        for k0 in range(0, K, BK):
            acc = np.matmul(arows[:, k0:k0 + BK], bcols[k0:k0 + BK], dtype=np.float32) + acc
        if activation == "leaky_relu":
            acc = np.where(acc >= 0, acc, np.float32(0.01) * acc)
        m0, n0 = pid_m * BM, pid_n * BN
        mm, nn = min(BM, M - m0), min(BN, N - n0)
        c[m0:m0 + mm, n0:n0 + nn] = acc[:mm, :nn]
    if bias is not None:
        return add_bias(c, bias, out)
    if activation == "softmax":
        return softmax_epilogue(c, out)
    return ROUND[out](c) if out in ROUND else c


def softmax_epilogue(c, out):
    """The 'softmax' epilogue of python/test/unit/hopper/test_gemm.py:223-228 on the fp32 product:
    z = c.to(out); z = z - max(z, 1); num = exp(z.to(fp32)).to(out); den = sum(num, 1);
    z = num / den, every step rounded to the output type (the row sum is accumulated in fp32 and
    rounded once)."""
    rnd = ROUND.get(out, lambda v: np.asarray(v, dtype=np.float32))
    z = rnd(c)
    z = rnd(z - z.max(axis=1, keepdims=True))
    num = rnd(np.exp(z, dtype=np.float32))
    den = rnd(num.sum(axis=1, keepdims=True, dtype=np.float32))
    return rnd(num / den)


def matmul_chain(a, b, w, out="fp16", storage="fp16", BM=128, BK=64):
    """The 'chain-dot' epilogue of python/test/unit/hopper/test_gemm.py:229-232 after the K loop of
    :205-210: z = (A @ B in fp32).to(out); z = dot(z.to(w.dtype), w) in fp32; z = z.to(out).
    BLOCK_N is N (the reference's condition for this epilogue, :187), so a program owns BM whole
    rows; `storage` is the operands' type."""
    a, b, w = (np.asarray(t, dtype=np.float32) for t in (a, b, w))
    M, K = a.shape
    N = b.shape[1]
    rnd_out = ROUND.get(out, lambda v: np.asarray(v, dtype=np.float32))
    c = np.zeros((M, w.shape[1]), dtype=np.float32)
    for m0 in range(0, M, BM):
        acc = np.zeros((min(BM, M - m0), N), dtype=np.float32)
        for k0 in range(0, K, BK):
            acc = np.matmul(a[m0:m0 + BM, k0:k0 + BK], b[k0:k0 + BK], dtype=np.float32) + acc
        z = ROUND[storage](rnd_out(acc))
        c[m0:m0 + BM] = rnd_out(np.matmul(z, w, dtype=np.float32))
    return c


def matmul_fp8(a_bits, b_bits, scale_a=None, scale_b=None, out="bf16", BM=128, BN=256, BK=128, pids=None):
    """e4m3 x e4m3 -> fp32 accumulator -> (acc * scale_a * scale_b) -> `out`.

    The accumulator part follows the fp8 matmul_kernel of
    python/test/unit/language/test_core.py:5110-5140 (column-major program order,
    unmasked loads so M, N, K must divide the tile, fp32 store); the interpreter widens
    fp8 operands before the product (interpreter.py:545-548), as done here.  The scale
    epilogue has no reference kernel; it is one fp32 multiply by (scale_a*scale_b) and
    one rounding.  out="fp32" with no scales returns the accumulator itself.  `pids`: run only
    these programs (tile of program pid: rows (pid % (M/BM)) * BM, columns (pid // (M/BM)) * BN).
    """
    a = decode_e4m3(a_bits)
    b = decode_e4m3(b_bits)
    M, K = a.shape
    N = b.shape[1]
    BM, BN, BK = min(BM, M), min(BN, N), min(BK, K)
    assert M % BM == 0 and N % BN == 0 and K % BK == 0
    c = np.zeros((M, N), dtype=np.float32)
    num_pid_m = M // BM
    for pid in (range(num_pid_m * (N // BN)) if pids is None else pids):
        pid_m, pid_n = pid % num_pid_m, pid // num_pid_m
        acc = np.zeros((BM, BN), dtype=np.float32)
        for k0 in range(0, K, BK):
            acc = np.matmul(a[pid_m * BM:(pid_m + 1) * BM, k0:k0 + BK],
                            b[k0:k0 + BK, pid_n * BN:(pid_n + 1) * BN], dtype=np.float32) + acc
        c[pid_m * BM:(pid_m + 1) * BM, pid_n * BN:(pid_n + 1) * BN] = acc
    if scale_a is not None:
        c = c * np.float32(np.float32(scale_a) * np.float32(scale_b))
    return ROUND[out](c) if out in ROUND else c


# -------------------------------------------------------------------------- attention


def _fwd_inner(acc, l_i, m_i, q, k, v, start_m, qk_scale, BM, BN, stage, offs_m, N_CTX, rnd):
    """_attn_fwd_inner, python/tutorials/06-fused-attention.py:25-75."""
    if stage == 1:
        lo, hi = 0, start_m * BM
    elif stage == 2:
        lo, hi = start_m * BM, (start_m + 1) * BM
    else:
        lo, hi = 0, N_CTX
    for start_n in range(lo, hi, BN):
        kb = k[start_n:start_n + BN]
        qk = np.matmul(q, kb.T, dtype=np.float32)
        if stage == 2:
            mask = offs_m[:, None] >= (start_n + np.arange(BN))[None, :]
            qk = qk * qk_scale + np.where(mask, np.float32(0), np.float32(-1.0e6))
            m_ij = np.maximum(m_i, qk.max(axis=1))
            qk = qk - m_ij[:, None]
        else:
            m_ij = np.maximum(m_i, qk.max(axis=1) * qk_scale)
            qk = qk * qk_scale - m_ij[:, None]
        p = np.exp2(qk, dtype=np.float32)
        l_ij = p.sum(axis=1, dtype=np.float32)
        alpha = np.exp2(m_i - m_ij, dtype=np.float32)
        l_i = l_i * alpha + l_ij
        acc = acc * alpha[:, None]
        acc = np.matmul(rnd(p), v[start_n:start_n + BN], dtype=np.float32) + acc
        m_i = m_ij
    return acc, l_i, m_i


def attention_fwd(q, k, v, causal, sm_scale, dtype="fp16", BM=128, BN=64):
    """O, M = attention forward.

    Follows _attn_fwd, python/tutorials/06-fused-attention.py:98-187: one program per
    (128-row Q block, batch*head); m=-inf, l=1, acc=0 (:156-158); qk_scale =
    sm_scale*1.44269504 (:160-161); causal runs the off-band stage then the diagonal
    stage (:166-181); M = m + log2(l), O = acc / l rounded to the storage type
    (:183-187).  q, k, v: fp32 arrays [Z,H,N,D] with values exact in `dtype`.
    Returns O (fp32 values exact in `dtype`) and M[Z,H,N] fp32 (base-2 log-sum-exp).
    """
    rnd = ROUND[dtype]
    Z, H, N, D = q.shape
    o = np.zeros_like(q, dtype=np.float32)
    Mout = np.zeros((Z, H, N), dtype=np.float32)
    qk_scale = np.float32(np.float32(sm_scale) * np.float32(1.44269504))
    for z in range(Z):
        for h in range(H):
            qq, kk, vv = q[z, h], k[z, h], v[z, h]
            for start_m in range(-(-N // BM)):
                offs_m = start_m * BM + np.arange(BM)
                m_i = np.full(BM, -np.inf, dtype=np.float32)
                l_i = np.ones(BM, dtype=np.float32)
                acc = np.zeros((BM, D), dtype=np.float32)
                qb = qq[start_m * BM:(start_m + 1) * BM]
                if causal:
                    acc, l_i, m_i = _fwd_inner(acc, l_i, m_i, qb, kk, vv, start_m, qk_scale, BM, BN, 1, offs_m, N, rnd)
                    acc, l_i, m_i = _fwd_inner(acc, l_i, m_i, qb, kk, vv, start_m, qk_scale, BM, BN, 2, offs_m, N, rnd)
                else:
                    acc, l_i, m_i = _fwd_inner(acc, l_i, m_i, qb, kk, vv, start_m, qk_scale, BM, BN, 3, offs_m, N, rnd)
                m_i = m_i + np.log2(l_i)
                acc = acc / l_i[:, None]
                Mout[z, h, start_m * BM:(start_m + 1) * BM] = m_i
                o[z, h, start_m * BM:(start_m + 1) * BM] = rnd(acc)
    return o, Mout


def attention_bwd_preprocess(o, do):
    """delta = rowsum(O * dO) in fp32 (_attn_bwd_preprocess, 06-fused-attention.py:190-204)."""
    return (np.asarray(o, np.float32) * np.asarray(do, np.float32)).sum(axis=-1, dtype=np.float32)


def _bwd_dkdv(dk, dv, q, k, v, do, M, delta, start_n, start_m, num_steps, BM1, BN1, mask, rnd):
    """_attn_bwd_dkdv, 06-fused-attention.py:208-257 (k is the pre-scaled K)."""
    offs_n = start_n + np.arange(BN1)
    curr_m = start_m
    for _ in range(num_steps):
        offs_m = curr_m + np.arange(BM1)
        qT = q[curr_m:curr_m + BM1].T
        m = M[curr_m:curr_m + BM1]
        qkT = np.matmul(k, qT, dtype=np.float32)
        pT = np.exp2(qkT - m[None, :], dtype=np.float32)
        if mask:
            pT = np.where(offs_m[None, :] >= offs_n[:, None], pT, np.float32(0))
        dob = do[curr_m:curr_m + BM1]
        dv = np.matmul(rnd(pT), dob, dtype=np.float32) + dv
        Di = delta[curr_m:curr_m + BM1]
        dpT = np.matmul(v, dob.T, dtype=np.float32)
        dsT = rnd(pT * (dpT - Di[None, :]))
        dk = np.matmul(dsT, qT.T, dtype=np.float32) + dk
        curr_m += BM1
    return dk, dv


def _bwd_dq(dq, q, k, v, do, m, Di, start_m, start_n, num_steps, BM2, BN2, mask, rnd):
    """_attn_bwd_dq, 06-fused-attention.py:261-305 (k is the pre-scaled K)."""
    offs_m = start_m + np.arange(BM2)
    curr_n = start_n
    for _ in range(num_steps):
        kT = k[curr_n:curr_n + BN2].T
        vT = v[curr_n:curr_n + BN2].T
        qk = np.matmul(q, kT, dtype=np.float32)
        p = np.exp2(qk - m[:, None], dtype=np.float32)
        if mask:
            offs_n = curr_n + np.arange(BN2)
            p = np.where(offs_m[:, None] >= offs_n[None, :], p, np.float32(0))
        dp = np.matmul(do, vT, dtype=np.float32)
        ds = rnd(p * (dp - Di[:, None]))
        dq = np.matmul(ds, kT.T, dtype=np.float32) + dq
        curr_n += BN2
    return dq


def attention_bwd(q, k, v, o, do, M, sm_scale, dtype="fp16"):
    """dQ, dK, dV for CAUSAL attention.

    Follows _attention.backward and _attn_bwd, 06-fused-attention.py:478-517, 308-435:
    K is pre-multiplied by sm_scale/ln2 and rounded to the storage type on the host
    (:491-492); per 128-row K/V block the diagonal is walked in masked 16-row Q slices
    and the rest in 32-row Q blocks (:362-391), dK is scaled by sm_scale at the end
    (:397); per 128-row Q block the diagonal is walked in masked 16-column slices and
    the earlier columns in 32-column blocks (:416-430), dQ is scaled by ln2 (:433).
    The reference's backward applies the causal mask whatever `causal` was in forward.
    """
    rnd = ROUND[dtype]
    Z, H, N, D = q.shape
    BM1, BN1, BM2, BN2, SLICE = 32, 128, 128, 32, 2
    LN2 = np.float32(0.6931471824645996)
    RCP_LN2 = 1.4426950408889634
    assert N % 128 == 0
    arg_k = rnd(np.asarray(k, np.float32) * np.float32(sm_scale * RCP_LN2))
    delta = attention_bwd_preprocess(o, do)
    dq = np.zeros_like(q, dtype=np.float32)
    dk = np.zeros_like(q, dtype=np.float32)
    dv = np.zeros_like(q, dtype=np.float32)
    for z in range(Z):
        for h in range(H):
            qq, kk, vv, dd, mm, de = q[z, h], arg_k[z, h], v[z, h], do[z, h], M[z, h], delta[z, h]
            for pid in range(N // BN1):
                start_n = pid * BN1
                kb, vb = kk[start_n:start_n + BN1], vv[start_n:start_n + BN1]
                dvb = np.zeros((BN1, D), np.float32)
                dkb = np.zeros((BN1, D), np.float32)
                mb = BM1 // SLICE
                steps = BN1 // mb
                dkb, dvb = _bwd_dkdv(dkb, dvb, qq, kb, vb, dd, mm, de, start_n, start_n, steps, mb, BN1, True, rnd)
                start_m = start_n + steps * mb
                steps = (N - start_m) // BM1
                dkb, dvb = _bwd_dkdv(dkb, dvb, qq, kb, vb, dd, mm, de, start_n, start_m, steps, BM1, BN1, False, rnd)
                dv[z, h, start_n:start_n + BN1] = rnd(dvb)
                dk[z, h, start_n:start_n + BN1] = rnd(dkb * np.float32(sm_scale))
                # dQ for the same 128 rows
                start_m = pid * BM2
                end_n = start_m + BM2
                nb = BN2 // SLICE
                qb, dob = qq[start_m:start_m + BM2], dd[start_m:start_m + BM2]
                m_rows, d_rows = mm[start_m:start_m + BM2], de[start_m:start_m + BM2]
                dqb = np.zeros((BM2, D), np.float32)
                steps = BM2 // nb
                dqb = _bwd_dq(dqb, qb, kk, vv, dob, m_rows, d_rows, start_m, end_n - steps * nb, steps, BM2, nb,
                              True, rnd)
                end_n -= steps * nb
                steps = end_n // BN2
                dqb = _bwd_dq(dqb, qb, kk, vv, dob, m_rows, d_rows, start_m, end_n - steps * BN2, steps, BM2, BN2,
                              False, rnd)
                dq[z, h, start_m:start_m + BM2] = rnd(dqb * LN2)
    return dq, dk, dv


def attention_bwd_full(q, k, v, o, do, M, sm_scale, causal, dtype="fp16"):
    """Dense-matrix backward with the same roundings (P and dS rounded to the storage
    type before the second products, fp32 elsewhere), for either mask.  Used for the
    non-causal backward, which the reference's kernel does not implement (its backward
    always masks); for causal inputs it agrees with `attention_bwd` to rounding noise.
    """
    rnd = ROUND[dtype]
    Z, H, N, D = q.shape
    scale2 = np.float32(sm_scale * 1.4426950408889634)
    delta = attention_bwd_preprocess(o, do)
    dq = np.zeros_like(q, dtype=np.float32)
    dk = np.zeros_like(q, dtype=np.float32)
    dv = np.zeros_like(q, dtype=np.float32)
    tri = np.tril(np.ones((N, N), dtype=bool))
    for z in range(Z):
        for h in range(H):
            s = np.matmul(q[z, h], k[z, h].T, dtype=np.float32) * scale2
            p = np.exp2(s - M[z, h][:, None], dtype=np.float32)
            if causal:
                p = np.where(tri, p, np.float32(0))
            dv[z, h] = rnd(np.matmul(rnd(p).T, do[z, h], dtype=np.float32))
            dp = np.matmul(do[z, h], v[z, h].T, dtype=np.float32)
            ds = rnd(p * (dp - delta[z, h][:, None]))
            dq[z, h] = rnd(np.matmul(ds, k[z, h], dtype=np.float32) * np.float32(sm_scale))
            dk[z, h] = rnd(np.matmul(ds.T, q[z, h], dtype=np.float32) * np.float32(sm_scale))
    return dq, dk, dv


# ------------------------------------------------------------------------------ flops


def matmul_flops(M, N, K):
    """2*M*N*K (python/tutorials/03-matrix-multiplication.py:437)."""
    return 2.0 * M * N * K


def attention_flops(Z, H, N, D, causal, mode="fwd"):
    """python/tutorials/06-fused-attention.py:630-636: two matmuls of 2*Z*H*N*N*D,
    halved when causal, times 2.5 for backward (2.0 backward + 0.5 recompute)."""
    total = 2 * (2.0 * Z * H * N * N * D)
    if causal:
        total *= 0.5
    if mode == "bwd":
        total *= 2.5
    return total
