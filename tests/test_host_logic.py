"""Host-side logic that needs no GPU: wrapper argument checks (the reference's asserts) and the
shard / gather arithmetic of the multi-GPU path, exercised with two gloo ranks on the CPU."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import triton_b200
from triton_b200 import dist as tdist


def test_matmul_asserts_match_reference_wrapper():
    a = torch.zeros(4, 8, dtype=torch.float16)
    b = torch.zeros(4, 8, dtype=torch.float16)
    with pytest.raises(AssertionError, match="Incompatible dimensions"):
        triton_b200.matmul(a, b)
    with pytest.raises(AssertionError, match="contiguous"):
        triton_b200.matmul(torch.zeros(8, 4, dtype=torch.float16).t(), torch.zeros(8, 4, dtype=torch.float16))
    with pytest.raises(AssertionError):
        triton_b200.matmul(torch.zeros(4, 8), torch.zeros(8, 4))  # fp32 inputs are not a dtype of this path
    with pytest.raises(AssertionError, match="activation"):
        triton_b200.matmul(a, b.t(), activation="gelu")


def test_out_tensor_is_checked_for_every_n():
    """A wrong-shape or wrong-type `out=` must be refused also when N == 1 (where a column
    stride other than 1 is allowed): the kernel would write M rows through it."""
    from triton_b200.ops import _check_out
    cpu = torch.device("cpu")
    _check_out(torch.zeros(5, 1, dtype=torch.float16), 5, 1, torch.float16, cpu)
    _check_out(torch.zeros(5, 2, dtype=torch.float16)[:, :1], 5, 1, torch.float16, cpu)  # N == 1: any column stride
    with pytest.raises(AssertionError):
        _check_out(torch.zeros(3, 1, dtype=torch.float16), 5, 1, torch.float16, cpu)  # too few rows
    with pytest.raises(AssertionError):
        _check_out(torch.zeros(5, 1, dtype=torch.float32), 5, 1, torch.float16, cpu)  # wrong type
    with pytest.raises(AssertionError):
        _check_out(torch.zeros(5, 8, dtype=torch.float16)[:, ::2], 5, 4, torch.float16, cpu)  # strided columns
    with pytest.raises(AssertionError):
        _check_out(torch.zeros(5, 4, dtype=torch.float16, device="meta"), 5, 4, torch.float16, cpu)  # other device


def test_attention_asserts_match_reference_wrapper():
    q = torch.zeros(1, 2, 128, 64, dtype=torch.float16)
    k = torch.zeros(1, 2, 128, 32, dtype=torch.float16)
    with pytest.raises(AssertionError):
        triton_b200.attention_forward(q, k, q, True, 0.5)
    q48 = torch.zeros(1, 2, 128, 48, dtype=torch.float16)
    with pytest.raises(AssertionError):
        triton_b200.attention_forward(q48, q48, q48, True, 0.5)


@pytest.mark.parametrize("total,world", [(8192, 8), (10, 4), (3, 8), (192, 5), (0, 2)])
def test_shard_range_partitions_exactly(total, world):
    covered = []
    for r in range(world):
        lo, hi = tdist.shard_range(total, world, r)
        assert 0 <= lo <= hi <= total
        covered += list(range(lo, hi))
    assert covered == list(range(total))
    sizes = [tdist.shard_range(total, world, r)[1] - tdist.shard_range(total, world, r)[0] for r in range(world)]
    assert max(sizes) - min(sizes) <= 1


def test_shard_rows_keeps_tile_multiples():
    a = torch.arange(1000 * 2).reshape(1000, 2)
    parts = [tdist.shard_rows(a, 3, r, multiple=128) for r in range(3)]
    assert torch.equal(torch.cat(parts), a)
    assert all(p.shape[0] % 128 == 0 for p in parts[:-1])


def test_shard_heads():
    t = torch.arange(2 * 3 * 4 * 5).reshape(2, 3, 4, 5)
    parts = [tdist.shard_heads(t, 4, r) for r in range(4)]
    assert torch.equal(torch.cat([p[0] for p in parts]), t.reshape(6, 4, 5))


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        a = torch.randn(301, 64, generator=g)
        b = torch.randn(64, 48, generator=g)
        a_local = tdist.shard_rows(a, world, rank)
        # the compute function is injected: on the GPU box it is triton_b200.matmul
        c = tdist.sharded_matmul(a_local, b, compute=torch.matmul, gather=True)
        ok = torch.allclose(c, a @ b, atol=1e-5)
        t = torch.arange(2 * 3 * 8 * 4, dtype=torch.float32).reshape(2, 3, 8, 4)
        local = tdist.shard_heads(t, world, rank)[0] * 2.0
        gathered = tdist.all_gather_rows(local)
        ok = ok and torch.equal(gathered, t.reshape(6, 8, 4) * 2.0)
        same = torch.full((3, 5), float(rank))
        both = tdist.all_gather_rows(same, equal_rows=True)
        ok = ok and torch.equal(both, torch.cat([torch.full((3, 5), float(r)) for r in range(world)]))
        q.put((rank, bool(ok), tuple(c.shape)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res)
    assert all(shape == (301, 48) for _, _, shape in res)


def test_custom_ops_are_registered_with_fake_implementations():
    """torch.ops.triton_b200.* exist in the dispatcher and trace on meta tensors (shapes and dtypes
    only, no kernel); on CPU tensors they raise: there is no CPU implementation."""
    import torch
    import triton_b200  # noqa: F401
    ns = torch.ops.triton_b200
    a = torch.empty(48, 32, dtype=torch.float16, device="meta")
    b = torch.empty(32, 80, dtype=torch.float16, device="meta")
    c = ns.matmul(a, b)
    assert c.shape == (48, 80) and c.dtype == torch.float16 and c.device.type == "meta"
    assert ns.matmul(a.to(torch.bfloat16), b.to(torch.bfloat16), "", torch.float32).dtype == torch.float32
    q = torch.empty(2, 3, 256, 64, dtype=torch.bfloat16, device="meta")
    o, M = ns.attention_fwd(q, q, q, True, 0.125)
    assert o.shape == q.shape and o.dtype == q.dtype and M.shape == (2, 3, 256) and M.dtype == torch.float32
    dq, dk, dv = ns.attention_bwd(q, q, q, o, M, o, True, 0.125)
    assert dq.shape == q.shape and dk.dtype == q.dtype and dv.shape == q.shape
    o2, M2 = ns.attention(q, q, q, False, 0.5)
    assert o2.shape == q.shape
    with pytest.raises((NotImplementedError, RuntimeError)):
        ns.matmul(torch.zeros(4, 4, dtype=torch.float16), torch.zeros(4, 4, dtype=torch.float16))
