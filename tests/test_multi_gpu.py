"""The multi-GPU use of the path on real GPUs: one process per GPU, NCCL.  The matmul is sharded by
M-row blocks and the attention by (batch, head); the only collective is the all-gather a caller
may ask for to assemble the output.  Needs two GPUs (skipped otherwise; the shard arithmetic and
the gather logic are also covered with two gloo ranks on the CPU in test_host_logic.py)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import triton_b200
        from triton_b200 import _lib
        from triton_b200 import dist as tdist
        g = torch.Generator().manual_seed(17)
        a = (torch.randn(1000, 512, generator=g) / 16).half().to(dev)   # 1000 rows: the shards differ in size
        b = (torch.randn(512, 384, generator=g) / 16).half().to(dev)
        a_local = tdist.shard_rows(a, world, rank, multiple=128)
        c = tdist.sharded_matmul(a_local.contiguous(), b, compute=triton_b200.matmul, gather=True)
        ok_mm = torch.equal(c, triton_b200.matmul(a, b))  # row blocks are independent: same bits as one GPU
        qkv = [(torch.randn(2, 3, 256, 64, generator=g) * 0.5).half().to(dev) for _ in range(3)]
        o_full, m_full = triton_b200.attention_forward(*qkv, True, 0.125)
        ql, kl, vl = (tdist.shard_heads(t, world, rank).contiguous() for t in qkv)
        o_l, m_l = triton_b200.attention_forward(ql, kl, vl, True, 0.125)
        o = tdist.all_gather_rows(o_l[0])   # [heads of this rank, N, D] -> all (batch, head) pairs
        ok_at = torch.equal(o, o_full.reshape(6, 256, 64))
        q.put((rank, bool(ok_mm), bool(ok_at), tuple(c.shape), _lib.status()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_nccl_shard_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok_mm, ok_at, shape, status in res:
        assert ok_mm, f"rank {rank}: gathered matmul differs from the single-GPU result"
        assert ok_at, f"rank {rank}: gathered attention output differs from the single-GPU result"
        assert shape == (1000, 384) and status == 0
