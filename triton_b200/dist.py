"""Multi-GPU use of the hot path: one process per GPU, independent shards, no data-path collective.

The path shards naturally: a matmul by M-row blocks (every rank holds all of B), attention
by (batch, head) pairs.  Each rank runs the single-GPU kernels on its shard; a collective
(all-gather over NCCL / NVLink) is issued only when a caller asks for the assembled output
on every rank.  The reference has no multi-device code at all; this module is the
partition arithmetic plus that optional gather.
"""
import torch
import torch.distributed as dist


def shard_range(total, world_size, rank):
    """[start, stop) of `total` units for `rank`: contiguous, sizes differ by at most one,
    earlier ranks take the larger shards."""
    assert 0 <= rank < world_size
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(a, world_size, rank, multiple=1):
    """Row block of `a` for `rank`; `multiple` keeps shard boundaries on tile multiples."""
    units = -(-a.shape[0] // multiple)
    lo, hi = shard_range(units, world_size, rank)
    return a[lo * multiple:min(hi * multiple, a.shape[0])]


def shard_heads(t, world_size, rank):
    """(batch*head) slice of a [Z, H, N, D] tensor as a [1, n_local, N, D] view."""
    Z, H, N, D = t.shape
    flat = t.reshape(Z * H, N, D)
    lo, hi = shard_range(Z * H, world_size, rank)
    return flat[lo:hi].unsqueeze(0)


def sharded_matmul(a_local, b, compute, gather=False, group=None):
    """C_local = compute(a_local, b); with gather=True returns the row-concatenation over ranks
    (ranks may hold different row counts)."""
    c_local = compute(a_local, b)
    if not gather:
        return c_local
    return all_gather_rows(c_local, group)


def all_gather_rows(x, group=None, equal_rows=False):
    """Concatenate `x` (leading dimension may differ per rank) over the ranks of `group`.
    equal_rows=True: the caller knows that every rank holds the same number of rows; one collective
    into the assembled tensor, no size exchange and no host synchronisation."""
    world = dist.get_world_size(group)
    if world == 1:
        return x
    if equal_rows:
        out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out
    n_local = torch.tensor([x.shape[0]], dtype=torch.int64, device=x.device)
    sizes = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(sizes, n_local, group=group)
    sizes = [int(s.item()) for s in sizes]
    nmax = max(sizes)
    pad = x
    if x.shape[0] != nmax:
        pad = torch.zeros((nmax,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pad[:x.shape[0]] = x
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad.contiguous(), group=group)
    return torch.cat([b[:n] for b, n in zip(bufs, sizes)], dim=0)
