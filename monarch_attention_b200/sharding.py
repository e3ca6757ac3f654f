"""Partitioning of independent (batch, head) units across the GPUs of one box.

Every (e, h) pair of a MonarchAttention call is independent in all four stages
(reference: ma/ma_torch.py:65-108 has no reduction over E or H; the Triton grids are
flat over E*H, ma/ma_triton.py:656-657), so the op shards across devices without any
data-path collective: each rank runs the library on its own slice of the batch or
head axis.  The only communication is a gather of per-rank timings and checksums
for reporting.
"""
from __future__ import annotations


def unit_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous [lo, hi) slice of ``total`` units for ``rank`` of ``world``.

    The first ``total % world`` ranks take one extra unit; a rank may get an empty
    slice when ``world > total``.
    """
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad partition request total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_heads(q, k, v, rank: int, world: int):
    """Slice (E, H, N, W) tensors along the flattened (E*H) axis for one rank.

    Splits along E when E is a multiple of ``world`` (views, no copy), else along H
    when H is a multiple of ``world`` (views), else falls back to a contiguous slice
    of the flattened (E*H) axis reshaped to (1, units, N, W).
    """
    E, H = q.shape[0], q.shape[1]
    if E % world == 0:
        lo, hi = unit_range(E, rank, world)
        return q[lo:hi], k[lo:hi], v[lo:hi]
    if H % world == 0:
        lo, hi = unit_range(H, rank, world)
        return q[:, lo:hi], k[:, lo:hi], v[:, lo:hi]
    lo, hi = unit_range(E * H, rank, world)

    def flat(t):
        return t.reshape(1, E * H, t.shape[2], t.shape[3])[:, lo:hi]

    return flat(q), flat(k), flat(v)


def gather_to_rank0(values, group=None):
    """All ranks contribute a picklable object; rank 0 receives the list (others get None).

    One collective, used for reporting only.  Works on any torch.distributed backend;
    returns ``[values]`` when no process group is initialised.
    """
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return [values]
    world = dist.get_world_size(group)
    out = [None] * world if dist.get_rank(group) == 0 else None
    dist.gather_object(values, out, dst=0, group=group)
    return out
