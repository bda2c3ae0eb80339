"""Sharding of the attention work across the GPUs of one box.

The unit of work is one (batch, KV head) pair together with its group of query heads (group size 1 for
MHA).  Units are independent, so rank r of W takes a contiguous range of units and no data-path
collective is needed; tables and theta are replicated.  In the flattened [B*Hkv, G, N, D] view a rank's
shard is a contiguous slice.
"""


def unit_range(n_units, rank, world_size):
    """Half-open range of unit indices owned by `rank`; remainders go to the lowest ranks."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size: %r/%r" % (rank, world_size))
    base, rem = divmod(n_units, world_size)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo, hi


def shard_units(B, Hkv, rank, world_size):
    """List of (b, kv_head) units owned by `rank`."""
    lo, hi = unit_range(B * Hkv, rank, world_size)
    return [(u // Hkv, u % Hkv) for u in range(lo, hi)]
