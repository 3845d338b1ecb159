"""KV-head sharding of the path over the GPUs of one node, the way ppl.nn's tensor parallelism
shards attention (tools/benchmark_llama/text_generator.cc:199-211): rank r of N owns kv heads
[r*Hkv/N, (r+1)*Hkv/N) with their query heads and a private cache holding only those heads; the
index tensors are replicated; the path itself needs no collective.  The only communication is an
all-gather of the per-rank outputs for whoever wants the full [T, Hq, Dh] tensor (verification)."""
from __future__ import annotations


def head_shard(num_heads: int, num_kv_heads: int, rank: int, world: int):
    """(query head slice, kv head slice) of `rank`.  Requires world | num_kv_heads."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank out of range")
    if num_kv_heads % world or num_heads % num_kv_heads:
        raise ValueError("the number of ranks must divide num_kv_heads, and num_kv_heads must divide num_heads")
    group = num_heads // num_kv_heads
    kv_per = num_kv_heads // world
    kv = slice(rank * kv_per, (rank + 1) * kv_per)
    q = slice(kv.start * group, kv.stop * group)
    return q, kv


def shard_call(query, current_key, current_value, num_heads: int, num_kv_heads: int, rank: int, world: int):
    """This rank's slices of the per-call tensors ([T, H, Dh] arrays or tensors, contiguous copies)."""
    q, kv = head_shard(num_heads, num_kv_heads, rank, world)

    def take(x, s):
        y = x[:, s]
        return y.contiguous() if hasattr(y, "contiguous") else y.copy()

    return take(query, q), take(current_key, kv), take(current_value, kv)


def gather_heads(local_out, world: int, group=None):
    """All-gather [T, Hq/N, Dh] outputs into [T, Hq, Dh] (torch.distributed; gloo or nccl)."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return local_out
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)
