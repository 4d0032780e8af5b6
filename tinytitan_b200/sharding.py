"""Multi-GPU partitioning of the attention path: sessions across ranks, or one long session's
KV range across ranks with a log-sum-exp merge of the per-rank partials.

The reference has no multi-device code; its split-KV chunk-partial format
(sources/TinyTitanCore/Metal/Attention/attention.metal:146-159) is used here as the shard
format: every rank produces one unnormalised (m, d, o) triple per q head for its key range
(tt_attn_decode_partial), the triples are all-gathered (16.5 KB per rank at 16 heads x 256),
and tt_attn_combine merges them. Independent sessions need no exchange at all.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_sessions(lengths: Sequence[int], world_size: int, policy: str = "greedy") -> List[List[int]]:
    """Session indices owned by each rank. "greedy" balances the KV bytes each rank streams
    (longest first onto the lightest rank); "round_robin" is session i -> rank i % world_size."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    shards: List[List[int]] = [[] for _ in range(world_size)]
    if policy == "round_robin":
        for i in range(len(lengths)):
            shards[i % world_size].append(i)
        return shards
    if policy != "greedy":
        raise ValueError(f"unknown policy {policy!r}")
    load = [0] * world_size
    for i in sorted(range(len(lengths)), key=lambda j: (-lengths[j], j)):
        r = min(range(world_size), key=lambda x: (load[x], x))
        shards[r].append(i)
        load[r] += lengths[i]
    for s in shards:
        s.sort()
    return shards


def kv_split_ranges(seq_len: int, world_size: int, kv_start: int = 0) -> List[Tuple[int, int]]:
    """Contiguous key ranges [lo, hi) per rank covering [kv_start, seq_len); trailing ranks may
    be empty, which yields the (-inf, 0, 0) partial the merge ignores."""
    n = max(0, seq_len - kv_start)
    per = -(-n // world_size) if n else 0
    out = []
    for r in range(world_size):
        lo = min(seq_len, kv_start + r * per)
        hi = min(seq_len, lo + per)
        out.append((lo, hi))
    return out


def pack_partial(m, d, o):
    """[H], [H], [H, hd] -> one [H, hd + 2] tensor so that a single all_gather moves the triple."""
    import torch
    return torch.cat([o, m.unsqueeze(1), d.unsqueeze(1)], dim=1).contiguous()


def unpack_partials(packed):
    """[G, H, hd + 2] -> contiguous m [G, H], d [G, H], o [G, H, hd] (tt_attn_combine's layout)."""
    hd = packed.shape[-1] - 2
    return packed[..., hd].contiguous(), packed[..., hd + 1].contiguous(), packed[..., :hd].contiguous()


def exchange_partials(m, d, o, group=None):
    """All-gather every rank's triple. Works on CUDA tensors over NCCL and on CPU tensors over
    gloo (the latter is what the CPU tests of this plumbing use)."""
    import torch
    import torch.distributed as dist
    packed = pack_partial(m, d, o)
    world = dist.get_world_size(group)
    gathered = torch.empty((world,) + tuple(packed.shape), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed, group=group) if packed.is_cuda else \
        dist.all_gather(list(gathered.unbind(0)), packed, group=group)
    return unpack_partials(gathered)


class LongContextDecode:
    """One session whose KV rows are split along the sequence across the ranks of a group.

    Rank r holds rows [lo_r, hi_r) of the logical sequence in its own buffers (local row 0 is
    logical position lo_r). `step` runs pass 1 on the local rows, all-gathers the triples and
    merges them on every rank."""

    def __init__(self, attention, head_dim: int, num_q_heads: int, num_kv_heads: int, scale: float, group=None,
                 fused: bool = False):
        import torch
        import torch.distributed as dist
        self.attention, self.hd, self.hq, self.hkv, self.scale, self.group = attention, head_dim, num_q_heads, num_kv_heads, scale, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        # fused: the triples travel by peer stores inside the merge kernel (tt_attn_exchange_combine)
        # instead of an NCCL all-gather followed by tt_attn_combine
        self.exchange = None
        if fused and self.world > 1:
            from .operators import PeerExchange

            def gather(handle: bytes):
                handles = [None] * self.world
                dist.all_gather_object(handles, handle, group=group)
                return handles
            self.exchange = PeerExchange(attention.context, dist.get_rank(group), self.world, num_q_heads, head_dim, gather)
        dev = torch.device("cuda", attention.context.device)
        self.m = torch.empty(num_q_heads, device=dev)
        self.d = torch.empty(num_q_heads, device=dev)
        self.o = torch.empty(num_q_heads, head_dim, device=dev)
        self.packed = torch.empty(num_q_heads, head_dim + 2, device=dev)
        self.gathered = torch.empty(self.world, num_q_heads, head_dim + 2, device=dev)

    def step(self, q, k_local, v_local, local_rows: int, out):
        import torch
        import torch.distributed as dist
        if self.exchange is not None:
            self.attention.encode_decode_exchange(q, k_local, v_local, self.hd, self.hq, self.hkv, local_rows, 0,
                                                  self.exchange, out, scale=self.scale)
            return out
        self.attention.encode_partial(q, k_local, v_local, self.hd, self.hq, self.hkv, local_rows, 0, self.m,
                                      self.d, self.o, scale=self.scale)
        torch.cat([self.o, self.m.unsqueeze(1), self.d.unsqueeze(1)], dim=1, out=self.packed)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.packed, group=self.group)
        else:
            self.gathered[0].copy_(self.packed)
        m, d, o = unpack_partials(self.gathered)
        self.attention.encode_combine(m, d, o, self.world, self.hq, self.hd, out)
        return out

    def close(self):
        """Collective: every rank stops using the exchange buffers, then unmaps and frees them."""
        if self.exchange is not None:
            import torch
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.exchange.close()
            self.exchange = None
