"""Sequence parallelism for the DiT step: tokens are sharded across ranks for quantizers, GEMMs and
epilogues (all row-local), and self-attention runs on head shards (Ulysses): one all-to-all turns
[tokens/P, H] into [tokens, H/P] before the attention pre-pass, a second one returns the output to
token sharding. One process per GPU, torch.distributed (NCCL over NVLink on GPUs, gloo in CPU tests).
The reference is single-GPU (its only mention of sequence parallelism is a dropped experiment,
docs/kernels.md:180), so this module has no reference counterpart.
"""
import torch
import torch.distributed as dist


def shard_bounds(total, world, align=64):
    """Contiguous, nearly equal token ranges [(start, stop)] per rank. Boundaries fall on multiples of
    `align` tokens (the last rank takes the ragged tail): the attention query quantizer works on blocks of
    64 tokens, so aligned shards see exactly the blocks the unsharded sequence has and the sequence-parallel
    step reproduces the single-GPU step bit for bit."""
    nblk = (total + align - 1) // align
    base, extra = divmod(nblk, world)
    out, a = [], 0
    for r in range(world):
        b = min(total, a + (base + (1 if r < extra else 0)) * align)
        out.append((a, b))
        a = b
    return out


def shard_segments(segments, lo, hi):
    """Intersect modality segments [(start, stop, row)] with this rank's rows [lo, hi), re-based to lo."""
    out = []
    for a, b, row in segments:
        a2, b2 = max(a, lo), min(b, hi)
        if b2 > a2:
            out.append((a2 - lo, b2 - lo, row))
    return out


class Ulysses:
    """Token <-> head re-sharding around self-attention for one packed sequence of `total` tokens."""

    def __init__(self, total, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.bounds = shard_bounds(total, self.world)
        self.counts = [b - a for a, b in self.bounds]
        self.total = total
        self.lo, self.hi = self.bounds[self.rank]

    def tokens_to_heads(self, qkv, heads, head_dim):
        """qkv [S_local, 3*H*D] -> q, k, v as [S_total, H/P, D] views (rows in global token order)."""
        p, s_loc = self.world, qkv.shape[0]
        if heads % p:
            raise RuntimeError(f"{heads} heads do not divide over {p} ranks")
        w = (heads // p) * head_dim
        send = qkv.view(s_loc, 3, p, w).permute(2, 0, 1, 3).contiguous().view(p * s_loc, 3, w)
        recv = torch.empty((self.total, 3, w), device=qkv.device, dtype=qkv.dtype)
        dist.all_to_all_single(recv, send, output_split_sizes=self.counts, input_split_sizes=[s_loc] * p,
                               group=self.group)
        return tuple(recv[:, i].view(self.total, heads // p, head_dim) for i in range(3))

    def heads_to_tokens(self, og):
        """og [S_total, H/P, D] (contiguous) -> [P, S_local, (H/P)*D]: this rank's tokens, grouped by the rank
        (= head group) that computed them; rapid_h3_b200.quantizers.quant_groups_i8 reads it in place."""
        p, s_loc = self.world, self.counts[self.rank]
        w = og.shape[1] * og.shape[2]
        send = og.reshape(self.total, w)
        recv = torch.empty((p * s_loc, w), device=og.device, dtype=og.dtype)
        dist.all_to_all_single(recv, send, output_split_sizes=[s_loc] * p, input_split_sizes=self.counts,
                               group=self.group)
        return recv.view(p, s_loc, w)

    def gather_tokens(self, x_local):
        """All ranks' token rows concatenated in token order: [S_total, ...] (shards padded to equal length
        for the collective, since shard sizes may differ by one)."""
        cmax = max(self.counts)
        tail = tuple(x_local.shape[1:])
        mine = torch.zeros((cmax,) + tail, device=x_local.device, dtype=x_local.dtype)
        mine[:x_local.shape[0]] = x_local
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        return torch.cat([p[:c] for p, c in zip(parts, self.counts)], 0)
