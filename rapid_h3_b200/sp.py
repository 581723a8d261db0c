"""Sequence parallelism for the DiT step: tokens are sharded across ranks for quantizers, GEMMs and
epilogues (all row-local), and self-attention runs on head shards (Ulysses): one all-to-all turns
[tokens/P, H] into [tokens, H/P] before the attention pre-pass, a second one returns the output to
token sharding. One process per GPU, torch.distributed (NCCL over NVLink on GPUs, gloo in CPU tests).
The reference is single-GPU (its only mention of sequence parallelism is a dropped experiment,
docs/kernels.md:180), so this module has no reference counterpart.
"""
import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from .timing import phase as _phase


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


def scatter_plan(bounds, rank, w, elem_bytes=2):
    """Where the attention epilogue of `rank` (owner of one head group of width `w`) stores the output rows of
    every token range: rank r's buffer is [P, count_r, w], slot `rank` of it belongs to this head group.
    Returns (byte offset into rank r's buffer for r = 0..P-1, row starts [P + 1])."""
    offsets = [rank * (b - a) * w * elem_bytes for a, b in bounds]
    starts = [a for a, _ in bounds] + [bounds[-1][1]]
    return offsets, starts


class PeerBuffers:
    """One device buffer of `nbytes` per rank, mapped into every rank of the group (ranks on one node): `local` is
    this rank's buffer as a uint8 tensor, `ptrs[r]` the address of rank r's buffer in this process. Tried in
    order: torch symmetric memory, then CUDA IPC handles exchanged through the process group. The peer addresses
    are only ever handed to this package's own kernels, which store to them; no library kernel and no bulk/TMA
    load touches another GPU's memory."""

    def __init__(self, nbytes, device, group=None):
        self.group = group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        nbytes = (int(nbytes) + 255) // 256 * 256
        self.how, self._keep = None, []
        errors = []
        # plain peer mappings are all that is needed: keep the buffers out of NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(nbytes, dtype=torch.uint8, device=device)
            hdl = symm.rendezvous(t, group if group is not None else dist.group.WORLD)
            self.local, self.ptrs, self.how = t, [int(x) for x in hdl.buffer_ptrs], "symmetric_memory"
            self._keep.append(hdl)
        except Exception as e:  # noqa: BLE001 - any failure of the optional path selects the IPC path
            errors.append(f"symmetric memory: {type(e).__name__}: {e}")
        # every rank must take the same path
        ok = torch.tensor([1 if self.how else 0], device=device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self.how = None
            t = torch.empty(nbytes, dtype=torch.uint8, device=device)
            handle = t.untyped_storage()._share_cuda_()
            offset = t.storage_offset()
            gathered = [None] * world
            dist.all_gather_object(gathered, (handle, offset), group=group)
            self.local, self.ptrs = t, []
            for r, (h, off) in enumerate(gathered):
                if r == rank:
                    self.ptrs.append(t.data_ptr())
                    continue
                st = torch.UntypedStorage._new_shared_cuda(*h)
                peer = torch.empty(0, dtype=torch.uint8, device=st.device).set_(st, off, (nbytes,))
                self._keep.append(peer)
                self.ptrs.append(peer.data_ptr())
            self.how = "cuda_ipc"
        self.errors = errors
        dist.barrier(group=group)


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
        self.fused = False

    # ---- exchanges done by the kernels themselves (stores into peer memory + a stream-ordered barrier) ----
    def enable_fused(self, heads, head_dim, device):
        """Allocate the two exchange buffers in every rank and map them everywhere. Afterwards `rope_scatter` and
        `attention_scatter` replace rms_rope + tokens_to_heads and attention + heads_to_tokens."""
        p = self.world
        if heads % p:
            raise RuntimeError(f"{heads} heads do not divide over {p} ranks")
        self._w = (heads // p) * head_dim
        self._heads, self._head_dim = heads, head_dim
        self._qkv_buf = PeerBuffers(self.total * 3 * self._w * 2, device, self.group)
        self._o_buf = PeerBuffers(p * max(self.counts) * self._w * 2, device, self.group)
        self._flag = torch.zeros(1, device=device, dtype=torch.int32)
        self.fused = True
        return self._qkv_buf.how

    def _barrier(self):
        """All ranks' kernels enqueued so far have finished (and their stores have landed) before anything enqueued
        after it starts: a one-element all-reduce on the compute stream."""
        with _phase("exchange_barrier"):
            dist.all_reduce(self._flag, group=self.group)

    def rope_scatter(self, qkv, q_weight, k_weight, eps, tab):
        """qkv [S_local, 3*H*D] (raw q | k | v of this rank's tokens) -> q, k, v [S_total, H/P, D] of this rank's
        heads: RMSNorm + RoPE of q and k fused with the token -> head exchange (rh3_rope_scatter_heads)."""
        _lib.require_cuda(qkv, q_weight, k_weight)
        s_loc = qkv.shape[0]
        if qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1 or qkv.shape[1] != 3 * self._heads * self._head_dim:
            raise RuntimeError("qkv must be bf16 [S_local, 3*H*D] with unit column stride")
        if tab is not None and (tab.dtype != torch.bfloat16 or tab.numel() != s_loc * 48 * 4 or not tab.is_contiguous()):
            raise RuntimeError("rope table must be contiguous bf16 [S_local, 48, 2, 2]")
        ptrs = (ctypes.c_void_p * self.world)(*self._qkv_buf.ptrs)
        _lib.call("rh3_rope_scatter_heads", qkv.data_ptr(), qkv.stride(0), s_loc, self._heads, self.world, self.lo,
                  q_weight.data_ptr(), k_weight.data_ptr(), float(eps), _lib.ptr(tab), ptrs, _lib.stream())
        self._barrier()
        recv = self._qkv_buf.local[: self.total * 3 * self._w * 2].view(torch.bfloat16).view(self.total, 3, self._w)
        return tuple(recv[:, i].view(self.total, self._heads // self.world, self._head_dim) for i in range(3))

    def attention_scatter(self, q, k, v, scale=None):
        """Attention on this rank's heads; the epilogue stores every token's output row into the rank that owns the
        token. Returns [P, S_local, (H/P)*D] as heads_to_tokens does."""
        from . import attn_int8
        pre = attn_int8.int8_prepass(q, k, v, _tag="self")
        w = self._w
        offsets, starts = scatter_plan(self.bounds, self.rank, w)
        ptrs = [self._o_buf.ptrs[r] + offsets[r] for r in range(self.world)]
        attn_int8.attention_pre(pre, scale, scatter=(ptrs, starts, w, self._head_dim), _tag="self")
        self._barrier()
        s_loc = self.counts[self.rank]
        return self._o_buf.local[: self.world * s_loc * w * 2].view(torch.bfloat16).view(self.world, s_loc, w)

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
