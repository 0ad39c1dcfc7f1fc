"""Tensor-parallel partition of the Q4 SwiGLU MLP block, and of the self-attention block, over the GPUs of one box.

The reference is single-process (src/mlp.rs); the partition is new.  Gate/up is
split by hidden unit in whole 32-unit interleave chunks (src/linear.rs:603-617),
so every (column, K-block) scale stays with its column and a rank's gate/up
columns are bit-identical to the one-GPU result; down is split by the same
hidden units = whole 32-deep K-blocks of W_down, so each rank's slice quantises
to the same codes and scales as the full matrix.  Each rank produces an f32
partial of the m x d output; one all-reduce sums them; the f16 store rounding
and the residual add follow on every rank.

Self-attention (src/self_attention.rs; single-process there too) is split by heads: a rank projects, caches and
attends its own query heads and the key/value heads they use, and multiplies by its rows of the out projection;
the f32 partial outputs are summed the same way.
"""
from __future__ import annotations

import os

import numpy as np

from .host import Gate, GatedLinear, KvCache, Linear, Mlp, Q4Params, SelfAttention, WeightLayout

FLAG_WORDS = 1288      # SMEG_TP_FLAG_WORDS of include/smeg_api.h


def shard_bounds(hidden_units: int, rank: int, world: int):
    """Hidden units [lo, hi) owned by `rank`: whole 32-unit chunks, sizes differing by at most one chunk."""
    assert hidden_units % 32 == 0, "the hidden width must be a whole number of 32-unit chunks to shard"
    chunks = hidden_units // 32
    assert world <= chunks
    lo = (chunks * rank // world) * 32
    hi = (chunks * (rank + 1) // world) * 32
    return lo, hi


def shard_weights(w_gate, w_up, w_down, rank: int, world: int):
    """(W_gate[lo:hi], W_up[lo:hi], W_down[:, lo:hi]) of OutIn f32 weights
    (W_gate, W_up: [hidden][d]; W_down: [d][hidden])."""
    f = w_gate.shape[0]
    lo, hi = shard_bounds(f, rank, world)
    return (np.ascontiguousarray(w_gate[lo:hi]), np.ascontiguousarray(w_up[lo:hi]),
            np.ascontiguousarray(w_down[:, lo:hi]))


class PeerReduce:
    """The ranks' partial buffers and flag arrays in memory every rank can address (torch symmetric
    memory: CUDA peer mappings over NVLink), and the one-kernel sum + f16 rounding + residual add over
    them (smeg_mlp_reduce_finish_dev).  Collective to construct; every rank then calls `finish` once
    per step, in the same order.  One object serves the exchanges of one shape and one form: above 64 rows the
    MLP block pushes its partial rows (other offsets inside the buffers, results as marked words), so an
    exchange that pulls -- the attention block's -- takes a PeerReduce of its own there."""

    def __init__(self, m: int, d: int, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", torch.cuda.current_device())
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert self.world <= 8 and (m * d) % 4 == 0
        # two buffers, taken in turn from step to step (the one-shot form of the kernel needs that); each holds
        # the f32 partial sums followed by the f16 results the owners of the other slices write back
        self._len = m * d
        # the pushed form keeps `world` slots of ceil(m / world) rows (one per sending rank) ahead of the f16 results
        self._rows = -(-m // self.world)
        self._recv = self.world * self._rows * d
        # (results: m * d f16 in the pulled form, m * d marked 4-byte words in the pushed form)
        self._stride = (max(self._len, self._recv) + self._len + 3) // 4 * 4   # floats per buffer, whole 16-byte vectors
        self.push = m > 64 and self.world > 1 and os.environ.get("SMEG_TP_PUSH", "1") != "0"
        self._both = symm.empty((2, self._stride), dtype=torch.float32, device=dev)
        self.flags = symm.empty((FLAG_WORDS,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        self._both.zero_()
        self._m, self._d = m, d
        torch.cuda.synchronize()
        self._hp = symm.rendezvous(self._both, group)
        self._hf = symm.rendezvous(self.flags, group)
        dist.barrier(group)                      # every rank's flags are zero before anyone's first call
        import ctypes as C
        self._C = C
        self._base = [int(p) for p in self._hp.buffer_ptrs]
        self._flags = (C.c_uint64 * self.world)(*[int(p) for p in self._hf.buffer_ptrs])
        # short vectors: every rank sums everything itself, one flag round instead of two
        self.oneshot = 1 if self._len * 4 <= 128 * 1024 else 0
        self.seq = 0
        # the ranks' buffers of either parity, as the C ABI takes them (built once: a step is a few calls long)
        self._bufs = [(C.c_uint64 * self.world)(*[b + par * self._stride * 4 for b in self._base]) for par in (0, 1)]

    @property
    def partial(self):
        """The buffer this rank's partial product of the coming step goes into."""
        return self._both[(self.seq + 1) & 1][: self._len].view(self._m, self._d)

    def next_bufs(self):
        """Every rank's buffer of the coming step, as the C ABI takes them."""
        return self._bufs[(self.seq + 1) & 1]

    def finish(self, y, pushed: bool = False) -> None:
        """y += f32(f16(sum over ranks of their `partial`)), on every rank.  pushed: the partials were stored into their
        owners' receive areas by smeg_mlp_partial_push_dev."""
        from ._lib import check, lib
        from .host import _ptr, _stream
        self.seq += 1
        bufs = self._bufs[self.seq & 1]
        if pushed:
            check("smeg_mlp_reduce_finish_pushed_dev",
                  lib().smeg_mlp_reduce_finish_pushed_dev(_ptr(y), bufs, self._flags, self.rank, self.world, self._m, self._d,
                                                          self.seq & 0xffffffff, _stream()))
            return
        check("smeg_mlp_reduce_finish_dev",
              lib().smeg_mlp_reduce_finish_dev(_ptr(y), bufs, self._flags, self.rank, self.world, y.numel(),
                                               self.seq & 0xffffffff, self.oneshot, _stream()))


class TpMlp:
    """One rank's shard of a gated MLP plus the collective.  `group` is a
    torch.distributed process group (None = the default group).  With `peer` (a PeerReduce for the
    step's m x d) the sum over ranks, the rounding and the residual add run as one kernel over peer
    memory; without it an all-reduce of the library behind torch.distributed and the finishing pass."""

    def __init__(self, mlp: Mlp, world: int, group=None, peer: "PeerReduce | None" = None):
        self.mlp, self.world, self.group, self.peer = mlp, world, group, peer

    @staticmethod
    def quantize(w_gate, w_up, w_down, rank: int, world: int, gate: Gate = Gate.Silu, p: Q4Params | None = None,
                 group=None) -> "TpMlp":
        wg, wu, wd = shard_weights(np.asarray(w_gate, np.float32), np.asarray(w_up, np.float32),
                                   np.asarray(w_down, np.float32), rank, world)
        fl, d = wg.shape
        up = GatedLinear.quantize(wg, wu, WeightLayout.OutIn, fl, d, gate, p)
        down = Linear.quantize(wd, WeightLayout.OutIn, wd.shape[0], fl, p)
        return TpMlp(Mlp.gated(up, down), world, group)

    def k(self) -> int:
        return self.mlp.k()

    def n(self) -> int:
        return self.mlp.n()

    def accumulate(self, x, y, m: int, partial=None) -> None:
        """y (m x d f32, replicated) += down(glu(x @ gate_up)) across the ranks."""
        import torch
        import torch.distributed as dist
        if self.world == 1:
            self.mlp.accumulate(x, y, m)
            return
        if self.peer is not None:
            if self.peer.push and m == self.peer._m:
                # the down projection's last stage stores each result row into its owner rank's receive area
                from ._lib import check, lib
                from .host import _ptr, _stream
                rc = lib().smeg_mlp_partial_push_dev(self.mlp._h, _ptr(x), self.peer.next_bufs(), self.peer.rank, self.world, m, _stream())
                if rc == 0:
                    self.peer.finish(y, pushed=True)
                    return
                if rc != -3:
                    check("smeg_mlp_partial_push_dev", rc)
            self.mlp.partial(x, self.peer.partial, m)
            self.peer.finish(y)
            return
        if partial is None:
            partial = torch.empty_like(y)
        self.mlp.partial(x, partial, m)
        dist.all_reduce(partial, group=self.group)
        Mlp.finish(y, partial)


def shard_heads(heads: int, kv_heads: int, rank: int, world: int):
    """(first query head, query heads, first KV head, KV heads) of `rank`: whole groups of heads / kv_heads query heads
    with the KV head they share, the same number on every rank."""
    assert heads % kv_heads == 0 and kv_heads % world == 0, "the KV heads divide evenly over the ranks"
    kvl = kv_heads // world
    hl = kvl * (heads // kv_heads)
    return rank * hl, hl, rank * kvl, kvl


def shard_attention_weights(w_qkv, w_out, heads: int, kv_heads: int, head_dim: int, rank: int, world: int):
    """A rank's rows of the fused projection W_qkv ([(heads + 2 kv_heads) * head_dim][d], rows [q | k | v] in head
    order) -- again [q | k | v] -- and its input columns of W_out ([d_out][heads * head_dim])."""
    h0, hl, kv0, kvl = shard_heads(heads, kv_heads, rank, world)
    q_len, kv_len = heads * head_dim, kv_heads * head_dim
    assert w_qkv.shape[0] == q_len + 2 * kv_len and w_out.shape[1] == q_len
    assert (hl * head_dim) % 32 == 0, "a rank's input columns of W_out are whole 32-deep K-blocks"
    q = w_qkv[h0 * head_dim:(h0 + hl) * head_dim]
    k = w_qkv[q_len + kv0 * head_dim:q_len + (kv0 + kvl) * head_dim]
    v = w_qkv[q_len + kv_len + kv0 * head_dim:q_len + kv_len + (kv0 + kvl) * head_dim]
    return (np.ascontiguousarray(np.concatenate([q, k, v], axis=0)),
            np.ascontiguousarray(w_out[:, h0 * head_dim:(h0 + hl) * head_dim]))


class TpSelfAttention:
    """One rank's heads of a self-attention block plus the sum over ranks: y (m x d f32, replicated) +=
    out(attention(qkv(x))).  The rank's KvCache (from `cache`) holds its own KV heads only.  With `peer` (a PeerReduce
    for the step's m x d) the sum, the f16 rounding and the residual add run as one kernel over peer memory; without it
    an all-reduce of the library behind torch.distributed and the finishing pass.  Block(norm1, TpSelfAttention, norm2,
    TpMlp) is a whole tensor-parallel layer over a replicated residual stream."""

    def __init__(self, attn: SelfAttention, world: int, group=None, peer: "PeerReduce | None" = None):
        self.attn, self.world, self.group, self.peer = attn, world, group, peer

    @staticmethod
    def quantize(w_qkv, w_out, heads: int, kv_heads: int, head_dim: int, rank: int, world: int,
                 p: Q4Params | None = None, group=None) -> "TpSelfAttention":
        wq, wo = shard_attention_weights(np.asarray(w_qkv, np.float32), np.asarray(w_out, np.float32), heads, kv_heads,
                                         head_dim, rank, world)
        _, hl, _, kvl = shard_heads(heads, kv_heads, rank, world)
        qkv = Linear.quantize(wq, WeightLayout.OutIn, wq.shape[0], wq.shape[1], p)
        out = Linear.quantize(wo, WeightLayout.OutIn, wo.shape[0], wo.shape[1], p)
        return TpSelfAttention(SelfAttention(qkv, out, hl, kvl, head_dim), world, group)

    def cache(self, capacity: int) -> KvCache:
        return self.attn.cache(capacity)

    def width(self) -> int:
        return self.attn.width()

    def out_width(self) -> int:
        return self.attn.out_width()

    def accumulate(self, x, cache: KvCache, y, m: int) -> None:
        import torch
        import torch.distributed as dist
        if self.world == 1:
            self.attn.accumulate(x, cache, y, m)
            return
        att16 = self.attn.attend(x, cache, m)
        if self.peer is not None:
            self.attn.out.partial(att16, self.peer.partial, m)
            self.peer.finish(y)
            return
        partial = torch.empty_like(y)
        self.attn.out.partial(att16, partial, m)
        dist.all_reduce(partial, group=self.group)
        Mlp.finish(y, partial)
