"""Tensor-parallel partition of the Q4 SwiGLU MLP block over the GPUs of one box.

The reference is single-process (src/mlp.rs); the partition is new.  Gate/up is
split by hidden unit in whole 32-unit interleave chunks (src/linear.rs:603-617),
so every (column, K-block) scale stays with its column and a rank's gate/up
columns are bit-identical to the one-GPU result; down is split by the same
hidden units = whole 32-deep K-blocks of W_down, so each rank's slice quantises
to the same codes and scales as the full matrix.  Each rank produces an f32
partial of the m x d output; one all-reduce sums them; the f16 store rounding
and the residual add follow on every rank.
"""
from __future__ import annotations

import numpy as np

from .host import Gate, GatedLinear, Linear, Mlp, Q4Params, WeightLayout


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


class TpMlp:
    """One rank's shard of a gated MLP plus the collective.  `group` is a
    torch.distributed process group (None = the default group)."""

    def __init__(self, mlp: Mlp, world: int, group=None):
        self.mlp, self.world, self.group = mlp, world, group

    @staticmethod
    def quantize(w_gate, w_up, w_down, rank: int, world: int, gate: Gate = Gate.Silu, p: Q4Params | None = None,
                 group=None) -> "TpMlp":
        wg, wu, wd = shard_weights(np.asarray(w_gate, np.float32), np.asarray(w_up, np.float32),
                                   np.asarray(w_down, np.float32), rank, world)
        fl, d = wg.shape
        up = GatedLinear.quantize(wg, wu, WeightLayout.OutIn, fl, d, gate, p)
        down = Linear.quantize(wd, WeightLayout.OutIn, wd.shape[0], fl, p)
        return TpMlp(Mlp.gated(up, down), world, group)

    def accumulate(self, x, y, m: int, partial=None) -> None:
        """y (m x d f32, replicated) += down(glu(x @ gate_up)) across the ranks."""
        import torch
        import torch.distributed as dist
        if self.world == 1:
            self.mlp.accumulate(x, y, m)
            return
        if partial is None:
            partial = torch.empty_like(y)
        self.mlp.partial(x, partial, m)
        dist.all_reduce(partial, group=self.group)
        Mlp.finish(y, partial)
