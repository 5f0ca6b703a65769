"""R-sharded BSI linear layers for one node with several GPUs.

The output rows (keys) of a linear layer are independent, so rank g of G keeps the keys of rows
[g*R/G, (g+1)*R/G) -- built once from its slice of the weight -- packs the (replicated) activations,
computes its [Q, R/G] block of the output and the blocks are exchanged with one all-gather over
NCCL (NVLink / NVSwitch). The reference has no distributed code; this is the multi-GPU extension of
its BSIQuantizedLinear (bsi_ops/benchmarks/verify_accuracy_bsi.py:46-215), with the same arithmetic
per output element, so a sharded model reproduces the single-GPU outputs bit for bit.

`shard_rows` / `gather_columns` carry the host-side logic and run on any backend (the CPU tests
drive them over gloo with a dense matmul standing in for the BSI dot).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


def shard_rows(R: int, world: int, rank: int, multiple: int = 1):
    """Half-open row range of `rank`: equal blocks of ceil(R/world) rounded up to `multiple`, the last
    ranks get what is left (possibly nothing)."""
    per = -(-R // world)
    per = -(-per // multiple) * multiple
    lo = min(R, rank * per)
    hi = min(R, lo + per)
    return lo, hi


def gather_columns(y_shard: torch.Tensor, R: int, world: int, group=None, multiple: int = 1) -> torch.Tensor:
    """All-gathers the per-rank column blocks [Q, r_g] into [Q, R].

    Ranks may hold blocks of different width (a ragged tail): every block is padded to the common
    width for the collective and trimmed afterwards."""
    if world == 1:
        return y_shard
    Q = y_shard.shape[0]
    per = shard_rows(R, world, 0, multiple)[1]
    if y_shard.shape[1] != per:
        pad = y_shard.new_zeros(Q, per)
        pad[:, : y_shard.shape[1]] = y_shard
        y_shard = pad
    gathered = y_shard.new_empty(world * Q, per)     # rank-major concatenation along dim 0
    dist.all_gather_into_tensor(gathered, y_shard.contiguous(), group=group)
    out = gathered.view(world, Q, per).permute(1, 0, 2).reshape(Q, world * per)
    return out[:, :R] if world * per != R else out


class BSIShardedLinear(nn.Module):
    """BSI linear whose keys are sharded along the output rows across the ranks of `group`."""

    def __init__(self, original_linear, rank: int, world: int, group=None, decimalPlaces=2, compress_threshold=0.2,
                 name: str = ""):
        super().__init__()
        from .linear import BSIQuantizedLinear

        self.in_features = original_linear.in_features
        self.out_features = original_linear.out_features
        self.rank, self.world, self.group = int(rank), int(world), group
        # 256-row blocks keep every shard a whole number of key tiles of the dot kernel
        self.multiple = 256 if self.out_features % (256 * self.world) == 0 else 32
        lo, hi = shard_rows(self.out_features, self.world, self.rank, self.multiple)
        self.lo, self.hi = lo, hi
        shard = nn.Linear(self.in_features, max(hi - lo, 1), bias=original_linear.bias is not None,
                          device=original_linear.weight.device, dtype=original_linear.weight.dtype)
        with torch.no_grad():
            if hi > lo:
                shard.weight.copy_(original_linear.weight[lo:hi])
                if original_linear.bias is not None:
                    shard.bias.copy_(original_linear.bias[lo:hi])
            else:
                shard.weight.zero_()
        self.empty = hi <= lo
        self.local = BSIQuantizedLinear(shard, decimalPlaces=decimalPlaces, compress_threshold=compress_threshold)
        self.weight_bsi_memory_bytes = self.local.weight_bsi_memory_bytes
        self.total_bsi_static_bytes = self.local.total_bsi_static_bytes

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        y = self.local(x2)
        if self.empty:
            y = y[:, :0]
        y = gather_columns(y, self.out_features, self.world, self.group, self.multiple)
        return y.view(*shape[:-1], self.out_features)


def sharded_layer_factory(rank: int, world: int, group=None):
    """`layer_factory` for `quantize_model_bsi`: every replaced Linear becomes a BSIShardedLinear."""
    def make(linear, decimalPlaces=2, compress_threshold=0.2, name=""):
        return BSIShardedLinear(linear, rank, world, group, decimalPlaces=decimalPlaces,
                                compress_threshold=compress_threshold, name=name)
    return make
