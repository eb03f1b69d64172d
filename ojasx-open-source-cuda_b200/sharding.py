"""Output-column sharding of a packed linear across the GPUs of one node.

Rows of W (output features) are independent, and when ``K % 32 == 0`` rank r's shard is a
contiguous byte range of the packed buffers - no repacking.  Each rank computes
``y[:, n0:n1]`` with the fused kernels; an NCCL all-gather over NVLink assembles the full output.
The reference has no multi-GPU form of this path (its only distributed code is a TCP pipeline,
``ojasx2/mesh_hal.py``), so this module has no counterpart there.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch


def shard_rows(n_rows: int, world_size: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """Contiguous row range ``[n0, n1)`` of ``rank``.  Ranges are multiples of ``multiple`` rows (the
    kernels' row tile) except possibly the last; all rows are covered exactly once."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    blocks = (n_rows + multiple - 1) // multiple
    b0 = blocks * rank // world_size
    b1 = blocks * (rank + 1) // world_size
    return min(b0 * multiple, n_rows), min(b1 * multiple, n_rows)


def shard_sizes(n_rows: int, world_size: int, multiple: int = 16) -> List[int]:
    return [b - a for a, b in (shard_rows(n_rows, world_size, r, multiple) for r in range(world_size))]


def slice_packed(packed: torch.Tensor, scales: torch.Tensor, in_features: int, n0: int, n1: int,
                 group_size: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Views of rows ``[n0, n1)`` of packed codes and scales (requires whole groups per row)."""
    if in_features % group_size != 0:
        raise ValueError("row slicing needs in_features % group_size == 0")
    bpr, spr = in_features * 3 // 16, in_features // group_size
    return packed[n0 * bpr: n1 * bpr], scales[n0 * spr: n1 * spr]


class ColumnShardedLinear:
    """One rank's shard of a packed linear plus the all-gather that follows it.

    ``forward(x)`` returns the full ``[M, N]`` output on every rank.  With ``world_size == 1`` no
    collective is issued.  ``compute`` is injectable so the sharding logic can be exercised on CPU
    ranks (gloo) with a stand-in for the CUDA kernel.
    """

    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor], out_features: int,
                 in_features: int, group_size: int = 32, rank: int = 0, world_size: int = 1, group=None,
                 compute=None):
        self.N, self.K, self.g = int(out_features), int(in_features), int(group_size)
        self.rank, self.world, self.group = rank, world_size, group
        self.n0, self.n1 = shard_rows(self.N, world_size, rank)
        self.sizes = shard_sizes(self.N, world_size)
        self.packed, self.scales = slice_packed(packed, scales, self.K, self.n0, self.n1, self.g)
        self.bias = bias[self.n0:self.n1] if bias is not None else None
        if compute is None:
            from . import ops
            compute = ops.linear
        self._compute = compute

    def forward_local(self, x2d: torch.Tensor) -> torch.Tensor:
        if self.n1 == self.n0:
            return x2d.new_empty((x2d.shape[0], 0))
        return self._compute(x2d, self.packed, self.scales, self.bias, self.n1 - self.n0, self.K, self.g)

    def forward(self, x2d: torch.Tensor) -> torch.Tensor:
        y_local = self.forward_local(x2d)
        if self.world == 1:
            return y_local
        import torch.distributed as dist
        m = x2d.shape[0]
        widest = max(self.sizes)
        if y_local.shape[1] != widest:
            # ragged last shards are padded so that one fixed-size collective serves every rank
            pad = y_local.new_zeros((m, widest))
            pad[:, : y_local.shape[1]] = y_local
            y_local = pad
        flat = y_local.new_empty((self.world * m, widest))
        dist.all_gather_into_tensor(flat, y_local.contiguous(), group=self.group)
        buf = flat.view(self.world, m, widest)
        if len(set(self.sizes)) == 1:
            return buf.permute(1, 0, 2).reshape(m, self.N)
        return torch.cat([buf[r, :, : s] for r, s in enumerate(self.sizes)], dim=1)

    __call__ = forward
