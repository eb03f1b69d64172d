"""Row-block packing entry points (mirror of the reference's ``ojasx2/streaming_e8.py:80-216``).

Because every row owns whole scale groups when ``in_features % group_size == 0``, packing a matrix
row block by row block yields exactly the bytes of packing it whole; the GPU encoder therefore
writes each block straight into its final byte range instead of concatenating pieces.
"""

from __future__ import annotations

from typing import Tuple

import torch

from . import ops
from .lattice import E8LatticeLinear, fwht_block32, _check_bitrate


def _validate_row_layout(out_features: int, in_features: int, bitrate: float, group_size: int) -> None:
    """Same rejections as the reference (``streaming_e8.py:90-109``)."""
    if float(bitrate) not in (1.0, 1.5, 2.0):
        raise ValueError(f"Unsupported E8 bitrate {bitrate!r}; expected one of [1.0, 1.5, 2.0]")
    if out_features <= 0 or in_features <= 0:
        raise ValueError("Streaming E8 requires non-empty two-dimensional weights")
    if group_size <= 0 or group_size % 32 != 0:
        raise ValueError("The current E8 packers require group_size to be a positive multiple of 32")
    if in_features % group_size != 0:
        raise ValueError(
            f"in_features={in_features} is not divisible by group_size={group_size}. "
            "Row-block packing would cross a scale-group boundary and change the packed layout.")
    _check_bitrate(bitrate)


def _pack_row_block(block: torch.Tensor, bitrate: float, group_size: int, use_hadamard: bool
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    _check_bitrate(bitrate)
    source = fwht_block32(block) if use_hadamard else block
    return ops.encode(source, group_size)


def pack_weight_rowwise(weight: torch.Tensor, *, bitrate: float = 1.5, group_size: int = 32, row_block: int = 32,
                        use_hadamard: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packs ``weight`` ``row_block`` rows at a time; the result equals whole-matrix packing byte for byte."""
    if weight.ndim != 2:
        raise ValueError(f"Expected a rank-2 weight, got shape {tuple(weight.shape)}")
    if row_block <= 0:
        raise ValueError("row_block must be positive")
    out_features, in_features = map(int, weight.shape)
    _validate_row_layout(out_features, in_features, bitrate, group_size)
    nbytes, nscales = ops.packed_sizes(out_features, in_features, group_size)
    packed = torch.empty(nbytes, dtype=torch.uint8, device=weight.device)
    scales = torch.empty(nscales, dtype=torch.float16, device=weight.device)
    bytes_per_row, scales_per_row = in_features * 3 // 16, in_features // group_size
    for start in range(0, out_features, row_block):
        stop = min(start + row_block, out_features)
        block = weight[start:stop]
        source = fwht_block32(block) if use_hadamard else block
        ops.encode(source, group_size, out=(packed[start * bytes_per_row: stop * bytes_per_row],
                                            scales[start * scales_per_row: stop * scales_per_row]))
    return packed, scales


def _copy_row_block_into_layer(layer: E8LatticeLinear, row_start: int, block: torch.Tensor, use_hadamard: bool) -> int:
    """Encodes ``block`` (rows ``row_start ..``) directly into the layer's packed buffers
    (reference ``streaming_e8.py:162-193``).  Returns the number of source bytes consumed."""
    if block.ndim != 2 or block.shape[1] != layer.in_features:
        raise ValueError(f"Unexpected row block shape {tuple(block.shape)} for "
                         f"{layer.out_features}x{layer.in_features} E8 layer")
    if not block.dtype.is_floating_point:
        raise TypeError(f"E8 packing requires floating-point source weights, got {block.dtype}")
    rows = int(block.shape[0])
    bytes_per_row = layer.in_features * 3 // 16
    scales_per_row = layer.in_features // layer.group_size
    p0, s0 = row_start * bytes_per_row, row_start * scales_per_row
    if p0 + rows * bytes_per_row > layer.packed_weight.numel():
        raise RuntimeError("Packed destination is smaller than the streamed source layout")
    if s0 + rows * scales_per_row > layer.block_scales.numel():
        raise RuntimeError("Scale destination is smaller than the streamed source layout")
    source = block.to(layer.packed_weight.device)
    source = fwht_block32(source) if use_hadamard else source
    with torch.no_grad():
        ops.encode(source, layer.group_size, out=(layer.packed_weight[p0: p0 + rows * bytes_per_row],
                                                  layer.block_scales[s0: s0 + rows * scales_per_row]))
    return int(block.numel() * block.element_size())
