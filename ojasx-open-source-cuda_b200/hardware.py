"""Kernel seam of the reference's lattice engine, bound to the sm_100a kernels.

The reference calls a module-level ``dispatch_tilelang_e8_gemm`` from
``_FusedE8GEMMFunction.forward`` and uses the result when it is not ``None``
(``ojasx2/math/lattice.py:51-55,583-589``; dispatcher at ``ojasx2/tilelang_kernels.py:370-419``).
This module provides a callable with that exact signature.  The reference's multi-backend
auto-tuner and source emitters are intentionally absent: there is one backend here.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops


def dispatch_tilelang_e8_gemm(x_2d: torch.Tensor, packed_weight: torch.Tensor, block_scales: torch.Tensor,
                              bias: Optional[torch.Tensor], out_features: int, in_features: int, group_size: int,
                              bitrate: float, lut_coords: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Fused ternary-E8 linear for CUDA tensors: returns ``y_2d`` ``[M, out_features]`` in x's dtype.

    Declines (returns ``None``, letting the caller's own path run) only for requests outside this
    backend's scope: another bit-rate or non-CUDA tensors.  Errors inside the backend raise; they are
    never swallowed.  ``lut_coords`` is ignored (the kernels carry their own tables).
    """
    del lut_coords
    if float(bitrate) != 1.5 or not x_2d.is_cuda:
        return None
    return ops.linear(x_2d, packed_weight, block_scales, bias, out_features, in_features, group_size)


def install_into_reference() -> bool:
    """Rebinds the reference's seam to this backend when the reference package is importable.
    Returns True when the patch was applied."""
    try:
        import ojasx2.math.lattice as ref_lattice   # type: ignore
    except Exception:
        return False
    ref_lattice.dispatch_tilelang_e8_gemm = dispatch_tilelang_e8_gemm
    return True
