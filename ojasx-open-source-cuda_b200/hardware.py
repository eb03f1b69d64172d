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


def fused_ternary_e8_gemm_fwd(x: torch.Tensor, packed_weight: torch.Tensor, block_scales: torch.Tensor,
                              bias: Optional[torch.Tensor] = None, group_size: int = 32) -> torch.Tensor:
    """Same schema as the reference's native op ``fused_ternary_e8_gemm_fwd(Tensor x, Tensor packed_weight,
    Tensor block_scales, Tensor? bias=None, int group_size=32) -> Tensor``
    (``ojasx2/math/csrc/ojasx_math_bindings.cpp:407-477,592``): ``x [M, K]``, row-major 2-D
    ``packed_weight [N, K*3/16]`` and ``block_scales [N, K/group]``; returns ``y [M, N]`` in x's dtype.
    The reference casts the scales to x's dtype before the call; fp16 scales are used as they are and any
    other dtype is converted back to fp16 (exact for values that were fp16 to begin with)."""
    if x.dim() != 2 or packed_weight.dim() != 2 or block_scales.dim() != 2:
        raise RuntimeError("fused_ternary_e8_gemm_fwd expects 2-D x, packed_weight and block_scales")
    n, k = int(packed_weight.shape[0]), int(x.shape[1])
    if int(packed_weight.shape[1]) * 16 != k * 3 or int(block_scales.shape[0]) != n:
        raise RuntimeError("fused_ternary_e8_gemm_fwd: packed_weight / block_scales do not match x")
    scales = block_scales if block_scales.dtype == torch.float16 else block_scales.to(torch.float16)
    return ops.linear(x.contiguous(), packed_weight.contiguous().view(-1), scales.contiguous().view(-1), bias, n, k, group_size)


def fused_ternary_e8_gemm_bwd_dx(grad_y: torch.Tensor, packed_weight: torch.Tensor, block_scales: torch.Tensor,
                                 in_features: int, group_size: int = 32) -> torch.Tensor:
    """Same schema as the reference's ``fused_ternary_e8_gemm_bwd_dx(Tensor grad_y, Tensor packed_weight,
    Tensor block_scales, int in_features, int group_size=32) -> Tensor``
    (``ojasx_math_bindings.cpp:479-533,594``): ``dX [M, K] = dY [M, N] . W [N, K]``, computed by the transposed
    tensor-core kernel straight from the packed codes for 16-bit gradients (``ops.linear_dx``)."""
    if grad_y.dim() != 2 or packed_weight.dim() != 2 or block_scales.dim() != 2:
        raise RuntimeError("fused_ternary_e8_gemm_bwd_dx expects 2-D grad_y, packed_weight and block_scales")
    n = int(packed_weight.shape[0])
    if int(grad_y.shape[1]) != n or int(packed_weight.shape[1]) * 16 != int(in_features) * 3:
        raise RuntimeError("fused_ternary_e8_gemm_bwd_dx: shapes do not match")
    scales = block_scales if block_scales.dtype == torch.float16 else block_scales.to(torch.float16)
    return ops.linear_dx(grad_y, packed_weight.contiguous().view(-1), scales.contiguous().view(-1), n, int(in_features), group_size)


def install_into_reference() -> bool:
    """Rebinds the reference's kernel seam (the module-level ``dispatch_tilelang_e8_gemm`` that
    ``_FusedE8GEMMFunction.forward`` calls first, ``ojasx2/math/lattice.py:51-55,583-589``) to this backend when the
    reference package is importable.  Returns True when the patch was applied.  The reference's second seam, the
    native module's ``fused_ternary_e8_gemm_fwd`` / ``_bwd_dx`` operators, is served by ``torch_ops.register()``:
    ``torch.ops.ojasx_math_native.*`` with the reference's schemas and a CUDA implementation."""
    try:
        import ojasx2.math.lattice as ref_lattice   # type: ignore
    except Exception:
        return False
    ref_lattice.dispatch_tilelang_e8_gemm = dispatch_tilelang_e8_gemm
    return True
