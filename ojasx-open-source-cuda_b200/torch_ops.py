"""``torch.ops.ojasx_math_native.fused_ternary_e8_gemm_fwd`` / ``_bwd_dx``, their 2.0-bit siblings ``fused_e8_gemm_fwd`` /
``_bwd_dx`` and ``conway_sloane_e8_project_tensor`` bound to the sm_100a kernels.

The reference registers these operators (with these schema strings) for its native CPU module
(``ojasx2/math/csrc/ojasx_math_bindings.cpp:586-595``) and reaches them as attributes of ``lattice._native``
(``ojasx2/math/lattice.py:591-608,656-681``).  Here they get a CUDA implementation (the fused decode-shape /
tcgen05 kernels behind ``hardware.fused_ternary_e8_gemm_fwd`` and the transposed kernel behind ``_bwd_dx``), a
fake (meta) implementation for tracing, and an autograd formula, so that a model holding ``E8LatticeLinear``
layers goes through ``torch.compile(fullgraph=True)`` without a graph break: the ctypes calls live inside
operators the compiler treats as opaque.  Operands are the reference's: ``x [M, K]``, row-major 2-D
``packed_weight [N, K*3/16]`` uint8 and ``block_scales [N, K/group]``.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import hardware, ops

NAMESPACE = "ojasx_math_native"
_FWD = "fused_ternary_e8_gemm_fwd(Tensor x, Tensor packed_weight, Tensor block_scales, Tensor? bias=None, int group_size=32) -> Tensor"
_BWD = "fused_ternary_e8_gemm_bwd_dx(Tensor grad_y, Tensor packed_weight, Tensor block_scales, int in_features, int group_size=32) -> Tensor"

_FWD2 = "fused_e8_gemm_fwd(Tensor x, Tensor packed_weight, Tensor block_scales, Tensor? bias=None, int group_size=32) -> Tensor"
_BWD2 = "fused_e8_gemm_bwd_dx(Tensor grad_y, Tensor packed_weight, Tensor block_scales, int in_features, int group_size=32) -> Tensor"
_PROJ = "conway_sloane_e8_project_tensor(Tensor x) -> Tensor"

_lib: Optional[torch.library.Library] = None


def _fwd2_cuda(x, packed_weight, block_scales, bias=None, group_size=32):
    # 2.0-bit operands as the reference's native module takes them: packed [N, K/4], scales [N, K/group]
    n, k = int(packed_weight.shape[0]), int(x.shape[1])
    return ops.linear_2bit(x, packed_weight.reshape(-1), block_scales.reshape(-1), bias, n, k, group_size)


def _bwd2_cuda(grad_y, packed_weight, block_scales, in_features, group_size=32):
    n = int(packed_weight.shape[0])
    return ops.linear_dx_lowbit(2, grad_y, packed_weight.reshape(-1), block_scales.reshape(-1), n, int(in_features), group_size)


def _proj_cuda(x):
    return ops.e8_project(x)


def _proj_fake(x):
    torch._check(x.shape[-1] == 8, lambda: "Last dimension must be 8 for E8 lattice")
    return torch.empty_like(x)


def _backward2(ctx, grad_y):
    packed_weight, block_scales = ctx.saved_tensors
    grad_x = torch.ops.ojasx_math_native.fused_e8_gemm_bwd_dx(grad_y.contiguous(), packed_weight, block_scales,
                                                              ctx.in_features, ctx.group_size)
    grad_bias = grad_y.sum(dim=0) if ctx.has_bias else None
    return grad_x, None, None, grad_bias, None


def _fwd_cuda(x, packed_weight, block_scales, bias=None, group_size=32):
    return hardware.fused_ternary_e8_gemm_fwd(x, packed_weight, block_scales, bias, group_size)


def _bwd_cuda(grad_y, packed_weight, block_scales, in_features, group_size=32):
    return hardware.fused_ternary_e8_gemm_bwd_dx(grad_y, packed_weight, block_scales, in_features, group_size)


def _fwd_fake(x, packed_weight, block_scales, bias=None, group_size=32):
    torch._check(x.dim() == 2 and packed_weight.dim() == 2 and block_scales.dim() == 2,
                 lambda: "fused_ternary_e8_gemm_fwd expects 2-D x, packed_weight and block_scales")
    return x.new_empty((x.shape[0], packed_weight.shape[0]))


def _bwd_fake(grad_y, packed_weight, block_scales, in_features, group_size=32):
    torch._check(grad_y.dim() == 2 and packed_weight.dim() == 2, lambda: "fused_ternary_e8_gemm_bwd_dx expects 2-D operands")
    return grad_y.new_empty((grad_y.shape[0], in_features))


def _setup_context(ctx, inputs, output):
    x, packed_weight, block_scales, bias, group_size = inputs
    ctx.save_for_backward(packed_weight, block_scales)
    ctx.in_features = x.shape[1]
    ctx.group_size = group_size
    ctx.has_bias = bias is not None


def _backward(ctx, grad_y):
    packed_weight, block_scales = ctx.saved_tensors
    grad_x = torch.ops.ojasx_math_native.fused_ternary_e8_gemm_bwd_dx(grad_y.contiguous(), packed_weight, block_scales,
                                                                      ctx.in_features, ctx.group_size)
    grad_bias = grad_y.sum(dim=0) if ctx.has_bias else None
    return grad_x, None, None, grad_bias, None


def register() -> bool:
    """Defines the operators (unless another library already did) and attaches the CUDA, fake and autograd
    implementations.  Idempotent; returns True when the operators are callable afterwards."""
    global _lib
    if _lib is not None:
        return True
    lib = torch.library.Library(NAMESPACE, "FRAGMENT")
    for schema in (_FWD, _BWD, _FWD2, _BWD2, _PROJ):
        name = schema.split("(")[0]
        if not hasattr(getattr(torch.ops, NAMESPACE), name):
            lib.define(schema)
    lib.impl("fused_ternary_e8_gemm_fwd", _fwd_cuda, "CUDA")
    lib.impl("fused_ternary_e8_gemm_bwd_dx", _bwd_cuda, "CUDA")
    torch.library.register_fake(f"{NAMESPACE}::fused_ternary_e8_gemm_fwd", _fwd_fake, lib=lib)
    torch.library.register_fake(f"{NAMESPACE}::fused_ternary_e8_gemm_bwd_dx", _bwd_fake, lib=lib)
    torch.library.register_autograd(f"{NAMESPACE}::fused_ternary_e8_gemm_fwd", _backward, setup_context=_setup_context, lib=lib)
    lib.impl("fused_e8_gemm_fwd", _fwd2_cuda, "CUDA")
    lib.impl("fused_e8_gemm_bwd_dx", _bwd2_cuda, "CUDA")
    lib.impl("conway_sloane_e8_project_tensor", _proj_cuda, "CUDA")
    torch.library.register_fake(f"{NAMESPACE}::fused_e8_gemm_fwd", _fwd_fake, lib=lib)
    torch.library.register_fake(f"{NAMESPACE}::fused_e8_gemm_bwd_dx", _bwd_fake, lib=lib)
    torch.library.register_fake(f"{NAMESPACE}::conway_sloane_e8_project_tensor", _proj_fake, lib=lib)
    torch.library.register_autograd(f"{NAMESPACE}::fused_e8_gemm_fwd", _backward2, setup_context=_setup_context, lib=lib)
    _lib = lib
    return True
