"""Host-side mirror of the reference's E8 quantized-linear interface, backed by the sm_100a kernels.

Same names, argument meaning and error behaviour as the reference module
``ojasx2/math/lattice.py`` (re-exported there as ``ojasx3.lattice``):

* :class:`TernaryE8LatticePacker`   (reference ``lattice.py:335-419``)  1.5 bits - the tensor-core path
* :class:`E8LatticePacker`          (reference ``lattice.py:207-279``)  2.0 bits
* :class:`RootE8LatticePacker`      (reference ``lattice.py:472-537``)  1.0 bit
* :class:`_FusedE8GEMMFunction`     (reference ``lattice.py:548-717``)
* :class:`E8LatticeLinear`          (reference ``lattice.py:724-846``)
* :func:`pack_model_e8`             (reference ``lattice.py:901-945``)
* :func:`fwht_block32`              (reference ``lattice.py:91-102``)
* :func:`conway_sloane_e8_project`, :class:`_E8STEFunction`, :class:`E8QuantizationAwareLinear`
                                    (reference ``lattice.py:162-203, 853-899``)
* :func:`_get_ternary_e8_luts`      (reference ``lattice.py:292-332``)

Differences, all deliberate: tensors must live on a CUDA device (the kernels are the only
implementation; nothing falls back to CPU or to PyTorch ops), and no dense weight matrix is ever
materialised in the forward pass (the 2.0- and 1.0-bit formats run one fused fp32 kernel instead of the
tensor-core kernels; their backward decodes the weights).
"""

from __future__ import annotations

import copy
import math
from typing import Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops

_SUPPORTED_BITRATES = (1.0, 1.5, 2.0)


def _check_bitrate(bitrate: float) -> None:
    """1.5 (ternary E8: the tensor-core path), 2.0 (four codes per byte) and 1.0 (one byte per 8-block) - the
    latter two with bit-exact packers and a fused fp32 linear."""
    if float(bitrate) not in _SUPPORTED_BITRATES:
        raise ValueError(f"Unsupported E8 bitrate {bitrate!r}; expected one of {list(_SUPPORTED_BITRATES)}")


class _Fwht32(torch.autograd.Function):
    """The transform is symmetric and orthogonal, so its adjoint is itself."""

    @staticmethod
    def forward(ctx, x):
        return ops.fwht32(x)

    @staticmethod
    def backward(ctx, grad):
        return ops.fwht32(grad)


def fwht_block32(x: torch.Tensor) -> torch.Tensor:
    """Normalised 32-point Walsh-Hadamard transform over consecutive blocks of the last dimension.

    Same butterfly order, roundings and final scaling as the reference (``lattice.py:91-102``), so results are
    bit-identical; tensors whose last dimension is not a multiple of 32 are returned unchanged.  CUDA tensors
    of the three float types take one kernel (``ops.fwht32``); anything else runs the tensor expression below.
    """
    if x.shape[-1] == 0 or x.shape[-1] % 32 != 0:
        return x
    if x.is_cuda and x.dtype in (torch.float32, torch.float16, torch.bfloat16) and x.numel() > 0 \
            and not torch.compiler.is_compiling():
        return _Fwht32.apply(x) if (x.requires_grad and torch.is_grad_enabled()) else ops.fwht32(x)
    h = x.reshape(-1, 32)
    span = 1
    while span < 32:
        v = h.reshape(-1, 32 // (2 * span), 2, span)
        a, b = v[:, :, 0, :], v[:, :, 1, :]
        h = torch.stack([a + b, a - b], dim=2).reshape(-1, 32)
        span *= 2
    return (h * 0.1767766952966369).reshape(x.shape)


def conway_sloane_e8_project(x: torch.Tensor, prefer_native: bool = True) -> torch.Tensor:
    """Snaps every 8-vector along the last dimension to the nearest point of E8 = D8 u (D8 + 1/2)
    (reference ``lattice.py:162-203``; ``prefer_native`` is accepted for signature compatibility - there is one
    implementation, the CUDA kernel)."""
    if torch.compiler.is_compiling() and x.numel() > 0:
        return torch.ops.ojasx_math_native.conway_sloane_e8_project_tensor(x)
    return ops.e8_project(x)


class _E8STEFunction(torch.autograd.Function):
    """E8 quantization with a straight-through gradient (reference ``lattice.py:853-867``)."""

    @staticmethod
    def forward(ctx, w: torch.Tensor) -> torch.Tensor:
        return ops.e8_ste_quantize(w)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor) -> torch.Tensor:
        return grad_output


class E8QuantizationAwareLinear(nn.Module):
    """Linear layer that trains dense weights through the E8 quantizer (reference ``lattice.py:870-899``)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, _E8STEFunction.apply(self.weight), self.bias)


_LUT_CACHE = {}


def _get_ternary_e8_luts(device: Optional[Union[str, torch.device]] = None):
    """``(rank_to_coords int8[3281,8], raw_to_rank int64[6561], powers int64[8])`` in the reference's
    enumeration order (``lattice.py:305-321``).  The kernels carry their own compiled-in tables; this
    function exists for callers that index the tables directly."""
    dev = torch.device("cpu") if device is None else torch.device(device)
    key = (dev.type, dev.index)
    if key not in _LUT_CACHE:
        raw = torch.arange(3 ** 8, dtype=torch.int64)
        digits = torch.stack([(raw // 3 ** i) % 3 for i in range(8)], dim=1) - 1
        valid = digits.sum(dim=1) % 2 == 0
        raw_to_rank = torch.zeros(3 ** 8, dtype=torch.int64)
        raw_to_rank[valid] = torch.arange(int(valid.sum()), dtype=torch.int64)
        coords = digits[valid].to(torch.int8)
        powers = torch.tensor([3 ** i for i in range(8)], dtype=torch.int64)
        _LUT_CACHE[key] = (coords.to(dev), raw_to_rank.to(dev), powers.to(dev))
    return _LUT_CACHE[key]


class TernaryE8LatticePacker:
    """Packs weight matrices into 1.50 bits/weight over D8 ∩ {-1, 0, +1}^8 (3,281 points)."""

    @staticmethod
    def pack(w: torch.Tensor, group_size: int = 32) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int]]:
        """Returns ``(packed uint8 1-D, scales float16 1-D, (rows, cols))``; bit-exact with the
        reference's CPU packer for fp32, fp16 and bf16 inputs."""
        if w.dim() != 2:
            raise ValueError(f"not enough values to unpack: expected a 2-D weight, got {tuple(w.shape)}")
        m, n = int(w.shape[0]), int(w.shape[1])
        src = w if w.dtype in (torch.float32, torch.float16, torch.bfloat16) else w.to(torch.float32)
        packed, scales = ops.encode(src, group_size)
        return packed, scales, (m, n)

    @staticmethod
    def unpack(packed_codes: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int],
               dtype: torch.dtype = torch.float32, use_workspace: bool = False) -> torch.Tensor:
        """Dense ``[rows, cols]`` weights in ``dtype``.  ``use_workspace`` is accepted for signature
        compatibility; the forward pass never needs a decoded matrix, so no cache is kept."""
        del use_workspace
        return ops.decode(packed_codes, scales, (int(shape[0]), int(shape[1])), dtype)


class E8LatticePacker:
    """2.0 bits/weight, four codes per byte (reference ``lattice.py:210-279``): same entry points and errors."""

    @staticmethod
    def pack(w: torch.Tensor, group_size: int = 8) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int]]:
        m, n = w.shape
        if group_size <= 0 or group_size % 8 != 0:
            raise ValueError(f"group_size ({group_size}) must be a positive multiple of 8.")
        src = w if w.dtype in (torch.float32, torch.float16, torch.bfloat16) else w.to(torch.float32)
        packed, scales = ops.encode_2bit(src, group_size)
        return packed, scales, (m, n)

    @staticmethod
    def unpack(packed_codes: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int],
               dtype: torch.dtype = torch.float32, use_workspace: bool = False) -> torch.Tensor:
        del use_workspace
        return ops.decode_2bit(packed_codes, scales, (int(shape[0]), int(shape[1])), dtype)


class RootE8LatticePacker:
    """1.0 bit/weight, one byte per 8-block indexing the 240 roots of E8 plus 16 axis vectors (reference
    ``lattice.py:472-537``): same entry points; codes and scales equal the reference's CPU results bit for bit."""

    @staticmethod
    def pack(w: torch.Tensor, group_size: int = 32) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int]]:
        m, n = w.shape
        src = w if w.dtype in (torch.float32, torch.float16, torch.bfloat16) else w.to(torch.float32)
        packed, scales = ops.encode_1bit(src, group_size)
        return packed, scales, (m, n)

    @staticmethod
    def unpack(packed_codes: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int],
               dtype: torch.dtype = torch.float32, use_workspace: bool = False) -> torch.Tensor:
        del use_workspace
        return ops.decode_1bit(packed_codes, scales, (int(shape[0]), int(shape[1])), dtype)


def _get_packer_for_bitrate(bitrate: float):
    if float(bitrate) == 1.0:
        return RootE8LatticePacker
    if float(bitrate) == 1.5:
        return TernaryE8LatticePacker
    return E8LatticePacker                      # the reference's default branch (lattice.py:536-541)


def _lowbit(bitrate: float) -> int:
    return 1 if float(bitrate) == 1.0 else 2


class _FusedE8GEMMFunction(torch.autograd.Function):
    """``y = x . dequant(W)^T + bias`` straight from the packed codes.

    Nine inputs and nine gradients, as in the reference (``lattice.py:551-563,717``).  Forward runs the
    fused kernels; x is not saved for backward (only the packed buffers are).  Backward computes
    ``dX = dY . W`` with the transposed tensor-core kernel straight from the packed codes for 16-bit
    gradients (``ops.linear_dx``); fp32 gradients decode W with the decode kernel and multiply.
    """

    @staticmethod
    def forward(ctx, x, packed_weight, block_scales, bias, out_features, in_features, group_size, bitrate,
                use_hadamard=False):
        _check_bitrate(bitrate)
        x_rot = fwht_block32(x) if (use_hadamard and in_features % 32 == 0) else x
        ctx.save_for_backward(packed_weight, block_scales)
        ctx.x_shape = x_rot.shape
        ctx.x_dtype = x_rot.dtype
        ctx.in_features = in_features
        ctx.out_features = out_features
        ctx.has_bias = bias is not None
        ctx.use_hadamard = use_hadamard
        ctx.group_size = group_size
        ctx.bitrate = float(bitrate)
        x_2d = x_rot.reshape(-1, in_features)
        if float(bitrate) == 1.0:
            y_2d = ops.linear_1bit(x_2d, packed_weight, block_scales, bias, out_features, in_features, group_size)
            return y_2d.reshape(*x_rot.shape[:-1], out_features)
        if float(bitrate) == 2.0:
            if torch.compiler.is_compiling() and in_features % group_size == 0:
                y_2d = torch.ops.ojasx_math_native.fused_e8_gemm_fwd(
                    x_2d, packed_weight.view(out_features, -1), block_scales.view(out_features, -1), bias, group_size)
            else:
                y_2d = ops.linear_2bit(x_2d, packed_weight, block_scales, bias, out_features, in_features, group_size)
            return y_2d.reshape(*x_rot.shape[:-1], out_features)
        eff = ops.effective_group(group_size)
        if torch.compiler.is_compiling() and in_features % eff == 0:
            # under torch.compile the kernels are reached through the registered operator, which the compiler
            # keeps as one opaque node (row-major 2-D operands, as the reference's native module takes them)
            y_2d = torch.ops.ojasx_math_native.fused_ternary_e8_gemm_fwd(
                x_2d, packed_weight.view(out_features, -1), block_scales.view(out_features, -1), bias, eff)
        else:
            y_2d = ops.linear(x_2d, packed_weight, block_scales, bias, out_features, in_features, group_size)
        return y_2d.reshape(*x_rot.shape[:-1], out_features)

    @staticmethod
    def backward(ctx, grad_y):
        packed_weight, block_scales = ctx.saved_tensors
        gy_2d = grad_y.reshape(-1, ctx.out_features).contiguous()
        eff = ops.effective_group(ctx.group_size)
        if ctx.bitrate == 1.0:
            grad_x = ops.linear_dx_lowbit(1, gy_2d.to(ctx.x_dtype), packed_weight, block_scales, ctx.out_features,
                                          ctx.in_features, ctx.group_size).reshape(ctx.x_shape)
        elif ctx.bitrate == 2.0:
            if torch.compiler.is_compiling() and ctx.in_features % ctx.group_size == 0:
                grad_x = torch.ops.ojasx_math_native.fused_e8_gemm_bwd_dx(
                    gy_2d.to(ctx.x_dtype), packed_weight.view(ctx.out_features, -1), block_scales.view(ctx.out_features, -1),
                    ctx.in_features, ctx.group_size).reshape(ctx.x_shape)
            else:
                grad_x = ops.linear_dx_lowbit(2, gy_2d.to(ctx.x_dtype), packed_weight, block_scales, ctx.out_features,
                                              ctx.in_features, ctx.group_size).reshape(ctx.x_shape)
        elif torch.compiler.is_compiling() and ctx.in_features % eff == 0:
            grad_x = torch.ops.ojasx_math_native.fused_ternary_e8_gemm_bwd_dx(
                gy_2d.to(ctx.x_dtype), packed_weight.view(ctx.out_features, -1), block_scales.view(ctx.out_features, -1),
                ctx.in_features, eff).reshape(ctx.x_shape)
        else:
            grad_x = ops.linear_dx(gy_2d.to(ctx.x_dtype), packed_weight, block_scales, ctx.out_features, ctx.in_features,
                                   ctx.group_size).reshape(ctx.x_shape)
        if ctx.use_hadamard and ctx.in_features % 32 == 0:
            grad_x = fwht_block32(grad_x)
        grad_bias = gy_2d.sum(dim=0) if ctx.has_bias else None
        return grad_x, None, None, grad_bias, None, None, None, None, None


class E8LatticeLinear(nn.Module):
    """Linear layer whose base weights are packed ternary-E8 codes (buffers ``packed_weight`` uint8 and
    ``block_scales`` float16, optional ``bias`` and LoRA factors ``lora_A [K, r]``, ``lora_B [r, N]``);
    state-dict compatible with the reference layer (``lattice.py:727-781``)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, rank: int = 0,
                 lora_alpha: float = 16.0, group_size: int = 8, bitrate: float = 2.0, use_hadamard: bool = False,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        _check_bitrate(bitrate)
        self.in_features = in_features
        self.out_features = out_features
        self.rank = rank
        self.lora_alpha = lora_alpha
        self.scaling = (lora_alpha / rank) if rank > 0 else 0.0
        self.bitrate = float(bitrate)
        self.use_hadamard = bool(use_hadamard and (in_features % 32 == 0))
        if self.bitrate == 1.5:
            eff_group = group_size if (group_size >= 16 and group_size % 16 == 0) else 16
            num_bytes, num_scales = ops.packed_sizes(out_features, in_features, eff_group)
        else:
            eff_group = group_size if (group_size >= 8 and group_size % 8 == 0) else 8
            num_bytes, num_scales = ops.packed_sizes_lowbit(_lowbit(self.bitrate), out_features, in_features, eff_group)
        self.group_size = eff_group
        self.register_buffer("packed_weight", torch.zeros(num_bytes, dtype=torch.uint8, device=device))
        self.register_buffer("block_scales", torch.ones(num_scales, dtype=torch.float16, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)
        if rank > 0:
            self.lora_A = nn.Parameter(torch.zeros(in_features, rank, dtype=dtype, device=device))
            self.lora_B = nn.Parameter(torch.zeros(rank, out_features, dtype=dtype, device=device))
            nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B)
        else:
            self.register_parameter("lora_A", None)
            self.register_parameter("lora_B", None)

    @classmethod
    def from_linear(cls, linear: nn.Linear, rank: int = 0, lora_alpha: float = 16.0, group_size: int = 8,
                    bitrate: float = 2.0, use_hadamard: bool = False) -> "E8LatticeLinear":
        _check_bitrate(bitrate)
        eff_gs = max(16, group_size) if float(bitrate) == 1.5 else group_size
        m = cls(linear.in_features, linear.out_features, bias=(linear.bias is not None), rank=rank,
                lora_alpha=lora_alpha, group_size=eff_gs, bitrate=bitrate, use_hadamard=use_hadamard,
                device=linear.weight.device, dtype=linear.weight.dtype)
        with torch.no_grad():
            encode = ops.encode if m.bitrate == 1.5 else (ops.encode_1bit if m.bitrate == 1.0 else ops.encode_2bit)
            encode(linear.weight, m.group_size, out=(m.packed_weight, m.block_scales), hadamard=m.use_hadamard)
            if linear.bias is not None:
                m.bias.copy_(linear.bias)
        return m

    def unpack_weights(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        w = _get_packer_for_bitrate(self.bitrate).unpack(self.packed_weight, self.block_scales,
                                                         (self.out_features, self.in_features), dtype=dtype)
        return fwht_block32(w) if self.use_hadamard else w

    def _forward_decode_with_adapter(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Inference at decode shapes with an adapter: the low-rank term rides in the GEMV's epilogue (one launch for
        the packed product, the adapter's second factor, the scaling and the addition); ``None`` when it does not apply."""
        if self.rank <= 0 or self.lora_A is None or not x.is_cuda or torch.compiler.is_compiling():
            return None
        if torch.is_grad_enabled() and (x.requires_grad or self.lora_A.requires_grad or self.lora_B.requires_grad
                                        or (self.bias is not None and self.bias.requires_grad)):
            return None
        x_2d = x.reshape(-1, self.in_features)
        if self.bitrate != 1.5:                          # the sibling formats: their int8 tensor-core decode kernels
            if not ops.lowbit_lora_fusable(int(x_2d.shape[0]), self.in_features, self.group_size, self.rank):
                return None
            t = (x_2d @ self.lora_A.to(x.dtype)).float() * self.scaling
            x_rot = fwht_block32(x_2d) if (self.use_hadamard and self.in_features % 32 == 0) else x_2d
            y = ops.linear_lowbit_lora(_lowbit(self.bitrate), x_rot, self.packed_weight, self.block_scales, self.bias,
                                       self.out_features, self.in_features, self.group_size, t, self.lora_B)
            return y.reshape(*x.shape[:-1], self.out_features)
        if not ops.lora_fusable(int(x_2d.shape[0]), self.in_features, self.group_size, x.dtype, self.rank):
            return None
        t = (x_2d @ self.lora_A.to(x.dtype)).float() * self.scaling
        x_rot = fwht_block32(x_2d) if self.use_hadamard else x_2d
        y = ops.linear_lora(x_rot, self.packed_weight, self.block_scales, self.bias, self.out_features, self.in_features,
                            self.group_size, t, self.lora_B)
        return y.reshape(*x.shape[:-1], self.out_features)

    def forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        fused = self._forward_decode_with_adapter(x)
        if fused is not None:
            return fused
        out = _FusedE8GEMMFunction.apply(x, self.packed_weight, self.block_scales, self.bias, self.out_features,
                                         self.in_features, self.group_size, self.bitrate, self.use_hadamard)
        if self.rank > 0 and self.lora_A is not None and self.lora_B is not None:
            lora_a = self.lora_A.to(x.dtype) if self.lora_A.dtype != x.dtype else self.lora_A
            lora_b = self.lora_B.to(x.dtype) if self.lora_B.dtype != x.dtype else self.lora_B
            out = out + self.scaling * ((x @ lora_a) @ lora_b)
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_fused(x)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bitrate={self.bitrate}, "
                f"group_size={self.group_size}, rank={self.rank}, use_hadamard={self.use_hadamard}")


def pack_model_e8(model: nn.Module, rank: int = 0, lora_alpha: float = 16.0, group_size: int = 32,
                  bitrate: float = 2.0, use_hadamard: bool = False,
                  target_modules: Optional[Union[list, tuple, str]] = None,
                  exclude_modules: Optional[Union[list, tuple]] = None, inplace: bool = True) -> nn.Module:
    """Recursively replaces ``nn.Linear`` children by :class:`E8LatticeLinear` (``lattice.py:901-945``);
    name filters are substring matches on the child name, as in the reference."""
    _check_bitrate(bitrate)
    target_model = model if inplace else copy.deepcopy(model)
    if isinstance(target_modules, str):
        target_modules = [target_modules]
    for name, module in target_model.named_children():
        if exclude_modules is not None and any(ex in name for ex in exclude_modules):
            continue
        targeted = True if target_modules is None else any(t in name for t in target_modules)
        if isinstance(module, nn.Linear) and targeted:
            setattr(target_model, name, E8LatticeLinear.from_linear(
                module, rank=rank, lora_alpha=lora_alpha, group_size=group_size, bitrate=bitrate,
                use_hadamard=use_hadamard))
        else:
            pack_model_e8(module, rank=rank, lora_alpha=lora_alpha, group_size=group_size, bitrate=bitrate,
                          use_hadamard=use_hadamard, target_modules=target_modules,
                          exclude_modules=exclude_modules, inplace=True)
    return target_model
