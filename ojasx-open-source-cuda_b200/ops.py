"""Tensor-level wrappers over the C ABI: encode, decode, decode-shape and prefill-shape linear.

torch is used only for device memory and streams; every computation is a call into
``libojx_e8t.so`` through plain pointers.  All functions require CUDA tensors and raise if
the library is missing - there is no CPU or PyTorch fallback on this path.
"""

from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _cabi

_DT = {torch.float32: _cabi.OJX_F32, torch.float16: _cabi.OJX_F16, torch.bfloat16: _cabi.OJX_BF16}

# Largest M handled by the decode-shape kernel; larger batches go to the tensor-core GEMM.
GEMV_MAX_M = 16

_scratch: Dict[Tuple[int, int, str], torch.Tensor] = {}


def _dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; expected float32, float16 or bfloat16") from None


def _require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("the B200 ternary-E8 backend needs CUDA tensors (no CPU fallback on this path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def scratch(device: torch.device, nbytes: int, tag: str = "ws") -> torch.Tensor:
    """Grow-only scratch buffer per (device, stream, tag) - the counterpart of the reference's
    ``_get_ephemeral_workspace`` (ojasx2/math/lattice.py:62-84), but only a few KB..MB of fp32
    partial sums instead of a full decoded weight matrix."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           int(torch.cuda.current_stream(device).cuda_stream), tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def effective_group(group_size: int) -> int:
    """The packer's coercion rule (ojasx2/math/lattice.py:346-347)."""
    return 16 if (group_size <= 0 or group_size % 16 != 0) else int(group_size)


def packed_sizes(rows: int, cols: int, group_size: int) -> Tuple[int, int]:
    g = effective_group(group_size)
    total = rows * cols
    padded = total + ((-total) % g)
    return padded * 3 // 16, padded // g


def fwht32(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Normalised 32-point Walsh-Hadamard transform of consecutive blocks of the last dimension, one kernel,
    bit-identical to the reference's ``fwht_block32`` (``ojasx2/math/lattice.py:91-102``)."""
    dev = _require_cuda(x)
    if x.shape[-1] % 32 != 0 or x.numel() == 0:
        raise ValueError("the last dimension must be a positive multiple of 32")
    xc = x.detach().contiguous()
    if xc.data_ptr() % 16:
        xc = xc.clone()
    res = torch.empty_like(xc) if out is None else out
    if res.shape != xc.shape or res.dtype != xc.dtype or not res.is_contiguous() or res.data_ptr() % 16:
        raise ValueError("output buffer has the wrong shape, dtype, layout or alignment")
    with torch.cuda.device(dev):
        st = _cabi.lib().ojx_e8t_fwht32(xc.data_ptr(), _dtype_code(xc.dtype), xc.numel(), res.data_ptr(), _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_fwht32")
    return res


def _lowbit_group(bits: int, group_size: int) -> int:
    """Group size as the reference's packers treat it: the 2.0-bit packer raises for anything that is not a positive
    multiple of 8 (``lattice.py:219-220``), the 1.0-bit packer replaces it by 8 (``lattice.py:485-486``)."""
    if group_size <= 0 or group_size % 8 != 0:
        if bits == 2:
            raise ValueError(f"group_size ({group_size}) must be a positive multiple of 8.")
        return 8
    return int(group_size)


def packed_sizes_lowbit(bits: int, rows: int, cols: int, group_size: int) -> Tuple[int, int]:
    """(code bytes, scales) of the 2.0-bit (four codes per byte) or 1.0-bit (one byte per eight weights) format."""
    g = _lowbit_group(bits, group_size)
    total = rows * cols
    padded = total + ((-total) % g)
    return (padded // 4 if bits == 2 else padded // 8), padded // g


def packed_sizes_2bit(rows: int, cols: int, group_size: int) -> Tuple[int, int]:
    return packed_sizes_lowbit(2, rows, cols, group_size)


def _encode_lowbit(bits: int, w: torch.Tensor, group_size: int, out, hadamard: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    if w.dim() != 2:
        raise ValueError(f"expected a 2-D weight, got shape {tuple(w.shape)}")
    dev = _require_cuda(w)
    rows, cols = int(w.shape[0]), int(w.shape[1])
    g = _lowbit_group(bits, group_size)
    nbytes, nscales = packed_sizes_lowbit(bits, rows, cols, g)
    if rows == 0 or cols == 0:
        raise ValueError("empty weight")
    wc = w.detach().contiguous()
    if hadamard and cols % 32 == 0:
        wc = fwht32(wc)
    if out is None:
        packed = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        scales = torch.empty(nscales, dtype=torch.float16, device=dev)
    else:
        packed, scales = out
        if packed.numel() != nbytes or scales.numel() != nscales or packed.dtype != torch.uint8 \
                or scales.dtype != torch.float16 or not packed.is_contiguous() or not scales.is_contiguous():
            raise ValueError("output buffers have the wrong size, dtype or layout")
    name = "ojx_e8t_encode_2bit" if bits == 2 else "ojx_e8t_encode_1bit"
    with torch.cuda.device(dev):
        st = getattr(_cabi.lib(), name)(wc.data_ptr(), _dtype_code(wc.dtype), rows, cols, g, packed.data_ptr(),
                                        scales.data_ptr(), _stream_ptr(dev))
    _cabi.check(st, name)
    return packed, scales


def _decode_lowbit(bits: int, packed: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int], dtype: torch.dtype) -> torch.Tensor:
    dev = _require_cuda(packed, scales)
    rows, cols = int(shape[0]), int(shape[1])
    group = (packed.numel() * (4 if bits == 2 else 8)) // max(1, scales.numel())
    out = torch.empty((rows, cols), dtype=dtype, device=dev)
    name = "ojx_e8t_decode_2bit" if bits == 2 else "ojx_e8t_decode_1bit"
    with torch.cuda.device(dev):
        st = getattr(_cabi.lib(), name)(packed.contiguous().data_ptr(), scales.contiguous().data_ptr(), rows, cols, group,
                                        _dtype_code(dtype), out.data_ptr(), _stream_ptr(dev))
    _cabi.check(st, name)
    return out


LOWBIT_GEMV_MAX_M = 8      # rows of x the decode kernels of the 2.0-bit / 1.0-bit formats take


def _linear_lowbit(bits: int, x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor],
                   n: int, k: int, group_size: int, out_dtype: Optional[torch.dtype]) -> torch.Tensor:
    dev = _require_cuda(x, packed, scales)
    x2 = x.detach().reshape(-1, k).contiguous()
    m = int(x2.shape[0])
    y = torch.empty((m, n), dtype=out_dtype or x2.dtype, device=dev)
    if m == 0:
        return y
    b = None if bias is None else bias.detach().to(x2.dtype).contiguous()
    lib = _cabi.lib()
    # the decode kernels on int8 tensor cores take groups of 32 with K % 2048 == 0; where only the fp32 decode kernel is
    # left, the prefill kernel is already the faster one from four rows on (measured on 14336 x 4096, groups of 8:
    # 59 against 50 us at four rows)
    decode_tc = int(group_size) == 32 and k % 2048 == 0
    if ((m > LOWBIT_GEMV_MAX_M or (m >= 4 and not decode_tc)) and int(group_size) in (8, 16, 32) and k % 256 == 0
            and x2.dtype in (torch.bfloat16, torch.float16)
            and packed.numel() * (4 if bits == 2 else 8) == n * k
            and (x2.data_ptr() | packed.data_ptr() | scales.data_ptr()) % 16 == 0):
        # batches of tokens: the tcgen05 prefill kernel with this format's decoder
        with torch.cuda.device(dev):
            ws = _gemm_scratch(dev, lib.ojx_e8t_gemm_workspace_bytes(m, n, k))
            st = lib.ojx_e8t_gemm_lowbit(bits, x2.data_ptr(), _dtype_code(x2.dtype), m, packed.data_ptr(), scales.data_ptr(),
                                         None if b is None else b.data_ptr(), n, k, int(group_size), y.data_ptr(), _dtype_code(y.dtype),
                                         ws.data_ptr(), ws.numel(), _stream_ptr(dev))
        _cabi.check(st, "ojx_e8t_gemm_lowbit")
        return y
    name = "ojx_e8t_linear_2bit" if bits == 2 else "ojx_e8t_linear_1bit"
    with torch.cuda.device(dev):
        st = getattr(_cabi.lib(), name)(x2.data_ptr(), _dtype_code(x2.dtype), m, packed.data_ptr(), scales.data_ptr(),
                                        None if b is None else b.data_ptr(), n, k, int(group_size), y.data_ptr(),
                                        _dtype_code(y.dtype), _stream_ptr(dev))
    _cabi.check(st, name)
    return y


def lowbit_lora_fusable(m: int, k: int, group_size: int, rank: int) -> bool:
    """Shapes for which the adapter term can ride in the epilogue of the 2.0-bit / 1.0-bit decode kernels
    (``ojx_e8t_linear_lowbit_lora``)."""
    return 1 <= m <= 8 and int(group_size) == 32 and k % 2048 == 0 and m * k <= 32768 and 0 < rank <= 64


def linear_lowbit_lora(bits: int, x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor],
                       n: int, k: int, group_size: int, lora_t: torch.Tensor, lora_b: torch.Tensor,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = x . W^T (+ bias) + lora_t . lora_b`` for the 2.0-bit (``bits`` 2) or 1.0-bit (``bits`` 1) format in ONE
    decode-shape launch; ``lora_t`` [M, r] fp32 is ``scaling * (x . A)``, ``lora_b`` [r, N]."""
    dev = _require_cuda(x, packed, scales)
    x2 = x.detach().reshape(-1, k).contiguous()
    m, r = int(x2.shape[0]), int(lora_b.shape[0])
    if not lowbit_lora_fusable(m, k, group_size, r):
        raise ValueError("this shape cannot take the fused adapter term; add it separately")
    if tuple(lora_t.shape) != (m, r) or tuple(lora_b.shape) != (r, n):
        raise ValueError("lora_t must be [M, r] and lora_b [r, N]")
    t = lora_t.detach().to(torch.float32).contiguous()
    bb = lora_b.detach().to(x2.dtype).contiguous()
    b = None if bias is None else bias.detach().to(x2.dtype).contiguous()
    y = torch.empty((m, n), dtype=out_dtype or x2.dtype, device=dev)
    with torch.cuda.device(dev):
        st = _cabi.lib().ojx_e8t_linear_lowbit_lora(bits, x2.data_ptr(), _dtype_code(x2.dtype), m, packed.data_ptr(), scales.data_ptr(),
                                                    None if b is None else b.data_ptr(), n, k, 32, t.data_ptr(), bb.data_ptr(), r,
                                                    y.data_ptr(), _dtype_code(y.dtype), _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_linear_lowbit_lora")
    return y


def encode_2bit(w: torch.Tensor, group_size: int = 8, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                hadamard: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w`` [rows, cols] -> (packed uint8[P/4], scales fp16[P/g]) in the 2.0-bit format; bit-exact with the
    reference's ``E8LatticePacker.pack`` (``ojasx2/math/lattice.py:210-248``)."""
    return _encode_lowbit(2, w, group_size, out, hadamard)


def decode_2bit(packed: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int],
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """2-bit codes + scales -> dense [rows, cols] in ``dtype``; the group size is inferred from the buffer sizes
    as the reference does (``ojasx2/math/lattice.py:262-264``)."""
    return _decode_lowbit(2, packed, scales, shape, dtype)


def linear_2bit(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor], n: int, k: int,
                group_size: int, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = x . W^T (+ bias)`` from 2-bit codes: up to eight rows of x run the decode kernels (int8 tensor cores for
    groups of 32 and K % 2048 == 0), more rows with 16-bit activations, groups of 8, 16 or 32 and K % 256 == 0 the tcgen05
    prefill kernel (weights rounded to fp16 once, as ``decode_2bit(..., torch.float16)`` gives them), anything else
    a scalar fp32 kernel."""
    return _linear_lowbit(2, x, packed, scales, bias, n, k, group_size, out_dtype)


def encode_1bit(w: torch.Tensor, group_size: int = 32, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                hadamard: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w`` [rows, cols] -> (packed uint8[P/8], scales fp16[P/g]) in the 1.0-bit format; bit-exact with the
    reference's ``RootE8LatticePacker.pack`` on its CPU path (``ojasx2/math/lattice.py:475-512``)."""
    return _encode_lowbit(1, w, group_size, out, hadamard)


def decode_1bit(packed: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int],
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Root codes + scales -> dense [rows, cols] in ``dtype`` (``ojasx2/math/lattice.py:514-537``)."""
    return _decode_lowbit(1, packed, scales, shape, dtype)


def linear_1bit(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor], n: int, k: int,
                group_size: int, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = x . W^T (+ bias)`` from root codes; routed as :func:`linear_2bit` (here the fp16 weights of the
    prefill kernel are exact)."""
    return _linear_lowbit(1, x, packed, scales, bias, n, k, group_size, out_dtype)


def _fp32_pass(x: torch.Tensor, name: str, vectors: bool) -> torch.Tensor:
    dev = _require_cuda(x)
    src = x.detach().to(torch.float32).contiguous()
    if src.data_ptr() % 16:
        src = src.clone()
    res = torch.empty_like(src)
    with torch.cuda.device(dev):
        fn = getattr(_cabi.lib(), name)
        st = fn(src.data_ptr(), src.numel() // 8 if vectors else src.numel(), res.data_ptr(), _stream_ptr(dev))
    _cabi.check(st, name)
    return res if x.dtype == torch.float32 else res.to(x.dtype)


def e8_project(x: torch.Tensor) -> torch.Tensor:
    """Nearest E8 lattice point of every 8-vector along the last dimension (one kernel; bit-identical to the
    reference's ``conway_sloane_e8_project`` on fp32 tensors; 16-bit tensors are projected in fp32 and
    rounded back)."""
    if x.shape[-1] != 8:
        raise ValueError(f"Last dimension must be 8 for E8 lattice (got {x.shape[-1]}).")
    if x.numel() == 0:
        return x.clone()
    return _fp32_pass(x, "ojx_e8t_project", True)


def e8_ste_quantize(w: torch.Tensor) -> torch.Tensor:
    """Forward of the reference's ``_E8STEFunction``: groups of eight consecutive elements scaled by their rms,
    projected to E8 and scaled back, one kernel (bit-identical on fp32 tensors)."""
    if w.numel() == 0:
        return w.clone()
    return _fp32_pass(w, "ojx_e8t_ste_quantize", False)


def encode(w: torch.Tensor, group_size: int = 32, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
           hadamard: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w`` [rows, cols] -> (packed uint8[P*3/16], scales fp16[P/g]); bit-exact with the
    reference's ``TernaryE8LatticePacker.pack``.  ``hadamard=True`` encodes ``fwht_block32(w)`` without
    materialising it (rotation fused into the encoder when the group is 32, one extra kernel otherwise)."""
    if w.dim() != 2:
        raise ValueError(f"expected a 2-D weight, got shape {tuple(w.shape)}")
    dev = _require_cuda(w)
    rows, cols = int(w.shape[0]), int(w.shape[1])
    if rows == 0 or cols == 0:
        raise ValueError("empty weight")
    wc = w.detach().contiguous()
    flags = 0
    if hadamard and cols % 32 == 0:
        if effective_group(group_size) == 32:
            flags = _cabi.OJX_ENCODE_HADAMARD
        else:
            wc = fwht32(wc)
    nbytes, nscales = packed_sizes(rows, cols, group_size)
    if out is None:
        packed = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        scales = torch.empty(nscales, dtype=torch.float16, device=dev)
    else:
        packed, scales = out
        if packed.numel() != nbytes or scales.numel() != nscales or packed.dtype != torch.uint8 \
                or scales.dtype != torch.float16 or not packed.is_contiguous() or not scales.is_contiguous():
            raise ValueError("output buffers have the wrong size, dtype or layout")
    with torch.cuda.device(dev):
        st = _cabi.lib().ojx_e8t_encode_ex(wc.data_ptr(), _dtype_code(wc.dtype), rows, cols, int(group_size), flags,
                                           packed.data_ptr(), scales.data_ptr(), _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_encode_ex")
    return packed, scales


def decode(packed: torch.Tensor, scales: torch.Tensor, shape: Tuple[int, int], dtype: torch.dtype = torch.float32,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed codes + scales -> dense [rows, cols] in ``dtype`` (the group size is inferred from the
    buffer sizes exactly as the reference does, ojasx2/math/lattice.py:407-409)."""
    dev = _require_cuda(packed, scales)
    rows, cols = int(shape[0]), int(shape[1])
    if packed.dtype != torch.uint8 or scales.dtype != torch.float16:
        raise TypeError("packed must be uint8 and scales float16")
    if packed.numel() % 3 != 0:
        raise ValueError("packed length must be a multiple of 3")
    padded = (packed.numel() // 3) * 16
    group = padded // max(1, scales.numel())
    if rows * cols > padded or group % 16 != 0 or group * scales.numel() != padded:
        raise ValueError("packed/scales sizes are inconsistent with the requested shape")
    pk, sc = packed.contiguous(), scales.contiguous()
    if out is None:
        out = torch.empty((rows, cols), dtype=dtype, device=dev)
    elif out.numel() != rows * cols or out.dtype != dtype or not out.is_contiguous():
        raise ValueError("output buffer has the wrong size, dtype or layout")
    with torch.cuda.device(dev):
        st = _cabi.lib().ojx_e8t_decode(pk.data_ptr(), sc.data_ptr(), rows, cols, group, _dtype_code(dtype),
                                        out.data_ptr(), _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_decode")
    return out.view(rows, cols)


def generate(count: int, seed: int, sigma: float, dtype: torch.dtype, device: torch.device, start: int = 0,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Seeded ~N(0, sigma) values produced on the device (same bits as the numpy generator of the test oracle)."""
    if out is None:
        out = torch.empty(count, dtype=dtype, device=device)
    with torch.cuda.device(device):
        st = _cabi.lib().ojx_e8t_generate(out.data_ptr(), _dtype_code(dtype), int(count), int(seed) & (2 ** 64 - 1),
                                          int(start), float(sigma), _stream_ptr(out.device))
    _cabi.check(st, "ojx_e8t_generate")
    return out


def _prep_linear(x2d, packed, scales, bias, n, k):
    dev = _require_cuda(x2d, packed, scales, bias)
    if x2d.dim() != 2 or x2d.shape[1] != k:
        raise ValueError(f"x must be [M, {k}], got {tuple(x2d.shape)}")
    if packed.dtype != torch.uint8 or scales.dtype != torch.float16:
        raise TypeError("packed must be uint8 and scales float16")
    x2d = x2d.contiguous()
    b = None
    if bias is not None:
        if bias.numel() != n:
            raise ValueError("bias has the wrong length")
        b = bias.detach().to(x2d.dtype).contiguous()       # the reference casts bias to x's dtype (lattice.py:622)
    return dev, x2d, packed.contiguous(), scales.contiguous(), b


def lora_fusable(m: int, k: int, group_size: int, dtype: torch.dtype, rank: int) -> bool:
    """Shapes for which the adapter term can ride in the decode kernel's epilogue (``ojx_e8t_gemv_lora``)."""
    return (1 <= m <= 8 and k % 256 == 0 and effective_group(group_size) == 32
            and dtype in (torch.bfloat16, torch.float16) and 0 < rank <= 64)


def linear_lora(x2d: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor],
                out_features: int, in_features: int, group_size: int, lora_t: torch.Tensor, lora_b: torch.Tensor,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = x . dequant(W)^T (+ bias) + lora_t . lora_b`` in ONE decode-shape launch: ``lora_t`` [M, r] fp32 is
    ``scaling * (x . A)``, ``lora_b`` [r, N]; the low-rank term is accumulated in fp32 in the kernel's epilogue
    (the reference adds it with three more tensor operations, ``ojasx2/math/lattice.py:839-842``)."""
    n, k = int(out_features), int(in_features)
    dev, x2d, pk, sc, b = _prep_linear(x2d, packed, scales, bias, n, k)
    _cabi.raise_pending()
    m, r = int(x2d.shape[0]), int(lora_b.shape[0])
    if not lora_fusable(m, k, group_size, x2d.dtype, r):
        raise ValueError("this shape cannot take the fused adapter term; add it separately")
    if tuple(lora_t.shape) != (m, r) or tuple(lora_b.shape) != (r, n):
        raise ValueError("lora_t must be [M, r] and lora_b [r, N]")
    t = lora_t.detach().to(torch.float32).contiguous()
    bb = lora_b.detach().to(x2d.dtype).contiguous()
    y = torch.empty((m, n), dtype=out_dtype or x2d.dtype, device=dev)
    lib = _cabi.lib()
    with torch.cuda.device(dev):
        need = lib.ojx_e8t_gemv_workspace_bytes(m, n, k)
        ws = scratch(dev, need, "gemv") if need else None
        st = lib.ojx_e8t_gemv_lora(x2d.data_ptr(), _dtype_code(x2d.dtype), m, pk.data_ptr(), sc.data_ptr(),
                                   b.data_ptr() if b is not None else None, n, k, 32, t.data_ptr(), bb.data_ptr(), r,
                                   y.data_ptr(), _dtype_code(y.dtype), ws.data_ptr() if ws is not None else None,
                                   ws.numel() if ws is not None else 0, _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_gemv_lora")
    return y


def linear(x2d: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor],
           out_features: int, in_features: int, group_size: int = 32,
           out_dtype: Optional[torch.dtype] = None, force: Optional[str] = None) -> torch.Tensor:
    """y[M, N] = x[M, K] . dequant(W)^T (+ bias), output in x's dtype unless ``out_dtype`` is given.

    Routing: M <= 16 -> decode-shape kernel (``ojx_e8t_gemv``); larger M with K % 256 == 0, 16-bit
    activations and groups of 32 or 16 -> tcgen05 kernel (``ojx_e8t_gemm``; groups of 16 take it from three rows on);
    everything else -> inside ``ojx_e8t_gemv`` the shared-memory fp32 kernel (up to eight rows, K % 64 == 0, groups
    of 16, 32, 64, ...; any activation dtype) or the scalar kernel.  ``force`` ("gemv" or "gemm") overrides the routing for tests.
    """
    n, k = int(out_features), int(in_features)
    dev, x2d, pk, sc, b = _prep_linear(x2d, packed, scales, bias, n, k)
    _cabi.raise_pending()
    m = int(x2d.shape[0])
    ydt = out_dtype or x2d.dtype
    y = torch.empty((m, n), dtype=ydt, device=dev)
    if m == 0:
        return y
    g = effective_group(group_size)
    lib = _cabi.lib()
    # groups of 16 (what the reference layer's default group size of 8 becomes for this format) have no tensor-core
    # decode kernel: one or two rows run the shared-memory fp32 kernel inside ojx_e8t_gemv, more rows the prefill kernel
    # (measured on 14336 x 4096 with the wrapper: 35 against 54 us at one row, 82 against 54 us at four)
    use_gemm = ((m > GEMV_MAX_M or (g == 16 and m > 2)) and k % 256 == 0 and g in (16, 32) and x2d.dtype in (torch.bfloat16, torch.float16)
                and (k * 3 // 16) * n == pk.numel())
    if force == "gemm":
        use_gemm = True
    elif force == "gemv":
        use_gemm = False
    with torch.cuda.device(dev):
        if use_gemm:
            need = lib.ojx_e8t_gemm_workspace_bytes(m, n, k)
            ws = _gemm_scratch(dev, need)
            st = lib.ojx_e8t_gemm(x2d.data_ptr(), _dtype_code(x2d.dtype), m, pk.data_ptr(), sc.data_ptr(),
                                  b.data_ptr() if b is not None else None, n, k, g, y.data_ptr(), _dtype_code(ydt),
                                  ws.data_ptr(), ws.numel(), _stream_ptr(dev))
            _cabi.check(st, "ojx_e8t_gemm")
        else:
            need = lib.ojx_e8t_gemv_workspace_bytes(m, n, k)
            ws = scratch(dev, need, "gemv") if need else None
            st = lib.ojx_e8t_gemv(x2d.data_ptr(), _dtype_code(x2d.dtype), m, pk.data_ptr(), sc.data_ptr(),
                                  b.data_ptr() if b is not None else None, n, k, g, y.data_ptr(), _dtype_code(ydt),
                                  ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                  _stream_ptr(dev))
            _cabi.check(st, "ojx_e8t_gemv")
    return y


def linear_dx(grad_y2d: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, out_features: int, in_features: int,
              group_size: int = 32, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """dX[M, K] = dY[M, N] . dequant(W)[N, K] straight from the packed codes (``ojx_e8t_gemm_dx``): the backward of
    :func:`linear` with respect to its input, without a decoded copy of W.  Shapes the tensor-core kernel does not
    take (fp32 gradients, K % 256 != 0, N % 8 != 0, another group size) decode W with the decode kernel and multiply."""
    n, k = int(out_features), int(in_features)
    dev = _require_cuda(grad_y2d, packed, scales)
    if grad_y2d.dim() != 2 or grad_y2d.shape[1] != n:
        raise ValueError(f"grad_y must be [M, {n}], got {tuple(grad_y2d.shape)}")
    if packed.dtype != torch.uint8 or scales.dtype != torch.float16:
        raise TypeError("packed must be uint8 and scales float16")
    gy = grad_y2d.contiguous()
    m = int(gy.shape[0])
    ydt = out_dtype or gy.dtype
    g = effective_group(group_size)
    if m == 0:
        return torch.empty((0, k), dtype=ydt, device=dev)
    fast = (gy.dtype in (torch.bfloat16, torch.float16) and k % 256 == 0 and n % 8 == 0 and g in (16, 32)
            and (k * 3 // 16) * n == packed.numel())
    if not fast:
        w = decode(packed, scales, (n, k), gy.dtype if gy.dtype.is_floating_point else torch.float32)
        return gy.matmul(w).to(ydt)
    _cabi.raise_pending()
    pk, sc = packed.contiguous(), scales.contiguous()
    dx = torch.empty((m, k), dtype=ydt, device=dev)
    lib = _cabi.lib()
    with torch.cuda.device(dev):
        ws = _gemm_scratch(dev, lib.ojx_e8t_gemm_dx_workspace_bytes(m, n, k))
        st = lib.ojx_e8t_gemm_dx(gy.data_ptr(), _dtype_code(gy.dtype), m, pk.data_ptr(), sc.data_ptr(), n, k, g,
                                 dx.data_ptr(), _dtype_code(ydt), ws.data_ptr(), ws.numel(), _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_gemm_dx")
    return dx


def linear_dx_lowbit(bits: int, grad_y2d: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, out_features: int,
                     in_features: int, group_size: int = 32, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """dX[M, K] = dY[M, N] . W[N, K] for the 2.0-bit (``bits`` 2) or 1.0-bit (``bits`` 1) format straight from the
    packed codes (``ojx_e8t_gemm_dx_lowbit``; the weights enter the tensor cores as fp16).  Shapes the kernel does not
    take (fp32 gradients, K % 256 != 0, N % 8 != 0, groups other than 8, 16 and 32) decode W and multiply."""
    n, k = int(out_features), int(in_features)
    dev = _require_cuda(grad_y2d, packed, scales)
    if grad_y2d.dim() != 2 or grad_y2d.shape[1] != n:
        raise ValueError(f"grad_y must be [M, {n}], got {tuple(grad_y2d.shape)}")
    gy = grad_y2d.contiguous()
    m = int(gy.shape[0])
    ydt = out_dtype or gy.dtype
    if m == 0:
        return torch.empty((0, k), dtype=ydt, device=dev)
    fast = (gy.dtype in (torch.bfloat16, torch.float16) and k % 256 == 0 and n % 8 == 0 and int(group_size) in (8, 16, 32)
            and packed.numel() * (4 if bits == 2 else 8) == n * k
            and (gy.data_ptr() | packed.data_ptr() | scales.data_ptr()) % 16 == 0)
    if not fast:
        w = _decode_lowbit(bits, packed, scales, (n, k), gy.dtype if gy.dtype.is_floating_point else torch.float32)
        return gy.matmul(w).to(ydt)
    _cabi.raise_pending()
    dx = torch.empty((m, k), dtype=ydt, device=dev)
    lib = _cabi.lib()
    with torch.cuda.device(dev):
        ws = _gemm_scratch(dev, lib.ojx_e8t_gemm_dx_workspace_bytes(m, n, k))
        st = lib.ojx_e8t_gemm_dx_lowbit(bits, gy.data_ptr(), _dtype_code(gy.dtype), m, packed.data_ptr(), scales.data_ptr(), n, k,
                                        int(group_size), dx.data_ptr(), _dtype_code(ydt), ws.data_ptr(), ws.numel(), _stream_ptr(dev))
    _cabi.check(st, "ojx_e8t_gemm_dx_lowbit")
    return dx


def _gemm_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """256-byte aligned scratch for the prefill kernel (status block + fp16 copy of bf16 activations)."""
    buf = scratch(device, nbytes + 256, "gemm")
    off = (-buf.data_ptr()) % 256
    return buf[off: off + max(nbytes, 256)]


def gemm_status(device: torch.device) -> None:
    """Raise if a bounded wait inside the last prefill GEMM on this device/stream expired."""
    ws = _gemm_scratch(device, 256)
    with torch.cuda.device(device):
        st = _cabi.lib().ojx_e8t_gemm_status(ws.data_ptr(), _stream_ptr(device))
    _cabi.check(st, "ojx_e8t_gemm (device status)")


class GroupedGemv:
    """Several independent decode-shape linears launched as ONE kernel.

    All buffers are fixed at construction (activations, outputs, packed weights), so the device
    descriptor table is built once and a call is a single launch - suitable for CUDA graphs.
    Typical groups: q/k/v of one layer, gate/up of one layer, or a benchmark's rotation of matrices.
    """

    def __init__(self, entries: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Optional[torch.Tensor], torch.Tensor]],
                 shapes: Sequence[Tuple[int, int]], peer_delta: Optional[Sequence[int]] = None,
                 static_weights: bool = False, peer_sync: Optional[int] = None, wait_peers: bool = False,
                 signal_peers: bool = False, extra_flags: int = 0, independent: bool = False):
        # entries: (x[M,K], packed, scales, bias-or-None, y[M,N]);  shapes: (N, K)
        # peer_delta: byte distances from this rank's output window to every rank's (see sharding.PeerWindow);
        #             when given, each result is stored into all ranks' windows by the kernel itself
        # static_weights: promise that nothing queued ahead of a call in its stream writes the packed buffers; the
        #             launch may then begin (set-up, first weight copies) while the previous kernel drains
        # independent: promise that nothing this launch reads or writes is touched by kernels queued ahead of it that may
        #             still be running (a sweep over different matrices with their own outputs): it never waits for them
        # peer_sync:  device address of this rank's ojx_e8t_peer_sync block inside the peer window (PeerWindow.sync_ptr);
        #             wait_peers: wait on the device until every rank has published the launch that produced x;
        #             signal_peers: publish this launch to every rank once all results are stored
        if not entries:
            raise ValueError("empty problem list")
        lib = _cabi.lib()
        self.device = _require_cuda(*[t for e in entries for t in e if t is not None])
        self.M = int(entries[0][0].shape[0])
        self.x_dtype = entries[0][0].dtype
        self.y_dtype = entries[0][4].dtype
        if not (1 <= self.M <= GEMV_MAX_M):
            raise ValueError(f"grouped decode-shape launch needs 1 <= M <= {GEMV_MAX_M}")
        if self.x_dtype not in (torch.bfloat16, torch.float16):
            raise TypeError("activations must be bfloat16 or float16")
        arr = (_cabi.GemvProblem * len(entries))()
        self._keep: List[torch.Tensor] = []
        tile_begin, partial_bytes = 0, 0
        offsets = []
        for (x, pk, sc, b, y), (n, k) in zip(entries, shapes):
            if k % 256 != 0:
                raise ValueError("grouped launch needs K % 256 == 0")
            if x.shape != (self.M, k) or y.shape != (self.M, n) or x.dtype != self.x_dtype or y.dtype != self.y_dtype:
                raise ValueError("inconsistent shapes or dtypes in the problem list")
            if y.stride(1) != 1 or (self.M > 1 and y.stride(0) < n):
                raise ValueError("y must have unit column stride (it may be a column block of a wider matrix)")
            if pk.numel() != n * k * 3 // 16 or sc.numel() != n * k // 32:
                raise ValueError("packed/scales sizes do not match (N, K)")
            for t in (x, pk, sc):
                if not t.is_contiguous() or t.data_ptr() % 16 != 0:
                    raise ValueError("buffers must be contiguous and 16-byte aligned")
            kc = lib.ojx_e8t_gemv_kchunks(k)
            offsets.append(partial_bytes if kc > 1 else -1)
            if kc > 1:
                partial_bytes += kc * self.M * n * 4
        self.partials = torch.empty(max(partial_bytes, 16), dtype=torch.uint8, device=self.device)
        for i, ((x, pk, sc, b, y), (n, k)) in enumerate(zip(entries, shapes)):
            bb = None
            if b is not None:
                bb = b.detach().to(self.x_dtype).contiguous()
                self._keep.append(bb)
            p = arr[i]
            p.x, p.packed, p.scales, p.y = x.data_ptr(), pk.data_ptr(), sc.data_ptr(), y.data_ptr()
            p.bias = bb.data_ptr() if bb is not None else None
            p.partial = (self.partials.data_ptr() + offsets[i]) if offsets[i] >= 0 else None
            p.N, p.K, p.tile_begin = n, k, tile_begin
            p.ldy = int(y.stride(0)) if (self.M > 1 and y.stride(0) != n) else 0
            tile_begin += lib.ojx_e8t_gemv_tiles(n, k)
            self._keep.extend([x, pk, sc, y])
        self.count = len(entries)
        self.total_tiles = tile_begin
        self.needs_reduce = 1 if partial_bytes > 0 else 0
        raw = bytes(arr)
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)
        self.packed_bytes = sum(n * k // 4 for n, k in shapes)
        if (wait_peers or signal_peers) and peer_sync is None:
            raise ValueError("wait_peers / signal_peers need the peer_sync block of the output window")
        if signal_peers and peer_delta is None:
            raise ValueError("signal_peers needs peer_delta")
        self.peer_sync = int(peer_sync) if peer_sync is not None else None
        self.flags = ((_cabi.OJX_GEMV_STATIC_WEIGHTS if static_weights else 0) | (_cabi.OJX_GEMV_INDEPENDENT if independent else 0) |
                      (_cabi.OJX_GEMV_WAIT_PEERS if wait_peers else 0) | (_cabi.OJX_GEMV_SIGNAL_PEERS if signal_peers else 0) |
                      int(extra_flags))
        self._peers = None
        if peer_delta is not None:
            if not (1 <= len(peer_delta) <= 8):
                raise ValueError("peer_delta needs one entry per rank, at most 8")
            self._peers = (ctypes.c_int64 * len(peer_delta))(*[int(d) for d in peer_delta])

    def __call__(self, independent: Optional[bool] = None) -> None:
        """Launches the group; ``independent`` overrides the constructor's choice for this call."""
        flags = self.flags
        if independent is not None:
            flags = (flags | _cabi.OJX_GEMV_INDEPENDENT) if independent else (flags & ~_cabi.OJX_GEMV_INDEPENDENT)
        _cabi.raise_pending()
        with torch.cuda.device(self.device):
            st = _cabi.lib().ojx_e8t_gemv_grouped_ex(
                self.table.data_ptr(), self.count, self.total_tiles, self.M, _dtype_code(self.x_dtype),
                _dtype_code(self.y_dtype), self.needs_reduce,
                ctypes.addressof(self._peers) if self._peers is not None else None,
                len(self._peers) if self._peers is not None else 1, self.peer_sync, flags, _stream_ptr(self.device))
        _cabi.check(st, "ojx_e8t_gemv_grouped_ex")
