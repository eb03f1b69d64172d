"""CPU oracle for the ternary-E8 (1.5 code bits / weight) quantized-linear path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy, the arithmetic
of the reference's ``TernaryE8LatticePacker`` and of its dequantize-then-matmul
forward.  It exists so that parity tests have an independent checker; nothing
in the shipped package may import it.  Only the test-suite, the smoke check and
the benchmark's CPU-baseline leg are allowed to call into this directory.

Parity status: PINNED.  The functions below are checked bit-for-bit against
outputs of the live reference (packed bytes, fp16 scales, fp32 decoded weights)
stored as fixtures under ``tests/golden/`` together with the script that
generated them from the reference.

Reference locations restated here (paths inside the reference project):

* ``ojasx2/math/lattice.py:292-332``  ``_get_ternary_e8_luts``  -> :func:`ternary_luts`
* ``ojasx2/math/lattice.py:338-384``  ``TernaryE8LatticePacker.pack``  -> :func:`encode`
* ``ojasx2/math/lattice.py:386-419``  ``TernaryE8LatticePacker.unpack``  -> :func:`decode`
* ``ojasx2/math/lattice.py:581,610-624``  ``_FusedE8GEMMFunction.forward``  -> :func:`linear_fp32`
* ``ojasx2/streaming_e8.py:90-159``  ``pack_weight_rowwise``  -> :func:`encode_rowwise`
"""

from __future__ import annotations

import math
from functools import lru_cache
from typing import Tuple

import numpy as np

F32 = np.float32
NUM_POINTS = 3281          # |D8 ∩ {-1,0,1}^8| : trit vectors with an even number of zeros
_SQRT_CACHE = {}


# ---------------------------------------------------------------------------
# Portable seeded generator (integer-exact; the same stream is produced by the
# CUDA generator kernel, so inputs never depend on a library RNG).
# ---------------------------------------------------------------------------

def _mix64(z: np.ndarray) -> np.ndarray:
    z = z.astype(np.uint64)
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def gen_normal(seed: int, n: int, sigma: float, start: int = 0) -> np.ndarray:
    """``n`` float32 values ~ N(0, sigma), element ``start + i`` of stream ``seed``.

    Sum of twelve 24-bit uniforms (Irwin-Hall) drawn from six splitmix64 outputs
    per element; every step is integer arithmetic or an exact power-of-two
    scaling, so numpy and CUDA agree bit-for-bit.
    """
    i = np.arange(start, start + n, dtype=np.uint64)
    s = np.zeros(n, dtype=np.int64)
    with np.errstate(over="ignore"):
        base = np.uint64(seed) * np.uint64(0xD1342543DE82EF95)
        for j in range(6):
            h = _mix64(base + i * np.uint64(6) + np.uint64(j))
            s += (h & np.uint64(0xFFFFFF)).astype(np.int64)
            s += ((h >> np.uint64(32)) & np.uint64(0xFFFFFF)).astype(np.int64)
    s -= 6 * (1 << 24)
    x = s.astype(F32) * F32(2.0 ** -24)
    return (x * F32(sigma)).astype(F32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32).astype(np.uint64)
    rounded = (u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(F32)


# ---------------------------------------------------------------------------
# Lookup tables
# ---------------------------------------------------------------------------

@lru_cache(maxsize=None)
def ternary_luts() -> Tuple[np.ndarray, np.ndarray]:
    """``(rank_to_coords int8[3281,8], raw_to_rank int64[6561])``.

    Follows lattice.py:305-321: enumerate raw = 0..3^8-1, digit i (little
    endian, base 3) minus one is coordinate i; keep vectors whose coordinate
    sum is even; rank = position in that increasing-raw order.
    """
    raw = np.arange(3 ** 8, dtype=np.int64)
    digits = np.stack([(raw // 3 ** i) % 3 for i in range(8)], axis=1) - 1
    valid = (digits.sum(axis=1) % 2) == 0
    raw_to_rank = np.zeros(3 ** 8, dtype=np.int64)
    raw_to_rank[valid] = np.arange(int(valid.sum()), dtype=np.int64)
    coords = digits[valid].astype(np.int8)
    assert coords.shape == (NUM_POINTS, 8)
    return coords, raw_to_rank


@lru_cache(maxsize=None)
def two_level_tables():
    """Small tables for rank <-> (hi, lo) with raw = hi*81 + lo.

    ``par4[h]``  parity of the number of 1-trits of the 4-trit number h
    ``off[h]``   number of valid codes whose high half is < h  (off[81] = 3281)
    ``lo_rank[p][l]`` index of l among 4-trit numbers of parity p
    ``lo_tab[p][r]``  inverse of lo_rank
    These are an implementation convenience shared with the CUDA kernels; they
    are validated against :func:`ternary_luts` in the tests.
    """
    ones = np.array([sum(1 for k in range(4) if (n // 3 ** k) % 3 == 1) for n in range(81)])
    par4 = (ones & 1).astype(np.int64)
    off = np.zeros(82, dtype=np.int64)
    for h in range(81):
        off[h + 1] = off[h] + (41 if par4[h] == 0 else 40)
    lo_rank = np.zeros((2, 81), dtype=np.int64)
    lo_tab = np.zeros((2, 41), dtype=np.int64)
    for p in (0, 1):
        c = 0
        for n in range(81):
            if par4[n] == p:
                lo_rank[p, n] = c
                lo_tab[p, c] = n
                c += 1
    return par4, off, lo_rank, lo_tab


# ---------------------------------------------------------------------------
# Encoder
# ---------------------------------------------------------------------------

def _effective_group(group_size: int) -> int:
    # lattice.py:346-347: anything that is not a positive multiple of 16 becomes 16.
    if group_size <= 0 or group_size % 16 != 0:
        return 16
    return group_size


def group_scales_f32(flat_groups: np.ndarray) -> np.ndarray:
    """Unrounded fp32 RMS scale of each row of ``flat_groups`` (shape [G, g]).

    lattice.py:356 computes ``torch.norm(w_groups, dim=-1) / sqrt(g) + 1e-8`` in
    fp32.  The sum of squares that ``torch.norm`` produces for a contiguous
    last dimension is: eight lane accumulators, lane j adding x[j]^2, x[j+8]^2,
    ... in order with separately rounded products (no FMA), then the lanes
    added sequentially 0..7.  That order is restated here.
    """
    x = np.ascontiguousarray(flat_groups, dtype=F32)
    g = x.shape[1]
    if g % 8 != 0:
        raise ValueError("group size must be a multiple of 8")
    acc = np.zeros((x.shape[0], 8), dtype=F32)
    for d in range(0, g, 8):
        v = x[:, d:d + 8]
        acc = (acc + (v * v).astype(F32)).astype(F32)
    s = acc[:, 0].copy()
    for j in range(1, 8):
        s = (s + acc[:, j]).astype(F32)
    nrm = np.sqrt(s).astype(F32)
    return ((nrm / F32(math.sqrt(g))).astype(F32) + F32(1e-8)).astype(F32)


def encode(w: np.ndarray, group_size: int = 32):
    """Restatement of ``TernaryE8LatticePacker.pack`` (lattice.py:338-384).

    ``w``: 2-D array (fp32, or fp16/bf16 already widened exactly to fp32).
    Returns ``(packed uint8[P*3/16], scales float16[P/g], (rows, cols))`` where P
    is rows*cols padded with zeros up to a multiple of g.
    """
    rows, cols = w.shape
    g = _effective_group(group_size)
    flat = np.ascontiguousarray(w, dtype=F32).reshape(-1)
    pad = (-flat.size) % g
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=F32)])
    groups = flat.reshape(-1, g)
    scale = group_scales_f32(groups)
    v = (groups / scale[:, None]).astype(F32).reshape(-1, 8)

    q = np.clip(np.rint(v), -1.0, 1.0).astype(F32)
    odd = (q.sum(axis=1).astype(np.int64) % 2) != 0
    alt = np.where(q == 0.0, np.where(v >= 0.0, F32(1), F32(-1)), F32(0)).astype(F32)
    da = (alt - v).astype(F32)
    dq = (q - v).astype(F32)
    pen = ((da * da).astype(F32) - (dq * dq).astype(F32)).astype(F32)
    worst = pen.argmin(axis=1)          # first index on ties, as torch.argmin
    idx = np.nonzero(odd)[0]
    q[idx, worst[idx]] = alt[idx, worst[idx]]

    digits = q.astype(np.int64) + 1
    raw = (digits * (3 ** np.arange(8, dtype=np.int64))).sum(axis=1)
    _, raw_to_rank = ternary_luts()
    codes = raw_to_rank[raw]
    packed = pack_codes(codes)
    return packed, scale.astype(np.float16), (rows, cols)


def pack_codes(codes: np.ndarray) -> np.ndarray:
    """Two 12-bit ranks -> three bytes (lattice.py:375-383)."""
    c = codes.reshape(-1, 2)
    c0, c1 = c[:, 0], c[:, 1]
    b0 = c0 & 0xFF
    b1 = ((c0 >> 8) & 0x0F) | ((c1 & 0x0F) << 4)
    b2 = (c1 >> 4) & 0xFF
    return np.stack([b0, b1, b2], axis=1).astype(np.uint8).reshape(-1)


def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """Three bytes -> two 12-bit ranks (lattice.py:397-405)."""
    t = packed.reshape(-1, 3).astype(np.int64)
    c0 = t[:, 0] | ((t[:, 1] & 0x0F) << 8)
    c1 = ((t[:, 1] >> 4) & 0x0F) | (t[:, 2] << 4)
    return np.stack([c0, c1], axis=1).reshape(-1)


def encode_rowwise(w: np.ndarray, group_size: int = 32, row_block: int = 32):
    """Restatement of ``pack_weight_rowwise`` (streaming_e8.py:126-159)."""
    if w.ndim != 2:
        raise ValueError(f"Expected a rank-2 weight, got shape {tuple(w.shape)}")
    if row_block <= 0:
        raise ValueError("row_block must be positive")
    rows, cols = w.shape
    if rows <= 0 or cols <= 0:
        raise ValueError("Streaming E8 requires non-empty two-dimensional weights")
    if group_size <= 0 or group_size % 32 != 0:
        raise ValueError("The current E8 packers require group_size to be a positive multiple of 32")
    if cols % group_size != 0:
        raise ValueError(f"in_features={cols} is not divisible by group_size={group_size}.")
    ps, ss = [], []
    for r0 in range(0, rows, row_block):
        p, s, _ = encode(w[r0:r0 + row_block], group_size)
        ps.append(p)
        ss.append(s)
    return np.concatenate(ps), np.concatenate(ss)


# ---------------------------------------------------------------------------
# Decoder
# ---------------------------------------------------------------------------

def decode_coords(packed: np.ndarray) -> np.ndarray:
    """int8[num_codes, 8] lattice coordinates of every packed code."""
    coords, _ = ternary_luts()
    return coords[unpack_codes(packed)]


def decode(packed: np.ndarray, scales: np.ndarray, shape: Tuple[int, int]) -> np.ndarray:
    """Restatement of ``TernaryE8LatticePacker.unpack(..., dtype=float32)``
    (lattice.py:386-419): ``W = float(coord) * float(scale_fp16)``; the group
    size is inferred as padded_elements // scales.size."""
    c = decode_coords(packed)
    padded = c.size
    g = padded // max(1, scales.size)
    w = c.reshape(-1, g).astype(F32) * scales.astype(F32).reshape(-1, 1)
    total = shape[0] * shape[1]
    return w.reshape(-1)[:total].reshape(shape).astype(F32)


def decode_two_level(packed: np.ndarray) -> np.ndarray:
    """Coordinates via the small-table unranking used on the GPU
    (hi = floor(2*rank/81), lo from a 41-entry table); must equal
    :func:`decode_coords`."""
    par4, off, _, lo_tab = two_level_tables()
    rank = unpack_codes(packed)
    hi = (2 * rank) // 81
    r = rank - off[hi]
    lo = np.where(par4[hi] == 0, lo_tab[0][np.minimum(r, 40)], lo_tab[1][np.minimum(r, 39)])
    raw = hi * 81 + lo
    return np.stack([(raw // 3 ** k) % 3 - 1 for k in range(8)], axis=1).astype(np.int8)


# ---------------------------------------------------------------------------
# Linear
# ---------------------------------------------------------------------------

def linear_fp32(x: np.ndarray, packed: np.ndarray, scales: np.ndarray, n: int, k: int,
                bias: np.ndarray | None = None) -> np.ndarray:
    """fp32 dequantize-then-matmul: ``y = x.float() @ decode(...).T (+ bias)``.

    This is the contract's GEMM oracle (lattice.py:618-624 evaluated in fp32).
    Accumulation is float64 then rounded once, so the oracle itself carries no
    summation-order noise.
    """
    w = decode(packed, scales, (n, k)).astype(np.float64)
    y = np.asarray(x, dtype=np.float64) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)[None, :]
    return y.astype(F32)


def gemm_tolerance(x: np.ndarray, k: int) -> Tuple[float, float]:
    """``(max_abs_bound, rel_l2_bound)`` of the GEMM contract:
    max-abs <= 1e-2 * ||x||_inf * sqrt(K), relative L2 <= 2e-3."""
    return 1e-2 * float(np.abs(np.asarray(x, dtype=np.float64)).max()) * math.sqrt(k), 2e-3


# ---------------------------------------------------------------------------------------------
# Nearest E8 lattice point and the straight-through quantizer built on it
# ---------------------------------------------------------------------------------------------

def _seq_sum_f32(a: np.ndarray) -> np.ndarray:
    """Sum over the last axis, left to right, every partial sum rounded to fp32 (the order torch's CPU
    reduction uses for rows of eight)."""
    s = a[..., 0].astype(np.float32).copy()
    for i in range(1, a.shape[-1]):
        s = (s + a[..., i]).astype(np.float32)
    return s


def _d8_candidate(v: np.ndarray) -> np.ndarray:
    """Nearest point of D8 (integer vectors with an even coordinate sum) to each row of ``v``: round every
    coordinate; when the sum is odd move the coordinate with the largest rounding error (first one on ties)
    one step in the direction of its error (+1 when the error is zero)."""
    f = np.rint(v).astype(np.float32)
    odd = (_seq_sum_f32(f).astype(np.int64) % 2) != 0
    diff = (v - f).astype(np.float32)
    worst = np.argmax(np.abs(diff), axis=-1)
    sign = np.sign(diff).astype(np.float32)
    sign[sign == 0] = 1.0
    rows = np.arange(v.shape[0])
    fixed = f.copy()
    fixed[rows, worst] = (f[rows, worst] + sign[rows, worst]).astype(np.float32)
    return np.where(odd[:, None], fixed, f).astype(np.float32)


def conway_sloane_project(x: np.ndarray) -> np.ndarray:
    """Nearest point of E8 = D8 u (D8 + 1/2) to every 8-vector (rows of ``x`` reshaped to [-1, 8]), fp32.
    Follows conway_sloane_e8_project (ojasx2/math/lattice.py:162-203) operation by operation: the D8 candidate of x,
    the D8 candidate of x - 1/2 shifted back, squared distances summed left to right, the first wins ties."""
    v = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 8)
    c1 = _d8_candidate(v)
    c2 = (_d8_candidate((v - np.float32(0.5)).astype(np.float32)) + np.float32(0.5)).astype(np.float32)
    e1, e2 = (v - c1).astype(np.float32), (v - c2).astype(np.float32)
    d1, d2 = _seq_sum_f32((e1 * e1).astype(np.float32)), _seq_sum_f32((e2 * e2).astype(np.float32))
    return np.where((d1 <= d2)[:, None], c1, c2).astype(np.float32).reshape(np.shape(x))


def ste_quantize(w: np.ndarray) -> np.ndarray:
    """Forward of the straight-through E8 quantizer (_E8STEFunction.forward, ojasx2/math/lattice.py:853-867): groups
    of eight consecutive elements of the flattened tensor (zero padded) are divided by rms + 1e-8, projected to E8
    and multiplied back; fp32."""
    flat = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    total = flat.size
    pad = (-total) % 8
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=np.float32)])
    g = flat.reshape(-1, 8)
    nrm = np.sqrt(_seq_sum_f32((g * g).astype(np.float32))).astype(np.float32)
    scale = ((nrm / np.float32(math.sqrt(8))).astype(np.float32) + np.float32(1e-8)).astype(np.float32)[:, None]
    q = conway_sloane_project((g / scale).astype(np.float32))
    return (q * scale).astype(np.float32).reshape(-1)[:total].reshape(np.shape(w))


# ---------------------------------------------------------------------------------------------
# 2.0-bit format: four 2-bit codes per byte, weight = (code - 1.5) * scale
# ---------------------------------------------------------------------------------------------

def encode_2bit(w: np.ndarray, group_size: int = 8):
    """Restatement of ``E8LatticePacker.pack`` (ojasx2/math/lattice.py:210-248).  ``group_size`` must be a positive
    multiple of 8 (the reference raises otherwise).  Every 8-block of the rms-normalised weights is moved to the
    half-integer grid {-1.5, -0.5, 0.5, 1.5}^8 with an even sum of the underlying integers: round(x - 1/2) clamped
    to [-2, 1]; when the sum is odd the coordinate whose move to its other neighbour costs least (first one on
    ties, clamping included) is moved.  Returns ``(packed uint8[P/4], scales float16[P/g], (rows, cols))``."""
    rows, cols = w.shape
    if group_size <= 0 or group_size % 8 != 0:
        raise ValueError(f"group_size ({group_size}) must be a positive multiple of 8.")
    flat = np.ascontiguousarray(w, dtype=F32).reshape(-1)
    pad = (-flat.size) % group_size
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=F32)])
    groups = flat.reshape(-1, group_size)
    scale = group_scales_f32(groups)
    xs = ((groups / scale[:, None]).astype(F32).reshape(-1, 8) - F32(0.5)).astype(F32)
    f = np.clip(np.rint(xs), -2.0, 1.0).astype(F32)
    odd = (f.sum(axis=1).astype(np.int64) % 2) != 0
    alt = np.where(xs >= f, np.clip(f + 1, -2.0, 1.0), np.clip(f - 1, -2.0, 1.0)).astype(F32)
    da, df = (alt - xs).astype(F32), (f - xs).astype(F32)
    pen = ((da * da).astype(F32) - (df * df).astype(F32)).astype(F32)
    worst = pen.argmin(axis=1)
    idx = np.nonzero(odd)[0]
    f[idx, worst[idx]] = alt[idx, worst[idx]]
    codes = np.clip(np.rint((f + F32(0.5)).astype(F32) + F32(1.5)), 0, 3).astype(np.uint8).reshape(-1, 4)
    packed = (codes[:, 0] | (codes[:, 1] << 2) | (codes[:, 2] << 4) | (codes[:, 3] << 6)).astype(np.uint8)
    return packed, scale.astype(np.float16), (rows, cols)


def decode_2bit(packed: np.ndarray, scales: np.ndarray, shape: Tuple[int, int]) -> np.ndarray:
    """Restatement of ``E8LatticePacker.unpack`` in fp32 (ojasx2/math/lattice.py:250-279)."""
    p = np.ascontiguousarray(packed, dtype=np.uint8)
    codes = np.stack([p & 3, (p >> 2) & 3, (p >> 4) & 3, (p >> 6) & 3], axis=-1).reshape(-1)
    g = codes.size // max(1, scales.size)
    vals = (codes.astype(F32) - F32(1.5)).reshape(-1, g) * scales.astype(F32).reshape(-1, 1)
    total = shape[0] * shape[1]
    return vals.astype(F32).reshape(-1)[:total].reshape(shape)


# ---------------------------------------------------------------------------------------------
# 1.0-bit format: one byte per 8-block, the index of one of 256 vectors (the 240 roots of E8 and 16 axis vectors,
# all doubled), weight = coordinate * scale with the least-squares scale of the group
# ---------------------------------------------------------------------------------------------

@lru_cache(maxsize=1)
def root_e8_table() -> np.ndarray:
    """The reference's 256 x 8 table in its order (``_get_root_e8_lut``, ojasx2/math/lattice.py:429-462), doubled:
    112 vectors with two entries +-2, 128 vectors (+-1)^8 with an even number of minus signs (the first coordinate
    varies slowest, minus before plus), 16 vectors with one entry +-2."""
    pts = []
    for i in range(8):
        for j in range(i + 1, 8):
            for s1 in (-1.0, 1.0):
                for s2 in (-1.0, 1.0):
                    v = [0.0] * 8
                    v[i], v[j] = s1, s2
                    pts.append(v)
    for b in range(256):
        signs = [0.5 if (b >> (7 - k)) & 1 else -0.5 for k in range(8)]
        if sum(1 for t in signs if t < 0) % 2 == 0:
            pts.append(signs)
    for i in range(8):
        for t in (-1.0, 1.0):
            v = [0.0] * 8
            v[i] = t
            pts.append(v)
    return (np.asarray(pts, dtype=F32) * F32(2.0)).astype(F32)


def _fma_f32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """fl32(a * b + c) with one rounding: the product of two fp32 values is exact in the 64-bit significand of the
    x87 extended type, and the sum is rounded to it before the final rounding to fp32 (double rounding would need an
    exact tie at bit 40 of the sum; none occurred in 25 M comparisons with the reference)."""
    assert np.finfo(np.longdouble).nmant >= 63, "needs the 80-bit extended type"
    return (a.astype(np.longdouble) * b.astype(np.longdouble) + c.astype(np.longdouble)).astype(F32)


def _sum_last_f32(a: np.ndarray) -> np.ndarray:
    """Sum over a contiguous last dimension as torch.sum does it on the CPU: chunks of eight go to four vector
    accumulators in turn, the accumulators are added 0..3, then the eight lanes 0..7."""
    n, g = a.shape
    acc = [np.zeros((n, 8), dtype=F32) for _ in range(4)]
    for ci, d in enumerate(range(0, g, 8)):
        acc[ci % 4] = (acc[ci % 4] + a[:, d:d + 8]).astype(F32)
    lanes = acc[0]
    for u in range(1, 4):
        lanes = (lanes + acc[u]).astype(F32)
    s = lanes[:, 0].copy()
    for j in range(1, 8):
        s = (s + lanes[:, j]).astype(F32)
    return s


def encode_1bit(w: np.ndarray, group_size: int = 32):
    """Restatement of ``RootE8LatticePacker.pack`` (ojasx2/math/lattice.py:475-512): every 8-block of the
    rms-normalised weights takes the table vector with the largest normalised dot product (the matrix product of
    the reference evaluates each dot product as a chain of fused multiply-adds over k = 0..7; the first maximum
    wins), then the group gets the least-squares scale <w, q> / <q, q>.  Group sizes that are not a positive
    multiple of 8 become 8.  Returns ``(packed uint8[P/8], scales float16[P/g], (rows, cols))``."""
    rows, cols = w.shape
    g = group_size if (group_size > 0 and group_size % 8 == 0) else 8
    flat = np.ascontiguousarray(w, dtype=F32).reshape(-1)
    pad = (-flat.size) % g
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=F32)])
    groups = flat.reshape(-1, g)
    v = (groups / group_scales_f32(groups)[:, None]).astype(F32).reshape(-1, 8)
    lut = root_e8_table()
    norms = np.maximum(np.sqrt((lut * lut).sum(axis=1, dtype=F32)).astype(F32), F32(1e-12))
    lut_n = (lut / norms[:, None]).astype(F32)
    dots = np.zeros((v.shape[0], 256), dtype=F32)
    for k in range(8):
        dots = _fma_f32(v[:, k:k + 1], lut_n[None, :, k], dots)
    packed = dots.argmax(axis=1).astype(np.uint8)
    q = lut[packed].reshape(-1, g)
    qn = np.maximum((q * q).sum(axis=1, dtype=F32), F32(1e-8)).astype(F32)
    scale = (_sum_last_f32((groups * q).astype(F32)) / qn).astype(F32)
    return packed, scale.astype(np.float16), (rows, cols)


def decode_1bit(packed: np.ndarray, scales: np.ndarray, shape: Tuple[int, int]) -> np.ndarray:
    """Restatement of ``RootE8LatticePacker.unpack`` in fp32 (ojasx2/math/lattice.py:514-537)."""
    coords = root_e8_table()[np.ascontiguousarray(packed, dtype=np.uint8).astype(np.int64)].reshape(-1)
    g = coords.size // max(1, scales.size)
    vals = (coords.reshape(-1, g) * scales.astype(F32).reshape(-1, 1)).astype(F32)
    total = shape[0] * shape[1]
    return vals.reshape(-1)[:total].reshape(shape)
