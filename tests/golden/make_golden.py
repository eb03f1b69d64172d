"""Generate golden vectors for the ternary-E8 path FROM THE LIVE REFERENCE.

Run once, in a container that has the reference checkout:

    OJASX_DISABLE_UPDATE_CHECK=1 PYTHONDONTWRITEBYTECODE=1 \
        python tests/golden/make_golden.py --ref /path/to/reference

It imports the reference's ``ojasx2.math.lattice`` / ``ojasx2.streaming_e8``,
feeds them inputs from the portable seeded generator in ``oracle/e8t_oracle.py``
(so inputs can be regenerated anywhere without a library RNG) and stores the
reference's outputs:

* ``e8t_golden.npz``  - full arrays for small cases (packed bytes, fp16 scales,
  fp32 decoded weights, fp32 linear outputs) and the reference's full
  rank->coords table;
* ``e8t_golden.json`` - case descriptions plus SHA-256 digests of the
  reference's outputs for the large cases.

Nothing here is read at test time except the two output files.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import logging
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import e8t_oracle as O  # noqa: E402  (input generator only)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# name, seed, rows, cols, sigma, dtype, group, store_full
CASES = [
    ("kat_64x128_f32", 1, 64, 128, 0.02, "f32", 32, True),
    ("kat_256x4096_f16", 2, 256, 4096, 0.02, "f16", 32, False),
    ("kat_128x14336_f32", 3, 128, 14336, 0.02, "f32", 32, False),
    ("kat_96x8192_f16", 4, 96, 8192, 0.02, "f16", 32, False),
    ("bf16_48x256", 5, 48, 256, 0.02, "bf16", 32, True),
    ("unit_sigma_32x512", 6, 32, 512, 1.0, "f32", 32, True),
    ("odd_7x13_g32", 7, 7, 13, 0.5, "f32", 32, True),
    ("odd_5x19_g16", 8, 5, 19, 0.5, "f32", 16, True),
    ("row_not_group_4x48_g32", 9, 4, 48, 0.1, "f32", 32, True),
    ("group64_16x256", 10, 16, 256, 0.02, "f32", 64, True),
    ("bad_group_8x64_g8", 11, 8, 64, 0.02, "f32", 8, True),      # coerced to 16 by the packer
    ("single_group_1x32", 12, 1, 32, 3.0, "f32", 32, True),
    ("llama_q_512x4096_bf16", 13, 512, 4096, 0.02, "bf16", 32, False),
    ("big_values_16x128", 14, 16, 128, 1.0e4, "f32", 32, True),
    ("tiny_values_16x128", 15, 16, 128, 1.0e-6, "f16", 32, True),   # fp16 denormals / zeros
]


def make_input(seed, rows, cols, sigma, dtype):
    import torch
    w = O.gen_normal(seed, rows * cols, sigma).reshape(rows, cols)
    t = torch.from_numpy(w.copy())
    if dtype == "f16":
        t = t.half()
    elif dtype == "bf16":
        t = t.bfloat16()
    return t


def special_inputs():
    """Hand-built edge inputs: all-zero groups, exact ties, half-way values, signed zeros."""
    import torch
    out = {}
    z = torch.zeros(2, 64)
    z[1, :32] = torch.linspace(-1, 1, 32)
    out["zeros_and_ramp_2x64"] = (z, 32)
    # values that sit exactly on rounding boundaries after division by the scale
    t = torch.tensor([0.5, -0.5, 1.5, -1.5, 0.0, -0.0, 2.5, -2.5] * 4, dtype=torch.float32).reshape(1, 32)
    out["halfway_1x32"] = (t, 32)
    # identical magnitudes -> argmin ties (first index must win)
    e = torch.full((1, 32), 0.3, dtype=torch.float32)
    e[0, ::3] = -0.3
    out["ties_1x32"] = (e, 32)
    c = torch.ones(3, 32, dtype=torch.float32)
    c[1] *= -1
    c[2, 16:] = 0
    out["constant_3x32"] = (c, 32)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("OJASX_REFERENCE_DIR"),
                    help="checkout of the reference project (or set OJASX_REFERENCE_DIR)")
    args = ap.parse_args()
    if not args.ref or not os.path.isdir(args.ref):
        ap.error("pass --ref /path/to/reference (or set OJASX_REFERENCE_DIR)")
    os.environ.setdefault("OJASX_DISABLE_UPDATE_CHECK", "1")
    logging.disable(logging.CRITICAL)
    sys.path.insert(0, args.ref)
    import torch
    import ojasx2.math.lattice as L
    from ojasx2.streaming_e8 import pack_weight_rowwise

    torch.set_num_threads(4)
    arrays, meta = {}, {"cases": [], "special": [], "generator_check": {}}

    x0 = O.gen_normal(1, 4, 1.0)
    meta["generator_check"] = {"seed": 1, "first4": [float(v) for v in x0]}

    r2c, raw2rank, _ = L._get_ternary_e8_luts()
    arrays["rank_to_coords"] = r2c.numpy().astype(np.int8)
    meta["rank_to_coords_sha256"] = sha(arrays["rank_to_coords"])
    meta["raw_to_rank_sha256"] = sha(raw2rank.numpy().astype(np.int64))

    for name, seed, rows, cols, sigma, dtype, group, full in CASES:
        w = make_input(seed, rows, cols, sigma, dtype)
        packed, scales, shape = L.TernaryE8LatticePacker.pack(w, group_size=group)
        dec = L.TernaryE8LatticePacker.unpack(packed, scales, (rows, cols), dtype=torch.float32)
        entry = dict(name=name, seed=seed, rows=rows, cols=cols, sigma=sigma, dtype=dtype, group=group,
                     full=full, packed_len=int(packed.numel()), scales_len=int(scales.numel()),
                     sha_input=sha(w.view(torch.int16).numpy() if dtype != "f32" else w.numpy()),
                     sha_packed=sha(packed.numpy()), sha_scales=sha(scales.view(torch.int16).numpy()),
                     sha_decoded=sha(dec.numpy()))
        if group % 32 == 0 and cols % group == 0:
            p2, s2 = pack_weight_rowwise(w, bitrate=1.5, group_size=group, row_block=5)
            entry["rowwise_equal"] = bool(torch.equal(p2, packed) and torch.equal(s2, scales))
        if cols % 32 == 0 and group == 32:
            xb = torch.from_numpy(O.gen_normal(seed + 100, 4 * cols, 1.0).reshape(4, cols).copy()).bfloat16()
            y = xb.float() @ dec.t()
            y_ref = L._FusedE8GEMMFunction.apply(xb.float(), packed, scales, None, rows, cols, group, 1.5, False)
            entry["y_norm"] = float(y.norm())
            entry["y_head"] = [float(v) for v in y[0, :3]]
            entry["ref_forward_matches_dequant_matmul"] = bool(torch.equal(y, y_ref))
            if full:
                arrays[name + "/y"] = y.numpy()
        if full:
            arrays[name + "/packed"] = packed.numpy()
            arrays[name + "/scales"] = scales.view(torch.int16).numpy().view(np.uint16)
            arrays[name + "/decoded"] = dec.numpy()
        meta["cases"].append(entry)
        print(name, entry["sha_packed"][:16], entry["sha_scales"][:16], entry["sha_decoded"][:16])

    for name, (w, group) in special_inputs().items():
        packed, scales, _ = L.TernaryE8LatticePacker.pack(w, group_size=group)
        dec = L.TernaryE8LatticePacker.unpack(packed, scales, tuple(w.shape), dtype=torch.float32)
        arrays["special/" + name + "/input"] = w.numpy()
        arrays["special/" + name + "/packed"] = packed.numpy()
        arrays["special/" + name + "/scales"] = scales.view(torch.int16).numpy().view(np.uint16)
        arrays["special/" + name + "/decoded"] = dec.numpy()
        meta["special"].append(dict(name=name, group=group, rows=int(w.shape[0]), cols=int(w.shape[1])))
        print("special", name, sha(packed.numpy())[:16])

    # Walsh-Hadamard rotation (lattice.py:91-102) in the three dtypes, and one layer packed and run with
    # use_hadamard=True (lattice.py:564-567,807,825): weights are rotated before packing, activations in forward
    xw = torch.from_numpy(O.gen_normal(77, 6 * 96, 1.0).reshape(6, 96).copy())
    for tag, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        xin = xw.to(dt)
        out = L.fwht_block32(xin)
        arrays["fwht/" + tag + "/input"] = xin.float().numpy()
        arrays["fwht/" + tag + "/output"] = out.float().numpy()
    lin = torch.nn.Linear(256, 48, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(O.gen_normal(78, 48 * 256, 0.02).reshape(48, 256).copy()))
        lin.bias.copy_(torch.from_numpy(O.gen_normal(79, 48, 0.1).copy()))
    layer = L.E8LatticeLinear.from_linear(lin, rank=0, bitrate=1.5, group_size=32, use_hadamard=True)
    xh = torch.from_numpy(O.gen_normal(80, 5 * 256, 1.0).reshape(5, 256).copy())
    with torch.no_grad():
        yh = layer(xh)
    arrays["hadamard/packed"] = layer.packed_weight.numpy()
    arrays["hadamard/scales"] = layer.block_scales.view(torch.int16).numpy().view(np.uint16)
    arrays["hadamard/unpacked"] = layer.unpack_weights(torch.float32).numpy()
    arrays["hadamard/y"] = yh.numpy()
    meta["hadamard"] = dict(in_features=256, out_features=48, weight_seed=78, bias_seed=79, x_seed=80, batch=5,
                            sha_packed=sha(layer.packed_weight.numpy()))
    print("hadamard", meta["hadamard"]["sha_packed"][:16])

    # nearest E8 point (lattice.py:162-203) and the straight-through quantizer's forward (lattice.py:853-867), fp32:
    # random vectors at four magnitudes, a quarter-integer grid (exact distance and rounding ties), integer
    # vectors (zero rounding error, odd sums), and weights whose element count is not a multiple of eight
    proj_in = np.concatenate([
        O.gen_normal(90, 384 * 8, 0.3), O.gen_normal(91, 384 * 8, 1.0), O.gen_normal(92, 384 * 8, 3.0),
        O.gen_normal(93, 128 * 8, 40.0),
        np.rint(O.gen_normal(94, 384 * 8, 2.0) * 4.0).astype(np.float32) * np.float32(0.25),
        np.rint(O.gen_normal(95, 128 * 8, 2.0)).astype(np.float32),
    ]).astype(np.float32).reshape(-1, 8)
    proj_out = L.conway_sloane_e8_project(torch.from_numpy(proj_in.copy()), prefer_native=False)
    arrays["project/input"] = proj_in
    arrays["project/output"] = proj_out.numpy()
    ste_in = O.gen_normal(96, 37 * 19, 0.05).reshape(37, 19).copy()
    ste_in[3, :] = 0.0
    arrays["ste/input"] = ste_in
    arrays["ste/output"] = L._E8STEFunction.apply(torch.from_numpy(ste_in.copy())).numpy()
    meta["project"] = dict(vectors=int(proj_in.shape[0]), sha_output=sha(arrays["project/output"]),
                           sha_ste_output=sha(arrays["ste/output"]))
    print("project", meta["project"]["sha_output"][:16], meta["project"]["sha_ste_output"][:16])

    # 2.0-bit packer (lattice.py:210-279): two group sizes, a heavy-tailed input (clamping active) and a half-integer
    # grid (rounding and penalty ties), with a padded tail in the first case
    two = {
        "g8": (torch.from_numpy(O.gen_normal(110, 33 * 100, 1.0).reshape(33, 100).copy()), 8),
        "g32": (torch.from_numpy(O.gen_normal(111, 48 * 256, 0.02).reshape(48, 256).copy()), 32),
        "heavy": (torch.from_numpy((O.gen_normal(112, 32 * 128, 1.0) ** 3).astype(np.float32).reshape(32, 128).copy()), 8),
        "grid": (torch.from_numpy((np.rint(O.gen_normal(113, 32 * 128, 2.0)) * 0.5).astype(np.float32).reshape(32, 128).copy()), 32),
    }
    for tag, (wt, g) in two.items():
        p2, s2, _ = L.E8LatticePacker.pack(wt, group_size=g)
        arrays[f"two_bit/{tag}/input"] = wt.numpy()
        arrays[f"two_bit/{tag}/group"] = np.int64(g)
        arrays[f"two_bit/{tag}/packed"] = p2.numpy()
        arrays[f"two_bit/{tag}/scales"] = s2.view(torch.int16).numpy().view(np.uint16)
        arrays[f"two_bit/{tag}/decoded"] = L.E8LatticePacker.unpack(p2, s2, tuple(wt.shape), dtype=torch.float32).numpy()
        print("two_bit", tag, sha(p2.numpy())[:16])

    # 1.0-bit root packer (lattice.py:472-537): two group sizes, a quarter-integer grid (many equal dot products: the
    # first maximum must win) and a sparse input with all-zero blocks
    sparse = np.zeros((16, 64), dtype=np.float32)
    sparse[1, :8] = 1.0
    sparse[2, 5] = -3.0
    sparse[3, 8:16] = O.gen_normal(123, 8, 1.0)
    one = {
        "g32": (torch.from_numpy(O.gen_normal(120, 48 * 256, 0.02).reshape(48, 256).copy()), 32),
        "g8": (torch.from_numpy(O.gen_normal(121, 33 * 100, 1.0).reshape(33, 100).copy()), 8),
        "grid": (torch.from_numpy((np.rint(O.gen_normal(122, 32 * 128, 2.0)) * 0.25).astype(np.float32).reshape(32, 128).copy()), 32),
        "sparse": (torch.from_numpy(sparse), 32),
    }
    for tag, (wt, g) in one.items():
        p1, s1, _ = L.RootE8LatticePacker.pack(wt, group_size=g)
        arrays[f"one_bit/{tag}/input"] = wt.numpy()
        arrays[f"one_bit/{tag}/group"] = np.int64(g)
        arrays[f"one_bit/{tag}/packed"] = p1.numpy()
        arrays[f"one_bit/{tag}/scales"] = s1.view(torch.int16).numpy().view(np.uint16)
        arrays[f"one_bit/{tag}/decoded"] = L.RootE8LatticePacker.unpack(p1, s1, tuple(wt.shape), dtype=torch.float32).numpy()
        print("one_bit", tag, sha(p1.numpy())[:16])

    # decode of every code: all 3281 ranks (padded to an even count) with unit scales
    ranks = np.arange(3282, dtype=np.int64) % 3281
    packed_all = O.pack_codes(ranks)
    sc = torch.ones(3282 * 8 // 32 + 1, dtype=torch.float16)[: (3282 * 8) // 32]
    # 3282*8 = 26256 weights = 820.5 groups of 32 -> use group 16 (1641 groups)
    sc16 = torch.ones(1641, dtype=torch.float16)
    dec_all = L.TernaryE8LatticePacker.unpack(torch.from_numpy(packed_all), sc16, (3282, 8), dtype=torch.float32)
    arrays["all_codes/packed"] = packed_all
    arrays["all_codes/decoded"] = dec_all.numpy().astype(np.int8)
    del sc

    np.savez_compressed(os.path.join(HERE, "e8t_golden.npz"), **arrays)
    with open(os.path.join(HERE, "e8t_golden.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays")


if __name__ == "__main__":
    main()
