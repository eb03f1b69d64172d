"""The CPU oracle (numpy and C) against golden vectors produced by the live reference.

Mirrors the reference's own checks for this path: exact byte counts
(tests/test_sub2bit_lattice.py:40-62), row-wise == whole-matrix packing
(tests/test_streaming_e8.py:15-39), odd shapes (tests/test_ojasx_exhaustive.py:303-320),
and adds bit-exact comparison with stored reference outputs.
"""

import hashlib

import numpy as np
import pytest

from conftest import case_input


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_generator_known_values(golden, oracle):
    meta, _ = golden
    got = oracle.gen_normal(1, 4, 1.0)
    assert [float(v) for v in got] == meta["generator_check"]["first4"]
    # start offset is consistent with one long stream
    a = oracle.gen_normal(3, 1000, 0.02)
    b = oracle.gen_normal(3, 400, 0.02, start=600)
    assert np.array_equal(a[600:], b)


def test_lut_matches_reference_table(golden, oracle):
    meta, arrays = golden
    coords, raw_to_rank = oracle.ternary_luts()
    assert np.array_equal(coords, arrays["rank_to_coords"])
    assert sha(coords) == meta["rank_to_coords_sha256"]
    assert sha(raw_to_rank.astype(np.int64)) == meta["raw_to_rank_sha256"]
    assert coords.shape == (3281, 8)
    # the all-zero vector is rank 1640
    assert np.array_equal(coords[1640], np.zeros(8, dtype=np.int8))


def test_two_level_unrank_is_exact(oracle):
    ranks = np.arange(3282) % 3281
    packed = oracle.pack_codes(ranks)
    assert np.array_equal(oracle.decode_two_level(packed), oracle.decode_coords(packed))
    par4, off, lo_rank, lo_tab = oracle.two_level_tables()
    assert off[81] == 3281
    r = np.arange(3281)
    hi = (2 * r) // 81
    assert np.all(off[hi] <= r) and np.all(r < off[hi + 1])


def test_all_codes_decode(golden, oracle):
    _, arrays = golden
    dec = oracle.decode_coords(arrays["all_codes/packed"])
    assert np.array_equal(dec, arrays["all_codes/decoded"])


def test_encode_decode_cases(golden, oracle, coracle):
    meta, arrays = golden
    for case in meta["cases"]:
        w = case_input(oracle, case)
        if case["dtype"] == "f16":
            assert sha(w.view(np.int16)) == case["sha_input"]
        elif case["dtype"] == "f32":
            assert sha(w) == case["sha_input"]
        else:
            assert sha(oracle.f32_to_bf16_bits(w).view(np.int16)) == case["sha_input"]
        w32 = w.astype(np.float32)
        packed, scales, shape = oracle.encode(w32, case["group"])
        eff_group = case["group"] if case["group"] % 16 == 0 and case["group"] > 0 else 16
        assert shape == (case["rows"], case["cols"])
        assert packed.size == case["packed_len"] and scales.size == case["scales_len"], case["name"]
        assert sha(packed) == case["sha_packed"], case["name"]
        assert sha(scales.view(np.int16)) == case["sha_scales"], case["name"]
        dec = oracle.decode(packed, scales, shape)
        assert sha(dec) == case["sha_decoded"], case["name"]
        # C restatement agrees with numpy and therefore with the reference
        cp, cs = coracle.encode(w32, eff_group)
        assert np.array_equal(cp, packed) and np.array_equal(cs.view(np.uint16), scales.view(np.uint16)), case["name"]
        cd = coracle.decode(packed, scales, shape, eff_group)
        assert np.array_equal(cd.view(np.uint32), dec.view(np.uint32)), case["name"]
        if case["full"]:
            assert np.array_equal(packed, arrays[case["name"] + "/packed"])
            assert np.array_equal(scales.view(np.uint16), arrays[case["name"] + "/scales"])
            assert np.array_equal(dec.view(np.uint32), arrays[case["name"] + "/decoded"].view(np.uint32))
        # exact storage law: 1.5 bits per (padded) weight, one fp16 scale per group
        padded = -(-case["rows"] * case["cols"] // eff_group) * eff_group
        assert packed.size == padded * 3 // 16 and scales.size == padded // eff_group


def test_special_inputs(golden, oracle, coracle):
    meta, arrays = golden
    for sp in meta["special"]:
        key = "special/" + sp["name"]
        w = arrays[key + "/input"]
        packed, scales, shape = oracle.encode(w, sp["group"])
        assert np.array_equal(packed, arrays[key + "/packed"]), sp["name"]
        assert np.array_equal(scales.view(np.uint16), arrays[key + "/scales"]), sp["name"]
        dec = oracle.decode(packed, scales, shape)
        assert np.array_equal(dec.view(np.uint32), arrays[key + "/decoded"].view(np.uint32)), sp["name"]
        cp, cs = coracle.encode(w, sp["group"])
        assert np.array_equal(cp, packed) and np.array_equal(cs.view(np.uint16), scales.view(np.uint16)), sp["name"]


def test_all_zero_group_is_rank_1640(oracle):
    packed, scales, _ = oracle.encode(np.zeros((1, 32), dtype=np.float32), 32)
    assert np.all(oracle.unpack_codes(packed) == 1640)
    assert scales.view(np.uint16)[0] == 0


def test_rowwise_equals_whole_matrix(golden, oracle):
    meta, _ = golden
    for case in meta["cases"]:
        if not case.get("rowwise_equal"):
            continue
        if case["rows"] * case["cols"] > 1 << 18:
            continue
        w = case_input(oracle, case).astype(np.float32)
        p, s, _ = oracle.encode(w, case["group"])
        for rb in (1, 5, 32):
            p2, s2 = oracle.encode_rowwise(w, case["group"], rb)
            assert np.array_equal(p, p2) and np.array_equal(s.view(np.uint16), s2.view(np.uint16))


def test_rowwise_rejects_bad_layout(oracle):
    w = np.zeros((4, 48), dtype=np.float32)
    with pytest.raises(ValueError):
        oracle.encode_rowwise(w, 32, 4)          # K % g != 0
    with pytest.raises(ValueError):
        oracle.encode_rowwise(np.zeros((4, 64), dtype=np.float32), 16, 4)   # g % 32 != 0
    with pytest.raises(ValueError):
        oracle.encode_rowwise(np.zeros((4, 64), dtype=np.float32), 32, 0)


def test_linear_oracle_against_reference_outputs(golden, oracle, coracle):
    meta, arrays = golden
    checked = 0
    for case in meta["cases"]:
        if "y_norm" not in case:
            continue
        if case["rows"] * case["cols"] > 1 << 21:
            continue
        w = case_input(oracle, case).astype(np.float32)
        packed, scales, _ = oracle.encode(w, case["group"])
        x = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(
            oracle.gen_normal(case["seed"] + 100, 4 * case["cols"], 1.0))).reshape(4, case["cols"])
        y = oracle.linear_fp32(x, packed, scales, case["rows"], case["cols"])
        assert abs(float(np.linalg.norm(y)) - case["y_norm"]) <= 1e-4 * case["y_norm"]
        assert np.allclose(y[0, :3], case["y_head"], rtol=1e-4, atol=1e-5)
        yc = coracle.linear(x, packed, scales, case["rows"], case["cols"])
        assert np.abs(yc - y).max() <= 1e-4 * max(1.0, np.abs(y).max())
        if case["full"]:
            assert np.abs(arrays[case["name"] + "/y"] - y).max() <= 1e-4 * max(1.0, np.abs(y).max())
        checked += 1
    assert checked >= 3


def test_multithreaded_c_oracle_matches_single(oracle, coracle):
    w = oracle.gen_normal(21, 64 * 512, 0.02).reshape(64, 512)
    p1, s1 = coracle.encode(w, 32, threads=1)
    p4, s4 = coracle.encode(w, 32, threads=4)
    assert np.array_equal(p1, p4) and np.array_equal(s1.view(np.uint16), s4.view(np.uint16))
    x = oracle.gen_normal(22, 3 * 512, 1.0).reshape(3, 512)
    y1 = coracle.linear(x, p1, s1, 64, 512, threads=1)
    y4 = coracle.linear(x, p1, s1, 64, 512, threads=4)
    assert np.array_equal(y1, y4)


def test_e8_projection_oracle_against_reference_outputs(golden, oracle):
    """conway_sloane_project / ste_quantize restate ojasx2/math/lattice.py:162-203 and :853-867; the golden file
    holds the reference's own outputs for random vectors at four magnitudes, a quarter-integer grid (ties in
    rounding, in the largest error and in the distance comparison) and integer vectors."""
    meta, arrays = golden
    x, want = arrays["project/input"], arrays["project/output"]
    got = oracle.conway_sloane_project(x)
    assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert hashlib.sha256(np.ascontiguousarray(got).tobytes()).hexdigest() == meta["project"]["sha_output"]
    # every output is a lattice point: all integers or all half-integers, even coordinate sum
    twice = got * 2
    assert np.array_equal(twice, np.rint(twice))
    frac = np.abs(got - np.floor(got))
    assert np.all((frac == 0).all(axis=1) | (frac == 0.5).all(axis=1))
    assert np.all(np.rint(got.sum(axis=1)) % 2 == 0)
    # and no lattice point one coordinate step (or the half-shifted twin) away is closer than the chosen one
    d = ((x - got) ** 2).sum(axis=1)
    assert np.all(d <= 2.0 + 1e-6)                                   # covering radius of E8 is 1
    w, wq = arrays["ste/input"], arrays["ste/output"]
    assert np.array_equal(oracle.ste_quantize(w).view(np.uint32), wq.view(np.uint32))
    assert np.all(wq[3] == 0)                                        # an all-zero row stays zero


def test_two_bit_oracle_against_reference_outputs(golden, oracle):
    """encode_2bit / decode_2bit restate E8LatticePacker (ojasx2/math/lattice.py:210-279); the golden file holds
    the reference's own codes, scales and decoded weights."""
    _, arrays = golden
    for tag in ("g8", "g32", "heavy", "grid"):
        w, g = arrays[f"two_bit/{tag}/input"], int(arrays[f"two_bit/{tag}/group"])
        p, s, shape = oracle.encode_2bit(w, g)
        assert shape == w.shape
        assert np.array_equal(p, arrays[f"two_bit/{tag}/packed"]), tag
        assert np.array_equal(s.view(np.uint16), arrays[f"two_bit/{tag}/scales"]), tag
        assert np.array_equal(oracle.decode_2bit(p, s, w.shape), arrays[f"two_bit/{tag}/decoded"]), tag
        # every 8-block is a point of D8 + 1/2 unless clamping blocked the parity fix: half-integers in [-1.5, 1.5]
        vals = oracle.decode_2bit(p, np.ones_like(s), w.shape)
        assert set(np.unique(vals)).issubset({-1.5, -0.5, 0.5, 1.5})
    with pytest.raises(ValueError):
        oracle.encode_2bit(np.zeros((2, 8), dtype=np.float32), 12)


def test_one_bit_oracle_against_reference_outputs(golden, oracle):
    """encode_1bit / decode_1bit restate RootE8LatticePacker (ojasx2/math/lattice.py:472-537); the golden file holds
    the reference's own codes, least-squares scales and decoded weights, ties and all-zero blocks included."""
    _, arrays = golden
    table = oracle.root_e8_table()
    assert table.shape == (256, 8) and len({tuple(r) for r in table}) == 256
    assert np.all((table * table).sum(axis=1)[:240] == 8) and np.all((table * table).sum(axis=1)[240:] == 4)
    for tag in ("g32", "g8", "grid", "sparse"):
        w, g = arrays[f"one_bit/{tag}/input"], int(arrays[f"one_bit/{tag}/group"])
        p, s, shape = oracle.encode_1bit(w, g)
        assert shape == w.shape
        assert np.array_equal(p, arrays[f"one_bit/{tag}/packed"]), tag
        assert np.array_equal(s.view(np.uint16), arrays[f"one_bit/{tag}/scales"]), tag
        assert np.array_equal(oracle.decode_1bit(p, s, w.shape), arrays[f"one_bit/{tag}/decoded"]), tag
