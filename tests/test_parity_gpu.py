"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle and the
golden vectors generated from the reference.  Bit-exact for codes, scales and decoded weights;
the GEMM contract (max-abs <= 1e-2*|x|_inf*sqrt(K), rel-L2 <= 2e-3) for the linear kernels."""

import hashlib
import math

import numpy as np
import pytest

from conftest import case_input, have_cuda, load_pkg

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def P():
    if not have_cuda():
        pytest.skip("no CUDA device")
    pkg = load_pkg()
    pkg._cabi.lib()          # fails loudly when the extension is missing
    return pkg


DEV = "cuda:0"
TD = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def to_dev(w_np, dtype):
    t = torch.from_numpy(np.ascontiguousarray(w_np).astype(np.float32))
    return t.to(TD[dtype]).to(DEV)       # values are already representable in the target dtype


def f16_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def test_generator_matches_oracle(P, oracle):
    for dt, name in ((torch.float32, "f32"), (torch.float16, "f16"), (torch.bfloat16, "bf16")):
        got = P.ops.generate(5000, 7, 0.02, dt, torch.device(DEV), start=123)
        ref = oracle.gen_normal(7, 5000, 0.02, start=123)
        if name == "f32":
            assert np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32))
        elif name == "f16":
            assert np.array_equal(f16_bits(got), ref.astype(np.float16).view(np.uint16))
        else:
            assert np.array_equal(f16_bits(got), oracle.f32_to_bf16_bits(ref))


def test_encode_bit_exact_golden_cases(P, golden, oracle):
    meta, arrays = golden
    for case in meta["cases"]:
        w = case_input(oracle, case)
        wt = to_dev(w, case["dtype"])
        packed, scales, shape = P.TernaryE8LatticePacker.pack(wt, group_size=case["group"])
        assert shape == (case["rows"], case["cols"])
        assert packed.numel() == case["packed_len"] and scales.numel() == case["scales_len"], case["name"]
        assert sha(packed.cpu().numpy()) == case["sha_packed"], case["name"]
        assert sha(f16_bits(scales).view(np.int16)) == case["sha_scales"], case["name"]
        dec = P.TernaryE8LatticePacker.unpack(packed, scales, shape, dtype=torch.float32)
        assert sha(dec.cpu().numpy()) == case["sha_decoded"], case["name"]


def test_encode_special_inputs(P, golden):
    meta, arrays = golden
    for sp in meta["special"]:
        key = "special/" + sp["name"]
        wt = torch.from_numpy(arrays[key + "/input"]).to(DEV)
        packed, scales, shape = P.TernaryE8LatticePacker.pack(wt, group_size=sp["group"])
        assert np.array_equal(packed.cpu().numpy(), arrays[key + "/packed"]), sp["name"]
        assert np.array_equal(f16_bits(scales), arrays[key + "/scales"]), sp["name"]
        dec = P.TernaryE8LatticePacker.unpack(packed, scales, shape)
        assert np.array_equal(dec.cpu().numpy().view(np.uint32), arrays[key + "/decoded"].view(np.uint32)), sp["name"]


def test_decode_every_code(P, golden):
    _, arrays = golden
    packed = torch.from_numpy(arrays["all_codes/packed"]).to(DEV)
    scales = torch.ones(1641, dtype=torch.float16, device=DEV)
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        dec = P.TernaryE8LatticePacker.unpack(packed, scales, (3282, 8), dtype=dt)
        assert np.array_equal(dec.float().cpu().numpy().astype(np.int8), arrays["all_codes/decoded"])


def test_decode_dtypes_follow_reference_rule(P, oracle):
    w = oracle.gen_normal(31, 64 * 512, 0.02).reshape(64, 512)
    packed_np, scales_np, _ = oracle.encode(w, 32)
    packed = torch.from_numpy(packed_np).to(DEV)
    scales = torch.from_numpy(scales_np.view(np.int16)).view(torch.float16).to(DEV)
    ref32 = oracle.decode(packed_np, scales_np, (64, 512))
    d32 = P.ops.decode(packed, scales, (64, 512), torch.float32).cpu().numpy()
    assert np.array_equal(d32.view(np.uint32), ref32.view(np.uint32))
    d16 = P.ops.decode(packed, scales, (64, 512), torch.float16).float().cpu().numpy()
    assert np.array_equal(d16, ref32)                                  # coord * fp16 scale is exact in fp16
    # bf16: coordinate times the bf16-rounded scale (the reference casts the scale first)
    coords = oracle.decode_coords(packed_np).reshape(-1, 32).astype(np.float32)
    sbf = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(scales_np.astype(np.float32)))
    refbf = (coords * sbf[:, None]).reshape(64, 512)
    dbf = P.ops.decode(packed, scales, (64, 512), torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(dbf, refbf)


def test_rowwise_pack_equals_whole_matrix(P, oracle):
    w = to_dev(oracle.gen_normal(41, 37 * 256, 0.02).reshape(37, 256), "f32")
    p, s, _ = P.TernaryE8LatticePacker.pack(w, 32)
    for rb in (1, 5, 32, 64):
        p2, s2 = P.pack_weight_rowwise(w, bitrate=1.5, group_size=32, row_block=rb)
        assert torch.equal(p, p2) and torch.equal(s, s2)
    with pytest.raises(ValueError):
        P.pack_weight_rowwise(w[:, :48].contiguous(), group_size=32)
    with pytest.raises(ValueError):
        P.pack_weight_rowwise(w, group_size=16)


def _linear_case(P, oracle, n, k, m, xdt, seed, bias=False, force=None, sigma=0.02):
    w = oracle.gen_normal(seed, n * k, sigma).reshape(n, k)
    packed_np, scales_np, _ = oracle.encode(w, 32)
    x32 = oracle.gen_normal(seed + 100, m * k, 1.0).reshape(m, k)
    if xdt == torch.bfloat16:
        x32 = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x32)).reshape(m, k)
    elif xdt == torch.float16:
        x32 = x32.astype(np.float16).astype(np.float32)
    b32 = None
    if bias:
        b32 = oracle.gen_normal(seed + 200, n, 0.5)
        b32 = (oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(b32)) if xdt == torch.bfloat16
               else b32.astype(np.float16).astype(np.float32) if xdt == torch.float16 else b32)
    y_ref = oracle.linear_fp32(x32, packed_np, scales_np, n, k, b32)
    packed = torch.from_numpy(packed_np).to(DEV)
    scales = torch.from_numpy(scales_np.view(np.int16)).view(torch.float16).to(DEV)
    x = torch.from_numpy(x32).to(xdt).to(DEV)
    b = torch.from_numpy(b32).to(xdt).to(DEV) if bias else None
    y = P.ops.linear(x, packed, scales, b, n, k, 32, force=force)
    torch.cuda.synchronize()
    assert y.dtype == xdt and tuple(y.shape) == (m, n)
    d = y.float().cpu().numpy().astype(np.float64) - y_ref
    max_abs, rel_l2 = float(np.abs(d).max()), float(np.linalg.norm(d) / max(np.linalg.norm(y_ref), 1e-30))
    bound_abs, bound_rel = oracle.gemm_tolerance(x32, k)
    assert max_abs <= bound_abs, (n, k, m, max_abs, bound_abs)
    assert rel_l2 <= bound_rel, (n, k, m, rel_l2)
    return max_abs, rel_l2


@pytest.mark.parametrize("n,k", [(16, 256), (100, 512), (64, 4096), (130, 14336), (48, 8192), (33, 3584)])
@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_gemv_bf16(P, oracle, n, k, m):
    _linear_case(P, oracle, n, k, m, torch.bfloat16, seed=n + k + m, bias=(m % 2 == 0))


@pytest.mark.parametrize("m", [1, 5, 16])
def test_gemv_fp16(P, oracle, m):
    _linear_case(P, oracle, 72, 1024, m, torch.float16, seed=77 + m, bias=True)


def test_gemv_fp32_out_is_tight(P, oracle):
    # with fp32 output what is left is the 13-bit fixed-point form of the activations inside the int8
    # tensor-core kernels (error <= 2^-13 of each 256-wide slice's maximum, exact for large elements)
    n, k, m = 96, 4096, 4
    w = oracle.gen_normal(5, n * k, 0.02).reshape(n, k)
    packed_np, scales_np, _ = oracle.encode(w, 32)
    x32 = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.gen_normal(6, m * k, 1.0))).reshape(m, k)
    y_ref = oracle.linear_fp32(x32, packed_np, scales_np, n, k)
    packed = torch.from_numpy(packed_np).to(DEV)
    scales = torch.from_numpy(scales_np.view(np.int16)).view(torch.float16).to(DEV)
    y = P.ops.linear(torch.from_numpy(x32).bfloat16().to(DEV), packed, scales, None, n, k, 32, out_dtype=torch.float32)
    rel = np.linalg.norm(y.cpu().numpy() - y_ref) / np.linalg.norm(y_ref)
    assert rel < 1e-4, rel


@pytest.mark.parametrize("n,k,m,xdt", [(7, 13, 3, torch.float32), (5, 19, 2, torch.float32), (4, 48, 2, torch.float32),
                                       (24, 128, 5, torch.bfloat16), (40, 96, 20, torch.float32)])
def test_generic_path_odd_shapes(P, oracle, n, k, m, xdt):
    # flat packing whose groups cross row boundaries, fp32 activations, K not a multiple of 256
    g = 16 if k % 32 else 32
    w = oracle.gen_normal(n * k, n * k, 0.5).reshape(n, k)
    packed_np, scales_np, _ = oracle.encode(w, g)
    x32 = oracle.gen_normal(3, m * k, 1.0).reshape(m, k)
    if xdt == torch.bfloat16:
        x32 = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x32)).reshape(m, k)
    wd = oracle.decode(packed_np, scales_np, (n, k)).astype(np.float64)
    y_ref = x32.astype(np.float64) @ wd.T
    packed = torch.from_numpy(packed_np).to(DEV)
    scales = torch.from_numpy(scales_np.view(np.int16)).view(torch.float16).to(DEV)
    y = P.ops.linear(torch.from_numpy(x32).to(xdt).to(DEV), packed, scales, None, n, k, g)
    tol = 2e-3 if xdt == torch.bfloat16 else 1e-5
    assert np.linalg.norm(y.float().cpu().numpy() - y_ref) <= tol * np.linalg.norm(y_ref) + 1e-6


@pytest.mark.parametrize("n,k,m", [(128, 256, 256), (256, 1024, 64), (200, 512, 300), (1000, 4096, 513)])
def test_gemm_tcgen05_bf16(P, oracle, n, k, m):
    _linear_case(P, oracle, n, k, m, torch.bfloat16, seed=n + k + m, bias=(m % 2 == 0), force="gemm")
    P.ops.gemm_status(torch.device(DEV))


def test_gemm_tcgen05_fp16(P, oracle):
    _linear_case(P, oracle, 384, 768, 100, torch.float16, seed=9, bias=True, force="gemm")
    P.ops.gemm_status(torch.device(DEV))


def test_gemm_large_magnitude_activations_are_rescaled(P, oracle):
    # bf16 activations far outside the fp16 range go through the power-of-two rescaling pre-pass
    n, k, m = 128, 512, 64
    w = oracle.gen_normal(21, n * k, 0.02).reshape(n, k)
    packed_np, scales_np, _ = oracle.encode(w, 32)
    x32 = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.gen_normal(22, m * k, 1.0) * np.float32(2.0 ** 30))).reshape(m, k)
    y_ref = oracle.linear_fp32(x32, packed_np, scales_np, n, k)
    packed = torch.from_numpy(packed_np).to(DEV)
    scales = torch.from_numpy(scales_np.view(np.int16)).view(torch.float16).to(DEV)
    y = P.ops.linear(torch.from_numpy(x32).bfloat16().to(DEV), packed, scales, None, n, k, 32, out_dtype=torch.float32, force="gemm")
    P.ops.gemm_status(torch.device(DEV))
    assert np.isfinite(y.cpu().numpy()).all()
    assert np.linalg.norm(y.cpu().numpy() - y_ref) / np.linalg.norm(y_ref) < 1e-5


def test_gemm_matches_gemv_small_batch(P, oracle):
    # the two independent kernels agree on the same inputs (M = 16 is legal for both)
    n, k, m = 256, 4096, 16
    w = oracle.gen_normal(1, n * k, 0.02).reshape(n, k)
    packed_np, scales_np, _ = oracle.encode(w, 32)
    packed = torch.from_numpy(packed_np).to(DEV)
    scales = torch.from_numpy(scales_np.view(np.int16)).view(torch.float16).to(DEV)
    x = P.ops.generate(m * k, 2, 1.0, torch.bfloat16, torch.device(DEV)).view(m, k)
    y1 = P.ops.linear(x, packed, scales, None, n, k, 32, out_dtype=torch.float32, force="gemv")
    y2 = P.ops.linear(x, packed, scales, None, n, k, 32, out_dtype=torch.float32, force="gemm")
    P.ops.gemm_status(torch.device(DEV))
    assert float((y1 - y2).norm() / y1.norm()) < 1e-4     # activation fixed-point error of the decode kernel


def test_grouped_gemv_matches_single(P, oracle):
    dev = torch.device(DEV)
    shapes = [(64, 4096), (32, 4096), (48, 14336), (80, 256)]
    m = 4
    entries, singles = [], []
    for i, (n, k) in enumerate(shapes):
        w = P.ops.generate(n * k, 50 + i, 0.02, torch.float16, dev).view(n, k)
        pk, sc = P.ops.encode(w, 32)
        x = P.ops.generate(m * k, 60 + i, 1.0, torch.bfloat16, dev).view(m, k)
        y = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
        entries.append((x, pk, sc, None, y))
        singles.append(P.ops.linear(x, pk, sc, None, n, k, 32))
    grp = P.ops.GroupedGemv(entries, shapes)
    grp()
    torch.cuda.synchronize()
    for (x, pk, sc, b, y), ref in zip(entries, singles):
        assert torch.equal(y, ref)


def test_module_forward_backward_and_state(P, oracle):
    dev = torch.device(DEV)
    lin = torch.nn.Linear(512, 96, bias=True).to(dev)
    layer = P.E8LatticeLinear.from_linear(lin, rank=4, bitrate=1.5, group_size=32)
    assert layer.packed_weight.numel() == 96 * 512 * 3 // 16 and layer.block_scales.numel() == 96 * 512 // 32
    assert layer.packed_weight.dtype == torch.uint8 and layer.block_scales.dtype == torch.float16
    x = torch.randn(3, 5, 512, device=dev, requires_grad=True)
    y = layer(x)
    assert tuple(y.shape) == (3, 5, 96)
    w = layer.unpack_weights(torch.float32)
    y_ref = torch.nn.functional.linear(x.detach(), w, layer.bias)
    assert float((y.detach() - y_ref).abs().max()) < 1e-3
    y.sum().backward()
    assert x.grad is not None and tuple(x.grad.shape) == (3, 5, 512)
    gx_ref = torch.ones(15, 96, device=dev) @ w
    assert float((x.grad.reshape(15, 512) - gx_ref).abs().max()) < 1e-3
    assert layer.lora_B.grad is not None
    sd = layer.state_dict()
    assert set(sd) == {"packed_weight", "block_scales", "bias", "lora_A", "lora_B"}
    # group_size below 16 is coerced to 16, other bit-rates are refused
    small = P.E8LatticeLinear.from_linear(torch.nn.Linear(64, 8).to(dev), bitrate=1.5, group_size=8)
    assert small.group_size == 16
    with pytest.raises(ValueError):
        P.E8LatticeLinear(64, 8, bitrate=3.0)


def test_seam_signature_and_errors(P):
    dev = torch.device(DEV)
    x = torch.zeros(2, 256, dtype=torch.bfloat16, device=dev)
    pk = torch.zeros(16 * 256 * 3 // 16, dtype=torch.uint8, device=dev)
    sc = torch.ones(16 * 256 // 32, dtype=torch.float16, device=dev)
    y = P.dispatch_tilelang_e8_gemm(x, pk, sc, None, 16, 256, 32, 1.5, None)
    assert y is not None and tuple(y.shape) == (2, 16)
    assert P.dispatch_tilelang_e8_gemm(x, pk, sc, None, 16, 256, 32, 2.0, None) is None
    assert P.dispatch_tilelang_e8_gemm(x.cpu(), pk.cpu(), sc.cpu(), None, 16, 256, 32, 1.5, None) is None
    with pytest.raises(RuntimeError):
        P.ops.encode(torch.zeros(4, 32))            # CPU tensor: no fallback
    st = P._cabi.lib().ojx_e8t_encode(None, 0, 4, 32, 32, None, None, None)
    assert st == -1 and P._cabi.status_name(st) == "OJX_ERR_NULL"


def test_full_size_properties_llama_q_proj(P, oracle, coracle):
    """BASELINE-size checks that do not need a slow CPU pass over everything: the encoder's output over a
    full 4096x4096 matrix hashes equal to the C oracle's, row-block packing equals whole packing, and the
    decode GEMV and the tensor-core GEMM agree with a dense fp32 product of the decoded matrix."""
    dev = torch.device(DEV)
    n = k = 4096
    w = P.ops.generate(n * k, 11, 0.02, torch.float16, dev).view(n, k)
    pk, sc = P.ops.encode(w, 32)
    w_host = oracle.gen_normal(11, n * k, 0.02).astype(np.float16).astype(np.float32)
    cp, cs = coracle.encode(w_host, 32, threads=8)
    assert sha(pk.cpu().numpy()) == sha(cp)
    assert sha(f16_bits(sc)) == sha(cs.view(np.uint16))
    p2, s2 = P.pack_weight_rowwise(w, row_block=512)
    assert torch.equal(pk, p2) and torch.equal(sc, s2)
    wd = P.ops.decode(pk, sc, (n, k), torch.float32)
    for m, force in ((1, "gemv"), (16, "gemv"), (2048, "gemm")):
        x = P.ops.generate(m * k, 12 + m, 1.0, torch.bfloat16, dev).view(m, k)
        y = P.ops.linear(x, pk, sc, None, n, k, 32, force=force)
        y_ref = x.float() @ wd.t()
        rel = float((y.float() - y_ref).norm() / y_ref.norm())
        max_abs = float((y.float() - y_ref).abs().max())
        assert rel <= 2e-3 and max_abs <= 1e-2 * float(x.float().abs().max()) * math.sqrt(k), (m, rel, max_abs)
    P.ops.gemm_status(dev)


def test_native_op_schema_entry_points(P, oracle):
    """fused_ternary_e8_gemm_fwd / _bwd_dx with the reference's 2-D row-major operands
    (ojasx_math_bindings.cpp:407-533): forward against the oracle, dX against a dense product."""
    dev = torch.device(DEV)
    n, k, m = 512, 1024, 8
    w = P.ops.generate(n * k, 321, 0.02, torch.float16, dev).view(n, k)
    pk, sc = P.ops.encode(w, 32)
    pk2, sc2 = pk.view(n, k * 3 // 16), sc.view(n, k // 32)
    x = P.ops.generate(m * k, 322, 1.0, torch.bfloat16, dev).view(m, k)
    bias = P.ops.generate(n, 323, 0.1, torch.bfloat16, dev)
    y = P.fused_ternary_e8_gemm_fwd(x, pk2, sc2, bias, 32)
    wd = P.ops.decode(pk, sc, (n, k), torch.float32)
    ref = x.float() @ wd.t() + bias.float()
    assert float((y.float() - ref).norm() / ref.norm()) <= 2e-3
    gy = P.ops.generate(m * n, 324, 1.0, torch.float32, dev).view(m, n)
    dx = P.fused_ternary_e8_gemm_bwd_dx(gy, pk2, sc2, k, 32)
    assert dx.shape == (m, k)
    assert float((dx - gy @ wd).norm() / (gy @ wd).norm()) <= 1e-5
    with pytest.raises(RuntimeError):
        P.fused_ternary_e8_gemm_fwd(x, pk, sc2, None, 32)


def test_gemm_tail_split_matches_dense_product(P):
    """150 big tiles on 148 SMs: the GEMM runs 148 tiles of 256 x 256 and hands the rest of the last token
    block to a second launch with small tiles.  Every output is checked against a dense fp32 product
    (bias included), with a ragged last row block and a ragged last token block."""
    dev = torch.device(DEV)
    n, k, m = 256 * 30 - 40, 512, 256 * 5 - 24
    w = P.ops.generate(n * k, 901, 0.02, torch.float16, dev).view(n, k)
    pk, sc = P.ops.encode(w, 32)
    x = P.ops.generate(m * k, 902, 1.0, torch.bfloat16, dev).view(m, k)
    bias = P.ops.generate(n, 903, 0.1, torch.bfloat16, dev)
    y = P.ops.linear(x, pk, sc, bias, n, k, 32, force="gemm")
    P.ops.gemm_status(dev)
    wd = P.ops.decode(pk, sc, (n, k), torch.float32)
    ref = x.float() @ wd.t() + bias.float()
    d = y.float() - ref
    assert float(d.norm() / ref.norm()) <= 2e-3
    assert float(d.abs().max()) <= 1e-2 * float(x.float().abs().max()) * k ** 0.5
    assert torch.isfinite(y.float()).all()


def test_gemm_long_rows_take_the_two_pass_normalisation(P):
    """K = 16640 is longer than the activation pre-pass keeps in registers (16384): the row is read twice."""
    dev = torch.device(DEV)
    n, k, m = 256, 16640, 40
    w = P.ops.generate(n * k, 911, 0.02, torch.float16, dev).view(n, k)
    pk, sc = P.ops.encode(w, 32)
    x = P.ops.generate(m * k, 912, 1.0, torch.bfloat16, dev).view(m, k)
    x[3] *= 3.0e4                                    # rows of very different magnitude: per-row factors matter
    x[7] *= 1.0e-6
    y = P.ops.linear(x, pk, sc, None, n, k, 32, force="gemm")
    P.ops.gemm_status(dev)
    ref = x.float() @ P.ops.decode(pk, sc, (n, k), torch.float32).t()
    for row in (0, 3, 7, 39):
        d = y[row].float() - ref[row]
        assert float(d.norm() / ref[row].norm()) <= 2e-3, row


def test_e8_projection_matches_reference_bits(P, golden, oracle):
    """ojx_e8t_project / ojx_e8t_ste_quantize against the reference's outputs in the golden file and, on a
    larger seeded input, against the oracle (ojasx2/math/lattice.py:162-203, 853-867)."""
    _, arrays = golden
    dev = torch.device(DEV)
    x = torch.from_numpy(arrays["project/input"]).to(dev)
    got = P.conway_sloane_e8_project(x).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), arrays["project/output"].view(np.uint32))
    w = torch.from_numpy(arrays["ste/input"]).to(dev)
    gq = P._E8STEFunction.apply(w).cpu().numpy()
    assert np.array_equal(gq.view(np.uint32), arrays["ste/output"].view(np.uint32))
    for sigma in (0.2, 1.0, 25.0):
        big = oracle.gen_normal(300, 1 << 20, sigma).reshape(-1, 8)
        assert np.array_equal(P.ops.e8_project(torch.from_numpy(big).to(dev)).cpu().numpy().view(np.uint32),
                              oracle.conway_sloane_project(big).view(np.uint32))
    grid = (np.rint(oracle.gen_normal(301, 1 << 18, 2.0) * 4.0) * 0.25).astype(np.float32).reshape(-1, 8)
    assert np.array_equal(P.ops.e8_project(torch.from_numpy(grid).to(dev)).cpu().numpy(), oracle.conway_sloane_project(grid))
    wbig = oracle.gen_normal(302, 1000 * 1003, 0.03).reshape(1000, 1003)          # element count not a multiple of 8
    assert np.array_equal(P.ops.e8_ste_quantize(torch.from_numpy(wbig).to(dev)).cpu().numpy().view(np.uint32),
                          oracle.ste_quantize(wbig).view(np.uint32))
    # idempotence: lattice points project onto themselves
    again = P.ops.e8_project(torch.from_numpy(got).to(dev)).cpu().numpy()
    assert np.array_equal(again, got)
    with pytest.raises(ValueError):
        P.conway_sloane_e8_project(torch.zeros(4, 7, device=dev))
    assert P.conway_sloane_e8_project(torch.zeros(0, 8, device=dev)).shape == (0, 8)


def test_quantization_aware_linear_trains_through_the_quantizer(P):
    """E8QuantizationAwareLinear (ojasx2/math/lattice.py:870-899): forward uses quantized weights, the gradient
    reaches the dense weights unchanged (straight-through)."""
    dev = torch.device(DEV)
    torch.manual_seed(5)
    layer = P.E8QuantizationAwareLinear(64, 24, bias=True, device=dev)
    x = torch.randn(6, 64, device=dev)
    wq = P.ops.e8_ste_quantize(layer.weight)
    y = layer(x)
    assert torch.allclose(y, torch.nn.functional.linear(x, wq, layer.bias), atol=1e-6)
    y.sum().backward()
    assert torch.allclose(layer.weight.grad, x.sum(0).expand(24, 64), atol=1e-5)
    wb = layer.weight.detach().to(torch.bfloat16)                   # 16-bit tensors: quantized in fp32, rounded back
    half = P.ops.e8_ste_quantize(wb)
    assert half.dtype == torch.bfloat16 and torch.equal(half, P.ops.e8_ste_quantize(wb.float()).to(torch.bfloat16))


@pytest.mark.parametrize("rows,cols,group,sigma,dtype", [(64, 256, 8, 0.02, "f32"), (33, 100, 8, 1.0, "f32"),
                                                         (128, 512, 32, 0.02, "f16"), (16, 256, 64, 0.5, "bf16"),
                                                         (7, 13, 16, 0.3, "f32"), (40, 64, 24, 2.0, "f32"),
                                                         (512, 4096, 8, 0.02, "bf16")])
def test_two_bit_packer_matches_oracle_bits(P, oracle, rows, cols, group, sigma, dtype):
    """ojx_e8t_encode_2bit / ojx_e8t_decode_2bit against the restatement of E8LatticePacker
    (ojasx2/math/lattice.py:210-279), which the golden vectors pin to the reference: codes and scales bit for
    bit for every group size and a padded tail, decoded weights bit for bit in fp32."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(500 + rows, rows * cols, sigma).reshape(rows, cols).copy()).to(TD[dtype])
    want_p, want_s, _ = oracle.encode_2bit(w.float().numpy(), group)
    got_p, got_s, shape = P.E8LatticePacker.pack(w.to(dev), group_size=group)
    assert shape == (rows, cols)
    assert np.array_equal(got_p.cpu().numpy(), want_p)
    assert np.array_equal(got_s.view(torch.int16).cpu().numpy(), want_s.view(np.int16))
    dec = P.E8LatticePacker.unpack(got_p, got_s, (rows, cols), dtype=torch.float32).cpu().numpy()
    assert np.array_equal(dec.view(np.uint32), oracle.decode_2bit(want_p, want_s, (rows, cols)).view(np.uint32))
    unit = torch.from_numpy(oracle.decode_2bit(want_p, np.ones_like(want_s), (rows, cols)))          # code - 1.5
    per_weight = torch.from_numpy(want_s).repeat_interleave(group)[: rows * cols].view(rows, cols)      # fp16 scales
    for dt in (torch.float16, torch.bfloat16):            # (code - 1.5) * cast(scale), rounded to the output type
        d16 = P.E8LatticePacker.unpack(got_p, got_s, (rows, cols), dtype=dt).cpu()
        assert torch.equal(d16, unit.to(dt) * per_weight.to(dt))
    with pytest.raises(ValueError):
        P.E8LatticePacker.pack(w.to(dev), group_size=12)


def test_two_bit_golden_and_special_inputs(P, golden, oracle):
    _, arrays = golden
    dev = torch.device(DEV)
    for tag in ("g8", "g32", "heavy", "grid"):
        w = torch.from_numpy(arrays[f"two_bit/{tag}/input"]).to(dev)
        g = int(arrays[f"two_bit/{tag}/group"])
        p, s, _ = P.E8LatticePacker.pack(w, group_size=g)
        assert np.array_equal(p.cpu().numpy(), arrays[f"two_bit/{tag}/packed"]), tag
        assert np.array_equal(s.view(torch.int16).cpu().numpy().view(np.uint16), arrays[f"two_bit/{tag}/scales"]), tag
        d = P.E8LatticePacker.unpack(p, s, tuple(w.shape), dtype=torch.float32).cpu().numpy()
        assert np.array_equal(d, arrays[f"two_bit/{tag}/decoded"]), tag


def test_two_bit_layer_with_reference_defaults(P, oracle):
    """E8LatticeLinear() with the reference's defaults (2.0 bits, groups of 8): forward against the fp32
    dequantize-then-matmul of the oracle within the GEMM contract, backward dX, rotation, streaming rows."""
    dev = torch.device(DEV)
    torch.manual_seed(9)
    lin = torch.nn.Linear(256, 96, bias=True).to(dev)
    for had in (False, True):
        layer = P.E8LatticeLinear.from_linear(lin, rank=4, use_hadamard=had)
        assert layer.bitrate == 2.0 and layer.group_size == 8 and layer.packed_weight.numel() == 96 * 256 // 4
        src = P.fwht_block32(lin.weight.detach()) if had else lin.weight.detach()
        want_p, want_s, _ = oracle.encode_2bit(src.cpu().numpy(), 8)
        assert np.array_equal(layer.packed_weight.cpu().numpy(), want_p)
        wd = torch.from_numpy(oracle.decode_2bit(want_p, want_s, (96, 256))).to(dev)
        assert torch.equal(layer.unpack_weights(torch.float32), P.fwht_block32(wd) if had else wd)
        for m, dt in ((1, torch.float32), (5, torch.bfloat16), (33, torch.float16)):
            x = torch.randn(m, 256, device=dev).to(dt).requires_grad_(True)
            y = layer(x)
            xr = P.fwht_block32(x.detach()) if had else x.detach()
            ref = xr.float() @ wd.t() + lin.bias.detach().to(dt).float()
            tol_abs, tol_rel = oracle.gemm_tolerance(x.detach().float().cpu().numpy(), 256)
            err = (y.float() - ref)
            assert float(err.abs().max()) <= tol_abs and float(err.norm() / ref.norm()) <= max(tol_rel, 4e-3 if dt != torch.float32 else 0)
            y.float().sum().backward()
            gref = torch.ones(m, 96, device=dev) @ wd
            gref = P.fwht_block32(gref) if had else gref
            assert float((x.grad.float() - gref).abs().max()) <= 2e-2 * float(gref.abs().max())
    rowwise_p, rowwise_s = P.pack_weight_rowwise(lin.weight.detach(), bitrate=2.0, group_size=32, row_block=7)
    whole_p, whole_s = P.ops.encode_2bit(lin.weight.detach(), 32)
    assert torch.equal(rowwise_p, whole_p) and torch.equal(rowwise_s, whole_s)
    model = P.pack_model_e8(torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8)).to(dev))
    assert all(isinstance(model[i], P.E8LatticeLinear) and model[i].bitrate == 2.0 for i in (0, 2))
    assert model(torch.randn(3, 64, device=dev)).shape == (3, 8)


def test_two_bit_and_projection_operators_compile_without_graph_breaks(P, oracle):
    """torch.ops.ojasx_math_native.fused_e8_gemm_fwd / _bwd_dx / conway_sloane_e8_project_tensor (schemas of
    ojasx2/math/csrc/ojasx_math_bindings.cpp:586-595) carry the 2.0-bit layer and the projection through
    torch.compile(fullgraph=True)."""
    dev = torch.device(DEV)
    torch.manual_seed(2)
    layer = P.E8LatticeLinear.from_linear(torch.nn.Linear(128, 40).to(dev), group_size=32)      # 2.0 bits
    x = torch.randn(6, 128, device=dev, requires_grad=True)
    eager = layer(x)
    compiled = torch.compile(layer, fullgraph=True, backend="aot_eager")
    y = compiled(x)
    assert torch.allclose(y, eager, atol=1e-5)
    y.sum().backward()
    wd = layer.unpack_weights(torch.float32)
    assert torch.allclose(x.grad, torch.ones(6, 40, device=dev) @ wd, atol=1e-4)
    ns = torch.ops.ojasx_math_native
    direct = ns.fused_e8_gemm_fwd(x.detach(), layer.packed_weight.view(40, -1), layer.block_scales.view(40, -1), layer.bias, 32)
    assert torch.allclose(direct, eager, atol=1e-5)
    v = torch.from_numpy(oracle.gen_normal(9, 64 * 8, 1.5).reshape(64, 8)).to(dev)
    snap = torch.compile(lambda t: P.conway_sloane_e8_project(t) * 2.0, fullgraph=True, backend="aot_eager")
    assert np.array_equal(snap(v).cpu().numpy(), oracle.conway_sloane_project(v.cpu().numpy()) * 2.0)


@pytest.mark.parametrize("rows,cols,group,sigma,dtype", [(64, 256, 32, 0.02, "f32"), (33, 100, 8, 1.0, "f32"),
                                                         (128, 512, 32, 0.02, "f16"), (16, 256, 64, 0.5, "bf16"),
                                                         (7, 13, 16, 0.3, "f32"), (40, 64, 24, 2.0, "f32"),
                                                         (64, 256, 128, 1.0, "f32"), (256, 4096, 32, 0.02, "bf16")])
def test_one_bit_packer_matches_oracle_bits(P, oracle, rows, cols, group, sigma, dtype):
    """ojx_e8t_encode_1bit / ojx_e8t_decode_1bit against the restatement of RootE8LatticePacker
    (ojasx2/math/lattice.py:472-537), which the golden vectors pin to the reference: codes, least-squares scales
    and decoded weights bit for bit, every group size (one that is not a multiple of 8 becomes 8), padded tails."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(700 + rows, rows * cols, sigma).reshape(rows, cols).copy()).to(TD[dtype])
    want_p, want_s, _ = oracle.encode_1bit(w.float().numpy(), group)
    got_p, got_s, shape = P.RootE8LatticePacker.pack(w.to(dev), group_size=group)
    assert shape == (rows, cols)
    assert np.array_equal(got_p.cpu().numpy(), want_p)
    assert np.array_equal(got_s.view(torch.int16).cpu().numpy(), want_s.view(np.int16))
    dec = P.RootE8LatticePacker.unpack(got_p, got_s, (rows, cols), dtype=torch.float32).cpu().numpy()
    assert np.array_equal(dec.view(np.uint32), oracle.decode_1bit(want_p, want_s, (rows, cols)).view(np.uint32))
    odd_p, odd_s, _ = P.RootE8LatticePacker.pack(w.to(dev), group_size=12)          # replaced by 8, as the reference does
    ref_p, ref_s, _ = oracle.encode_1bit(w.float().numpy(), 12)
    assert np.array_equal(odd_p.cpu().numpy(), ref_p) and odd_s.numel() == ref_s.size


def test_one_bit_golden_ties_and_layer(P, golden, oracle):
    _, arrays = golden
    dev = torch.device(DEV)
    for tag in ("g32", "g8", "grid", "sparse"):
        w = torch.from_numpy(arrays[f"one_bit/{tag}/input"]).to(dev)
        g = int(arrays[f"one_bit/{tag}/group"])
        p, s, _ = P.RootE8LatticePacker.pack(w, group_size=g)
        assert np.array_equal(p.cpu().numpy(), arrays[f"one_bit/{tag}/packed"]), tag
        assert np.array_equal(s.view(torch.int16).cpu().numpy().view(np.uint16), arrays[f"one_bit/{tag}/scales"]), tag
        d = P.RootE8LatticePacker.unpack(p, s, tuple(w.shape), dtype=torch.float32).cpu().numpy()
        assert np.array_equal(d, arrays[f"one_bit/{tag}/decoded"]), tag
    torch.manual_seed(4)
    lin = torch.nn.Linear(256, 48, bias=True).to(dev)
    layer = P.E8LatticeLinear.from_linear(lin, rank=2, bitrate=1.0, group_size=32)
    wd = layer.unpack_weights(torch.float32)
    x = torch.randn(5, 256, device=dev, requires_grad=True)
    y = layer(x)
    assert torch.allclose(y, x.detach() @ wd.t() + lin.bias.detach(), atol=1e-4)
    y.sum().backward()
    assert torch.allclose(x.grad, torch.ones(5, 48, device=dev) @ wd, atol=1e-4)
    rp, rs = P.pack_weight_rowwise(lin.weight.detach(), bitrate=1.0, group_size=32, row_block=5)
    wp, ws = P.ops.encode_1bit(lin.weight.detach(), 32)
    assert torch.equal(rp, wp) and torch.equal(rs, ws)


@pytest.mark.parametrize("bits", [2, 1])
@pytest.mark.parametrize("m,k,n,group,dt", [(1, 4096, 4096, 32, torch.bfloat16), (3, 256, 40, 8, torch.float16),
                                             (8, 4096, 96, 64, torch.bfloat16), (1, 14336, 64, 32, torch.float32),
                                             (2, 1024, 33, 16, torch.bfloat16), (9, 512, 24, 32, torch.bfloat16), (9, 512, 24, 32, torch.float32), (12, 320, 24, 32, torch.bfloat16),
                                             (5, 512, 40, 8, torch.bfloat16), (3, 512, 40, 8, torch.bfloat16), (6, 768, 16, 32, torch.float16)])
def test_low_bit_decode_linear_matches_dense_product(P, oracle, bits, m, k, n, group, dt):
    """ojx_e8t_linear_2bit / _1bit at decode shapes (the tensor-core or the shared-memory kernel for up to eight rows;
    beyond, the prefill kernel or the scalar kernel) against the fp32 product with the decoded weights: fp32
    accumulation of exact products, so the error stays within 1e-5 of sum |x||w| per output."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(900 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    enc, dec, lin = ((P.ops.encode_2bit, P.ops.decode_2bit, P.ops.linear_2bit) if bits == 2
                     else (P.ops.encode_1bit, P.ops.decode_1bit, P.ops.linear_1bit))
    pk, sc = enc(w, group)
    # more than eight rows of 16-bit activations with groups of 32 and K % 256 == 0 run the prefill kernel, whose
    # operand is the weight rounded to fp16
    prefill = (m > 8 or (m >= 4 and not (group == 32 and k % 2048 == 0))) and group in (8, 16, 32) and k % 256 == 0 and dt != torch.float32
    wd = dec(pk, sc, (n, k), torch.float16).float() if prefill else dec(pk, sc, (n, k), torch.float32)
    x = torch.from_numpy(oracle.gen_normal(901 + m, m * k, 1.0).reshape(m, k).copy()).to(dt).to(dev)
    bias = torch.from_numpy(oracle.gen_normal(902, n, 0.1).copy()).to(dt).to(dev)
    y = lin(x, pk, sc, bias, n, k, group, out_dtype=torch.float32)
    ref = x.float() @ wd.t() + bias.float()
    magnitude = x.float().abs() @ wd.abs().t() + bias.float().abs()
    assert float(((y - ref).abs() / magnitude).max()) < 1e-5
    y16 = lin(x, pk, sc, None, n, k, group)
    assert y16.dtype == dt and float((y16.float() - (ref - bias.float())).abs().max()) <= 2.0 ** -7 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize("m,k,n,dt", [(1, 2048, 40, torch.bfloat16), (1, 4096, 4096, torch.bfloat16), (1, 14336, 100, torch.float16),
                                      (1, 8192, 17, torch.float32), (2, 4096, 100, torch.bfloat16), (3, 2048, 33, torch.float16),
                                      (4, 8192, 64, torch.bfloat16), (5, 2048, 48, torch.float32), (8, 4096, 4096, torch.bfloat16),
                                      (7, 4096, 20, torch.float16)])
@pytest.mark.parametrize("bits", [2, 1])
def test_low_bit_tensor_core_kernels(P, oracle, bits, m, k, n, dt):
    """gemv_b2_kernel / gemv_b1_kernel (one to eight rows, groups of 32, K % 2048 == 0) against the dense fp32 product: within 1e-5 of
    sum |x||w| per output (row counts that are not multiples of 16 included), outliers do not hurt their neighbours,
    scaling x by a power of two scales y exactly, Inf / NaN give the dense product's pattern and leave the other rows
    of x within the same bound."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(950 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    enc, dec, lin = ((P.ops.encode_2bit, P.ops.decode_2bit, P.ops.linear_2bit) if bits == 2
                     else (P.ops.encode_1bit, P.ops.decode_1bit, P.ops.linear_1bit))
    pk, sc = enc(w, 32)
    wd = dec(pk, sc, (n, k), torch.float32)
    x = torch.from_numpy(oracle.gen_normal(951 + m, m * k, 1.0).reshape(m, k).copy()).to(dt).to(dev)
    for r in range(m):
        x[r, 7 + r::256] *= 1.0e3                                    # one outlier per 256-wide round
        x[r] *= 2.0 ** (r - 4 if dt == torch.float16 else 2 * r)     # every row on its own scale
    bias = torch.from_numpy(oracle.gen_normal(952, n, 0.1).copy()).to(dt).to(dev)
    y = lin(x, pk, sc, bias, n, k, 32, out_dtype=torch.float32)
    ref = x.float() @ wd.t() + bias.float()
    magnitude = x.float().abs() @ wd.abs().t() + bias.float().abs()
    assert float(((y - ref).abs() / magnitude).max()) < 1e-5
    y0 = lin(x, pk, sc, None, n, k, 32, out_dtype=torch.float32)
    for s in (-30, 20):
        if dt == torch.float16:
            continue                                                 # would leave fp16's range
        ys = lin(x * 2.0 ** s, pk, sc, None, n, k, 32, out_dtype=torch.float32)
        assert torch.equal(ys, y0 * 2.0 ** s), s
    xi = x.clone()
    xi[0, 5] = float("inf")
    xi[m - 1, k - 1] = float("-inf")
    yi = lin(xi, pk, sc, None, n, k, 32, out_dtype=torch.float32)
    ri = xi.float() @ wd.t()
    assert torch.equal(torch.isnan(yi), torch.isnan(ri)) and torch.equal(torch.isposinf(yi), torch.isposinf(ri))
    assert torch.equal(torch.isneginf(yi), torch.isneginf(ri))
    fin = torch.isfinite(ri)
    if bool(fin.any()):
        assert float((((yi - ri).abs() / (magnitude - bias.float().abs()))[fin]).max()) < 1e-5
    xn = x.clone()
    xn[m // 2, 100] = float("nan")
    yn = lin(xn, pk, sc, None, n, k, 32, out_dtype=torch.float32)
    assert torch.isnan(yn[m // 2]).all() and int(torch.isnan(yn).sum()) == n


@pytest.mark.parametrize("bits", [2, 1])
@pytest.mark.parametrize("m,k,n,dt,with_bias,group", [(64, 256, 40, torch.float16, False, 32), (17, 512, 256, torch.float16, True, 32),
                                                      (300, 1024, 500, torch.bfloat16, True, 32), (2048, 4096, 4096, torch.bfloat16, False, 32),
                                                      (129, 2048, 8, torch.bfloat16, False, 32), (300, 1024, 500, torch.bfloat16, True, 8),
                                                      (70, 512, 264, torch.float16, False, 16), (512, 4096, 1024, torch.bfloat16, False, 8)])
def test_low_bit_prefill_gemm_matches_dense_product(P, oracle, bits, m, k, n, dt, with_bias, group):
    """ojx_e8t_gemm_lowbit (the tcgen05 prefill kernel with the 2.0-bit / 1.0-bit decoders) against the fp32 product
    with the weights decoded to fp16 - the operand the tensor cores see: fp32 accumulation of exact products, so the
    error stays within 2e-5 of sum |x||w| per output; tile edges in both directions and scale groups of 8, 16 and 32
    weights (the reference layer's default is 8) included."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(970 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    enc, dec, lin = ((P.ops.encode_2bit, P.ops.decode_2bit, P.ops.linear_2bit) if bits == 2
                     else (P.ops.encode_1bit, P.ops.decode_1bit, P.ops.linear_1bit))
    pk, sc = enc(w, group)
    wd = dec(pk, sc, (n, k), torch.float16).float()
    x = torch.from_numpy(oracle.gen_normal(971 + m, m * k, 1.0).reshape(m, k).copy()).to(dt).to(dev)
    x[m // 2] *= 64.0                                                    # rows on different scales
    bias = torch.from_numpy(oracle.gen_normal(972, n, 0.1).copy()).to(dt).to(dev) if with_bias else None
    y = lin(x, pk, sc, bias, n, k, group, out_dtype=torch.float32)
    P.ops.gemm_status(dev)
    ref = x.float() @ wd.t() + (bias.float() if with_bias else 0.0)
    magnitude = x.float().abs() @ wd.abs().t() + (bias.float().abs() if with_bias else 0.0)
    assert float(((y - ref).abs() / magnitude.clamp_min(1e-30)).max()) < 2e-5
    y16 = lin(x, pk, sc, bias, n, k, group)
    assert y16.dtype == dt and float((y16.float() - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max()) + 1e-3
    if bits == 2:                                                        # the fp16 rounding of (code - 1.5) * scale is within the tolerance of the path
        exact = x.float() @ dec(pk, sc, (n, k), torch.float32).t() + (bias.float() if with_bias else 0.0)
        assert float((y - exact).norm() / exact.norm()) <= 2e-3


def test_low_bit_layer_prefill_runs_on_the_tensor_core_kernel(P):
    """E8LatticeLinear with the reference's default bit-rate (2.0) and with 1.0 on a batch of tokens: forward through the
    prefill kernel equals the product with the unpacked fp16 weights; backward still gives dY . W."""
    dev = torch.device(DEV)
    torch.manual_seed(11)
    for bitrate in (2.0, 1.0):
        lin = torch.nn.Linear(512, 96, bias=True).to(dev).to(torch.bfloat16)
        layer = P.E8LatticeLinear.from_linear(lin, rank=0, bitrate=bitrate)           # the reference's default group size: 8
        assert layer.group_size == 8
        wd = layer.unpack_weights(torch.float16).float()
        x = torch.randn(3, 40, 512, device=dev, dtype=torch.bfloat16, requires_grad=True)
        y = layer(x)
        ref = x.detach().float() @ wd.t() + layer.bias.float()
        assert y.shape == (3, 40, 96) and float((y.float() - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max()) + 1e-3
        y.float().sum().backward()
        gref = torch.ones(120, 96, device=dev) @ layer.unpack_weights(torch.float32)
        assert float((x.grad.float().reshape(120, 512) - gref).abs().max()) <= 2.0 ** -6 * float(gref.abs().max()) + 1e-3


@pytest.mark.parametrize("bits", [2, 1])
@pytest.mark.parametrize("m,k,n,dt,group", [(64, 256, 40, torch.float16, 32), (300, 1024, 504, torch.bfloat16, 32),
                                            (2048, 4096, 4096, torch.bfloat16, 32), (33, 512, 8, torch.bfloat16, 32),
                                            (300, 1024, 504, torch.bfloat16, 8), (64, 512, 72, torch.float16, 16),
                                            (512, 4096, 1024, torch.bfloat16, 8)])
def test_low_bit_backward_dx_matches_dense_product(P, oracle, bits, m, k, n, dt, group):
    """ojx_e8t_gemm_dx_lowbit: dX = dY . W for the 2.0-bit / 1.0-bit formats against the fp32 product with the weights
    decoded to fp16 (the tensor cores' operand), within 2e-5 of sum |dy||w| per output; a weight-row count that is not a
    multiple of the 64-row contraction block included."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(980 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    enc, dec = (P.ops.encode_2bit, P.ops.decode_2bit) if bits == 2 else (P.ops.encode_1bit, P.ops.decode_1bit)
    pk, sc = enc(w, group)
    wd = dec(pk, sc, (n, k), torch.float16).float()
    gy = torch.from_numpy(oracle.gen_normal(981 + m, m * n, 1.0).reshape(m, n).copy()).to(dt).to(dev)
    gy[m // 3] *= 32.0
    dx = P.ops.linear_dx_lowbit(bits, gy, pk, sc, n, k, group, out_dtype=torch.float32)
    P.ops.gemm_status(dev)
    ref = gy.float() @ wd
    magnitude = gy.float().abs() @ wd.abs()
    assert float(((dx - ref).abs() / magnitude.clamp_min(1e-30)).max()) < 2e-5
    # fp32 gradients take the decode-and-multiply route
    dx32 = P.ops.linear_dx_lowbit(bits, gy.float(), pk, sc, n, k, group)
    assert dx32.dtype == torch.float32 and float((dx32 - gy.float() @ dec(pk, sc, (n, k), torch.float32)).abs().max()) <= 1e-3 * float(ref.abs().max())


@pytest.mark.parametrize("m,k,n,dt", [(1, 512, 40, torch.bfloat16), (5, 4096, 1000, torch.float16), (300, 1024, 520, torch.bfloat16),
                                      (2048, 4096, 4096, torch.bfloat16), (2, 14336, 40, torch.bfloat16), (12, 1024, 72, torch.float16),
                                      (8, 2048, 24, torch.bfloat16)])
def test_ternary_groups_of_16_run_the_tensor_core_kernels(P, oracle, m, k, n, dt):
    """Ternary codes with one scale per 16 weights (what the reference layer's default group size of 8 becomes for this
    format, ojasx2/math/lattice.py:750-751): forward (the shared-memory fp32 kernel for one or two rows, the tcgen05 kernel
    beyond) and backward (tcgen05) against the fp32 products with the decoded weights, which are exact in fp16 -
    within 2e-5 of sum |x||w| per output."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(990 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    pk, sc = P.ops.encode(w, 16)
    assert sc.numel() == n * k // 16
    wd = P.ops.decode(pk, sc, (n, k), torch.float32)
    x = torch.from_numpy(oracle.gen_normal(991 + m, m * k, 1.0).reshape(m, k).copy()).to(dt).to(dev)
    bias = torch.from_numpy(oracle.gen_normal(992, n, 0.1).copy()).to(dt).to(dev)
    y = P.ops.linear(x, pk, sc, bias, n, k, 16, out_dtype=torch.float32)
    P.ops.gemm_status(dev)
    ref = x.float() @ wd.t() + bias.float()
    magnitude = x.float().abs() @ wd.abs().t() + bias.float().abs()
    assert float(((y - ref).abs() / magnitude).max()) < 2e-5
    gy = torch.from_numpy(oracle.gen_normal(993 + m, m * n, 1.0).reshape(m, n).copy()).to(dt).to(dev)
    dx = P.ops.linear_dx(gy, pk, sc, n, k, 16, out_dtype=torch.float32)
    P.ops.gemm_status(dev)
    assert float(((dx - gy.float() @ wd).abs() / (gy.float().abs() @ wd.abs()).clamp_min(1e-30)).max()) < 2e-5
    # a layer built with the reference's defaults except the bit-rate
    if m == 5:
        lin = torch.nn.Linear(k, 64, bias=True).to(dev).to(dt)
        layer = P.E8LatticeLinear.from_linear(lin, rank=0, bitrate=1.5)
        assert layer.group_size == 16
        out = layer(x)
        refl = x.float() @ layer.unpack_weights(torch.float32).t() + layer.bias.float()
        assert float((out.float() - refl).abs().max()) <= 2.0 ** -7 * float(refl.abs().max()) + 1e-3


@pytest.mark.parametrize("m,k,n,group", [(1, 4096, 4096, 32), (4, 1024, 40, 32), (8, 2048, 17, 64), (2, 320, 24, 32)])
def test_ternary_fp32_activations_at_decode_shapes(P, oracle, m, k, n, group):
    """fp32 activations (the dtype of the reference's CPU tests) at decode shapes run the shared-memory fp32 kernel
    (K % 64 == 0, power-of-two groups from 16) or the scalar one: exact products, fp32 accumulation - within 1e-5 of
    sum |x||w| per output."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(995 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    pk, sc = P.ops.encode(w, group)
    wd = P.ops.decode(pk, sc, (n, k), torch.float32)
    x = torch.from_numpy(oracle.gen_normal(996 + m, m * k, 1.0).reshape(m, k).copy()).to(dev)
    x[0, 3::97] *= 1.0e3
    bias = torch.from_numpy(oracle.gen_normal(997, n, 0.1).copy()).to(dev)
    y = P.ops.linear(x, pk, sc, bias, n, k, group)
    ref = x @ wd.t() + bias
    magnitude = x.abs() @ wd.abs().t() + bias.abs()
    assert y.dtype == torch.float32 and float(((y - ref).abs() / magnitude).max()) < 1e-5


@pytest.mark.parametrize("bits", [2, 1])
@pytest.mark.parametrize("m,k,n,r,dt", [(1, 4096, 100, 8, torch.bfloat16), (4, 2048, 48, 16, torch.float16), (8, 4096, 33, 3, torch.float32)])
def test_low_bit_adapter_epilogue(P, oracle, bits, m, k, n, r, dt):
    """ojx_e8t_linear_lowbit_lora: the packed product, bias and the low-rank term in one launch of the int8 tensor-core
    decode kernels, against the fp32 sum of the three - within 1e-5 of sum |x||w| + |bias| + sum |t||B| per output;
    then a layer with an adapter at decode shapes against the reference's formula (lattice.py:839-842)."""
    dev = torch.device(DEV)
    w = torch.from_numpy(oracle.gen_normal(1000 + n, n * k, 0.02).reshape(n, k).copy()).to(dev)
    enc, dec = (P.ops.encode_2bit, P.ops.decode_2bit) if bits == 2 else (P.ops.encode_1bit, P.ops.decode_1bit)
    pk, sc = enc(w, 32)
    wd = dec(pk, sc, (n, k), torch.float32)
    x = torch.from_numpy(oracle.gen_normal(1001 + m, m * k, 1.0).reshape(m, k).copy()).to(dt).to(dev)
    bias = torch.from_numpy(oracle.gen_normal(1002, n, 0.1).copy()).to(dt).to(dev)
    t = torch.from_numpy(oracle.gen_normal(1003, m * r, 1.0).reshape(m, r).copy()).to(dev)
    b = torch.from_numpy(oracle.gen_normal(1004, r * n, 0.05).reshape(r, n).copy()).to(dt).to(dev)
    y = P.ops.linear_lowbit_lora(bits, x, pk, sc, bias, n, k, 32, t, b, out_dtype=torch.float32)
    ref = x.float() @ wd.t() + bias.float() + t @ b.float()
    magnitude = x.float().abs() @ wd.abs().t() + bias.float().abs() + t.abs() @ b.float().abs()
    assert float(((y - ref).abs() / magnitude).max()) < 1e-5
    with pytest.raises(ValueError):
        P.ops.linear_lowbit_lora(bits, x[:1].repeat(9, 1), pk, sc, bias, n, k, 32, t[:1].repeat(9, 1), b)
    if dt == torch.bfloat16:
        torch.manual_seed(5)
        lin = torch.nn.Linear(k, 64, bias=True).to(dev).to(dt)
        layer = P.E8LatticeLinear.from_linear(lin, rank=r, bitrate=float(bits), group_size=32)
        with torch.no_grad():
            layer.lora_B.copy_(torch.randn_like(layer.lora_B) * 0.05)
            out = layer(x)
            wl = layer.unpack_weights(torch.float32)
            refl = (x.float() @ wl.t() + layer.bias.float()
                    + layer.scaling * ((x.float() @ layer.lora_A.float()) @ layer.lora_B.float()))
        assert float((out.float() - refl).abs().max()) <= 2.0 ** -6 * float(refl.abs().max()) + 1e-3
