"""CPU-side checks: the C-ABI library loads and exports every declared symbol (no compute calls),
the header and the binding agree, the host mirror keeps the reference's names/signatures/errors,
and the column-sharding logic works across two gloo ranks."""

import ctypes
import importlib
import inspect
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, load_pkg

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def P():
    pkg = load_pkg()
    pkg._cabi.build()              # nvcc cross-compiles sm_100a without a GPU
    return pkg


def header_functions():
    text = open(os.path.join(ROOT, "include", "ojx_e8t.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ojx_e8t_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(P):
    lib = ctypes.CDLL(P._cabi.LIB_PATH)
    declared = header_functions()
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ojx_e8t.h but not exported"
    assert sorted(P._cabi.EXPORTED_SYMBOLS) == declared
    assert P._cabi.lib().ojx_e8t_version() >= 100
    assert P._cabi.status_name(0) == "OJX_OK" and P._cabi.status_name(-7) == "OJX_ERR_TIMEOUT"


def test_pure_host_entry_points(P):
    lib = P._cabi.lib()
    # tile / chunk arithmetic is host-only
    assert lib.ojx_e8t_gemv_kchunks(4096) == 1 and lib.ojx_e8t_gemv_kchunks(14336) == 4
    assert lib.ojx_e8t_gemv_kchunks(8192) == 2 and lib.ojx_e8t_gemv_kchunks(100) == 0
    assert lib.ojx_e8t_gemv_tiles(4096, 4096) == 128 and lib.ojx_e8t_gemv_tiles(4096, 14336) == 512      # 32-row tiles x K chunks
    assert lib.ojx_e8t_gemv_tiles(17, 256) == 1 and lib.ojx_e8t_gemv_tiles(33, 256) == 2
    assert lib.ojx_e8t_gemv_workspace_bytes(4, 4096, 4096) == 0
    assert lib.ojx_e8t_gemv_workspace_bytes(4, 4096, 14336) == 4 * 4 * 4096 * 4
    assert lib.ojx_e8t_gemm_workspace_bytes(2048, 4096, 4096) >= 16
    assert ctypes.sizeof(P._cabi.GemvProblem) == 88


def test_argument_validation_needs_no_gpu(P):
    lib = P._cabi.lib()
    assert lib.ojx_e8t_encode(None, 0, 4, 32, 32, None, None, None) == -1          # null
    assert lib.ojx_e8t_decode(None, None, 4, 32, 32, 0, None, None) == -1
    buf = (ctypes.c_uint8 * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.ojx_e8t_encode(p, 0, 0, 32, 32, p, p, None) == -2                   # empty shape
    assert lib.ojx_e8t_gemv(p, 2, 0, p, p, None, 4, 256, 32, p, 2, None, 0, None) == -2
    assert lib.ojx_e8t_gemv(p, 9, 1, p, p, None, 4, 256, 32, p, 2, None, 0, None) == -4   # bad dtype


def test_mirror_keeps_reference_signatures(P):
    sig = inspect.signature
    assert list(sig(P.TernaryE8LatticePacker.pack).parameters) == ["w", "group_size"]
    assert list(sig(P.TernaryE8LatticePacker.unpack).parameters) == ["packed_codes", "scales", "shape", "dtype", "use_workspace"]
    assert list(sig(P._FusedE8GEMMFunction.forward).parameters) == [
        "ctx", "x", "packed_weight", "block_scales", "bias", "out_features", "in_features", "group_size", "bitrate", "use_hadamard"]
    assert list(sig(P.E8LatticeLinear.__init__).parameters) == [
        "self", "in_features", "out_features", "bias", "rank", "lora_alpha", "group_size", "bitrate", "use_hadamard", "device", "dtype"]
    # native-op schemas (ojasx_math_bindings.cpp:592-594)
    assert list(sig(P.fused_ternary_e8_gemm_fwd).parameters) == ["x", "packed_weight", "block_scales", "bias", "group_size"]
    assert sig(P.fused_ternary_e8_gemm_fwd).parameters["group_size"].default == 32
    assert list(sig(P.fused_ternary_e8_gemm_bwd_dx).parameters) == ["grad_y", "packed_weight", "block_scales", "in_features", "group_size"]
    assert list(sig(P.dispatch_tilelang_e8_gemm).parameters) == [
        "x_2d", "packed_weight", "block_scales", "bias", "out_features", "in_features", "group_size", "bitrate", "lut_coords"]
    prw = sig(P.pack_weight_rowwise).parameters
    assert [prw[k].default for k in ("bitrate", "group_size", "row_block", "use_hadamard")] == [1.5, 32, 32, False]
    assert sig(P.E8LatticeLinear.__init__).parameters["bitrate"].default == 2.0
    assert sig(P.pack_model_e8).parameters["group_size"].default == 32


def test_layer_buffers_and_errors_on_cpu(P):
    layer = P.E8LatticeLinear(128, 64, bias=True, rank=2, group_size=32, bitrate=1.5)
    assert layer.packed_weight.numel() == 64 * 128 * 3 // 16 and layer.packed_weight.dtype == torch.uint8
    assert layer.block_scales.numel() == 64 * 128 // 32 and layer.block_scales.dtype == torch.float16
    assert tuple(layer.lora_A.shape) == (128, 2) and tuple(layer.lora_B.shape) == (2, 64)
    odd = P.E8LatticeLinear(13, 7, bias=False, group_size=8, bitrate=1.5)      # padded flat layout, group coerced to 16
    assert odd.group_size == 16 and odd.packed_weight.numel() == 96 * 3 // 16 and odd.block_scales.numel() == 6
    two = P.E8LatticeLinear(64, 8)                     # the reference's defaults: 2.0 bits, groups of 8
    assert two.bitrate == 2.0 and two.group_size == 8
    assert two.packed_weight.numel() == 64 * 8 // 4 and two.block_scales.numel() == 64 * 8 // 8
    one = P.E8LatticeLinear(64, 8, bitrate=1.0, group_size=32)
    assert one.packed_weight.numel() == 64 * 8 // 8 and one.block_scales.numel() == 64 * 8 // 32
    with pytest.raises(ValueError):
        P.E8LatticeLinear(64, 8, bitrate=3.0)
    with pytest.raises(RuntimeError):
        layer(torch.zeros(1, 128))                     # CPU tensors: the CUDA path is the only path
    with pytest.raises(ValueError):
        P.pack_weight_rowwise(torch.zeros(4, 48), group_size=32)
    with pytest.raises(ValueError):
        P.pack_weight_rowwise(torch.zeros(4, 64), group_size=16)
    with pytest.raises(ValueError):
        P.pack_weight_rowwise(torch.zeros(4, 64), row_block=0)
    with pytest.raises(ValueError):
        P.pack_weight_rowwise(torch.zeros(64), group_size=32)
    assert P.dispatch_tilelang_e8_gemm(torch.zeros(1, 32), torch.zeros(6, dtype=torch.uint8),
                                       torch.ones(1, dtype=torch.float16), None, 1, 32, 32, 1.5) is None


def test_luts_and_fwht_match_oracle(P, oracle):
    coords, raw_to_rank, powers = P._get_ternary_e8_luts()
    oc, orr = oracle.ternary_luts()
    assert np.array_equal(coords.numpy(), oc) and np.array_equal(raw_to_rank.numpy(), orr)
    assert powers.tolist() == [3 ** i for i in range(8)]
    x = torch.from_numpy(oracle.gen_normal(3, 4 * 64, 1.0).reshape(4, 64))
    y = P.fwht_block32(x)
    # orthonormal and an involution; untouched when the last dimension is not a multiple of 32
    assert torch.allclose(P.fwht_block32(y), x, atol=1e-5)
    assert torch.allclose(y.norm(), x.norm(), rtol=1e-5)
    z = torch.zeros(2, 33)
    assert P.fwht_block32(z) is z
    h = P.fwht_block32(torch.eye(32))
    assert torch.allclose(h.abs(), torch.full((32, 32), 32 ** -0.5))


def test_fwht_equals_reference_output_bit_for_bit(P, golden):
    """fwht_block32 against outputs of the reference's own function (ojasx2/math/lattice.py:91-102) stored by
    tests/golden/make_golden.py, in the three dtypes the packer is fed with."""
    _, arrays = golden
    for tag, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        x = torch.from_numpy(arrays[f"fwht/{tag}/input"]).to(dt)
        y = P.fwht_block32(x)
        assert y.dtype == dt
        assert np.array_equal(y.float().numpy().view(np.uint32), arrays[f"fwht/{tag}/output"].view(np.uint32)), tag


def test_native_operator_schemas_and_shape_inference(P):
    """The two operators of the reference's native module (ojasx_math_bindings.cpp:592-595) exist under the same
    namespace with the same schema strings, and infer shapes without touching data."""
    ns = torch.ops.ojasx_math_native
    assert "Tensor? bias=None, int group_size=32" in str(ns.fused_ternary_e8_gemm_fwd.default._schema)
    assert "int in_features, int group_size=32" in str(ns.fused_ternary_e8_gemm_bwd_dx.default._schema)
    assert "Tensor? bias=None, int group_size=32" in str(ns.fused_e8_gemm_fwd.default._schema)          # 2.0-bit siblings
    assert "int in_features, int group_size=32" in str(ns.fused_e8_gemm_bwd_dx.default._schema)
    assert str(ns.conway_sloane_e8_project_tensor.default._schema).endswith("(Tensor x) -> Tensor")
    xm2 = torch.empty(5, 256, device="meta", dtype=torch.bfloat16)
    y2 = ns.fused_e8_gemm_fwd(xm2, torch.empty(24, 64, device="meta", dtype=torch.uint8),
                              torch.empty(24, 8, device="meta", dtype=torch.float16), None, 32)
    assert tuple(y2.shape) == (5, 24) and y2.dtype == torch.bfloat16
    assert tuple(ns.conway_sloane_e8_project_tensor(torch.empty(7, 8, device="meta")).shape) == (7, 8)
    x = torch.empty(5, 256, device="meta", dtype=torch.float16)
    pk = torch.empty(24, 48, device="meta", dtype=torch.uint8)
    sc = torch.empty(24, 8, device="meta", dtype=torch.float16)
    y = ns.fused_ternary_e8_gemm_fwd(x, pk, sc, None, 32)
    assert tuple(y.shape) == (5, 24) and y.dtype == torch.float16
    dx = ns.fused_ternary_e8_gemm_bwd_dx(y, pk, sc, 256, 32)
    assert tuple(dx.shape) == (5, 256)
    with pytest.raises((RuntimeError, NotImplementedError)):
        ns.fused_ternary_e8_gemm_fwd(torch.zeros(5, 256), torch.zeros(24, 48, dtype=torch.uint8),
                                     torch.ones(24, 8, dtype=torch.float16), None, 32)     # no CPU implementation


def test_shard_rows_cover_everything(P):
    from importlib import import_module
    sh = import_module(P.__name__ + ".sharding")
    for n in (1, 15, 16, 17, 1024, 4096, 14336, 100):
        for world in (1, 2, 3, 4, 8):
            spans = [sh.shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(s[0] % 16 == 0 for s in spans)
    with pytest.raises(ValueError):
        sh.shard_rows(10, 2, 2)


_WORKER = r'''
import importlib, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["OJX_ROOT"])
from oracle import e8t_oracle as O
pkg = importlib.import_module("ojasx-open-source-cuda_b200")
sh = importlib.import_module("ojasx-open-source-cuda_b200.sharding")
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
N, K, M = int(os.environ["OJX_N"]), 256, 3
w = O.gen_normal(5, N * K, 0.02).reshape(N, K)
packed_np, scales_np, _ = O.encode(w, 32)
x = O.gen_normal(6, M * K, 1.0).reshape(M, K)
bias = O.gen_normal(7, N, 0.1)
def cpu_compute(x2d, pk, sc, b, n, k, g):      # stand-in for the CUDA kernel: the test's own oracle
    y = O.linear_fp32(x2d.numpy(), pk.numpy(), sc.numpy().view(np.float16), n, k, None if b is None else b.numpy())
    return torch.from_numpy(y)
lin = sh.ColumnShardedLinear(torch.from_numpy(packed_np), torch.from_numpy(scales_np.view(np.int16)).view(torch.float16),
                             torch.from_numpy(bias), N, K, 32, rank, world, None, compute=cpu_compute)
y = lin(torch.from_numpy(x))
ref = O.linear_fp32(x, packed_np, scales_np, N, K, bias)
assert tuple(y.shape) == (M, N), y.shape
assert np.array_equal(y.numpy(), ref), "sharded result differs"
if len(set(lin.sizes)) != 1:                    # the fused exchange needs equal shards and says so before touching a GPU
    try:
        lin.enable_fused_gather(torch.device("cpu"))
    except ValueError:
        pass
    else:
        raise SystemExit("ragged shards were accepted by enable_fused_gather")
dist.barrier()
if rank == 0:
    print("SHARD_OK", lin.sizes)
dist.destroy_process_group()
'''


@pytest.mark.parametrize("n_rows", [64, 50])      # equal shards, and a ragged last shard
def test_column_sharding_two_gloo_ranks(tmp_path, n_rows):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, OJX_ROOT=ROOT, OJX_N=str(n_rows), MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29611 + n_rows % 7), str(script)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "SHARD_OK" in proc.stdout


def test_checkpoint_file_discovery_and_layout_rules(P, tmp_path):
    """Host-only parts of checkpoint ingestion (ojasx2/streaming_e8.py:90-109, 231-252): which shard files a
    directory yields, refusal of shards outside it, and the row-layout rules of the three formats."""
    import json
    se = importlib.import_module(P.__name__ + ".streaming_e8")
    with pytest.raises(FileNotFoundError):
        se._checkpoint_files(tmp_path)
    (tmp_path / "b.safetensors").write_bytes(b"x")
    (tmp_path / "a.safetensors").write_bytes(b"x")
    assert [f.name for f in se._checkpoint_files(tmp_path)] == ["a.safetensors", "b.safetensors"]
    (tmp_path / "model.safetensors").write_bytes(b"x")
    assert [f.name for f in se._checkpoint_files(tmp_path)] == ["model.safetensors"]
    index = tmp_path / "model.safetensors.index.json"
    index.write_text(json.dumps({"weight_map": {"w1": "b.safetensors", "w2": "a.safetensors", "w3": "b.safetensors"}}))
    assert [f.name for f in se._checkpoint_files(tmp_path)] == ["a.safetensors", "b.safetensors"]
    index.write_text(json.dumps({"weight_map": {"w": "missing.safetensors"}}))
    with pytest.raises(FileNotFoundError):
        se._checkpoint_files(tmp_path)
    index.write_text(json.dumps({"weight_map": {"w": "../escape.safetensors"}}))
    (tmp_path.parent / "escape.safetensors").write_bytes(b"x")
    with pytest.raises(ValueError, match="inside the checkpoint directory"):
        se._checkpoint_files(tmp_path)
    index.write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(ValueError, match="weight_map"):
        se._checkpoint_files(tmp_path)

    for bitrate in (1.0, 1.5, 2.0):
        se._validate_row_layout(64, 256, bitrate, 32)
        with pytest.raises(ValueError):
            se._validate_row_layout(64, 100, bitrate, 32)          # a row would not own whole groups
        with pytest.raises(ValueError):
            se._validate_row_layout(64, 256, bitrate, 8)           # row packing wants groups of 32 k
    with pytest.raises(ValueError):
        se._validate_row_layout(64, 256, 3.0, 32)
    assert se._bytes_per_row(4096, 1.0) == 512 and se._bytes_per_row(4096, 1.5) == 768 and se._bytes_per_row(4096, 2.0) == 1024
    ops = P.ops
    assert ops.packed_sizes_lowbit(2, 7, 13, 8) == (24, 12)            # 91 weights padded to 96
    assert ops.packed_sizes_lowbit(1, 7, 13, 12) == (12, 12)           # group 12 -> 8, as the reference's root packer
    with pytest.raises(ValueError):
        ops.packed_sizes_lowbit(2, 7, 13, 12)                          # the 2-bit packer raises instead
    assert se._matches_any("model.layers.0.mlp.up_proj", ("*.mlp.*",)) and not se._matches_any("lm_head", ("model.*",))
    with pytest.raises(ValueError, match="row_block"):
        P.load_hf_checkpoint_e8(str(tmp_path), row_block=0)
    with pytest.raises(NotADirectoryError):
        P.load_hf_checkpoint_e8(str(tmp_path / "nowhere"))


def test_adapter_epilogue_shape_rules(P):
    """Which decode shapes may carry the adapter term in the kernels' epilogue (host-side predicates only): the ternary
    kernels take 1-8 rows of 16-bit activations with K % 256 == 0 and groups of 32; the 2.0-bit / 1.0-bit kernels 1-8
    rows with groups of 32, K % 2048 == 0 and operands of x that fit shared memory; ranks 1-64."""
    import torch
    ops = P.ops
    assert ops.lora_fusable(1, 4096, 32, torch.bfloat16, 8) and ops.lora_fusable(8, 256, 32, torch.float16, 64)
    assert not ops.lora_fusable(9, 4096, 32, torch.bfloat16, 8)          # the 9-16 row kernels have no registers for it
    assert not ops.lora_fusable(1, 4096, 32, torch.float32, 8)           # fp32 activations do not reach those kernels
    assert not ops.lora_fusable(1, 4000, 32, torch.bfloat16, 8) and not ops.lora_fusable(1, 4096, 32, torch.bfloat16, 65)
    assert not ops.lora_fusable(1, 4096, 32, torch.bfloat16, 0)
    assert ops.lowbit_lora_fusable(1, 4096, 32, 8) and ops.lowbit_lora_fusable(8, 4096, 32, 64) and ops.lowbit_lora_fusable(4, 8192, 32, 1)
    assert not ops.lowbit_lora_fusable(8, 8192, 32, 8)                   # eight rows of 8192 activations do not fit shared memory
    assert not ops.lowbit_lora_fusable(1, 4096, 8, 8) and not ops.lowbit_lora_fusable(1, 4352, 32, 8)
    assert not ops.lowbit_lora_fusable(9, 2048, 32, 8) and not ops.lowbit_lora_fusable(0, 2048, 32, 8)
