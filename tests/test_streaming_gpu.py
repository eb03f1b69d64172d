"""GPU tests of the rotation kernel, the encoder's fused rotation and checkpoint ingestion: safetensors row
blocks -> pinned host slots -> encoder -> a layer's packed buffers, and a whole (tiny) Hugging Face
checkpoint loaded without a dense copy of any quantized weight."""

import numpy as np
import pytest

from conftest import have_cuda, load_pkg

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

DEV = "cuda:0"


@pytest.fixture(scope="module")
def P():
    if not have_cuda():
        pytest.skip("no CUDA device")
    pkg = load_pkg()
    pkg._cabi.lib()
    return pkg


def bits(t):
    """Raw bit pattern of a float tensor as a numpy integer array."""
    if t.dtype == torch.float32:
        return t.detach().cpu().view(torch.int32).numpy()
    return t.detach().cpu().view(torch.int16).numpy()


def special_inputs(dtype, seed):
    """Blocks that stress the per-stage roundings: mixed exponents, values near the type's limits, denormals,
    signed zeros, exact ties."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(64, 256, generator=g)
    x[0] *= 1e-3
    x[1] *= torch.logspace(-12, 2 if dtype == torch.float16 else 4, 256)
    x[2] = 0.0
    x[3, ::2] = -0.0
    x[4] = torch.randint(-3, 4, (256,), generator=g).float()                 # small integers: exact sums, ties
    x[5] = torch.randint(-3, 4, (256,), generator=g).float() * 2.0 ** -9     # half-ulp patterns for 8-bit significands
    x[6] = 1.0 + torch.randint(0, 2, (256,), generator=g).float() * 2.0 ** -8
    big = 6.0e4 if dtype == torch.float16 else 1.0e38
    x[7] = (torch.rand(256, generator=g) - 0.5) * big / 16                    # sums stay finite, magnitudes near the top
    tiny = 6.0e-8 if dtype == torch.float16 else 1.0e-40
    x[8] = torch.randint(-5, 6, (256,), generator=g).float() * tiny           # denormal range
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_rotation_kernel_equals_the_tensor_expression_bit_for_bit(P, dtype):
    """ops.fwht32 (one kernel, packed 16-bit arithmetic) against the tensor expression evaluated by torch on the
    host, which the golden vectors pin to the reference's fwht_block32 (ojasx2/math/lattice.py:91-102)."""
    x = special_inputs(dtype, 11)
    want = P.fwht_block32(x)                       # host tensors take the tensor expression
    got = P.ops.fwht32(x.to(DEV))
    assert got.dtype == dtype and got.shape == x.shape
    assert np.array_equal(bits(got), bits(want))
    again = P.fwht_block32(x.to(DEV))               # the public name routes CUDA tensors to the kernel
    assert np.array_equal(bits(again), bits(want))
    inplace = x.to(DEV).clone()
    P.ops.fwht32(inplace, out=inplace)
    assert np.array_equal(bits(inplace), bits(want))


def test_rotation_is_differentiable_and_self_adjoint(P):
    x = torch.randn(8, 64, device=DEV, requires_grad=True)
    g = torch.randn(8, 64, device=DEV)
    y = P.fwht_block32(x)
    y.backward(g)
    assert np.array_equal(bits(x.grad), bits(P.ops.fwht32(g)))
    twice = P.ops.fwht32(P.ops.fwht32(x.detach()))
    assert torch.allclose(twice, x.detach(), atol=1e-5)        # the normalised transform is an involution


def test_rotation_rejects_bad_shapes(P):
    with pytest.raises(ValueError):
        P.ops.fwht32(torch.zeros(4, 48, device=DEV))
    assert P.fwht_block32(torch.ones(4, 48, device=DEV)).equal(torch.ones(4, 48, device=DEV))   # unchanged, as the reference


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_encoder_with_fused_rotation_equals_rotate_then_encode(P, dtype):
    """OJX_ENCODE_HADAMARD: bytes and scales equal encode(fwht_block32(w)) - the reference's _pack_row_block
    with use_hadamard=True (ojasx2/streaming_e8.py:112-125) - for every input type."""
    w = special_inputs(dtype, 12)
    w = torch.cat([w, (torch.randn(192, 256, generator=torch.Generator().manual_seed(5)) * 0.02).to(dtype)])
    rotated_on_host = P.fwht_block32(w)
    want_p, want_s = P.ops.encode(rotated_on_host.to(DEV), 32)
    got_p, got_s = P.ops.encode(w.to(DEV), 32, hadamard=True)
    assert torch.equal(got_p, want_p)
    assert np.array_equal(bits(got_s), bits(want_s))
    # group 64: the rotation runs as its own kernel in front of the encoder
    want_p, want_s = P.ops.encode(rotated_on_host.to(DEV), 64)
    got_p, got_s = P.ops.encode(w.to(DEV), 64, hadamard=True)
    assert torch.equal(got_p, want_p) and np.array_equal(bits(got_s), bits(want_s))
    # a width that is not a multiple of 32 is left unrotated, as fwht_block32 leaves it
    odd = w[:, :48].contiguous().to(DEV)
    a, b = P.ops.encode(odd, 16, hadamard=True), P.ops.encode(odd, 16)
    assert torch.equal(a[0], b[0]) and np.array_equal(bits(a[1]), bits(b[1]))


def test_encode_ex_rejects_what_it_cannot_fuse(P):
    lib = P._cabi.lib()
    w = torch.zeros(4, 64, device=DEV)
    p = torch.zeros(4 * 64 * 3 // 16, dtype=torch.uint8, device=DEV)
    s = torch.zeros(4 * 64 // 16, dtype=torch.float16, device=DEV)
    args = (w.data_ptr(), 0, 4, 64)
    assert lib.ojx_e8t_encode_ex(*args, 64, 1, p.data_ptr(), s.data_ptr(), None) == -2      # group != 32
    assert lib.ojx_e8t_encode_ex(*args, 32, 2, p.data_ptr(), s.data_ptr(), None) == -9      # unknown flag
    w2 = torch.zeros(4, 48, device=DEV)
    assert lib.ojx_e8t_encode_ex(w2.data_ptr(), 0, 4, 48, 32, 1, p.data_ptr(), s.data_ptr(), None) == -2


@pytest.mark.parametrize("dtype,rows,row_block,had", [(torch.bfloat16, 96, 32, False), (torch.float16, 70, 32, True),
                                                      (torch.float32, 33, 7, True), (torch.bfloat16, 5, 64, False)])
def test_safetensors_rows_stream_into_a_layer(P, tmp_path, dtype, rows, row_block, had):
    """_stream_safetensor_weight (ojasx2/streaming_e8.py:196-216): every row-block size, a ragged last block and
    a block larger than the matrix give the bytes of packing the matrix whole; the return value is the size of
    the largest source block."""
    st = pytest.importorskip("safetensors.torch")
    from safetensors import safe_open
    k = 256
    w = (torch.randn(rows, k, generator=torch.Generator().manual_seed(rows)) * 0.05).to(dtype)
    path = tmp_path / "w.safetensors"
    st.save_file({"proj.weight": w, "other": torch.zeros(3)}, str(path))
    layer = P.E8LatticeLinear(k, rows, bias=False, group_size=32, bitrate=1.5, use_hadamard=had, device=torch.device(DEV))
    with safe_open(str(path), framework="pt", device="cpu") as handle:
        largest = P._stream_safetensor_weight(handle, "proj.weight", layer, row_block, had)
        assert largest == min(row_block, rows) * k * w.element_size()
        want_p, want_s = P.ops.encode(w.to(DEV), 32, hadamard=had)
        torch.cuda.synchronize()
        assert torch.equal(layer.packed_weight, want_p)
        assert np.array_equal(bits(layer.block_scales), bits(want_s))
        wrong = P.E8LatticeLinear(k, rows + 1, bias=False, group_size=32, bitrate=1.5, device=torch.device(DEV))
        with pytest.raises(ValueError, match="has shape"):
            P._stream_safetensor_weight(handle, "proj.weight", wrong, row_block, had)


def _tiny_llama(transformers, tie):
    return transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                    tie_word_embeddings=tie)


def test_sharded_checkpoint_loads_packed_and_trains_adapters(P, tmp_path):
    """load_hf_checkpoint_e8 (ojasx2/streaming_e8.py:255-558) on a sharded checkpoint: every linear arrives
    packed exactly as E8LatticeLinear.from_linear packs the dense module, nothing is left on the meta device,
    only the adapters train, and a forward/backward pass through the packed model is finite."""
    transformers = pytest.importorskip("transformers")
    pytest.importorskip("safetensors")
    torch.manual_seed(411)
    source = transformers.LlamaForCausalLM(_tiny_llama(transformers, tie=False))
    source.save_pretrained(tmp_path, safe_serialization=True, max_shard_size="20KB")
    assert (tmp_path / "model.safetensors.index.json").is_file()

    model, report = P.load_hf_checkpoint_e8(str(tmp_path), bitrate=1.5, group_size=32, lora_rank=2, row_block=3,
                                            use_hadamard=True)
    assert len(report.checkpoint_files) > 1
    assert report.quantized_linear_layers == 15                      # 2 x (q, k, v, o, gate, up, down) + lm_head
    dense = dict(source.named_modules())
    packed_layers = {n: m for n, m in model.named_modules() if isinstance(m, P.E8LatticeLinear)}
    assert len(packed_layers) == 15
    assert report.quantized_source_parameters == sum(dense[n].weight.numel() for n in packed_layers)
    assert report.max_source_row_block_bytes <= 3 * 128 * 4
    assert report.estimated_persistent_tensor_bytes == (report.parameter_bytes + report.packed_weight_bytes
                                                        + report.packed_scale_bytes + report.other_buffer_bytes)
    assert not [n for n, p in model.named_parameters() if p.is_meta]
    assert not [n for n, b in model.named_buffers() if b.is_meta]
    assert all(p.is_cuda for p in model.parameters()) and all(b.is_cuda for b in model.buffers())
    for name, layer in packed_layers.items():
        want = P.E8LatticeLinear.from_linear(dense[name].to(DEV), rank=2, bitrate=1.5, group_size=32, use_hadamard=True)
        assert torch.equal(layer.packed_weight, want.packed_weight), name
        assert np.array_equal(bits(layer.block_scales), bits(want.block_scales)), name
    assert torch.equal(model.model.embed_tokens.weight.cpu(), source.model.embed_tokens.weight.detach())

    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all(n.endswith(("lora_A", "lora_B")) for n in trainable)
    assert report.trainable_parameters == sum(p.numel() for p in model.parameters() if p.requires_grad)
    ids = torch.tensor([[1, 2, 3, 4]], device=DEV)
    out = model(input_ids=ids, labels=ids)
    assert torch.isfinite(out.loss) and out.logits.shape == (1, 4, 128)
    out.loss.backward()
    grads = dict(model.named_parameters())
    assert all(grads[n].grad is not None and torch.isfinite(grads[n].grad).all() for n in trainable)
    assert report.to_dict()["row_block"] == 3 and model.ojasx_streaming_report is report


def test_loader_refuses_tied_head_and_partial_checkpoints(P, tmp_path):
    transformers = pytest.importorskip("transformers")
    st = pytest.importorskip("safetensors.torch")
    tied_dir, partial_dir = tmp_path / "tied", tmp_path / "partial"
    tied = transformers.LlamaForCausalLM(_tiny_llama(transformers, tie=True))
    tied.save_pretrained(tied_dir, safe_serialization=True)
    with pytest.raises(ValueError, match="shares its weight"):
        P.load_hf_checkpoint_e8(str(tied_dir))
    model, report = P.load_hf_checkpoint_e8(str(tied_dir), exclude_modules=("lm_head",), lora_rank=0)
    assert report.quantized_linear_layers == 14 and report.trainable_parameters == 0
    assert model.lm_head.weight is model.model.embed_tokens.weight          # the tie survives shard-wise assignment

    full = transformers.LlamaForCausalLM(_tiny_llama(transformers, tie=False))
    full.save_pretrained(partial_dir, safe_serialization=True)
    # copies: load_file maps the file, and the file is rewritten below
    state = {k: v.clone() for k, v in st.load_file(str(partial_dir / "model.safetensors")).items()}
    state.pop("model.norm.weight")
    st.save_file(state, str(partial_dir / "model.safetensors"), metadata={"format": "pt"})
    with pytest.raises(ValueError, match="missing required dense"):
        P.load_hf_checkpoint_e8(str(partial_dir))
    state.pop("model.layers.0.mlp.up_proj.weight")
    st.save_file(state, str(partial_dir / "model.safetensors"), metadata={"format": "pt"})
    with pytest.raises(ValueError, match="required by converted E8 layers"):
        P.load_hf_checkpoint_e8(str(partial_dir))
    state["surprise"] = torch.zeros(2)
    st.save_file(state, str(partial_dir / "model.safetensors"), metadata={"format": "pt"})
    with pytest.raises(ValueError, match="Unexpected checkpoint tensor"):
        P.load_hf_checkpoint_e8(str(partial_dir))
    with pytest.raises(ValueError, match="row_block"):
        P.load_hf_checkpoint_e8(str(partial_dir), row_block=0)
    with pytest.raises(NotADirectoryError):
        P.load_hf_checkpoint_e8(str(tmp_path / "absent"))
