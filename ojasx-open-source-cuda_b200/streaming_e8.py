"""Row-block packing and checkpoint ingestion (mirror of the reference's ``ojasx2/streaming_e8.py``).

Because every row owns whole scale groups when ``in_features % group_size == 0``, packing a matrix
row block by row block yields exactly the bytes of packing it whole; the GPU encoder therefore
writes each block straight into its final byte range instead of concatenating pieces, and the
optional Hadamard rotation happens in the encoder's registers.

Checkpoint ingestion keeps the reference's contract - a dense weight never exists as a whole, only
``row_block`` rows of it at a time - and adds what a GPU target needs: row blocks travel through two
pinned host slots and one side stream, so reading block ``i + 1`` from the file overlaps the
host-to-device copy and the encoding of block ``i``.
"""

from __future__ import annotations

import contextlib
import dataclasses
import fnmatch
import json
import pathlib
from typing import Dict, Iterable, List, Optional, Sequence, Set, Tuple

import torch
from torch import nn

from . import ops
from .lattice import E8LatticeLinear, _check_bitrate


def _validate_row_layout(out_features: int, in_features: int, bitrate: float, group_size: int) -> None:
    """Same rejections as the reference (``streaming_e8.py:90-109``)."""
    if float(bitrate) not in (1.0, 1.5, 2.0):
        raise ValueError(f"Unsupported E8 bitrate {bitrate!r}; expected one of [1.0, 1.5, 2.0]")
    if out_features <= 0 or in_features <= 0:
        raise ValueError("Streaming E8 requires non-empty two-dimensional weights")
    if group_size <= 0 or group_size % 32 != 0:
        raise ValueError("The current E8 packers require group_size to be a positive multiple of 32")
    if in_features % group_size != 0:
        raise ValueError(
            f"in_features={in_features} is not divisible by group_size={group_size}. "
            "Row-block packing would cross a scale-group boundary and change the packed layout.")
    _check_bitrate(bitrate)


def _encoder_for(bitrate: float):
    _check_bitrate(bitrate)
    return {1.0: ops.encode_1bit, 1.5: ops.encode, 2.0: ops.encode_2bit}[float(bitrate)]


def _bytes_per_row(in_features: int, bitrate: float) -> int:
    return {1.0: in_features // 8, 1.5: in_features * 3 // 16, 2.0: in_features // 4}[float(bitrate)]


def _pack_row_block(block: torch.Tensor, bitrate: float, group_size: int, use_hadamard: bool
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    return _encoder_for(bitrate)(block, group_size, hadamard=use_hadamard)


def pack_weight_rowwise(weight: torch.Tensor, *, bitrate: float = 1.5, group_size: int = 32, row_block: int = 32,
                        use_hadamard: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packs ``weight`` ``row_block`` rows at a time; the result equals whole-matrix packing byte for byte."""
    if weight.ndim != 2:
        raise ValueError(f"Expected a rank-2 weight, got shape {tuple(weight.shape)}")
    if row_block <= 0:
        raise ValueError("row_block must be positive")
    out_features, in_features = map(int, weight.shape)
    _validate_row_layout(out_features, in_features, bitrate, group_size)
    encode = _encoder_for(bitrate)
    bytes_per_row, scales_per_row = _bytes_per_row(in_features, bitrate), in_features // group_size
    packed = torch.empty(out_features * bytes_per_row, dtype=torch.uint8, device=weight.device)
    scales = torch.empty(out_features * scales_per_row, dtype=torch.float16, device=weight.device)
    for start in range(0, out_features, row_block):
        stop = min(start + row_block, out_features)
        encode(weight[start:stop], group_size, hadamard=use_hadamard,
                   out=(packed[start * bytes_per_row: stop * bytes_per_row],
                        scales[start * scales_per_row: stop * scales_per_row]))
    return packed, scales


def _destination_ranges(layer: E8LatticeLinear, row_start: int, block: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Checks ``block`` against the layer and returns the slices of its packed buffers that rows
    ``row_start ..`` occupy (the checks and messages of the reference's ``streaming_e8.py:168-189``)."""
    if block.ndim != 2 or block.shape[1] != layer.in_features:
        raise ValueError(f"Unexpected row block shape {tuple(block.shape)} for "
                         f"{layer.out_features}x{layer.in_features} E8 layer")
    if not block.dtype.is_floating_point:
        raise TypeError(f"E8 packing requires floating-point source weights, got {block.dtype}")
    rows = int(block.shape[0])
    bytes_per_row = _bytes_per_row(layer.in_features, layer.bitrate)
    scales_per_row = layer.in_features // layer.group_size
    p0, s0 = row_start * bytes_per_row, row_start * scales_per_row
    if p0 + rows * bytes_per_row > layer.packed_weight.numel():
        raise RuntimeError("Packed destination is smaller than the streamed source layout")
    if s0 + rows * scales_per_row > layer.block_scales.numel():
        raise RuntimeError("Scale destination is smaller than the streamed source layout")
    return layer.packed_weight[p0: p0 + rows * bytes_per_row], layer.block_scales[s0: s0 + rows * scales_per_row]


def _copy_row_block_into_layer(layer: E8LatticeLinear, row_start: int, block: torch.Tensor, use_hadamard: bool) -> int:
    """Encodes ``block`` (rows ``row_start ..``) directly into the layer's packed buffers
    (reference ``streaming_e8.py:162-193``).  Returns the number of source bytes consumed."""
    out = _destination_ranges(layer, row_start, block)
    source = block.to(layer.packed_weight.device)
    with torch.no_grad():
        _encoder_for(layer.bitrate)(source, layer.group_size, out=out, hadamard=use_hadamard)
    return int(block.numel() * block.element_size())


class _RowBlockPipe:
    """Two pinned host slots feeding one side stream: host -> device copy and encoding of a block are
    queued on the side stream while the caller fills the other slot with the next block."""

    def __init__(self, device: torch.device, slot_bytes: int) -> None:
        self.device = device
        self.stream = torch.cuda.Stream(device=device)
        self.stream.wait_stream(torch.cuda.current_stream(device))
        self.slots = [torch.empty(slot_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self.copied = [None, None]          # event: the slot's bytes have left host memory
        self.turn = 0

    def push(self, layer: E8LatticeLinear, row_start: int, block: torch.Tensor, use_hadamard: bool) -> None:
        out = _destination_ranges(layer, row_start, block)
        i = self.turn
        self.turn ^= 1
        if self.copied[i] is not None:
            self.copied[i].synchronize()
        nbytes = block.numel() * block.element_size()
        host = self.slots[i][:nbytes].view(block.dtype).view(block.shape)
        host.copy_(block)
        with torch.cuda.stream(self.stream), torch.no_grad():
            staged = host.to(self.device, non_blocking=True)
            self.copied[i] = torch.cuda.Event()
            self.copied[i].record(self.stream)
            _encoder_for(layer.bitrate)(staged, layer.group_size, out=out, hadamard=use_hadamard)

    def finish(self) -> None:
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        for ev in self.copied:
            if ev is not None:
                ev.synchronize()


def _stream_safetensor_weight(handle: object, key: str, layer: E8LatticeLinear, row_block: int, use_hadamard: bool) -> int:
    """Packs checkpoint tensor ``key`` into ``layer`` ``row_block`` rows at a time (reference
    ``streaming_e8.py:196-216``): only one row block of the dense weight exists on the host, and two on the
    device, at any moment.  Returns the size in bytes of the largest source block."""
    source = handle.get_slice(key)
    shape = tuple(int(v) for v in source.get_shape())
    expected = (int(layer.out_features), int(layer.in_features))
    if shape != expected:
        raise ValueError(f"Checkpoint tensor {key!r} has shape {shape}, expected {expected}")
    pipe: Optional[_RowBlockPipe] = None
    largest = 0
    for start in range(0, expected[0], row_block):
        block = source[start: min(start + row_block, expected[0])]
        nbytes = int(block.numel() * block.element_size())
        if pipe is None:
            pipe = _RowBlockPipe(layer.packed_weight.device, max(nbytes, 16))
        pipe.push(layer, start, block, use_hadamard)
        largest = max(largest, nbytes)
        del block
    if pipe is not None:
        pipe.finish()
    return largest


@dataclasses.dataclass(frozen=True)
class StreamingE8LoadReport:
    """What a finished checkpoint load left resident (same fields as the reference's report,
    ``streaming_e8.py:45-76``).  Counts persistent tensors only."""

    checkpoint_dir: str
    architectures: Tuple[str, ...]
    bitrate: float
    group_size: int
    lora_rank: int
    row_block: int
    checkpoint_files: Tuple[str, ...]
    quantized_linear_layers: int
    quantized_source_parameters: int
    packed_weight_bytes: int
    packed_scale_bytes: int
    parameter_bytes: int
    other_buffer_bytes: int
    estimated_persistent_tensor_bytes: int
    trainable_parameters: int
    trainable_parameter_bytes: int
    dense_source_parameters: int
    max_source_row_block_bytes: int
    ignored_checkpoint_keys: Tuple[str, ...]
    memory_scope: str = ("persistent tensors only; excludes process memory, allocator overhead, activations, "
                         "autograd state, gradients, optimizer state and workspaces")

    def to_dict(self) -> Dict[str, object]:
        return dataclasses.asdict(self)


def _matches_any(name: str, patterns: Sequence[str]) -> bool:
    return any(fnmatch.fnmatchcase(name, p) for p in patterns)


def _checkpoint_files(checkpoint_dir: pathlib.Path) -> Tuple[pathlib.Path, ...]:
    """Shard files of a local checkpoint: those the index names, else ``model.safetensors``, else every
    ``*.safetensors`` (reference ``streaming_e8.py:231-252``); shards must lie inside the directory."""
    index = checkpoint_dir / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text(encoding="utf-8")).get("weight_map")
        if not isinstance(weight_map, dict) or not weight_map:
            raise ValueError(f"Invalid or empty weight_map in {index}")
        files = tuple(checkpoint_dir / n for n in sorted({str(v) for v in weight_map.values()}))
    elif (checkpoint_dir / "model.safetensors").is_file():
        files = (checkpoint_dir / "model.safetensors",)
    else:
        files = tuple(sorted(checkpoint_dir.glob("*.safetensors")))
    if not files:
        raise FileNotFoundError(f"No safetensors checkpoint found under {checkpoint_dir}")
    for f in files:
        if not f.is_file():
            raise FileNotFoundError(f"Checkpoint index references missing file: {f}")
        if f.resolve().parent != checkpoint_dir.resolve():
            raise ValueError("Checkpoint shard paths must remain inside the checkpoint directory")
    return files


@contextlib.contextmanager
def _parameters_on_meta():
    """While active, every parameter a module registers is replaced by a meta-device parameter, so building
    a large model allocates nothing for its weights; buffers are created normally."""
    original = nn.Module.register_parameter

    def register(module, name, param):
        if param is not None and not param.is_meta:
            param = nn.Parameter(torch.empty_like(param, device="meta"), requires_grad=param.requires_grad)
        original(module, name, param)

    nn.Module.register_parameter = register
    try:
        yield
    finally:
        nn.Module.register_parameter = original


def _resolve(model: nn.Module, dotted: str) -> Tuple[nn.Module, str]:
    parent = model
    parts = dotted.split(".")
    for part in parts[:-1]:
        parent = getattr(parent, part)
    return parent, parts[-1]


def load_hf_checkpoint_e8(checkpoint_dir: str, *, bitrate: float = 1.5, group_size: int = 32, lora_rank: int = 8,
                          lora_alpha: float = 16.0, row_block: int = 32, use_hadamard: bool = False,
                          adapter_dtype: torch.dtype = torch.float32, exclude_modules: Iterable[str] = (),
                          allow_unexpected_keys: bool = False, device: Optional[torch.device] = None
                          ) -> Tuple[nn.Module, StreamingE8LoadReport]:
    """Builds a Hugging Face causal LM from a local safetensors checkpoint with every selected ``nn.Linear``
    replaced by a packed :class:`E8LatticeLinear` on ``device`` (default: the current CUDA device), never holding
    a dense copy of a quantized weight (reference ``streaming_e8.py:255-558``: same arguments, checks, freezing
    policy and report).  Differences: the result lives on the GPU; weights are created on the meta device by a
    local context manager, so the ``accelerate`` package is not needed.

    Selected linears whose weight is shared with another module are refused (exclude a tied ``lm_head``);
    missing, duplicate or unexpected checkpoint tensors are errors unless ``allow_unexpected_keys``.
    Only the LoRA factors of the packed layers are left trainable.
    """
    if row_block <= 0:
        raise ValueError("row_block must be positive")
    if lora_rank < 0:
        raise ValueError("lora_rank must be non-negative")
    if float(bitrate) not in (1.0, 1.5, 2.0):
        raise ValueError(f"Unsupported E8 bitrate {bitrate!r}; expected one of [1.0, 1.5, 2.0]")
    if group_size <= 0 or group_size % 32 != 0:
        raise ValueError("group_size must be a positive multiple of 32")
    _check_bitrate(bitrate)
    root = pathlib.Path(checkpoint_dir).expanduser().resolve()
    if not root.is_dir():
        raise NotADirectoryError(f"Local checkpoint directory does not exist: {root}")
    try:
        from safetensors import safe_open
        from transformers import AutoConfig, AutoModelForCausalLM
    except ImportError as exc:
        raise ImportError("Checkpoint ingestion needs the transformers and safetensors packages") from exc
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)

    files = _checkpoint_files(root)
    config = AutoConfig.from_pretrained(str(root), local_files_only=True, trust_remote_code=False)
    with _parameters_on_meta():
        model = AutoModelForCausalLM.from_config(config, trust_remote_code=False)
    model.tie_weights()

    patterns = tuple(exclude_modules)
    selected = {name for name, mod in model.named_modules()
                if isinstance(mod, nn.Linear) and not _matches_any(name, patterns)}
    owners: Dict[int, List[str]] = {}
    for name, param in model.named_parameters(remove_duplicate=False):
        owners.setdefault(id(param), []).append(name)
    shared_groups = [names for names in owners.values() if len(names) > 1]
    for names in shared_groups:
        if any(n.endswith(".weight") and n[:-len(".weight")] in selected for n in names):
            raise ValueError("A selected E8 linear shares its weight with another module: " + ", ".join(names)
                             + ". Independent packing would break weight tying. Exclude the tied head/module "
                             "explicitly, or add a separately validated tying policy.")

    weight_to_layer: Dict[str, E8LatticeLinear] = {}
    bias_to_layer: Dict[str, E8LatticeLinear] = {}
    quantized_source_parameters = 0
    for name in sorted(selected):
        parent, leaf = _resolve(model, name)
        linear = getattr(parent, leaf)
        _validate_row_layout(int(linear.out_features), int(linear.in_features), float(bitrate), int(group_size))
        layer = E8LatticeLinear(int(linear.in_features), int(linear.out_features), bias=linear.bias is not None,
                                rank=int(lora_rank), lora_alpha=float(lora_alpha), bitrate=float(bitrate),
                                group_size=int(group_size), use_hadamard=bool(use_hadamard), device=dev,
                                dtype=adapter_dtype)
        setattr(parent, leaf, layer)
        weight_to_layer[f"{name}.weight"] = layer
        if layer.bias is not None:
            layer.bias.requires_grad_(False)
            bias_to_layer[f"{name}.bias"] = layer
        quantized_source_parameters += int(linear.in_features) * int(linear.out_features)
    if not weight_to_layer:
        raise ValueError("No eligible nn.Linear modules were selected for E8 conversion")

    state_keys = set(model.state_dict())
    packed_state_keys = {f"{k[:-len('.weight')]}.{suffix}" for k in weight_to_layer
                         for suffix in ("packed_weight", "block_scales", "lora_A", "lora_B")}
    shared_keys = {n for names in shared_groups for n in names}
    need_dense = state_keys - packed_state_keys - shared_keys - set(bias_to_layer)
    need_packed = set(weight_to_layer) | set(bias_to_layer)
    seen: Set[str] = set()
    ignored: List[str] = []
    largest_block = 0
    dense_source_parameters = 0

    for file in files:
        dense: Dict[str, torch.Tensor] = {}
        with safe_open(str(file), framework="pt", device="cpu") as handle:
            for key in handle.keys():
                if key in seen:
                    raise ValueError(f"Duplicate checkpoint tensor across shards: {key}")
                seen.add(key)
                if key in weight_to_layer:
                    largest_block = max(largest_block, _stream_safetensor_weight(
                        handle, key, weight_to_layer[key], int(row_block), bool(use_hadamard)))
                elif key in bias_to_layer:
                    layer = bias_to_layer[key]
                    value = handle.get_tensor(key)
                    if tuple(value.shape) != (int(layer.out_features),):
                        raise ValueError(f"Unexpected bias shape for {key}: {tuple(value.shape)}")
                    with torch.no_grad():
                        layer.bias.copy_(value)
                    dense_source_parameters += int(value.numel())
                elif key in state_keys:
                    dense[key] = handle.get_tensor(key).to(dev)
                    dense_source_parameters += int(dense[key].numel())
                elif allow_unexpected_keys:
                    ignored.append(key)
                else:
                    raise ValueError(f"Unexpected checkpoint tensor {key!r} in {file.name}; "
                                     "refusing a silent partial load")
        if dense:
            model.load_state_dict(dense, strict=False, assign=True)

    missing = sorted(need_packed - seen)
    if missing:
        raise ValueError("Checkpoint is missing tensors required by converted E8 layers: " + ", ".join(missing[:20]))
    missing = sorted(need_dense - seen)
    if missing:
        raise ValueError("Checkpoint is missing required dense parameters or persistent buffers: "
                         + ", ".join(missing[:20]))
    for names in shared_groups:
        if not any(n in seen for n in names):
            raise ValueError("Checkpoint contains no stored tensor for shared parameter group: " + ", ".join(names))
        members = []
        for n in names:
            parent, leaf = _resolve(model, n)
            members.append(getattr(parent, leaf))
        real = next((p for p in members if not p.is_meta), None)
        if real is not None:                               # safetensors stores one member of a tied group
            for n in names:
                parent, leaf = _resolve(model, n)
                setattr(parent, leaf, real)

    leftovers = [n for n, p in model.named_parameters() if p.is_meta] + [n for n, b in model.named_buffers() if b.is_meta]
    if leftovers:
        raise ValueError("Checkpoint load left uninitialized meta tensors: " + ", ".join(leftovers[:30]))
    model.to(dev)                                          # buffers the architecture built on the host

    for param in model.parameters():
        param.requires_grad_(False)
    for layer in weight_to_layer.values():
        if layer.lora_A is not None and layer.lora_A.numel():
            layer.lora_A.requires_grad_(True)
            layer.lora_B.requires_grad_(True)

    def nbytes(t: torch.Tensor) -> int:
        return int(t.numel() * t.element_size())

    params = list(model.parameters())
    packed_ids = {id(b) for layer in weight_to_layer.values() for b in (layer.packed_weight, layer.block_scales)}
    parameter_bytes = sum(nbytes(p) for p in params)
    packed_weight_bytes = sum(nbytes(layer.packed_weight) for layer in weight_to_layer.values())
    packed_scale_bytes = sum(nbytes(layer.block_scales) for layer in weight_to_layer.values())
    other_buffer_bytes = sum(nbytes(b) for b in model.buffers() if id(b) not in packed_ids)
    report = StreamingE8LoadReport(
        checkpoint_dir=str(root),
        architectures=tuple(getattr(config, "architectures", ()) or (type(model).__name__,)),
        bitrate=float(bitrate), group_size=int(group_size), lora_rank=int(lora_rank), row_block=int(row_block),
        checkpoint_files=tuple(f.name for f in files),
        quantized_linear_layers=len(weight_to_layer),
        quantized_source_parameters=quantized_source_parameters,
        packed_weight_bytes=packed_weight_bytes, packed_scale_bytes=packed_scale_bytes,
        parameter_bytes=parameter_bytes, other_buffer_bytes=other_buffer_bytes,
        estimated_persistent_tensor_bytes=parameter_bytes + packed_weight_bytes + packed_scale_bytes + other_buffer_bytes,
        trainable_parameters=sum(int(p.numel()) for p in params if p.requires_grad),
        trainable_parameter_bytes=sum(nbytes(p) for p in params if p.requires_grad),
        dense_source_parameters=dense_source_parameters,
        max_source_row_block_bytes=largest_block,
        ignored_checkpoint_keys=tuple(sorted(ignored)),
    )
    model.ojasx_streaming_report = report
    return model, report
