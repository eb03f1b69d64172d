"""Output-column sharding of a packed linear across the GPUs of one node.

Rows of W (output features) are independent, and when ``K % 32 == 0`` rank r's shard is a
contiguous byte range of the packed buffers - no repacking.  Each rank computes
``y[:, n0:n1]`` with the fused kernels; an NCCL all-gather over NVLink assembles the full output.
The reference has no multi-GPU form of this path (its only distributed code is a TCP pipeline,
``ojasx2/mesh_hal.py``), so this module has no counterpart there.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch


def shard_rows(n_rows: int, world_size: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """Contiguous row range ``[n0, n1)`` of ``rank``.  Ranges are multiples of ``multiple`` rows (the
    kernels' row tile) except possibly the last; all rows are covered exactly once."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    blocks = (n_rows + multiple - 1) // multiple
    b0 = blocks * rank // world_size
    b1 = blocks * (rank + 1) // world_size
    return min(b0 * multiple, n_rows), min(b1 * multiple, n_rows)


def shard_sizes(n_rows: int, world_size: int, multiple: int = 16) -> List[int]:
    return [b - a for a, b in (shard_rows(n_rows, world_size, r, multiple) for r in range(world_size))]


def slice_packed(packed: torch.Tensor, scales: torch.Tensor, in_features: int, n0: int, n1: int,
                 group_size: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Views of rows ``[n0, n1)`` of packed codes and scales (requires whole groups per row)."""
    if in_features % group_size != 0:
        raise ValueError("row slicing needs in_features % group_size == 0")
    bpr, spr = in_features * 3 // 16, in_features // group_size
    return packed[n0 * bpr: n1 * bpr], scales[n0 * spr: n1 * spr]


class ColumnShardedLinear:
    """One rank's shard of a packed linear plus the all-gather that follows it.

    ``forward(x)`` returns the full ``[M, N]`` output on every rank.  With ``world_size == 1`` no
    collective is issued.  ``compute`` is injectable so the sharding logic can be exercised on CPU
    ranks (gloo) with a stand-in for the CUDA kernel.
    """

    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor], out_features: int,
                 in_features: int, group_size: int = 32, rank: int = 0, world_size: int = 1, group=None,
                 compute=None):
        self.N, self.K, self.g = int(out_features), int(in_features), int(group_size)
        self.rank, self.world, self.group = rank, world_size, group
        self.n0, self.n1 = shard_rows(self.N, world_size, rank)
        self.sizes = shard_sizes(self.N, world_size)
        self.packed, self.scales = slice_packed(packed, scales, self.K, self.n0, self.n1, self.g)
        self.bias = bias[self.n0:self.n1] if bias is not None else None
        if compute is None:
            from . import ops
            compute = ops.linear
        self._compute = compute

    def forward_local(self, x2d: torch.Tensor) -> torch.Tensor:
        if self.n1 == self.n0:
            return x2d.new_empty((x2d.shape[0], 0))
        return self._compute(x2d, self.packed, self.scales, self.bias, self.n1 - self.n0, self.K, self.g)

    def forward(self, x2d: torch.Tensor) -> torch.Tensor:
        y_local = self.forward_local(x2d)
        if self.world == 1:
            return y_local
        import torch.distributed as dist
        m = x2d.shape[0]
        widest = max(self.sizes)
        if y_local.shape[1] != widest:
            # ragged last shards are padded so that one fixed-size collective serves every rank
            pad = y_local.new_zeros((m, widest))
            pad[:, : y_local.shape[1]] = y_local
            y_local = pad
        flat = y_local.new_empty((self.world * m, widest))
        dist.all_gather_into_tensor(flat, y_local.contiguous(), group=self.group)
        buf = flat.view(self.world, m, widest)
        if len(set(self.sizes)) == 1:
            return buf.permute(1, 0, 2).reshape(m, self.N)
        return torch.cat([buf[r, :, : s] for r, s in enumerate(self.sizes)], dim=1)

    __call__ = forward

    # ---- fused form: the decode kernel stores this rank's columns into every rank's output window ----
    def enable_fused_gather(self, device: torch.device, x_dtype: torch.dtype = torch.bfloat16,
                            y_dtype: torch.dtype = torch.bfloat16, max_rows: int = 16) -> None:
        """Collective.  Builds two alternating peer-mapped output windows ``[world, max_rows, N / world]`` (a window
        is rewritten only two calls later, after every rank has passed the fence of the call in between) for
        ``forward_fused``.  Needs equal shards, K % 256 == 0 and group 32."""
        if len(set(self.sizes)) != 1 or self.K % 256 != 0 or self.g != 32:
            raise ValueError("fused gather needs equal column shards, K % 256 == 0 and group_size 32")
        self._fg = {"dev": device, "xd": x_dtype, "yd": y_dtype, "rows": int(max_rows), "calls": 0, "groups": {},
                    "windows": [PeerWindow(self.world * max_rows * self.sizes[0], y_dtype, device, self.group) for _ in range(2)]}

    def forward_fused(self, x2d: torch.Tensor) -> torch.Tensor:
        """``[M, N]`` on every rank for M <= max_rows: one kernel launch that writes all ranks' windows, one fence.
        The result is a view of this rank's window: use it before the call after next."""
        from . import ops
        fg, m, nl = self._fg, int(x2d.shape[0]), self.sizes[0]
        if not (1 <= m <= fg["rows"]) or x2d.dtype != fg["xd"]:
            raise ValueError("forward_fused: row count or dtype outside what enable_fused_gather set up")
        which = fg["calls"] % 2
        fg["calls"] += 1
        key = (m, which)
        if key not in fg["groups"]:
            window = fg["windows"][which]
            x_stage = torch.empty((m, self.K), dtype=fg["xd"], device=fg["dev"])
            slot = window.local.view(self.world, fg["rows"], nl)[self.rank, :m]
            fg["groups"][key] = (x_stage, ops.GroupedGemv([(x_stage, self.packed, self.scales, self.bias, slot)],
                                                          [(nl, self.K)], peer_delta=window.delta))
        x_stage, group = fg["groups"][key]
        x_stage.copy_(x2d)
        group()
        window = fg["windows"][which]
        window.fence()
        return window.local.view(self.world, fg["rows"], nl)[:, :m].permute(1, 0, 2).reshape(m, self.N)


class PeerWindow:
    """One buffer of the same size on every rank of a single-node process group, each rank holding a mapping of
    every other rank's copy (CUDA IPC), for kernels that store their shard of a result into all ranks' buffers
    themselves - the fused form of "compute a column shard, then all-gather"
    (see ``GroupedGemv(..., peer_delta=window.delta)``).

    ``local`` is this rank's buffer, laid out by the caller (for example ``[world, ...]`` with slot r belonging
    to rank r, or full ``[M, N]`` matrices of which every rank fills its column block);
    ``delta[r]`` is the byte distance from ``local`` to rank r's copy as mapped here (0 for this rank).
    Between the kernels that write a window and anyone reading it the ranks must either meet (``fence()``), or
    the launches order themselves on the device through the window's ``sync_ptr`` block
    (``GroupedGemv(..., peer_sync=window.sync_ptr, wait_peers=..., signal_peers=...)``).
    Construction is collective; it raises if the device memory cannot be shared between the ranks.
    """

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed as dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        from . import _cabi
        my_index = device.index if device.index is not None else torch.cuda.current_device()
        # the payload, then (256-byte aligned) the ojx_e8t_peer_sync block, in ONE allocation: one mapping serves both
        itemsize = torch.empty(0, dtype=dtype).element_size()
        payload = (numel * itemsize + 255) // 256 * 256
        self._raw = torch.zeros(payload + 256, dtype=torch.uint8, device=device)
        self.local = self._raw[: numel * itemsize].view(dtype)
        self.sync_ptr = int(self._raw.data_ptr()) + payload
        self._sync_words = self._raw[payload: payload + _cabi.PEER_SYNC_BYTES].view(torch.int32)
        handle = self._raw.untyped_storage()._share_cuda_()
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self._peer_storages = []
        self.delta = []
        with torch.cuda.device(device):
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.delta.append(0)
                    continue
                # Kernels of THIS device will store into the peer's memory: peer access must be on in that direction,
                # and the handle is opened with this device current (h[0] is the exporter's device index).
                _cabi.check(_cabi.lib().ojx_e8t_enable_peer_access(int(h[0])), "ojx_e8t_enable_peer_access")
                storage = torch.UntypedStorage._new_shared_cuda(my_index, *h[1:])
                self._peer_storages.append(storage)             # keeps the mapping alive
                self.delta.append(int(storage.data_ptr()) - int(self.local.data_ptr()))
        self._token = torch.zeros(1, dtype=torch.int32, device=device)

    def close(self) -> None:
        """Drops this rank's mappings of the peers' buffers.  Collective by convention: every rank closes before any
        rank frees its own buffer or exits."""
        self._peer_storages.clear()
        self.delta = [0] * len(self.delta)

    def sync_status(self) -> int:
        """Status word of the device-side ordering block: 0, or the (negative) code of a wait that gave up.
        Synchronises the current stream."""
        return int(self._sync_words[2].item())

    def set_spin_limit(self, polls: int) -> None:
        """Polls per awaited rank before a device-side wait gives up (0: the library default, about a second)."""
        self._sync_words[3] = int(polls)

    def wait_peers(self) -> None:
        """Stream-ordered, device-side: what follows on the current stream runs once every rank has published the
        launch this rank signalled last (for work of other libraries that reads the window)."""
        from . import _cabi
        with torch.cuda.device(self.local.device):
            st = _cabi.lib().ojx_e8t_peer_wait(self.sync_ptr, self.world,
                                               int(torch.cuda.current_stream(self.local.device).cuda_stream))
        _cabi.check(st, "ojx_e8t_peer_wait")

    def fence(self) -> None:
        """All ranks' earlier kernels on their current streams have completed once this returns on the stream
        (one tiny all-reduce: stream-ordered, no host synchronisation)."""
        import torch.distributed as dist
        dist.all_reduce(self._token, group=self.group)
