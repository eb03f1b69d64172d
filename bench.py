#!/usr/bin/env python
"""Benchmark of the ternary-E8 decode GEMV sweep (and, as extra lines of evidence, the prefill GEMM
and the encoder) on B200.

    python bench.py --gpus 1 --steps 20 --warmup 3            # this framework, one GPU
    torchrun ... bench.py --gpus N ...                        # output-column shards + NCCL all-gather
    python bench.py --impl reference                          # the reference's CPU kernel on host cores

Workload ("step"): one pass over the decode sweep at Llama-3-8B linear shapes
(K->N: 4096->4096, 4096->1024, 4096->14336, 14336->4096), batches 1, 4 and 16, over a rotation of
distinct seeded matrices per shape (the whole sweep is ~2.1 GB of packed weights, far larger than
L2, and a matrix is only revisited after the rest of the sweep has streamed through).  Every
(shape, batch) pair is ONE grouped launch over the rotation.  The metric is packed bytes streamed
per second.  Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)]      # (K, N)
BATCHES = [1, 4, 16]
METRIC = "E8 fused dequant-GEMM: decode GB/s on packed bytes @8B shapes"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (K=4096, N=14336, 16 matrices per launch: 234.9 MB of codes + scales, plus x and y, are the algorithmic bytes).
# The 16-row kernel has the largest share of the sweep's time, so its figure is the headline `traffic`.
NCU_TRAFFIC = {
    "gemv_b1_kernel (1 row)": {"dram_bytes": 238.7e6, "algorithmic_bytes": 235.5e6, "profile": "profiles/gemv_b1_kernel_K4096_N14336_R16_M1.md"},
    "gemv_bn_kernel<1,false,false> (4 rows)": {"dram_bytes": 240.7e6, "algorithmic_bytes": 237.2e6, "profile": "profiles/gemv_bn_kernel_K4096_N14336_R16_M4.md"},
    "gemv_bn_kernel<2,true,false> (16 rows)": {"dram_bytes": 243.1e6, "algorithmic_bytes": 244.3e6, "profile": "profiles/gemv_bn_kernel_K4096_N14336_R16_M16.md"},
}
TRAFFIC_PER_LAUNCH = NCU_TRAFFIC["gemv_bn_kernel<2,true,false> (16 rows)"]["dram_bytes"]


class _SubWindow:
    """A slice of a peer-mapped arena: same offsets on every rank, so the arena's deltas apply."""

    def __init__(self, arena, offset, numel):
        self.arena, self.local, self.delta = arena, arena.local[offset: offset + numel], arena.delta

    def fence(self):
        self.arena.fence()

    def close(self):
        self.arena.close()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in self.samples:
            try:
                sm.append(float(p[0])); mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(names, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# CPU baseline (the reference's native fused kernel compiled in place, else the oracle's C port)
# --------------------------------------------------------------------------------------------------

def cpu_baseline_run(repeats: int = 1, batches=(1, 4, 16)):
    """One bounded sample of the sweep on host cores: ONE matrix per shape at every batch, random valid
    codes (timing does not depend on the values).  Threads follow the reference's own wrapper, which
    parallelises over the rows of x only."""
    import numpy as np
    cores = os.cpu_count() or 1
    ref_so = os.path.join(ROOT, "oracle", "_ref", "libojx_ref.so")
    port_so = os.path.join(ROOT, "oracle", "libe8t_oracle.so")
    kind = None
    if os.path.exists(ref_so):
        lib = ctypes.CDLL(ref_so)
        lib.ojx_ref_ternary_forward.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 4 + [ctypes.c_int]
        kind = "reference"
    else:
        if not os.path.exists(port_so):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "all"], stdout=subprocess.DEVNULL)
        lib = ctypes.CDLL(port_so)
        lib.e8t_oracle_linear_mt.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 3 + [ctypes.c_int, ctypes.c_int]
        kind = "port"
    rng = np.random.default_rng(0)
    total_bytes, total_time, used_threads = 0, 0.0, 1
    for (k, n) in SHAPES:
        codes = rng.integers(0, 3281, size=n * k // 8, dtype=np.int64).reshape(-1, 2)
        packed = np.stack([codes[:, 0] & 0xFF, ((codes[:, 0] >> 8) & 0xF) | ((codes[:, 1] & 0xF) << 4), (codes[:, 1] >> 4) & 0xFF],
                          axis=1).astype(np.uint8).reshape(-1)
        for b in batches:
            x = rng.standard_normal((b, k)).astype(np.float32)
            y = np.zeros((b, n), dtype=np.float32)
            threads = max(1, min(b, cores))
            used_threads = max(used_threads, threads)
            if kind == "reference":
                scales = np.full(n * k // 32, 0.02, dtype=np.float32)
                fn = lambda: lib.ojx_ref_ternary_forward(x.ctypes.data, packed.ctypes.data, scales.ctypes.data, None,
                                                         y.ctypes.data, b, k, n, 32, threads)
            else:
                scales = np.full(n * k // 32, 0.02, dtype=np.float16).view(np.uint16)
                fn = lambda: lib.e8t_oracle_linear_mt(x.ctypes.data, packed.ctypes.data, scales.ctypes.data, None,
                                                      y.ctypes.data, b, k, n, 32, threads)
            for _ in range(repeats):
                t0 = time.perf_counter()
                fn()
                total_time += time.perf_counter() - t0
                total_bytes += n * k // 4
    return {"value": total_bytes / total_time / 1e9, "unit": "GB/s", "cores": used_threads, "kind": kind,
            "sample": f"one matrix per shape x batches {list(batches)}, {repeats} pass(es), fp32 activations, "
                      f"threads=min(batch, {cores} cores) as in the reference's wrapper",
            "seconds": total_time}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # bounded: every step is one pass of the sample; keep the whole run within a few minutes
    times, total = [], None
    for i in range(args.warmup + args.steps):
        r = cpu_baseline_run(1)
        if i >= args.warmup:
            times.append(r["seconds"])
        total = r
    bytes_per_step = sum(n * k // 4 for k, n in SHAPES) * len(BATCHES)
    val = bytes_per_step / (sum(times) / len(times)) / 1e9
    line = {"metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": "decode GEMV sweep, Llama-3-8B linear shapes, batch 1/4/16 (bounded sample: one matrix per shape)",
                       "shapes_K_N": SHAPES, "batches": BATCHES},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": total["cores"], "kind": total["kind"], "sample": total["sample"]},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rotation", type=int, default=64, help="distinct matrices per shape")
    ap.add_argument("--no-extras", action="store_true", help="skip prefill/encoder/per-shape extras")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--merge", default="off", choices=["auto", "on", "off"],
                    help="fused gather only: one grouped launch per batch size over all shapes instead of one per shape and "
                         "batch (auto: from 4 GPUs up); slower at 1 and 2 GPUs, where uneven item sizes cost more than the "
                         "saved launch start-ups")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: kernels store their column shard into every rank's output window (fused), or NCCL all-gather")
    ap.add_argument("--case", default=None, choices=["gemv", "gemm", "encode", "decode"],
                    help="run a few launches of ONE kernel on a small case and exit (used for ncu captures)")
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.case is not None:
        run_case(args)
        return

    import torch
    pkg = importlib.import_module("ojasx-open-source-cuda_b200")
    pkg._cabi.lib()                                        # no library -> loud failure, never a fallback
    ops = pkg.ops
    sharding = importlib.import_module("ojasx-open-source-cuda_b200.sharding")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    json_out = sys.stdout
    if world > 1:
        # NCCL prints its version banner with printf: everything that goes to file descriptor 1 from here on is
        # sent to stderr, and the one JSON line is written to the saved descriptor at the end
        sys.stdout.flush()
        json_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    hbm_peak, tf_peak, tf_sustained, peak_src = measured_peaks()

    # ---- build the sweep: per shape, R matrices (this rank's row shard of each), x and y buffers ----
    R = args.rotation
    groups = {}          # (shape index, batch) -> GroupedGemv
    gathers = {}         # (shape index, batch) -> (local flat y, gathered buffer)
    xs = {}
    packed_store = []
    launches_per_step = 0
    bytes_per_step = 0
    h2d_per_step = 0
    d2h_per_step = 0
    # N > 1, fused gather: one peer-mapped output window per (shape, batch).  Any rank that cannot map its peers'
    # memory sends every rank back to the NCCL all-gather.
    fused, windows = False, {}
    if world > 1 and args.gather == "fused":
        good = 1
        try:
            # ONE peer-mapped arena holds the windows of all (shape, batch) pairs, so every launch shares one delta list
            sizes = {(si, b): world * R * b * (sharding.shard_rows(n, world, rank)[1] - sharding.shard_rows(n, world, rank)[0])
                     for si, (k, n) in enumerate(SHAPES) for b in BATCHES}
            arena = sharding.PeerWindow(sum(sizes.values()), torch.bfloat16, dev)
            off = 0
            for key, size in sizes.items():
                windows[key] = _SubWindow(arena, off, size)
                off += size
        except Exception as exc:                                  # noqa: BLE001
            print(f"[bench] rank {rank}: peer windows unavailable ({exc}); using NCCL all-gather", file=sys.stderr)
            good = 0
        flag = torch.tensor([good], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        fused = int(flag.item()) == 1
        if fused:      # equal shard sizes are what makes the windows line up
            fused = all(sharding.shard_rows(n, world, r)[1] - sharding.shard_rows(n, world, r)[0] ==
                        sharding.shard_rows(n, world, 0)[1] - sharding.shard_rows(n, world, 0)[0]
                        for (k, n) in SHAPES for r in range(world))
    tmp = torch.empty(max(k * n for k, n in SHAPES), dtype=torch.float16, device=dev)
    for si, (k, n) in enumerate(SHAPES):
        n0, n1 = sharding.shard_rows(n, world, rank)
        nl = n1 - n0
        mats = []
        for r in range(R):
            seed = 1000 * (si + 1) + r
            w = ops.generate(nl * k, seed, 0.02, torch.float16, dev, start=n0 * k, out=tmp[: nl * k]).view(nl, k)
            pk, sc = ops.encode(w, 32)
            mats.append((pk, sc))
        packed_store.append(mats)
        for b in BATCHES:
            x = ops.generate(b * k, 7 + b + si, 1.0, torch.bfloat16, dev).view(b, k)
            xs[(si, b)] = x
            if fused:
                # every rank's window holds all ranks' shards: [world, R, b, nl]; this rank's kernels fill slot `rank`
                # of every window themselves
                window = windows[(si, b)]
                y_all = window.local.view(world, R, b, nl)[rank]
                delta = window.delta
            else:
                y_all = torch.zeros((R, b, nl), dtype=torch.bfloat16, device=dev)
                delta = None
            entries = [(x, pk, sc, None, y_all[r]) for r, (pk, sc) in enumerate(mats)]
            groups[(si, b)] = ops.GroupedGemv(entries, [(nl, k)] * R, peer_delta=delta)
            launches_per_step += 1 + groups[(si, b)].needs_reduce
            gathered = torch.empty((world, R, b, nl), dtype=torch.bfloat16, device=dev) if (world > 1 and not fused) else None
            gathers[(si, b)] = (y_all, gathered)
            bytes_per_step += R * (n * k // 4) // 1            # whole-job packed bytes (all ranks)
            h2d_per_step += b * k * 2
            d2h_per_step += R * b * n * 2
    merged = fused and (args.merge == "on" or (args.merge == "auto" and world >= 4))
    sweep = {}
    if merged:
        for b in BATCHES:
            ents, shps = [], []
            for si, (k, n) in enumerate(SHAPES):
                n0, n1 = sharding.shard_rows(n, world, rank)
                y_all = gathers[(si, b)][0]
                ents += [(xs[(si, b)], pk, sc, None, y_all[r]) for r, (pk, sc) in enumerate(packed_store[si])]
                shps += [(n1 - n0, k)] * R
            sweep[b] = ops.GroupedGemv(ents, shps, peer_delta=windows[(0, b)].delta)
        launches_per_step = sum(1 + sweep[b].needs_reduce for b in BATCHES)
    del tmp
    torch.cuda.synchronize()

    def step():
        # Fused: the kernels write every rank's window; the ranks meet once at the end of the pass.
        # NCCL: the groups are independent, so each all-gather (own buffers, NCCL's stream) overlaps the next
        # group's kernel; the compute stream joins all of them at the end of the pass.
        pending = []
        if merged:
            for b in BATCHES:
                sweep[b]()
            windows[(0, BATCHES[0])].fence()
            return
        for b in BATCHES:
            for si in range(len(SHAPES)):
                groups[(si, b)]()
                if world > 1 and not fused:
                    y_all, gathered = gathers[(si, b)]
                    pending.append(dist.all_gather_into_tensor(gathered.view(world, -1), y_all.view(1, -1).squeeze(0), async_op=True))
        for work in pending:
            work.wait()
        if fused:
            windows[(0, BATCHES[0])].fence()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region ----
    x_host = {key: x.cpu().pin_memory() for key, x in xs.items()}
    y_host = {key: torch.empty(ya.shape, dtype=ya.dtype).pin_memory() for key, (ya, _) in gathers.items()}

    # Uploads run ahead on their own stream and read-backs trail on another, so the PCIe transfers of one
    # (shape, batch) group overlap the kernels of its neighbours; everything is drained before the step ends.
    up_stream, down_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    keys = [(si, b) for b in BATCHES for si in range(len(SHAPES))]
    ev_x = {key: torch.cuda.Event() for key in keys}
    ev_y = {key: torch.cuda.Event() for key in keys}

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        with torch.cuda.stream(up_stream):
            for key in keys:
                xs[key].copy_(x_host[key], non_blocking=True)
                ev_x[key].record(up_stream)
        for key in keys:
            cur.wait_event(ev_x[key])
            groups[key]()
            if world > 1 and not fused:
                y_all, gathered = gathers[key]
                dist.all_gather_into_tensor(gathered.view(world, -1), y_all.view(-1))
            ev_y[key].record(cur)
            with torch.cuda.stream(down_stream):
                down_stream.wait_event(ev_y[key])
                y_host[key].copy_(gathers[key][0], non_blocking=True)
        if fused:
            windows[(0, BATCHES[0])].fence()
        torch.cuda.synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3 * 0.0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9

    extras = {}
    if not args.no_extras and world == 1:
        extras = run_extras(torch, ops, dev, groups, packed_store, hbm_peak, tf_peak)

    if rank == 0:
        # x and y traffic counted with the packed bytes in the roofline numerator
        act_bytes = sum(R * (b * k * 2 + b * n * 2) for k, n in SHAPES for b in BATCHES)
        algo_bytes = bytes_per_step + act_bytes
        achieved = algo_bytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "decode GEMV sweep, Llama-3-8B linear shapes (K->N 4096->4096, 4096->1024, 4096->14336, 14336->4096), "
                                   "batch 1/4/16, bf16 activations, bf16 outputs",
                       "rotation": R, "l2": "inputs larger than L2: %.2f GB of packed weights per pass, a matrix is revisited only after the whole sweep" % (bytes_per_step / 3 / 1e9),
                       "parallelism": (("output-column shards, kernels store into every rank's output window over NVLink (one fence per pass)"
                                        + (", one grouped launch per batch size" if merged else "")) if fused
                                       else "output-column shards + NCCL all-gather") if world > 1 else "single GPU",
                       "launches_per_step": launches_per_step},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak * world, "unit": "GB/s", "frac": achieved / (hbm_peak * world),
                         "traffic": TRAFFIC_PER_LAUNCH, "traffic_per_kernel": NCU_TRAFFIC,
                         "kernel": "gemv_b1_kernel / gemv_bn_kernel (one grouped launch per shape and batch)",
                         "peak_source": peak_src + " (MEASURED_PEAKS.json hbm_gbs)" if peak_src == "measured" else peak_src,
                         "note": "achieved = (packed + activation + output bytes of a pass) / time of a pass, all GPUs together; launch gaps included; peak = measured per-GPU HBM bandwidth x n_gpus"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d_per_step, "d2h_bytes_per_step": d2h_per_step,
                    "ms_per_step": e2e_ms},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline_run(1)
            cb.pop("seconds", None)
            line["cpu_baseline"] = cb
        line.update(extras)
        json_out.write(json.dumps(line) + "\n")
        json_out.flush()
    if world > 1:
        for w in windows.values():
            w.close()
        barrier()
        dist.destroy_process_group()


def run_case(args):
    """A few launches of one kernel on one shape, timed with CUDA events; prints one JSON line."""
    import torch
    pkg = importlib.import_module("ojasx-open-source-cuda_b200")
    ops = pkg.ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    k, n, m = args.K, args.N, args.M
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w = ops.generate(n * k, 3, 0.02, torch.float16, dev).view(n, k)
    info = {"case": args.case, "K": k, "N": n, "M": m, "launches": args.launches}
    if args.case == "gemv":
        R = args.rotation
        mats = []
        for r in range(R):
            ops.generate(n * k, 100 + r, 0.02, torch.float16, dev, out=w.view(-1))
            mats.append(ops.encode(w, 32))
        x = ops.generate(m * k, 7, 1.0, torch.bfloat16, dev).view(m, k)
        y = torch.zeros((R, m, n), dtype=torch.bfloat16, device=dev)
        grp = ops.GroupedGemv([(x, pk, sc, None, y[r]) for r, (pk, sc) in enumerate(mats)], [(n, k)] * R)
        fn = grp
        info["bytes_per_launch"] = grp.packed_bytes + R * (m * k * 2 + m * n * 2)
    elif args.case == "gemm":
        pk, sc = ops.encode(w, 32)
        x = ops.generate(m * k, 7, 1.0, torch.bfloat16, dev).view(m, k)
        fn = lambda: ops.linear(x, pk, sc, None, n, k, 32, force="gemm")
        info["flops_per_launch"] = 2.0 * m * n * k
    elif args.case == "encode":
        pk = torch.empty(n * k * 3 // 16, dtype=torch.uint8, device=dev)
        sc = torch.empty(n * k // 32, dtype=torch.float16, device=dev)
        fn = lambda: ops.encode(w, 32, out=(pk, sc))
        info["bytes_per_launch"] = n * k * 2.25
    else:
        pk, sc = ops.encode(w, 32)
        out = torch.empty((n, k), dtype=torch.float16, device=dev)
        fn = lambda: ops.decode(pk, sc, (n, k), torch.float16, out=out)
        info["bytes_per_launch"] = n * k * 2.25
    torch.cuda.synchronize()
    times = []
    for _ in range(args.launches):
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    info["ms"] = times
    if "bytes_per_launch" in info:
        info["GBps_last"] = info["bytes_per_launch"] / (times[-1] * 1e-3) / 1e9
    else:
        info["TFLOPs_last"] = info["flops_per_launch"] / (times[-1] * 1e-3) / 1e12
    print(json.dumps(info))


def run_extras(torch, ops, dev, groups, packed_store, hbm_peak, tf_peak):
    """Per-(shape, batch) decode numbers, the prefill GEMM and the encoder, each timed with CUDA events."""
    out = {"decode_detail": [], "prefill": [], "encoder": None, "decoder": None}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)       # > L2

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    for (si, b), grp in sorted(groups.items()):
        k, n = SHAPES[si]
        ms = timed(grp, 5)
        gbs = grp.packed_bytes / (ms * 1e-3) / 1e9
        out["decode_detail"].append({"K": k, "N": n, "batch": b, "ms": ms, "packed_GBps": gbs, "frac_hbm": gbs / hbm_peak})

    # Prefill: M = 2048 tokens through eight DISTINCT matrices of the shape, issued back to back like the
    # linears of consecutive layers (weights cold, launch latency overlapped); also one cold call on its own.
    m = 2048
    for si, (k, n) in enumerate(SHAPES):
        x = ops.generate(m * k, 99 + si, 1.0, torch.bfloat16, dev).view(m, k)
        mats = packed_store[si][:8]

        def stream_of_calls():
            for pk, sc in mats:
                ops.linear(x, pk, sc, None, n, k, 32, force="gemm")

        ms = timed(stream_of_calls, 5) / len(mats)
        ops.gemm_status(dev)
        pk, sc = packed_store[si][0]
        ms_single = timed(lambda: ops.linear(x, pk, sc, None, n, k, 32, force="gemm"), 5)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out["prefill"].append({"K": k, "N": n, "M": m, "ms": ms, "TFLOPs": tf, "frac_bf16_peak": tf / tf_peak,
                               "calls_per_timing": len(mats),
                               "single_cold_call_ms": ms_single, "single_cold_call_TFLOPs": 2.0 * m * n * k / (ms_single * 1e-3) / 1e12})

    k, n = 8192, 28672
    w = ops.generate(n * k, 5, 0.02, torch.float16, dev).view(n, k)
    pk = torch.empty(n * k * 3 // 16, dtype=torch.uint8, device=dev)
    sc = torch.empty(n * k // 32, dtype=torch.float16, device=dev)
    ms = timed(lambda: ops.encode(w, 32, out=(pk, sc)), 3)
    gbs = n * k * 2.25 / (ms * 1e-3) / 1e9
    out["encoder"] = {"rows": n, "cols": k, "dtype": "f16", "ms": ms, "GBps": gbs, "frac_hbm": gbs / hbm_peak,
                      "Gweights_per_s": n * k / (ms * 1e-3) / 1e9}
    out["stack"] = run_stack(torch, ops, dev, timed, hbm_peak)
    # decoder (unpack): packed codes + scales -> dense fp16 weights, 0.25 B read + 2 B written per weight
    ms = timed(lambda: ops.decode(pk, sc, (n, k), torch.float16, out=w), 3)
    gbs = n * k * 2.25 / (ms * 1e-3) / 1e9
    out["decoder"] = {"rows": n, "cols": k, "dtype": "f16", "ms": ms, "GBps": gbs, "frac_hbm": gbs / hbm_peak}
    return out


def run_stack(torch, ops, dev, timed, hbm_peak, layers=32):
    """The linears of a Llama-3-8B-shaped decoder stack (32 layers x {q, k, v, o, gate, up, down} = 224 matrices,
    1.74 GB packed) run as a chain with real data flow - q,k,v <- h; a <- o(q); g,u <- a; h <- down(g + u) - four
    launches per layer (q/k/v grouped, o, gate/up grouped, down).  Attention, norms and activations are not part
    of the path and are left out; every matrix is distinct, so the weights always come from HBM."""
    H, KV, F = 4096, 1024, 14336
    w = torch.empty(F * H, dtype=torch.float16, device=dev)

    def make(n, k, seed):
        ops.generate(n * k, seed, 0.02, torch.float16, dev, out=w[: n * k])
        return ops.encode(w[: n * k].view(n, k), 32)

    mats = [[make(*shape, 5000 + 10 * layer + j) for j, shape in enumerate([(H, H), (KV, H), (KV, H), (H, H), (F, H), (F, H), (H, F)])]
            for layer in range(layers)]
    packed_bytes = layers * sum(n * k // 4 for n, k in [(H, H), (KV, H), (KV, H), (H, H), (F, H), (F, H), (H, F)])
    results = []
    for b in (1, 16):
        h = ops.generate(b * H, 9, 1.0, torch.bfloat16, dev).view(b, H)
        q = torch.empty((b, H), dtype=torch.bfloat16, device=dev)
        kk, v = (torch.empty((b, KV), dtype=torch.bfloat16, device=dev) for _ in range(2))
        a = torch.empty((b, H), dtype=torch.bfloat16, device=dev)
        g, u, mid = (torch.empty((b, F), dtype=torch.bfloat16, device=dev) for _ in range(3))
        steps = []
        for m in mats:
            steps.append(ops.GroupedGemv([(h, m[0][0], m[0][1], None, q), (h, m[1][0], m[1][1], None, kk), (h, m[2][0], m[2][1], None, v)],
                                         [(H, H), (KV, H), (KV, H)]))
            steps.append(ops.GroupedGemv([(q, m[3][0], m[3][1], None, a)], [(H, H)]))
            steps.append(ops.GroupedGemv([(a, m[4][0], m[4][1], None, g), (a, m[5][0], m[5][1], None, u)], [(F, H), (F, H)]))
            steps.append(ops.GroupedGemv([(mid, m[6][0], m[6][1], None, h)], [(H, F)]))

        def forward():
            for i, st in enumerate(steps):
                if i % 4 == 3:
                    torch.add(g, u, out=mid)
                st()

        ms_eager = timed(forward, 3)
        # the same chain replayed from a CUDA graph: no per-launch host work
        ms = ms_eager
        mode = "eager"
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                forward()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                forward()
            ms = timed(graph.replay, 3)
            mode = "cuda graph"
        except Exception as exc:                                  # noqa: BLE001
            print(f"[bench] layer-stack graph capture unavailable: {exc}", file=sys.stderr)
        gbs = packed_bytes / (ms * 1e-3) / 1e9
        results.append({"batch": b, "layers": layers, "matrices": 7 * layers, "launches": 4 * layers, "ms": ms, "mode": mode,
                        "ms_eager": ms_eager,
                        "packed_GBps": gbs, "frac_hbm": gbs / hbm_peak, "tokens_per_s_linears_only": b / (ms * 1e-3)})
    return results


if __name__ == "__main__":
    main()
