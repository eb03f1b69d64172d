"""Two or more ranks on one node: the grouped GEMV that stores its column shard into every rank's output window
must leave every window equal to an NCCL all-gather of the shards; and a chain of such launches that orders itself
on the device (epoch flags in the windows, no collective in between) must give what the same chain gives with an
all-gather after every launch.  Run by tests/test_multi_gpu.py under torchrun."""

import importlib
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    dist.init_process_group("nccl", device_id=dev)
    P = importlib.import_module("ojasx-open-source-cuda_b200")
    ops, sharding = P.ops, importlib.import_module("ojasx-open-source-cuda_b200.sharding")
    ok = True
    for (k, n, m, mats) in [(4096, 1024, 1, 3), (4096, 4096, 4, 2), (14336, 1024, 16, 2)]:
        n0, n1 = sharding.shard_rows(n, world, rank)
        nl = n1 - n0
        assert all(sharding.shard_rows(n, world, r)[1] - sharding.shard_rows(n, world, r)[0] == nl for r in range(world))
        window = sharding.PeerWindow(world * mats * m * nl, torch.bfloat16, dev)
        slots = window.local.view(world, mats, m, nl)
        x = ops.generate(m * k, 11, 1.0, torch.bfloat16, dev).view(m, k)
        entries, plain = [], []
        y_plain = torch.zeros((mats, m, nl), dtype=torch.bfloat16, device=dev)
        for j in range(mats):
            w = ops.generate(nl * k, 100 + j, 0.02, torch.float16, dev, start=n0 * k).view(nl, k)
            pk, sc = ops.encode(w, 32)
            entries.append((x, pk, sc, None, slots[rank, j]))
            plain.append((x, pk, sc, None, y_plain[j]))
        fused = ops.GroupedGemv(entries, [(nl, k)] * mats, peer_delta=window.delta)
        ref = ops.GroupedGemv(plain, [(nl, k)] * mats)
        for _ in range(2):
            fused()
            window.fence()
        ref()
        gathered = torch.empty((world, mats, m, nl), dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(gathered.view(world, -1), y_plain.view(-1))
        torch.cuda.synchronize()
        same = torch.equal(slots, gathered)
        window.close()
        dist.barrier()
        if not same:
            ok = False
            print(f"rank {rank}: mismatch at K={k} N={n} M={m}", flush=True)
    # the module form: ColumnShardedLinear.forward_fused against its NCCL forward, several calls in a row
    n, k = 2048, 4096
    w = ops.generate(n * k, 77, 0.02, torch.float16, dev).view(n, k)
    pk, sc = ops.encode(w, 32)
    bias = ops.generate(n, 78, 0.1, torch.bfloat16, dev)
    lin = sharding.ColumnShardedLinear(pk, sc, bias, n, k, 32, rank=rank, world_size=world)
    lin.enable_fused_gather(dev)
    for call, m in enumerate([1, 4, 16, 4, 1]):
        x = ops.generate(m * k, 200 + call, 1.0, torch.bfloat16, dev).view(m, k)
        y_fused = lin.forward_fused(x).clone()
        y_nccl = lin.forward(x)
        torch.cuda.synchronize()
        if not torch.equal(y_fused, y_nccl):
            ok = False
            print(f"rank {rank}: module mismatch at call {call} (M={m})", flush=True)
    for wdw in lin._fg["windows"]:
        wdw.close()
    dist.barrier()

    # a chain that orders itself on the device: y1 = A x, y2 = B y1, y3 = C y2 (K = 14336: partial sums + reduce
    # kernel), every matrix column-sharded, every launch reading the FULL previous output from this rank's window
    for m in (1, 16):
        dims = [(4096, 2048), (2048, 14336), (14336, 1024)]                     # (K, N) of A, B, C
        arena = sharding.PeerWindow(m * (2048 + 14336 + 1024), torch.bfloat16, dev)
        y1 = arena.local[: m * 2048].view(m, 2048)
        y2 = arena.local[m * 2048: m * (2048 + 14336)].view(m, 14336)
        y3 = arena.local[m * (2048 + 14336):].view(m, 1024)
        x0 = ops.generate(m * 4096, 300 + m, 1.0, torch.bfloat16, dev).view(m, 4096)
        shards, fulls = [], []
        for j, (k, n) in enumerate(dims):
            n0, n1 = sharding.shard_rows(n, world, rank, 32)
            wf = ops.generate(n * k, 310 + j, 0.02 if j == 0 else 0.05, torch.float16, dev).view(n, k)
            fulls.append(ops.encode(wf, 32))
            shards.append(ops.encode(wf[n0:n1].contiguous(), 32) + (n0, n1))
        ins, outs = [x0, y1, y2], [y1, y2, y3]
        chain = [ops.GroupedGemv([(ins[j], shards[j][0], shards[j][1], None, outs[j][:, shards[j][2]: shards[j][3]])],
                                 [(shards[j][3] - shards[j][2], dims[j][0])], peer_delta=arena.delta, peer_sync=arena.sync_ptr,
                                 wait_peers=(j > 0), signal_peers=True, static_weights=True) for j in range(3)]
        for _ in range(3):
            for g in chain:
                g()
        arena.wait_peers()                                   # the last launch of every rank has been published
        torch.cuda.synchronize()
        r1 = ops.linear(x0, fulls[0][0], fulls[0][1], None, 2048, 4096, 32)
        r2 = ops.linear(r1, fulls[1][0], fulls[1][1], None, 14336, 2048, 32)
        r3 = ops.linear(r2, fulls[2][0], fulls[2][1], None, 1024, 14336, 32)
        same = torch.equal(y1, r1) and torch.equal(y2, r2) and torch.equal(y3, r3) and arena.sync_status() == 0
        dist.barrier()
        arena.close()
        if not same:
            ok = False
            print(f"rank {rank}: device-ordered chain differs at M={m}", flush=True)
    dist.barrier()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PEER_WINDOW_OK" if int(flag.item()) == 1 else "PEER_WINDOW_MISMATCH", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
