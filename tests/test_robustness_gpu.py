"""Error paths and device-side ordering of the decode-shape kernels, on one GPU and without ever hanging or
faulting it: every wait in the kernels is bounded, so the tests make a wait run out (a flag that nothing sets,
a copy whose completion is never reported) and check that the kernel returns, that the failure is reported
through every channel, and that the next normal call is correct."""

import numpy as np
import pytest

from conftest import have_cuda, load_pkg

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

DEV = "cuda:0"
TIMEOUT = -7


@pytest.fixture(scope="module")
def P():
    if not have_cuda():
        pytest.skip("no CUDA device")
    pkg = load_pkg()
    pkg._cabi.lib()
    return pkg


def _problem(P, n, k, m, seed):
    dev = torch.device(DEV)
    w = P.ops.generate(n * k, seed, 0.02, torch.float16, dev).view(n, k)
    pk, sc = P.ops.encode(w, 32)
    x = P.ops.generate(m * k, seed + 1, 1.0, torch.bfloat16, dev).view(m, k)
    return pk, sc, x


def test_chain_orders_itself_on_the_device(P):
    """Two dependent grouped launches - the second reads what the first wrote - ordered by the peer-sync block
    alone (one rank, so 'every rank' is this one): results equal the unsynchronised path, the epoch counts the
    signalled launches, and K > 4096 (partial sums + reduce kernel) signals from the reduce kernel."""
    dev = torch.device(DEV)
    m = 4
    pk1, sc1, x = _problem(P, 512, 4096, m, 10)
    pk2, sc2, _ = _problem(P, 256, 512, m, 20)
    pk3, sc3, x3 = _problem(P, 128, 14336, m, 30)
    mid = torch.zeros((m, 512), dtype=torch.bfloat16, device=dev)
    out = torch.zeros((m, 256), dtype=torch.bfloat16, device=dev)
    out3 = torch.zeros((m, 128), dtype=torch.bfloat16, device=dev)
    sync = torch.zeros(64, dtype=torch.int32, device=dev)
    first = P.ops.GroupedGemv([(x, pk1, sc1, None, mid)], [(512, 4096)], peer_delta=[0], peer_sync=sync.data_ptr(),
                              signal_peers=True, static_weights=True)
    second = P.ops.GroupedGemv([(mid, pk2, sc2, None, out)], [(256, 512)], peer_delta=[0], peer_sync=sync.data_ptr(),
                               wait_peers=True, signal_peers=True, static_weights=True)
    third = P.ops.GroupedGemv([(x3, pk3, sc3, None, out3)], [(128, 14336)], peer_delta=[0], peer_sync=sync.data_ptr(),
                              wait_peers=True, signal_peers=True, static_weights=True)
    for _ in range(3):
        first(); second(); third()
    torch.cuda.synchronize()
    ref_mid = P.ops.linear(x, pk1, sc1, None, 512, 4096, 32)
    ref_out = P.ops.linear(ref_mid, pk2, sc2, None, 256, 512, 32)
    ref3 = P.ops.linear(x3, pk3, sc3, None, 128, 14336, 32)
    assert torch.equal(mid, ref_mid) and torch.equal(out, ref_out) and torch.equal(out3, ref3)
    words = sync.cpu().numpy()
    assert words[0] == 9 and words[1] == 0 and words[2] == 0 and words[4] == 9      # epoch, arrived, status, flag[0]
    assert P._cabi.lib().ojx_e8t_device_status() == 0


def test_wait_on_a_rank_that_never_signals_gives_up(P):
    dev = torch.device(DEV)
    lib = P._cabi.lib()
    pk, sc, x = _problem(P, 256, 1024, 2, 40)
    y = torch.zeros((2, 256), dtype=torch.bfloat16, device=dev)
    sync = torch.zeros(64, dtype=torch.int32, device=dev)
    sync[0] = 5          # this rank believes five launches are done; nobody has published them into flag[0]
    sync[3] = 2000       # polls before giving up (about a millisecond)
    grp = P.ops.GroupedGemv([(x, pk, sc, None, y)], [(256, 1024)], peer_delta=[0], peer_sync=sync.data_ptr(), wait_peers=True)
    grp()
    torch.cuda.synchronize()                                  # the kernel returned
    assert int(sync[2].item()) == TIMEOUT
    with pytest.raises(P._cabi.OjxError):                     # the next call through a wrapper raises, no sync needed
        P.ops.linear(x, pk, sc, None, 256, 1024, 32)
    assert lib.ojx_e8t_poll_status() == 0                     # reported once
    assert lib.ojx_e8t_device_status() == TIMEOUT and lib.ojx_e8t_device_status() == 0
    sync.zero_()
    grp()                                                     # epoch 0, flag 0: nothing to wait for
    torch.cuda.synchronize()
    assert torch.equal(y, P.ops.linear(x, pk, sc, None, 256, 1024, 32))
    assert lib.ojx_e8t_device_status() == 0


def test_copy_that_never_completes_gives_up(P):
    """The loader withholds one arrival on the first work item's 'copies landed' barrier: every warp's wait on it
    runs into the (shortened) limit, the CTAs stop touching their inputs, keep their barriers matched, wait for
    the copies that are in flight, and return."""
    dev = torch.device(DEV)
    lib = P._cabi.lib()
    pk, sc, x = _problem(P, 4096, 4096, 16, 50)
    y = torch.zeros((16, 4096), dtype=torch.bfloat16, device=dev)
    good = P.ops.GroupedGemv([(x, pk, sc, None, y)], [(4096, 4096)])
    bad = P.ops.GroupedGemv([(x, pk, sc, None, y)], [(4096, 4096)], extra_flags=P._cabi.OJX_GEMV_TEST_LOSE_COPY)
    lib.ojx_e8t_set_wait_limit(3000)
    try:
        bad()
        torch.cuda.synchronize()
    finally:
        lib.ojx_e8t_set_wait_limit(0)
    with pytest.raises(P._cabi.OjxError):
        good()
    assert lib.ojx_e8t_device_status() == TIMEOUT
    good()
    torch.cuda.synchronize()
    wd = P.ops.decode(pk, sc, (4096, 4096), torch.float32)
    ref = x.float() @ wd.t()
    assert float((y.float() - ref).norm() / ref.norm()) <= 2e-3
    assert lib.ojx_e8t_device_status() == 0 and lib.ojx_e8t_poll_status() == 0


def test_two_devices_in_one_process(P):
    """Kernel attributes and the SM count are kept per device: the same process drives cuda:0 and cuda:1."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    outs = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        w = P.ops.generate(512 * 4096, 3, 0.02, torch.float16, dev).view(512, 4096)
        pk, sc = P.ops.encode(w, 32)
        x = P.ops.generate(16 * 4096, 4, 1.0, torch.bfloat16, dev).view(16, 4096)
        outs.append(P.ops.linear(x, pk, sc, None, 512, 4096, 32).cpu())
        outs.append(P.ops.linear(x.repeat(8, 1), pk, sc, None, 512, 4096, 32, force="gemm")[:16].cpu())
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])


def test_independent_launches_overlap_without_changing_results(P):
    """OJX_GEMV_INDEPENDENT: launches over different matrices with their own activations and outputs never wait for
    the launch queued ahead of them; their results equal the ordered launches' bit for bit, a dependent reader queued
    after them sees complete outputs, and the flag is refused together with the cross-GPU ordering flags."""
    dev = torch.device(DEV)
    groups, ordered = [], []
    for i, (n, k, m) in enumerate([(512, 4096, 1), (1024, 14336, 4), (384, 4096, 16), (2048, 4096, 1)]):
        mats = [_problem(P, n, k, m, 40 + 10 * i + j) for j in range(6)]
        y_a = torch.zeros((6, m, n), dtype=torch.bfloat16, device=dev)
        y_b = torch.zeros((6, m, n), dtype=torch.bfloat16, device=dev)
        groups.append((P.ops.GroupedGemv([(x, pk, sc, None, y_a[j]) for j, (pk, sc, x) in enumerate(mats)], [(n, k)] * 6,
                                         static_weights=True, independent=True), y_a))
        ordered.append((P.ops.GroupedGemv([(x, pk, sc, None, y_b[j]) for j, (pk, sc, x) in enumerate(mats)], [(n, k)] * 6), y_b))
    for grp, _ in ordered:
        grp()
    for _ in range(3):                                      # back to back: the tail of one launch is filled by the next
        for grp, _ in groups:
            grp()
    total = sum(y.float().sum() for _, y in groups)         # a dependent reader, queued after the launches
    torch.cuda.synchronize()
    for (_, ya), (_, yb) in zip(groups, ordered):
        assert torch.equal(ya, yb)
    assert torch.isfinite(total)
    groups[0][0](independent=False)                         # per-call override back to an ordered launch
    torch.cuda.synchronize()
    assert torch.equal(groups[0][1], ordered[0][1])
    lib = P._cabi.lib()
    g0 = groups[0][0]
    sync = torch.zeros(16, dtype=torch.int32, device=dev)
    st = lib.ojx_e8t_gemv_grouped_ex(g0.table.data_ptr(), g0.count, g0.total_tiles, g0.M, 2, 2, g0.needs_reduce, None, 1,
                                     sync.data_ptr(), P._cabi.OJX_GEMV_INDEPENDENT | P._cabi.OJX_GEMV_WAIT_PEERS, None)
    assert st == -9
