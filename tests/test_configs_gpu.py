"""GPU parity at the shapes of the remaining benchmark configurations, reduced in count but not in shape:
a Llama-3-8B-shaped layer stack run through grouped launches with teacher-forced checks, and the encoder
over Llama-3-70B-shaped matrices compared with the C oracle by SHA-256."""

import hashlib

import numpy as np
import pytest

from conftest import have_cuda, load_pkg

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

DEV = "cuda:0"


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def P():
    if not have_cuda():
        pytest.skip("no CUDA device")
    pkg = load_pkg()
    pkg._cabi.lib()
    return pkg


@pytest.mark.parametrize("batch", [1, 16])
def test_llama8b_shaped_layers_grouped_and_teacher_forced(P, batch):
    """Two layers of the 8B-shaped stack (q,k,v <- h; a <- o(q); g,u <- a; h <- down(g + u)), q/k/v and gate/up
    each as ONE grouped launch.  Every matrix is checked against a dense fp32 product of its decoded weights with
    the bf16 input that was actually fed to it (teacher forcing), with the GEMM contract as the bar."""
    dev = torch.device(DEV)
    ops = P.ops
    H, KV, F = 4096, 1024, 14336

    def make(n, k, seed):
        w = ops.generate(n * k, seed, 0.02, torch.float16, dev).view(n, k)
        pk, sc = ops.encode(w, 32)
        return pk, sc, (n, k)

    def check(x, y, pk, sc, n, k):
        wd = ops.decode(pk, sc, (n, k), torch.float32)
        ref = x.float() @ wd.t()
        d = y.float() - ref
        assert float(d.norm() / ref.norm()) <= 2e-3
        assert float(d.abs().max()) <= 1e-2 * float(x.float().abs().max()) * k ** 0.5

    h = ops.generate(batch * H, 1, 1.0, torch.bfloat16, dev).view(batch, H)
    for layer in range(2):
        base = 100 * (layer + 1)
        q, kk, v, o = make(H, H, base + 1), make(KV, H, base + 2), make(KV, H, base + 3), make(H, H, base + 4)
        g, u, dn = make(F, H, base + 5), make(F, H, base + 6), make(H, F, base + 7)
        yq = torch.empty((batch, H), dtype=torch.bfloat16, device=dev)
        yk = torch.empty((batch, KV), dtype=torch.bfloat16, device=dev)
        yv = torch.empty((batch, KV), dtype=torch.bfloat16, device=dev)
        ops.GroupedGemv([(h, q[0], q[1], None, yq), (h, kk[0], kk[1], None, yk), (h, v[0], v[1], None, yv)],
                        [q[2], kk[2], v[2]])()
        for y, m in ((yq, q), (yk, kk), (yv, v)):
            check(h, y, m[0], m[1], *m[2])
        a = ops.linear(yq, o[0], o[1], None, H, H, 32)
        check(yq, a, o[0], o[1], H, H)
        yg = torch.empty((batch, F), dtype=torch.bfloat16, device=dev)
        yu = torch.empty((batch, F), dtype=torch.bfloat16, device=dev)
        ops.GroupedGemv([(a, g[0], g[1], None, yg), (a, u[0], u[1], None, yu)], [g[2], u[2]])()
        check(a, yg, g[0], g[1], F, H)
        check(a, yu, u[0], u[1], F, H)
        mid = (yg.float() + yu.float()).bfloat16()
        h = ops.linear(mid, dn[0], dn[1], None, H, F, 32)          # K = 14336: four K chunks + reduce pass
        check(mid, h, dn[0], dn[1], H, F)
        assert torch.isfinite(h.float()).all()
    assert P._cabi.lib().ojx_e8t_device_status() == 0


@pytest.mark.parametrize("rows,cols", [(1024, 8192), (2048, 28672), (8192, 8192)])
def test_encoder_llama70b_shapes_match_oracle_hash(P, oracle, coracle, rows, cols):
    """fp16 weights generated on the device (same bits as the host generator), encoded whole and in two row
    shards (the multi-GPU partition), compared with the C oracle by hash."""
    dev = torch.device(DEV)
    w = P.ops.generate(rows * cols, 70 + rows, 0.02, torch.float16, dev).view(rows, cols)
    pk, sc = P.ops.encode(w, 32)
    w_host = oracle.gen_normal(70 + rows, rows * cols, 0.02).astype(np.float16).astype(np.float32)
    cp, cs = coracle.encode(w_host, 32, threads=8)
    assert sha(pk.cpu().numpy()) == sha(cp)
    assert sha(sc.view(torch.int16).cpu().numpy().view(np.uint16)) == sha(cs.view(np.uint16))
    # row-sharded encode (two ranks' shares) reproduces the same bytes
    half = rows // 2
    p0, s0 = P.ops.encode(w[:half], 32)
    p1, s1 = P.ops.encode(w[half:], 32)
    assert torch.equal(torch.cat([p0, p1]), pk) and torch.equal(torch.cat([s0, s1]), sc)
    # decode -> dense matches the oracle's decode of the same bytes on a sample of rows
    dec = P.ops.decode(pk, sc, (rows, cols), torch.float32)[:4].cpu().numpy()
    ref = oracle.decode(cp[: 4 * cols * 3 // 16], cs[: 4 * cols // 32], (4, cols))
    assert np.array_equal(dec.view(np.uint32), ref.view(np.uint32))
