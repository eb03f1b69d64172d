"""The scratch-free decode entry point (collected last on purpose).

``ojx_e8t_gemv_static_scratch`` serves hosts that give a plug-in only its inputs and outputs - no
workspace, no right to call cudaMalloc (a serving process with a pre-carved device arena, a callback
where allocation would synchronise the device).  It keeps the fp32 partial sums of long-K problems in
an array inside the library image.  The check: called straight through the C ABI, twice in a row, it
must return exactly what ``ojx_e8t_gemv`` returns with caller-provided scratch (both run the same
deterministic kernels, so the comparison is bit-for-bit), and it must refuse problems that exceed its
built-in capacity.
"""

import ctypes

import pytest

from conftest import have_cuda, load_pkg

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_static_scratch_entry_matches_workspace_entry_twice():
    if not have_cuda():
        pytest.skip("no CUDA device")
    pkg = load_pkg()
    lib = pkg._cabi.lib()
    dev = torch.device("cuda:0")
    n, k, m = 512, 14336, 5                       # K spans four chunks -> partial sums in scratch
    need = lib.ojx_e8t_gemv_workspace_bytes(m, n, k)
    assert 0 < need <= lib.ojx_e8t_gemv_static_scratch_capacity()
    w = pkg.ops.generate(n * k, 321, 0.02, torch.float16, dev).view(n, k)
    packed, scales = pkg.ops.encode(w, 32)
    bias = pkg.ops.generate(n, 322, 0.5, torch.bfloat16, dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for attempt in range(2):                      # the shared array keeps the previous call's contents
        x = pkg.ops.generate(m * k, 400 + attempt, 1.0, torch.bfloat16, dev).view(m, k)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        y_ref = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        y_new = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        st = lib.ojx_e8t_gemv(x.data_ptr(), 2, m, packed.data_ptr(), scales.data_ptr(), bias.data_ptr(), n, k, 32,
                              y_ref.data_ptr(), 2, ws.data_ptr(), ws.numel(), stream)
        assert st == 0, pkg._cabi.status_name(st)
        st = lib.ojx_e8t_gemv_static_scratch(x.data_ptr(), 2, m, packed.data_ptr(), scales.data_ptr(), bias.data_ptr(),
                                             n, k, 32, y_new.data_ptr(), 2, stream)
        assert st == 0, pkg._cabi.status_name(st)
        torch.cuda.synchronize()
        assert torch.equal(y_new.view(torch.int16), y_ref.view(torch.int16)), f"call {attempt} differs"
        assert torch.isfinite(y_new.float()).all()
    # a problem whose partial sums exceed the built-in array is refused with a clear status, nothing is launched
    big_n = 65536
    assert lib.ojx_e8t_gemv_workspace_bytes(16, big_n, 14336) > lib.ojx_e8t_gemv_static_scratch_capacity()
    st = lib.ojx_e8t_gemv_static_scratch(x.data_ptr(), 2, 16, packed.data_ptr(), scales.data_ptr(), None, big_n, 14336, 32,
                                         y_new.data_ptr(), 2, stream)
    assert pkg._cabi.status_name(st) == "OJX_ERR_WORKSPACE"
    # short-K problems need no scratch at all and go straight through
    x2 = pkg.ops.generate(3 * 4096, 9, 1.0, torch.bfloat16, dev).view(3, 4096)
    w2 = pkg.ops.generate(64 * 4096, 10, 0.02, torch.float16, dev).view(64, 4096)
    p2, s2 = pkg.ops.encode(w2, 32)
    y2 = torch.empty((3, 64), dtype=torch.bfloat16, device=dev)
    st = lib.ojx_e8t_gemv_static_scratch(x2.data_ptr(), 2, 3, p2.data_ptr(), s2.data_ptr(), None, 64, 4096, 32,
                                         y2.data_ptr(), 2, stream)
    assert st == 0
    torch.cuda.synchronize()
    assert torch.equal(y2, pkg.ops.linear(x2, p2, s2, None, 64, 4096, 32))
