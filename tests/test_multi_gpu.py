"""Multi-GPU parity (needs at least two GPUs on the node; skipped otherwise)."""

import os
import socket
import subprocess
import sys

import pytest

from conftest import have_cuda

pytestmark = pytest.mark.gpu


def test_fused_gather_equals_nccl_all_gather():
    torch = pytest.importorskip("torch")
    if not have_cuda() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    with socket.socket() as sock:                   # a port nobody else on this shared machine is using right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(here, "peer_window_check.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "PEER_WINDOW_OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-2000:]
