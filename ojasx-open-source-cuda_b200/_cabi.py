"""ctypes binding of the C ABI declared in ``include/ojx_e8t.h``.

The shared library is built in-tree (``csrc/`` -> ``lib/libojx_e8t.so``) by :func:`build`.
There is no CPU fallback: if the library is missing or a call returns a negative status,
a ``RuntimeError`` carrying the status name is raised.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libojx_e8t.so")

OJX_F32, OJX_F16, OJX_BF16 = 0, 1, 2
OJX_GEMV_STATIC_WEIGHTS, OJX_GEMV_SIGNAL_PEERS, OJX_GEMV_WAIT_PEERS, OJX_GEMV_TEST_LOSE_COPY = 1, 2, 4, 8
OJX_GEMV_INDEPENDENT = 16
OJX_ENCODE_HADAMARD = 1
PEER_SYNC_BYTES = 48        # sizeof(ojx_e8t_peer_sync): epoch, arrived, status, spin_limit, flag[8]

EXPORTED_SYMBOLS = (
    "ojx_e8t_version", "ojx_e8t_status_string", "ojx_e8t_encode", "ojx_e8t_encode_ex", "ojx_e8t_fwht32", "ojx_e8t_encode_2bit", "ojx_e8t_decode_2bit", "ojx_e8t_linear_2bit", "ojx_e8t_encode_1bit", "ojx_e8t_decode_1bit", "ojx_e8t_linear_1bit", "ojx_e8t_linear_lowbit_lora", "ojx_e8t_project", "ojx_e8t_ste_quantize", "ojx_e8t_decode",
    "ojx_e8t_gemv_workspace_bytes", "ojx_e8t_gemv", "ojx_e8t_gemv_lora", "ojx_e8t_gemv_tiles", "ojx_e8t_gemv_kchunks",
    "ojx_e8t_gemv_grouped", "ojx_e8t_gemv_grouped_peers", "ojx_e8t_gemv_grouped_ex", "ojx_e8t_peer_wait", "ojx_e8t_enable_peer_access", "ojx_e8t_gemm_workspace_bytes", "ojx_e8t_gemm", "ojx_e8t_gemm_lowbit", "ojx_e8t_gemm_status", "ojx_e8t_gemm_dx", "ojx_e8t_gemm_dx_lowbit", "ojx_e8t_gemm_dx_workspace_bytes",
    "ojx_e8t_generate", "ojx_e8t_last_cuda_error", "ojx_e8t_device_status", "ojx_e8t_poll_status", "ojx_e8t_set_wait_limit",
    "ojx_e8t_gemv_static_scratch", "ojx_e8t_gemv_static_scratch_capacity",
)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class OjxError(RuntimeError):
    """A C-ABI call returned a negative status."""


def sources():
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".inc"))] + [
        os.path.join(os.path.dirname(HERE), "include", "ojx_e8t.h")]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > built for s in sources())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``csrc/ojx_e8t.cu`` for sm_100a into ``lib/libojx_e8t.so`` (nvcc cross-compiles
    without a GPU).  Returns the library path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libojx_e8t.so")
    os.makedirs(LIB_DIR, exist_ok=True)
    tmp = LIB_PATH + ".tmp.%d" % os.getpid()
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", tmp, os.path.join(CSRC, "ojx_e8t.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    os.replace(tmp, LIB_PATH)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


class GemvProblem(ctypes.Structure):
    """Mirror of ``ojx_e8t_gemv_problem`` (88 bytes)."""
    _fields_ = [
        ("x", ctypes.c_void_p), ("packed", ctypes.c_void_p), ("scales", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("y", ctypes.c_void_p), ("partial", ctypes.c_void_p),
        ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("tile_begin", ctypes.c_int32), ("ldy", ctypes.c_int32),
        ("lora_t", ctypes.c_void_p), ("lora_b", ctypes.c_void_p), ("lora_rank", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


def _declare(lib: ctypes.CDLL) -> None:
    vp, i32, i64, u64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t
    lib.ojx_e8t_version.restype = i32
    lib.ojx_e8t_version.argtypes = []
    lib.ojx_e8t_status_string.restype = ctypes.c_char_p
    lib.ojx_e8t_status_string.argtypes = [i32]
    lib.ojx_e8t_encode.restype = i32
    lib.ojx_e8t_encode.argtypes = [vp, i32, i64, i64, i32, vp, vp, vp]
    lib.ojx_e8t_encode_ex.restype = i32
    lib.ojx_e8t_encode_ex.argtypes = [vp, i32, i64, i64, i32, ctypes.c_uint32, vp, vp, vp]
    lib.ojx_e8t_encode_2bit.restype = i32
    lib.ojx_e8t_encode_2bit.argtypes = [vp, i32, i64, i64, i32, vp, vp, vp]
    lib.ojx_e8t_decode_2bit.restype = i32
    lib.ojx_e8t_decode_2bit.argtypes = [vp, vp, i64, i64, i32, i32, vp, vp]
    lib.ojx_e8t_linear_lowbit_lora.restype = i32
    lib.ojx_e8t_linear_lowbit_lora.argtypes = [i32, vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, vp, i32, vp, i32, vp]
    lib.ojx_e8t_linear_2bit.restype = i32
    lib.ojx_e8t_linear_2bit.argtypes = [vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, i32, vp]
    lib.ojx_e8t_encode_1bit.restype = i32
    lib.ojx_e8t_encode_1bit.argtypes = [vp, i32, i64, i64, i32, vp, vp, vp]
    lib.ojx_e8t_decode_1bit.restype = i32
    lib.ojx_e8t_decode_1bit.argtypes = [vp, vp, i64, i64, i32, i32, vp, vp]
    lib.ojx_e8t_linear_1bit.restype = i32
    lib.ojx_e8t_linear_1bit.argtypes = [vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, i32, vp]
    lib.ojx_e8t_project.restype = i32
    lib.ojx_e8t_project.argtypes = [vp, i64, vp, vp]
    lib.ojx_e8t_ste_quantize.restype = i32
    lib.ojx_e8t_ste_quantize.argtypes = [vp, i64, vp, vp]
    lib.ojx_e8t_fwht32.restype = i32
    lib.ojx_e8t_fwht32.argtypes = [vp, i32, i64, vp, vp]
    lib.ojx_e8t_decode.restype = i32
    lib.ojx_e8t_decode.argtypes = [vp, vp, i64, i64, i32, i32, vp, vp]
    lib.ojx_e8t_gemv_lora.restype = i32
    lib.ojx_e8t_gemv_lora.argtypes = [vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, vp, i32, vp, i32, vp, sz, vp]
    lib.ojx_e8t_gemv_workspace_bytes.restype = sz
    lib.ojx_e8t_gemv_workspace_bytes.argtypes = [i64, i64, i64]
    lib.ojx_e8t_gemv.restype = i32
    lib.ojx_e8t_gemv.argtypes = [vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, i32, vp, sz, vp]
    lib.ojx_e8t_gemv_static_scratch.restype = i32
    lib.ojx_e8t_gemv_static_scratch.argtypes = [vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, i32, vp]
    lib.ojx_e8t_gemv_static_scratch_capacity.restype = sz
    lib.ojx_e8t_gemv_static_scratch_capacity.argtypes = []
    lib.ojx_e8t_gemv_tiles.restype = i32
    lib.ojx_e8t_gemv_tiles.argtypes = [i64, i64]
    lib.ojx_e8t_gemv_kchunks.restype = i32
    lib.ojx_e8t_gemv_kchunks.argtypes = [i64]
    lib.ojx_e8t_gemv_grouped.restype = i32
    lib.ojx_e8t_gemv_grouped.argtypes = [vp, i32, i32, i64, i32, i32, i32, vp]
    lib.ojx_e8t_enable_peer_access.restype = i32
    lib.ojx_e8t_enable_peer_access.argtypes = [i32]
    lib.ojx_e8t_gemv_grouped_peers.restype = i32
    lib.ojx_e8t_gemv_grouped_peers.argtypes = [vp, i32, i32, i64, i32, i32, i32, vp, i32, vp]
    lib.ojx_e8t_gemv_grouped_ex.restype = i32
    lib.ojx_e8t_gemv_grouped_ex.argtypes = [vp, i32, i32, i64, i32, i32, i32, vp, i32, vp, i32, vp]
    lib.ojx_e8t_peer_wait.restype = i32
    lib.ojx_e8t_peer_wait.argtypes = [vp, i32, vp]
    lib.ojx_e8t_gemm_workspace_bytes.restype = sz
    lib.ojx_e8t_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    lib.ojx_e8t_gemm.restype = i32
    lib.ojx_e8t_gemm.argtypes = [vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, i32, vp, sz, vp]
    lib.ojx_e8t_gemm_lowbit.restype = i32
    lib.ojx_e8t_gemm_lowbit.argtypes = [i32, vp, i32, i64, vp, vp, vp, i64, i64, i32, vp, i32, vp, sz, vp]
    lib.ojx_e8t_gemm_dx_workspace_bytes.restype = sz
    lib.ojx_e8t_gemm_dx_workspace_bytes.argtypes = [i64, i64, i64]
    lib.ojx_e8t_gemm_dx.restype = i32
    lib.ojx_e8t_gemm_dx.argtypes = [vp, i32, i64, vp, vp, i64, i64, i32, vp, i32, vp, sz, vp]
    lib.ojx_e8t_gemm_dx_lowbit.restype = i32
    lib.ojx_e8t_gemm_dx_lowbit.argtypes = [i32] + [vp, i32, i64, vp, vp, i64, i64, i32, vp, i32, vp, sz, vp]
    lib.ojx_e8t_gemm_status.restype = i32
    lib.ojx_e8t_gemm_status.argtypes = [vp, vp]
    lib.ojx_e8t_last_cuda_error.restype = ctypes.c_char_p
    lib.ojx_e8t_last_cuda_error.argtypes = []
    lib.ojx_e8t_device_status.restype = i32
    lib.ojx_e8t_device_status.argtypes = []
    lib.ojx_e8t_poll_status.restype = i32
    lib.ojx_e8t_poll_status.argtypes = []
    lib.ojx_e8t_set_wait_limit.restype = None
    lib.ojx_e8t_set_wait_limit.argtypes = [ctypes.c_uint32]
    lib.ojx_e8t_generate.restype = i32
    lib.ojx_e8t_generate.argtypes = [vp, i32, i64, u64, i64, ctypes.c_float, vp]


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built: the CUDA path is the only path."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing. Build it with this module's build() (needs nvcc); "
                        "this package has no CPU or PyTorch fallback.")
                handle = ctypes.CDLL(LIB_PATH)
                _declare(handle)
                _lib = handle
    return _lib


def status_name(code: int) -> str:
    return lib().ojx_e8t_status_string(int(code)).decode()


def raise_pending() -> None:
    """Raises if a kernel launched earlier ran into the limit of one of its bounded waits (read from the library's
    pinned status word: no synchronisation).  Called by the wrappers at the start of every decode-shape call."""
    if lib().ojx_e8t_poll_status() != 0:
        raise OjxError("an earlier launch gave up on a bounded device-side wait (OJX_ERR_TIMEOUT): its outputs are invalid")


def check(code: int, what: str) -> None:
    if code != 0:
        detail = ""
        if code == -6:
            detail = " - CUDA: " + lib().ojx_e8t_last_cuda_error().decode()
        raise OjxError(f"{what} failed: {status_name(code)} ({code}){detail}")
