"""Shared fixtures: repository paths, the golden vectors, the CPU oracle (numpy + C)."""

from __future__ import annotations

import ctypes
import importlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG_NAME = "ojasx-open-source-cuda_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_pkg():
    """The package directory name contains hyphens; import it by string."""
    return importlib.import_module(PKG_NAME)


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


@pytest.fixture(scope="session")
def golden():
    gdir = os.path.join(ROOT, "tests", "golden")
    with open(os.path.join(gdir, "e8t_golden.json")) as f:
        meta = json.load(f)
    arrays = np.load(os.path.join(gdir, "e8t_golden.npz"))
    return meta, arrays


@pytest.fixture(scope="session")
def oracle():
    from oracle import e8t_oracle
    return e8t_oracle


class COracle:
    """ctypes view of oracle/libe8t_oracle.so (built on demand with make)."""

    def __init__(self):
        odir = os.path.join(ROOT, "oracle")
        so = os.path.join(odir, "libe8t_oracle.so")
        src = os.path.join(odir, "e8t_oracle.c")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", odir, "all"], stdout=subprocess.DEVNULL)
        self.lib = ctypes.CDLL(so)
        p = ctypes.c_void_p
        self.lib.e8t_oracle_encode.argtypes = [p, ctypes.c_int64, ctypes.c_int, p, p]
        self.lib.e8t_oracle_decode.argtypes = [p, p, ctypes.c_int64, ctypes.c_int, p]
        self.lib.e8t_oracle_linear.argtypes = [p, p, p, p, p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
        self.lib.e8t_oracle_linear_mt.argtypes = self.lib.e8t_oracle_linear.argtypes + [ctypes.c_int]
        self.lib.e8t_oracle_encode_mt.argtypes = self.lib.e8t_oracle_encode.argtypes + [ctypes.c_int]

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    def encode(self, w, group=32, threads=1):
        flat = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        ngr = (flat.size + group - 1) // group
        packed = np.zeros(ngr * group * 3 // 16, dtype=np.uint8)
        scales = np.zeros(ngr, dtype=np.uint16)
        if threads > 1:
            self.lib.e8t_oracle_encode_mt(self._p(flat), flat.size, group, self._p(packed), self._p(scales), threads)
        else:
            self.lib.e8t_oracle_encode(self._p(flat), flat.size, group, self._p(packed), self._p(scales))
        return packed, scales.view(np.float16)

    def decode(self, packed, scales, shape, group=32):
        out = np.zeros(shape[0] * shape[1], dtype=np.float32)
        sc = np.ascontiguousarray(scales).view(np.uint16)
        pk = np.ascontiguousarray(packed)
        self.lib.e8t_oracle_decode(self._p(pk), self._p(sc), out.size, group, self._p(out))
        return out.reshape(shape)

    def linear(self, x, packed, scales, n, k, bias=None, group=32, threads=1):
        x = np.ascontiguousarray(x, dtype=np.float32)
        m = x.shape[0]
        y = np.zeros((m, n), dtype=np.float32)
        sc = np.ascontiguousarray(scales).view(np.uint16)
        pk = np.ascontiguousarray(packed)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        bp = None if b is None else self._p(b)
        if threads > 1:
            self.lib.e8t_oracle_linear_mt(self._p(x), self._p(pk), self._p(sc), bp, self._p(y), m, k, n, group, threads)
        else:
            self.lib.e8t_oracle_linear(self._p(x), self._p(pk), self._p(sc), bp, self._p(y), m, k, n, group)
        return y


@pytest.fixture(scope="session")
def coracle():
    return COracle()


def case_input(oracle_mod, case):
    """Regenerate a golden case's input exactly (fp32 array holding the stored dtype's values)."""
    w = oracle_mod.gen_normal(case["seed"], case["rows"] * case["cols"], case["sigma"]).reshape(case["rows"], case["cols"])
    if case["dtype"] == "f16":
        return w.astype(np.float16)
    if case["dtype"] == "bf16":
        return oracle_mod.bf16_bits_to_f32(oracle_mod.f32_to_bf16_bits(w)).reshape(w.shape)
    return w


def have_cuda():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
