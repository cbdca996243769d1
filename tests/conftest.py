"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on CPU."""
from __future__ import annotations

import ctypes
import importlib
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("6s894_project_2025_b200")


@pytest.fixture(scope="session")
def lib():
    return importlib.import_module("6s894_project_2025_b200._lib")


@pytest.fixture(scope="session")
def oracle():
    return importlib.import_module("oracle.fwht_oracle")


@pytest.fixture(scope="session")
def coracle():
    """The C restatement (oracle/liboracle.so), built on demand with gcc."""
    so = ROOT / "oracle" / "liboracle.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    c = ctypes.CDLL(str(so))
    fp, dp, sz = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double), ctypes.c_size_t
    c.oracle_fwht_f32.argtypes = [fp, sz, sz, ctypes.c_float]
    c.oracle_fwht_f64.argtypes = [dp, sz, sz, ctypes.c_double]
    c.oracle_fused_gemm_f32.argtypes = [fp, fp, fp, sz, sz, sz, ctypes.c_float]
    c.oracle_fused_gemm_f64.argtypes = [dp, dp, dp, sz, sz, sz, ctypes.c_double]
    c.oracle_fused_gemv_f32.argtypes = [fp, fp, fp, sz, sz, sz, ctypes.c_float]
    c.oracle_fused_gemv_f64.argtypes = [dp, dp, dp, sz, sz, sz, ctypes.c_double]
    return c


@pytest.fixture(scope="session")
def golden():
    g = ROOT / "tests" / "golden"
    return {
        "fwht": np.load(g / "fwht_golden.npz"),
        "fused": np.load(g / "fused_golden.npz"),
    }


def fptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def dptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))
