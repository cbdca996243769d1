"""Pins the CPU oracle (numpy and C) to the golden vectors made from the
reference's own hadamard_ref (bench/bench.py:55-59) and to scipy's Sylvester
matrix, which the reference uses as its truth (HadaCore/test.py:27)."""
import math

import numpy as np
import pytest
import scipy.linalg

from conftest import dptr, fptr


@pytest.mark.parametrize("n", [1, 2, 4, 8, 64, 256, 1024])
def test_sylvester_is_scipy_hadamard(oracle, n):
    assert np.array_equal(oracle.sylvester(n), scipy.linalg.hadamard(n).astype(np.float64))


@pytest.mark.parametrize("n", [2, 8, 64, 512])
def test_butterfly_equals_explicit_matrix(oracle, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal((7, n))
    ref = x @ oracle.sylvester(n)
    got = oracle.fwht_butterfly(x)
    assert np.allclose(got, ref, rtol=0, atol=1e-9 * n)


@pytest.mark.parametrize("logn", range(1, 13))
def test_numpy_oracle_matches_reference_golden(oracle, golden, logn):
    n = 1 << logn
    g = golden["fwht"]
    x, y32 = g[f"x_{n}"], g[f"y32_{n}"]
    # fp32 explicit-matrix restatement: same arithmetic as the reference
    got = oracle.hadamard_ref(x, dtype=np.float32)
    assert oracle.rel_fro(got, y32) < 2e-6
    # fp64 butterfly: the reference's fp32 result is within fp32 rounding of it
    got64 = oracle.fwht_rows(x.astype(np.float64))
    assert oracle.rel_fro(y32, got64) < 1e-6
    assert np.max(np.abs(y32 - got64)) < 1e-5 * max(1.0, np.max(np.abs(got64)))


@pytest.mark.parametrize("logn", [1, 3, 8, 10, 12])
def test_golden_16bit_outputs_within_reference_tolerance(oracle, golden, logn):
    # HadaCore/test.py:93,99: atol 1e-2 (fp16) / 5e-2 (bf16) against the 16-bit matmul truth
    n = 1 << logn
    g = golden["fwht"]
    import torch

    x = torch.from_numpy(g[f"x_{n}"])
    for key, dt, atol in (("yf16", torch.float16, 1e-2), ("yb16", torch.bfloat16, 5e-2)):
        xin = x.to(dt).double().numpy()
        ref = oracle.fwht_rows(xin)
        assert np.max(np.abs(g[f"{key}_{n}"] - ref)) <= atol


def test_c_oracle_fwht_matches_numpy_and_golden(oracle, coracle, golden):
    g = golden["fwht"]
    for n in (2, 16, 256, 4096):
        x = g[f"x_{n}"]
        a = np.ascontiguousarray(x, dtype=np.float32).copy()
        coracle.oracle_fwht_f32(fptr(a), a.shape[0], n, np.float32(math.sqrt(1 / n)))
        assert oracle.rel_fro(a, g[f"y32_{n}"]) < 2e-6
        d = np.ascontiguousarray(x, dtype=np.float64).copy()
        coracle.oracle_fwht_f64(dptr(d), d.shape[0], n, math.sqrt(1 / n))
        assert np.allclose(d, oracle.fwht_rows(x.astype(np.float64)), rtol=0, atol=1e-12)


def test_fused_oracles_match_reference_golden(oracle, coracle, golden):
    g = golden["fused"]
    # GEMV layout, K=64, B=8, M=32
    W, X, Y = g["c1_W"], g["c1_X"], g["c1_Y"]
    got = oracle.fused_gemv_ref(W, X)
    assert oracle.rel_fro(got, Y) < 2e-6
    M, K = W.shape
    B = X.shape[1]
    yc = np.zeros((M, B), dtype=np.float32)
    assert coracle.oracle_fused_gemv_f32(fptr(np.ascontiguousarray(W)), fptr(np.ascontiguousarray(X)), fptr(yc),
                                         M, K, B, np.float32(math.sqrt(1 / K))) == 0
    assert oracle.rel_fro(yc, Y) < 2e-6
    # token-major GEMM layout
    Xg, Wg, Cg = g["g_X"], g["g_W"], g["g_C"]
    got = oracle.fused_gemm_ref(Xg, Wg)
    assert oracle.rel_fro(got, Cg) < 2e-6
    Mg, Kg = Wg.shape
    Ng = Xg.shape[0]
    cc = np.zeros((Mg, Ng), dtype=np.float64)
    assert coracle.oracle_fused_gemm_f64(dptr(Xg.astype(np.float64)), dptr(Wg.astype(np.float64)), dptr(cc),
                                         Mg, Ng, Kg, math.sqrt(1 / Kg)) == 0
    assert oracle.rel_fro(cc, got) < 1e-12


def test_transform_is_an_involution_and_isometry(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 1024))
    y = oracle.fwht_rows(x)
    assert np.allclose(oracle.fwht_rows(y), x, atol=1e-12)
    assert np.allclose(np.linalg.norm(y, axis=1), np.linalg.norm(x, axis=1))


def test_seeded_inputs_are_reproducible(oracle):
    a = oracle.make_inputs("c1")
    b = oracle.make_inputs("c1")
    assert (a["W"] == b["W"]).all() and (a["X"] == b["X"]).all()
    c5 = oracle.make_inputs("c5", K=64, M=8, N=4)
    assert set(np.unique(c5["d"].numpy())) <= {-1.0, 1.0}
