"""The allocation-free fused entry point, b200ht_fused_gemm_static.

It exists for callers that cannot allocate device memory at the call site (a
server whose pool owns the whole GPU, a plugin hook that may not allocate, a
loop that must not touch the driver's allocator): the transformed tokens go to
a fixed array inside the library instead of a caller workspace.  This test
calls it through the C ABI twice in a row (the second call reuses the array
with a different, smaller problem, so stale contents of the first call would
show) and compares each result with b200ht_fused_gemm on the same inputs, using
the tolerances of the other fused tests (1e-5 fp32, 2e-2 bf16).  The file name
makes pytest collect it last, so a failure here cannot hide other results.
"""
import importlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, X, W, out_dtype, layout):
    l = lib.load()
    N, K = X.shape
    M = W.shape[0]
    dt = {torch.float32: lib.F32, torch.bfloat16: lib.BF16}
    shape = (M, N) if layout == lib.OUT_MN else (N, M)
    st = torch.cuda.current_stream().cuda_stream
    c_static = torch.empty(shape, dtype=out_dtype, device="cuda")
    rc = l.b200ht_fused_gemm_static(X.data_ptr(), W.data_ptr(), c_static.data_ptr(), M, N, K, dt[X.dtype],
                                    dt[out_dtype], layout, float(K ** -0.5), st)
    assert rc == 0, lib.error_string(rc)
    ws = torch.empty(l.b200ht_fused_gemm_workspace_bytes(M, N, K, dt[X.dtype]), dtype=torch.uint8, device="cuda")
    c_ws = torch.empty(shape, dtype=out_dtype, device="cuda")
    rc = l.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), c_ws.data_ptr(), M, N, K, dt[X.dtype], dt[out_dtype],
                             layout, float(K ** -0.5), ws.data_ptr(), ws.numel(), st)
    assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    return c_static, c_ws


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-5)])
def test_static_scratch_entry_matches_workspace_entry_twice(lib, dtype, tol):
    oracle = importlib.import_module("oracle.fwht_oracle")
    g = torch.Generator().manual_seed(11)
    cases = [(384, 700, 1024, lib.OUT_MN), (130, 96, 512, lib.OUT_NM)]   # second call: smaller, other layout
    for M, N, K, layout in cases:
        X = torch.randn(N, K, generator=g).to(dtype).cuda()
        W = torch.randn(M, K, generator=g).to(dtype).cuda()
        c_static, c_ws = _both(lib, X, W, torch.float32, layout)
        a, b = c_static.double().cpu().numpy(), c_ws.double().cpu().numpy()
        assert oracle.rel_fro(a, b) <= tol and oracle.rel_max(a, b) <= tol
        ref = oracle.fused_gemm_ref(X.double().cpu().numpy(), W.double().cpu().numpy())
        got = a if layout == lib.OUT_MN else a.T
        assert oracle.rel_fro(got, ref) <= tol
    assert lib.load().b200ht_device_status(1) == 0


def test_static_scratch_entry_rejects_oversized_problems(lib):
    l = lib.load()
    K = 8192
    n_fit = lib.STATIC_SCRATCH_BYTES // (K * 2)
    x = torch.zeros(16, dtype=torch.uint8, device="cuda")
    p = x.data_ptr()
    # one token too many for the built-in array: refused before anything is launched
    rc = l.b200ht_fused_gemm_static(p, p, p, 128, n_fit + 1, K, lib.BF16, lib.F32, lib.OUT_MN, 1.0, None)
    assert rc == -9
    assert "static scratch" in lib.error_string(rc)
    rc = l.b200ht_fused_gemm_static(p, p, p, 128, n_fit // 2 + 1, K, lib.F32, lib.F32, lib.OUT_MN, 1.0, None)
    assert rc == -9


def test_static_entry_back_to_back_through_the_two_launch_contraction(lib):
    """M=4096, N=2560, K=64 needs 16 x 10 = 160 tiles of 256 rows on 148 SMs, so the contraction is two launches
    (whole waves of 256-row tiles, then a 128-row tail) tied together by programmatic dependencies.  Two such calls
    are enqueued back to back on one stream with no synchronisation in between: the second call's transform
    overwrites the built-in array while the first call's tail may still be draining, unless the ordering inside the
    library holds.  Both results must equal the workspace entry's, bit for bit (same kernels, same inputs)."""
    l = lib.load()
    g = torch.Generator().manual_seed(12)
    M, N, K = 4096, 2560, 64
    Xa = torch.randn(N, K, generator=g).bfloat16().cuda()
    Xb = torch.randn(N, K, generator=g).bfloat16().cuda()
    W = torch.randn(M, K, generator=g).bfloat16().cuda()
    st = torch.cuda.current_stream().cuda_stream
    sc = float(K ** -0.5)
    ca = torch.empty(N, M, dtype=torch.bfloat16, device="cuda")
    cb = torch.empty(N, M, dtype=torch.bfloat16, device="cuda")
    for X, C in ((Xa, ca), (Xb, cb)):      # no sync between the two calls
        rc = l.b200ht_fused_gemm_static(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, lib.BF16, lib.BF16,
                                        lib.OUT_NM, sc, st)
        assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    ws = torch.empty(l.b200ht_fused_gemm_workspace_bytes(M, N, K, lib.BF16), dtype=torch.uint8, device="cuda")
    for X, C in ((Xa, ca), (Xb, cb)):
        ref = torch.empty_like(C)
        rc = l.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), ref.data_ptr(), M, N, K, lib.BF16, lib.BF16, lib.OUT_NM,
                                 sc, ws.data_ptr(), ws.numel(), st)
        assert rc == 0, lib.error_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(C, ref)
    assert l.b200ht_device_status(1) == 0


def test_static_entry_leaves_free_device_memory_unchanged(lib):
    """The point of the entry: after one warm-up call of a given shape class (which may make the driver load the
    kernels it needs), further calls change the device's free memory by nothing."""
    l = lib.load()
    g = torch.Generator().manual_seed(13)
    M, N, K = 512, 640, 1024
    X = torch.randn(N, K, generator=g).bfloat16().cuda()
    W = torch.randn(M, K, generator=g).bfloat16().cuda()
    C = torch.empty(M, N, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def call():
        rc = l.b200ht_fused_gemm_static(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, lib.BF16, lib.F32,
                                        lib.OUT_MN, float(K ** -0.5), st)
        assert rc == 0, lib.error_string(rc)

    call()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_static_entry_checks_the_transform_size_before_the_scratch_size(lib):
    l = lib.load()
    x = torch.zeros(16, dtype=torch.uint8, device="cuda")
    p = x.data_ptr()
    # K not a power of two, and so large that N*K would also exceed the array: the size error wins
    rc = l.b200ht_fused_gemm_static(p, p, p, 128, 1 << 20, 3000, lib.BF16, lib.F32, lib.OUT_MN, 1.0, None)
    assert rc == -2
