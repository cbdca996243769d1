"""GPU parity of the fused W . H(X) entry points against the CPU oracle.
Tolerances from the task statement: relative error <= 1e-5 for fp32, <= 2e-2
for bf16 inputs with fp32 accumulation (both as ||.||_F ratio and max ratio)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 2e-2


def _check(oracle, got, ref, tol):
    got = np.asarray(got, dtype=np.float64)
    assert oracle.rel_fro(got, ref) <= tol, oracle.rel_fro(got, ref)
    assert oracle.rel_max(got, ref) <= tol, oracle.rel_max(got, ref)


def test_c1_fp32_gemv(pkg, oracle):
    inp = oracle.make_inputs("c1")
    W, X = inp["W"], inp["X"]
    ref = oracle.fused_gemv_ref(W.numpy(), X.numpy())
    Y = pkg.fused_ht_gemv(W.cuda(), X.cuda())
    assert Y.shape == (32, 8)
    _check(oracle, Y.cpu().numpy(), ref, F32_TOL)
    # the same numbers through the GEMM entry (tokens = columns of X)
    C = pkg.fused_ht_gemm(X.t().contiguous().cuda(), W.cuda())
    _check(oracle, C.cpu().numpy(), ref, F32_TOL)


def test_golden_fused_vectors(pkg, oracle, golden):
    g = golden["fused"]
    W, X, Y = map(torch.from_numpy, (g["c1_W"], g["c1_X"], g["c1_Y"]))
    got = pkg.fused_ht_gemv(W.cuda(), X.cuda()).cpu().numpy()
    _check(oracle, got, Y.numpy(), 2e-5)   # the golden itself is an fp32 computation
    Xg, Wg, Cg = map(torch.from_numpy, (g["g_X"], g["g_W"], g["g_C"]))
    got = pkg.fused_ht_gemm(Xg.cuda(), Wg.cuda()).cpu().numpy()
    _check(oracle, got, Cg.numpy(), 2e-5)
    got = pkg.fused_ht_gemm(Xg.cuda(), Wg.cuda(), out_layout="nm").cpu().numpy()
    _check(oracle, got.T, Cg.numpy(), 2e-5)


@pytest.mark.parametrize("M,N,K", [(32, 8, 64), (1, 1, 2), (7, 5, 4), (130, 67, 16), (128, 256, 128),
                                   (300, 129, 1024), (64, 33, 8192)])
def test_fp32_gemm_shapes(pkg, oracle, M, N, K):
    inp = oracle.make_inputs("c3", K=K, N=N, M=M)
    X, W = inp["X"], inp["W"]
    ref = oracle.fused_gemm_ref(X.numpy(), W.numpy())
    for layout in ("mn", "nm"):
        C = pkg.fused_ht_gemm(X.cuda(), W.cuda(), out_layout=layout).cpu().numpy()
        _check(oracle, C if layout == "mn" else C.T, ref, F32_TOL)
    # reference executable convention: unscaled transform
    ref1 = oracle.fused_gemm_ref(X.numpy(), W.numpy(), scale=1.0)
    C = pkg.fused_ht_gemm(X.cuda(), W.cuda(), scale=1.0).cpu().numpy()
    _check(oracle, C, ref1, F32_TOL)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 128), (256, 512, 256), (100, 77, 64),
                                   (129, 257, 1024), (384, 300, 4096), (8, 4, 32), (5, 3, 2),
                                   (2048, 1024, 2048)])
def test_bf16_gemm_shapes(pkg, oracle, M, N, K):
    inp = oracle.make_inputs("c3", K=K, N=N, M=M)
    X, W = inp["X"].bfloat16(), inp["W"].bfloat16()
    ref = oracle.fused_gemm_ref(X.double().numpy(), W.double().numpy())
    for layout, odt in (("mn", torch.float32), ("nm", torch.float32), ("mn", torch.bfloat16), ("nm", torch.bfloat16)):
        C = pkg.fused_ht_gemm(X.cuda(), W.cuda(), out_layout=layout, out_dtype=odt)
        assert pkg.device_status() == 0
        C = C.float().cpu().numpy()
        _check(oracle, C if layout == "mn" else C.T, ref, BF16_TOL)


def test_c3_full_size_fp32_and_bf16(pkg, oracle):
    inp = oracle.make_inputs("c3")
    X, W = inp["X"], inp["W"]                       # 4096 x 1024 each
    rows = np.array([0, 1, 127, 128, 2047, 4095])
    Y = oracle.fwht_rows(X.double().numpy())        # 4096 x 1024
    ref_rows = W.double().numpy()[rows] @ Y.T       # 6 x 4096
    C = pkg.fused_ht_gemm(X.cuda(), W.cuda())
    _check(oracle, C[rows].cpu().numpy(), ref_rows, F32_TOL)
    Xb, Wb = X.bfloat16(), W.bfloat16()
    Yb = oracle.fwht_rows(Xb.double().numpy())
    refb = Wb.double().numpy()[rows] @ Yb.T
    Cb = pkg.fused_ht_gemm(Xb.cuda(), Wb.cuda())
    assert pkg.device_status() == 0
    _check(oracle, Cb[rows].cpu().numpy(), refb, BF16_TOL)
    # checksum of checksums: column sums of C equal (sum of W rows) . H(X)
    colsum = Cb.double().sum(dim=0).cpu().numpy()
    ref_colsum = Wb.double().numpy().sum(axis=0) @ Yb.T
    assert oracle.rel_fro(colsum, ref_colsum) <= BF16_TOL


@pytest.mark.parametrize("B", [1, 4, 16])
def test_c4_bf16_gemv(pkg, oracle, B):
    inp = oracle.make_inputs("c4", B=B)
    W, X = inp["W"], inp["X"]
    ref = oracle.fused_gemv_ref(W.double().numpy(), X.double().numpy())
    Y = pkg.fused_ht_gemv(W.cuda(), X.cuda())
    assert Y.shape == (4096, B)
    _check(oracle, Y.cpu().numpy(), ref, BF16_TOL)
    Yb = pkg.fused_ht_gemv(W.cuda(), X.cuda(), out_dtype=torch.bfloat16)
    _check(oracle, Yb.float().cpu().numpy(), ref, BF16_TOL)


@pytest.mark.parametrize("M,N,B,dtype", [(32, 64, 8, torch.float32), (64, 128, 16, torch.float32),
                                         (128, 256, 32, torch.float32), (5, 2, 1, torch.float32),
                                         (33, 32, 3, torch.bfloat16), (100, 512, 9, torch.bfloat16),
                                         (17, 2048, 64, torch.bfloat16), (40, 32768, 2, torch.bfloat16),
                                         (9, 16384, 5, torch.float32)])
def test_gemv_shapes_including_reference_self_tests(pkg, oracle, M, N, B, dtype):
    # (32,64,8), (64,128,16), (128,256,32) are the shapes of fwht_gemv_fusion.cu:632-634;
    # inputs uniform in [-1, 1] and the unscaled transform, as there (:278-282)
    g = torch.Generator().manual_seed(42)
    W = (torch.rand(M, N, generator=g) * 2 - 1).to(dtype)
    X = (torch.rand(N, B, generator=g) * 2 - 1).to(dtype)
    ref = oracle.fused_gemv_ref(W.double().numpy(), X.double().numpy(), scale=1.0)
    Y = pkg.fused_ht_gemv(W.cuda(), X.cuda(), scale=1.0).cpu().numpy()
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    _check(oracle, Y, ref, tol)
    if dtype == torch.float32 and N <= 256:
        assert np.max(np.abs(Y - ref)) < 1e-3   # the reference's own absolute gate (:293-312)


def test_c5_reduced_and_sharded(pkg, oracle):
    """C5 distribution at a reduced shape; 2-way and 4-way token shards must
    reproduce the unsharded result bit for bit."""
    inp = oracle.make_inputs("c5", K=8192, M=512, N=768)
    X, W = inp["X"], inp["W"]
    ref = oracle.fused_gemm_ref(X.double().numpy(), W.double().numpy())
    Xd, Wd = X.cuda(), W.cuda()
    full = pkg.fused_ht_gemm(Xd, Wd, out_layout="nm")
    assert pkg.device_status() == 0
    _check(oracle, full.cpu().numpy().T, ref, BF16_TOL)
    for world in (2, 4):
        parts = [pkg.fused_ht_gemm(pkg.shard_tokens(Xd, r, world), Wd, out_layout="nm") for r in range(world)]
        assert torch.equal(torch.cat(parts, dim=0), full)


def test_c5_full_size_sampled(pkg, oracle):
    inp = oracle.make_inputs("c5")
    X, W = inp["X"], inp["W"]                        # 16384 x 8192, 28672 x 8192
    Xd, Wd = X.cuda(), W.cuda()
    C = pkg.fused_ht_gemm(Xd, Wd, out_layout="nm", out_dtype=torch.bfloat16)   # 16384 x 28672
    assert pkg.device_status() == 0
    toks = np.array([0, 255, 256, 8191, 12345, 16383])
    rows = np.array([0, 127, 128, 14335, 20000, 28671])
    Y = oracle.fwht_rows(X[toks].double().numpy())            # 6 x 8192
    ref = Y @ W[rows].double().numpy().T                      # 6 tokens x 6 rows
    got = C[toks][:, rows].float().cpu().numpy()
    _check(oracle, got, ref, BF16_TOL)
    # checksum over all rows of W for the sampled tokens
    ref_sum = Y @ W.double().numpy().sum(axis=0)
    got_sum = C[toks].double().sum(dim=1).cpu().numpy()
    assert oracle.rel_fro(got_sum, ref_sum) <= BF16_TOL


def test_host_pipeline_matches_single_call(pkg, oracle):
    inp = oracle.make_inputs("c5", K=1024, M=384, N=1000)
    X, W = inp["X"], inp["W"]
    Wd = W.cuda()
    ref = pkg.fused_ht_gemm(X.cuda(), Wd, out_layout="nm", out_dtype=torch.bfloat16).cpu()
    pipe = pkg.HostPipeline(Wd, 1000, chunk_tokens=256, n_streams=3)
    Xh = X.pin_memory()
    out = torch.empty(1000, 384, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        out.zero_()
        pipe(Xh, out)
        torch.cuda.synchronize()
        assert torch.equal(out, ref)
    assert pkg.device_status() == 0


def test_fused_gemm_with_sign_diagonal(pkg, oracle):
    inp = oracle.make_inputs("c5", K=2048, M=300, N=260)
    W, d = inp["W"], inp["d"]
    X0 = torch.randn(260, 2048, generator=torch.Generator().manual_seed(9)).bfloat16()   # tokens before the diagonal
    ref = oracle.fused_gemm_ref((X0.double() * d.double()).numpy(), W.double().numpy())
    C = pkg.fused_ht_gemm(X0.cuda(), W.cuda(), signs=d)
    _check(oracle, C.cpu().numpy(), ref, BF16_TOL)
    C2 = pkg.fused_ht_gemm((X0 * d.bfloat16()).cuda(), W.cuda())
    assert torch.equal(C, C2)


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
@pytest.mark.parametrize("layout", ["mn", "nm"])
def test_output_of_more_than_2_31_elements(pkg, dtype, out_dtype, layout):
    """Output offsets past 2^31 elements: M x N = 65664 x 33000 (2.17e9 entries) with a small K.  Rows and
    columns sampled across the whole output are compared with a torch product of the transformed tokens."""
    M, N, K = 65664, 33000, 64
    g = torch.Generator(device="cuda").manual_seed(11)
    X = torch.randn(N, K, generator=g, device="cuda").to(dtype)
    W = (torch.randn(M, K, generator=g, device="cuda") / 8).to(dtype)
    C = pkg.fused_ht_gemm(X, W, out_dtype=out_dtype, out_layout=layout)
    assert pkg.device_status() == 0
    H = torch.ones(1, 1, dtype=torch.float64, device="cuda")
    while H.shape[0] < K:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    HX = (X.double() @ H * K ** -0.5).float()                    # explicit Sylvester matrix, as the reference's check
    if dtype == torch.bfloat16:
        HX = HX.bfloat16().float()                               # the kernel rounds H(X) to bf16 before the product
    ref_full = lambda ms, ns: W[ms].double() @ HX[ns].double().t()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    ms = torch.tensor(sorted({0, 1, 127, 128, M // 2, 65535, 65536, M - 1}), device="cuda")
    ns = torch.tensor(sorted({0, 1, 255, 256, N // 2, 32767, 32768, N - 1}), device="cuda")
    all_n = torch.arange(N, device="cuda")
    all_m = torch.arange(M, device="cuda")
    Cv = C if layout == "mn" else C.t()
    for got, ref in ((Cv[ms].double(), ref_full(ms, all_n)), (Cv[:, ns].double(), ref_full(all_m, ns))):
        err = (got - ref).norm() / ref.norm()
        assert float(err) <= tol, float(err)
    del C, Cv
    torch.cuda.empty_cache()


@pytest.mark.parametrize("M,N,B", [(4096, 256, 2), (300, 1024, 8), (6000, 4096, 24), (1000, 8192, 8),
                                   (4741, 512, 12), (77, 4096, 40), (4096, 2048, 5), (10000, 256, 1),
                                   (9000, 4096, 16), (8, 8192, 4), (29, 1024, 32),
                                   (7000, 2048, 4), (20000, 1024, 8), (6000, 1024, 32), (12000, 8192, 2)])
def test_bf16_gemv_streaming_path_shapes(pkg, oracle, M, N, B):
    """The bf16 path for 256 <= N <= 8192: every copy-in variant of X (B = 1, 2, 4, multiples of 8, others),
    1 to 4 column tiles, column splits (B > 32), one and several row groups per CTA (the latter with two warp
    groups of eight on 8 x 64 k items where N allows, four of four otherwise), ragged last rows."""
    g = torch.Generator().manual_seed(1000 + M + N + B)
    W = (torch.randn(M, N, generator=g) / N ** 0.5).bfloat16()
    X = torch.randn(N, B, generator=g).bfloat16()
    ref = oracle.fused_gemv_ref(W.double().numpy(), X.double().numpy())
    Y = pkg.fused_ht_gemv(W.cuda(), X.cuda())
    assert pkg.device_status() == 0
    _check(oracle, Y.cpu().numpy(), ref, BF16_TOL)
    Yb = pkg.fused_ht_gemv(W.cuda(), X.cuda(), out_dtype=torch.bfloat16)
    _check(oracle, Yb.float().cpu().numpy(), ref, BF16_TOL)


@pytest.mark.parametrize("M,N,B", [(256, 256, 512), (64, 128, 256), (128, 256, 512), (512, 512, 1024)])
def test_gemv_with_the_reference_benchmark_batches(pkg, oracle, M, N, B):
    """The reference's own benchmark calls its GEMV kernel with B up to 2048 (fwht_gemv_fusion.cu:643-653).  The
    Python entry serves B > 64 through the fused GEMM; the C entry loops over column groups.  Both must agree
    with the oracle (fp32, unscaled as there)."""
    g = torch.Generator().manual_seed(5)
    W = torch.rand(M, N, generator=g) * 2 - 1
    X = torch.rand(N, B, generator=g) * 2 - 1
    ref = oracle.fused_gemv_ref(W.double().numpy(), X.double().numpy(), scale=1.0)
    Wd, Xd = W.cuda(), X.cuda()
    Y = pkg.fused_ht_gemv(Wd, Xd, scale=1.0)
    assert Y.shape == (M, B)
    _check(oracle, Y.cpu().numpy(), ref, F32_TOL)
    lib = pkg._lib.load()
    Y2 = torch.empty(M, B, device="cuda")
    rc = lib.b200ht_fused_gemv(Wd.data_ptr(), Xd.data_ptr(), Y2.data_ptr(), M, N, B, pkg._lib.F32, pkg._lib.F32, 1.0,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    _check(oracle, Y2.cpu().numpy(), ref, F32_TOL)
    # bf16: the streaming path in column groups of 32
    Yb = torch.empty(M, B, device="cuda")
    Wb, Xb = Wd.bfloat16(), Xd.bfloat16()
    rc = lib.b200ht_fused_gemv(Wb.data_ptr(), Xb.data_ptr(), Yb.data_ptr(), M, N, B,
                               pkg._lib.BF16, pkg._lib.F32, 1.0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    refb = oracle.fused_gemv_ref(W.bfloat16().double().numpy(), X.bfloat16().double().numpy(), scale=1.0)
    _check(oracle, Yb.cpu().numpy(), refb, BF16_TOL)


@pytest.mark.parametrize("M,N,K", [(1024, 768, 1024), (600, 900, 4096), (4096, 4096, 32), (2000, 3000, 128)])
def test_fp32_tensor_core_contraction(pkg, oracle, M, N, K):
    """fp32 inputs on shapes large enough for the split-bf16 tensor-core contraction (three bf16 terms per operand,
    six products): same 1e-5 bar as the FFMA kernel, both layouts and output types, and `exact=True` still gives
    the FFMA result."""
    lib = pkg._lib.load()
    assert lib.b200ht_fused_gemm_tc_workspace_bytes(M, N, K, pkg._lib.F32) > \
        lib.b200ht_fused_gemm_workspace_bytes(M, N, K, pkg._lib.F32)
    inp = oracle.make_inputs("c3", K=K, N=N, M=M)
    X, W = inp["X"], inp["W"]
    ref = oracle.fused_gemm_ref(X.numpy(), W.numpy())
    Xd, Wd = X.cuda(), W.cuda()
    for layout in ("mn", "nm"):
        C = pkg.fused_ht_gemm(Xd, Wd, out_layout=layout).cpu().numpy()
        _check(oracle, C if layout == "mn" else C.T, ref, F32_TOL)
    Ce = pkg.fused_ht_gemm(Xd, Wd, exact=True).cpu().numpy()
    _check(oracle, Ce, ref, F32_TOL)
    Cb = pkg.fused_ht_gemm(Xd, Wd, out_dtype=torch.bfloat16).float().cpu().numpy()
    _check(oracle, Cb, ref, 1e-2)   # bf16 rounding of the result only
    assert pkg.device_status() == 0


def test_fp32_long_rows_keep_the_ffma_kernel(pkg):
    # K = 8192: the tensor-core accumulator's truncation error would reach the 1e-5 bar, so the split path is off
    lib = pkg._lib.load()
    assert lib.b200ht_fused_gemm_tc_workspace_bytes(2048, 2048, 8192, pkg._lib.F32) == \
        lib.b200ht_fused_gemm_workspace_bytes(2048, 2048, 8192, pkg._lib.F32)
    assert lib.b200ht_fused_gemm_tc_workspace_bytes(64, 64, 64, pkg._lib.F32) == \
        lib.b200ht_fused_gemm_workspace_bytes(64, 64, 64, pkg._lib.F32)
    assert lib.b200ht_fused_gemm_tc_workspace_bytes(4096, 4096, 1024, pkg._lib.BF16) == \
        lib.b200ht_fused_gemm_workspace_bytes(4096, 4096, 1024, pkg._lib.BF16)


@pytest.mark.parametrize("dtype,M,N,K", [(torch.bfloat16, 300, 200, 256), (torch.bfloat16, 4096, 2560, 64),
                                         (torch.bfloat16, 640, 777, 32), (torch.float32, 130, 67, 128),
                                         (torch.float32, 1024, 768, 1024)])
def test_epilogue_scales(pkg, oracle, dtype, M, N, K):
    """Per-channel and per-token factors in the epilogue (b200ht_fused_gemm_scaled): every store path of the
    tensor-core kernel (both layouts, both output types, whole and ragged tiles, the two-launch form, K < 64), the
    FFMA path and the fp32 tensor-core path, each factor alone and both, with and without the sign diagonal."""
    inp = oracle.make_inputs("c3", K=K, N=N, M=M)
    X, W = inp["X"].to(dtype), inp["W"].to(dtype)
    g = torch.Generator().manual_seed(3)
    rs = torch.rand(M, generator=g) + 0.5
    ts = torch.rand(N, generator=g) * 2 - 1
    base = oracle.fused_gemm_ref(X.double().numpy(), W.double().numpy())
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    Xd, Wd = X.cuda(), W.cuda()
    for r, t in ((rs, ts), (rs, None), (None, ts)):
        ref = base * (r.double().numpy()[:, None] if r is not None else 1.0) * (t.double().numpy()[None, :] if t is not None else 1.0)
        for layout in ("mn", "nm"):
            for od in (torch.float32, torch.bfloat16):
                C = pkg.fused_ht_gemm(Xd, Wd, out_layout=layout, out_dtype=od, row_scale=r, token_scale=t)
                got = C.float().cpu().numpy()
                _check(oracle, got if layout == "mn" else got.T, ref, tol if od == torch.float32 else max(tol, 1e-2))
    if dtype == torch.bfloat16:
        d = torch.where(torch.rand(K, generator=g) < 0.5, -1.0, 1.0)
        ref = oracle.fused_gemm_ref((X.double() * d.double()).numpy(), W.double().numpy()) * rs.double().numpy()[:, None]
        C = pkg.fused_ht_gemm(Xd, Wd, signs=d, row_scale=rs)
        _check(oracle, C.cpu().numpy(), ref, tol)
    else:
        Ce = pkg.fused_ht_gemm(Xd, Wd, exact=True, row_scale=rs, token_scale=ts)
        _check(oracle, Ce.cpu().numpy(), base * rs.double().numpy()[:, None] * ts.double().numpy()[None, :], tol)
    assert pkg.device_status() == 0


@pytest.mark.parametrize("M,N,B", [(6000, 4096, 24), (77, 4096, 40), (500, 8192, 20), (333, 2048, 70), (100, 512, 50)])
def test_gemv_c_abi_with_more_columns_than_fit_in_shared_memory(pkg, oracle, M, N, B):
    """Straight through the C ABI with more columns than b200ht_fused_gemv_max_batch: the entry serves them in column
    groups (W is then streamed once per group; the Python wrapper would send such a batch to the fused GEMM)."""
    lib = pkg._lib.load()
    assert 0 < lib.b200ht_fused_gemv_max_batch(N, pkg._lib.BF16) < B
    g = torch.Generator().manual_seed(2000 + M + N + B)
    W = (torch.randn(M, N, generator=g) / N ** 0.5).bfloat16().cuda()
    X = torch.randn(N, B, generator=g).bfloat16().cuda()
    Y = torch.empty(M, B, dtype=torch.float32, device="cuda")
    rc = lib.b200ht_fused_gemv(W.data_ptr(), X.data_ptr(), Y.data_ptr(), M, N, B, pkg._lib.BF16, pkg._lib.F32,
                               float(N ** -0.5), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, pkg._lib.error_string(rc)
    assert pkg.device_status() == 0
    ref = oracle.fused_gemv_ref(W.double().cpu().numpy(), X.double().cpu().numpy())
    _check(oracle, Y.cpu().numpy(), ref, BF16_TOL)


def test_gemv_max_batch_table(pkg):
    lib = pkg._lib.load()
    got = {n: lib.b200ht_fused_gemv_max_batch(n, pkg._lib.BF16) for n in (128, 256, 1024, 2048, 4096, 8192, 16384)}
    assert got == {128: 0, 256: 32, 1024: 32, 2048: 24, 4096: 16, 8192: 8, 16384: 0}
    assert lib.b200ht_fused_gemv_max_batch(4096, pkg._lib.F32) == 0


def test_gemv_tcgen05_kernel_agrees_with_the_oracle():
    """The tcgen05 GEMV kernel (B200HT_GEMV_TCGEN05=1, read once per process) in a child process: every copy-in
    variant of X, 8 / 16 / 32 / 64 operand rows, one and several row groups per CTA, ragged last rows, column
    groups, both output types."""
    import os
    import subprocess
    import sys
    import textwrap
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    code = textwrap.dedent(f"""
        import importlib, sys
        sys.path.insert(0, {str(root)!r})
        import torch
        pkg = importlib.import_module("6s894_project_2025_b200")
        oracle = importlib.import_module("oracle.fwht_oracle")
        lib = pkg._lib.load()
        g = torch.Generator().manual_seed(5)
        shapes = ((4096, 4096, 4), (300, 1024, 8), (1000, 8192, 8), (4096, 4096, 16), (4096, 256, 2), (4741, 512, 12),
                  (10000, 256, 1), (9000, 4096, 16), (8, 8192, 4), (29, 1024, 32), (333, 1024, 64), (77, 4096, 40),
                  (28672, 8192, 3))
        for M, N, B in shapes:
            W = (torch.randn(M, N, generator=g) / N ** 0.5).bfloat16()
            X = torch.randn(N, B, generator=g).bfloat16()
            ref = oracle.fused_gemv_ref(W.double().numpy(), X.double().numpy())
            Wd, Xd = W.cuda(), X.cuda()
            for odt, code in ((torch.float32, pkg._lib.F32), (torch.bfloat16, pkg._lib.BF16)):
                Y = torch.empty(M, B, dtype=odt, device="cuda")
                rc = lib.b200ht_fused_gemv(Wd.data_ptr(), Xd.data_ptr(), Y.data_ptr(), M, N, B, pkg._lib.BF16, code,
                                           float(N ** -0.5), torch.cuda.current_stream().cuda_stream)
                assert rc == 0, (M, N, B, rc)
                got = Y.float().cpu().numpy()
                assert oracle.rel_fro(got, ref) <= 2e-2 and oracle.rel_max(got, ref) <= 2e-2, (M, N, B)
        assert pkg.device_status() == 0
        print("ok")
    """)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, B200HT_GEMV_TCGEN05="1"))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("env", [{"B200HT_GEMM_CHUNK_MB": "1"}, {"B200HT_GEMM_ORDER": "1", "B200HT_GEMM_GROUP": "3"},
                                 {"B200HT_GEMM_ORDER": "0", "B200HT_GEMM_GROUP": "5", "B200HT_GEMM_CHUNK_MB": "2"},
                                 {"B200HT_GEMM_SPLIT": "0", "B200HT_GEMM_CHUNK_MB": "0"}])
def test_fused_gemm_chunking_and_tile_orders_agree_bit_for_bit(pkg, oracle, tmp_path, env):
    """The token range is processed in L2-sized chunks, the tiles of the contraction are visited in groups along rows
    or tokens, and a partial last wave of 256-row tiles is recomputed as 128-row tiles by a second launch.  None of
    that may change a single bit: every output element is the same K-ordered sum whatever tile holds it.  A child
    process runs the library with the knobs set (they are read once per process) on shapes with ragged edges, more
    than one wave and both rectangle forms of the split; the parent compares with its own default-configuration
    result over the FULL matrix and checks that against the oracle."""
    import os
    import subprocess
    import sys
    import textwrap
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    shapes = [(4096, 2560, 64, "nm"), (2900, 3333, 512, "mn"), (6400, 6144, 128, "nm"), (9000, 5000, 64, "mn")]
    code = textwrap.dedent(f"""
        import importlib, sys
        sys.path.insert(0, {str(root)!r})
        import torch
        pkg = importlib.import_module("6s894_project_2025_b200")
        for i, (M, N, K, layout) in enumerate({shapes!r}):
            g = torch.Generator().manual_seed(77 + i)
            X = torch.randn(N, K, generator=g).bfloat16().cuda()
            W = torch.randn(M, K, generator=g).bfloat16().cuda()
            rs = torch.rand(M, generator=g).cuda() + 0.5
            ts = torch.rand(N, generator=g).cuda() + 0.5
            C = pkg.fused_ht_gemm(X, W, out_layout=layout, out_dtype=torch.bfloat16, row_scale=rs, token_scale=ts)
            C2 = pkg.fused_ht_gemm(X, W, out_layout=layout)     # twice in a row on the stream, fp32 out
            torch.save((C.cpu(), C2.cpu()), {str(tmp_path)!r} + f"/c{{i}}.pt")
        assert pkg.device_status() == 0
        print("ok")
    """)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, **env))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
    for i, (M, N, K, layout) in enumerate(shapes):
        g = torch.Generator().manual_seed(77 + i)
        X = torch.randn(N, K, generator=g).bfloat16()
        W = torch.randn(M, K, generator=g).bfloat16()
        rs = torch.rand(M, generator=g) + 0.5
        ts = torch.rand(N, generator=g) + 0.5
        C = pkg.fused_ht_gemm(X.cuda(), W.cuda(), out_layout=layout, out_dtype=torch.bfloat16, row_scale=rs.cuda(),
                              token_scale=ts.cuda()).cpu()
        C2 = pkg.fused_ht_gemm(X.cuda(), W.cuda(), out_layout=layout).cpu()
        Cc, C2c = torch.load(tmp_path / f"c{i}.pt")
        assert torch.equal(C, Cc) and torch.equal(C2, C2c), (env, M, N, K, layout)
        ref = oracle.fused_gemm_ref(X.double().numpy(), W.double().numpy())
        got = C2.double().numpy() if layout == "mn" else C2.double().numpy().T
        assert oracle.rel_fro(got, ref) <= BF16_TOL
    assert pkg.device_status() == 0
