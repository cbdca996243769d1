"""torch.library registration: dispatcher ops, fake-tensor shapes (CPU), and on the GPU opcheck, autograd of
the transform and CUDA-graph capture/replay of all three operators."""
import math

import pytest
import torch


def test_ops_are_registered_with_fake_impls(pkg):
    assert hasattr(torch.ops.b200ht, "hadamard_transform")
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(3, 5, 256, dtype=torch.bfloat16, device="cuda")
        y = torch.ops.b200ht.hadamard_transform(x, 1.0 / 16)
        assert y.shape == x.shape and y.dtype == x.dtype
        X = torch.empty(100, 1024, dtype=torch.bfloat16, device="cuda")
        W = torch.empty(64, 1024, dtype=torch.bfloat16, device="cuda")
        assert torch.ops.b200ht.fused_ht_gemm(X, W, 1.0, True, True).shape == (100, 64)
        assert torch.ops.b200ht.fused_ht_gemm(X, W, 1.0, False, False).shape == (64, 100)
        assert torch.ops.b200ht.fused_ht_gemm(X, W, 1.0, False, False).dtype == torch.float32
        Xc = torch.empty(1024, 4, dtype=torch.bfloat16, device="cuda")
        assert torch.ops.b200ht.fused_ht_gemv(W, Xc, 1.0, False).shape == (64, 4)


@pytest.mark.gpu
def test_opcheck_and_autograd(pkg, oracle):
    x = torch.randn(4, 512, device="cuda").bfloat16()
    torch.library.opcheck(torch.ops.b200ht.hadamard_transform, (x, 512 ** -0.5),
                          test_utils=("test_schema", "test_faketensor"))
    # H is symmetric and (with scale 1/sqrt(n)) orthogonal: d/dx sum(H(x) * g) = H(g)
    xr = torch.randn(3, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(3, 256, device="cuda", dtype=torch.bfloat16)
    y = torch.ops.b200ht.hadamard_transform(xr, 1.0 / 16)
    y.backward(g)
    ref = oracle.fwht_rows(g.double().cpu().numpy())
    assert abs(xr.grad.double().cpu().numpy() - ref).max() <= 5e-2


@pytest.mark.gpu
def test_cuda_graph_capture_and_replay(pkg):
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(64, 4096, generator=g, device="cuda").bfloat16()
    X = torch.randn(512, 1024, generator=g, device="cuda").bfloat16()
    W = torch.randn(256, 1024, generator=g, device="cuda").bfloat16()
    Wv = (torch.randn(512, 4096, generator=g, device="cuda") / 64).bfloat16()
    Xv = torch.randn(4096, 4, generator=g, device="cuda").bfloat16()
    expect = (pkg.hadamard_transform(x), pkg.fused_ht_gemm(X, W), pkg.fused_ht_gemv(Wv, Xv))
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            got = (pkg.hadamard_transform(x), pkg.fused_ht_gemm(X, W), pkg.fused_ht_gemv(Wv, Xv))
        for _ in range(3):
            graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(got, expect):
        assert torch.equal(a, b)
    assert pkg.device_status() == 0


@pytest.mark.gpu
def test_cuda_graph_with_the_two_launch_gemm(pkg):
    """A shape whose 256-row tiles leave a partial wave (16 x 10 = 160 tiles on 148 SMs): the contraction is two
    launches tied together by programmatic dependencies.  Captured in a graph and replayed, with the transform in
    front and another call behind, it must give the eager result bit for bit."""
    g = torch.Generator(device="cuda").manual_seed(6)
    X = torch.randn(2560, 64, generator=g, device="cuda").bfloat16()
    W = torch.randn(4096, 64, generator=g, device="cuda").bfloat16()
    expect = pkg.fused_ht_gemm(X, W, out_layout="nm", out_dtype=torch.bfloat16)
    expect2 = pkg.fused_ht_gemm(X, W)
    ref = (W.float() @ pkg.hadamard_transform(X).float().t())
    assert float((expect2 - ref).norm() / ref.norm()) < 2e-2
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            got = pkg.fused_ht_gemm(X, W, out_layout="nm", out_dtype=torch.bfloat16)
            got2 = pkg.fused_ht_gemm(X, W)
        for _ in range(3):
            graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, expect) and torch.equal(got2, expect2)
    assert pkg.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_torch_compile_fullgraph_matches_eager(pkg, backend):
    """A module whose forward calls the three registered operators compiles with fullgraph=True (no graph break at
    the custom ops: the fake-tensor functions give the compiler their shapes) and returns what eager returns, bit
    for bit; the backward of the compiled transform is the transform of the incoming gradient."""

    class Block(torch.nn.Module):
        def __init__(self, W, Wv):
            super().__init__()
            self.W = torch.nn.Parameter(W, requires_grad=False)
            self.Wv = torch.nn.Parameter(Wv, requires_grad=False)

        def forward(self, x, X, Xv):
            y = torch.ops.b200ht.hadamard_transform(x, x.shape[-1] ** -0.5)
            c = torch.ops.b200ht.fused_ht_gemm(X, self.W, X.shape[-1] ** -0.5, True, True)
            v = torch.ops.b200ht.fused_ht_gemv(self.Wv, Xv, Xv.shape[0] ** -0.5, False)
            return y * 2, c, v + 1

    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(32, 1024, generator=g, device="cuda").bfloat16()
    X = torch.randn(300, 512, generator=g, device="cuda").bfloat16()
    W = torch.randn(192, 512, generator=g, device="cuda").bfloat16()
    Wv = (torch.randn(256, 2048, generator=g, device="cuda") / 45).bfloat16()
    Xv = torch.randn(2048, 4, generator=g, device="cuda").bfloat16()
    mod = Block(W, Wv)
    eager = mod(x, X, Xv)
    torch._dynamo.reset()
    compiled = torch.compile(mod, fullgraph=True, backend=backend)
    got = compiled(x, X, Xv)
    for a, b in zip(got, eager):
        assert a.shape == b.shape and a.dtype == b.dtype
        assert torch.equal(a, b)

    # backward through the compiled transform
    def f(t):
        return torch.ops.b200ht.hadamard_transform(t, 1.0 / 16).float().square().sum()

    t0 = torch.randn(8, 256, generator=g, device="cuda").bfloat16()
    te = t0.clone().requires_grad_(True)
    f(te).backward()
    tc = t0.clone().requires_grad_(True)
    torch.compile(f, fullgraph=True, backend=backend)(tc).backward()
    assert torch.allclose(tc.grad.float(), te.grad.float(), atol=2e-2, rtol=2e-2)
    assert pkg.device_status() == 0
