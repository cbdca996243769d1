"""Out-of-bounds writes, checked without a sanitizer: every output (and workspace) of a call sits between two guard
zones filled with a known pattern; after the call the zones must be untouched.  Small, ragged shapes over every
kernel family, so that tail tiles, partial chunks and partial row groups are all exercised."""
import pytest
import torch

pytestmark = pytest.mark.gpu

GUARD = 4096          # bytes on each side
PATTERN = 0xA5


class Guarded:
    """A device buffer of `nbytes` bytes with guard zones on both sides."""

    def __init__(self, nbytes: int):
        self.nbytes = nbytes
        pad = (-nbytes) % 256
        self.raw = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device="cuda")
        self.pad = pad

    def ptr(self) -> int:
        return self.raw.data_ptr() + GUARD

    def view(self, dtype, shape):
        return self.raw[GUARD: GUARD + self.nbytes].view(dtype).view(shape)

    def intact(self) -> bool:
        tail = self.raw[GUARD + self.nbytes + self.pad:]
        return bool((self.raw[:GUARD] == PATTERN).all()) and bool((tail == PATTERN).all())


@pytest.mark.parametrize("n", [2, 8, 64, 256, 512, 2048, 4096, 8192, 16384, 32768])
@pytest.mark.parametrize("rows", [1, 3, 37])
def test_transform_writes_only_its_rows(pkg, lib, n, rows):
    l = lib.load()
    x = torch.randn(rows, n, device="cuda").bfloat16()
    out = Guarded(rows * n * 2)
    rc = l.b200ht_fwht(x.data_ptr(), out.ptr(), rows, n, lib.BF16, float(n ** -0.5), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    assert out.intact()
    assert torch.equal(out.view(torch.bfloat16, (rows, n)), pkg.hadamard_transform(x))


@pytest.mark.parametrize("M,N,K,layout,odt", [(130, 96, 512, 0, torch.float32), (384, 700, 1024, 1, torch.bfloat16),
                                               (4096, 2560, 64, 1, torch.bfloat16), (33, 77, 128, 0, torch.bfloat16),
                                               (1000, 1500, 256, 0, torch.float32), (5, 3, 32, 1, torch.float32)])
@pytest.mark.parametrize("idt", [torch.bfloat16, torch.float32])
def test_fused_gemm_writes_only_c_and_its_workspace(pkg, lib, M, N, K, layout, odt, idt):
    l = lib.load()
    dt = {torch.float32: lib.F32, torch.bfloat16: lib.BF16}
    X = torch.randn(N, K, device="cuda").to(idt)
    W = torch.randn(M, K, device="cuda").to(idt)
    esz = 4 if odt == torch.float32 else 2
    C = Guarded(M * N * esz)
    nws = int(l.b200ht_fused_gemm_tc_workspace_bytes(M, N, K, dt[idt]))
    ws = Guarded(nws)
    rc = l.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), C.ptr(), M, N, K, dt[idt], dt[odt], layout, float(K ** -0.5),
                             ws.ptr(), nws, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    assert C.intact() and ws.intact()
    assert l.b200ht_device_status(1) == 0


@pytest.mark.parametrize("M,N,B", [(29, 1024, 5), (300, 4096, 16), (4741, 512, 12), (8, 8192, 4), (100, 64, 3), (77, 32768, 2)])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_fused_gemv_writes_only_y(pkg, lib, M, N, B, odt):
    l = lib.load()
    W = (torch.randn(M, N, device="cuda") / N ** 0.5).bfloat16()
    X = torch.randn(N, B, device="cuda").bfloat16()
    Y = Guarded(M * B * (4 if odt == torch.float32 else 2))
    rc = l.b200ht_fused_gemv(W.data_ptr(), X.data_ptr(), Y.ptr(), M, N, B, lib.BF16,
                             lib.F32 if odt == torch.float32 else lib.BF16, float(N ** -0.5),
                             torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.error_string(rc)
    torch.cuda.synchronize()
    assert Y.intact()
    assert l.b200ht_device_status(1) == 0
