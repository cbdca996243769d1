"""Host-side operators: the reference's op boundary over the b200ht C ABI.

``hadamard_transform(x, inplace=False)`` keeps the name, arguments, defaults,
error messages and aliasing rules of the reference's pybind op
(csrc/hadamard_transform.cpp:12-92).  ``fused_ht_gemm`` and ``fused_ht_gemv``
give the reference's two fused kernels (fused_ht/fusion_pipelined.cu:306-310,
fused_ht/fwht_gemv_fusion.cu:98-105 — launched only from ``main()`` there) a
Python entry with the same argument order and memory layouts.

PyTorch is used for device memory, streams and the caching allocator only; all
arithmetic happens in libb200ht.so.  There is no CPU path: CPU tensors are
rejected exactly as the reference rejects them.
"""
from __future__ import annotations

import math

import torch

from . import _lib

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def _is_pow2(v: int) -> bool:
    return v > 0 and (v & (v - 1)) == 0


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def sign_mask(signs: torch.Tensor, n: int, device: torch.device) -> torch.Tensor:
    """+-1 diagonal (length n, any real dtype) -> the 16-bit sign-bit table the library takes
    (0x8000 where the entry is negative), padded to a whole 16-byte vector."""
    if signs.dim() != 1 or int(signs.shape[0]) != n:
        raise RuntimeError(f"signs must be a vector of length {n}")
    m = torch.where(signs.to(device) < 0, -32768, 0).to(torch.int16)
    if n < 8:
        m = torch.cat([m, m.new_zeros(8 - n)])
    return m.contiguous()


def hadamard_transform(x: torch.Tensor, inplace: bool = False, *, scale: float | None = None,
                       signs: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ H_n * scale`` along the last dimension, H_n in Sylvester order.

    Same contract as ``csrc.hadamard_transform`` (csrc/hadamard_transform.cpp:12-70):
    fp16/bf16 CUDA tensor of any shape whose last dimension n is a power of two
    <= 2**15; the result has the input's shape; with ``inplace=True`` the data
    of ``x`` is overwritten and ``x`` itself is returned, also when a temporary
    was needed.  ``scale`` defaults to the reference's ``1/sqrt(n)``.  Unlike
    the reference, any n >= 2 and any number of rows is accepted.  ``signs`` (a
    vector of n entries, negative = flip) applies a +-1 diagonal to the columns
    before the transform (randomised Hadamard transform) at no extra pass.
    """
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("Only fp16 and bf16 supported currently")
    if not x.is_cuda:
        raise RuntimeError("Expected in.is_cuda() to be true, but got false.")
    if x.dim() == 0:
        raise RuntimeError("Only power of two Hadamard sizes up to 2^15 are supported, got 1")
    n = int(x.shape[-1])
    if not _is_pow2(n) or n > (1 << 15) or n < 2:
        raise RuntimeError(f"Only power of two Hadamard sizes up to 2^15 are supported, got {n}")
    if scale is None:
        scale = math.sqrt(1.0 / n)

    lib = _lib.load()
    work = x
    if not work.is_contiguous() or work.data_ptr() % 16 != 0:
        work = x.contiguous()
        if work.data_ptr() % 16 != 0:  # contiguous view at an odd storage offset
            work = work.clone()
    out = work if inplace else torch.empty_like(work)
    rows = work.numel() // n
    if rows > 0:
        with torch.cuda.device(x.device):
            if signs is None:
                rc = lib.b200ht_fwht(work.data_ptr(), out.data_ptr(), rows, n, _DT[x.dtype], float(scale),
                                     _stream_ptr(x.device))
            else:
                mask = sign_mask(signs, n, x.device)
                rc = lib.b200ht_fwht_signed(work.data_ptr(), out.data_ptr(), rows, n, _DT[x.dtype], float(scale),
                                            mask.data_ptr(), _stream_ptr(x.device))
        _lib.check(rc, "b200ht_fwht")
    if inplace:
        if work is not x:
            x.copy_(out.view(x.shape))
        return x
    return out.view(x.shape)


def fused_gemm_workspace_bytes(M: int, N: int, K: int, dtype: torch.dtype, exact: bool = False) -> int:
    """Workspace size for ``fused_ht_gemm``.  For fp32 inputs the default size selects the tensor-core
    contraction (three bf16 terms per operand), ``exact=True`` the size of the FFMA path."""
    lib = _lib.load()
    fn = lib.b200ht_fused_gemm_workspace_bytes if exact else lib.b200ht_fused_gemm_tc_workspace_bytes
    return int(fn(M, N, K, _DT[dtype]))


def fused_ht_gemm(X: torch.Tensor, W: torch.Tensor, *, scale: float | None = None,
                  out_dtype: torch.dtype | None = None, out_layout: str = "mn",
                  out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                  signs: torch.Tensor | None = None, exact: bool = False,
                  row_scale: torch.Tensor | None = None, token_scale: torch.Tensor | None = None) -> torch.Tensor:
    """C = W . H(X): ``C[m, t] = sum_k W[m, k] * (scale * H_K x_t)[k]``.

    ``X`` is (N tokens, K) token-major and ``W`` is (M, K) row-major, the
    layouts of fused_ht/fusion_pipelined.cu:148-221; argument order X, W as in
    ``fused_ht_gemm_pipelined`` (:306-310).  Both fp32 (exact FFMA path) or
    both bf16 (tensor cores, fp32 accumulate).  ``out_layout="mn"`` returns the
    reference's (M, N) matrix, ``"nm"`` the token-major (N, M) one.  ``scale``
    defaults to 1/sqrt(K); the reference executable computes ``scale=1.0``.
    ``signs`` (K entries, negative = flip; bf16 inputs only) computes W . H(d * X).
    fp32 inputs on large shapes with K <= 4096 are contracted on the tensor
    cores as six bf16 products per fp32 product (relative error up to 4.4e-6
    at K = 4096, about 4x faster than FFMA);
    ``exact=True``, or a caller ``workspace`` of only the minimal size, keeps
    the FFMA kernel.  ``row_scale`` (M floats, per output channel) and
    ``token_scale`` (N floats, per token) multiply the fp32 accumulator in the
    epilogue, before the one rounding of the store.
    """
    if X.dtype != W.dtype or X.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("fused_ht_gemm: X and W must both be float32 or both bfloat16")
    if not (X.is_cuda and W.is_cuda):
        raise RuntimeError("fused_ht_gemm: X and W must be CUDA tensors")
    if X.dim() != 2 or W.dim() != 2 or X.shape[1] != W.shape[1]:
        raise RuntimeError("fused_ht_gemm: expected X (N, K) and W (M, K)")
    N, K = int(X.shape[0]), int(X.shape[1])
    M = int(W.shape[0])
    if not _is_pow2(K) or K < 2 or K > (1 << 15):
        raise RuntimeError(f"Only power of two Hadamard sizes up to 2^15 are supported, got {K}")
    if out_layout not in ("mn", "nm"):
        raise RuntimeError("fused_ht_gemm: out_layout must be 'mn' or 'nm'")
    if scale is None:
        scale = math.sqrt(1.0 / K)
    out_dtype = out_dtype or torch.float32
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("fused_ht_gemm: out_dtype must be float32 or bfloat16")
    lib = _lib.load()
    X = X.contiguous()
    W = W.contiguous()
    shape = (M, N) if out_layout == "mn" else (N, M)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=X.device)
    elif tuple(out.shape) != shape or out.dtype != out_dtype or not out.is_contiguous():
        raise RuntimeError("fused_ht_gemm: out has the wrong shape, dtype or strides")
    need = int(lib.b200ht_fused_gemm_workspace_bytes(M, N, K, _DT[X.dtype]))
    if workspace is None:
        want = need if exact else int(lib.b200ht_fused_gemm_tc_workspace_bytes(M, N, K, _DT[X.dtype]))
        workspace = torch.empty(max(want, 256), dtype=torch.uint8, device=X.device)
    elif workspace.numel() * workspace.element_size() < need:
        raise RuntimeError("fused_ht_gemm: workspace too small")
    if M > 0 and N > 0:
        with torch.cuda.device(X.device):
            layout = _lib.OUT_MN if out_layout == "mn" else _lib.OUT_NM
            wsb = need if exact else workspace.numel() * workspace.element_size()
            if row_scale is not None or token_scale is not None:
                def _vec(v, n, what):
                    if v is None:
                        return None
                    if v.dim() != 1 or int(v.shape[0]) != n:
                        raise RuntimeError(f"fused_ht_gemm: {what} must be a vector of length {n}")
                    return v.to(device=X.device, dtype=torch.float32).contiguous()
                rs, ts = _vec(row_scale, M, "row_scale"), _vec(token_scale, N, "token_scale")
                mask = sign_mask(signs, K, X.device) if signs is not None else None
                rc = lib.b200ht_fused_gemm_scaled(X.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, _DT[X.dtype],
                                                  _DT[out_dtype], layout, float(scale),
                                                  mask.data_ptr() if mask is not None else None,
                                                  rs.data_ptr() if rs is not None else None,
                                                  ts.data_ptr() if ts is not None else None,
                                                  workspace.data_ptr(), wsb, _stream_ptr(X.device))
            elif signs is None:
                rc = lib.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, _DT[X.dtype],
                                           _DT[out_dtype], layout, float(scale), workspace.data_ptr(), wsb,
                                           _stream_ptr(X.device))
            else:
                mask = sign_mask(signs, K, X.device)
                rc = lib.b200ht_fused_gemm_signed(X.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, _DT[X.dtype],
                                                  _DT[out_dtype], layout, float(scale), mask.data_ptr(),
                                                  workspace.data_ptr(), wsb, _stream_ptr(X.device))
        _lib.check(rc, "b200ht_fused_gemm")
    return out


class HostPipeline:
    """Host-to-host fused W . H(X) for token batches that live in (pinned) host memory.

    The tokens are cut into chunks; chunk i is copied in, multiplied and copied
    out on stream i % n_streams, so the copy engines (one per direction) and the
    SMs work on different chunks at the same time.  Device buffers are allocated
    once.  The reference has no counterpart (its programs copy everything in,
    run, copy everything out: fused_ht/fusion_pipelined.cu:626-704).
    """

    def __init__(self, W: torch.Tensor, max_tokens: int, *, chunk_tokens: int = 2048, n_streams: int = 3,
                 out_dtype: torch.dtype = torch.bfloat16, scale: float | None = None):
        if not W.is_cuda or W.dtype not in (torch.float32, torch.bfloat16):
            raise RuntimeError("HostPipeline: W must be a float32 or bfloat16 CUDA tensor")
        self.W = W.contiguous()
        self.M, self.K = int(W.shape[0]), int(W.shape[1])
        self.chunk = int(min(chunk_tokens, max(max_tokens, 1)))
        self.out_dtype = out_dtype
        self.scale = scale
        dev = W.device
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
        self.x = [torch.empty(self.chunk, self.K, dtype=W.dtype, device=dev) for _ in range(n_streams)]
        self.c = [torch.empty(self.chunk, self.M, dtype=out_dtype, device=dev) for _ in range(n_streams)]
        nbytes = fused_gemm_workspace_bytes(self.M, self.chunk, self.K, W.dtype)
        self.ws = [torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev) for _ in range(n_streams)]

    def __call__(self, X_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """``out_host[t, m] = (W . H(x_t))[m]`` (token-major).  Both tensors should be pinned; returns
        ``out_host`` after all chunks have been enqueued (synchronise before reading it)."""
        n = int(X_host.shape[0])
        if tuple(out_host.shape) != (n, self.M) or out_host.dtype != self.out_dtype:
            raise RuntimeError("HostPipeline: out_host has the wrong shape or dtype")
        cur = torch.cuda.current_stream(self.W.device)
        for st in self.streams:
            st.wait_stream(cur)
        for i, t0 in enumerate(range(0, n, self.chunk)):
            t1 = min(t0 + self.chunk, n)
            k = i % len(self.streams)
            with torch.cuda.stream(self.streams[k]):
                xd = self.x[k][: t1 - t0]
                cd = self.c[k][: t1 - t0]
                xd.copy_(X_host[t0:t1], non_blocking=True)
                fused_ht_gemm(xd, self.W, scale=self.scale, out_dtype=self.out_dtype, out_layout="nm", out=cd,
                              workspace=self.ws[k])
                out_host[t0:t1].copy_(cd, non_blocking=True)
        for st in self.streams:
            cur.wait_stream(st)
        return out_host


def fused_ht_gemv(W: torch.Tensor, X: torch.Tensor, *, scale: float | None = None,
                  out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Y = W . H(X) for a small batch: ``Y[m, b] = sum_k W[m, k] * (scale * H_N x_b)[k]``.

    ``W`` is (M, N) row-major, ``X`` is (N, B) with b fastest and the result is
    (M, B) with b fastest — the layouts and the argument order (W, X) of
    ``fused_hadamard_gemv_kernel`` (fused_ht/fwht_gemv_fusion.cu:98-159).
    ``scale`` defaults to 1/sqrt(N); the reference uses 1.0.  Built for small
    batches: when the transformed columns no longer fit in shared memory beside
    the stream of W (more than 16 columns at N = 4096, 64 at N <= 1024; the
    reference's benchmark goes up to 2048, :643-653) the call is served by the
    fused GEMM, which also reads W once.
    """
    if X.dtype != W.dtype or X.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("fused_ht_gemv: W and X must both be float32 or both bfloat16")
    if not (X.is_cuda and W.is_cuda):
        raise RuntimeError("fused_ht_gemv: W and X must be CUDA tensors")
    if X.dim() == 1:
        X = X[:, None]
    if X.dim() != 2 or W.dim() != 2 or X.shape[0] != W.shape[1]:
        raise RuntimeError("fused_ht_gemv: expected W (M, N) and X (N, B)")
    M, N = int(W.shape[0]), int(W.shape[1])
    B = int(X.shape[1])
    if not _is_pow2(N) or N < 2 or N > (1 << 15):
        raise RuntimeError(f"Only power of two Hadamard sizes up to 2^15 are supported, got {N}")
    if B < 1:
        raise RuntimeError(f"fused_ht_gemv: batch must be at least 1, got {B}")
    if scale is None:
        scale = math.sqrt(1.0 / N)
    out_dtype = out_dtype or torch.float32
    lib = _lib.load()
    once = int(lib.b200ht_fused_gemv_max_batch(N, _DT[W.dtype]))   # columns served by one pass over W
    if B > 64 or (once and B > once and N >= 64):
        return fused_ht_gemm(X.t().contiguous(), W, scale=scale, out_dtype=out_dtype, out_layout="mn", out=out)
    X = X.contiguous()
    W = W.contiguous()
    if out is None:
        out = torch.empty((M, B), dtype=out_dtype, device=W.device)
    elif tuple(out.shape) != (M, B) or out.dtype != out_dtype or not out.is_contiguous():
        raise RuntimeError("fused_ht_gemv: out has the wrong shape, dtype or strides")
    if M > 0:
        with torch.cuda.device(W.device):
            rc = lib.b200ht_fused_gemv(W.data_ptr(), X.data_ptr(), out.data_ptr(), M, N, B, _DT[W.dtype],
                                       _DT[out_dtype], float(scale), _stream_ptr(W.device))
        _lib.check(rc, "b200ht_fused_gemv")
    return out


def device_status(clear: bool = True) -> int:
    """0, or the error code a kernel left after a bounded wait expired."""
    return int(_lib.load().b200ht_device_status(1 if clear else 0))
