"""Sharding of W . H(X) across the GPUs of one node.

Large batches split by tokens: every token (row of the (N, K) matrix X) is
transformed and multiplied independently and W is read-only, so W is
replicated and there is no collective on the data path; the only exchange is
the optional assembly of the full result, which the caller times separately.

Small batches (the GEMV, B <= 64) cannot split by tokens; they split by ROWS
of W instead: every rank keeps M/world rows of W, transforms the same small X
and produces its rows of Y, and one all-gather of M x B values assembles Y.
The reference is single-GPU; this module has no counterpart there.
"""
from __future__ import annotations

import torch


def token_range(n_tokens: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of token rows owned by ``rank``: equal contiguous blocks,
    the first ``n_tokens % world`` ranks take one extra row."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n_tokens, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_tokens(X: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's rows of the token-major (N, K) matrix (a view, no copy)."""
    a, b = token_range(int(X.shape[0]), rank, world)
    return X[a:b]


def gather_result(C_local: torch.Tensor, n_tokens: int, out_layout: str = "nm", group=None) -> torch.Tensor:
    """Assemble the full result on every rank from the per-rank blocks.

    ``out_layout="nm"`` (token-major, (N, M)): blocks are contiguous row ranges,
    one ``all_gather``.  ``"mn"`` ((M, N), the reference layout): blocks are
    column ranges; they are gathered token-major and transposed back.  With
    NCCL the transfer runs over NVLink; with gloo (CPU tests) over sockets.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if out_layout not in ("nm", "mn"):
        raise ValueError("out_layout must be 'nm' or 'mn'")
    local_nm = C_local if out_layout == "nm" else C_local.t().contiguous()
    M = int(local_nm.shape[1])
    sizes = [token_range(n_tokens, r, world) for r in range(world)]
    full = _gather_row_blocks(local_nm.contiguous(), sizes, group)
    return full if out_layout == "nm" else full.t().contiguous()


def _gather_row_blocks(local: torch.Tensor, sizes, group) -> torch.Tensor:
    """All-gather of per-rank row blocks ``sizes[r] = (start, stop)``.  Collectives need equal shapes on every
    rank, so uneven blocks are padded to the largest one and trimmed after the exchange."""
    import torch.distributed as dist

    world = len(sizes)
    total = sizes[-1][1]
    cols = int(local.shape[1])
    if len({b - a for a, b in sizes}) == 1:
        full = torch.empty((total, cols), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(full, local, group=group)
        return full
    big = max(b - a for a, b in sizes)
    padded = torch.zeros((big, cols), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    buf = torch.empty((world * big, cols), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    return torch.cat([buf[r * big: r * big + (b - a)] for r, (a, b) in enumerate(sizes)], dim=0)


def row_range(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of rows of W owned by ``rank`` (same split rule as ``token_range``)."""
    return token_range(n_rows, rank, world)


def shard_rows(W: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's rows of the (M, N) matrix W (a view, no copy)."""
    a, b = row_range(int(W.shape[0]), rank, world)
    return W[a:b]


def gather_rows(Y_local: torch.Tensor, n_rows: int, group=None) -> torch.Tensor:
    """Assemble the (M, B) result of a row-sharded GEMV on every rank: one all-gather of the per-rank row blocks
    (M x B values in total; NCCL over NVLink, gloo in CPU tests)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [row_range(n_rows, r, world) for r in range(world)]
    return _gather_row_blocks(Y_local.contiguous(), sizes, group)


class RowShardedGemv:
    """Small-batch ``Y = W . H(X)`` with the rows of W split over the ranks of one node, the exchange done by the
    kernel's own stores.

    Every rank keeps ``shard_rows(W)`` and the same X.  The GEMV kernel writes its rows of Y into its own result
    buffer and sends every value, together with the number of the call, as one 8-byte store into a slot array on
    each other rank (peer-mapped pointers); its CTAs then collect the other ranks' rows from the local slot array,
    waiting for each slot's tag (``b200ht_fused_gemv_peers``).  There is no collective, no fence and no flag on the
    path: at W 4096 x 4096 an NCCL all-gather of the 64 KB result costs several times the kernel.

    Set-up (once): each rank allocates one exchange buffer -- two result buffers and two slot arrays used
    alternately, plus the kernel's counter word -- exports it (CUDA IPC), the handles go round with
    ``all_gather_object`` and every rank maps the others'.
    ``__call__`` returns a view of the result buffer of this call; it stays valid until the call after next.  All
    ranks must make the same sequence of calls.  bf16, 256 <= N <= 8192, B <= ``max_batch``.

    The kernel counts the calls of an exchange on the device, so no argument changes from one call to the next and
    a CUDA graph can replay calls (which takes the host's launch pace and jitter, the larger part of a call's time
    on 4 and 8 GPUs, out of the loop).  A captured graph must hold an even number of calls of each op: the two
    result buffers and slot arrays alternate.
    """

    def __init__(self, W_local: torch.Tensor, n_rows: int, max_batch: int, *, out_dtype: torch.dtype = torch.float32,
                 group=None, backend=None):
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.W = W_local.contiguous()
        self.n_rows = int(n_rows)
        self.N = int(W_local.shape[1])
        self.max_batch = int(max_batch)
        self.out_dtype = out_dtype
        self.row_begin, self.row_end = row_range(self.n_rows, self.rank, self.world)
        if int(W_local.shape[0]) != self.row_end - self.row_begin:
            raise RuntimeError("RowShardedGemv: W_local does not hold this rank's rows (see shard_rows)")
        self.calls = 0
        self._plans = {}
        esz = 4 if out_dtype == torch.float32 else 2
        self.y_bytes = (self.n_rows * self.max_batch * esz + 255) & ~255
        self.slot_bytes = (self.n_rows * self.max_batch * 8 + 255) & ~255
        self.backend = backend if backend is not None else _IpcBackend(W_local.device)
        # exchange buffer (zeroed): [counter word: 256 bytes][result 0][result 1][slot array 0][slot array 1]
        self.buf = self.backend.allocate(256 + 2 * self.y_bytes + 2 * self.slot_bytes)
        handle = self.backend.export(self.buf)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        # base address of every rank's exchange buffer as seen from this GPU (own buffer: its own address)
        self.bases = [self.backend.address(self.buf) if r == self.rank else self.backend.open(handles[r])
                      for r in range(self.world)]
        self.peers = [r for r in range(self.world) if r != self.rank]
        dist.barrier(group=group)   # every rank has zeroed and mapped its buffers before the first call

    # layout of the exchange buffer
    def _local_count(self, base: int) -> int:
        return base + 128                      # kernel scratch word, then the kernel's count of calls
    def _result(self, base: int, parity: int) -> int:
        return base + 256 + parity * self.y_bytes
    def _slots(self, base: int, parity: int) -> int:
        return base + 256 + 2 * self.y_bytes + parity * self.slot_bytes

    def plan(self, batch: int) -> dict:
        """Addresses and number of the NEXT call (also what the host-side tests check)."""
        if not (1 <= batch <= self.max_batch):
            raise RuntimeError(f"RowShardedGemv: batch must be in [1, {self.max_batch}]")
        parity = self.calls & 1
        p = self._plans.get(parity)
        if p is None:
            mine = self.bases[self.rank]
            p = {
                "parity": parity,
                "y_full": self._result(mine, parity),
                "my_slots": self._slots(mine, parity),
                "peer_slots": [self._slots(self.bases[r], parity) for r in self.peers],
                "local_count": self._local_count(mine),
                "views": {},
            }
            self._plans[parity] = p
        p["call"] = self.calls + 1      # the tag of this call's values (the kernel keeps its own count)
        return p

    def __call__(self, X: torch.Tensor, *, scale: float | None = None) -> torch.Tensor:
        if X.dim() == 1:
            X = X[:, None]
        batch = int(X.shape[1])
        p = self.plan(batch)
        if not X.is_contiguous():
            X = X.contiguous()
        self.backend.launch(self, X, batch, p, scale)
        self.calls += 1
        y = p["views"].get(batch)
        if y is None:
            y = self.backend.view(self.buf, p["y_full"] - self.bases[self.rank], (self.n_rows, batch), self.out_dtype)
            p["views"][batch] = y
        return y

    def close(self) -> None:
        for r in self.peers:
            self.backend.close(self.bases[r])
        self.peers = []


class _IpcBackend:
    """CUDA side of RowShardedGemv: device buffers through torch, mapping through the library's IPC wrappers."""

    def __init__(self, device):
        from . import _lib
        self.device = device
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self._lib = _lib
        self.lib = _lib.load()
        self._opened = {}
        self._args = {}
        # the current stream's handle, by the shortest route torch offers (the call is short enough for this to show)
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (
            lambda index: torch.cuda.current_stream(index).cuda_stream)

    def allocate(self, nbytes: int) -> torch.Tensor:
        # a private cudaMalloc block (IPC handles cover whole allocations): bypass the caching allocator's pooling
        # by asking for a block larger than its small-allocation pools hand out piecemeal
        t = torch.zeros(max(nbytes, 2 << 20), dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize(self.device)
        return t

    def address(self, buf: torch.Tensor) -> int:
        return int(buf.data_ptr())

    def export(self, buf: torch.Tensor):
        import ctypes
        h = ctypes.create_string_buffer(64)
        off = ctypes.c_ulonglong(0)
        with torch.cuda.device(self.device):
            self._lib.check(self.lib.b200ht_ipc_export(buf.data_ptr(), h, ctypes.byref(off)), "b200ht_ipc_export")
        return (bytes(h.raw), int(off.value))

    def open(self, handle) -> int:
        import ctypes
        raw, off = handle
        base = ctypes.c_void_p(0)
        with torch.cuda.device(self.device):
            self._lib.check(self.lib.b200ht_ipc_open(raw, ctypes.byref(base)), "b200ht_ipc_open")
        self._opened[int(base.value) + off] = int(base.value)
        return int(base.value) + off

    def close(self, addr: int) -> None:
        base = self._opened.pop(addr, None)
        if base is not None:
            self.lib.b200ht_ipc_close(base)

    def launch(self, op: "RowShardedGemv", X: torch.Tensor, batch: int, p: dict, scale) -> None:
        import ctypes
        import math
        # the pointer array of a parity never changes: build it once
        key = (id(op), p["parity"])
        args = self._args.get(key)
        if args is None:
            n = len(p["peer_slots"])
            vp = ctypes.c_void_p
            dt = {torch.float32: self._lib.F32, torch.bfloat16: self._lib.BF16}
            args = ((vp * max(n, 1))(*p["peer_slots"]), n, dt[op.W.dtype], dt[op.out_dtype], math.sqrt(1.0 / op.N),
                    op.W.data_ptr())
            self._args[key] = args
        peer_slots, n, in_dt, out_dt, default_scale, w_ptr = args
        sc = default_scale if scale is None else scale

        def enqueue():
            return self.lib.b200ht_fused_gemv_peers(
                w_ptr, X.data_ptr(), p["y_full"], op.row_end - op.row_begin, op.N, batch, in_dt, out_dt,
                float(sc), op.row_begin, op.n_rows, n, peer_slots, p["my_slots"], p["local_count"],
                0, self._raw_stream(self.index))   # 0: calls counted on the device

        # (switching the device costs more host time than the call; one process per GPU is already on it)
        if torch.cuda.current_device() == self.index:
            rc = enqueue()
        else:
            with torch.cuda.device(self.device):
                rc = enqueue()
        if rc:
            self._lib.check(rc, "b200ht_fused_gemv_peers")

    def view(self, buf: torch.Tensor, offset: int, shape, dtype) -> torch.Tensor:
        n = shape[0] * shape[1] * (4 if dtype == torch.float32 else 2)
        return buf[offset: offset + n].view(dtype).view(shape)
