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
