"""Token sharding of W . H(X) across the GPUs of one node.

Every token (row of the (N, K) matrix X) is transformed and multiplied
independently and W is read-only, so the work splits by tokens with W
replicated and no collective on the data path.  The only exchange is the
optional assembly of the full result, which the caller times separately.
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
    if len({b - a for a, b in sizes}) == 1:
        full = torch.empty((n_tokens, M), dtype=local_nm.dtype, device=local_nm.device)
        dist.all_gather_into_tensor(full, local_nm.contiguous(), group=group)
    else:
        parts = [torch.empty((b - a, M), dtype=local_nm.dtype, device=local_nm.device) for a, b in sizes]
        dist.all_gather(parts, local_nm.contiguous(), group=group)
        full = torch.cat(parts, dim=0)
    return full if out_layout == "nm" else full.t().contiguous()
