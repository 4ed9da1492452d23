"""Partitioning of independent sequences across GPUs (one process per GPU, no data-path collective).

Batched decode of independent sequences has no cross-sequence arithmetic, so a job of ``n`` sequences
on ``world`` ranks is ``world`` independent engines, each decoding a contiguous slice.  Results are gathered
on the host (``torch.distributed`` object/tensor gather) only to report them.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np


def shard_range(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced slice [begin, end) of ``n_items`` owned by ``rank`` (earlier ranks take the remainder)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank/world out of range")
    base, rem = divmod(n_items, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_rows(array: np.ndarray, rank: int, world: int) -> np.ndarray:
    b, e = shard_range(array.shape[0], rank, world)
    return array[b:e]


def gather_token_streams(local: Sequence[np.ndarray], n_total: int, rank: int, world: int, max_tokens: int):
    """Gather per-sequence token streams on rank 0 (gloo or nccl); returns the list on rank 0, else None."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return list(local)
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    counts = [shard_range(n_total, r, world) for r in range(world)]
    width = max_tokens + 1
    per = max(e - b for b, e in counts)
    buf = torch.full((per, width), -1, dtype=torch.int64, device=device)
    for i, t in enumerate(local):
        buf[i, 0] = len(t)
        if len(t):
            buf[i, 1:1 + len(t)] = torch.as_tensor(np.asarray(t, dtype=np.int64), device=device)
    gathered = [torch.empty_like(buf) for _ in range(world)] if rank == 0 else None
    dist.gather(buf, gathered, dst=0)
    if rank != 0:
        return None
    out = []
    for r, (b, e) in enumerate(counts):
        g = gathered[r].cpu().numpy()
        for i in range(e - b):
            n = int(g[i, 0])
            out.append(g[i, 1:1 + n].astype(np.uint32))
    return out


# ---- tensor parallelism: which slice of each tensor a rank holds -------------------------------------------------

_ROW_SPLIT = ("wq", "wk", "wv", "w1", "w3", "lm_head", "bq", "bk", "bv", "b1")   # split along the output dimension
_COL_SPLIT = ("wo", "w2")                                                          # split along the input dimension


def tp_shard(name: str, tensor, rank: int, world: int):
    """Megatron shard of one tensor for ``rank`` of ``world`` (works on numpy arrays and torch tensors).

    Matrices whose rows are per-head or per-hidden-unit outputs (wq, wk, wv, w1, w3, lm_head and their biases) are
    split by rows; wo and w2 consume those outputs and are split by columns; embeddings, norm gains and the
    output-side biases (bo, b2: added once, by rank 0) stay whole."""
    if world <= 1:
        return tensor
    leaf = name.rsplit("/", 1)[-1]
    if leaf in _ROW_SPLIT:
        b, e = shard_range(tensor.shape[0], rank, world)
        if tensor.shape[0] % world:
            raise ValueError(f"{name}: {tensor.shape[0]} rows do not divide by {world}")
        return tensor[b:e]
    if leaf in _COL_SPLIT:
        if tensor.shape[1] % world:
            raise ValueError(f"{name}: {tensor.shape[1]} columns do not divide by {world}")
        b, e = shard_range(tensor.shape[1], rank, world)
        return tensor[:, b:e]
    return tensor
