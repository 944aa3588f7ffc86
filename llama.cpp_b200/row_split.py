"""Row-split of weight matrices over ranks (one process per GPU): the host-side rules.

Mirrors the reference's split buffers (ggml/src/ggml-cuda/ggml-cuda.cu:714-1040): rank r of n holds the rows
[row_low, row_high) of every split matrix, where the boundaries are the equal-share cumulative fractions rounded
down to a multiple of 128 rows and the last rank takes the remainder (get_row_split, :725-742, with the MMQ tile
height get_mmq_y_host = 128 as the rounding, ggml/src/ggml-cuda/mmq.cuh:125-128).  A rank with an empty range
holds nothing of that matrix.  Whole tensors are scattered on upload and dst slices gathered after MUL_MAT
(:837-911, :1520-1660); on the GPUs the gather is done by the kernels themselves with stores into peer memory,
and torch.distributed only carries set-up data (IPC handles) and the benchmark's timing reductions.
"""
from __future__ import annotations

import numpy as np

ROUNDING = 128


def row_range(n_rows: int, rank: int, n_ranks: int) -> tuple[int, int]:
    """[row_low, row_high) of `rank`; the same arithmetic as b200_row_split_range in the C-ABI."""
    def bound(r: int) -> int:
        if r <= 0:
            return 0
        if r >= n_ranks:
            return n_rows
        b = n_rows * r // n_ranks
        return b - b % ROUNDING
    return bound(rank), bound(rank + 1)


def slice_rows(data: np.ndarray, full_rows: int, row_low: int, n_rows: int) -> np.ndarray:
    """The bytes of rows [row_low, row_low + n_rows) of a row-major tensor given as flat bytes."""
    data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    if data.size % full_rows:
        raise ValueError("tensor bytes are not a whole number of rows")
    rb = data.size // full_rows
    return data[row_low * rb:(row_low + n_rows) * rb]


def gather_bytes(dist):
    """A gather function for Llama.attach_peers built on an initialised torch.distributed process group."""
    def gather(mine: bytes) -> list[bytes]:
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, mine)
        return out
    return gather


def gather_rows(dist, local: np.ndarray, n_rows: int) -> np.ndarray:
    """All-gather of dst row slices: local is [n_cols, rows of this rank]; returns [n_cols, n_rows].

    The host-side statement of what the GPUs do with peer stores; used to check the split rules on CPU ranks."""
    import torch
    world, rank = dist.get_world_size(), dist.get_rank()
    lo, hi = row_range(n_rows, rank, world)
    local = np.ascontiguousarray(local, dtype=np.float32)
    if local.shape[-1] != hi - lo:
        raise ValueError(f"rank {rank} holds {local.shape[-1]} rows, expected {hi - lo}")
    n_cols = local.shape[0]
    width = max(row_range(n_rows, r, world)[1] - row_range(n_rows, r, world)[0] for r in range(world))
    pad = torch.zeros(n_cols, width, dtype=torch.float32)
    pad[:, :hi - lo] = torch.from_numpy(local)
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    out = np.empty((n_cols, n_rows), dtype=np.float32)
    for r in range(world):
        a, b = row_range(n_rows, r, world)
        out[:, a:b] = parts[r][:, :b - a].numpy()
    return out
