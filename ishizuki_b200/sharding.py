"""N-sharding of a projection across the GPUs of one node.

A projection's output rows are independent: GGUF rows are self-contained runs of blocks and an
affine row carries its own scales and biases, so rank r of G simply holds rows
[r*N/G, (r+1)*N/G) of the weight (the only precedent in the reference is
PackedLinear.channels(from:), Sources/IshizukiKit/Core/Hadamard.swift:254-262). Activations are
replicated; every rank computes its rows transposed, y^T [N/G, M], so that its slab is contiguous,
and one all-gather per projection assembles y^T [N, M]. No other collective is involved.

The shard arithmetic and the gather are plain torch.distributed and run on CPU (gloo) as well as
on GPUs (nccl); the local product is the C-ABI library on GPUs.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

GGML_TYPE_SIZE = {12: 144, 14: 210, 17: 74}


def row_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of an N-row projection held by `rank`: contiguous, sizes differing by at most one."""
    return rank * n // world, (rank + 1) * n // world


def shard_ggml(blocks: np.ndarray, type_id: int, n: int, k: int, rank: int, world: int) -> np.ndarray:
    """The byte range of raw GGUF blocks [n][k/256][type size] that holds this rank's rows."""
    row_bytes = (k // 256) * GGML_TYPE_SIZE[type_id]
    lo, hi = row_range(n, rank, world)
    flat = blocks.reshape(-1)
    assert flat.size >= n * row_bytes
    return flat[lo * row_bytes: hi * row_bytes]


def shard_affine(w: np.ndarray, scales: np.ndarray, biases: np.ndarray, rank: int, world: int):
    """Row slices of an affine pack's three arrays."""
    lo, hi = row_range(w.shape[0], rank, world)
    return w[lo:hi], scales[lo:hi], biases[lo:hi]


def gather_rows(y_local_t: torch.Tensor, n: int, group=None) -> torch.Tensor:
    """All-gathers the ranks' slabs y^T [N/G, M] into y^T [N, M] (one collective)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m = y_local_t.shape[1]
    lo, hi = row_range(n, rank, world)
    assert y_local_t.shape[0] == hi - lo
    out = torch.empty((n, m), dtype=y_local_t.dtype, device=y_local_t.device)
    if n % world == 0:
        dist.all_gather_into_tensor(out, y_local_t.contiguous(), group=group)
    else:  # uneven slabs: pad every slab to the largest, gather, then drop the padding
        cap = -(-n // world)
        padded = torch.zeros((cap, m), dtype=y_local_t.dtype, device=y_local_t.device)
        padded[: hi - lo] = y_local_t
        buf = torch.empty((world * cap, m), dtype=y_local_t.dtype, device=y_local_t.device)
        dist.all_gather_into_tensor(buf, padded, group=group)
        for r in range(world):
            a, b = row_range(n, r, world)
            out[a:b] = buf[r * cap: r * cap + (b - a)]
    return out


class ShardedLinear:
    """This rank's rows of a projection plus the gather: y = x . W^T for the whole projection."""

    def __init__(self, local, n: int, group=None):
        self.local = local  # an interface.PackedLinear over this rank's rows
        self.n = n
        self.group = group

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y_local_t = self.local(x, transposed=True)
        return gather_rows(y_local_t, self.n, self.group).t()
