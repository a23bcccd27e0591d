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

GGML_TYPE_SIZE = {10: 84, 12: 144, 14: 210, 16: 66, 17: 74, 18: 98, 19: 50, 21: 110, 22: 82, 23: 136, 29: 56}


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


class NcclGroup:
    """The NCCL all-gather path of the C ABI (ishi_group_*): one communicator per process, created
    from an id that rank 0 draws and the host process group passes around."""

    def __init__(self, group=None, timeout_ms: int = 30000):
        import ctypes

        from . import _lib
        from .interface import IshizukiError

        self.lib = _lib.load()
        self._err = IshizukiError
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        blob = ctypes.create_string_buffer(_lib.GROUP_ID_BYTES)
        if self.rank == 0:
            rc = self.lib.ishi_group_unique_id(blob)
            if rc != 0:
                raise IshizukiError(rc, "ishi_group_unique_id failed")
        ids = [bytes(blob.raw)]
        if self.world > 1:
            dist.broadcast_object_list(ids, src=0, group=group)
        handle = ctypes.c_void_p()
        rc = self.lib.ishi_group_create(ctypes.create_string_buffer(ids[0], _lib.GROUP_ID_BYTES), self.rank, self.world,
                                        timeout_ms, ctypes.byref(handle))
        self.handle = handle
        if rc != 0:
            raise IshizukiError(rc, self.lib.ishi_group_last_error(handle).decode())

    def apply(self, local, x: torch.Tensor, y_all: torch.Tensor) -> None:
        """local: interface.PackedLinear over this rank's rows; y_all [world * n_local, rows] fp16."""
        import ctypes

        rc = self.lib.ishi_projection_apply_sharded(self.handle, local.handle, ctypes.c_void_p(x.data_ptr()), x.shape[0],
                                                    ctypes.c_void_p(y_all.data_ptr()),
                                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise self._err(rc, self.lib.ishi_group_last_error(self.handle).decode() or local.ctx.last_error())

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ishi_group_destroy(self.handle)
            self.handle = None


class _DeviceView:
    """A raw device range as something torch.as_tensor accepts (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class OutputExchange:
    """Outputs of N-sharded projections exchanged by the product kernels themselves over NVLink
    (ishi_exchange_* in the C ABI) instead of one all-gather per projection: every rank's kernel
    stores its rows into every rank's copy of the output and the ranks signal each other with
    arrival words, so a whole step has no collective and can be captured in one CUDA graph.

    The buffer holds fp16 arrays [rows of all shards][8] at offsets handed out by reserve();
    all ranks must reserve and apply in the same order. The handles are exchanged once over the
    (host) process group."""

    def __init__(self, nbytes: int, group=None, device: int | None = None):
        import ctypes

        from . import _lib
        from .interface import Context, IshizukiError

        self._err = IshizukiError
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.ctx = Context.get(torch.cuda.current_device() if device is None else device)
        self.lib = self.ctx.lib
        self.nbytes = int(nbytes)
        self.used = 0
        handle = ctypes.c_void_p()
        self._check(self.lib.ishi_exchange_create(self.ctx.handle, self.rank, self.world, self.nbytes, ctypes.byref(handle)))
        self.handle = handle
        if self.world > 1:
            blob = ctypes.create_string_buffer(_lib.EXCHANGE_HANDLE_BYTES)
            self._check(self.lib.ishi_exchange_export(self.handle, blob))
            blobs = [None] * self.world
            dist.all_gather_object(blobs, bytes(blob.raw), group=group)
            joined = ctypes.create_string_buffer(b"".join(blobs), _lib.EXCHANGE_HANDLE_BYTES * self.world)
            self._check(self.lib.ishi_exchange_connect(self.handle, joined))
            dist.barrier(group=group)
        base = self.lib.ishi_exchange_buffer(self.handle)
        self.buffer = torch.as_tensor(_DeviceView(base, self.nbytes), device=torch.device("cuda", self.ctx.device))

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise self._err(rc, self.ctx.last_error())

    def reserve(self, n_total: int, rows: int = 8) -> tuple[int, torch.Tensor]:
        """Room for one output [n_total, 8] fp16 ([n_total, 16] for calls with more than 8 drafted
        rows): its byte offset and a view of the local copy."""
        width = 16 if rows > 8 else 8
        off = self.used
        size = n_total * width * 2
        if off + size > self.nbytes:
            raise ValueError(f"exchange buffer of {self.nbytes} bytes is full")
        self.used = off + ((size + 255) & ~255)
        return off, self.buffer[off: off + size].view(torch.float16).view(n_total, width)

    def apply(self, local, x: torch.Tensor, offset: int, row_offset: int, wait_previous: bool = True) -> None:
        """local: interface.PackedLinear over this rank's rows; x [rows <= 16, K] fp16 on this GPU
        (more than 8 rows need an output reserved with rows > 8)."""
        import ctypes

        rows = x.shape[0]
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._check(self.lib.ishi_exchange_apply(self.handle, local.handle, ctypes.c_void_p(x.data_ptr()), rows, offset,
                                                 row_offset, 1 if wait_previous else 0, stream))

    def wait(self) -> None:
        """Enqueues, on the current stream, a wait for every rank's latest apply to have landed here."""
        import ctypes

        self._check(self.lib.ishi_exchange_wait(self.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def close(self, barrier: bool = True) -> None:
        """Disconnects from the peers, waits for every rank to have done so, then frees the buffer
        (a peer's last launch may still be storing into it until then). All ranks call it."""
        if getattr(self, "handle", None):
            self.lib.ishi_exchange_disconnect(self.handle)
            if barrier and self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            self.lib.ishi_exchange_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close(barrier=False)  # a finaliser cannot count on the other ranks
        except Exception:
            pass
