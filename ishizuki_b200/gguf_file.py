"""A GGUF file's header and tensor table, with the weight bytes left on disk: the host-side mirror
of the reference's GGUFFile (Sources/IshizukiKit/Config/GGUFFile.swift:179-397) over the C ABI
(ishi_gguf_*). Opening a file needs no GPU; `blocks()` uploads one tensor as GGUFBlocks."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib


class GGUFError(RuntimeError):
    """The file was refused (the reference throws BonsaiError.unsupportedModel / shapeMismatch)."""


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple[int, ...]  # row-major: a [5120, 248320] table in the file is 248320 rows of 5120
    type: int               # GGML type id
    offset: int             # relative to GGUFFile.dataOffset
    byteCount: int          # noqa: N815 (reference spelling)
    index: int

    @property
    def elementCount(self) -> int:  # noqa: N802
        return int(np.prod(self.shape))


class GGUFFile:
    magic = 0x46554747

    def __init__(self, path):
        self.lib = _lib.load()
        self.path = str(path)
        handle = ctypes.c_void_p()
        err = ctypes.create_string_buffer(512)
        rc = self.lib.ishi_gguf_open(self.path.encode(), ctypes.byref(handle), err, len(err))
        if rc != _lib.OK:
            raise GGUFError(err.value.decode(errors="replace") or f"status {rc}")
        self.handle = handle
        self.version = int(self.lib.ishi_gguf_version(handle))
        self.dataOffset = int(self.lib.ishi_gguf_data_offset(handle))  # noqa: N815
        self.alignment = int(self.lib.ishi_gguf_alignment(handle))
        self.tensors: list[TensorInfo] = []
        info = _lib.GGUFTensorInfo()
        for i in range(int(self.lib.ishi_gguf_tensor_count(handle))):
            assert self.lib.ishi_gguf_tensor(handle, i, ctypes.byref(info)) == _lib.OK
            self.tensors.append(TensorInfo(info.name.decode(), tuple(int(info.shape[d]) for d in range(info.rank)),
                                           int(info.ggml_type), int(info.offset), int(info.byte_count), i))
        self._index = {t.name: t for t in self.tensors}

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.ishi_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor(self, name: str) -> TensorInfo | None:
        return self._index.get(name)

    # ---- metadata ------------------------------------------------------------------------------
    @property
    def keys(self) -> list[str]:
        n = int(self.lib.ishi_gguf_metadata_count(self.handle))
        return [self.lib.ishi_gguf_metadata_key(self.handle, i).decode() for i in range(n)]

    def __getitem__(self, key: str):
        """The value of a metadata key as int, float, bool, str or list, or None."""
        k = key.encode()
        kind = int(self.lib.ishi_gguf_metadata_kind(self.handle, k))
        if kind == 0:
            return None
        if kind in (1, 2, 4):
            out = ctypes.c_int64()
            self.lib.ishi_gguf_metadata_int(self.handle, k, ctypes.byref(out))
            return bool(out.value) if kind == 4 else int(out.value)
        if kind == 3:
            out = ctypes.c_double()
            self.lib.ishi_gguf_metadata_float(self.handle, k, ctypes.byref(out))
            return float(out.value)
        if kind == 5:
            return self.lib.ishi_gguf_metadata_string(self.handle, k).decode(errors="replace")
        items = []
        for i in range(int(self.lib.ishi_gguf_metadata_array_length(self.handle, k))):
            s = self.lib.ishi_gguf_metadata_array_string(self.handle, k, i)
            if s is not None:
                items.append(s.decode(errors="replace"))
                continue
            out = ctypes.c_int64()
            if self.lib.ishi_gguf_metadata_array_int(self.handle, k, i, ctypes.byref(out)) == _lib.OK:
                items.append(int(out.value))
        return items

    @property
    def architecture(self) -> str:
        return self["general.architecture"] or ""

    def architectureValue(self, suffix: str):  # noqa: N802
        return self[f"{self.architecture}.{suffix}"]

    @property
    def typeHistogram(self) -> list[tuple[int, int]]:  # noqa: N802
        counts: dict[int, int] = {}
        for t in self.tensors:
            counts[t.type] = counts.get(t.type, 0) + 1
        return sorted(counts.items(), key=lambda kv: -kv[1])

    # ---- tensor data ---------------------------------------------------------------------------
    def data(self, tensor: TensorInfo | str) -> np.ndarray:
        """The raw bytes of one tensor (GGUFFile.data(for:))."""
        t = self._index[tensor] if isinstance(tensor, str) else tensor
        out = np.empty(t.byteCount, dtype=np.uint8)
        rc = self.lib.ishi_gguf_read_tensor(self.handle, t.index, out.ctypes.data_as(ctypes.c_void_p), out.size)
        if rc != _lib.OK:
            raise GGUFError(self.lib.ishi_gguf_last_error(self.handle).decode(errors="replace"))
        return out

    def blocks(self, tensor: TensorInfo | str):
        """One quantized tensor on the current GPU, still in its GGML blocks (GGUFWeights.load keeps
        every quantized tensor like this, Sources/IshizukiKit/Core/GGUFWeights.swift:63-68)."""
        import torch

        from .interface import GGMLType, GGUFBlocks

        t = self._index[tensor] if isinstance(tensor, str) else tensor
        dev = torch.empty(t.byteCount, dtype=torch.uint8, device="cuda")
        rc = self.lib.ishi_gguf_upload_tensor(self.handle, t.index, ctypes.c_void_p(dev.data_ptr()), dev.numel(),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != _lib.OK:
            raise GGUFError(self.lib.ishi_gguf_last_error(self.handle).decode(errors="replace"))
        rows = int(np.prod(t.shape[:-1]))
        return GGUFBlocks(dev, GGMLType(t.type), (rows, t.shape[-1]))
