"""Host-side mirror of the reference's projection interface on top of the C ABI.

The reference's host language is Swift; no Swift toolchain exists where this library is built
and tested, so the same surface is written here in Python over ctypes. Names, argument meaning
and "declined" behaviour follow the reference:

  GGMLType, GGUFBlocks      Sources/IshizukiKit/Config/GGUFFile.swift:13-121,
                            Sources/IshizukiKit/Core/GGUFWeights.swift:13-26
  GGMLKernels               Sources/IshizukiKit/Core/GGMLKernels.swift:60-95,146,177-253
  VerifyMatmul              Sources/IshizukiKit/Core/VerifyMatmul.swift:11-120
  PackedLinear              Sources/IshizukiKit/Core/Hadamard.swift:25-263
  BonsaiRuntime             Sources/IshizukiKit/Core/RuntimeOptions.swift:43-54

Where the reference returns nil ("declined, the caller falls back"), these return None for a
shape guard and raise for anything else; there is no fallback path behind them. Device memory
is held in torch tensors (plumbing only): every product is computed by libishizuki_cuda.so.
"""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass

import torch

from . import _lib


class IshizukiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{_status_name(status)}: {message}")
        self.status = status


def _status_name(status: int) -> str:
    return _lib.load().ishi_status_string(status).decode()


class GGMLType(enum.IntEnum):
    """GGUF tensor types this library decodes, numbered as in the file format (the quantized
    members of the reference's GGMLDequant.supported)."""

    q2K = 10
    q4K = 12
    q6K = 14
    iq2Xxs = 16
    iq2Xs = 17
    iq3Xxs = 18
    iq1S = 19
    iq3S = 21
    iq2S = 22
    iq4Xs = 23
    iq1M = 29

    @property
    def blockSize(self) -> int:  # noqa: N802 (reference spelling)
        return 256

    @property
    def typeSize(self) -> int:  # noqa: N802
        return _lib.GGML_TYPE_SIZE[int(self)]

    @property
    def isQuantized(self) -> bool:  # noqa: N802
        return True

    def byteCount(self, elements: int) -> int:  # noqa: N802
        return elements // self.blockSize * self.typeSize


@dataclass
class GGUFBlocks:
    """One tensor still in its GGML blocks: raw bytes (uint8, on the GPU), type, [N, K] shape."""

    bytes: torch.Tensor
    type: GGMLType
    shape: tuple[int, int]

    @property
    def outputDim(self) -> int:  # noqa: N802
        return self.shape[0]

    @property
    def inputDim(self) -> int:  # noqa: N802
        return self.shape[-1]


class BonsaiRuntime:
    """Global switches the dispatch reads (reference: RuntimeOptions.swift:43-54)."""

    useVerifyMatmul = True
    # B200 additions: force one kernel family, or move the GEMV -> tensor-core crossover.
    route = _lib.ROUTE_AUTO
    crossoverRows = 0


class Context:
    """One per GPU; owns the library's tables and the scratch of the kernel-level calls."""

    _by_device: dict[int, "Context"] = {}

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("ishizuki_b200 needs a CUDA device: there is no CPU path")
        handle = ctypes.c_void_p()
        rc = self.lib.ishi_ctx_create(device, ctypes.byref(handle))
        if rc != _lib.OK:
            raise IshizukiError(rc, f"ishi_ctx_create({device}) failed")
        self.handle = handle
        self.device = device

    @classmethod
    def get(cls, device: int | None = None) -> "Context":
        device = torch.cuda.current_device() if device is None else device
        ctx = cls._by_device.get(device)
        if ctx is None:
            ctx = cls._by_device[device] = Context(device)
        return ctx

    def last_error(self) -> str:
        return self.lib.ishi_last_error(self.handle).decode()

    def check(self, rc: int, declined=( _lib.E_SHAPE,)):
        """OK -> True, a shape guard -> False (the reference's nil), anything else raises."""
        if rc == _lib.OK:
            return True
        if rc in declined:
            return False
        raise IshizukiError(rc, self.last_error())

    def poll(self) -> None:
        rc = self.lib.ishi_ctx_poll(self.handle)
        if rc != _lib.OK:
            raise IshizukiError(rc, self.last_error())

    def sync_route(self) -> None:
        rc = self.lib.ishi_ctx_set_route(self.handle, BonsaiRuntime.route, BonsaiRuntime.crossoverRows)
        if rc != _lib.OK:
            raise IshizukiError(rc, self.last_error())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_SCALE_DT = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16, torch.float32: _lib.DT_F32}
_OUT_DT = _SCALE_DT


def _as_half_rows(x: torch.Tensor) -> torch.Tensor | None:
    if x.dim() != 2 or x.dtype != torch.float16 or not x.is_cuda:
        return None
    return x.contiguous()


class GGMLKernels:
    """Runs a tensor's GGML blocks on the GPU, expanded or folded into a product."""

    matvecBatch = range(1, 17)
    # The reference's few-row kernel takes 2...8 rows; this one takes every count the matvec does.
    matmulFewRows = range(1, 17)

    @staticmethod
    def dequantize(blocks: torch.Tensor, type: GGMLType, shape, dtype=torch.bfloat16):
        ctx = Context.get(blocks.device.index)
        count = 1
        for s in shape:
            count *= s
        try:
            type = GGMLType(type)
        except ValueError:
            return None
        if count % type.blockSize != 0:
            return None
        n_blocks = count // type.blockSize
        if blocks.numel() < n_blocks * type.typeSize:
            return None
        out = torch.empty(count, dtype=dtype, device=blocks.device)
        rc = ctx.lib.ishi_ggml_dequantize(ctx.handle, int(type), _ptr(blocks), n_blocks, _ptr(out),
                                          _OUT_DT[dtype], _stream())
        if not ctx.check(rc, declined=(_lib.E_SHAPE, _lib.E_UNSUPPORTED)):
            return None
        return out.reshape(tuple(shape))

    @staticmethod
    def gather(ids: torch.Tensor, blocks: torch.Tensor, type: GGMLType, inputDim: int, dtype=torch.bfloat16):  # noqa: N803
        """The rows named by ids, decoded into [ids.numel(), inputDim] (the embedding lookup)."""
        try:
            type = GGMLType(type)
        except ValueError:
            return None
        if inputDim % type.blockSize != 0 or ids.numel() == 0:
            return None
        ctx = Context.get(blocks.device.index)
        idx = ids.reshape(-1).to(torch.int32).contiguous()
        per_row = inputDim // type.blockSize * type.typeSize
        table_rows = blocks.numel() // per_row
        out = torch.empty((idx.numel(), inputDim), dtype=dtype, device=blocks.device)
        rc = ctx.lib.ishi_ggml_gather(ctx.handle, _ptr(idx), idx.numel(), _ptr(blocks), blocks.numel(), int(type),
                                      table_rows, inputDim, _ptr(out), _OUT_DT[dtype], _stream())
        return out if ctx.check(rc, declined=(_lib.E_SHAPE, _lib.E_UNSUPPORTED)) else None

    @staticmethod
    def _product(fn_name: str, x, blocks, type, outputDim):
        x = _as_half_rows(x)
        if x is None:
            return None
        try:
            type = GGMLType(type)
        except ValueError:
            return None
        ctx = Context.get(x.device.index)
        m, k = x.shape
        y = torch.empty((m, outputDim), dtype=torch.float16, device=x.device)
        fn = getattr(ctx.lib, fn_name)
        rc = fn(ctx.handle, _ptr(x), m, _ptr(blocks), blocks.numel(), int(type), outputDim, k, _ptr(y),
                _stream())
        return y if ctx.check(rc) else None

    @staticmethod
    def matvec(x, blocks: torch.Tensor, type: GGMLType, outputDim: int):  # noqa: N803
        """x [M, K] against the blocks of w [N, K] on CUDA cores; None when declined."""
        return GGMLKernels._product("ishi_ggml_matvec", x, blocks, type, outputDim)

    @staticmethod
    def matmulFew(x, blocks: torch.Tensor, type: GGMLType, outputDim: int, rowBlocks: int = 2):  # noqa: N802,N803
        """The same product through tensor-core fragments. rowBlocks is accepted for source
        compatibility; the tile shape is fixed by the launch plan here."""
        return GGMLKernels._product("ishi_ggml_matmul_few", x, blocks, type, outputDim)


class VerifyMatmul:
    """A few-row affine matmul for the speculative verify."""

    supportedRows = range(1, 17)  # the reference's Metal kernel stops at 8

    @staticmethod
    def minimumRows(bytes: int) -> int:  # noqa: N802,A002
        """The reference's Apple-M1 crossover table, unchanged (VerifyMatmul.swift:19-26)."""
        return int(_lib.load().ishi_reference_minimum_rows(bytes))

    @staticmethod
    def applyAny(x, w, scales, biases, groupSize: int, bits: int, route: int = _lib.ROUTE_MMA):  # noqa: N802,N803
        x = _as_half_rows(x)
        if x is None:
            return None
        ctx = Context.get(x.device.index)
        m, k = x.shape
        n = w.shape[0]
        if w.shape[1] * 32 != k * bits or scales.dtype != biases.dtype:
            return None
        scales, biases = scales.contiguous(), biases.contiguous()
        y = torch.empty((m, n), dtype=torch.float16, device=x.device)
        rc = ctx.lib.ishi_verify_matmul(ctx.handle, _ptr(x), m, _ptr(w), _ptr(scales), _ptr(biases),
                                        _SCALE_DT[scales.dtype], groupSize, bits, n, k, route, _ptr(y),
                                        _stream())
        return y if ctx.check(rc, declined=(_lib.E_SHAPE, _lib.E_UNSUPPORTED)) else None

    @staticmethod
    def apply(x, w, scales, biases, groupSize: int, bits: int):  # noqa: N803
        if x.dim() != 2 or x.shape[0] not in VerifyMatmul.supportedRows:
            return None
        return VerifyMatmul.applyAny(x, w, scales, biases, groupSize, bits)


class PackedLinear:
    """A projection whose weight stays packed: GGUF blocks or an MLX affine pack, optionally
    with a Hadamard-rotated input. Construct with the affine arguments or with ggml=GGUFBlocks."""

    def __init__(self, weight=None, scales=None, biases=None, signs=None, block: int = 0,
                 groupSize: int = 128, bits: int = 2, ggml: GGUFBlocks | None = None):  # noqa: N803
        self.ggml = ggml
        self.signs = signs
        self.block = block
        if ggml is not None:
            self.weight = ggml.bytes
            self.scales = self.biases = None
            self.groupSize, self.bits = ggml.type.blockSize, 0
            self.outputDim, self.inputDim = ggml.outputDim, ggml.inputDim
        else:
            self.weight, self.scales, self.biases = weight, scales, biases
            self.groupSize, self.bits = groupSize, bits
            self.outputDim = weight.shape[0]
            self.inputDim = scales.shape[1] * groupSize
            if block > 0 and signs is not None and signs.shape[0] != self.inputDim:
                raise ValueError(f"sign vector is {signs.shape[0]} wide, expected {self.inputDim}")
        if block > 0 and self.inputDim % block != 0:
            raise ValueError(f"Hadamard block {block} does not divide input width {self.inputDim}")
        self.ctx = Context.get(self.weight.device.index)
        d = self._describe(self.weight, self.scales, self.biases, self.outputDim)
        handle = ctypes.c_void_p()
        rc = self.ctx.lib.ishi_projection_create(self.ctx.handle, ctypes.byref(d), ctypes.byref(handle))
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())
        self.handle = handle

    def _describe(self, weight, scales, biases, n) -> "_lib.WeightDesc":
        d = _lib.WeightDesc()
        d.kind = _lib.KIND_GGML if self.ggml is not None else _lib.KIND_AFFINE
        d.ggml_type = int(self.ggml.type) if self.ggml is not None else 0
        d.bits, d.group_size = self.bits, self.groupSize
        d.scale_dtype = _SCALE_DT[scales.dtype] if scales is not None else 0
        d.hadamard_block = self.block
        d.n, d.k = n, self.inputDim
        d.weight_dev = weight.data_ptr()
        d.weight_bytes = weight.numel() * weight.element_size()
        d.scales_dev = 0 if scales is None else scales.data_ptr()
        d.biases_dev = 0 if biases is None else biases.data_ptr()
        d.signs_dev = 0 if self.signs is None else self.signs.data_ptr()
        return d

    def __del__(self):
        handle = getattr(self, "handle", None)
        if handle:
            self.ctx.lib.ishi_projection_destroy(handle)
            self.handle = None

    @property
    def weightBytes(self) -> int:  # noqa: N802
        return int(self.ctx.lib.ishi_projection_weight_bytes(self.handle))

    @property
    def crossoverRows(self) -> int:  # noqa: N802
        return int(self.ctx.lib.ishi_projection_crossover_rows(self.handle))

    @property
    def plan(self) -> tuple[int, int, int, int]:
        """The launch plan create settled on (K split, warps per panel, panels in parallel, ring);
        zeros for a format outside the warp-level kernel."""
        out = (ctypes.c_int * 4)()
        self.ctx.check(self.ctx.lib.ishi_projection_plan(self.handle, out), declined=())
        return tuple(int(v) for v in out)

    def set_plan(self, plan) -> None:
        """Imposes another projection's plan: partial sums are then added in the same order."""
        arr = (ctypes.c_int * 4)(*[int(v) for v in plan])
        self.ctx.check(self.ctx.lib.ishi_projection_set_plan(self.handle, arr), declined=())

    def _rows(self, x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, ...]]:
        if x.dtype != torch.float16 or not x.is_cuda:
            raise TypeError("activations must be fp16 CUDA tensors")
        shape = tuple(x.shape)
        return x.reshape(-1, shape[-1]).contiguous(), shape

    def _out(self, h: torch.Tensor, transposed: bool) -> torch.Tensor:
        m = h.shape[0]
        if transposed:
            return torch.empty((self.outputDim, m), dtype=torch.float16, device=h.device)
        return torch.empty((m, self.outputDim), dtype=torch.float16, device=h.device)

    def __call__(self, x: torch.Tensor, transposed: bool = False, out: torch.Tensor | None = None):
        """y = x . W^T for 1...16 rows of x, rotating x first when the pack is rotated."""
        self.ctx.sync_route()
        h, shape = self._rows(x)
        y = self._out(h, transposed) if out is None else out
        rc = self.ctx.lib.ishi_projection_apply(self.handle, _ptr(h), h.shape[0], _ptr(y), y.stride(0),
                                                _lib.OUT_TRANSPOSED if transposed else 0, _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())
        return y if transposed or out is not None else y.reshape(shape[:-1] + (self.outputDim,))

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        """Per row of x the index of its largest logit (int32): the head of a greedy verify step."""
        self.ctx.sync_route()
        h, _ = self._rows(x)
        out = torch.empty(h.shape[0], dtype=torch.int32, device=h.device)
        rc = self.ctx.lib.ishi_projection_apply_argmax(self.handle, _ptr(h), h.shape[0], _ptr(out), _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())
        return out

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        h, shape = self._rows(x)
        xr = torch.empty_like(h)
        rc = self.ctx.lib.ishi_projection_rotate(self.handle, _ptr(h), h.shape[0], _ptr(xr), _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())
        return xr.reshape(shape)

    def applyRotated(self, h: torch.Tensor) -> torch.Tensor:  # noqa: N802
        self.ctx.sync_route()
        rows, shape = self._rows(h)
        y = self._out(rows, False)
        rc = self.ctx.lib.ishi_projection_apply_rotated(self.handle, _ptr(rows), rows.shape[0], _ptr(y),
                                                        y.stride(0), 0, _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())
        return y.reshape(shape[:-1] + (self.outputDim,))

    def apply_host(self, x_host, y_host) -> None:
        """Host-buffer form: x_host [M, K] and y_host [M, N] are C-contiguous fp16 numpy arrays."""
        rc = self.ctx.lib.ishi_projection_apply_host(
            self.handle, x_host.ctypes.data_as(ctypes.c_void_p), x_host.shape[0],
            y_host.ctypes.data_as(ctypes.c_void_p), _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())

    def apply_host_async(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Host-buffer form without the wait: x_host [M, K] and y_host [M, N] are contiguous fp16 CPU
        tensors (page-locked ones make the copies asynchronous); y_host is valid once the current
        stream has been synchronised."""
        rc = self.ctx.lib.ishi_projection_apply_host_async(self.handle, _ptr(x_host), x_host.shape[0], _ptr(y_host),
                                                           _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())


class HostBatch:
    """A fixed list of projections with page-locked host inputs and outputs, run by one C call
    (ishi_projection_apply_host_batch): the copies in, the products and the copies out overlap."""

    def __init__(self, layers, xs, ys):
        """layers: PackedLinear objects of one context; xs[i] [rows, k_i], ys[i] [rows, n_i]: contiguous
        fp16 CPU tensors (pinned for the copies to be asynchronous)."""
        self.layers, self.xs, self.ys = list(layers), list(xs), list(ys)
        n = len(self.layers)
        self.rows = self.xs[0].shape[0]
        self._p = (ctypes.c_void_p * n)(*[lin.handle.value for lin in self.layers])
        self._x = (ctypes.c_void_p * n)(*[x.data_ptr() for x in self.xs])
        self._y = (ctypes.c_void_p * n)(*[y.data_ptr() for y in self.ys])
        self.ctx = self.layers[0].ctx

    def run(self) -> None:
        """Enqueues the whole list; the outputs are valid once the current stream is synchronised."""
        rc = self.ctx.lib.ishi_projection_apply_host_batch(self._p, self._x, self.rows, self._y, len(self.layers), _stream())
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())


class FusedLinear(PackedLinear):
    """Several projections that read the same input, as one: y = [x . W0^T | x . W1^T | ...].

    The reference runs q / k / v (Sources/IshizukiKit/Text/Attention.swift:75-83) and gate / up
    (Attention.swift:251) as separate kernels on the same input; here their weights are stacked
    along the output rows at create time and one launch streams them all. ``parts`` is a list of
    GGUFBlocks (same type and input width) or of (weight, scales, biases) affine packs (same
    width, group size and scale dtype). ``split(y)`` gives the parts' outputs back as views.

    ``gated=True`` takes exactly two parts, the MLP's gate and up projections, and makes the
    launch's output ``silu(x . gate^T) * (x . up^T)`` (the input of the reference's downProj,
    Attention.swift:251): the rows of the two weights are interleaved by eights at create time so
    that one accumulator fragment holds a gate row and its up row, and the kernel's epilogue
    combines them. ``outputDim`` is then the height of one part."""

    def __init__(self, parts, signs=None, block: int = 0, groupSize: int = 128, bits: int = 2,  # noqa: N803
                 gated: bool = False):
        first = parts[0]
        self.signs, self.block = signs, block
        if isinstance(first, GGUFBlocks):
            self.ggml = first
            self.groupSize, self.bits = first.type.blockSize, 0
            self.inputDim = first.inputDim
            self.outputDims = [p.outputDim for p in parts]
            triples = [(p.bytes, None, None) for p in parts]
            if any(p.type != first.type or p.inputDim != first.inputDim for p in parts):
                raise ValueError("stacked GGUF weights must share type and input width")
        else:
            self.ggml = None
            self.groupSize, self.bits = groupSize, bits
            self.inputDim = first[1].shape[1] * groupSize
            self.outputDims = [w.shape[0] for w, _, _ in parts]
            triples = list(parts)
        self.weight, self.scales, self.biases = triples[0]
        self.outputDim = sum(self.outputDims)
        self.ctx = Context.get(self.weight.device.index)
        descs = (_lib.WeightDesc * len(triples))()
        for i, (w, s, b) in enumerate(triples):
            descs[i] = self._describe(w, s, b, self.outputDims[i])
        handle = ctypes.c_void_p()
        self.gated = gated
        if gated:
            if len(triples) != 2:
                raise ValueError("a gated pair is two weights: gate and up")
            rc = self.ctx.lib.ishi_projection_create_gated(self.ctx.handle, ctypes.byref(descs[0]), ctypes.byref(descs[1]),
                                                           ctypes.byref(handle))
            self.outputDim = self.outputDims[0]
        else:
            rc = self.ctx.lib.ishi_projection_create_fused(self.ctx.handle, descs, len(triples), ctypes.byref(handle))
        if rc != _lib.OK:
            raise IshizukiError(rc, self.ctx.last_error())
        self.handle = handle
        self.weight = self.scales = self.biases = None  # the library keeps its own tiled copy

    def split(self, y: torch.Tensor, transposed: bool = False):
        if self.gated:
            raise ValueError("a gated pair has one output: silu(gate) * up")
        return torch.split(y, self.outputDims, dim=0 if transposed else -1)


def hadamardRotate(x: torch.Tensor, block: int, signs: torch.Tensor | None) -> torch.Tensor:  # noqa: N802
    """xr = WHT_block(x * signs) / sqrt(block) along the last axis (forward form only)."""
    ctx = Context.get(x.device.index)
    h = x.reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty_like(h)
    rc = ctx.lib.ishi_hadamard_rotate(ctx.handle, _ptr(h), h.shape[0], h.shape[1], block, _ptr(signs), _ptr(y),
                                      _stream())
    if rc != _lib.OK:
        raise IshizukiError(rc, ctx.last_error())
    return y.reshape(x.shape)


def rmsNorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:  # noqa: N802
    """MLXFast.rmsNorm(x, weight:, eps:) ahead of a projection (TextModel.swift:151-161): fp32 or
    fp16 rows in, fp16 out."""
    ctx = Context.get(x.device.index)
    h = x.reshape(-1, x.shape[-1]).contiguous()
    w = weight.contiguous()
    y = torch.empty(h.shape, dtype=torch.float16, device=x.device)
    ctx.check(ctx.lib.ishi_rms_norm(ctx.handle, _ptr(h), _OUT_DT[h.dtype], h.shape[0], h.shape[1], _ptr(w), _OUT_DT[w.dtype],
                                    ctypes.c_float(eps), _ptr(y), _stream()), declined=())
    return y.reshape(x.shape)


class EXL3Tensor:
    """An EXL3 trellis-coded weight (reference: EXL3Tensor, Sources/IshizukiKit/Core/EXL3.swift:9-79):
    ``trellis`` int16 [k / 16, n / 16, 16 * bits], fp16 scale vectors of the input and the output
    side, and one of the three codebooks."""

    threeInst, mcg, mul1 = _lib.EXL3_3INST, _lib.EXL3_MCG, _lib.EXL3_MUL1

    def __init__(self, trellis: torch.Tensor, inputScales: torch.Tensor | None, outputScales: torch.Tensor | None,  # noqa: N803
                 codebook: int):
        if trellis.ndim != 3 or trellis.dtype != torch.int16:
            raise ValueError("EXL3 trellis must be int16 [k/16, n/16, words]")
        self.trellis = trellis.contiguous()
        self.inputScales = None if inputScales is None else inputScales.to(torch.float16).reshape(-1).contiguous()
        self.outputScales = None if outputScales is None else outputScales.to(torch.float16).reshape(-1).contiguous()
        self.codebook = int(codebook)
        self.bits = trellis.shape[2] / 16
        self.inputDim, self.outputDim = trellis.shape[0] * 16, trellis.shape[1] * 16

    def _desc(self) -> "_lib.EXL3Desc":
        d = _lib.EXL3Desc()
        d.trellis_dev = self.trellis.data_ptr()
        d.k, d.n = self.inputDim, self.outputDim
        d.words_per_tile = self.trellis.shape[2]
        d.codebook = self.codebook
        d.input_scales_dev = 0 if self.inputScales is None else self.inputScales.data_ptr()
        d.output_scales_dev = 0 if self.outputScales is None else self.outputScales.data_ptr()
        return d


class EXL3Kernels:
    """EXL3Kernels of the reference (EXL3.swift:81-164): decode, rotations, the few-row product
    that decodes inside the multiply, and their composition."""

    matvecRows = range(1, 9)

    @staticmethod
    def dequantize(t: EXL3Tensor, dtype: torch.dtype = torch.float16) -> torch.Tensor:
        ctx = Context.get(t.trellis.device.index)
        w = torch.empty((t.inputDim, t.outputDim), dtype=dtype, device=t.trellis.device)
        ctx.check(ctx.lib.ishi_exl3_dequantize(ctx.handle, ctypes.byref(t._desc()), _OUT_DT[dtype], _ptr(w), _stream()), declined=())
        return w

    @staticmethod
    def rotate(x: torch.Tensor, scales: torch.Tensor, before: bool, to: torch.dtype) -> torch.Tensor:
        ctx = Context.get(x.device.index)
        h = x.reshape(-1, x.shape[-1]).contiguous()
        s = scales.to(torch.float16).contiguous()
        y = torch.empty(h.shape, dtype=to, device=x.device)
        ctx.check(ctx.lib.ishi_exl3_rotate(ctx.handle, _ptr(h), _OUT_DT[h.dtype], h.shape[0], h.shape[1], _ptr(s), int(before),
                                           _ptr(y), _OUT_DT[to], _stream()), declined=())
        return y.reshape(x.shape)

    @staticmethod
    def matvec(x: torch.Tensor, t: EXL3Tensor) -> torch.Tensor | None:
        """fp32 [rows, n] for 1...8 fp16 rows, None outside (as the reference)."""
        if x.ndim != 2 or x.shape[1] != t.inputDim or x.shape[0] not in EXL3Kernels.matvecRows:
            return None
        ctx = Context.get(x.device.index)
        h = x.to(torch.float16).contiguous()
        y = torch.empty((h.shape[0], t.outputDim), dtype=torch.float32, device=x.device)
        ctx.check(ctx.lib.ishi_exl3_matvec(ctx.handle, ctypes.byref(t._desc()), _ptr(h), h.shape[0], _ptr(y), _stream()), declined=())
        return y

    @staticmethod
    def apply(x: torch.Tensor, t: EXL3Tensor) -> torch.Tensor:
        """rotate -> product -> rotate, 1...16 fp16 rows."""
        ctx = Context.get(x.device.index)
        shape = x.shape
        h = x.reshape(-1, t.inputDim).to(torch.float16).contiguous()
        y = torch.empty((h.shape[0], t.outputDim), dtype=torch.float16, device=x.device)
        ctx.check(ctx.lib.ishi_exl3_apply(ctx.handle, ctypes.byref(t._desc()), _ptr(h), h.shape[0], _ptr(y), _stream()), declined=())
        return y.reshape(shape[:-1] + (t.outputDim,))


class EXL3Linear:
    """PackedLinear(exl3:) of the reference (EXL3Tests.projectionMatchesCheckpoint): a projection
    over an EXL3Tensor, y = EXL3Kernels.apply(x, tensor)."""

    def __init__(self, exl3: EXL3Tensor):
        if exl3.inputScales is None or exl3.outputScales is None:
            raise ValueError("an EXL3 projection needs both scale vectors")
        self.exl3 = exl3
        self.inputDim, self.outputDim = exl3.inputDim, exl3.outputDim
        self.ctx = Context.get(exl3.trellis.device.index)

    @property
    def weightBytes(self) -> int:  # noqa: N802
        return self.exl3.trellis.numel() * 2 + (self.inputDim + self.outputDim) * 2

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return EXL3Kernels.apply(x, self.exl3)
