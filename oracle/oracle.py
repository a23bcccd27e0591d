"""ctypes front end of the CPU oracle (``ishi_oracle.c``). TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and bench.py's CPU-baseline leg import this module; the product
package never does. Each function forwards to the C restatement, whose header lists the
reference lines it follows.
"""
from __future__ import annotations

import ctypes
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libishi_oracle.so"

Q2_K, Q4_K, Q6_K, IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ4_XS, IQ1_M = 10, 12, 14, 16, 17, 18, 19, 21, 22, 23, 29
TYPE_SIZE = {Q2_K: 84, Q4_K: 144, Q6_K: 210, IQ2_XXS: 66, IQ2_XS: 74, IQ3_XXS: 98, IQ1_S: 50, IQ3_S: 110, IQ2_S: 82,
             IQ4_XS: 136, IQ1_M: 56}
SCALE_DTYPE = {np.dtype(np.float16): 0, np.dtype(np.float32): 2}  # bf16 is passed as uint16 + flag


def build() -> pathlib.Path:
    """Compiles the oracle with the committed Makefile (gcc only; a few seconds)."""
    subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


def _load() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        build()
    lib = ctypes.CDLL(str(_LIB_PATH))
    c = ctypes
    lib.oracle_dequant.argtypes = [c.c_int, c.c_void_p, c.c_int64, c.c_void_p]
    lib.oracle_dequant.restype = c.c_int
    lib.oracle_affine_dequant.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int64,
                                          c.c_int64, c.c_int, c.c_int, c.c_void_p]
    lib.oracle_affine_dequant.restype = c.c_int
    lib.oracle_hadamard_rotate.argtypes = [c.c_void_p, c.c_int64, c.c_int64, c.c_int, c.c_void_p,
                                           c.c_void_p]
    lib.oracle_hadamard_rotate.restype = c.c_int
    lib.oracle_matmul.argtypes = [c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int64,
                                  c.c_void_p, c.c_void_p]
    lib.oracle_matmul.restype = None
    lib.oracle_ggml_matmul.argtypes = [c.c_int, c.c_void_p, c.c_void_p, c.c_int64, c.c_int64,
                                       c.c_int64, c.c_void_p, c.c_void_p]
    lib.oracle_ggml_matmul.restype = c.c_int
    lib.oracle_affine_matmul.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                         c.c_int, c.c_void_p, c.c_int64, c.c_int64, c.c_int64,
                                         c.c_void_p, c.c_void_p]
    lib.oracle_affine_matmul.restype = c.c_int
    lib.oracle_reference_minimum_rows.argtypes = [c.c_int64]
    lib.oracle_reference_minimum_rows.restype = c.c_int
    lib.oracle_threads.restype = c.c_int
    lib.oracle_set_threads.argtypes = [c.c_int]
    lib.oracle_set_threads.restype = c.c_int
    lib.oracle_float_to_half.argtypes = [c.c_float]
    lib.oracle_float_to_half.restype = c.c_uint16
    return lib


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a)


def threads() -> int:
    return int(lib().oracle_threads())


def use_all_cores() -> int:
    """Runs the products on every core this process may use, whatever OMP_NUM_THREADS says."""
    import os

    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(n)
    return threads()


def dequantize(type_id: int, blocks: np.ndarray) -> np.ndarray:
    """GGUF blocks (uint8, a whole number of blocks) to fp32, as ggml's to_float does."""
    blocks = _c(blocks.view(np.uint8).reshape(-1))
    ts = TYPE_SIZE[type_id]
    assert blocks.size % ts == 0, "not a whole number of blocks"
    nb = blocks.size // ts
    out = np.empty(nb * 256, dtype=np.float32)
    rc = lib().oracle_dequant(type_id, _ptr(blocks), nb, _ptr(out))
    assert rc == 0
    return out


def _scale_args(scales: np.ndarray, biases: np.ndarray, bf16: bool):
    if bf16:
        assert scales.dtype == np.uint16 and biases.dtype == np.uint16
        return _c(scales), _c(biases), 1
    assert scales.dtype == biases.dtype
    return _c(scales), _c(biases), SCALE_DTYPE[scales.dtype]


def affine_dequantize(w: np.ndarray, scales: np.ndarray, biases: np.ndarray, bits: int,
                      group_size: int, bf16: bool = False) -> np.ndarray:
    """MLX affine pack to fp32 [N, K]: w = float(code) * scale + bias."""
    w = _c(w.astype(np.uint32, copy=False))
    n = w.shape[0]
    k = w.shape[1] * 32 // bits
    s, b, dt = _scale_args(scales, biases, bf16)
    out = np.empty((n, k), dtype=np.float32)
    rc = lib().oracle_affine_dequant(_ptr(w), _ptr(s), _ptr(b), dt, n, k, bits, group_size,
                                     _ptr(out))
    assert rc == 0
    return out


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """MLXFast.rmsNorm as DecoderLayer uses it (Sources/IshizukiKit/Text/TextModel.swift:151-161):
    x * rsqrt(mean(x^2) + eps) * weight in fp32, fp16 out. Pinned by the formula only (MLX)."""
    h = x.astype(np.float32)
    r = np.float32(1) / np.sqrt((h.astype(np.float64) ** 2).mean(axis=-1, keepdims=True).astype(np.float32) + np.float32(eps))
    return (h * r * weight.astype(np.float32)).astype(np.float16)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """silu(gate) * up on fp16 arrays, the input of the reference's downProj
    (Sources/IshizukiKit/Text/Attention.swift:251: downProj(silu(gateProj(x)) * upProj(x))). Each
    element-wise operation of the reference yields an fp16 array, so sigmoid, gate * sigmoid and the
    product with up are each rounded to fp16; the arithmetic in between is fp32. The reference
    holds no vector for this stage (it runs through MLX): pinned by the formula only."""
    assert gate.dtype == np.float16 and up.dtype == np.float16
    g = gate.astype(np.float32)
    with np.errstate(over="ignore"):
        sig = (np.float32(1) / (np.float32(1) + np.exp(-g))).astype(np.float16).astype(np.float32)
    act = (g * sig).astype(np.float16).astype(np.float32)
    return (act * up.astype(np.float32)).astype(np.float16)


def hadamard_rotate(x: np.ndarray, block: int, signs: np.ndarray | None = None) -> np.ndarray:
    """Block Hadamard rotation of fp16 rows, fp32 inside, fp16 out."""
    assert x.dtype == np.float16
    x = _c(x)
    rows = x.size // x.shape[-1]
    s = None if signs is None else _c(signs.astype(np.float32))
    out = np.empty_like(x)
    rc = lib().oracle_hadamard_rotate(_ptr(x), rows, x.shape[-1], block, _ptr(s), _ptr(out))
    assert rc == 0
    return out


def matmul(w: np.ndarray, x: np.ndarray):
    """Dense fp32 w [N, K] against fp16 x [M, K] -> (fp32 [M, N], fp16 [M, N])."""
    w = _c(w.astype(np.float32, copy=False))
    x = _c(x)
    assert x.dtype == np.float16
    m, k = x.shape
    n = w.shape[0]
    y32 = np.empty((m, n), dtype=np.float32)
    y16 = np.empty((m, n), dtype=np.float16)
    lib().oracle_matmul(_ptr(w), _ptr(x), m, n, k, _ptr(y32), _ptr(y16))
    return y32, y16


def ggml_matmul(type_id: int, blocks: np.ndarray, x: np.ndarray, n: int):
    """GGUF blocks [N][K/256][type size] against fp16 x [M, K] -> (fp32, fp16) [M, N]."""
    blocks = _c(blocks.view(np.uint8).reshape(-1))
    x = _c(x)
    assert x.dtype == np.float16
    m, k = x.shape
    assert blocks.size >= n * (k // 256) * TYPE_SIZE[type_id]
    y32 = np.empty((m, n), dtype=np.float32)
    y16 = np.empty((m, n), dtype=np.float16)
    rc = lib().oracle_ggml_matmul(type_id, _ptr(blocks), _ptr(x), m, n, k, _ptr(y32), _ptr(y16))
    assert rc == 0
    return y32, y16


def affine_matmul(w: np.ndarray, scales: np.ndarray, biases: np.ndarray, bits: int,
                  group_size: int, x: np.ndarray, bf16: bool = False):
    """Affine pack against fp16 x [M, K] (already rotated if the pack is) -> (fp32, fp16)."""
    w = _c(w.astype(np.uint32, copy=False))
    x = _c(x)
    assert x.dtype == np.float16
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] * 32 == k * bits
    s, b, dt = _scale_args(scales, biases, bf16)
    y32 = np.empty((m, n), dtype=np.float32)
    y16 = np.empty((m, n), dtype=np.float16)
    rc = lib().oracle_affine_matmul(_ptr(w), _ptr(s), _ptr(b), dt, bits, group_size, _ptr(x), m,
                                    n, k, _ptr(y32), _ptr(y16))
    assert rc == 0
    return y32, y16


def reference_minimum_rows(nbytes: int) -> int:
    return int(lib().oracle_reference_minimum_rows(nbytes))


def read_ggml_fixture(path) -> dict[int, tuple[np.ndarray, np.ndarray]]:
    """Parses the reference's ggml fixture: {type id: (raw block bytes, expected fp32)}."""
    data = pathlib.Path(path).read_bytes()
    assert data[:8] == b"GGMLREF1"
    cur = 8
    count = int(np.frombuffer(data, "<u4", 1, cur)[0])
    cur += 4
    out = {}
    for _ in range(count):
        tid, _nb, raw, nf = (int(v) for v in np.frombuffer(data, "<u4", 4, cur))
        cur += 16
        blocks = np.frombuffer(data, np.uint8, raw, cur).copy()
        cur += raw
        want = np.frombuffer(data, "<f4", nf, cur).copy()
        cur += 4 * nf
        out[tid] = (blocks, want)
    return out

# ---- EXL3 trellis-coded weights (reference: Sources/IshizukiKit/Core/EXL3.swift) ----------------
#
# A 16 x 16 tile of W [k, n] is one ring of 256 * bits bits (half-integer rates: 128 * (2 * whole + 1)),
# stored as 16 * bits int16 (read as 32-bit little-endian words, bits counted from each word's top).
# Weight p of the tile (0...255) is a function of the 16 ring bits that end where p's own code ends
# (EXL3.swift:184-186, 200-214); the function is one of three procedural codebooks
# (EXL3.swift:171-182). Weight p = 8 * lane + i sits at row (lane % 4) * 2 + {0, 1, 8, 9}[i % 4],
# column lane / 4 + 8 * (i / 4) of the tile (EXL3.swift:286-290): the layout of a 16 x 8 x 16
# matrix-multiply fragment.
EXL3_3INST, EXL3_MCG, EXL3_MUL1 = 0, 1, 2


def _exl3_codes_end(whole: int, half: bool) -> np.ndarray:
    p = np.arange(256)
    if half:
        return (p >> 1) * (2 * whole + 1) + whole + (p & 1) * (whole + 1)
    return (p + 1) * whole


def _bits_to_half(bits: np.ndarray) -> np.ndarray:
    return bits.astype(np.uint16).view(np.float16)


def exl3_decode(state: np.ndarray, codebook: int) -> np.ndarray:
    """The weight of a 16-bit trellis state, as float32 (EXL3.swift:171-182). All values are fp16
    numbers: the codebooks end in one fp16 operation (an add, or a fused multiply-add)."""
    s = state.astype(np.uint64)
    if codebook == EXL3_MUL1:
        x = (s * 0x83DCD12D) & 0xFFFFFFFF
        p = (x & 0x00FF00FF) + ((x >> 8) & 0x00FF00FF)
        h = _bits_to_half((p & 0xFFFF) + (p >> 16) + 0x6400).astype(np.float64)
        a = float(_bits_to_half(np.array([0x1EEE]))[0])
        b = float(_bits_to_half(np.array([0xC931]))[0])
        return (h * a + b).astype(np.float16).astype(np.float32)  # exact in float64, rounded once
    x = (s * 0xCBAC1FED) & 0xFFFFFFFF if codebook == EXL3_MCG else (s * 89226354 + 64248484) & 0xFFFFFFFF
    x = (x & 0x8FFF8FFF) ^ 0x3B603B60
    lo, hi = _bits_to_half(x & 0xFFFF).astype(np.float64), _bits_to_half(x >> 16).astype(np.float64)
    return (lo + hi).astype(np.float16).astype(np.float32)


def exl3_dequantize(trellis: np.ndarray, codebook: int) -> np.ndarray:
    """int16 [k / 16, n / 16, 16 * bits] -> float32 W [k, n] (EXL3.swift:275-292)."""
    assert trellis.dtype == np.int16 and trellis.ndim == 3
    tk, tn, words16 = trellis.shape
    whole, half = words16 // 16, words16 % 16 != 0
    assert words16 in (16 * whole, 16 * whole + 8)
    ring = 16 * words16
    words = np.ascontiguousarray(trellis).view(np.uint32).reshape(tk * tn, ring // 32)
    # the ring as bits, each 32-bit word from its top bit down
    bits = np.unpackbits(words.byteswap().view(np.uint8).reshape(tk * tn, ring // 8), axis=1)
    end = _exl3_codes_end(whole, half)
    idx = (end[:, None] - 16 + np.arange(16)[None, :]) % ring                 # [256, 16]
    state = (bits[:, idx].astype(np.uint32) << (15 - np.arange(16, dtype=np.uint32))).sum(axis=2)  # [tiles, 256]
    v = exl3_decode(state, codebook)
    lane, i = np.arange(256) // 8, np.arange(256) % 8
    row = (lane % 4) * 2 + np.array([0, 1, 8, 9])[i % 4]
    col = lane // 4 + 8 * (i // 4)
    tiles = np.empty((tk * tn, 16, 16), dtype=np.float32)
    tiles[:, row, col] = v
    return tiles.reshape(tk, tn, 16, 16).transpose(0, 2, 1, 3).reshape(tk * 16, tn * 16)


def exl3_rotate(x: np.ndarray, scales: np.ndarray, before: bool, dtype=np.float16) -> np.ndarray:
    """Block Hadamard of 128 with a scale vector on the input (before) or the output side, fp32
    inside (EXL3.swift:114-122, 219-262)."""
    rows, width = x.shape
    h = x.astype(np.float32)
    s = scales.astype(np.float32)
    if before:
        h = h * s
    hm = np.array([[1.0]], dtype=np.float32)
    while hm.shape[0] < 128:
        hm = np.block([[hm, hm], [hm, -hm]])
    h = (h.reshape(-1, 128).astype(np.float64) @ hm.astype(np.float64)).astype(np.float32) * np.float32(0.08838834764831845)
    h = h.reshape(rows, width)
    if not before:
        h = h * s
    return h.astype(dtype)


def exl3_apply(x: np.ndarray, trellis: np.ndarray, input_scales: np.ndarray, output_scales: np.ndarray, codebook: int):
    """EXL3Kernels.apply (EXL3.swift:83-106): rotate x (scales first) to fp16, multiply by the
    decoded W in fp32, rotate the fp32 product (scales last) to fp16."""
    xh = exl3_rotate(x, input_scales, True, np.float16)
    w = exl3_dequantize(trellis, codebook).astype(np.float64)
    yh = (xh.astype(np.float64) @ w).astype(np.float32)
    return exl3_rotate(yh, output_scales, False, np.float16)
