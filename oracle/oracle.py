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
