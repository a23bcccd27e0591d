"""Seeded synthetic weights and activations with the shapes and value distributions of the
benchmark configurations (numpy, host side). Real GGUF files and packs are not available where
this library is built, so these stand in for them in tests and in bench.py.

Every generator takes a numpy Generator so callers control the seed and the draw order.
"""
from __future__ import annotations

import numpy as np

Q2_K, Q4_K, Q6_K, IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ4_XS, IQ1_M = 10, 12, 14, 16, 17, 18, 19, 21, 22, 23, 29
TYPE_SIZE = {Q2_K: 84, Q4_K: 144, Q6_K: 210, IQ2_XXS: 66, IQ2_XS: 74, IQ3_XXS: 98, IQ1_S: 50, IQ3_S: 110, IQ2_S: 82,
             IQ4_XS: 136, IQ1_M: 56}
# byte offsets of the fp16 block scales of every type but IQ1_M (whose scale is spread over four words)
_SCALE_AT = {Q2_K: (80, 82), Q4_K: (0, 2), Q6_K: (208,), IQ2_XXS: (0,), IQ2_XS: (0,), IQ3_XXS: (0,), IQ1_S: (0,), IQ3_S: (0,),
             IQ2_S: (0,), IQ4_XS: (0,)}


def _half_bytes(values: np.ndarray) -> np.ndarray:
    return values.astype(np.float16).view(np.uint8).reshape(values.shape + (2,))


def q4k_blocks(rng: np.random.Generator, n: int, k: int, d_scale: float = 2e-3) -> np.ndarray:
    """[n][k/256][144] bytes: d, dmin = fp16 |N(0,1)| * d_scale, uniform scale bytes (each 6-bit
    field is then uniform in 0..63) and uniform 4-bit codes."""
    nb = n * (k // 256)
    out = rng.integers(0, 256, size=(nb, 144), dtype=np.uint8)
    out[:, 0:2] = _half_bytes(np.abs(rng.standard_normal(nb)) * d_scale)
    out[:, 2:4] = _half_bytes(np.abs(rng.standard_normal(nb)) * d_scale)
    return out.reshape(-1)


def iq2xs_blocks(rng: np.random.Generator, n: int, k: int, d_scale: float = 1e-2) -> np.ndarray:
    """[n][k/256][74] bytes: d = fp16 |N(0,1)| * d_scale, 32 uniform u16 (9-bit grid index and
    7 sign bits), eight uniform scale bytes (two 4-bit sub-scales each)."""
    nb = n * (k // 256)
    out = rng.integers(0, 256, size=(nb, 74), dtype=np.uint8)
    out[:, 0:2] = _half_bytes(np.abs(rng.standard_normal(nb)) * d_scale)
    return out.reshape(-1)


def q6k_blocks(rng: np.random.Generator, n: int, k: int, d_scale: float = 1e-4) -> np.ndarray:
    """[n][k/256][210] bytes: uniform 6-bit codes and int8 sub-scales, d = fp16 |N(0,1)| * d_scale."""
    nb = n * (k // 256)
    out = rng.integers(0, 256, size=(nb, 210), dtype=np.uint8)
    out[:, 208:210] = _half_bytes(np.abs(rng.standard_normal(nb)) * d_scale)
    return out.reshape(-1)


def other_blocks(rng: np.random.Generator, type_id: int, n: int, k: int, d_scale: float = 2e-3) -> np.ndarray:
    """[n][k/256][type size] bytes of any block type: uniform random bytes with the fp16 block
    scales set to |N(0,1)| * d_scale (for IQ1_M the scale's four nibbles sit on top of its words)."""
    nb = n * (k // 256)
    ts = TYPE_SIZE[type_id]
    out = rng.integers(0, 256, size=(nb, ts), dtype=np.uint8)
    if type_id == IQ1_M:
        d = (np.abs(rng.standard_normal(nb)) * d_scale).astype(np.float16).view(np.uint16)
        words = out[:, 48:56].copy().view("<u2")  # [nb, 4]
        for i in range(4):
            words[:, i] = (words[:, i] & 0x0FFF) | (((d >> (4 * i)) & 0xF) << 12).astype(np.uint16)
        out[:, 48:56] = words.view(np.uint8)
    else:
        for at in _SCALE_AT[type_id]:
            out[:, at:at + 2] = _half_bytes(np.abs(rng.standard_normal(nb)) * d_scale)
    return out.reshape(-1)


def ggml_blocks(rng: np.random.Generator, type_id: int, n: int, k: int) -> np.ndarray:
    special = {Q4_K: q4k_blocks, Q6_K: q6k_blocks, IQ2_XS: iq2xs_blocks}
    if type_id in special:
        return special[type_id](rng, n, k)
    return other_blocks(rng, type_id, n, k)


def lcg_blocks(type_id: int, rows: int, k: int, seed: int) -> np.ndarray:
    """Block bytes as the reference's kernel tests draw them
    (Tests/IshizukiKitTests/GGMLKernelTests.swift:102-109): a 64-bit LCG, one byte per step, bit 6
    cleared so that no two bytes form an fp16 with a saturated exponent."""
    count = rows * (k // 256) * TYPE_SIZE[type_id]
    out = np.empty(count, dtype=np.uint8)
    state = seed & 0xFFFFFFFFFFFFFFFF
    for i in range(count):
        state = (state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = (state >> 33) & 0xBF
    return out


def pack_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    """[n, k] integer codes to MLX's affine layout: code i of a row at bit i * bits of the row's
    little-endian uint32 stream (Sources/IshizukiKit/Quantize/WeightedAffineQuantizer.swift:142-161)."""
    n, k = codes.shape
    assert (k * bits) % 32 == 0
    if 32 % bits == 0:
        per = 32 // bits
        shifts = (np.arange(per, dtype=np.uint64) * bits)[None, None, :]
        words = (codes.reshape(n, k // per, per).astype(np.uint64) << shifts).sum(axis=-1)
        return words.astype(np.uint32)
    bitsarr = ((codes[:, :, None].astype(np.uint32) >> np.arange(bits, dtype=np.uint32)) & 1).reshape(n, -1, 32)
    return (bitsarr.astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(axis=-1).astype(np.uint32)


def affine_pack(rng: np.random.Generator, n: int, k: int, bits: int = 4, group_size: int = 64,
                scale_dtype=np.float16):
    """Uniform codes; scales |N(0,1)| * 0.01; biases -2^(bits-1) * scale + N(0, 1e-3)."""
    codes = rng.integers(0, 1 << bits, size=(n, k), dtype=np.uint32)
    scales = (np.abs(rng.standard_normal((n, k // group_size))) * 0.01).astype(scale_dtype)
    biases = (-(1 << (bits - 1)) * scales.astype(np.float32)
              + rng.standard_normal((n, k // group_size)) * 1e-3).astype(scale_dtype)
    return pack_codes(codes, bits), scales, biases


def to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = values.astype(np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def ternary_pack(rng: np.random.Generator, n: int, k: int, group_size: int = 128):
    """Bonsai-style ternary 2-bit pack: codes {0,1,2} with probabilities .3/.4/.3, sixteen per
    uint32, bf16 scales |N(0,1)| * 0.02 (returned as uint16 bit patterns) and bias = -scale."""
    codes = rng.choice(np.array([0, 1, 2], dtype=np.uint32), size=(n, k), p=[0.3, 0.4, 0.3])
    s = np.abs(rng.standard_normal((n, k // group_size))) * 0.02
    sbits = to_bf16_bits(s)
    bbits = sbits ^ np.uint16(0x8000)
    return pack_codes(codes, 2), sbits, bbits


def activations(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    return rng.standard_normal((m, k)).astype(np.float16)
