#!/usr/bin/env python3
"""Copies the reference's golden vectors for the verify-matmul path into tests/golden/.

Run once in a container that has the reference checkout; the outputs are committed because the
reference tree is not present where the GPU tests run.

  ggml-reference.bin    verbatim copy of Tests/IshizukiKitTests/Fixtures/ggml-reference.bin
                        (ggml's own to_float on 8 pseudo-random blocks of each of 14 types,
                        written by Scripts/gen-ggml-reference.c: "GGMLREF1", u32 count, then per
                        type {u32 type, u32 nblocks, u32 raw bytes, u32 n floats, raw, f32[]}).
  hadamard_case1.npz    case1_x and case1_hadamard ([3, 5120] fp16 each) out of
                        Tests/Golden/hadamard_golden.safetensors: an activation and its
                        block-1024 rotated form, plus the +-1 sign vector recovered from them
                        (the pack's own sign tensor is not in the reference tree).

  exl3_reference.npz    every array of Tests/IshizukiKitTests/Fixtures/exl3-reference.safetensors:
                        eleven EXL3 trellis tensors "r<bits>[h5]c<codebook>" (int16 [k/16, n/16,
                        16 * bits]) with the exllamav3 reconstruction of each ("expected", fp32
                        [k, n]), and one projection of two checkpoints ("qwen3": codebook 3INST,
                        "qwen38": mul1) with trellis, input / output scale vectors and the fp16
                        weight it was quantized from.

Usage: python tests/golden/make_golden.py /path/to/reference
"""
import pathlib
import shutil
import sys

import numpy as np


def sylvester(n: int) -> np.ndarray:
    h = np.array([[1.0]])
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return h


def main() -> None:
    ref = pathlib.Path(sys.argv[1])
    here = pathlib.Path(__file__).parent
    shutil.copyfile(ref / "Tests/IshizukiKitTests/Fixtures/ggml-reference.bin",
                    here / "ggml-reference.bin")

    from safetensors import safe_open

    with safe_open(str(ref / "Tests/Golden/hadamard_golden.safetensors"), "np") as f:
        x = f.get_tensor("case1_x")
        h = f.get_tensor("case1_hadamard")
    # y = WHT(x * s) / sqrt(B)  =>  x * s = WHT(y) / sqrt(B): the signs are the signs of the
    # inverse transform of the rotated rows divided by x, agreed on by all three rows.
    block = 1024
    H = sylvester(block) / np.sqrt(block)
    back = (h.astype(np.float64).reshape(3, -1, block) @ H).reshape(3, -1)
    ratio = back / np.where(x == 0, 1, x.astype(np.float64))
    signs = np.sign(np.median(ratio, axis=0)).astype(np.float32)
    assert np.all(np.abs(signs) == 1)
    np.savez_compressed(here / "hadamard_case1.npz", x=x, rotated=h, signs=signs,
                        block=np.int32(block))
    print("negatives in sign vector:", int((signs < 0).sum()))

    with safe_open(str(ref / "Tests/IshizukiKitTests/Fixtures/exl3-reference.safetensors"), "np") as f:
        arrays = {name: f.get_tensor(name) for name in f.keys()}
    np.savez_compressed(here / "exl3_reference.npz", **arrays)
    print("EXL3 arrays:", len(arrays))


if __name__ == "__main__":
    main()
