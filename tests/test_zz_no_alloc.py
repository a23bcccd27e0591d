"""The entry point for hosts that cannot allocate device memory, against the ordinary one.

ishi_q4k_matmul_few_static takes no context and no projection: a caller that owns nothing but the
input and output buffers it was handed (a plugin inside a runtime that reserved the GPU, a loop
that may not allocate after start-up) passes x, the raw Q4_K blocks and y, and the kernel's
scratch is a fixed array inside the library. It must give what ishi_ggml_matmul_few gives, on
repeated calls, because the array carries the previous call's contents into the next one.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from ishizuki_b200 import _lib, synth
from ishizuki_b200.interface import GGMLKernels, GGMLType
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def static_product(x: torch.Tensor, blocks: torch.Tensor, n: int) -> tuple[int, torch.Tensor]:
    lib = _lib.load()
    m, k = x.shape
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ishi_q4k_matmul_few_static(ctypes.c_void_p(x.data_ptr()), m, ctypes.c_void_p(blocks.data_ptr()),
                                        blocks.numel(), n, k, ctypes.c_void_p(y.data_ptr()), stream)
    return rc, y


@pytest.mark.parametrize("n,k,m", [(1024, 5120, 8), (17, 512, 3), (4096, 4096, 16)])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(n, k, m):
    torch.cuda.set_device(0)
    rng = np.random.default_rng(n + m)
    blocks = dev(synth.q4k_blocks(rng, n, k))
    results = []
    for call in range(2):  # the second call finds the first one's leftovers in the array
        x = dev(synth.activations(rng, m, k))
        rc, got = static_product(x, blocks, n)
        assert rc == _lib.OK, _lib.load().ishi_status_string(rc).decode()
        want = GGMLKernels.matmulFew(x, blocks, GGMLType.q4K, n)
        torch.cuda.synchronize()
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.abs(g - w).max() <= TOL * np.abs(w).max()
        # ... and what the CPU oracle gives (this entry point runs its own decoder)
        want32, _ = oracle.ggml_matmul(oracle.Q4_K, blocks.cpu().numpy(), x.cpu().numpy(), n)
        assert np.abs(g - want32).max() <= TOL * np.abs(want32).max()
        results.append(g)
    assert not np.array_equal(results[0], results[1])  # different activations, different answers


def test_a_weight_beyond_the_built_in_scratch_is_refused():
    torch.cuda.set_device(0)
    n, k = 17408, 5120  # 50 MB of blocks: more than the array's 12 MiB for the tiled copy
    blocks = torch.zeros(n * (k // 256) * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros((8, k), dtype=torch.float16, device="cuda")
    rc, y = static_product(x, blocks, n)
    assert rc == _lib.E_TOO_LARGE
    assert "scratch" in _lib.load().ishi_status_string(rc).decode()
    assert float(y.abs().max()) == 0.0  # nothing was launched
