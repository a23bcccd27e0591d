"""The NVLink output exchange of N-sharded projections (ishi_exchange_* in the C ABI).

On one GPU the exchange degenerates to "the kernel writes its rows into the local [N, 8] array and
raises its own arrival word": that path is checked against the plain projection. With two or more
GPUs a two-process run (one rank per GPU) checks that every rank ends up with the whole output.
"""
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from ishizuki_b200 import synth
from ishizuki_b200 import _lib
from ishizuki_b200.interface import GGMLType, GGUFBlocks, IshizukiError, PackedLinear
from ishizuki_b200.sharding import OutputExchange

pytestmark = pytest.mark.gpu


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _projection(fmt, rng, n, k):
    if fmt == "q4_k":
        return PackedLinear(ggml=GGUFBlocks(dev(synth.q4k_blocks(rng, n, k)), GGMLType.q4K, (n, k)))
    if fmt == "q6_k":
        return PackedLinear(ggml=GGUFBlocks(dev(synth.q6k_blocks(rng, n, k)), GGMLType.q6K, (n, k)))
    if fmt in ("iq2_xs", "iq4_xs"):
        type_id = GGMLType.iq2Xs if fmt == "iq2_xs" else GGMLType.iq4Xs
        return PackedLinear(ggml=GGUFBlocks(dev(synth.ggml_blocks(rng, int(type_id), n, k)), type_id, (n, k)))
    if fmt == "affine8":  # the tcgen05 kernel: the product, then a publishing kernel
        w, s, b = synth.affine_pack(rng, n, k, 8, 64, np.float16)
        return PackedLinear(dev(w), dev(s), dev(b), None, 0, groupSize=64, bits=8)
    w, s, b = synth.affine_pack(rng, n, k, 4, 64, np.float16)
    return PackedLinear(dev(w), dev(s), dev(b), None, 0, groupSize=64, bits=4)


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "affine4", "iq2_xs", "iq4_xs", "affine8"])
@pytest.mark.parametrize("rows", [1, 5, 8])
def test_single_rank_exchange_matches_projection(rows, fmt):
    rng = np.random.default_rng(rows)
    n, k = 1000, 2048  # a ragged last panel
    lin = _projection(fmt, rng, n, k)
    ex = OutputExchange(4 << 20)
    off_a, view_a = ex.reserve(n)
    off_b, view_b = ex.reserve(n)
    x = dev(synth.activations(rng, rows, k))
    want = lin(x, transposed=True)
    for _ in range(3):  # the launch numbers advance; every call waits for the one before
        ex.apply(lin, x, off_a, 0)
        ex.apply(lin, x, off_b, 0)
    ex.wait()
    torch.cuda.synchronize()
    lin.ctx.poll()
    assert torch.equal(view_a[:, :rows], want)
    assert torch.equal(view_b[:, :rows], want)
    assert not view_a[:, rows:].any()
    ex.close()


def test_single_rank_exchange_of_thirteen_rows():
    """More than eight drafted rows: two launches, the pieces side by side in a [N, 16] array."""
    rng = np.random.default_rng(13)
    n, k, rows = 1000, 2048, 13
    lin = _projection("q4_k", rng, n, k)
    ex = OutputExchange(1 << 20)
    off, view = ex.reserve(n, rows)
    x = dev(synth.activations(rng, rows, k))
    want = lin(x, transposed=True)
    for _ in range(2):
        ex.apply(lin, x, off, 0)
    ex.wait()
    torch.cuda.synchronize()
    lin.ctx.poll()
    assert view.shape == (n, 16)
    assert torch.equal(view[:, :rows], want)
    assert not view[:, rows:].any()
    ex.close()


def test_single_rank_exchange_in_a_replayed_graph():
    rng = np.random.default_rng(7)
    n, k = 768, 1024
    w, s, b = synth.affine_pack(rng, n, k, 4, 64, np.float16)
    lin = PackedLinear(dev(w), dev(s), dev(b), None, 0, groupSize=64, bits=4)
    ex = OutputExchange(1 << 20)
    off, view = ex.reserve(n)
    x = dev(synth.activations(rng, 8, k))
    want = lin(x, transposed=True)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ex.apply(lin, x, off, 0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            ex.apply(lin, x, off, 0)
            ex.apply(lin, x, off, 0)
            ex.wait()
        for _ in range(4):
            view.zero_()
            graph.replay()
        torch.cuda.synchronize()
    lin.ctx.poll()
    assert torch.equal(view, want)
    ex.close()


def test_a_wait_nobody_answers_gives_up_and_reports():
    """Failure detection without a fault: the rank is made to expect one launch more than was
    issued, so the wait's arrival word never comes. The kernel must return after its bound, the
    context must report ISHI_E_TIMEOUT once, and the GPU must stay usable."""
    rng = np.random.default_rng(1)
    n, k = 256, 512
    lin = PackedLinear(ggml=GGUFBlocks(dev(synth.q4k_blocks(rng, n, k)), GGMLType.q4K, (n, k)))
    x = dev(synth.activations(rng, 8, k))
    want = lin(x, transposed=True)
    ex = OutputExchange(1 << 16)
    off, view = ex.reserve(n)
    ex.apply(lin, x, off, 0)
    assert ex.lib.ishi_exchange_debug_expect(ex.handle, 1) == _lib.OK
    t0 = time.time()
    ex.wait()
    torch.cuda.synchronize()
    assert time.time() - t0 < 20.0
    with pytest.raises(IshizukiError) as err:
        ex.ctx.poll()
    assert err.value.status == _lib.E_TIMEOUT
    ex.ctx.poll()  # reported once
    assert torch.equal(view, want)  # the rows of the launch that did happen are there
    assert torch.equal(lin(x, transposed=True), want)  # and the context still works
    ex.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_all_ranks_end_up_with_whole_outputs():
    """One rank per visible GPU: the NVLink exchange inside a replayed CUDA graph and the NCCL
    all-gather of the C ABI, both bit for bit against each shard recomputed locally."""
    world = min(torch.cuda.device_count(), 8)
    world = 1 << (world.bit_length() - 1)  # 2, 4 or 8
    script = os.path.join(os.path.dirname(__file__), "exchange_ranks.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world, "--master-addr",
           "127.0.0.1", "--master-port", "29533", script]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    assert done.stdout.count("exchange ok") == world
    assert done.stdout.count("all-gather ok") == world
