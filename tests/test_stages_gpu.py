"""The layer stages around the projections: RMS norm ahead of q/k/v and gate/up (its own launch in
the dependent-launch chain). silu(gate) * up is covered with the gated pair in test_ggml_gpu.py."""
import numpy as np
import pytest
import torch

from ishizuki_b200 import _lib, synth
from ishizuki_b200.interface import FusedLinear, GGMLType, GGUFBlocks, IshizukiError, rmsNorm
from oracle import oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,width", [(1, 5120), (8, 5120), (13, 1024), (3, 8192), (2, 200)])
@pytest.mark.parametrize("xdt,wdt", [(np.float32, np.float16), (np.float16, np.float32), (np.float32, np.float32)])
def test_rms_norm_matches_the_oracle(rows, width, xdt, wdt):
    rng = np.random.default_rng(rows * width)
    x = (rng.standard_normal((rows, width)) * 3).astype(xdt)
    x[0, 5] = 900.0  # an outlier of the residual stream
    w = (1 + 0.1 * rng.standard_normal(width)).astype(wdt)
    got = rmsNorm(dev(x), dev(w), 1e-6).cpu().numpy()
    want = oracle.rms_norm(x, w, 1e-6)
    # fp32 sums in another order: a unit in the last place of fp16 at most
    diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert np.all(diff <= np.abs(want.astype(np.float32)) * 2.0 ** -10 + 1e-7)
    assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.01


def test_norm_then_stacked_projection_in_one_graph():
    """rmsNorm -> q+k+v as consecutive dependent launches, captured and replayed: the product of the
    normalised rows, against the oracle's."""
    rng = np.random.default_rng(4)
    k, sizes = 2048, (512, 128, 128)
    parts = [synth.q4k_blocks(rng, n, k) for n in sizes]
    fused = FusedLinear([GGUFBlocks(dev(b), GGMLType.q4K, (n, k)) for b, n in zip(parts, sizes)])
    x = (rng.standard_normal((8, k)) * 2).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    xd, wd = dev(x), dev(w)
    y = torch.empty((8, sum(sizes)), dtype=torch.float16, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fused(rmsNorm(xd, wd, 1e-6), out=y)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            normed = rmsNorm(xd, wd, 1e-6)
            fused(normed, out=y)
        y.zero_()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    fused.ctx.poll()
    xn = oracle.rms_norm(x, w, 1e-6)
    for piece, blocks, n in zip(fused.split(y), parts, sizes):
        want32, _ = oracle.ggml_matmul(int(GGMLType.q4K), blocks, xn, n)
        assert float(np.abs(piece.cpu().numpy().astype(np.float64) - want32).max() / np.abs(want32).max()) < 2e-3


def test_rms_norm_guards():
    x = dev(np.zeros((2, 8200), dtype=np.float32))
    w = dev(np.ones(8200, dtype=np.float16))
    with pytest.raises(IshizukiError) as err:
        rmsNorm(x, w, 1e-6)  # wider than the kernel keeps in registers
    assert err.value.status == _lib.E_SHAPE
