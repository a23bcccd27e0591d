"""GGUF block kernels on the GPU against the CPU oracle and the reference's fixture.

Mirrors Tests/IshizukiKitTests/GGMLKernelTests.swift: the decode is held to the reference bit
for bit, and the fused products are compared with "expand the weight and multiply".
"""
import numpy as np
import pytest
import torch

from ishizuki_b200 import synth
from ishizuki_b200.interface import GGMLKernels, GGMLType, GGUFBlocks, PackedLinear
from oracle import oracle

pytestmark = pytest.mark.gpu

TYPES = [GGMLType.q4K, GGMLType.q6K, GGMLType.iq2Xs]
MATMUL_TYPES = [GGMLType.q4K, GGMLType.q6K, GGMLType.iq2Xs]
TOL = 2e-3  # max |got - want| / max |want|, fp16 output, fp32 accumulate


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same_bits(got: np.ndarray, want: np.ndarray) -> bool:
    return bool(((got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))).all())


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    return float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max() / np.abs(want).max())


@pytest.mark.parametrize("type_id", TYPES)
def test_decode_matches_ggml_fixture(ggml_fixture, type_id):
    blocks, want = ggml_fixture[int(type_id)]
    got = GGMLKernels.dequantize(dev(blocks), type_id, [want.size], dtype=torch.float32)
    assert got is not None
    assert same_bits(got.cpu().numpy(), want)


@pytest.mark.parametrize("type_id", TYPES)
def test_decode_matches_oracle_on_a_projection(type_id):
    rng = np.random.default_rng(11)
    n, k = 1024, 5120
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    got = GGMLKernels.dequantize(dev(blocks), type_id, [n, k], dtype=torch.float32)
    want = oracle.dequantize(int(type_id), blocks).reshape(n, k)
    assert same_bits(got.cpu().numpy(), want)
    half = GGMLKernels.dequantize(dev(blocks), type_id, [n, k], dtype=torch.float16)
    assert np.array_equal(half.cpu().numpy().view(np.uint16), want.astype(np.float16).view(np.uint16))


def test_decode_refuses_what_the_reference_refuses():
    blocks = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    assert GGMLKernels.dequantize(blocks, 11, [256]) is None  # Q3_K: no decoder
    assert GGMLKernels.dequantize(blocks, GGMLType.iq2Xs, [100]) is None  # not whole blocks
    assert GGMLKernels.dequantize(blocks[:73], GGMLType.iq2Xs, [256]) is None  # short buffer


@pytest.mark.parametrize("type_id", MATMUL_TYPES)
@pytest.mark.parametrize("m", list(range(1, 17)))
def test_few_row_product_ragged_tile(type_id, m):
    """K = 512, N = 17 (a ragged tile), the reference's LCG bytes, every row count 1...16
    (GGMLKernelTests.swift:111-175)."""
    k, n = 512, 17
    blocks = synth.lcg_blocks(int(type_id), n, k, 0xFE11)
    x = synth.activations(np.random.default_rng(m), m, k)
    got = GGMLKernels.matmulFew(dev(x), dev(blocks), type_id, n)
    assert got is not None and got.shape == (m, n)
    assert torch.equal(got, GGMLKernels.matvec(dev(x), dev(blocks), type_id, n))
    want32, want16 = oracle.ggml_matmul(int(type_id), blocks, x, n)
    gotn = got.cpu().numpy()
    # random block bytes can decode to weights whose products overflow fp16: those outputs must
    # be the same infinities the rounded oracle has, the rest are compared as numbers
    finite = np.isfinite(want16.astype(np.float32))
    assert np.array_equal(gotn[~finite].view(np.uint16), want16[~finite].view(np.uint16))
    # per element against the sum of the magnitudes that formed it (the reference's yardstick),
    # loosened from 1e-5 to fp16 output precision
    w = np.abs(oracle.dequantize(int(type_id), blocks).reshape(n, k))
    bound = np.abs(x.astype(np.float32)) @ w.T
    err = np.abs(gotn.astype(np.float32) - want32)[finite] / np.maximum(bound, 1e-6)[finite]
    assert err.max() < 1e-3
    assert rel_err(gotn[finite], want32[finite]) < TOL


@pytest.mark.parametrize("type_id", MATMUL_TYPES)
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408), (1024, 5120), (6144, 5120), (5120, 6144)])
@pytest.mark.parametrize("m", [1, 8, 16])
def test_projection_shapes(type_id, n, k, m):
    rng = np.random.default_rng(n + k + m)
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    x = synth.activations(rng, m, k)
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks), type_id, (n, k)))
    y = lin(dev(x))
    torch.cuda.synchronize()
    lin.ctx.poll()
    want32, _ = oracle.ggml_matmul(int(type_id), blocks, x, n)
    assert rel_err(y.cpu().numpy(), want32) < TOL
    # a second call reuses the projection's scratch and must give the same bits
    y2 = lin(dev(x))
    assert torch.equal(y, y2)
    yt = lin(dev(x), transposed=True)
    assert torch.equal(yt.t().contiguous(), y)


def test_product_guards():
    blocks = torch.zeros(4 * 74, dtype=torch.uint8, device="cuda")
    wide = torch.zeros((17, 256), dtype=torch.float16, device="cuda")
    assert GGMLKernels.matmulFew(wide, blocks, GGMLType.q4K, 1) is None  # too many rows
    assert GGMLKernels.matvec(wide, blocks, GGMLType.iq2Xs, 4) is None
    ragged = torch.zeros((1, 100), dtype=torch.float16, device="cuda")
    assert GGMLKernels.matmulFew(ragged, blocks, GGMLType.q4K, 1) is None  # k not whole blocks
    x = torch.zeros((1, 256), dtype=torch.float16, device="cuda")
    assert GGMLKernels.matmulFew(x, blocks, GGMLType.q4K, 4) is None  # buffer too short for 4 rows


def test_host_buffer_entry_points_agree():
    """apply_host (waits) and apply_host_async (one synchronisation for several calls) give the
    device path's result."""
    rng = np.random.default_rng(5)
    n, k = 1536, 2048
    lin = PackedLinear(ggml=GGUFBlocks(dev(synth.q4k_blocks(rng, n, k)), GGMLType.q4K, (n, k)))
    xs = [synth.activations(rng, m, k) for m in (1, 8, 13)]
    want = [lin(dev(x)).cpu() for x in xs]
    outs = [torch.empty((x.shape[0], n), dtype=torch.float16).pin_memory() for x in xs]
    pinned = [torch.from_numpy(x).pin_memory() for x in xs]
    for xh, yh in zip(pinned, outs):
        lin.apply_host_async(xh, yh)
    torch.cuda.current_stream().synchronize()
    lin.ctx.poll()
    for yh, w, x in zip(outs, want, xs):
        assert torch.equal(yh, w)
        y2 = np.empty((x.shape[0], n), dtype=np.float16)
        lin.apply_host(x, y2)
        assert np.array_equal(y2.view(np.uint16), w.numpy().view(np.uint16))


@pytest.mark.parametrize("plan", ["1,2,1", "1,3,2", "2,1,2", "2,2,4", "3,1,2", "4,2,2", "5,1,4", "8,1,4"])
def test_every_launch_plan_gives_the_same_product(plan, monkeypatch):
    """The warp-level kernel under forced launch plans (K split = cluster size, units per warp,
    panels in parallel), on a shape with a ragged last panel and an uneven K split."""
    monkeypatch.setenv("ISHI_FRAG_PLAN", plan)
    rng = np.random.default_rng(21)
    n, k = 1000, 5120 + 256
    blocks = synth.q4k_blocks(rng, n, k)
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks), GGMLType.q4K, (n, k)))
    for m in (1, 8, 11):
        x = synth.activations(rng, m, k)
        got = lin(dev(x)).cpu().numpy()
        want32, _ = oracle.ggml_matmul(int(GGMLType.q4K), blocks, x, n)
        err = float(np.abs(got.astype(np.float64) - want32.astype(np.float64)).max() / np.abs(want32).max())
        assert err < 2e-3, (plan, m, err)
    lin.ctx.poll()
