"""EXL3 trellis-coded projections through the C ABI against the oracle and the reference's fixture
(reference tests: Tests/IshizukiKitTests/EXL3Tests.swift)."""
import numpy as np
import pytest
import torch

from ishizuki_b200 import _lib
from ishizuki_b200.interface import EXL3Kernels, EXL3Tensor, IshizukiError
from oracle import oracle

pytestmark = pytest.mark.gpu

RATES = [("r1c0", 0), ("r2c1", 1), ("r3c2", 2), ("r4c0", 0), ("r5c2", 2), ("r6c1", 1), ("r7c2", 2), ("r8c0", 0),
         ("r1h5c2", 2), ("r2h5c2", 2), ("r3h5c2", 2)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def padded(trellis: np.ndarray) -> np.ndarray:
    """The fixture's 32 x 48 tensors padded with zero tiles to whole 128 blocks, as the reference's test does."""
    tk, tn, words = trellis.shape
    out = np.zeros(((tk * 16 + 127) // 128 * 8, (tn * 16 + 127) // 128 * 8, words), dtype=np.int16)
    out[:tk, :tn] = trellis
    return out


@pytest.mark.parametrize("name,codebook", RATES)
def test_decode_is_bit_exact_on_the_reference_fixture(golden_dir, name, codebook):
    # EXL3Tests.decodeMatchesReference
    g = np.load(golden_dir / "exl3_reference.npz")
    want = g[name + ".expected"]
    t = EXL3Tensor(dev(padded(g[name + ".trellis"])), None, None, codebook)
    for dtype in (torch.float32, torch.float16):
        w = EXL3Kernels.dequantize(t, dtype).float().cpu().numpy()
        assert np.array_equal(w[: want.shape[0], : want.shape[1]].view(np.uint32), want.view(np.uint32))


def random_trellis(rng, k, n, words):
    return rng.integers(-32768, 32768, size=(k // 16, n // 16, words), dtype=np.int16)


@pytest.mark.parametrize("words,codebook", [(16, 0), (32, 1), (48, 2), (64, 0), (64, 2), (96, 1), (128, 0), (24, 2), (40, 2), (56, 2)])
def test_decode_and_product_on_random_trellises(words, codebook):
    """Every rate on a larger random tensor: the decode bit for bit against the oracle, the fused
    product against the expanded weight with the reference's bound (EXL3Tests.matvecMatchesExpanded:
    |y - x W| / max(|x| |W|) < 1e-5), for every row count."""
    rng = np.random.default_rng(words * 3 + codebook)
    k, n = 1024, 384
    trellis = random_trellis(rng, k, n, words)
    t = EXL3Tensor(dev(trellis), None, None, codebook)
    want_w = oracle.exl3_dequantize(trellis, codebook)
    w = EXL3Kernels.dequantize(t, torch.float32).cpu().numpy()
    assert np.array_equal(w.view(np.uint32), want_w.view(np.uint32))
    for m in (1, 2, 5, 8):
        x = rng.standard_normal((m, k)).astype(np.float16)
        y = EXL3Kernels.matvec(dev(x), t).cpu().numpy()
        want = x.astype(np.float64) @ want_w.astype(np.float64)
        bound = (np.abs(x).astype(np.float64) @ np.abs(want_w).astype(np.float64)).max()
        assert np.abs(y - want).max() / bound < 1e-5
    assert EXL3Kernels.matvec(dev(rng.standard_normal((9, k)).astype(np.float16)), t) is None


@pytest.mark.parametrize("n", [8192, 17408])
def test_product_with_several_tile_columns_per_block(n):
    """Wide outputs: a thread block takes two or four adjacent tile columns. Checked against the
    expanded weight (whose decode the tests above hold to the oracle bit for bit)."""
    rng = np.random.default_rng(n)
    k = 512
    for words, codebook in ((64, EXL3Tensor.mul1), (48, EXL3Tensor.threeInst)):
        trellis = random_trellis(rng, k, n, words)
        t = EXL3Tensor(dev(trellis), None, None, codebook)
        w = EXL3Kernels.dequantize(t, torch.float32).double()
        sample = oracle.exl3_dequantize(trellis[:, :16], codebook)  # the first 256 columns against the oracle
        assert np.array_equal(w[:, :256].float().cpu().numpy().view(np.uint32), sample.view(np.uint32))
        for m in (1, 8):
            x = dev(rng.standard_normal((m, k)).astype(np.float16))
            y = EXL3Kernels.matvec(x, t).double()
            want = x.double() @ w
            bound = (x.double().abs() @ w.abs()).max()
            assert float((y - want).abs().max() / bound) < 1e-5


def test_rotation_matches_the_oracle():
    # EXL3Tests.rotationMatchesHadamard
    rng = np.random.default_rng(5)
    for rows, width in ((1, 5120), (7, 1024), (40, 256)):
        x = rng.standard_normal((rows, width)).astype(np.float32)
        s = rng.standard_normal(width).astype(np.float16)
        for before in (True, False):
            got = EXL3Kernels.rotate(dev(x), dev(s), before, torch.float32).cpu().numpy()
            assert np.abs(got - oracle.exl3_rotate(x, s, before, np.float32)).max() < 1e-4
            got16 = EXL3Kernels.rotate(dev(x.astype(np.float16)), dev(s), before, torch.float16).cpu().numpy()
            want16 = oracle.exl3_rotate(x.astype(np.float16), s, before, np.float16)
            assert np.abs(got16.astype(np.float32) - want16.astype(np.float32)).max() <= 2.0 ** -9 * np.abs(want16).max()


def test_projection_reproduces_its_checkpoint(golden_dir):
    # EXL3Tests.projectionMatchesCheckpoint: both rotations around the product; drift against the
    # fp16 weight the projection was quantized from below 0.12, and the oracle's apply within 2e-3
    g = np.load(golden_dir / "exl3_reference.npz")
    rng = np.random.default_rng(3)
    for name, codebook in (("qwen3", EXL3Tensor.threeInst), ("qwen38", EXL3Tensor.mul1)):
        t = EXL3Tensor(dev(g[name + ".trellis"]), dev(g[name + ".suh"]), dev(g[name + ".svh"]), codebook)
        batch = rng.standard_normal((16, 128)).astype(np.float16)
        for rows in (1, 5, 12, 16):
            x = batch[:rows]
            y = EXL3Kernels.apply(dev(x), t).float().cpu().numpy()
            want = x.astype(np.float64) @ g[name + ".weight"].astype(np.float64)
            assert np.sqrt(((y - want) ** 2).sum() / (want ** 2).sum()) < 0.12
            exact = oracle.exl3_apply(x, g[name + ".trellis"], g[name + ".suh"], g[name + ".svh"], codebook).astype(np.float32)
            assert np.abs(y - exact).max() / np.abs(exact).max() < 2e-3


def test_projection_at_a_model_shape():
    """A 4-bit projection of the 27B hidden size through apply, against the oracle."""
    rng = np.random.default_rng(8)
    k, n = 5120, 1024
    trellis = random_trellis(rng, k, n, 64)
    su = np.where(rng.random(k) < 0.5, -1, 1).astype(np.float16)
    sv = np.where(rng.random(n) < 0.5, -1, 1).astype(np.float16)
    t = EXL3Tensor(dev(trellis), dev(su), dev(sv), EXL3Tensor.mul1)
    for rows in (1, 8, 13):
        x = rng.standard_normal((rows, k)).astype(np.float16)
        y = EXL3Kernels.apply(dev(x), t).float().cpu().numpy()
        want = oracle.exl3_apply(x, trellis, su, sv, EXL3Tensor.mul1).astype(np.float32)
        assert np.abs(y - want).max() / np.abs(want).max() < 2e-3


def test_guards():
    rng = np.random.default_rng(1)
    ok = random_trellis(rng, 128, 128, 64)
    with pytest.raises(IshizukiError) as err:
        EXL3Kernels.dequantize(EXL3Tensor(dev(random_trellis(rng, 128, 128, 72)), None, None, 0))  # 4.5 bits is not a rate
    assert err.value.status == _lib.E_UNSUPPORTED
    with pytest.raises(IshizukiError) as err:
        EXL3Kernels.dequantize(EXL3Tensor(dev(random_trellis(rng, 128, 128, 24)), None, None, 0))  # half rates need mul1
    assert err.value.status == _lib.E_UNSUPPORTED
    with pytest.raises(IshizukiError) as err:
        EXL3Kernels.dequantize(EXL3Tensor(dev(random_trellis(rng, 64, 128, 64)), None, None, 0))  # k not a multiple of 128
    assert err.value.status == _lib.E_SHAPE
    t = EXL3Tensor(dev(ok), None, None, 0)
    with pytest.raises(IshizukiError) as err:
        EXL3Kernels.apply(dev(rng.standard_normal((2, 128)).astype(np.float16)), t)  # no scale vectors
    assert err.value.status == _lib.E_INVALID
    s = dev(np.ones(128, dtype=np.float16))
    with pytest.raises(IshizukiError) as err:
        EXL3Kernels.apply(dev(rng.standard_normal((17, 128)).astype(np.float16)), EXL3Tensor(dev(ok), s, s, 0))
    assert err.value.status == _lib.E_SHAPE
