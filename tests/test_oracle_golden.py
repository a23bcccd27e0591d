"""The CPU oracle against the reference's own golden vectors (no GPU)."""
import numpy as np
import pytest

from ishizuki_b200 import synth
from oracle import oracle


def _same_bits(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    return (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))


ALL_TYPES = sorted(oracle.TYPE_SIZE)  # the eleven quantized block types of GGMLDequant.supported


@pytest.mark.parametrize("type_id", ALL_TYPES)
def test_dequant_matches_ggml_bit_for_bit(ggml_fixture, type_id):
    # Tests/IshizukiKitTests/GGMLDequantTests.swift:60-85: bit patterns equal, NaN == NaN
    blocks, want = ggml_fixture[type_id]
    got = oracle.dequantize(type_id, blocks)
    assert got.shape == want.shape
    assert _same_bits(got, want).all()


def test_fixture_has_the_fourteen_types(ggml_fixture):
    assert sorted(ggml_fixture) == [0, 1, 10, 12, 14, 16, 17, 18, 19, 21, 22, 23, 29, 30]
    for type_id, size in oracle.TYPE_SIZE.items():
        assert ggml_fixture[type_id][0].size == 8 * size  # GGUFTests.blockGeometry


@pytest.mark.parametrize("type_id", ALL_TYPES)
def test_dequant_matches_gguf_py(type_id):
    """ggml's own Python reference on larger seeded inputs (independent cross-check)."""
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(type_id)
    blocks = synth.ggml_blocks(rng, type_id, 8, 1024)
    want = gguf.quants.dequantize(blocks.reshape(-1, oracle.TYPE_SIZE[type_id]),
                                  gguf.GGMLQuantizationType(type_id)).reshape(-1)
    got = oracle.dequantize(type_id, blocks)
    assert _same_bits(got, want.astype(np.float32)).all()


def test_hadamard_matches_golden(golden_dir):
    g = np.load(golden_dir / "hadamard_case1.npz")
    got = oracle.hadamard_rotate(g["x"], int(g["block"]), g["signs"])
    # the golden rows were produced by MLX's transform; fp16 results agree to the last bit here
    assert np.array_equal(got.view(np.uint16), g["rotated"].view(np.uint16))


def test_hadamard_is_orthonormal():
    rng = np.random.default_rng(3)
    x = synth.activations(rng, 4, 1024)
    for block in (128, 256, 1024):
        y = oracle.hadamard_rotate(x, block)
        back = oracle.hadamard_rotate(y, block)  # H is symmetric and orthonormal: H(Hx) = x
        assert np.abs(back.astype(np.float32) - x.astype(np.float32)).max() < 4e-3


def test_affine_formula_and_packing():
    rng = np.random.default_rng(5)
    for bits, gs in [(2, 128), (4, 64), (4, 128), (8, 128), (3, 128)]:
        n, k = 8, 512
        codes = rng.integers(0, 1 << bits, size=(n, k), dtype=np.uint32)
        scales = (np.abs(rng.standard_normal((n, k // gs))) * 0.01).astype(np.float16)
        biases = (rng.standard_normal((n, k // gs)) * 0.01).astype(np.float16)
        w = synth.pack_codes(codes, bits)
        assert w.shape == (n, k * bits // 32)
        got = oracle.affine_dequantize(w, scales, biases, bits, gs)
        s = np.repeat(scales.astype(np.float32), gs, axis=1)
        b = np.repeat(biases.astype(np.float32), gs, axis=1)
        want = codes.astype(np.float32) * s + b  # VerifyMatmul.swift:286-287
        assert np.array_equal(got, want)


def test_reference_row_floor():
    # Tests/IshizukiKitTests/VerifyMatmulTests.swift:75-87
    def rows(n, k, bits=2):
        return oracle.reference_minimum_rows(n * k * bits // 8)

    assert rows(248_320, 5120) == 2
    assert rows(17_408, 5120) == 3
    assert rows(12_288, 5120) == 3
    assert rows(6144, 5120) == 4
    assert rows(1024, 5120) == 6
    assert rows(4096, 5120, bits=8) == 3
    assert rows(1024, 5120, bits=8) == 4


def test_matmul_agrees_with_numpy():
    rng = np.random.default_rng(7)
    blocks = synth.q4k_blocks(rng, 17, 512)
    x = synth.activations(rng, 5, 512)
    y32, y16 = oracle.ggml_matmul(oracle.Q4_K, blocks, x, 17)
    w = oracle.dequantize(oracle.Q4_K, blocks).reshape(17, 512)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(y32 - want).max() <= 1e-6 * np.abs(want).max()
    assert np.array_equal(y16, y32.astype(np.float16))


# The reference's EXL3 fixture (Tests/IshizukiKitTests/EXL3Tests.swift:23-27): rate and codebook per tensor
EXL3_RATES = [("r1c0", 0), ("r2c1", 1), ("r3c2", 2), ("r4c0", 0), ("r5c2", 2), ("r6c1", 1), ("r7c2", 2), ("r8c0", 0),
              ("r1h5c2", 2), ("r2h5c2", 2), ("r3h5c2", 2)]


def test_exl3_decode_is_bit_exact_on_the_reference_fixture(golden_dir):
    # EXL3Tests.decodeMatchesReference: every rate (1...8 bits and the half rates) and codebook
    g = np.load(golden_dir / "exl3_reference.npz")
    for name, codebook in EXL3_RATES:
        got = oracle.exl3_dequantize(g[name + ".trellis"], codebook)
        want = g[name + ".expected"]
        assert got.shape == want.shape
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name


def test_exl3_projection_reproduces_its_checkpoint(golden_dir):
    # EXL3Tests.projectionMatchesCheckpoint: relative drift below 0.12 against the fp16 weight the
    # projection was quantized from, both rotations included
    g = np.load(golden_dir / "exl3_reference.npz")
    rng = np.random.default_rng(3)
    for name, codebook in (("qwen3", oracle.EXL3_3INST), ("qwen38", oracle.EXL3_MUL1)):
        x = rng.standard_normal((12, 128)).astype(np.float16)
        y = oracle.exl3_apply(x, g[name + ".trellis"], g[name + ".suh"], g[name + ".svh"], codebook).astype(np.float64)
        want = x.astype(np.float64) @ g[name + ".weight"].astype(np.float64)
        assert np.sqrt(((y - want) ** 2).sum() / (want ** 2).sum()) < 0.12


def test_exl3_rotation_is_the_scaled_block_hadamard():
    # EXL3Tests.rotationMatchesHadamard
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 1024)).astype(np.float32)
    s = rng.standard_normal(1024).astype(np.float16)
    h = np.array([[1.0]])
    while h.shape[0] < 128:
        h = np.block([[h, h], [h, -h]])
    h /= np.sqrt(128.0)
    before = ((x * s.astype(np.float32)).reshape(-1, 128) @ h).reshape(7, 1024)
    after = (x.reshape(-1, 128) @ h).reshape(7, 1024) * s.astype(np.float32)
    assert np.abs(oracle.exl3_rotate(x, s, True, np.float32) - before).max() < 1e-4
    assert np.abs(oracle.exl3_rotate(x, s, False, np.float32) - after).max() < 1e-4
