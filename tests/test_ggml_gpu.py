"""GGUF block kernels on the GPU against the CPU oracle and the reference's fixture.

Mirrors Tests/IshizukiKitTests/GGMLKernelTests.swift: the decode is held to the reference bit
for bit, and the fused products are compared with "expand the weight and multiply".
"""
import numpy as np
import pytest
import torch

from ishizuki_b200 import synth
from ishizuki_b200 import _lib
from ishizuki_b200.interface import BonsaiRuntime, FusedLinear, GGMLKernels, GGMLType, GGUFBlocks, IshizukiError, PackedLinear
from oracle import oracle

pytestmark = pytest.mark.gpu

TYPES = list(GGMLType)  # all eleven block formats the reference reads
MATMUL_TYPES = list(GGMLType)
STREAMED = [GGMLType.q4K, GGMLType.q6K, GGMLType.iq2Xs]  # formats with a streaming product kernel
OTHERS = [t for t in GGMLType if t not in STREAMED]
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


@pytest.mark.parametrize("type_id", STREAMED)
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408), (1024, 5120), (6144, 5120), (5120, 6144)])
@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
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


@pytest.mark.parametrize("type_id", STREAMED)
def test_properties_at_full_size(type_id):
    """Size-independent properties on the benchmark's gate shape: doubling the activations doubles
    every output exactly (powers of two pass through fp16 and fp32 unchanged), a zero row gives
    zeros, the rows of x do not influence each other, and the product is additive in x within
    the fp16 tolerance."""
    n, k = 17408, 5120
    rng = np.random.default_rng(int(type_id))
    lin = PackedLinear(ggml=GGUFBlocks(dev(synth.ggml_blocks(rng, int(type_id), n, k)), type_id, (n, k)))
    x = dev(synth.activations(rng, 8, k))
    y = lin(x)
    assert torch.equal(lin(x * 2), y * 2)
    x0 = x.clone()
    x0[3] = 0
    y0 = lin(x0)
    assert not y0[3].any()
    assert torch.equal(y0[[0, 1, 2, 4, 5, 6, 7]], y[[0, 1, 2, 4, 5, 6, 7]])
    assert torch.equal(lin(x[[7, 6, 5, 4, 3, 2, 1, 0]]), y[[7, 6, 5, 4, 3, 2, 1, 0]])
    x2 = dev(synth.activations(rng, 8, k))
    both = lin(x + x2).float()
    parts = y.float() + lin(x2).float()
    assert float((both - parts).abs().max() / parts.abs().max()) < 2 * TOL
    lin.ctx.poll()


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


@pytest.mark.parametrize("type_id", STREAMED)
@pytest.mark.parametrize("plan", ["1,2,1", "1,3,2", "2,1,2", "2,2,4", "3,1,2", "4,2,2", "5,1,4", "8,1,4",
                                  "2,11,12", "1,21,16", "2,4,6,2", "3,7,8", "2,6,5"])
def test_every_launch_plan_gives_the_same_product(plan, type_id, monkeypatch):
    """The warp-level kernel under forced launch plans (K split = cluster size, units per warp,
    panels in parallel, optionally the ring depth), on a shape with a ragged last panel and an
    uneven K split: plans with and without clusters, with several warps per panel and with a warp
    owning whole panels."""
    monkeypatch.setenv("ISHI_FRAG_PLAN", plan)
    rng = np.random.default_rng(21)
    n, k = 1000, 5120 + 256
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks), type_id, (n, k)))
    want_plan = [int(v) for v in plan.split(",")]
    if lin.plan[0] == 0:
        pytest.skip("this plan does not fit shared memory for this format (the tcgen05 kernel took the weight)")
    assert lin.plan[0] == want_plan[0] and lin.plan[2] == want_plan[2], "the forced plan was not taken"
    for m in (1, 8, 11):
        x = synth.activations(rng, m, k)
        got = lin(dev(x)).cpu().numpy()
        want32, _ = oracle.ggml_matmul(int(type_id), blocks, x, n)
        err = float(np.abs(got.astype(np.float64) - want32.astype(np.float64)).max() / np.abs(want32).max())
        assert err < 2e-3, (plan, m, err)
    lin.ctx.poll()


@pytest.mark.parametrize("type_id", OTHERS)
@pytest.mark.parametrize("m", [1, 8, 16])
def test_projection_of_the_other_block_formats(type_id, m):
    """The eight formats without a streaming kernel go through one warp per output row."""
    rng = np.random.default_rng(int(type_id) * 31 + m)
    n, k = 1000, 5120
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    x = synth.activations(rng, m, k)
    raw = dev(blocks)
    lin = PackedLinear(ggml=GGUFBlocks(raw, type_id, (n, k)))
    raw.zero_()  # the projection keeps its own copy of the blocks
    y = lin(dev(x))
    torch.cuda.synchronize()
    want32, _ = oracle.ggml_matmul(int(type_id), blocks, x, n)
    assert rel_err(y.cpu().numpy(), want32) < TOL
    yt = lin(dev(x), transposed=True)
    assert torch.equal(yt.t().contiguous(), y)


def test_single_row_on_cuda_cores_at_a_projection_shape():
    """ISHI_ROUTE_GEMV: the CUDA-core variant of the warp-level kernel on the 27B gate shape."""
    rng = np.random.default_rng(77)
    n, k = 17408, 5120
    blocks = synth.q4k_blocks(rng, n, k)
    x = synth.activations(rng, 1, k)
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks), GGMLType.q4K, (n, k)))
    want32, _ = oracle.ggml_matmul(int(GGMLType.q4K), blocks, x, n)
    BonsaiRuntime.route = _lib.ROUTE_GEMV
    try:
        y = lin(dev(x))
    finally:
        BonsaiRuntime.route = _lib.ROUTE_AUTO
    assert rel_err(y.cpu().numpy(), want32) < TOL
    assert rel_err(lin(dev(x)).cpu().numpy(), want32) < TOL


@pytest.mark.parametrize("sizes", [(6144, 1024, 1024), (17, 40, 64), (1000, 24)])
def test_stacked_projections_are_one_launch_with_the_same_products(sizes):
    """ishi_projection_create_fused: q / k / v style weights stacked along the output rows."""
    rng = np.random.default_rng(sum(sizes))
    k = 5120 if sizes[0] > 100 else 1024
    parts = [synth.q4k_blocks(rng, n, k) for n in sizes]
    fused = FusedLinear([GGUFBlocks(dev(b), GGMLType.q4K, (n, k)) for b, n in zip(parts, sizes)])
    assert fused.outputDim == sum(sizes)
    for m in (1, 8, 13):
        x = synth.activations(rng, m, k)
        y = fused(dev(x))
        torch.cuda.synchronize()
        fused.ctx.poll()
        for piece, blocks, n in zip(fused.split(y), parts, sizes):
            want32, _ = oracle.ggml_matmul(int(GGMLType.q4K), blocks, x, n)
            assert rel_err(piece.cpu().numpy(), want32) < TOL


def test_stacked_q6k_matrices():
    """Q6_K has a fragment decoder too: matrices that share an input stack into one launch."""
    rng = np.random.default_rng(12)
    k, sizes = 1024, (48, 200)
    parts = [synth.q6k_blocks(rng, n, k) for n in sizes]
    fused = FusedLinear([GGUFBlocks(dev(b), GGMLType.q6K, (n, k)) for b, n in zip(parts, sizes)])
    x = synth.activations(rng, 8, k)
    y = fused(dev(x))
    torch.cuda.synchronize()
    fused.ctx.poll()
    for piece, blocks, n in zip(fused.split(y), parts, sizes):
        want32, _ = oracle.ggml_matmul(int(GGMLType.q6K), blocks, x, n)
        assert rel_err(piece.cpu().numpy(), want32) < TOL


def test_stacked_matrices_of_another_block_type():
    """The other GGML block types run on the warp-level kernel through the dense decoder and stack
    like the rest."""
    rng = np.random.default_rng(14)
    k, sizes = 1024, (40, 128)
    parts = [synth.ggml_blocks(rng, int(GGMLType.iq4Xs), n, k) for n in sizes]
    fused = FusedLinear([GGUFBlocks(dev(b), GGMLType.iq4Xs, (n, k)) for b, n in zip(parts, sizes)])
    x = synth.activations(rng, 8, k)
    y = fused(dev(x))
    torch.cuda.synchronize()
    fused.ctx.poll()
    assert all(v > 0 for v in fused.plan)
    for piece, blocks, n in zip(fused.split(y), parts, sizes):
        want32, _ = oracle.ggml_matmul(int(GGMLType.iq4Xs), blocks, x, n)
        assert rel_err(piece.cpu().numpy(), want32) < TOL


def test_stacked_affine_packs():
    rng = np.random.default_rng(9)
    k, sizes = 2048, (256, 100)
    packs = [synth.affine_pack(rng, n, k, 4, 64, np.float16) for n in sizes]
    fused = FusedLinear([(dev(w), dev(s), dev(b)) for w, s, b in packs], groupSize=64, bits=4)
    x = synth.activations(rng, 8, k)
    y = fused(dev(x))
    for piece, (w, s, b) in zip(fused.split(y), packs):
        want32, _ = oracle.affine_matmul(w, s, b, 4, 64, x)
        assert rel_err(piece.cpu().numpy(), want32) < TOL


def test_a_projection_under_another_ones_plan_gives_the_same_bits():
    """create measures its launch plan; the plan fixes the order of the partial sums. A second
    projection of the same weight agrees bit for bit once it is given the first one's plan."""
    rng = np.random.default_rng(21)
    n, k = 2048, 4096
    blocks = dev(synth.q4k_blocks(rng, n, k))
    a = PackedLinear(ggml=GGUFBlocks(blocks, GGMLType.q4K, (n, k)))
    b = PackedLinear(ggml=GGUFBlocks(blocks, GGMLType.q4K, (n, k)))
    assert all(v > 0 for v in a.plan)
    x = dev(synth.activations(rng, 8, k))
    b.set_plan(a.plan)
    assert b.plan == a.plan
    assert torch.equal(a(x), b(x))
    with pytest.raises(IshizukiError):
        b.set_plan((2, 25, 8, 3))  # more warps than a block holds: not a plan of this projection


@pytest.mark.parametrize("type_id", [GGMLType.q4K, GGMLType.q6K])
def test_rotated_input_ahead_of_a_gguf_projection(type_id):
    """A GGUF projection with a rotation block: the input goes through the stand-alone rotation
    kernel first (the GGUF decoders' staging does not rotate), the product is that of the rotated
    rows."""
    rng = np.random.default_rng(int(type_id))
    n, k = 96, 1024
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    lin = PackedLinear(None, None, None, None, 128, ggml=GGUFBlocks(dev(blocks), type_id, (n, k)))
    for m in (1, 8):
        x = synth.activations(rng, m, k)
        want32, _ = oracle.ggml_matmul(int(type_id), blocks, oracle.hadamard_rotate(x, 128), n)
        assert rel_err(lin(dev(x)).cpu().numpy(), want32) < TOL
    lin.ctx.poll()


@pytest.mark.parametrize("type_id", [GGMLType.q2K, GGMLType.iq2S, GGMLType.iq3Xxs, GGMLType.iq4Xs, GGMLType.iq1M])
def test_the_dense_decoder_path_of_the_other_block_types(type_id, monkeypatch):
    """ISHI_DENSE_DECODER=1 at create sends the eight other block types through the dense decoder
    (decode8 into fp16 fragments) instead of their own fragment decoders: the same products."""
    rng = np.random.default_rng(int(type_id) + 500)
    n, k = 200, 1024
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    own = PackedLinear(ggml=GGUFBlocks(dev(blocks), type_id, (n, k)))
    monkeypatch.setenv("ISHI_DENSE_DECODER", "1")
    dense = PackedLinear(ggml=GGUFBlocks(dev(blocks), type_id, (n, k)))
    monkeypatch.delenv("ISHI_DENSE_DECODER")
    for m in (1, 8):
        x = synth.activations(rng, m, k)
        want32, _ = oracle.ggml_matmul(int(type_id), blocks, x, n)
        assert rel_err(own(dev(x)).cpu().numpy(), want32) < TOL
        assert rel_err(dense(dev(x)).cpu().numpy(), want32) < TOL
    own.ctx.poll()


def _check_gated(gated, stacked, x, want_gate, want_up):
    """The gated launch against (a) the oracle's silu(gate) * up on the oracle's fp16 products and
    (b) the same formula on this library's own stacked products, which differ from the kernel's
    only where the device's exp rounds another way: a unit in the last place, rarely."""
    f = gated.outputDim
    h = gated(dev(x))
    torch.cuda.synchronize()
    gated.ctx.poll()
    assert h.shape == (x.shape[0], f)
    want = oracle.swiglu(want_gate, want_up).astype(np.float32)
    assert rel_err(h.cpu().numpy().astype(np.float32), want) < TOL
    gate_y, up_y = stacked.split(stacked(dev(x)))
    own = oracle.swiglu(gate_y.cpu().numpy(), up_y.cpu().numpy())
    got = h.cpu().numpy()
    differing = got.view(np.uint16) != own.view(np.uint16)
    assert differing.mean() < 1e-3
    assert np.all(np.abs(got.astype(np.float32) - own.astype(np.float32))[differing] <= np.abs(own.astype(np.float32))[differing] * 2.0 ** -9 + 1e-7)


@pytest.mark.parametrize("f,k", [(17408, 5120), (1000, 1024), (8, 512)])
def test_gated_pair_writes_silu_gate_times_up(f, k):
    """ishi_projection_create_gated: gate and up interleaved by eights in the tiled copy, the
    kernel's epilogue writes silu(x . gate^T) * (x . up^T), [rows, f]."""
    rng = np.random.default_rng(f + k)
    gate, up = synth.q4k_blocks(rng, f, k), synth.q4k_blocks(rng, f, k)
    parts = [GGUFBlocks(dev(gate), GGMLType.q4K, (f, k)), GGUFBlocks(dev(up), GGMLType.q4K, (f, k))]
    gated = FusedLinear(parts, gated=True)
    stacked = FusedLinear(parts)
    stacked.set_plan(gated.plan)  # the same order of partial sums
    assert gated.outputDim == f and stacked.outputDim == 2 * f
    for m in (1, 8, 11):
        x = synth.activations(rng, m, k)
        _, g16 = oracle.ggml_matmul(int(GGMLType.q4K), gate, x, f)
        _, u16 = oracle.ggml_matmul(int(GGMLType.q4K), up, x, f)
        _check_gated(gated, stacked, x, g16, u16)


def test_gated_pair_other_formats_and_a_single_row_on_cuda_cores():
    rng = np.random.default_rng(77)
    f, k = 264, 2048
    x = synth.activations(rng, 8, k)
    packs = [synth.affine_pack(rng, f, k, 4, 64, np.float16) for _ in range(2)]
    parts = [(dev(w), dev(s), dev(b)) for w, s, b in packs]
    gated, stacked = FusedLinear(parts, groupSize=64, bits=4, gated=True), FusedLinear(parts, groupSize=64, bits=4)
    stacked.set_plan(gated.plan)
    wants = [oracle.affine_matmul(w, s, b, 4, 64, x)[1] for w, s, b in packs]
    _check_gated(gated, stacked, x, *wants)
    blocks = [synth.q6k_blocks(rng, f, k) for _ in range(2)]
    parts = [GGUFBlocks(dev(b), GGMLType.q6K, (f, k)) for b in blocks]
    gated, stacked = FusedLinear(parts, gated=True), FusedLinear(parts)
    stacked.set_plan(gated.plan)
    wants = [oracle.ggml_matmul(int(GGMLType.q6K), b, x, f)[1] for b in blocks]
    _check_gated(gated, stacked, x, *wants)
    # one row through the CUDA-core route
    blocks = [synth.q4k_blocks(rng, f, k) for _ in range(2)]
    parts = [GGUFBlocks(dev(b), GGMLType.q4K, (f, k)) for b in blocks]
    gated = FusedLinear(parts, gated=True)
    x1 = synth.activations(rng, 1, k)
    wants = [oracle.ggml_matmul(int(GGMLType.q4K), b, x1, f)[1] for b in blocks]
    want = oracle.swiglu(*wants).astype(np.float32)
    BonsaiRuntime.route = _lib.ROUTE_GEMV
    try:
        h = gated(dev(x1))
    finally:
        BonsaiRuntime.route = _lib.ROUTE_AUTO
    assert rel_err(h.cpu().numpy().astype(np.float32), want) < TOL
    gated.ctx.poll()


def test_gated_pair_guards():
    rng = np.random.default_rng(3)
    a = GGUFBlocks(dev(synth.q4k_blocks(rng, 32, 512)), GGMLType.q4K, (32, 512))
    b = GGUFBlocks(dev(synth.q4k_blocks(rng, 40, 512)), GGMLType.q4K, (40, 512))
    c = GGUFBlocks(dev(synth.q4k_blocks(rng, 20, 512)), GGMLType.q4K, (20, 512))
    with pytest.raises(IshizukiError) as err:
        FusedLinear([a, b], gated=True)  # different heights
    assert err.value.status == _lib.E_SHAPE
    with pytest.raises(IshizukiError) as err:
        FusedLinear([c, c], gated=True)  # height not a multiple of 8
    assert err.value.status == _lib.E_SHAPE
    with pytest.raises(ValueError):
        FusedLinear([a, a, a], gated=True)


def test_stacking_guards():
    rng = np.random.default_rng(2)
    a = GGUFBlocks(dev(synth.q4k_blocks(rng, 32, 512)), GGMLType.q4K, (32, 512))
    b = GGUFBlocks(dev(synth.q4k_blocks(rng, 32, 1024)), GGMLType.q4K, (32, 1024))
    with pytest.raises(ValueError):
        FusedLinear([a, b])  # different input widths
    packs = [synth.affine_pack(rng, 64, 512, 8, 64, np.float16) for _ in range(2)]
    with pytest.raises(IshizukiError) as err:
        FusedLinear([(dev(w), dev(sc), dev(b)) for w, sc, b in packs], groupSize=64, bits=8)  # 8-bit packs run on the tcgen05 kernel: cannot be stacked
    assert err.value.status == _lib.E_UNSUPPORTED


@pytest.mark.parametrize("type_id", [GGMLType.q4K, GGMLType.q6K, GGMLType.iq4Xs, GGMLType.iq2Xxs])
def test_gather_decodes_the_requested_rows(type_id):
    """GGMLKernels.gather: the quantized embedding lookup, bit-exact against the decoder."""
    rng = np.random.default_rng(int(type_id))
    rows, k = 300, 1024
    blocks = synth.ggml_blocks(rng, int(type_id), rows, k)
    table = oracle.dequantize(int(type_id), blocks).reshape(rows, k)
    ids = np.array([0, 299, 17, 17, 123, 4], dtype=np.int64)
    got = GGMLKernels.gather(torch.from_numpy(ids).cuda(), dev(blocks), type_id, k, dtype=torch.float32)
    assert same_bits(got.cpu().numpy(), table[ids])
    half = GGMLKernels.gather(torch.from_numpy(ids).cuda(), dev(blocks), type_id, k, dtype=torch.float16)
    assert np.array_equal(half.cpu().numpy().view(np.uint16), table[ids].astype(np.float16).view(np.uint16))
    outside = GGMLKernels.gather(torch.tensor([5, rows, -1]).cuda(), dev(blocks), type_id, k, dtype=torch.float32)
    assert same_bits(outside[0].cpu().numpy(), table[5]) and not outside[1:].any()
    assert GGMLKernels.gather(torch.tensor([1]).cuda(), dev(blocks), type_id, 100) is None


@pytest.mark.parametrize("type_id", [GGMLType.q4K, GGMLType.q6K, GGMLType.iq4Xs])
@pytest.mark.parametrize("m", [1, 8, 16])
def test_head_argmax_matches_argmax_of_the_logits(type_id, m):
    """The verify step's head: index of the largest fp16 logit per row, lowest index among equals."""
    rng = np.random.default_rng(m + int(type_id))
    n, k = 20000, 1024  # a vocabulary-like output dimension with a ragged last panel
    blocks = synth.ggml_blocks(rng, int(type_id), n, k)
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks), type_id, (n, k)))
    x = synth.activations(rng, m, k)
    got = lin.argmax(dev(x)).cpu().numpy()
    logits = lin(dev(x)).float().cpu().numpy()
    assert np.array_equal(got, logits.argmax(axis=1))  # numpy also returns the first of equals
    want32, _ = oracle.ggml_matmul(int(type_id), blocks, x, n)
    top = want32.max(axis=1)
    assert np.all(want32[np.arange(m), got] >= top - 2e-3 * np.abs(want32).max())


def test_head_argmax_on_rows_that_are_not_16_byte_aligned():
    """n not a multiple of 8: every logits row but the first starts off the 16-byte grid and is read
    value by value; repeated calls reuse the kernel's counters."""
    rng = np.random.default_rng(31)
    n, k = 9004, 256
    blocks = synth.q4k_blocks(rng, n, k)
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks), GGMLType.q4K, (n, k)))
    for m in (3, 16, 1):
        x = synth.activations(rng, m, k)
        logits = lin(dev(x)).float().cpu().numpy()
        for _ in range(2):
            assert np.array_equal(lin.argmax(dev(x)).cpu().numpy(), logits.argmax(axis=1))


def test_argmax_ties_take_the_lowest_index():
    n, k = 4096, 256
    blocks = np.zeros((n, 144), dtype=np.uint8)  # every weight decodes to zero: all logits equal
    lin = PackedLinear(ggml=GGUFBlocks(dev(blocks.reshape(-1)), GGMLType.q4K, (n, k)))
    x = synth.activations(np.random.default_rng(0), 4, k)
    assert lin.argmax(dev(x)).cpu().tolist() == [0, 0, 0, 0]


def test_misaligned_rotation_signs_are_refused_before_anything_runs():
    rng = np.random.default_rng(4)
    n, k = 64, 512
    w, sb, bb = synth.ternary_pack(rng, n, k, 128)
    signs = torch.ones(k + 1, dtype=torch.float32, device="cuda")
    with pytest.raises(IshizukiError) as err:
        PackedLinear(dev(w), dev(sb).view(torch.bfloat16), dev(bb).view(torch.bfloat16), signs[1:], 128, groupSize=128, bits=2)
    assert err.value.status == _lib.E_INVALID


def test_a_projection_and_an_embedding_read_straight_off_a_gguf_file(tmp_path):
    """Tests/IshizukiKitTests/GGUFWeightsTests.swift:119-177: an IQ2_S projection and an IQ1_M
    embedding table out of a GGUF file, against decode-then-multiply."""
    gguf = pytest.importorskip("gguf")
    from ishizuki_b200.gguf_file import GGUFFile

    rng = np.random.default_rng(33)
    hidden, vocab = 256, 16
    table = synth.ggml_blocks(rng, int(GGMLType.iq1M), vocab, hidden)
    up = synth.ggml_blocks(rng, int(GGMLType.iq2S), hidden, hidden)
    path = tmp_path / "modules.gguf"
    w = gguf.GGUFWriter(str(path), "qwen35")
    w.add_tensor("token_embd.weight", table.reshape(vocab, -1), raw_dtype=gguf.GGMLQuantizationType(29))
    w.add_tensor("blk.0.ffn_up.weight", up.reshape(hidden, -1), raw_dtype=gguf.GGMLQuantizationType(22))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    f = GGUFFile(path)
    blocks = f.blocks("blk.0.ffn_up.weight")
    assert (blocks.type, blocks.shape) == (GGMLType.iq2S, (hidden, hidden))
    assert np.array_equal(blocks.bytes.cpu().numpy(), up)
    lin = PackedLinear(ggml=blocks)
    x = synth.activations(rng, 1, hidden)
    want32, _ = oracle.ggml_matmul(int(GGMLType.iq2S), up, x, hidden)
    assert rel_err(lin(dev(x)).cpu().numpy(), want32) < TOL

    emb = f.blocks("token_embd.weight")
    rows = GGMLKernels.gather(torch.tensor([3, 11]).cuda(), emb.bytes, emb.type, hidden, dtype=torch.float32)
    full = oracle.dequantize(int(GGMLType.iq1M), table).reshape(vocab, hidden)
    assert same_bits(rows.cpu().numpy(), full[[3, 11]])
