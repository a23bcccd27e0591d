"""Affine group-quantized packs on the GPU against the CPU oracle.

Mirrors Tests/IshizukiKitTests/VerifyMatmulTests.swift: (bits, group) pairs, N = 384, K = 1024,
rows 5...8 (plus 1 and 16 here), scale dtypes fp16 / bf16 / fp32, tolerance max|d| / max|want| <
2e-3 for fp16 activations; then the model's own shapes.
"""
import numpy as np
import pytest
import torch

from ishizuki_b200 import synth
from ishizuki_b200.interface import PackedLinear, VerifyMatmul, hadamardRotate
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(got, want) -> float:
    return float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max() / np.abs(want).max())


def make_pack(rng, n, k, bits, gs, dtype):
    w, s, b = synth.affine_pack(rng, n, k, bits, gs, np.float32)
    if dtype == "f32":
        return w, s, b, dev(s), dev(b), False
    if dtype == "f16":
        s, b = s.astype(np.float16), b.astype(np.float16)
        return w, s, b, dev(s), dev(b), False
    sb, bb = synth.to_bf16_bits(s), synth.to_bf16_bits(b)
    return w, sb, bb, dev(sb).view(torch.bfloat16), dev(bb).view(torch.bfloat16), True


@pytest.mark.parametrize("bits,gs", [(2, 128), (4, 128), (8, 128), (4, 64), (2, 64), (4, 32), (8, 32), (2, 32)])
@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_matches_expanded_matmul(bits, gs, dtype):
    rng = np.random.default_rng(bits * 1000 + gs)
    n, k = 384, 1024
    w, s, b, sd, bd, bf16 = make_pack(rng, n, k, bits, gs, dtype)
    for rows in (1, 5, 8, 13, 16):
        x = (rng.standard_normal((rows, k)) * 2).astype(np.float16)
        got = VerifyMatmul.applyAny(dev(x), dev(w), sd, bd, gs, bits)
        assert got is not None
        want32, _ = oracle.affine_matmul(w, s, b, bits, gs, x, bf16=bf16)
        assert rel_err(got.cpu().numpy(), want32) < TOL, (bits, gs, dtype, rows)


def test_decode_matches_formula():
    rng = np.random.default_rng(9)
    for bits, gs in [(2, 128), (4, 64), (8, 128), (3, 128), (5, 32), (6, 64)]:
        n, k = 64, 1024
        codes = rng.integers(0, 1 << bits, size=(n, k), dtype=np.uint32)
        w = synth.pack_codes(codes, bits)
        s = (np.abs(rng.standard_normal((n, k // gs))) * 0.01).astype(np.float16)
        b = (rng.standard_normal((n, k // gs)) * 0.01).astype(np.float16)
        from ishizuki_b200 import _lib
        from ishizuki_b200.interface import Context, _ptr, _stream
        ctx = Context.get(0)
        out = torch.empty((n, k), dtype=torch.float32, device="cuda")
        wd, sd, bd = dev(w), dev(s), dev(b)  # keep the device copies alive across the call
        rc = ctx.lib.ishi_affine_dequantize(ctx.handle, _ptr(wd), _ptr(sd), _ptr(bd), _lib.DT_F16, gs, bits,
                                            n, k, _ptr(out), _stream())
        assert rc == 0
        torch.cuda.synchronize()
        want = oracle.affine_dequantize(w, s, b, bits, gs)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_declines_what_the_reference_declines():
    x = torch.zeros((8, 1024), dtype=torch.float16, device="cuda")
    w = torch.zeros((384, 1024 * 3 // 32), dtype=torch.int32, device="cuda")
    s = torch.zeros((384, 8), dtype=torch.float16, device="cuda")
    assert VerifyMatmul.applyAny(x, w, s, s, 128, 3) is None  # 3 bits: no kernel here
    w4 = torch.zeros((384, 128), dtype=torch.int32, device="cuda")
    assert VerifyMatmul.applyAny(torch.zeros((17, 1024), dtype=torch.float16, device="cuda"), w4, s, s, 128, 4) is None
    assert VerifyMatmul.applyAny(x[:, :1000].contiguous(), w4, s, s, 128, 4) is None  # width mismatch


@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 5120), (6144, 5120), (5120, 6144), (17408, 5120), (5120, 17408)])
def test_config_shapes_four_bit_group_64(n, k):
    """The single-projection configuration: 4-bit, group 64, fp16 scales, rows 1 and 8."""
    rng = np.random.default_rng(0)
    w, s, b = synth.affine_pack(rng, n, k, 4, 64, np.float16)
    lin = PackedLinear(dev(w), dev(s), dev(b), None, 0, groupSize=64, bits=4)
    for rows in (1, 8):
        x = synth.activations(rng, rows, k)
        y = lin(dev(x))
        want32, _ = oracle.affine_matmul(w, s, b, 4, 64, x)
        assert rel_err(y.cpu().numpy(), want32) < TOL
    lin.ctx.poll()


@pytest.mark.parametrize("n,k", [(6144, 5120), (1024, 5120), (5120, 6144), (17408, 5120), (5120, 17408)])
def test_ternary_rotated_projection(n, k):
    """Bonsai-style ternary pack: 2 bits, group 128, bf16 scales, bias = -scale, input rotated by
    an orthonormal block Hadamard of 128 (no sign vector)."""
    rng = np.random.default_rng(4)
    w, sbits, bbits = synth.ternary_pack(rng, n, k, 128)
    lin = PackedLinear(dev(w), dev(sbits).view(torch.bfloat16), dev(bbits).view(torch.bfloat16), None, 128,
                       groupSize=128, bits=2)
    for rows in (1, 8):
        x = synth.activations(rng, rows, k)
        y = lin(dev(x))
        xr = oracle.hadamard_rotate(x, 128)
        want32, _ = oracle.affine_matmul(w, sbits, bbits, 2, 128, xr, bf16=True)
        assert rel_err(y.cpu().numpy(), want32) < TOL
        # rotate + applyRotated is the same product in two calls. The product kernel rotates this
        # case on the tensor cores, the rotation kernel by butterflies: the two agree to fp32
        # rounding, the outputs to a unit in the last place of fp16
        xr_dev = lin.rotate(dev(x))
        assert np.array_equal(xr_dev.cpu().numpy().view(np.uint16), xr.view(np.uint16))
        two = lin.applyRotated(xr_dev).cpu().numpy().astype(np.float32)
        assert rel_err(two, y.cpu().numpy().astype(np.float32)) < 5e-4
        if rows == 1:
            # the same staging feeds the single-row CUDA-core route
            from ishizuki_b200 import _lib
            from ishizuki_b200.interface import BonsaiRuntime

            BonsaiRuntime.route = _lib.ROUTE_GEMV
            try:
                assert rel_err(lin(dev(x)).cpu().numpy(), want32) < TOL
            finally:
                BonsaiRuntime.route = _lib.ROUTE_AUTO
    lin.ctx.poll()


def test_rotation_matches_golden(golden_dir):
    g = np.load(golden_dir / "hadamard_case1.npz")
    got = hadamardRotate(dev(g["x"]), int(g["block"]), dev(g["signs"]))
    assert np.array_equal(got.cpu().numpy().view(np.uint16), g["rotated"].view(np.uint16))
    for block in (128, 512, 4096):
        x = synth.activations(np.random.default_rng(block), 5, 8192)
        want = oracle.hadamard_rotate(x, block)
        got = hadamardRotate(dev(x), block, None)
        assert np.array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("bits,gs", [(4, 32), (4, 64), (4, 128), (2, 64), (2, 128)])
def test_single_row_on_cuda_cores(bits, gs):
    """One activation row through the CUDA-core route (fp32 FMA, warp-shuffle reduction) gives the
    product of the tensor-core route within the same tolerance."""
    from ishizuki_b200 import _lib

    rng = np.random.default_rng(bits * 100 + gs)
    n, k = 400, 1536  # a ragged last panel
    w, s, b, sd, bd, bf16 = make_pack(rng, n, k, bits, gs, "bf16")
    x = synth.activations(rng, 1, k)
    got = VerifyMatmul.applyAny(dev(x), dev(w), sd, bd, gs, bits, route=_lib.ROUTE_GEMV)
    assert got is not None
    want32, _ = oracle.affine_matmul(w, s, b, bits, gs, x, bf16=bf16)
    assert rel_err(got.cpu().numpy(), want32) < TOL


@pytest.mark.parametrize("block", [32, 64, 128, 256, 512])
@pytest.mark.parametrize("signed", [False, True])
def test_rotation_inside_the_product_kernel(block, signed):
    """apply(x) on a rotated projection equals applyRotated(rotate(x)) bit for bit, whether the
    rotation runs inside the product kernel (blocks up to 256) or as its own kernel (512), with and
    without a sign vector; and it matches the oracle's product on the oracle's rotation."""
    rng = np.random.default_rng(block + int(signed))
    n, k = 272, 2048
    w, s, b = synth.affine_pack(rng, n, k, 4, 64, np.float16)
    signs = np.where(rng.random(k) < 0.5, -1.0, 1.0).astype(np.float32) if signed else None
    lin = PackedLinear(dev(w), dev(s), dev(b), None if signs is None else dev(signs), block, groupSize=64, bits=4)
    for rows in (1, 3, 8, 11):
        x = synth.activations(rng, rows, k)
        y = lin(dev(x))
        xr_dev = lin.rotate(dev(x))
        assert torch.equal(lin.applyRotated(xr_dev), y)
        xr = oracle.hadamard_rotate(x, block, signs) if signs is not None else oracle.hadamard_rotate(x, block)
        assert np.array_equal(xr_dev.cpu().numpy().view(np.uint16), xr.view(np.uint16))
        want32, _ = oracle.affine_matmul(w, s, b, 4, 64, xr)
        assert rel_err(y.cpu().numpy(), want32) < TOL
    lin.ctx.poll()
