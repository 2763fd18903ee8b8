"""Bit-exactness of the CUDA rowwise quantizers / dequantizers and of the table-row packing
against the CPU oracle (which is itself pinned to the FBGEMM CPU kernels and to
torch.ops.quantized.embedding_bag_*_prepack in test_oracle_pins.py)."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def rows(rng, kind, n, d):
    if kind == "normal":
        return rng.normal(0.0, 0.1, (n, d)).astype(np.float32)
    if kind == "uniform":
        return rng.uniform(-0.1, 0.1, (n, d)).astype(np.float32)
    if kind == "const":
        return np.full((n, d), 0.37, dtype=np.float32)
    if kind == "tiny":
        return (rng.normal(0.0, 1.0, (n, d)) * 1e-9).astype(np.float32)
    if kind == "huge":
        return (rng.normal(0.0, 1.0, (n, d)) * 1e30).astype(np.float32)
    if kind == "mixed":
        x = rng.normal(0.0, 1.0, (n, d)).astype(np.float32)
        x[::3] *= 1e-4
        x[1::3] *= 300.0
        x[:, 0] = 0.0
        return x
    raise ValueError(kind)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


SHAPES = [(2000, 128), (500, 64), (300, 7), (50, 1), (17, 16), (33, 260), (5, 4096), (1, 3), (1000, 36)]
KINDS = ["normal", "uniform", "const", "tiny", "huge", "mixed"]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("kind", KINDS)
def test_quantize_8bit_bit_exact(shape, kind):
    import fbgemm_ascend_b200  # noqa: F401
    rng = np.random.default_rng(hash(shape) % 1000 + KINDS.index(kind))
    x = rows(rng, kind, *shape)
    want = O.quantize_8bit_rowwise(x)
    got = torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(dev(x)).cpu().numpy()
    assert got.shape == want.shape and got.dtype == np.uint8
    assert np.array_equal(got, want), f"{int((got != want).sum())} bytes differ"
    back = torch.ops.fbgemm.Fused8BitRowwiseQuantizedToFloat(dev(want)).cpu().numpy()
    assert np.array_equal(back.view(np.uint32), O.dequantize_8bit_rowwise(want).view(np.uint32))


def test_quantize_8bit_unaligned_input_view_and_3d():
    import fbgemm_ascend_b200  # noqa: F401
    rng = np.random.default_rng(4)
    x = rng.normal(0, 1, (6, 10, 24)).astype(np.float32)
    got = torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(dev(x)).cpu().numpy()
    assert got.shape == (6, 10, 32)
    assert np.array_equal(got.reshape(60, 32), O.quantize_8bit_rowwise(x.reshape(60, 24)))
    # a storage offset that breaks 16-byte alignment of the input
    base = dev(rng.normal(0, 1, (1 + 40 * 20,)).astype(np.float32))
    view = base[1:].view(40, 20)
    got = torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(view).cpu().numpy()
    assert np.array_equal(got, O.quantize_8bit_rowwise(view.cpu().numpy()))


def test_half_variants():
    import fbgemm_ascend_b200  # noqa: F401
    rng = np.random.default_rng(9)
    x = rng.normal(0, 0.1, (100, 48)).astype(np.float16)
    got = torch.ops.fbgemm.HalfToFused8BitRowwiseQuantized(dev(x)).cpu().numpy()
    assert np.array_equal(got, O.quantize_8bit_rowwise(x.astype(np.float32)))
    back = torch.ops.fbgemm.Fused8BitRowwiseQuantizedToHalf(dev(got)).cpu().numpy()
    assert np.array_equal(back, O.dequantize_8bit_rowwise(got).astype(np.float16))


@pytest.mark.parametrize("bit_rate", [4, 2])
@pytest.mark.parametrize("shape", [(2000, 128), (500, 64), (300, 8), (10, 16), (100, 256), (7, 4096), (64, 24), (77, 32), (1001, 96),
                                   (33, 160), (5, 128), (1, 256)])
@pytest.mark.parametrize("kind", KINDS)
def test_quantize_nbit_bit_exact(bit_rate, shape, kind):
    import fbgemm_ascend_b200  # noqa: F401
    if kind == "huge":
        pytest.skip("1e30 overflows the fp16 bias of the n-bit format; the result is implementation-defined")
    rng = np.random.default_rng(bit_rate * 100 + KINDS.index(kind))
    x = rows(rng, kind, *shape)
    want = O.quantize_nbit_rowwise_sbhalf(x, bit_rate)
    got = torch.ops.fbgemm.FloatToFusedNBitRowwiseQuantizedSBHalf(dev(x), bit_rate).cpu().numpy()
    assert np.array_equal(got, want), f"{int((got != want).sum())} bytes differ"
    back = torch.ops.fbgemm.FusedNBitRowwiseQuantizedSBHalfToFloat(dev(want), bit_rate).cpu().numpy()
    assert np.array_equal(back.view(np.uint32), O.dequantize_nbit_rowwise_sbhalf(want, bit_rate).view(np.uint32))


@pytest.mark.parametrize("ty", [O.INT8, O.INT4, O.INT2, O.FP16])
@pytest.mark.parametrize("shape", [(1000, 128), (333, 64), (50, 16), (20, 1024), (101, 96), (9, 256), (45, 32)])
@pytest.mark.parametrize("row_alignment", [16, 1])
def test_table_rows_bit_exact(ty, shape, row_alignment):
    """Direct fp32 -> table rows equals oracle quantize + pack; and so does quantize then pack on the GPU."""
    import fbgemm_ascend_b200  # noqa: F401
    rng = np.random.default_rng(ty * 7 + shape[1])
    x = rows(rng, "normal", *shape)
    want = O.pack_table(x, ty, row_alignment)
    rb = want.shape[1]
    got = torch.ops.tbe_b200.quantize_to_table_rows(dev(x), ty, rb).cpu().numpy()
    assert np.array_equal(got, want)
    if ty == O.INT8:
        fused = torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(dev(x))
        assert np.array_equal(torch.ops.tbe_b200.pack_table_rows(fused, 8, shape[1], rb).cpu().numpy(), want)
    elif ty in (O.INT4, O.INT2):
        bits = 4 if ty == O.INT4 else 2
        fused = torch.ops.fbgemm.FloatToFusedNBitRowwiseQuantizedSBHalf(dev(x), bits)
        assert np.array_equal(torch.ops.tbe_b200.pack_table_rows(fused, bits, shape[1], rb).cpu().numpy(), want)


def test_quantize_dequantize_round_trip_large():
    """Size-independent property at a benchmark-sized table chunk (1M x 128): the round trip error is
    at most half a quantization step per element, and re-quantizing the dequantized rows gives the
    same codes."""
    import fbgemm_ascend_b200  # noqa: F401
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(1_000_000, 128, device="cuda", generator=g) * 0.05
    q = torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(x)
    y = torch.ops.fbgemm.Fused8BitRowwiseQuantizedToFloat(q)
    scale = q[:, 128:132].contiguous().view(torch.float32)
    assert bool(((x - y).abs() <= 0.5001 * scale + 1e-12).all())
    q2 = torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(y)
    assert float((q2[:, :128] != q[:, :128]).float().mean()) < 1e-3
    # spot-check 4096 rows bit-exactly against the oracle
    sel = torch.randint(0, 1_000_000, (4096,), device="cuda", generator=g)
    assert np.array_equal(q[sel].cpu().numpy(), O.quantize_8bit_rowwise(x[sel].cpu().numpy()))
