"""Pins the CPU oracle (oracle/tbe_oracle.c) before anything is compared with it.

Three independent anchors:
  1. the committed golden vectors (tests/golden/tbe_golden.npz), produced by the FBGEMM CPU kernels
     and the torch.ops.quantized embedding-bag operators;
  2. the same FBGEMM kernels and torch operators called live on seeded random inputs;
  3. the known-answer vectors of the reference's permute tests.
Integer / byte results must be identical; pooled fp32 / fp16 results are identical too (the C
restatement reproduces FBGEMM's operation order), except bf16 ties, which FBGEMM rounds away from zero
and the reference's device kernel (and the oracle) round to even.
"""
import os

import numpy as np
import pytest
import torch

import oracle as O
from helpers import make_case, oracle_lookup

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "tbe_golden.npz"))


def bits(a):
    return a.view(np.uint32 if a.dtype == np.float32 else np.uint16)


# ---- 1. golden vectors -------------------------------------------------------------

def test_golden_quantizers():
    assert np.array_equal(O.quantize_8bit_rowwise(GOLD["q8_in"]), GOLD["q8_out"])
    assert np.array_equal(bits(O.dequantize_8bit_rowwise(GOLD["q8_out"])), bits(GOLD["q8_back"]))
    assert np.array_equal(O.quantize_nbit_rowwise_sbhalf(GOLD["q4_in"], 4), GOLD["q4_out"])
    assert np.array_equal(O.quantize_nbit_rowwise_sbhalf(GOLD["q4_in"], 4), GOLD["q4_out_fbgemm"])
    assert np.array_equal(O.quantize_nbit_rowwise_sbhalf(GOLD["q4_in"], 2), GOLD["q2_out_fbgemm"])


@pytest.mark.parametrize("pname,pm", [("sum", O.SUM), ("mean", O.MEAN)])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("oname,od", [("f32", O.FP32), ("f16", O.FP16)])
def test_golden_lookup(pname, pm, weighted, oname, od):
    g = GOLD
    out = O.tbe_lookup(g["lk_dev"], g["lk_wo"], g["lk_wt"], g["lk_do"], g["lk_idx"], g["lk_offs"], pm,
                       g["lk_w"] if weighted else None, od)
    want = g[f"lk_{pname}_{'w' if weighted else 'u'}_{oname}"]
    assert np.array_equal(bits(out), bits(want))


def test_golden_fp8_and_fused_row_lookup():
    g = GOLD
    a = O.tbe_lookup(g["f8_dev"], g["f8_wo"], g["f8_wt"], g["f8_do"], g["f8_idx"], g["f8_offs"], O.SUM, None, O.FP32, 16, 4, 7)
    assert np.array_equal(bits(a), bits(g["f8_sum_e4b7"]))
    b = O.tbe_lookup(g["f8_dev"], g["f8_wo"], g["f8_wt"], g["f8_do"], g["f8_idx"], g["f8_offs"], O.MEAN, None, O.FP32, 16, 5, 15)
    assert np.array_equal(bits(b), bits(g["f8_mean_e5b15"]))
    # fused 8-bit rows with fp16-representable scale/bias == table rows; compare with torch-core's lookup
    fused = g["eb_fused"]
    rows = np.zeros((fused.shape[0], 48), dtype=np.uint8)
    O._lib("port").orc_pack_int8_rows(O._ptr(np.ascontiguousarray(fused)), fused.shape[0], 32, 48, O._ptr(rows))
    dev, wo, wt, do = O.concat_tables([rows], [O.INT8], [32])
    out = O.tbe_lookup(dev, wo, wt, do, g["eb_idx"], g["eb_offs"], O.SUM, None, O.FP32)
    assert np.array_equal(bits(out), bits(g["eb_out"]))


# ---- 2. live cross-checks -----------------------------------------------------------

@pytest.mark.parametrize("n,d,kind", [(2000, 128, "n"), (500, 64, "u"), (300, 7, "n"), (50, 1, "n"), (10, 16, "c"), (64, 36, "t")])
def test_quantize_8bit_against_fbgemm_and_torch(n, d, kind):
    rng = np.random.default_rng(n + d)
    x = rng.normal(0, 0.1, (n, d)).astype(np.float32) if kind != "u" else rng.uniform(-.1, .1, (n, d)).astype(np.float32)
    if kind == "c":
        x[:] = 0.37
    if kind == "t":
        x *= 1e-7
    a = O.quantize_8bit_rowwise(x, "port")
    assert np.array_equal(a, O.quantize_8bit_rowwise(x, "ref"))
    assert np.array_equal(a, torch.ops.quantized.embedding_bag_byte_prepack(torch.from_numpy(x)).numpy())
    da = O.dequantize_8bit_rowwise(a, "port")
    assert np.array_equal(bits(da), bits(O.dequantize_8bit_rowwise(a, "ref")))
    assert np.array_equal(bits(da), bits(torch.ops.quantized.embedding_bag_byte_unpack(torch.from_numpy(a)).numpy()))


@pytest.mark.parametrize("bit_rate", [4, 2])
@pytest.mark.parametrize("n,d,kind", [(2000, 128, "n"), (500, 64, "u"), (300, 8, "n"), (10, 16, "c"), (100, 256, "t")])
def test_quantize_nbit_against_fbgemm_and_torch(bit_rate, n, d, kind):
    rng = np.random.default_rng(n + d + bit_rate)
    x = rng.normal(0, 0.1, (n, d)).astype(np.float32) if kind != "u" else rng.uniform(-.1, .1, (n, d)).astype(np.float32)
    if kind == "c":
        x[:] = 0.37
    if kind == "t":
        x *= 1e-9
    a = O.quantize_nbit_rowwise_sbhalf(x, bit_rate, "port")
    assert np.array_equal(a, O.quantize_nbit_rowwise_sbhalf(x, bit_rate, "ref"))
    if bit_rate == 4:
        assert np.array_equal(a, torch.ops.quantized.embedding_bag_4bit_prepack(torch.from_numpy(x)).numpy())
    assert np.array_equal(bits(O.dequantize_nbit_rowwise_sbhalf(a, bit_rate, "port")),
                          bits(O.dequantize_nbit_rowwise_sbhalf(a, bit_rate, "ref")))


@pytest.mark.parametrize("tys,dims", [([O.INT8], [128]), ([O.INT4, O.INT8, O.FP16], [64, 128, 32]),
                                      ([O.INT2, O.FP32], [32, 20]), ([O.INT4, O.INT4, O.INT4], [64, 128, 256])])
@pytest.mark.parametrize("index_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("pm", [O.SUM, O.MEAN])
@pytest.mark.parametrize("od", [O.FP32, O.FP16, O.BF16])
def test_lookup_port_equals_fbgemm(tys, dims, index_dtype, weighted, pm, od):
    rng = np.random.default_rng(1)
    c = make_case(rng, tys, dims, [3000] * len(tys), 37, [30] * len(tys), index_dtype, weighted, prune_frac=0.02)
    a = oracle_lookup(c, pm, od, "port")
    b = oracle_lookup(c, pm, od, "ref")
    if od == O.BF16:
        # FBGEMM rounds bf16 ties half away from zero, the oracle half to even: they may differ only
        # where the fp32 sum lies exactly half way between two bf16 values
        f32 = oracle_lookup(c, pm, O.FP32, "ref")
        tie = (f32.view(np.uint32) & 0xffff) == 0x8000
        assert np.all((a == b) | tie)
        ulp = np.maximum(np.abs(a), 2.0 ** -126) * 2.0 ** -7
        assert np.all(np.abs(a - b) <= ulp)
    else:
        assert np.array_equal(bits(a), bits(b))


@pytest.mark.parametrize("ebits,ebias", [(4, 7), (5, 15), (4, 14)])
@pytest.mark.parametrize("weighted", [False, True])
def test_lookup_fp8_port_equals_fbgemm(ebits, ebias, weighted):
    """FP8 rows are the one weight type the reference's device kernel implements
    (c310/op_kernel/common.h:120-167); its bit-placement decode is restated in the oracle."""
    rng = np.random.default_rng(2)
    c = make_case(rng, [O.FP8, O.FP8], [64, 20], [3000, 100], 37, [30, 30], np.int32, weighted)
    for pm in (O.SUM, O.MEAN):
        a = oracle_lookup(c, pm, O.FP32, "port", fp8=(ebits, ebias))
        b = oracle_lookup(c, pm, O.FP32, "ref", fp8=(ebits, ebias))
        assert np.array_equal(bits(a), bits(b))


def test_fp8_decode_all_codes():
    """Every byte against an independent formula: (-1)^s * 2^(e-bias) * (1 + m/2^mbits), subnormals
    m/2^mbits * 2^(1-bias)."""
    lib = O._lib("port")
    for ebits, ebias in ((4, 7), (5, 15)):
        mbits = 7 - ebits
        for b in range(256):
            s, e, m = b >> 7, (b >> mbits) & ((1 << ebits) - 1), b & ((1 << mbits) - 1)
            want = (m / (1 << mbits)) * 2.0 ** (1 - ebias) if e == 0 else (1 + m / (1 << mbits)) * 2.0 ** (e - ebias)
            want = -want if s else want
            assert lib.orc_fp8_to_f32(b, ebits, ebias) == np.float32(want)


def test_half_and_bf16_conversions_match_numpy_and_torch():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 1, 5000), rng.normal(0, 1e-6, 2000), rng.normal(0, 1e4, 2000),
                        [0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 2.0 ** -24, 2.0 ** -25, np.inf, -np.inf]]).astype(np.float32)
    lib = O._lib("port")
    got16 = np.array([lib.orc_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got16, x.astype(np.float16).view(np.uint16))
    gotbf = np.array([lib.orc_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(gotbf, torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))


# ---- 3. reference known answers ------------------------------------------------------

def test_permute_known_answers():
    # permute_pooled_embedding_test.py:79-86 with the net of common.py:69-78
    out = O.permute_pooled_embs(np.arange(10, dtype=np.float32)[None], [0, 2, 5, 6, 10], [3, 0, 2, 1], [0, 4, 6, 7, 10])
    assert out.reshape(-1).tolist() == [6, 7, 8, 9, 0, 1, 5, 2, 3, 4]
    # permute_pooled_embedding_modules.py:45-80
    x = np.arange(48, dtype=np.float32).reshape(3, 16)
    out = O.permute_pooled_embs(x, [0, 4, 8, 16], [2, 0, 1], [0, 8, 12, 16])
    assert out[0].tolist() == [8, 9, 10, 11, 12, 13, 14, 15, 0, 1, 2, 3, 4, 5, 6, 7]
    assert out[2].tolist() == [40, 41, 42, 43, 44, 45, 46, 47, 32, 33, 34, 35, 36, 37, 38, 39]
    # permute_pooled_embedding_test.py:120-160: equals concatenating the parts in the new order
    rng = np.random.default_rng(0)
    dims, order = [1, 2, 3, 4, 5], [2, 1, 3, 0, 4]
    parts = [rng.random((4, d)).astype(np.float16) for d in dims]
    off = np.concatenate([[0], np.cumsum(dims)])
    inv_off = np.concatenate([[0], np.cumsum([dims[i] for i in order])])
    out = O.permute_pooled_embs(np.concatenate(parts, 1), off, order, inv_off)
    assert np.array_equal(out, np.concatenate([parts[i] for i in order], 1))
    with pytest.raises(RuntimeError):
        O.permute_pooled_embs(x, [0, 4, 8, 16], [2, 0, 3], [0, 8, 12, 16])
