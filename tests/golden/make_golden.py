"""Generates tests/golden/tbe_golden.npz: small input/output vectors for the quantized TBE path.

Outputs come from code that is NOT this repository's: the FBGEMM CPU kernels inside
libtorch_cpu.so (through oracle/_ref/libfbgemm_cpu_ref.so) and the torch.ops.quantized
embedding-bag pack/unpack/lookup operators built on the same library.  The reference's own
golden path (fbgemm_gpu 1.2.0 CPU operators) cannot be installed here; FBGEMM is the library it
is built on.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tbe_golden.npz")


def main():
    rng = np.random.default_rng(20240607)
    g = {}
    # --- quantizers: torch-core prepack ops (fp32 scale/bias for 8-bit, fp16 for 4-bit) ---
    x8 = rng.normal(0, 0.1, (48, 40)).astype(np.float32)
    x8[3] = 0.25            # constant row
    x8[4, :] = 0.0
    x8[5] *= 1e-6
    g["q8_in"] = x8
    g["q8_out"] = torch.ops.quantized.embedding_bag_byte_prepack(torch.from_numpy(x8)).numpy()
    g["q8_back"] = torch.ops.quantized.embedding_bag_byte_unpack(torch.from_numpy(g["q8_out"])).numpy()
    x4 = rng.uniform(-0.1, 0.1, (48, 64)).astype(np.float32)
    x4[7] = -0.5
    g["q4_in"] = x4
    g["q4_out"] = torch.ops.quantized.embedding_bag_4bit_prepack(torch.from_numpy(x4)).numpy()
    g["q4_out_fbgemm"] = O.quantize_nbit_rowwise_sbhalf(x4, 4, impl="ref")
    g["q2_out_fbgemm"] = O.quantize_nbit_rowwise_sbhalf(x4, 2, impl="ref")
    # --- lookups: FBGEMM EmbeddingSpMDM kernels in the table-batched layout ---
    tys = [O.INT8, O.INT4, O.FP16, O.INT2, O.FP32, O.INT8]
    dims = [32, 64, 16, 32, 12, 128]
    E, B = 60, 6
    tabs = [O.pack_table(rng.normal(0, 0.05, (E, d)).astype(np.float32), ty, impl="ref") for ty, d in zip(tys, dims)]
    dev, wo, wt, do = O.concat_tables(tabs, tys, dims)
    lens = rng.integers(0, 9, len(tys) * B)
    lens[4] = 0
    offs = np.zeros(len(tys) * B + 1, dtype=np.int64)
    offs[1:] = np.cumsum(lens)
    idx = rng.integers(0, E, int(offs[-1])).astype(np.int64)
    idx[::11] = -1
    w = rng.random(idx.size).astype(np.float32)
    g.update(lk_dev=dev, lk_wo=wo, lk_wt=wt, lk_do=do, lk_idx=idx, lk_offs=offs, lk_w=w)
    for pm, pname in ((O.SUM, "sum"), (O.MEAN, "mean")):
        for weighted in (False, True):
            for od, oname in ((O.FP32, "f32"), (O.FP16, "f16")):
                out = O.tbe_lookup(dev, wo, wt, do, idx, offs, pm, w if weighted else None, od, impl="ref")
                g[f"lk_{pname}_{'w' if weighted else 'u'}_{oname}"] = out
    # FP8 rows (the weight type the reference's device kernel implements), no pruned indices
    fp8 = rng.integers(0, 256, (E, 24), dtype=np.uint8) & np.uint8(0xBF)
    dev8, wo8, wt8, do8 = O.concat_tables([O.pack_table(fp8, O.FP8)], [O.FP8], [24])
    offs8 = np.arange(0, 6 * 5 + 1, 5, dtype=np.int32)
    idx8 = rng.integers(0, E, 30).astype(np.int32)
    g.update(f8_dev=dev8, f8_wo=wo8, f8_wt=wt8, f8_do=do8, f8_idx=idx8, f8_offs=offs8)
    g["f8_sum_e4b7"] = O.tbe_lookup(dev8, wo8, wt8, do8, idx8, offs8, O.SUM, None, O.FP32, 16, 4, 7, impl="ref")
    g["f8_mean_e5b15"] = O.tbe_lookup(dev8, wo8, wt8, do8, idx8, offs8, O.MEAN, None, O.FP32, 16, 5, 15, impl="ref")
    # torch-core fused-row lookups with fp16-representable scale/bias (independent entry point)
    xq = rng.normal(0, 0.1, (200, 32)).astype(np.float32)
    fused = O.quantize_8bit_rowwise(xq, impl="ref").copy()
    sb = fused[:, 32:40].copy().view(np.float32).astype(np.float16).astype(np.float32)
    fused[:, 32:40] = sb.view(np.uint8)
    eidx = rng.integers(0, 200, 50).astype(np.int64)
    eoffs = np.arange(0, 51, 5, dtype=np.int64)
    g.update(eb_fused=fused, eb_idx=eidx, eb_offs=eoffs)
    g["eb_out"] = torch.ops.quantized.embedding_bag_byte_rowwise_offsets(
        torch.from_numpy(fused), torch.from_numpy(eidx), torch.from_numpy(eoffs), False, 0, False, None, None, True).numpy()
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes;", len(g), "arrays")


if __name__ == "__main__":
    main()
