"""Parity at the sizes that are benchmarked: the five benchmark configurations at their full table
sizes, batch sizes, bag-length and index distributions and index widths.

Configuration 2 is compared with the CPU oracle in full (its 3.7 GB of tables fit the host).  The
tables of configurations 3, 4 and 5 (30-110 GB) do not, so a sample of at least 4096 (table, bag)
pairs per run is checked, the longest bags of the batch always among them: only the rows those bags
reference are copied to the host and pooled by the oracle (``oracle.sampling``).  Sampled table rows are
also compared byte for byte with the CPU quantizer's packing of the same fp32 source rows.
Tolerances are the reference's (test_int_nbit_split_embedding_codegen_lookup_function.py:345-366).
"""
import numpy as np
import pytest

import oracle as O
from oracle.sampling import check_sampled_bags

pytestmark = pytest.mark.gpu


def _free_gib():
    import torch
    free, _ = torch.cuda.mem_get_info()
    return free / 2 ** 30


class RowSampler:
    """Keeps a few fp32 source rows of every table while the tables are generated."""

    def __init__(self, per_chunk=4, every=8):
        self.per_chunk, self.every, self.n, self.kept = per_chunk, every, 0, []

    def __call__(self, t, r0, x):
        self.n += 1
        if self.n % self.every == 1:
            ids = [0, x.shape[0] // 3, x.shape[0] - 1][: self.per_chunk]
            self.kept.append((t, [r0 + i for i in ids], x[ids].cpu().numpy()))


def _check_rows(tables, sampler):
    """Quantized table rows byte for byte against the CPU quantizer + packing."""
    import torch
    for t, row_ids, x in sampler.kept:
        ty = int(tables.specs[t].weight_ty)
        want = O.pack_table(x, ty, tables.row_alignment)
        got = tables.table_rows(t).index_select(0, torch.tensor(row_ids, device=tables.device)).cpu().numpy()
        assert np.array_equal(got, want), f"table {t} rows {row_ids}: quantized bytes differ from the CPU packing"
    return len(sampler.kept)


def _build(name, **kw):
    import torch
    from fbgemm_ascend_b200 import workloads as W
    ws = W.spec(name, **kw)
    need = W.table_bytes(ws) / 2 ** 30 + 12
    if _free_gib() < need:
        pytest.skip(f"{name} needs about {need:.0f} GiB of free device memory")
    sampler = RowSampler()
    tables = W.build_tables(ws, torch.device("cuda"), row_hook=sampler)
    return W, ws, tables, sampler


def test_config2_full_against_oracle():
    """Configuration 2, every bag: T=26 x 1M x 128 INT8, B=2048, Poisson(30) lengths, Zipf(1.05), int64, SUM -> fp16."""
    import torch
    W, ws, tables, sampler = _build("c2")
    assert _check_rows(tables, sampler) > 0
    dev_h = tables.weights_dev.cpu().numpy()
    wo, wt, do = (tables.weights_offsets.cpu().numpy(), tables.weights_tys.cpu().numpy(), tables.D_offsets.cpu().numpy())
    for seed in (0, 1):
        b = W.make_batch(ws, tables.device, batch_seed=seed)
        got = tables.forward(b.indices, b.offsets, b.weights).float().cpu().numpy()
        want = O.tbe_lookup(dev_h, wo, wt, do, b.indices.cpu().numpy(), b.offsets.cpu().numpy(), O.SUM, None, O.FP16,
                            impl="ref").astype(np.float32)
        err = np.abs(got - want)
        assert np.all(err <= 1e-3 + 1e-3 * np.abs(want)), f"c2 batch {seed}: max err {err.max():.3e}"
        lens = np.diff(b.offsets.cpu().numpy())
        assert lens.max() >= 45        # long bags of the folded INT8 -> fp16 path are in the batch
    del tables
    torch.cuda.empty_cache()


@pytest.mark.parametrize("name", ["c3", "c5", "c4"])
def test_large_config_sampled_against_oracle(name):
    """Configurations 3 (INT4 mixed widths, MEAN -> fp32), 5 (weighted INT8/INT4/FP16, jagged with empty bags, -> fp32)
    and 4 (one rank's 64 INT8 tables of 12M rows, Poisson(32) up to 128 rows per bag, -> fp16; int64 and int32
    indices) at full size, on a sample of bags that includes the longest ones."""
    import torch
    W, ws, tables, sampler = _build(name)
    assert _check_rows(tables, sampler) > 0
    b = W.make_batch(ws, tables.device, batch_seed=0)
    variants = [(b.indices, b.offsets)]
    if name == "c4":
        variants.append((b.indices.to(torch.int32), b.offsets.to(torch.int32)))
    for idx, offs in variants:
        out = tables.forward(idx, offs, b.weights)
        r = check_sampled_bags(tables, idx, offs, b.weights, out, n_samples=4096, n_longest=512, seed=1)
        assert r["ok"], f"{name} {idx.dtype}: {r}"
        assert r["bags"] >= 4096
        if name == "c4":
            assert r["max_len"] >= 60, r     # the tail of Poisson(32): the long bags of the folded path
        if name == "c5":
            assert r["max_len"] == 200, r
        del out
    if name == "c4":
        # Poisson(32) hardly ever gives a bag of more than 70 rows; the configuration allows up to 128.  The same tables
        # with bags of 100 to 128 rows (a smaller batch) put the folded INT8 -> fp16 accumulation at its longest.
        ws.length_dist = "uniform:100:128"
        ws.B = 4096
        bl = W.make_batch(ws, tables.device, batch_seed=7)
        out = tables.forward(bl.indices, bl.offsets, None)
        r = check_sampled_bags(tables, bl.indices, bl.offsets, None, out, n_samples=4096, n_longest=512, seed=2)
        assert r["ok"] and r["max_len"] == 128, f"c4 long bags: {r}"
        del out, bl
    del tables, b
    torch.cuda.empty_cache()


def test_sampled_check_detects_a_wrong_result():
    """The sampled comparison is not vacuous: a perturbed output is reported."""
    import torch
    from fbgemm_ascend_b200 import workloads as W
    ws = W.spec("c2", scale_E=0.01, scale_B=0.25)
    tables = W.build_tables(ws, torch.device("cuda"))
    b = W.make_batch(ws, tables.device, batch_seed=3)
    out = tables.forward(b.indices, b.offsets, b.weights)
    assert check_sampled_bags(tables, b.indices, b.offsets, None, out, n_samples=512)["ok"]
    out += 0.05
    assert not check_sampled_bags(tables, b.indices, b.offsets, None, out, n_samples=512)["ok"]
