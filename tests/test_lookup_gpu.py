"""Parity of the CUDA lookup with the CPU oracle, on the reference's own test grids
(bench/tbe_inference/.../test_int_nbit_split_embedding_codegen_lookup_function.py:372-487) extended
to every weight type, plus the edge cases of the domain (empty bags, pruned indices, ragged
bags, unaligned rows, very wide rows)."""
import random
import zlib

import numpy as np
import pytest

import oracle as O
from helpers import Case, assert_close, gpu_lookup, make_case, oracle_lookup

pytestmark = pytest.mark.gpu

ALIGN = {O.FP32: 1, O.FP16: 2, O.INT8: 4, O.INT4: 8, O.INT2: 16, O.FP8: 4}
OUT_ALIGN = {O.FP32: 1, O.FP16: 2, O.BF16: 2}


def seed_of(*args):
    return zlib.crc32(repr(args).encode()) & 0x7fffffff


def round_up(a, b):
    return (a + b - 1) // b * b


def run(c: Case, pooling, out_ty, what, fp8=(4, 7)):
    want = oracle_lookup(c, pooling, out_ty, fp8=fp8)
    got = gpu_lookup(c, pooling, out_ty, fp8=fp8)
    assert_close(got, want, out_ty, what)


@pytest.mark.parametrize("weights_ty", [O.INT8, O.INT4, O.FP16, O.FP8, O.FP32, O.INT2])
@pytest.mark.parametrize("pooling", [O.SUM, O.MEAN])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("index_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("out_ty", [O.FP16, O.FP32, O.BF16])
@pytest.mark.parametrize("table_num", [1, 4, 10])
def test_random_multi_table_forward(weights_ty, pooling, weighted, index_dtype, out_ty, table_num):
    """Random tables: E in [1, 20000], D = 4*rand(1..1024) rounded to the type's alignment, B = 64,
    per-table bag length in [1, 100] (the reference's generator, :238-277)."""
    seed = seed_of(weights_ty, pooling, weighted, index_dtype.__name__, out_ty, table_num) & 0xffff
    rnd = random.Random(10000 + seed)
    rng = np.random.default_rng(10000 + seed)
    rows = [rnd.randint(1, 20000) for _ in range(table_num)]
    dims = [round_up(4 * rnd.randint(1, 1024), max(ALIGN[weights_ty], OUT_ALIGN[out_ty])) for _ in range(table_num)]
    if table_num == 10:
        dims = [min(d, 1024) for d in dims]   # keeps the CPU oracle quick; 4096-wide rows are covered below
    L = [rnd.randint(1, 100) for _ in range(table_num)]
    B = 64
    lens = np.concatenate([np.full(B, l) for l in L])
    c = make_case(rng, [weights_ty] * table_num, dims, rows, B, lens, index_dtype, weighted)
    run(c, pooling, out_ty, f"ty={weights_ty} dims={dims}")


BAG_TABLES = [
    [(1000, 16), (2000, 16)], [(2000, 256), (1000, 256)], [(2000, 512), (1000, 512)], [(2000, 1024), (1000, 1024)],
    [(2000, 2048), (1000, 2048)], [(2000, 4096), (1000, 4096)], [(2000, 16), (1000, 256)], [(2000, 16), (1000, 512)],
    [(2000, 16), (1000, 1024)], [(2000, 16), (1000, 2048)], [(2000, 16), (1000, 4096)],
]


@pytest.mark.parametrize("weights_ty", [O.INT8, O.FP8])
@pytest.mark.parametrize("pooling", [O.SUM, O.MEAN])
@pytest.mark.parametrize("weighted", [True, False])
@pytest.mark.parametrize("index_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("out_ty", [O.FP16, O.FP32, O.BF16])
@pytest.mark.parametrize("tables", BAG_TABLES)
def test_double_table_forward_bag(weights_ty, pooling, weighted, index_dtype, out_ty, tables):
    """The reference's fixed two-table grid (:418-460), bag lengths 40 and 50, B = 64."""
    rng = np.random.default_rng(seed_of(weights_ty, pooling, weighted, out_ty, tables))
    rows = [e for e, _ in tables]
    dims = [d for _, d in tables]
    lens = np.concatenate([np.full(64, 40), np.full(64, 50)])
    c = make_case(rng, [weights_ty] * 2, dims, rows, 64, lens, index_dtype, weighted)
    run(c, pooling, out_ty, f"tables={tables}")


NOBAG_TABLES = [
    [(1000, 16), (2000, 16)], [(1000, 32), (2000, 32)], [(1000, 64), (2000, 64)], [(1000, 128), (2000, 128)],
    [(2000, 256), (1000, 256)], [(2000, 512), (1000, 512)], [(2000, 1024), (1000, 1024)],
    [(2000, 2048), (1000, 2048)], [(2000, 4096), (1000, 4096)],
]


@pytest.mark.parametrize("weights_ty", [O.INT8, O.INT4, O.FP8, O.FP16])
@pytest.mark.parametrize("out_ty", [O.FP16, O.FP32, O.BF16])
@pytest.mark.parametrize("index_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("tables", NOBAG_TABLES)
def test_double_table_forward_nobag(weights_ty, out_ty, index_dtype, tables):
    """Pooling NONE, equal D across tables (:463-487)."""
    rng = np.random.default_rng(seed_of(weights_ty, out_ty, tables))
    rows = [e for e, _ in tables]
    dims = [d for _, d in tables]
    lens = np.concatenate([np.full(64, 40), np.full(64, 50)])
    c = make_case(rng, [weights_ty] * 2, dims, rows, 64, lens, index_dtype, False)
    run(c, O.NONE, out_ty, f"nobag tables={tables}")


@pytest.mark.parametrize("index_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("out_ty", [O.FP32, O.FP16])
@pytest.mark.parametrize("pooling", [O.SUM, O.MEAN])
def test_mixed_types_jagged_empty_pruned(index_dtype, out_ty, pooling):
    """Mixed weight types in one launch, bag lengths uniform in [0, 200] (empty bags included),
    2% pruned (-1) indices, per-sample weights: the shape of benchmark configuration 5."""
    rng = np.random.default_rng(5)
    tys = [O.INT8, O.INT4, O.FP16, O.INT8, O.INT4, O.FP16, O.FP8, O.FP32, O.INT2]
    dims = [128, 128, 128, 64, 256, 32, 96, 20, 48]
    rows = [5000] * len(tys)
    B = 33
    lens = rng.integers(0, 201, len(tys) * B)
    lens[::7] = 0
    c = make_case(rng, tys, dims, rows, B, lens, index_dtype, True, prune_frac=0.02)
    run(c, pooling, out_ty, "mixed")


@pytest.mark.parametrize("weights_ty", [O.INT8, O.INT4, O.FP16, O.FP32, O.FP8, O.INT2])
@pytest.mark.parametrize("row_alignment", [1, 4, 16])
def test_row_alignment_and_unaligned_tables(weights_ty, row_alignment):
    """row_alignment 1 (unpadded rows, the layout upstream uses for CPU-built modules) and tables
    that start at odd byte offsets take the byte-wise path; results must not change."""
    rng = np.random.default_rng(row_alignment * 10 + weights_ty)
    dims = [round_up(d, ALIGN[weights_ty]) for d in (36, 128, 200)]
    c = make_case(rng, [weights_ty] * 3, dims, [777, 1000, 50], 16, [30, 5, 64], np.int64, True,
                  prune_frac=0.05, row_alignment=row_alignment, table_alignment=1 if row_alignment == 1 else 4)
    run(c, O.SUM, O.FP32, f"align={row_alignment}")


def test_all_bags_empty_through_c_abi():
    """No index at all: every output element must be zero.  (The operator, like the reference
    adapter, rejects an empty `indices`; the C ABI accepts it.)"""
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(0)
    c = make_case(rng, [O.INT8, O.FP16], [64, 32], [100, 100], 8, 0, np.int32)
    d = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    out = torch.full((8, 96), 7.0, dtype=torch.float16, device=d)
    cabi.lookup(t(c.dev_weights), t(c.weights_offsets), t(c.weights_tys), t(c.D_offsets), 96, 64,
                torch.zeros(0, dtype=torch.int32, device=d), t(c.offsets), O.SUM, out)
    assert float(out.abs().max()) == 0.0


def test_config1_full_size_matches_oracle_and_fbgemm():
    """Benchmark configuration 1 in full: T=1, E=100000, D=128 INT8 from N(0, 0.1) seed 0, B=512,
    L=20, int32, SUM, fp16 out -- against both the C restatement and the FBGEMM CPU kernels."""
    rng = np.random.default_rng(0)
    x = rng.normal(0.0, 0.1, (100_000, 128)).astype(np.float32)
    rows = O.pack_table(x, O.INT8)
    dev, wo, wt, do = O.concat_tables([rows], [O.INT8], [128])
    idx = rng.integers(0, 100_000, 512 * 20).astype(np.int32)
    offs = np.arange(0, 512 * 20 + 1, 20, dtype=np.int32)
    c = Case(dev, wo, wt, do, idx, offs, None, [O.INT8], [128], [100_000], 512)
    got = gpu_lookup(c, O.SUM, O.FP16)
    assert_close(got, oracle_lookup(c, O.SUM, O.FP16, impl="port"), O.FP16, "c1 vs port")
    assert_close(got, oracle_lookup(c, O.SUM, O.FP16, impl="ref"), O.FP16, "c1 vs fbgemm")


def test_error_flag_and_bad_arguments():
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(1)
    c = make_case(rng, [O.INT8], [32], [50], 4, 3, np.int64)
    c.indices[2] = -5   # invalid (only -1 means "pruned")
    d = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    out = torch.empty((4, 32), dtype=torch.float32, device=d)
    args = (t(c.dev_weights), t(c.weights_offsets), t(c.weights_tys), t(c.D_offsets), 32, 32, t(c.indices), t(c.offsets))
    cabi.lookup(*args, O.SUM, out, error_flag=flag)
    assert int(flag.item()) == 1
    c.indices[2] = -1
    assert_close(out.cpu().numpy(), oracle_lookup(c, O.SUM, O.FP32), O.FP32, "bad index skipped")
    with pytest.raises(RuntimeError, match="pooling_mode"):
        cabi.lookup(*args, 7, out)
    with pytest.raises(RuntimeError, match="rows_per_dest"):
        cabi.lookup(*args, O.SUM, out, dest_outputs=torch.zeros(1, dtype=torch.int64, device=d), rows_per_dest=0)
    # operator-level checks mirror the reference adapter's messages
    with pytest.raises(RuntimeError, match="indices can not be empty"):
        c2 = make_case(rng, [O.INT8], [32], [50], 4, 0, np.int64)
        gpu_lookup(c2, O.SUM, O.FP32)
    with pytest.raises(RuntimeError, match="is incorrect for feature count"):
        c3 = make_case(rng, [O.INT8, O.INT8], [32, 32], [50, 50], 4, 3, np.int64)
        c3.offsets = c3.offsets[:-1]
        gpu_lookup(c3, O.SUM, O.FP32)
    with pytest.raises(RuntimeError, match="Unsupported output_dtype"):
        gpu_lookup(c, O.SUM, 3)


def test_scatter_to_destinations_with_column_remap():
    """dest_outputs + output_col_offsets: the batch is split over several destination buffers and
    each table lands at a remapped column -- equal to lookup, split by rows, then permute."""
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(3)
    dims = [64, 128, 32, 128]
    c = make_case(rng, [O.INT8, O.INT4, O.FP16, O.INT8], dims, [300] * 4, 24, [20, 40, 3, 9], np.int64)
    want = oracle_lookup(c, O.SUM, O.FP16)
    perm = [2, 0, 3, 1]
    inv_dims = [dims[p] for p in perm]
    inv_off = np.concatenate([[0], np.cumsum(inv_dims)])
    off = np.concatenate([[0], np.cumsum(dims)])
    want_perm = np.concatenate([want[:, off[p]:off[p + 1]] for p in perm], axis=1)
    col = np.zeros(4, dtype=np.int64)
    for i, p in enumerate(perm):
        col[p] = inv_off[i]
    d = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    parts = [torch.zeros((8, sum(dims)), dtype=torch.float16, device=d) for _ in range(3)]
    ptrs = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=d)
    cabi.lookup(t(c.dev_weights), t(c.weights_offsets), t(c.weights_tys), t(c.D_offsets), sum(dims), max(dims),
                t(c.indices), t(c.offsets), O.SUM, parts[0], output_col_offsets=t(col), dest_outputs=ptrs,
                rows_per_dest=8)
    got = torch.cat(parts, 0).float().cpu().numpy()
    assert_close(got, want_perm, O.FP16, "scatter+remap")


@pytest.mark.parametrize("weights_ty,D", [(O.INT8, 128), (O.INT4, 64), (O.FP16, 32), (O.INT8, 20)])
@pytest.mark.parametrize("pooling", [O.SUM, O.NONE])
def test_row_past_the_table_is_skipped_and_reported(weights_ty, D, pooling):
    """An index >= the table's row count is never dereferenced: with dev_weights_bytes known the row is
    treated like a pruned one (-1) and bit 4 of the error word is set.  Checked for a table in the
    middle of dev_weights (the row would belong to the next table) and for the last one (the row would
    lie outside the buffer)."""
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(11)
    E = [40, 30, 50]
    c = make_case(rng, [weights_ty] * 3, [D] * 3, E, 8, np.concatenate([np.full(8, 9), np.full(8, 12), np.full(8, 5)]), np.int64)
    offs = c.offsets
    bad_positions = [int(offs[8]) + 3, int(offs[16]) + 1, int(offs[23]) + 2]   # one in the middle table, two in the last
    for q in bad_positions:
        t = int(np.searchsorted(offs[::8], q, side="right") - 1)
        c.indices[q] = E[t] + (0 if q == bad_positions[0] else 1000)
    d = torch.device("cuda")
    t_ = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    n_out = c.indices.size if pooling == O.NONE else 8
    width = D if pooling == O.NONE else 3 * D
    out = torch.full((n_out, width), 3.0, dtype=torch.float32, device=d)
    cabi.lookup(t_(c.dev_weights), t_(c.weights_offsets), t_(c.weights_tys), t_(c.D_offsets), 3 * D, D, t_(c.indices),
                t_(c.offsets), pooling, out, error_flag=flag)
    assert int(flag.item()) == 4
    for q in bad_positions:
        c.indices[q] = -1
    assert_close(out.cpu().numpy(), oracle_lookup(c, pooling, O.FP32), O.FP32, "rows past the table pruned")


def test_offsets_that_disagree_with_the_index_count_are_reported():
    """offsets[T*B] != indices.numel() (the reference kernel asserts on it) sets bit 8; positions past
    `indices` are never read."""
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(12)
    c = make_case(rng, [O.INT8, O.INT8], [64, 64], [100, 100], 8, 6, np.int32)
    d = torch.device("cuda")
    t_ = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    flag = torch.zeros(1, dtype=torch.int32, device=d)
    out = torch.zeros((8, 128), dtype=torch.float16, device=d)
    short = c.indices[:-5]                      # offsets describe 5 more positions than there are indices
    cabi.lookup(t_(c.dev_weights), t_(c.weights_offsets), t_(c.weights_tys), t_(c.D_offsets), 128, 64, t_(short), t_(c.offsets),
                O.SUM, out, error_flag=flag)
    assert int(flag.item()) & 8
    flag.zero_()
    cabi.lookup(t_(c.dev_weights), t_(c.weights_offsets), t_(c.weights_tys), t_(c.D_offsets), 128, 64, t_(c.indices), t_(c.offsets),
                O.SUM, out, error_flag=flag)
    assert int(flag.item()) == 0
    assert_close(out.float().cpu().numpy(), oracle_lookup(c, O.SUM, O.FP16), O.FP16, "consistent offsets")


@pytest.mark.parametrize("out_dtype", ["float16", "float32"])
def test_scatter_with_rows_that_are_not_16_byte_aligned(out_dtype):
    """Destination scatter with an output row of 68 elements (136 or 272 bytes: alternate rows are
    misaligned for 16-byte stores), a batch that is not a multiple of the lane-group count, and bag lengths
    that differ a lot, so that bags straddle the lane groups' ranges."""
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(13)
    dims = [32, 16, 20]
    B = 13
    lens = rng.integers(0, 60, 3 * B)
    lens[5] = 300
    c = make_case(rng, [O.INT8, O.INT8, O.INT8], dims, [200] * 3, B, lens, np.int32)
    out_ty = O.FP16 if out_dtype == "float16" else O.FP32
    want = oracle_lookup(c, O.SUM, out_ty)
    d = torch.device("cuda")
    t_ = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    rows_per_dest = 5
    parts = [torch.zeros((rows_per_dest, 68), dtype=getattr(torch, out_dtype), device=d) for _ in range(3)]
    ptrs = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=d)
    cabi.lookup(t_(c.dev_weights), t_(c.weights_offsets), t_(c.weights_tys), t_(c.D_offsets), 68, 32, t_(c.indices),
                t_(c.offsets), O.SUM, parts[0], dest_outputs=ptrs, rows_per_dest=rows_per_dest, output_stride=68)
    got = torch.cat(parts, 0)[:B].float().cpu().numpy()
    assert_close(got, want, out_ty, "misaligned scatter")

@pytest.mark.parametrize("index_dtype", [np.int32, np.int64])
@pytest.mark.parametrize("weighted", [False, True])
def test_one_wave_launch_with_ragged_bags(index_dtype, weighted):
    """A launch that fills the GPU about once (12 000 bags, 400 000 rows: every warp takes a handful of bags) with bags
    as unequal as they get: empty bags at the very start and end and in long stretches, one bag of 5000 rows, stretches
    of one-row bags, three table types and widths."""
    rng = np.random.default_rng(seed_of("one-wave", index_dtype.__name__, weighted))
    T, B = 3, 4000
    lens = rng.poisson(33, T * B).astype(np.int64)
    lens[:200] = 0
    lens[-300:] = 0
    lens[5000:5600] = 0
    lens[2000:2600] = 1
    lens[7000] = 5000
    lens[7001:7040] = 0
    lens[9000:9010] = 700
    c = make_case(rng, [O.INT8, O.INT4, O.FP16], [128, 64, 32], [5000, 3000, 2000], B, lens, index_dtype, weighted, prune_frac=0.01)
    assert c.indices.size > 350_000
    for pooling, out_ty in ((O.SUM, O.FP16), (O.MEAN, O.FP32)):
        run(c, pooling, out_ty, f"one wave, ragged bags, {index_dtype.__name__}")



@pytest.mark.parametrize("weights_ty", [O.INT8, O.INT4, O.FP16, O.FP8, O.FP32])
@pytest.mark.parametrize("D", [64, 128, 256, 512])
@pytest.mark.parametrize("weighted", [False, True])
def test_bags_that_straddle_lane_group_ranges(weights_ty, D, weighted):
    """Few, very unequal bags per table: one bag of a thousand rows next to empty and tiny ones, so that a
    bag is summed in pieces by several lane groups and put together by its owner; also a table whose bags
    are all empty and a batch of a single bag."""
    rng = np.random.default_rng(seed_of(weights_ty, D, weighted))
    for B, lens in ((5, [0, 1000, 0, 3, 1, 0, 0, 0, 0, 0, 2, 0, 0, 777, 1]), (1, [613, 0, 5]), (3, [1, 1, 1, 0, 0, 0, 64, 64, 65])):
        c = make_case(rng, [weights_ty] * 3, [D] * 3, [300, 50, 1000], B, np.asarray(lens), np.int64, weighted, prune_frac=0.01)
        for pooling, out_ty in ((O.SUM, O.FP16), (O.MEAN, O.FP32)):
            run(c, pooling, out_ty, f"straddle B={B}")
