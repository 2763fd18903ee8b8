"""Seeded synthetic workloads for the quantized TBE inference path.

Each generator builds, on the GPU, the tables and one or more request batches of one of the
five benchmark configurations (or a scaled-down version of it for tests):

    c1  T=1,   E=1e5,   D=128 INT8,            B=512,   L=20,               uniform, int32, SUM  -> fp16
    c2  T=26,  E=1e6,   D=128 INT8,            B=2048,  L~Poisson(30)[1,100], Zipf 1.05, int64, SUM  -> fp16
    c3  T=64,  E=1e7,   D in {64,128,256} INT4, B=16384, L=40,               Zipf 1.1,  int32, MEAN -> fp32
    c4  64 tables per rank, E=1.2e7, D=128 INT8, B=65536, L~Poisson(32)[1,128], Zipf 1.05, int64, SUM -> fp16
    c5  T=96,  E=2e6,   D=128 INT8/INT4/FP16,  B=8192,  L~U{0..200},        uniform, int64, weighted SUM -> fp32

No public dataset is involved; these generators are the benchmark inputs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .modules import IntNBitTableBatchedEmbeddingBags
from .types import PoolingMode, SparseType, row_bytes


@dataclass
class WorkloadSpec:
    name: str
    T: int
    E: int
    dims: List[int]
    tys: List[SparseType]
    B: int
    pooling: PoolingMode
    output_dtype: SparseType
    index_dtype: torch.dtype
    length_dist: str                 # "fixed:L" | "poisson:mean:lo:hi" | "uniform:lo:hi"
    index_dist: str                  # "uniform" | "zipf:alpha"
    weighted: bool
    table_dist: str                  # "normal:std" | "uniform:half_range"
    seed: int


def spec(name: str, scale_E: float = 1.0, scale_B: float = 1.0, scale_T: float = 1.0, tables: Optional[int] = None) -> WorkloadSpec:
    """The named configuration, optionally scaled down (rows E, batch B, table count T)."""
    S, P = SparseType, PoolingMode

    def sc(v, f):
        return max(1, int(round(v * f)))

    if name == "c1":
        T = 1
        return WorkloadSpec("c1", T, sc(100_000, scale_E), [128], [S.INT8], sc(512, scale_B), P.SUM, S.FP16, torch.int32,
                            "fixed:20", "uniform", False, "normal:0.1", 0)
    if name == "c2":
        T = tables or sc(26, scale_T)
        return WorkloadSpec("c2", T, sc(1_000_000, scale_E), [128] * T, [S.INT8] * T, sc(2048, scale_B), P.SUM, S.FP16,
                            torch.int64, "poisson:30:1:100", "zipf:1.05", False, "normal:0.05", 1)
    if name == "c3":
        T = tables or sc(64, scale_T)
        return WorkloadSpec("c3", T, sc(10_000_000, scale_E), [[64, 128, 256][t % 3] for t in range(T)], [S.INT4] * T,
                            sc(16384, scale_B), P.MEAN, S.FP32, torch.int32, "fixed:40", "zipf:1.1", False,
                            "uniform:0.1", 2)
    if name == "c4":
        T = tables or sc(64, scale_T)   # tables held by one rank
        return WorkloadSpec("c4", T, sc(12_000_000, scale_E), [128] * T, [S.INT8] * T, sc(65536, scale_B), P.SUM, S.FP16,
                            torch.int64, "poisson:32:1:128", "zipf:1.05", False, "normal:0.05", 3)
    if name == "c5":
        T = tables or sc(96, scale_T)
        return WorkloadSpec("c5", T, sc(2_000_000, scale_E), [128] * T, [[S.INT8, S.INT4, S.FP16][t % 3] for t in range(T)],
                            sc(8192, scale_B), P.SUM, S.FP32, torch.int64, "uniform:0:200", "uniform", True,
                            "normal:0.05", 4)
    raise ValueError(f"unknown workload {name!r}")


def table_bytes(ws: WorkloadSpec, row_alignment: int = 16) -> int:
    return sum(ws.E * row_bytes(ty, d, row_alignment) for ty, d in zip(ws.tys, ws.dims))


def build_tables(ws: WorkloadSpec, device: torch.device, table_seed_offset: int = 0,
                 chunk_rows: int = 1 << 20, row_hook: Optional[Callable] = None) -> IntNBitTableBatchedEmbeddingBags:
    """Generate fp32 rows on the device chunk by chunk, quantize them into the flat table buffer
    and drop the fp32 (so a 110 GB shard never needs a second copy).  ``row_hook(t, r0, x)`` sees every
    fp32 chunk (rows r0.. of table t) before it is dropped, e.g. to keep a sample of source rows."""
    specs = [(f"t{t}", ws.E, ws.dims[t], ws.tys[t]) for t in range(ws.T)]
    m = IntNBitTableBatchedEmbeddingBags(specs, device=device, pooling_mode=ws.pooling, output_dtype=ws.output_dtype,
                                         indices_dtype=ws.index_dtype)
    kind, val = ws.table_dist.split(":")
    val = float(val)

    row0 = {}

    def make_rows(t, n, D, gen):
        if kind == "normal":
            x = torch.randn(n, D, device=device, generator=gen) * val
        else:
            x = (torch.rand(n, D, device=device, generator=gen) * 2.0 - 1.0) * val
        if row_hook is not None:
            row_hook(t, row0.get(t, 0), x)
            row0[t] = row0.get(t, 0) + n
        return x

    m.fill_random_weights(make_rows, seed=ws.seed * 1000 + table_seed_offset, chunk_rows=chunk_rows)
    return m


@dataclass
class Batch:
    indices: torch.Tensor
    offsets: torch.Tensor
    weights: Optional[torch.Tensor]
    lengths_sum_per_table: List[int] = field(default_factory=list)

    @property
    def num_rows(self) -> int:
        return self.indices.numel()


class _ZipfSampler:
    """Bounded Zipf over ranks 1..E by inverse CDF on a float64 cumulative sum; rank r maps to row
    perm[r-1] with a per-table seeded permutation, so hot rows are scattered over the table."""

    def __init__(self, E: int, alpha: float, device: torch.device):
        ranks = torch.arange(1, E + 1, device=device, dtype=torch.float64)
        self.cdf = torch.cumsum(ranks.pow_(-alpha), 0)
        self.E = E
        self.device = device

    def sample(self, n: int, gen: torch.Generator, perm: torch.Tensor) -> torch.Tensor:
        u = torch.rand(n, device=self.device, dtype=torch.float64, generator=gen) * self.cdf[-1]
        r = torch.searchsorted(self.cdf, u).clamp_(max=self.E - 1)
        return perm[r]


def make_batch(ws: WorkloadSpec, device: torch.device, batch_seed: int = 0, table_ids: Optional[Sequence[int]] = None) -> Batch:
    """One request batch: table-major offsets [T*B+1] and indices, all on the device.

    ``table_ids`` are the global ids of the tables (they seed the per-table row permutation, so a
    table keeps its hot rows from batch to batch and from rank to rank)."""
    gen = torch.Generator(device=device)
    gen.manual_seed((ws.seed + 1) * 1_000_003 + batch_seed)
    T, B = ws.T, ws.B
    parts = ws.length_dist.split(":")
    if parts[0] == "fixed":
        lengths = torch.full((T * B,), int(parts[1]), device=device, dtype=torch.int64)
    elif parts[0] == "poisson":
        mean, lo, hi = float(parts[1]), int(parts[2]), int(parts[3])
        lengths = torch.poisson(torch.full((T * B,), mean, device=device), generator=gen).to(torch.int64).clamp_(lo, hi)
    else:
        lo, hi = int(parts[1]), int(parts[2])
        lengths = torch.randint(lo, hi + 1, (T * B,), device=device, generator=gen, dtype=torch.int64)
    offsets = torch.zeros(T * B + 1, device=device, dtype=torch.int64)
    torch.cumsum(lengths, 0, out=offsets[1:])
    per_table = lengths.view(T, B).sum(1).tolist()
    N = int(sum(per_table))
    indices = torch.empty(N, device=device, dtype=torch.int64)
    ids = list(table_ids) if table_ids is not None else list(range(T))
    sampler = None
    if ws.index_dist.startswith("zipf"):
        sampler = _ZipfSampler(ws.E, float(ws.index_dist.split(":")[1]), device)
    pos = 0
    for t in range(T):
        n = int(per_table[t])
        if sampler is not None:
            pg = torch.Generator(device=device)
            pg.manual_seed(ws.seed * 7919 + 17 * ids[t] + 1)
            perm = torch.randperm(ws.E, device=device, generator=pg)
            indices[pos:pos + n] = sampler.sample(n, gen, perm)
        else:
            indices[pos:pos + n] = torch.randint(0, ws.E, (n,), device=device, generator=gen, dtype=torch.int64)
        pos += n
    weights = torch.rand(N, device=device, generator=gen) if ws.weighted else None
    return Batch(indices.to(ws.index_dtype), offsets.to(ws.index_dtype), weights, [int(x) for x in per_table])


def algorithmic_bytes(ws: WorkloadSpec, batch: Batch) -> Dict[str, int]:
    """Bytes one lookup call must move: unpadded rows (D+4 INT8, D/2+4 INT4, 2D FP16, ...), indices,
    offsets, per-sample weights, output.  Also the padded-stride and 32-byte-sector figures."""
    isz = 4 if ws.index_dtype == torch.int32 else 8
    osz = 4 if ws.output_dtype == SparseType.FP32 else 2
    rows_unpadded = rows_padded = rows_sector = 0
    for t in range(ws.T):
        n = batch.lengths_sum_per_table[t]
        ub = row_bytes(ws.tys[t], ws.dims[t], 1)
        pb = row_bytes(ws.tys[t], ws.dims[t], 16)
        rows_unpadded += n * ub
        rows_padded += n * pb
        # 16-byte-aligned rows of pb bytes: average number of 32-byte sectors touched by the used bytes
        # rows are 16-byte aligned: with a stride that is not a multiple of 32 they start at byte 0 or
        # 16 of a sector in turn
        sect = ((ub + 31) // 32 + (ub + 16 + 31) // 32) / 2 if pb % 32 else (ub + 31) // 32
        rows_sector += int(n * sect * 32)
    other = batch.num_rows * isz + (ws.T * ws.B + 1) * isz + (batch.num_rows * 4 if ws.weighted else 0) \
        + ws.B * sum(ws.dims) * osz
    return {"algorithmic": rows_unpadded + other, "padded": rows_padded + other, "sector": rows_sector + other,
            "rows": batch.num_rows}
