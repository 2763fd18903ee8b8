"""Shared test helpers: random table-batched cases built on the CPU, the oracle call, and the
comparison with the tolerances the reference's tests use
(test_int_nbit_split_embedding_codegen_lookup_function.py:358-363: rtol = atol = 1e-3 for fp16,
2**-7 for bf16, 1e-4 for fp32)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

import oracle as O

TOL = {O.FP16: 1e-3, O.BF16: 2.0 ** -7, O.FP32: 1e-4}


@dataclass
class Case:
    dev_weights: np.ndarray
    weights_offsets: np.ndarray
    weights_tys: np.ndarray
    D_offsets: np.ndarray
    indices: np.ndarray
    offsets: np.ndarray
    weights: Optional[np.ndarray]
    tys: List[int]
    dims: List[int]
    rows: List[int]
    B: int
    row_alignment: int = 16

    @property
    def T(self):
        return len(self.tys)

    @property
    def total_D(self):
        return int(self.D_offsets[-1])

    @property
    def max_D(self):
        return max(self.dims)

    def max_d_of(self, ty):
        return max([d for d, t in zip(self.dims, self.tys) if t == ty], default=0)


def random_table(rng, ty, E, D, row_alignment=16, std=0.05):
    if ty == O.FP8:
        x = rng.integers(0, 256, (E, D), dtype=np.uint8) & np.uint8(0xBF)   # exponent field <= 7: |v| < 2
    else:
        x = rng.normal(0.0, std, (E, D)).astype(np.float32)
    return O.pack_table(x, ty, row_alignment)


def make_case(rng, tys: Sequence[int], dims: Sequence[int], rows: Sequence[int], B: int, lengths,
              index_dtype=np.int32, weighted=False, prune_frac=0.0, row_alignment=16, table_alignment=16) -> Case:
    """``lengths``: an int (fixed L), a list with one max-L per table (uniform in [0, L]), or an
    explicit array of T*B lengths."""
    T = len(tys)
    tabs = [random_table(rng, ty, E, D, row_alignment) for ty, D, E in zip(tys, dims, rows)]
    dev, wo, wt, do = O.concat_tables(tabs, tys, dims, table_alignment)
    if isinstance(lengths, (int, np.integer)):
        lens = np.full(T * B, int(lengths), dtype=np.int64)
    elif len(lengths) == T:
        lens = np.concatenate([rng.integers(0, int(l) + 1, B) for l in lengths]).astype(np.int64)
    else:
        lens = np.asarray(lengths, dtype=np.int64)
    offsets = np.zeros(T * B + 1, dtype=index_dtype)
    offsets[1:] = np.cumsum(lens)
    idx = np.concatenate([rng.integers(0, rows[t], int(lens[t * B:(t + 1) * B].sum())) for t in range(T)] +
                         [np.zeros(0, dtype=np.int64)]).astype(index_dtype)
    if prune_frac > 0 and idx.size:
        idx[rng.random(idx.size) < prune_frac] = -1
    w = rng.random(idx.size).astype(np.float32) if weighted else None
    return Case(dev, wo, wt, do, idx, offsets, w, list(tys), list(dims), list(rows), B, row_alignment)


def oracle_lookup(c: Case, pooling, out_ty, impl="port", fp8=(4, 7)) -> np.ndarray:
    out = O.tbe_lookup(c.dev_weights, c.weights_offsets, c.weights_tys, c.D_offsets, c.indices, c.offsets, pooling,
                       c.weights, out_ty, c.row_alignment, fp8[0], fp8[1], impl=impl)
    return O.bf16_bits_to_f32(out) if out_ty == O.BF16 else out.astype(np.float32)


def assert_close(got: np.ndarray, want: np.ndarray, out_ty: int, what: str = "") -> None:
    tol = TOL[out_ty]
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    err = np.abs(got - want)
    bad = err > tol + tol * np.abs(want)
    if bad.any() or not np.isfinite(got).all():
        i = np.argwhere(bad)[:5]
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} elements beyond rtol=atol={tol}; max err "
                             f"{float(err.max()):.3e}; first at {i.tolist()}")


# ---- GPU side ------------------------------------------------------------------

def gpu_lookup(c: Case, pooling, out_ty, fp8=(4, 7), device="cuda"):
    """Run the torch operator on the case; returns a float32 numpy array."""
    import torch
    import fbgemm_ascend_b200  # noqa: F401  (registers the operators)

    d = torch.device(device)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(d)
    out = torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function(
        dev_weights=t(c.dev_weights), uvm_weights=torch.empty(0, dtype=torch.uint8, device=d),
        weights_placements=torch.zeros(c.T, dtype=torch.int32, device=d), weights_offsets=t(c.weights_offsets),
        weights_tys=t(c.weights_tys), D_offsets=t(c.D_offsets), total_D=c.total_D,
        max_int2_D=c.max_d_of(O.INT2), max_int4_D=c.max_d_of(O.INT4), max_int8_D=c.max_d_of(O.INT8),
        max_float16_D=c.max_d_of(O.FP16), max_float32_D=c.max_d_of(O.FP32), indices=t(c.indices), offsets=t(c.offsets),
        pooling_mode=int(pooling), indice_weights=None if c.weights is None else t(c.weights), output_dtype=int(out_ty),
        lxu_cache_weights=None, lxu_cache_locations=None, row_alignment=c.row_alignment,
        max_float8_D=c.max_d_of(O.FP8), fp8_exponent_bits=fp8[0], fp8_exponent_bias=fp8[1])
    return out.float().cpu().numpy()
