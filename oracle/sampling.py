"""Checks of a GPU lookup at sizes whose tables do not fit the host.  TEST INFRASTRUCTURE ONLY.

A lookup over tens of gigabytes of table rows cannot be repeated on the CPU in full, so a sample of
(table, bag) pairs is checked instead: the rows those bags reference are copied to the host, the
indices are renumbered onto that compact set of rows, the CPU oracle pools the compact case, and the
result is compared with the corresponding slices of the GPU output.  The sample always contains the
longest bags of the batch, because the error of fp32 accumulation (and of the folded INT8 form) grows
with the bag length.  The tolerances are the ones the reference's test uses
(test_int_nbit_split_embedding_codegen_lookup_function.py:358-363).

Used by ``tests/`` and by the benchmark's verification step; never by the GPU package.
"""
from __future__ import annotations

from typing import Dict

import numpy as np

from . import BF16, FP16, FP32, bf16_bits_to_f32, tbe_lookup

TOL = {FP16: 1e-3, BF16: 2.0 ** -7, FP32: 1e-4}


def check_sampled_bags(tables, indices, offsets, weights, out, n_samples: int = 4096, n_longest: int = 512,
                       seed: int = 0, impl: str = "ref") -> Dict[str, object]:
    """Compare ``out`` (the GPU result of ``tables.forward(indices, offsets, weights)``) with the CPU
    oracle on ``n_samples`` sampled bags.  ``tables`` is the GPU table container (``specs``,
    ``table_rows(t)``, ``D_offsets``, ``pooling_mode``, ``output_dtype``, ``row_alignment``).

    Returns {"ok", "bags", "rows", "max_len", "max_err", "bad"}."""
    import torch

    T = len(tables.specs)
    offs = offsets.detach().cpu().numpy().astype(np.int64)
    B = (offs.size - 1) // T
    lengths = np.diff(offs)
    rng = np.random.default_rng(seed)
    nbags = T * B
    n_samples = min(n_samples, nbags)
    n_longest = min(n_longest, n_samples)
    longest = np.argpartition(lengths, nbags - n_longest)[nbags - n_longest:] if n_longest > 0 else np.zeros(0, np.int64)
    others = rng.choice(nbags, size=n_samples, replace=False)
    sample = np.unique(np.concatenate([longest, others]))      # sorted, so a table's bags are contiguous
    samp_len = lengths[sample]
    # positions of all sampled rows in `indices`, one device gather for the whole sample
    starts = offs[sample]
    total = int(samp_len.sum())
    seg_off = np.zeros(sample.size + 1, dtype=np.int64)
    np.cumsum(samp_len, out=seg_off[1:])
    pos = np.repeat(starts - seg_off[:-1], samp_len) + np.arange(total, dtype=np.int64)
    dev = indices.device
    pos_t = torch.from_numpy(pos).to(dev)
    idx_h = indices.index_select(0, pos_t).cpu().numpy().astype(np.int64) if total else np.zeros(0, np.int64)
    w_h = weights.index_select(0, pos_t).cpu().numpy() if (weights is not None and total) else None
    d_off = tables.D_offsets.cpu().numpy()
    out_ty = int(tables.output_dtype)
    tol = TOL[out_ty]
    tab_of = sample // B
    max_err, bad, rows_checked = 0.0, 0, 0
    for t in np.unique(tab_of):
        sel = np.nonzero(tab_of == t)[0]
        bags = sample[sel] - t * B
        lens = samp_len[sel]
        lo, hi = seg_off[sel[0]], seg_off[sel[-1] + 1]            # the sample is sorted, so a table's rows are contiguous
        idx = idx_h[lo:hi]
        valid = idx >= 0
        uniq, inv = np.unique(idx[valid], return_inverse=True)
        compact = np.full(idx.shape, -1, dtype=np.int64)
        compact[valid] = inv
        if uniq.size:
            rows = tables.table_rows(int(t)).index_select(0, torch.from_numpy(uniq).to(dev)).cpu().numpy()
        else:
            rows = np.zeros((1, tables.table_row_bytes(int(t))), dtype=np.uint8)
        spec = tables.specs[int(t)]
        c_off = np.zeros(lens.size + 1, dtype=np.int64)
        np.cumsum(lens, out=c_off[1:])
        want = tbe_lookup(rows.reshape(-1), np.zeros(1, np.int64), np.array([int(spec.weight_ty)], np.uint8),
                          np.array([0, spec.embedding_dim], np.int32), compact, c_off, int(tables.pooling_mode),
                          None if w_h is None else w_h[lo:hi], out_ty, tables.row_alignment,
                          tables.fp8_exponent_bits, tables.fp8_exponent_bias, impl=impl)
        want = bf16_bits_to_f32(want) if out_ty == BF16 else want.astype(np.float32)
        got = out[torch.from_numpy(bags).to(dev), int(d_off[t]):int(d_off[t + 1])].float().cpu().numpy()
        err = np.abs(got - want)
        bad += int((err > tol + tol * np.abs(want)).sum()) + int((~np.isfinite(got)).sum())
        max_err = max(max_err, float(err.max()) if err.size else 0.0)
        rows_checked += int(idx.size)
    return {"ok": bad == 0, "bags": int(sample.size), "rows": rows_checked, "max_len": int(samp_len.max()) if sample.size else 0,
            "max_err": max_err, "bad": bad, "tolerance": tol}
