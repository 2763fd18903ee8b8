"""CPU checkers for the quantized TBE inference path.  TEST INFRASTRUCTURE ONLY.

Two shared libraries are wrapped here with ctypes + numpy:

* ``port``  -- ``oracle/_build/libtbe_oracle.so``, the plain-C restatement
  (``tbe_oracle.c``);
* ``ref``   -- ``oracle/_ref/libfbgemm_cpu_ref.so``, a harness over the FBGEMM CPU
  kernels inside ``libtorch_cpu.so`` (``fbgemm_cpu_ref.cpp``), the library the
  reference's golden path (fbgemm_gpu's CPU operators) is built on.

Only ``tests/``, the smoke test and the benchmark's CPU-baseline leg import this
package.  The GPU package never does; it fails loudly without its CUDA library.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "_build", "libtbe_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libfbgemm_cpu_ref.so")

# SparseType / PoolingMode values: int_nbit_split_embedding_codegen_lookup_function.cpp:18-33
FP32, FP16, INT8, INT4, INT2, BF16, FP8 = 0, 1, 2, 3, 4, 5, 6
SUM, MEAN, NONE = 0, 1, 2

_c = ctypes
_vp, _i64, _i32 = _c.c_void_p, _c.c_int64, _c.c_int


def build(force: bool = False) -> None:
    """Compile both checkers with ``make`` (a few seconds)."""
    if force or not (os.path.exists(PORT_SO) and os.path.exists(REF_SO)):
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True,
                       stdout=subprocess.DEVNULL)


_libs = {}


def _lib(impl: str):
    if impl in _libs:
        return _libs[impl]
    build()
    if impl == "port":
        lib = _c.CDLL(PORT_SO)
        p = "orc_"
        lib.orc_tbe_lookup.restype = _i64
        lib.orc_tbe_lookup.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i32, _vp, _i32, _i32,
                                       _i64, _i32, _i32, _vp, _i64, _i64]
        lib.orc_permute_pooled_embs.restype = _i32
        lib.orc_permute_pooled_embs.argtypes = [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp]
        lib.orc_row_bytes.restype = _i64
        lib.orc_row_bytes.argtypes = [_i32, _i64, _i64]
        lib.orc_pack_int8_rows.restype = None
        lib.orc_pack_int8_rows.argtypes = [_vp, _i64, _i64, _i64, _vp]
        lib.orc_pack_nbit_rows.restype = None
        lib.orc_pack_nbit_rows.argtypes = [_vp, _i64, _i64, _i64, _vp]
        lib.orc_fp8_to_f32.restype = _c.c_float
        lib.orc_fp8_to_f32.argtypes = [_c.c_uint8, _i32, _i32]
        lib.orc_f32_to_f16.restype = _c.c_uint16
        lib.orc_f32_to_f16.argtypes = [_c.c_float]
        lib.orc_f32_to_bf16.restype = _c.c_uint16
        lib.orc_f32_to_bf16.argtypes = [_c.c_float]
        lib.orc_num_threads.restype = _i32
    elif impl == "ref":
        import torch  # noqa: F401  (makes libtorch_cpu.so resident before dlopen)

        lib = _c.CDLL(REF_SO)
        p = "fbr_"
        lib.fbr_tbe_lookup.restype = _i64
        lib.fbr_tbe_lookup.argtypes = [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i32, _vp, _i32,
                                       _i32, _i64, _i32, _i32, _vp, _i64]
        lib.fbr_num_threads.restype = _i32
    else:
        raise ValueError(impl)
    getattr(lib, p + "quantize_8bit_rowwise").restype = None
    getattr(lib, p + "quantize_8bit_rowwise").argtypes = [_vp, _i64, _i64, _vp]
    getattr(lib, p + "dequantize_8bit_rowwise").restype = None
    getattr(lib, p + "dequantize_8bit_rowwise").argtypes = [_vp, _i64, _i64, _vp]
    getattr(lib, p + "quantize_nbit_rowwise_sbhalf").restype = None
    getattr(lib, p + "quantize_nbit_rowwise_sbhalf").argtypes = [_i32, _vp, _i64, _i64, _vp]
    getattr(lib, p + "dequantize_nbit_rowwise_sbhalf").restype = None
    getattr(lib, p + "dequantize_nbit_rowwise_sbhalf").argtypes = [_i32, _vp, _i64, _i64, _vp]
    _libs[impl] = lib
    return lib


def _fn(impl: str, name: str):
    return getattr(_lib(impl), ("orc_" if impl == "port" else "fbr_") + name)


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(_vp)


def num_threads(impl: str = "port") -> int:
    return int(_fn(impl, "num_threads")())


# ---- quantizers -------------------------------------------------------------

def quantize_8bit_rowwise(x: np.ndarray, impl: str = "port") -> np.ndarray:
    """fp32 [N, D] -> uint8 [N, D + 8] (codes, fp32 scale, fp32 bias)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, d = x.shape
    out = np.empty((n, d + 8), dtype=np.uint8)
    _fn(impl, "quantize_8bit_rowwise")(_ptr(x), n, d, _ptr(out))
    return out


def dequantize_8bit_rowwise(q: np.ndarray, impl: str = "port") -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    n, dq = q.shape
    out = np.empty((n, dq - 8), dtype=np.float32)
    _fn(impl, "dequantize_8bit_rowwise")(_ptr(q), n, dq, _ptr(out))
    return out


def quantize_nbit_rowwise_sbhalf(x: np.ndarray, bit_rate: int, impl: str = "port") -> np.ndarray:
    """fp32 [N, D] -> uint8 [N, D*bit_rate/8 + 4] (codes, fp16 scale, fp16 bias)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, d = x.shape
    per = 8 // bit_rate
    out = np.empty((n, (d + per - 1) // per + 4), dtype=np.uint8)
    _fn(impl, "quantize_nbit_rowwise_sbhalf")(bit_rate, _ptr(x), n, d, _ptr(out))
    return out


def dequantize_nbit_rowwise_sbhalf(q: np.ndarray, bit_rate: int, impl: str = "port") -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    n, dq = q.shape
    out = np.empty((n, (dq - 4) * (8 // bit_rate)), dtype=np.float32)
    _fn(impl, "dequantize_nbit_rowwise_sbhalf")(bit_rate, _ptr(q), n, dq, _ptr(out))
    return out


# ---- table construction -----------------------------------------------------

def row_bytes(ty: int, D: int, row_alignment: int = 16) -> int:
    return int(_lib("port").orc_row_bytes(ty, D, row_alignment))


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def pack_table(x: np.ndarray, ty: int, row_alignment: int = 16, impl: str = "port") -> np.ndarray:
    """fp32 [E, D] -> TBE rows uint8 [E, row_bytes] of weight type ``ty``.

    INT8: FloatToFused8BitRowwiseQuantized, then scale/bias fp32 -> fp16 (RNE) moved to
    the front of the row.  INT4/INT2: the SBHalf quantizer's row with its fp16 scale/bias
    moved to the front.  FP16/FP32: a cast.  FP8: ``x`` must already be uint8 codes.
    """
    e, d = x.shape
    rb = row_bytes(ty, d, row_alignment)
    rows = np.zeros((e, rb), dtype=np.uint8)
    lib = _lib("port")
    if ty == INT8:
        fused = quantize_8bit_rowwise(x, impl)
        lib.orc_pack_int8_rows(_ptr(fused), e, d, rb, _ptr(rows))
    elif ty in (INT4, INT2):
        bits = 4 if ty == INT4 else 2
        fused = quantize_nbit_rowwise_sbhalf(x, bits, impl)
        lib.orc_pack_nbit_rows(_ptr(fused), e, fused.shape[1] - 4, rb, _ptr(rows))
    elif ty == FP16:
        rows[:, : 2 * d] = np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint8).reshape(e, 2 * d)
    elif ty == FP32:
        rows[:, : 4 * d] = np.ascontiguousarray(x, dtype=np.float32).view(np.uint8).reshape(e, 4 * d)
    elif ty == FP8:
        assert x.dtype == np.uint8
        rows[:, :d] = x
    else:
        raise ValueError(f"weight type {ty}")
    return rows


def concat_tables(tables: Sequence[np.ndarray], tys: Sequence[int], Ds: Sequence[int],
                  table_alignment: int = 16) -> Tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """Row blocks -> (dev_weights uint8, weights_offsets int64, weights_tys uint8, D_offsets int32)."""
    offs, cur = [], 0
    for t in tables:
        cur = (cur + table_alignment - 1) // table_alignment * table_alignment
        offs.append(cur)
        cur += t.size
    dev = np.zeros(max(cur, 1), dtype=np.uint8)
    for t, o in zip(tables, offs):
        dev[o:o + t.size] = t.reshape(-1)
    d_offsets = np.zeros(len(Ds) + 1, dtype=np.int32)
    d_offsets[1:] = np.cumsum(Ds)
    return dev, np.asarray(offs, dtype=np.int64), np.asarray(tys, dtype=np.uint8), d_offsets


# ---- lookup / permute -------------------------------------------------------

_OUT_NP = {FP32: np.float32, FP16: np.float16, BF16: np.uint16}


def tbe_lookup(dev_weights: np.ndarray, weights_offsets: np.ndarray, weights_tys: np.ndarray,
               D_offsets: np.ndarray, indices: np.ndarray, offsets: np.ndarray, pooling_mode: int = SUM,
               indice_weights: Optional[np.ndarray] = None, output_dtype: int = FP16, row_alignment: int = 16,
               fp8_exponent_bits: int = 4, fp8_exponent_bias: int = 7, impl: str = "port") -> np.ndarray:
    """CPU result of int_nbit_split_embedding_codegen_lookup_function.

    Returns [B, total_D] (pooled) or [N, max_D] (pooling NONE) in fp32 / fp16; bf16 output
    is returned as its uint16 bit pattern.
    """
    dev_weights = np.ascontiguousarray(dev_weights, dtype=np.uint8)
    weights_offsets = np.ascontiguousarray(weights_offsets, dtype=np.int64)
    weights_tys = np.ascontiguousarray(weights_tys, dtype=np.uint8)
    D_offsets = np.ascontiguousarray(D_offsets, dtype=np.int32)
    assert indices.dtype in (np.int32, np.int64)
    indices = np.ascontiguousarray(indices)
    offsets = np.ascontiguousarray(offsets.astype(indices.dtype))
    bits = 32 if indices.dtype == np.int32 else 64
    T = weights_offsets.size
    B = (offsets.size - 1) // T
    total_D = int(D_offsets[-1])
    max_D = int(np.max(np.diff(D_offsets))) if T else 0
    w = None if indice_weights is None else np.ascontiguousarray(indice_weights, dtype=np.float32)
    if pooling_mode == NONE:
        out = np.zeros((indices.size, max_D), dtype=_OUT_NP[output_dtype])
        stride = max_D
    else:
        out = np.zeros((B, total_D), dtype=_OUT_NP[output_dtype])
        stride = total_D
    if impl == "port":
        rc = _lib("port").orc_tbe_lookup(_ptr(dev_weights), _ptr(weights_offsets), _ptr(weights_tys),
                                         _ptr(D_offsets), T, B, total_D, _ptr(indices), _ptr(offsets), bits,
                                         _ptr(w), pooling_mode, output_dtype, row_alignment, fp8_exponent_bits,
                                         fp8_exponent_bias, _ptr(out), stride, max_D)
    else:
        rc = _lib("ref").fbr_tbe_lookup(_ptr(dev_weights), dev_weights.size, _ptr(weights_offsets),
                                        _ptr(weights_tys), _ptr(D_offsets), T, B, total_D, _ptr(indices),
                                        _ptr(offsets), bits, _ptr(w), pooling_mode, output_dtype, row_alignment,
                                        fp8_exponent_bits, fp8_exponent_bias, _ptr(out), stride)
    if rc != 0:
        raise RuntimeError(f"oracle lookup ({impl}) rejected its input: status {rc}")
    return out


def permute_pooled_embs(pooled: np.ndarray, offset_dim_list: np.ndarray, permute_list: np.ndarray,
                        inv_offset_dim_list: np.ndarray) -> np.ndarray:
    pooled = np.ascontiguousarray(pooled)
    B = int(np.prod(pooled.shape[:-1]))
    total_D = pooled.shape[-1]
    out = np.empty_like(pooled)
    o = np.ascontiguousarray(offset_dim_list, dtype=np.int64)
    p = np.ascontiguousarray(permute_list, dtype=np.int64)
    io = np.ascontiguousarray(inv_offset_dim_list, dtype=np.int64)
    rc = _lib("port").orc_permute_pooled_embs(_ptr(pooled), B, total_D, pooled.dtype.itemsize, _ptr(o), _ptr(p),
                                              _ptr(io), p.size, _ptr(out))
    if rc != 0:
        raise RuntimeError("permute_list must be a permutation of 0..T-1")
    return out


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def complete_cumsum(x: np.ndarray) -> np.ndarray:
    """out[0] = 0, out[i + 1] = x[0] + ... + x[i], in x's integer type (sums wrap like the type does).

    Restates what the reference's tests expect of ``asynchronous_complete_cumsum``
    (bench/sparse/asynchronous_complete_cumsum_test/test_asynchronous_complete_cumsum.py:39-48: the
    operator against the CPU operator of the same name, i.e. a zero followed by the running sums).
    """
    x = np.ascontiguousarray(x)
    out = np.zeros(x.size + 1, dtype=x.dtype)
    np.cumsum(x, out=out[1:], dtype=x.dtype)
    return out


def permute_2d_sparse_data(permute: np.ndarray, lengths: np.ndarray, values: np.ndarray,
                           weights: Optional[np.ndarray] = None):
    """(lengths[permute], value segments of the tables permute[0], permute[1], ..., weights alike).

    Restates ``permute_2d_sparse_data_reference``, the CPU model the reference's own test checks the
    operator against (bench/sparse/permute_sparse_data/test_permute2d_sparse_data.py:41-72): table t
    owns ``sum(lengths[t, :])`` consecutive entries of ``values``; entries of ``permute`` may repeat and
    ``len(permute)`` need not equal ``lengths.shape[0]``; 1-D or 2-D weights are cut along dim 0.
    With an empty dimension the inputs come back unchanged (same test, :48-53).
    """
    lengths = np.ascontiguousarray(lengths)
    values = np.ascontiguousarray(values)
    if lengths.shape[0] == 0 or lengths.shape[1] == 0 or permute.size == 0:
        return lengths.copy(), values.copy(), None if weights is None else weights.copy()
    seg = lengths.astype(np.int64).sum(axis=1)
    off = np.zeros(seg.size + 1, dtype=np.int64)
    off[1:] = np.cumsum(seg)
    rows = [int(r) for r in permute]
    out_v = np.concatenate([values[off[r]:off[r + 1]] for r in rows]) if rows else values[:0]
    out_w = None
    if weights is not None:
        out_w = np.concatenate([weights[off[r]:off[r + 1]] for r in rows], axis=0)
    return lengths[np.asarray(rows, dtype=np.int64)], out_v, out_w
