"""ctypes view of the C ABI in ``include/tbe_b200.h`` for callers holding torch tensors.

The torch operators go through the same entry points from C++; this module exists for
callers that need arguments the operator schema does not have (destination scatter,
column remap, error flag) and for tests that exercise the boundary directly.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .types import PoolingMode, SparseType

_vp, _i64, _i32 = C.c_void_p, C.c_int64, C.c_int32


class LookupArgs(C.Structure):
    """Mirror of ``tbe_b200_lookup_args`` (field order and types must match the header)."""
    _fields_ = [
        ("dev_weights", _vp), ("dev_weights_bytes", _i64), ("weights_offsets", _vp), ("weights_tys", _vp),
        ("D_offsets", _vp), ("T", _i32), ("B", _i64), ("total_D", _i64), ("max_D", _i32), ("indices", _vp),
        ("offsets", _vp), ("index_bits", _i32), ("num_indices", _i64), ("indice_weights", _vp),
        ("pooling_mode", _i32), ("output_dtype", _i32), ("row_alignment", _i32), ("fp8_exponent_bits", _i32),
        ("fp8_exponent_bias", _i32), ("output", _vp), ("output_stride", _i64), ("output_col_offsets", _vp),
        ("dest_outputs", _vp), ("rows_per_dest", _i64), ("error_flag", _vp),
    ]


EXPORTS = {
    "tbe_b200_int_nbit_lookup": (_i32, [C.POINTER(LookupArgs), _vp]),
    "tbe_b200_quantize_8bit_rowwise": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp]),
    "tbe_b200_dequantize_8bit_rowwise": (_i32, [_vp, _i64, _i64, _vp, _i32, _vp]),
    "tbe_b200_quantize_nbit_rowwise_sbhalf": (_i32, [_i32, _vp, _i64, _i64, _vp, _vp]),
    "tbe_b200_dequantize_nbit_rowwise_sbhalf": (_i32, [_i32, _vp, _i64, _i64, _vp, _vp]),
    "tbe_b200_pack_table_rows": (_i32, [_i32, _vp, _i64, _i64, _i64, _vp, _vp]),
    "tbe_b200_quantize_to_table_rows": (_i32, [_i32, _vp, _i64, _i64, _i64, _vp, _vp]),
    "tbe_b200_permute_pooled_embs": (_i32, [_vp, _i64, _i64, _i32, _i64, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "tbe_b200_permute_pooled_embs_blocked": (_i32, [_vp, _i64, _i64, _i32, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _vp,
                                                    _vp, _vp]),
    "tbe_b200_complete_cumsum_scratch_bytes": (_i64, [_i64]),
    "tbe_b200_complete_cumsum": (_i32, [_vp, _i64, _i32, _vp, _vp, _i64, _vp]),
    "tbe_b200_complete_cumsum_static_max_elements": (_i64, []),
    "tbe_b200_complete_cumsum_static": (_i32, [_vp, _i64, _i32, _vp, _vp]),
    "tbe_b200_permute_2d_sparse_scratch_bytes": (_i64, [_i64, _i64]),
    "tbe_b200_permute_2d_sparse_offsets": (_i32, [_vp, _i64, _vp, _i32, _i64, _i64, _vp, _vp, _i64, _vp, _vp]),
    "tbe_b200_permute_2d_sparse_copy": (_i32, [_vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _vp]),
    "tbe_b200_permute_2d_sparse_copy_to_dests": (_i32, [_vp, _i64, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _vp, _vp, _vp]),
    "tbe_b200_signal_peers": (_i32, [_vp, _i32, _i32, _i64, _vp]),
    "tbe_b200_wait_flags": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp]),
    "tbe_b200_last_error": (C.c_char_p, []),
    "tbe_b200_version": (_i32, []),
}

_lib = None


def lib():
    """The loaded ``libtbe_b200.so`` with argument types declared."""
    global _lib
    if _lib is None:
        from . import cabi_lib
        for name, (res, args) in EXPORTS.items():
            fn = getattr(cabi_lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = cabi_lib
    return _lib


def last_error() -> str:
    return lib().tbe_b200_last_error().decode()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (status {rc}): {last_error()}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_OUT_DTYPE = {torch.float32: SparseType.FP32, torch.float16: SparseType.FP16, torch.bfloat16: SparseType.BF16}


def lookup(dev_weights: torch.Tensor, weights_offsets: torch.Tensor, weights_tys: torch.Tensor,
           D_offsets: torch.Tensor, total_D: int, max_D: int, indices: torch.Tensor, offsets: torch.Tensor,
           pooling_mode: int, output: torch.Tensor, indice_weights: Optional[torch.Tensor] = None,
           row_alignment: int = 16, fp8_exponent_bits: int = 4, fp8_exponent_bias: int = 7,
           output_stride: Optional[int] = None, output_col_offsets: Optional[torch.Tensor] = None,
           dest_outputs: Optional[torch.Tensor] = None, rows_per_dest: int = 0,
           error_flag: Optional[torch.Tensor] = None, B: Optional[int] = None) -> torch.Tensor:
    """``tbe_b200_int_nbit_lookup`` on the current stream, writing into ``output``.

    ``dest_outputs`` is an int64 CUDA tensor of base addresses (one per ``rows_per_dest`` rows of
    the batch); ``output_col_offsets`` an int64 CUDA tensor [T].  All tensors must be contiguous
    and on the current device; nothing is copied or converted here.
    """
    T = weights_offsets.numel()
    assert weights_offsets.dtype == torch.int64 and weights_tys.dtype == torch.uint8 and D_offsets.dtype == torch.int32
    assert indices.dtype in (torch.int32, torch.int64) and offsets.dtype == indices.dtype
    a = LookupArgs()
    a.dev_weights = _ptr(dev_weights)
    a.dev_weights_bytes = dev_weights.numel()
    a.weights_offsets = _ptr(weights_offsets)
    a.weights_tys = _ptr(weights_tys)
    a.D_offsets = _ptr(D_offsets)
    a.T = T
    a.B = (offsets.numel() - 1) // T if B is None else B
    a.total_D = total_D
    a.max_D = max_D
    a.indices = _ptr(indices)
    a.offsets = _ptr(offsets)
    a.index_bits = 32 if indices.dtype == torch.int32 else 64
    a.num_indices = indices.numel()
    a.indice_weights = _ptr(indice_weights)
    a.pooling_mode = int(pooling_mode)
    a.output_dtype = int(_OUT_DTYPE[output.dtype])
    a.row_alignment = row_alignment
    a.fp8_exponent_bits = fp8_exponent_bits
    a.fp8_exponent_bias = fp8_exponent_bias
    a.output = _ptr(output)
    if output_stride is None:
        output_stride = max_D if int(pooling_mode) == int(PoolingMode.NONE) else total_D
    a.output_stride = output_stride
    a.output_col_offsets = _ptr(output_col_offsets)
    a.dest_outputs = _ptr(dest_outputs)
    a.rows_per_dest = rows_per_dest
    a.error_flag = _ptr(error_flag)
    check(lib().tbe_b200_int_nbit_lookup(C.byref(a), _stream()), "tbe_b200_int_nbit_lookup")
    return output


def permute_pooled_embs(pooled: torch.Tensor, offset_dim_list: torch.Tensor, permute_list: torch.Tensor,
                        inv_offset_dim_list: torch.Tensor, output: torch.Tensor,
                        error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    total_D = pooled.shape[-1]
    B = pooled.numel() // total_D
    check(lib().tbe_b200_permute_pooled_embs(_ptr(pooled), B, total_D, pooled.element_size(), pooled.stride(-2),
                                             output.stride(-2), _ptr(offset_dim_list), _ptr(permute_list),
                                             _ptr(inv_offset_dim_list), permute_list.numel(), _ptr(output),
                                             _ptr(error_flag), _stream()), "tbe_b200_permute_pooled_embs")
    return output


def quantize_to_table_rows(x: torch.Tensor, weight_ty: int, row_bytes_: int, rows_out: torch.Tensor) -> torch.Tensor:
    """fp32 [E, D] -> table rows written in place into ``rows_out`` (uint8, E*row_bytes bytes)."""
    assert x.dtype == torch.float32 and x.is_contiguous() and rows_out.dtype == torch.uint8
    assert rows_out.numel() >= x.shape[0] * row_bytes_
    check(lib().tbe_b200_quantize_to_table_rows(int(weight_ty), _ptr(x), x.shape[0], x.shape[1], row_bytes_,
                                                _ptr(rows_out), _stream()), "tbe_b200_quantize_to_table_rows")
    return rows_out


def permute_pooled_embs_blocked(blocks: torch.Tensor, offset_dim_list: torch.Tensor, permute_list: torch.Tensor,
                                inv_offset_dim_list: torch.Tensor, output: torch.Tensor,
                                error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``blocks`` is [nblocks, B, block_cols] (contiguous); the logical source is their concatenation along
    the columns, [B, nblocks * block_cols]; ``output`` is [B, nblocks * block_cols]."""
    nblk, B, bc = blocks.shape
    check(lib().tbe_b200_permute_pooled_embs_blocked(_ptr(blocks), B, nblk * bc, blocks.element_size(), bc, output.stride(0),
                                                     bc, B * bc, _ptr(offset_dim_list), _ptr(permute_list),
                                                     _ptr(inv_offset_dim_list), permute_list.numel(), _ptr(output),
                                                     _ptr(error_flag), _stream()), "tbe_b200_permute_pooled_embs_blocked")
    return output


def permute_2d_sparse_offsets(permute: torch.Tensor, lengths: torch.Tensor, scratch: torch.Tensor,
                              error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``tbe_b200_permute_2d_sparse_offsets`` on the current stream: returns ``lengths[permute]`` ([T_out, B]) and leaves
    the segment offsets in ``scratch`` (int64, at least ``permute_2d_sparse_scratch_elems(T_in, T_out)`` entries)."""
    assert permute.dtype == torch.int32 and lengths.dim() == 2 and lengths.is_contiguous() and scratch.dtype == torch.int64
    T_in, B = lengths.shape
    T_out = permute.numel()
    out = torch.empty((T_out, B), dtype=lengths.dtype, device=lengths.device)
    check(lib().tbe_b200_permute_2d_sparse_offsets(_ptr(permute), T_out, _ptr(lengths), 32 if lengths.dtype == torch.int32 else 64,
                                                   T_in, B, _ptr(out), _ptr(scratch), scratch.numel() * 8, _ptr(error_flag), _stream()),
          "tbe_b200_permute_2d_sparse_offsets")
    return out


def permute_2d_sparse_scratch_elems(T_in: int, T_out: int) -> int:
    return (lib().tbe_b200_permute_2d_sparse_scratch_bytes(T_in, T_out) + 7) // 8


def permute_2d_sparse_copy_to_dests(permute: torch.Tensor, T_in: int, values: torch.Tensor, dest_bases: torch.Tensor,
                                    tables_per_dest: int, dest_capacity: int, scratch: torch.Tensor,
                                    error_flag: Optional[torch.Tensor] = None) -> None:
    """``tbe_b200_permute_2d_sparse_copy_to_dests`` on the current stream; ``dest_bases`` is an int64 CUDA tensor of
    addresses (local or peer memory), ``scratch`` what :func:`permute_2d_sparse_offsets` left."""
    assert values.is_contiguous() and dest_bases.dtype == torch.int64
    vb = values.element_size() * (values.numel() // max(values.shape[0], 1) if values.dim() > 1 else 1)
    check(lib().tbe_b200_permute_2d_sparse_copy_to_dests(_ptr(permute), permute.numel(), T_in, _ptr(values), vb, _ptr(dest_bases),
                                                         tables_per_dest, dest_capacity, values.shape[0], _ptr(scratch), _ptr(error_flag),
                                                         _stream()), "tbe_b200_permute_2d_sparse_copy_to_dests")


def signal_peers(peer_flag_ptrs: torch.Tensor, world: int, rank: int, value: int) -> None:
    """``tbe_b200_signal_peers`` on the current stream; ``peer_flag_ptrs`` is an int64 CUDA tensor of ``world``
    addresses, one per rank, each of an int64 flag array of ``world`` entries in that rank's memory."""
    check(lib().tbe_b200_signal_peers(_ptr(peer_flag_ptrs), world, rank, value, _stream()), "tbe_b200_signal_peers")


def wait_flags(flags: torch.Tensor, world: int, value: int, max_polls: int, error_flag: Optional[torch.Tensor] = None) -> None:
    """``tbe_b200_wait_flags`` on the current stream: a bounded device-side wait for ``flags[r] >= value``."""
    assert flags.dtype == torch.int64 and flags.numel() >= world
    check(lib().tbe_b200_wait_flags(_ptr(flags), world, value, max_polls, _ptr(error_flag), _stream()), "tbe_b200_wait_flags")
