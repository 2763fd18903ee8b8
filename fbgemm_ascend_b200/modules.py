"""Host-side modules over the operators: the table container that drives the lookup and the
pooled-embedding permutation.

They mirror the two upstream modules the reference's tests drive the operators through:
``IntNBitTableBatchedEmbeddingBagsCodegen`` (attribute names as read by ``call_operator`` in
bench/tbe_inference/.../test_int_nbit_split_embedding_codegen_lookup_function.py:88-118) and
``PermutePooledEmbeddings``
(bench/pooled_embedding/permute_pooled_embs/permute_pooled_embedding_modules.py:94-142).
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import accumulate
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch

from . import cabi
from .types import PoolingMode, SparseType, row_bytes


@dataclass
class TableSpec:
    name: str
    num_embeddings: int
    embedding_dim: int
    weight_ty: SparseType


class IntNBitTableBatchedEmbeddingBags:
    """Quantized tables in one flat device buffer + the lookup over them.

    ``embedding_specs`` is a list of ``(name, E, D, SparseType)`` (a trailing location entry, as in
    the upstream spec tuples, is accepted and ignored: every table lives in device memory).
    Table ``t`` occupies ``weights_dev[weights_offsets[t] : weights_offsets[t] + E_t * row_bytes_t]``;
    rows are ``[fp16 scale][fp16 bias][payload]`` for INT8/INT4/INT2 and plain payload otherwise,
    padded to ``row_alignment`` bytes.
    """

    def __init__(self, embedding_specs: Sequence[Tuple], device: Union[str, torch.device] = "cuda",
                 pooling_mode: PoolingMode = PoolingMode.SUM, output_dtype: SparseType = SparseType.FP16,
                 indices_dtype: torch.dtype = torch.int32, row_alignment: int = 16,
                 fp8_exponent_bits: int = 4, fp8_exponent_bias: int = 7) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("IntNBitTableBatchedEmbeddingBags needs a CUDA device: there is no CPU path")
        self.specs = [TableSpec(s[0], int(s[1]), int(s[2]), SparseType(int(s[3]))) for s in embedding_specs]
        self.pooling_mode = PoolingMode(int(pooling_mode))
        self.output_dtype = int(output_dtype)
        self.indices_dtype = indices_dtype
        self.row_alignment = int(row_alignment)
        self.fp8_exponent_bits = fp8_exponent_bits
        self.fp8_exponent_bias = fp8_exponent_bias
        offs, cur = [], 0
        for s in self.specs:
            if s.embedding_dim % s.weight_ty.align_size() != 0:
                raise ValueError(f"table {s.name}: D={s.embedding_dim} must be a multiple of "
                                 f"{s.weight_ty.align_size()} for {s.weight_ty.name}")
            cur = (cur + 15) // 16 * 16
            offs.append(cur)
            cur += s.num_embeddings * row_bytes(s.weight_ty, s.embedding_dim, self.row_alignment)
        self.weights_dev = torch.zeros(max(cur, 1), dtype=torch.uint8, device=self.device)
        self.weights_uvm = torch.empty(0, dtype=torch.uint8, device=self.device)
        self.weights_placements = torch.zeros(len(self.specs), dtype=torch.int32, device=self.device)
        self.weights_offsets = torch.tensor(offs, dtype=torch.int64, device=self.device)
        self.weights_tys = torch.tensor([int(s.weight_ty) for s in self.specs], dtype=torch.uint8, device=self.device)
        dims = [s.embedding_dim for s in self.specs]
        self.D_offsets = torch.tensor([0] + list(accumulate(dims)), dtype=torch.int32, device=self.device)
        self.total_D = sum(dims)
        self.max_D = max(dims) if dims else 0
        self._host_offsets = offs

        def max_d(ty):
            return max([s.embedding_dim for s in self.specs if s.weight_ty == ty], default=0)

        self.max_int2_D = max_d(SparseType.INT2)
        self.max_int4_D = max_d(SparseType.INT4)
        self.max_int8_D = max_d(SparseType.INT8)
        self.max_float8_D = max_d(SparseType.FP8)
        self.max_float16_D = max_d(SparseType.FP16)
        self.max_float32_D = max_d(SparseType.FP32)

    # -- weights ---------------------------------------------------------------

    def table_row_bytes(self, t: int) -> int:
        s = self.specs[t]
        return row_bytes(s.weight_ty, s.embedding_dim, self.row_alignment)

    def table_rows(self, t: int) -> torch.Tensor:
        """uint8 view [E_t, row_bytes_t] of table ``t`` inside ``weights_dev``."""
        s, rb = self.specs[t], self.table_row_bytes(t)
        o = self._host_offsets[t]
        return self.weights_dev[o:o + s.num_embeddings * rb].view(s.num_embeddings, rb)

    def split_embedding_weights(self) -> List[Tuple[torch.Tensor, Optional[torch.Tensor]]]:
        return [(self.table_rows(t), None) for t in range(len(self.specs))]

    def assign_rows_from_float(self, t: int, x: torch.Tensor, row_start: int = 0) -> None:
        """Quantize fp32 ``x`` [n, D_t] into rows ``row_start .. row_start+n`` of table ``t``."""
        s = self.specs[t]
        if s.weight_ty in (SparseType.FP32, SparseType.FP8, SparseType.BF16):
            raise ValueError("assign_rows_from_float covers FP16 / INT8 / INT4 / INT2 tables")
        x = x.to(self.device, torch.float32).contiguous()
        rows = self.table_rows(t)[row_start:row_start + x.shape[0]]
        cabi.quantize_to_table_rows(x, int(s.weight_ty), self.table_row_bytes(t), rows)

    def fill_random_weights(self, make_rows: Optional[Callable[[int, int, int, torch.Generator], torch.Tensor]] = None,
                            seed: int = 0, chunk_rows: int = 1 << 20) -> None:
        """Fill every table.  ``make_rows(t, n, D, gen)`` returns fp32 [n, D] on the device; the
        default draws N(0, 0.05).  FP8 and FP32 tables get raw random payloads."""
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        for t, s in enumerate(self.specs):
            if s.weight_ty == SparseType.FP8:
                b = torch.randint(0, 256, (s.num_embeddings, s.embedding_dim), dtype=torch.uint8, device=self.device, generator=gen)
                b[(b & 0x7f) >= 0x78] = 0x3c   # keep clear of the top exponent
                self.table_rows(t)[:, :s.embedding_dim] = b
                continue
            for r0 in range(0, s.num_embeddings, chunk_rows):
                n = min(chunk_rows, s.num_embeddings - r0)
                x = make_rows(t, n, s.embedding_dim, gen) if make_rows else \
                    torch.randn(n, s.embedding_dim, device=self.device, generator=gen) * 0.05
                if s.weight_ty == SparseType.FP32:
                    self.table_rows(t)[r0:r0 + n, :4 * s.embedding_dim] = x.contiguous().view(torch.uint8).view(n, -1)
                else:
                    self.assign_rows_from_float(t, x, r0)

    # -- lookup ----------------------------------------------------------------

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor,
                per_sample_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        return torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function(
            dev_weights=self.weights_dev, uvm_weights=self.weights_uvm,
            weights_placements=self.weights_placements, weights_offsets=self.weights_offsets,
            weights_tys=self.weights_tys, D_offsets=self.D_offsets, total_D=self.total_D,
            max_int2_D=self.max_int2_D, max_int4_D=self.max_int4_D, max_int8_D=self.max_int8_D,
            max_float16_D=self.max_float16_D, max_float32_D=self.max_float32_D,
            indices=indices, offsets=offsets, pooling_mode=int(self.pooling_mode),
            indice_weights=per_sample_weights, output_dtype=self.output_dtype,
            lxu_cache_weights=None, lxu_cache_locations=None, row_alignment=self.row_alignment,
            max_float8_D=self.max_float8_D, fp8_exponent_bits=self.fp8_exponent_bits,
            fp8_exponent_bias=self.fp8_exponent_bias)

    __call__ = forward


class PermutePooledEmbeddings:
    """Permute pooled embeddings along the feature dimension: feature ``permute[i]`` moves to
    position ``i``.  Same constructor and call signature as the upstream module."""

    def __init__(self, embs_dims: List[int], permute: List[int], device: Optional[torch.device] = None) -> None:
        embs_dims = [int(d) for d in embs_dims]
        self._offset_dim_list = torch.tensor([0] + list(accumulate(embs_dims)), device=device, dtype=torch.int64)
        self._permute = torch.tensor(permute, device=device, dtype=torch.int64)
        inv_permute = [0] * len(permute)
        for i, p in enumerate(permute):
            inv_permute[p] = i
        self._inv_permute = torch.tensor(inv_permute, device=device, dtype=torch.int64)
        inv_embs_dims = [embs_dims[i] for i in permute]
        self._inv_offset_dim_list = torch.tensor([0] + list(accumulate(inv_embs_dims)), device=device, dtype=torch.int64)

    def __call__(self, pooled_embs: torch.Tensor) -> torch.Tensor:
        dev = pooled_embs.device
        return torch.ops.fbgemm.permute_pooled_embs_auto_grad(
            pooled_embs, self._offset_dim_list.to(device=dev), self._permute.to(device=dev),
            self._inv_offset_dim_list.to(device=dev), self._inv_permute.to(device=dev))
