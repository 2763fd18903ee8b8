"""Host-side logic that needs no GPU: row geometry, the permutation module's lists, workload
accounting."""
import inspect

import pytest
import torch

import oracle as O


def test_row_bytes_matches_oracle():
    from fbgemm_ascend_b200.types import SparseType, row_bytes
    for ty in (O.FP32, O.FP16, O.INT8, O.INT4, O.INT2, O.FP8):
        for D in (4, 16, 36, 64, 128, 256, 1000, 4096):
            if D % SparseType(ty).align_size():
                continue
            for al in (1, 4, 16, 32):
                assert row_bytes(ty, D, al) == O.row_bytes(ty, D, al)
    assert row_bytes(O.INT8, 128) == 144 and row_bytes(O.INT4, 128) == 80 and row_bytes(O.INT4, 64) == 48
    assert row_bytes(O.FP16, 128) == 256 and row_bytes(O.INT8, 128, 1) == 132


def test_permute_module_lists_and_signature():
    from fbgemm_ascend_b200 import PermutePooledEmbeddings
    m = PermutePooledEmbeddings([2, 3, 1, 4], [3, 0, 2, 1])
    assert m._offset_dim_list.tolist() == [0, 2, 5, 6, 10]
    assert m._inv_offset_dim_list.tolist() == [0, 4, 6, 7, 10]
    assert m._inv_permute.tolist() == [1, 3, 2, 0]
    # the reference pins this API (bench/pooled_embedding/permute_pooled_embs/common.py:30-36)
    assert inspect.getfullargspec(PermutePooledEmbeddings.__init__).args == ["self", "embs_dims", "permute", "device"]
    assert inspect.getfullargspec(PermutePooledEmbeddings.__call__).args == ["self", "pooled_embs"]


def test_table_module_needs_cuda():
    from fbgemm_ascend_b200 import IntNBitTableBatchedEmbeddingBags, SparseType
    with pytest.raises(RuntimeError, match="no CPU path"):
        IntNBitTableBatchedEmbeddingBags([("t", 10, 16, SparseType.INT8)], device="cpu")


def test_workload_specs_and_bytes():
    from fbgemm_ascend_b200 import workloads as W
    c2 = W.spec("c2")
    assert (c2.T, c2.E, c2.B, c2.dims[0]) == (26, 1_000_000, 2048, 128) and c2.index_dtype == torch.int64
    assert W.table_bytes(c2) == 26 * 1_000_000 * 144
    c3 = W.spec("c3")
    assert sum(c3.dims) == 9472 and W.table_bytes(c3) == 10_000_000 * (22 * 48 + 21 * 80 + 21 * 144)
    c4 = W.spec("c4")
    assert W.table_bytes(c4) == 64 * 12_000_000 * 144
    b = W.Batch(torch.zeros(1000, dtype=torch.int64), torch.zeros(26 * 2048 + 1, dtype=torch.int64), None, [1000] + [0] * 25)
    ab = W.algorithmic_bytes(c2, b)
    assert ab["algorithmic"] == 1000 * 132 + 1000 * 8 + (26 * 2048 + 1) * 8 + 2048 * 3328 * 2
    assert ab["padded"] - ab["algorithmic"] == 1000 * 12
    assert ab["sector"] - ab["algorithmic"] == 1000 * 28     # a 144-byte-stride row touches five 32-byte sectors
