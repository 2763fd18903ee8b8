"""The C-ABI library loads without a GPU and exports every symbol include/tbe_b200.h declares.
No compute call is made here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tbe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tbe_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from fbgemm_ascend_b200 import CABI_LIB_PATH, cabi
    lib = ctypes.CDLL(CABI_LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tbe_b200.h but not exported"
        assert n in cabi.EXPORTS, f"{n} has no ctypes signature in cabi.EXPORTS"
    assert set(cabi.EXPORTS) == set(names)
    assert cabi.lib().tbe_b200_version() >= 100
    assert cabi.last_error() == ""


def test_struct_layout_matches_header():
    """Field order of the ctypes mirror equals the header's struct."""
    from fbgemm_ascend_b200 import cabi
    text = open(os.path.join(ROOT, "include", "tbe_b200.h")).read()
    body = re.search(r"typedef struct \{(.*?)\} tbe_b200_lookup_args;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"([A-Za-z_0-9]+)\s*;", body)
    assert fields == [f[0] for f in cabi.LookupArgs._fields_]


def test_argument_validation_without_gpu():
    """Host-side argument checks return a status and a message before any CUDA call."""
    from fbgemm_ascend_b200 import cabi
    lib = cabi.lib()
    assert lib.tbe_b200_int_nbit_lookup(None, None) == -1
    assert "NULL" in cabi.last_error()
    a = cabi.LookupArgs()
    a.T = 0
    assert lib.tbe_b200_int_nbit_lookup(ctypes.byref(a), None) == -1
    assert "T must be positive" in cabi.last_error()
    assert lib.tbe_b200_permute_pooled_embs(None, 4, 4, 3, 4, 4, None, None, None, 1, None, None, None) == -2
    assert "elem_bytes" in cabi.last_error()
    assert lib.tbe_b200_quantize_nbit_rowwise_sbhalf(3, None, 0, 0, None, None) == -2
    assert lib.tbe_b200_quantize_to_table_rows(6, None, 0, 0, 0, None, None) == -2
    # producers of the lookup's inputs and the step flags
    assert lib.tbe_b200_complete_cumsum(None, -1, 64, None, None, 0, None) == -1
    assert lib.tbe_b200_complete_cumsum(None, 4, 16, None, None, 0, None) == -1 and "index_bits" in cabi.last_error()
    assert lib.tbe_b200_complete_cumsum_scratch_bytes(8192) == 0 and lib.tbe_b200_complete_cumsum_scratch_bytes(8193) == 16 + 2 * 16
    assert lib.tbe_b200_permute_2d_sparse_copy_to_dests(None, 6, 6, None, 8, None, 4, 10, 10, None, None, None) == -1
    assert "multiple of tables_per_dest" in cabi.last_error()
    assert lib.tbe_b200_permute_2d_sparse_copy_to_dests(None, 6, 6, None, 8, None, 3, 10, 10, None, None, None) == -1
    assert "NULL" in cabi.last_error()
    assert lib.tbe_b200_wait_flags(None, 2, 1, 0, None, None) != 0


def test_operators_registered_and_cpu_tensors_rejected():
    import pytest
    import torch
    import fbgemm_ascend_b200  # noqa: F401
    for name in ("int_nbit_split_embedding_codegen_lookup_function", "FloatToFused8BitRowwiseQuantized",
                 "Fused8BitRowwiseQuantizedToFloat", "permute_pooled_embs", "permute_pooled_embs_auto_grad",
                 "FloatToFusedNBitRowwiseQuantizedSBHalf", "FusedNBitRowwiseQuantizedSBHalfToFloat"):
        assert hasattr(torch.ops.fbgemm, name)
    assert hasattr(torch.ops.mxrec, "permute_pooled_embs")
    # there is no CPU implementation to fall back to
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.fbgemm.FloatToFused8BitRowwiseQuantized(torch.zeros(2, 4))
    with pytest.raises((RuntimeError, NotImplementedError)):
        z = torch.zeros(2, dtype=torch.int64)
        torch.ops.fbgemm.permute_pooled_embs(torch.zeros(2, 4), z, z, z, z)
    schema = torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function.default._schema
    assert [a.name for a in schema.arguments] == [
        "dev_weights", "uvm_weights", "weights_placements", "weights_offsets", "weights_tys", "D_offsets", "total_D",
        "max_int2_D", "max_int4_D", "max_int8_D", "max_float16_D", "max_float32_D", "indices", "offsets", "pooling_mode",
        "indice_weights", "output_dtype", "lxu_cache_weights", "lxu_cache_locations", "row_alignment", "max_float8_D",
        "fp8_exponent_bits", "fp8_exponent_bias"]
