"""B200 (sm_100a) implementation of fbgemm-ascend's quantized TBE inference path.

Importing this package loads two in-tree shared libraries

* ``lib/libtbe_b200.so`` -- the CUDA kernels behind a C ABI (``include/tbe_b200.h``);
* ``lib/libtbe_b200_torch.so`` -- the ``torch.ops.fbgemm.*`` registrations
  (``int_nbit_split_embedding_codegen_lookup_function``,
  ``FloatToFused8BitRowwiseQuantized`` / ``Fused8BitRowwiseQuantizedToFloat``,
  ``permute_pooled_embs`` and relatives) for the CUDA dispatch key,

which is what ``import fbgemm_ascend`` does for the reference through chip detection
and ``torch.ops.load_library`` (fbgemm_ascend/__init__.py:189-231).  There is one
architecture and no CPU fallback: a missing library is an ImportError.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .types import PoolingMode, SparseType  # noqa: F401

_PKG = os.path.dirname(os.path.abspath(__file__))
CABI_LIB_PATH = os.path.join(_PKG, "lib", "libtbe_b200.so")
TORCH_LIB_PATH = os.path.join(_PKG, "lib", "libtbe_b200_torch.so")


def _load():
    for path in (CABI_LIB_PATH, TORCH_LIB_PATH):
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build the CUDA libraries first with "
                "`python -m fbgemm_ascend_b200.build` (needs nvcc; sm_100a only). "
                "This package has no CPU or PyTorch fallback.")
    cabi = ctypes.CDLL(CABI_LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(TORCH_LIB_PATH)
    return cabi


cabi_lib = _load()

from . import cabi  # noqa: E402,F401
from .modules import IntNBitTableBatchedEmbeddingBags, PermutePooledEmbeddings, TableSpec  # noqa: E402,F401

__all__ = ["PoolingMode", "SparseType", "cabi", "cabi_lib", "IntNBitTableBatchedEmbeddingBags",
           "PermutePooledEmbeddings", "TableSpec", "CABI_LIB_PATH", "TORCH_LIB_PATH"]
