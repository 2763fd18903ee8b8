"""Table-wise sharded pooled lookup across the GPUs of one box.

The reference has no multi-device code; this module composes its single-device operators the way
a table-wise sharded server does (benchmark configuration 4):

  1. every rank owns whole tables (global table ``r + world * j`` lives on rank ``r``) and pools its
     tables for the GLOBAL batch                          -> ``[B_global, sum(D_local)]``
  2. the pooled rows are exchanged so that rank ``s`` ends up with rows ``[s * B/world, (s+1) * B/world)``
     of every rank's result                                -> ``world`` blocks ``[B/world, sum(D_r)]``
  3. the blocks are put into feature order by ``permute_pooled_embs``  -> ``[B/world, sum(D_all)]``

Two data paths produce identical bytes:

``exchange="nccl"``   lookup kernel, then ``all_to_all_single`` into a local receive buffer, then the
                      blocked permute kernel reading that buffer (no concatenation pass);
``exchange="direct"`` one lookup kernel per rank whose epilogue stores every pooled segment straight
                      into the destination rank's output buffer at its final (permuted) column, over
                      NVLink peer memory; a barrier replaces the exchange and no permute pass is left.

Peer buffers come from ``torch.distributed._symmetric_memory`` (plain peer mappings; no multicast).
Everything that can be tested without a GPU -- ownership, column maps, permute lists, split sizes --
is in :class:`ShardPlan`; the operators themselves are injectable so the plumbing also runs on CPU
ranks (gloo) in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import accumulate
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class ShardPlan:
    """Who owns which table and where every pooled segment ends up."""
    world: int
    rank: int
    dims: List[int]                 # D of every global table
    feature_order: List[int]        # output position k holds global table feature_order[k]
    global_batch: int

    def __post_init__(self) -> None:
        T = len(self.dims)
        if sorted(self.feature_order) != list(range(T)):
            raise ValueError("feature_order must be a permutation of the global table ids")
        if self.global_batch % self.world != 0:
            raise ValueError(f"global batch {self.global_batch} must be divisible by the world size {self.world}")
        if not (0 <= self.rank < self.world):
            raise ValueError("rank out of range")

    # -- ownership -------------------------------------------------------------
    def tables_of(self, r: int) -> List[int]:
        """Global ids of the tables rank ``r`` owns (round-robin)."""
        return list(range(r, len(self.dims), self.world))

    @property
    def local_tables(self) -> List[int]:
        return self.tables_of(self.rank)

    @property
    def local_batch(self) -> int:
        return self.global_batch // self.world

    @property
    def total_D(self) -> int:
        return sum(self.dims)

    def width_of(self, r: int) -> int:
        return sum(self.dims[t] for t in self.tables_of(r))

    # -- layouts ---------------------------------------------------------------
    @property
    def exchanged_order(self) -> List[int]:
        """Global table ids in the order the exchange leaves them: rank-major, then owner-local."""
        return [t for r in range(self.world) for t in self.tables_of(r)]

    def permute_lists(self):
        """(offset_dim_list, permute_list, inv_offset_dim_list, inv_permute_list) taking the exchanged
        layout to feature order, as ``permute_pooled_embs`` wants them."""
        ex = self.exchanged_order
        pos = {t: i for i, t in enumerate(ex)}
        ex_dims = [self.dims[t] for t in ex]
        permute = [pos[t] for t in self.feature_order]
        inv_permute = [0] * len(permute)
        for i, q in enumerate(permute):
            inv_permute[q] = i
        offset = [0] + list(accumulate(ex_dims))
        inv_offset = [0] + list(accumulate(ex_dims[q] for q in permute))
        return offset, permute, inv_offset, inv_permute

    def final_col_of(self, t: int) -> int:
        """First output column of global table ``t`` in feature order."""
        col = 0
        for u in self.feature_order:
            if u == t:
                return col
            col += self.dims[u]
        raise KeyError(t)

    def local_final_cols(self) -> List[int]:
        return [self.final_col_of(t) for t in self.local_tables]

    def equal_widths(self) -> bool:
        return len({self.width_of(r) for r in range(self.world)}) == 1


class TableWiseShardedLookup:
    """Lookup -> exchange -> permute for the tables of one rank.

    ``lookup_fn(indices, offsets, weights) -> [B_global, width_local]`` pools the local tables;
    by default it is ``tables.forward``.  ``group`` is the process group of the box.
    """

    def __init__(self, plan: ShardPlan, tables=None, group=None, exchange: str = "nccl",
                 lookup_fn: Optional[Callable] = None, permute_fn: Optional[Callable] = None,
                 device: Optional[torch.device] = None, out_dtype: torch.dtype = torch.float16) -> None:
        if exchange not in ("nccl", "direct"):
            raise ValueError("exchange must be 'nccl' or 'direct'")
        self.plan = plan
        self.tables = tables
        self.group = group
        self.exchange = exchange
        self.device = device if device is not None else (tables.device if tables is not None else torch.device("cpu"))
        self.out_dtype = out_dtype
        self.lookup_fn = lookup_fn or (lambda i, o, w: tables.forward(i, o, w))
        self.permute_fn = permute_fn
        off, perm, inv_off, inv_perm = plan.permute_lists()
        t = lambda v: torch.tensor(v, dtype=torch.int64, device=self.device)
        self.offset_dim_list, self.permute_list = t(off), t(perm)
        self.inv_offset_dim_list, self.inv_permute_list = t(inv_off), t(inv_perm)
        if not plan.equal_widths():
            raise ValueError("every rank must hold the same pooled width (same sum of D) for the exchange")
        self._recv = None
        self._out = None
        self._symm = None
        if exchange == "direct":
            self._setup_direct()

    # -- NCCL path -------------------------------------------------------------
    def _buffers(self):
        p = self.plan
        if self._recv is None:
            self._recv = torch.empty((p.world, p.local_batch, p.width_of(p.rank)), dtype=self.out_dtype, device=self.device)
            self._out = torch.empty((p.local_batch, p.total_D), dtype=self.out_dtype, device=self.device)
        return self._recv, self._out

    def forward_nccl(self, indices, offsets, weights=None) -> torch.Tensor:
        p = self.plan
        pooled = self.lookup_fn(indices, offsets, weights)               # [B_global, width]
        recv, out = self._buffers()
        if p.world == 1:
            recv = pooled.view(1, p.local_batch, -1)
        else:
            # block s of `pooled` (rows of rank s) goes to rank s; block r of `recv` comes from rank r
            dist.all_to_all_single(recv.view(-1), pooled.view(-1), group=self.group)
        if self.permute_fn is not None:
            return self.permute_fn(recv, self.offset_dim_list, self.permute_list, self.inv_offset_dim_list, out)
        from . import cabi
        return cabi.permute_pooled_embs_blocked(recv, self.offset_dim_list, self.permute_list, self.inv_offset_dim_list, out)

    # -- direct peer-store path --------------------------------------------------
    def _setup_direct(self) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        p = self.plan
        # one output buffer per rank, mapped into every peer; double-buffered so a rank may start writing
        # step n+1 while a slow peer still reads step n
        self._symm = symm_mem.empty((2, p.local_batch, p.total_D), dtype=self.out_dtype, device=self.device)
        self._hdl = symm_mem.rendezvous(self._symm, self.group.group_name if self.group is not None else dist.group.WORLD.group_name)
        ptrs = [int(x) for x in self._hdl.buffer_ptrs]
        half = p.local_batch * p.total_D * self._symm.element_size()
        self._dest_ptrs = [torch.tensor([q + k * half for q in ptrs], dtype=torch.int64, device=self.device) for k in range(2)]
        self._col_offsets = torch.tensor(p.local_final_cols(), dtype=torch.int64, device=self.device)
        self._step = 0

    def forward_direct(self, indices, offsets, weights=None) -> torch.Tensor:
        from . import cabi
        p, tb = self.plan, self.tables
        k = self._step & 1
        self._step += 1
        out = self._symm[k]
        cabi.lookup(tb.weights_dev, tb.weights_offsets, tb.weights_tys, tb.D_offsets, tb.total_D, tb.max_D, indices, offsets,
                    int(tb.pooling_mode), out, indice_weights=weights, row_alignment=tb.row_alignment,
                    output_stride=p.total_D, output_col_offsets=self._col_offsets, dest_outputs=self._dest_ptrs[k],
                    rows_per_dest=p.local_batch, B=p.global_batch)
        # every rank's stores into this rank's buffer are complete once all ranks passed this point
        self._hdl.barrier(channel=k)
        return out

    def forward(self, indices, offsets, weights=None) -> torch.Tensor:
        return self.forward_direct(indices, offsets, weights) if self.exchange == "direct" else \
            self.forward_nccl(indices, offsets, weights)

    __call__ = forward
