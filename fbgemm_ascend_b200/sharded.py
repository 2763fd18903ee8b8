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
                      NVLink peer memory; step flags with a bounded device-side wait replace the exchange
                      and no permute pass is left.

Peer buffers come from ``torch.distributed._symmetric_memory`` (plain peer mappings; no multicast).
Everything that can be tested without a GPU -- ownership, column maps, permute lists, split sizes --
is in :class:`ShardPlan`; the operators themselves are injectable so the plumbing also runs on CPU
ranks (gloo) in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import accumulate
from typing import Callable, List, Optional

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
                 device: Optional[torch.device] = None, out_dtype: torch.dtype = torch.float16,
                 max_polls: Optional[int] = None) -> None:
        if max_polls is not None:
            self.MAX_POLLS = int(max_polls)      # how long a rank waits for its peers' step flags before it reports
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
    #: polls (about a microsecond apart) after which a wait for the peers' step flags gives up and records bit 16 in
    #: ``status``; about two seconds
    MAX_POLLS = 1 << 21

    def _setup_direct(self) -> None:
        p = self.plan
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)   # error word of the lookup and of the waits
        self._col_offsets = torch.tensor(p.local_final_cols(), dtype=torch.int64, device=self.device)
        self._step = 0
        if p.world == 1:
            # one rank: the "exchange" is the column remap alone; plain local buffers, nothing to wait for
            self._out2 = torch.empty((2, p.local_batch, p.total_D), dtype=self.out_dtype, device=self.device)
            self._dest_ptrs = [None, None]
            return
        import torch.distributed._symmetric_memory as symm_mem

        gname = self.group.group_name if self.group is not None else dist.group.WORLD.group_name
        # one output buffer per rank, mapped into every peer; double-buffered so a rank may start writing
        # step n+1 while a slow peer still reads step n
        self._symm = symm_mem.empty((2, p.local_batch, p.total_D), dtype=self.out_dtype, device=self.device)
        self._hdl = symm_mem.rendezvous(self._symm, gname)
        self._out2 = self._symm
        ptrs = [int(x) for x in self._hdl.buffer_ptrs]
        half = p.local_batch * p.total_D * self._symm.element_size()
        self._dest_ptrs = [torch.tensor([q + k * half for q in ptrs], dtype=torch.int64, device=self.device) for k in range(2)]
        # step flags: flags[k][r] on rank s = the last step of buffer k that rank r has finished storing into rank s
        self._flags = symm_mem.empty((2, p.world), dtype=torch.int64, device=self.device)
        self._flags.zero_()
        self._fhdl = symm_mem.rendezvous(self._flags, gname)
        fptrs = [int(x) for x in self._fhdl.buffer_ptrs]
        self._flag_ptrs = [torch.tensor([q + k * p.world * 8 for q in fptrs], dtype=torch.int64, device=self.device) for k in range(2)]
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)        # every rank's flags are zero before anyone raises one

    def forward_direct(self, indices, offsets, weights=None) -> torch.Tensor:
        from . import cabi
        p, tb = self.plan, self.tables
        k = self._step & 1
        self._step += 1
        out = self._out2[k]
        cabi.lookup(tb.weights_dev, tb.weights_offsets, tb.weights_tys, tb.D_offsets, tb.total_D, tb.max_D, indices, offsets,
                    int(tb.pooling_mode), out, indice_weights=weights, row_alignment=tb.row_alignment,
                    output_stride=p.total_D, output_col_offsets=self._col_offsets, dest_outputs=self._dest_ptrs[k],
                    rows_per_dest=p.local_batch if p.world > 1 else 0, B=p.global_batch, error_flag=self.status)
        if p.world > 1:
            # this rank's stores into every peer are in place -> raise its flag there; then wait (bounded) until
            # every peer has raised its flag here: the buffer then holds the whole step
            value = (self._step + 1) // 2
            cabi.signal_peers(self._flag_ptrs[k], p.world, p.rank, value)
            cabi.wait_flags(self._flags[k], p.world, value, self.MAX_POLLS, self.status)
        return out

    def check_status(self) -> int:
        """Reads the error word (a device-to-host copy): 0, or the bits of ``tbe_b200_lookup_args.error_flag`` and bit 16
        (a peer's step flag did not arrive in time)."""
        return int(self.status.item())

    def forward(self, indices, offsets, weights=None) -> torch.Tensor:
        return self.forward_direct(indices, offsets, weights) if self.exchange == "direct" else \
            self.forward_nccl(indices, offsets, weights)

    __call__ = forward


class FeatureMajorInputDist:
    """Turns the feature-major request every rank holds for ITS samples into the table-major request over the
    GLOBAL batch that the rank's lookup needs (the step in front of the sharded lookup).

    Rank ``s`` starts with ``lengths [T_global, B_local]`` and the matching ``indices`` (all tables, its own
    ``B_local = B_global / world`` samples).  Per call:

      1. ``permute_2D_sparse_data`` groups the tables by owning rank (the order of ``ShardPlan.exchanged_order``);
      2. the lengths go through an all-to-all with equal splits, the send / receive counts of the indices are
         summed on the device and read by the host once (the collective needs them as host integers -- the
         reference reads its output size the same way, permute2d_sparse_data.cpp:100-108), then the indices (and
         per-sample weights) go through an all-to-all with those splits into local memory;
      3. what arrived is ordered (source rank, local table, sample); a second ``permute_2D_sparse_data`` over the
         ``world * T_local`` segments puts it into (local table, source rank, sample) order, which is table-major
         over the global batch, and ``asynchronous_complete_cumsum`` turns the lengths into offsets.

    The three operators are the package's own (``torch.ops.fbgemm.*``) unless replaced through the hooks, which
    lets the plumbing run on CPU ranks (gloo) in the tests.

    ``exchange="direct"`` (GPUs of one box, symmetric memory) replaces step 2's index all-to-all: the permute of step 1
    stores owner ``r``'s values straight into slot ``rank`` of ``r``'s receive buffer (``world`` slots of
    ``slot_capacity`` entries, double-buffered; plain peer stores, no multicast), raises its step flag at every peer
    and waits -- bounded, ``max_polls`` -- for theirs; step 3 reads the slots in place, the unused rest of every slot
    being one more segment that its permute list leaves out.  Only the lengths still go through a (small) collective.
    Per-sample weights are not moved on this path.  A slot that is too small drops values and sets bit 2 of ``status``;
    the ranks that see the count on the host (the sender and the owner) raise ``ValueError`` after the step, the others
    find out at their next collective.  ``wire_dtype=torch.int32`` narrows the indices before they are permuted and
    exchanged (row numbers fit 31 bits), on either path.
    """

    def __init__(self, plan: ShardPlan, group=None, device: Optional[torch.device] = None,
                 permute_fn: Optional[Callable] = None, cumsum_fn: Optional[Callable] = None,
                 index_dtype: torch.dtype = torch.int64, wire_dtype: Optional[torch.dtype] = None,
                 exchange: str = "nccl", slot_capacity: int = 0, max_polls: int = 1 << 21) -> None:
        self.plan = plan
        self.group = group
        self.device = device if device is not None else torch.device("cpu")
        self.index_dtype = index_dtype        # dtype of the indices and offsets handed to the lookup
        self.wire_dtype = wire_dtype          # dtype of the indices while they are permuted and exchanged (None: as given);
                                              # row numbers fit 31 bits, so int32 halves the bytes moved
        self.stages: Optional[list] = None    # set to [] to have one call record (name, CUDA event) after every stage
        self.permute_fn = permute_fn or (lambda perm, lengths, values, weights, total:
                                         torch.ops.fbgemm.permute_2D_sparse_data(perm, lengths, values, weights, total))
        self.cumsum_fn = cumsum_fn or (lambda x: torch.ops.fbgemm.asynchronous_complete_cumsum(x))
        p = plan
        self.T_loc = len(p.local_tables)
        if any(len(p.tables_of(r)) != self.T_loc for r in range(p.world)):
            raise ValueError("every rank must own the same number of tables")
        t32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.device)
        self.by_owner = t32(p.exchanged_order)                                            # step 1
        self.to_table_major = t32([s * self.T_loc + j for j in range(self.T_loc) for s in range(p.world)])   # step 3
        # "direct": no index all-to-all -- the first permute stores every owner's values straight into a slot of that
        # owner's receive buffer (peer memory, plain stores over NVLink), step flags say when a buffer is complete
        self.exchange = exchange if p.world > 1 else "nccl"
        if exchange not in ("nccl", "direct"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.max_polls = max_polls
        if self.exchange == "direct":
            if slot_capacity <= 0:
                raise ValueError("exchange='direct' needs slot_capacity: the most indices one rank sends to one owner")
            self._setup_direct(int(slot_capacity))

    def _setup_direct(self, cap: int) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        from . import cabi
        p, w = self.plan, self.plan.world
        wire = self.wire_dtype or self.index_dtype
        esz = torch.empty((), dtype=wire).element_size()
        agreed = torch.tensor([cap], dtype=torch.int64, device=self.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=self.group)      # every rank's buffer must have one size
        cap = (int(agreed.item()) + 15) // 16 * 16          # slots stay 16-byte aligned for every element size
        self.slot_capacity = cap
        gname = self.group.group_name if self.group is not None else dist.group.WORLD.group_name
        # receive buffer of this rank: [2 buffers][world slots][cap]; slot s is written by rank s alone
        self._recv = symm_mem.empty((2, w, cap), dtype=wire, device=self.device)
        hdl = symm_mem.rendezvous(self._recv, gname)
        ptrs = [int(x) for x in hdl.buffer_ptrs]
        self._dest_bases = [torch.tensor([q + (k * w + p.rank) * cap * esz for q in ptrs], dtype=torch.int64, device=self.device)
                            for k in range(2)]
        self._flags = symm_mem.empty((2, w), dtype=torch.int64, device=self.device)
        self._flags.zero_()
        fhdl = symm_mem.rendezvous(self._flags, gname)
        self._flag_ptrs = [torch.tensor([q + k * w * 8 for q in fhdl.buffer_ptrs], dtype=torch.int64, device=self.device) for k in range(2)]
        self._handles = (hdl, fhdl)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch = torch.empty(cabi.permute_2d_sparse_scratch_elems(len(p.dims), len(p.dims)), dtype=torch.int64, device=self.device)
        # second permute over world x (T_loc + 1) segments: the extra one per source stands for the unused rest of its slot
        self._to_table_major_slots = torch.tensor(self.slot_permute_list(w, self.T_loc), dtype=torch.int32, device=self.device)
        self._step = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    @staticmethod
    def slot_permute_list(world: int, T_loc: int) -> List[int]:
        """Permute list of the second ``permute_2D_sparse_data`` when the values sit in ``world`` slots: slot ``s`` is
        ``T_loc`` segments (source ``s``'s values for the local tables) followed by one more for the unused rest of the
        slot, which the list leaves out; the result is (local table, source rank) order."""
        return [s * (T_loc + 1) + j for j in range(T_loc) for s in range(world)]

    @staticmethod
    def slot_segment_lengths(len_recv: torch.Tensor, recv_counts: torch.Tensor, cap: int) -> torch.Tensor:
        """``len_recv`` [world, T_loc, B_loc] -> [world, T_loc + 1, B_loc]: every slot gets one more "table" whose first
        length is the unused rest of the slot (``cap`` minus what the source sent), so that the running sum of all
        lengths gives every segment's position inside the ``world * cap`` receive buffer."""
        w, T_loc, B_loc = len_recv.shape
        ext = torch.zeros((w, T_loc + 1, B_loc), dtype=len_recv.dtype, device=len_recv.device)
        ext[:, :T_loc] = len_recv
        ext[:, T_loc, 0] = cap - recv_counts.to(len_recv.dtype)
        return ext

    def check_status(self) -> int:
        """0, or bit 2 (a slot was too small: values were dropped) / bit 16 (a peer's step flag did not arrive in time)."""
        return int(self.status.item()) if self.exchange == "direct" else 0

    def _call_direct(self, lengths, indices):
        from . import cabi
        p, w, T_loc, B_loc, cap = self.plan, self.plan.world, self.T_loc, self.plan.local_batch, self.slot_capacity
        k = self._step & 1
        self._step += 1
        value = (self._step + 1) // 2
        self._mark("start")
        if self.wire_dtype is not None and indices.dtype != self.wire_dtype:
            indices = indices.to(self.wire_dtype)
            self._mark("narrow")
        # 1. permute by owner, stored straight into slot `rank` of every owner's buffer k; then this rank's flag there
        len_by_owner = cabi.permute_2d_sparse_offsets(self.by_owner, lengths.contiguous(), self._scratch, self.status)
        cabi.permute_2d_sparse_copy_to_dests(self.by_owner, len(p.dims), indices.contiguous(), self._dest_bases[k], T_loc, cap, self._scratch,
                                             self.status)
        cabi.signal_peers(self._flag_ptrs[k], w, p.rank, value)
        self._mark("permute_by_owner_into_peer_slots")
        # 2. lengths: a small all-to-all; the host needs the number of values that arrive to size the result
        len_recv = torch.empty_like(len_by_owner)
        dist.all_to_all_single(len_recv.view(-1), len_by_owner.view(-1), group=self.group)
        send_counts = len_by_owner.view(w, -1).sum(1, dtype=torch.int64)
        recv_counts = len_recv.view(w, -1).sum(1, dtype=torch.int64)
        self._mark("lengths_all_to_all")
        counts = torch.stack([send_counts, recv_counts]).cpu()
        if int(counts.max()) > cap:
            raise ValueError(f"slot_capacity {cap} is too small: a rank sends or receives {int(counts.max())} values for one owner")
        total = int(counts[1].sum())
        self._mark("host_read_of_counts")
        cabi.wait_flags(self._flags[k], w, value, self.max_polls, self.status)
        self._mark("wait_for_peer_stores")
        # 3. slots -> table-major: every source's slot is its T_loc segments plus one segment of unused space
        len_ext = self.slot_segment_lengths(len_recv.view(w, T_loc, B_loc), recv_counts, cap)
        len_tm, idx_tm, _ = self.permute_fn(self._to_table_major_slots, len_ext.view(w * (T_loc + 1), B_loc), self._recv[k].view(-1), None, total)
        self._mark("permute_to_table_major")
        offsets = self.cumsum_fn(len_tm.reshape(-1)).to(self.index_dtype)
        idx_tm = idx_tm.to(self.index_dtype)
        self._mark("cumsum")
        return idx_tm, offsets, None

    def __call__(self, lengths: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor] = None):
        p, w, T_loc, B_loc = self.plan, self.plan.world, self.T_loc, self.plan.local_batch
        if tuple(lengths.shape) != (len(p.dims), B_loc):
            raise ValueError(f"lengths must be [{len(p.dims)}, {B_loc}], got {tuple(lengths.shape)}")
        if self.exchange == "direct":
            if weights is not None:
                raise NotImplementedError("exchange='direct' moves indices only; use exchange='nccl' for per-sample weights")
            return self._call_direct(lengths, indices)
        self._mark("start")
        if self.wire_dtype is not None and indices.dtype != self.wire_dtype:
            indices = indices.to(self.wire_dtype)
            self._mark("narrow")
        # 1. tables grouped by owner: owner r's tables are rows [r * T_loc, (r + 1) * T_loc) of the result
        len_by_owner, idx_by_owner, w_by_owner = self.permute_fn(self.by_owner, lengths, indices, weights, indices.numel())
        self._mark("permute_by_owner")
        # 2. exchange
        send_counts = len_by_owner.view(w, -1).sum(1, dtype=torch.int64)
        if w == 1:
            len_recv, idx_recv, w_recv = len_by_owner, idx_by_owner, w_by_owner
            total = idx_by_owner.numel()
        else:
            len_recv = torch.empty_like(len_by_owner)
            dist.all_to_all_single(len_recv.view(-1), len_by_owner.contiguous().view(-1), group=self.group)
            recv_counts = len_recv.view(w, -1).sum(1, dtype=torch.int64)
            self._mark("lengths_all_to_all")
            counts = torch.stack([send_counts, recv_counts]).cpu()                        # the one host read of the step
            send_l, recv_l = counts[0].tolist(), counts[1].tolist()
            total = int(sum(recv_l))
            self._mark("host_read_of_split_sizes")
            idx_recv = torch.empty(total, dtype=indices.dtype, device=indices.device)
            dist.all_to_all_single(idx_recv, idx_by_owner.contiguous(), recv_l, send_l, group=self.group)
            self._mark("indices_all_to_all")
            w_recv = None
            if weights is not None:
                w_recv = torch.empty(total, dtype=weights.dtype, device=weights.device)
                dist.all_to_all_single(w_recv, w_by_owner.contiguous(), recv_l, send_l, group=self.group)
        # 3. (source rank, local table, sample) -> (local table, source rank, sample) = table-major over the global batch
        len_tm, idx_tm, w_tm = self.permute_fn(self.to_table_major, len_recv.view(w * T_loc, B_loc), idx_recv, w_recv, total)
        self._mark("permute_to_table_major")
        offsets = self.cumsum_fn(len_tm.reshape(-1)).to(self.index_dtype)
        idx_tm = idx_tm.to(self.index_dtype)
        self._mark("cumsum")
        return idx_tm, offsets, w_tm

    def _mark(self, name: str) -> None:
        if self.stages is not None and self.device.type == "cuda":
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.stages.append((name, e))

    def stage_ms(self) -> dict:
        """Milliseconds between consecutive marks of the recorded call (device time on the current stream)."""
        torch.cuda.synchronize()
        st = self.stages or []
        return {st[i][0]: round(st[i - 1][1].elapsed_time(st[i][1]), 4) for i in range(1, len(st))}
