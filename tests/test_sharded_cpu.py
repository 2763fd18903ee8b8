"""Table-wise sharding plumbing on CPU ranks (gloo, world size 2): ownership, the exchange and the
permute lists.  The CUDA operators are replaced by the CPU oracle through the injectable hooks of
TableWiseShardedLookup, so this runs without a GPU; the GPU data paths are covered by
tests/test_sharded_gpu.py."""
import os
import socket
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from helpers import make_case



def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_shard_plan_lists():
    from fbgemm_ascend_b200.sharded import ShardPlan
    dims = [8, 16, 8, 16]
    plan = ShardPlan(world=2, rank=1, dims=dims, feature_order=[3, 0, 2, 1], global_batch=8)
    assert plan.tables_of(0) == [0, 2] and plan.local_tables == [1, 3]
    assert plan.exchanged_order == [0, 2, 1, 3]
    off, perm, inv_off, inv_perm = plan.permute_lists()
    assert off == [0, 8, 16, 32, 48]
    assert perm == [3, 0, 1, 2]                  # feature 3 sits at exchanged position 3, feature 0 at 0, ...
    assert inv_off == [0, 16, 24, 32, 48]
    assert [perm[i] for i in inv_perm] == [0, 1, 2, 3]
    assert plan.local_final_cols() == [32, 0]    # table 1 is last (after 16 + 8 + 8), table 3 first
    assert plan.local_batch == 4 and plan.total_D == 48
    with pytest.raises(ValueError):
        ShardPlan(world=2, rank=0, dims=dims, feature_order=[0, 1, 2, 2], global_batch=8)
    with pytest.raises(ValueError):
        ShardPlan(world=2, rank=0, dims=dims, feature_order=[0, 1, 2, 3], global_batch=7)


def _global_case():
    rng = np.random.default_rng(11)
    dims = [32, 64, 32, 16, 16, 16, 48, 32]     # both ranks hold 128 columns
    tys = [O.INT8, O.INT4, O.FP16, O.INT8, O.INT8, O.INT4, O.FP16, O.INT8]
    c = make_case(rng, tys, dims, [200] * 8, 12, [9] * 8, np.int64)
    order = [5, 2, 7, 0, 3, 6, 1, 4]
    return c, dims, tys, order


def _rank_main(rank, world, port, fail, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import datetime
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
        from fbgemm_ascend_b200.sharded import ShardPlan, TableWiseShardedLookup
        c, dims, tys, order = _global_case()
        B = c.B
        plan = ShardPlan(world=world, rank=rank, dims=dims, feature_order=order, global_batch=B)
        mine = plan.local_tables
        # the local shard: this rank's tables, and the global batch's bags of those tables
        offs = c.offsets
        l_tabs, l_idx, l_lens = [], [], []
        for t in mine:
            rb = O.row_bytes(tys[t], dims[t])
            start = int(c.weights_offsets[t])
            l_tabs.append(c.dev_weights[start:start + 200 * rb].reshape(200, rb))
            l_idx.append(c.indices[offs[t * B]:offs[(t + 1) * B]])
            l_lens.append(np.diff(offs[t * B:(t + 1) * B + 1]))
        dev, wo, wt, do = O.concat_tables(l_tabs, [tys[t] for t in mine], [dims[t] for t in mine])
        idx = np.concatenate(l_idx)
        loffs = np.concatenate([[0], np.cumsum(np.concatenate(l_lens))]).astype(np.int64)

        def lookup_fn(i, o, w):
            return torch.from_numpy(O.tbe_lookup(dev, wo, wt, do, i.numpy(), o.numpy(), O.SUM, None, O.FP16))

        def permute_fn(blocks, off, perm, inv_off, out):
            cat = torch.cat([blocks[r] for r in range(blocks.shape[0])], dim=1).numpy()
            out.copy_(torch.from_numpy(O.permute_pooled_embs(cat, off.numpy(), perm.numpy(), inv_off.numpy())))
            return out

        sh = TableWiseShardedLookup(plan, tables=None, group=None, exchange="nccl", lookup_fn=lookup_fn,
                                    permute_fn=permute_fn, device=torch.device("cpu"))
        if fail and rank == 1:
            raise RuntimeError("injected failure before the exchange")
        got = sh(torch.from_numpy(idx), torch.from_numpy(loffs)).numpy()
        # reference: everything on one process
        full = O.tbe_lookup(c.dev_weights, c.weights_offsets, c.weights_tys, c.D_offsets, c.indices, c.offsets, O.SUM, None, O.FP16)
        goff = np.concatenate([[0], np.cumsum(dims)])
        want = np.concatenate([full[:, goff[t]:goff[t + 1]] for t in order], axis=1)[rank * (B // world):(rank + 1) * (B // world)]
        q.put((rank, bool(np.array_equal(got.view(np.uint16), want.view(np.uint16))), ""))
        dist.destroy_process_group()
    except Exception as e:   # report instead of hanging the parent
        q.put((rank, False, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-600:]}"))


def _run(world, fail):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, fail, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for pr in procs:
        pr.join(timeout=60)
        if pr.is_alive():
            pr.kill()
    return sorted(res)


def test_two_rank_exchange_and_permute_bit_exact():
    res = _run(2, fail=False)
    assert all(ok for _, ok, _ in res), res


def test_rank_failure_before_exchange_surfaces_on_peer():
    """A rank that raises before the collective must not leave its peer hanging: the peer's exchange
    ends with an error (connection closed or the process-group timeout)."""
    res = _run(2, fail=True)
    assert res[1][1] is False and "injected failure" in res[1][2]
    assert res[0][1] is False and res[0][2] != ""


def _local_request(c, rank, world):
    """The feature-major request rank `rank` holds: every table's bags for its own B/world samples."""
    T, B = c.T, c.B
    Bl = B // world
    lens = np.diff(c.offsets).reshape(T, B)
    l_loc = lens[:, rank * Bl:(rank + 1) * Bl]
    idx = np.concatenate([c.indices[c.offsets[t * B + rank * Bl]:c.offsets[t * B + (rank + 1) * Bl]] for t in range(T)])
    return np.ascontiguousarray(l_loc), idx


def _dist_main(rank, world, port, weighted, q, narrow=False):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import datetime
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
        from fbgemm_ascend_b200.sharded import FeatureMajorInputDist, ShardPlan
        c, dims, tys, order = _global_case()
        B = c.B
        plan = ShardPlan(world=world, rank=rank, dims=dims, feature_order=order, global_batch=B)

        def permute_fn(perm, lengths, values, weights, total):
            l, v, w = O.permute_2d_sparse_data(perm.numpy(), lengths.numpy(), values.numpy(), None if weights is None else weights.numpy())
            assert v.size == total
            return torch.from_numpy(l), torch.from_numpy(v), None if w is None else torch.from_numpy(w)

        kw = dict(wire_dtype=torch.int32, index_dtype=torch.int32) if narrow else {}
        ind = FeatureMajorInputDist(plan, group=None, device=torch.device("cpu"), permute_fn=permute_fn,
                                    cumsum_fn=lambda x: torch.from_numpy(O.complete_cumsum(x.numpy())), **kw)
        l_loc, idx_loc = _local_request(c, rank, world)
        wts = None
        if weighted:
            wts = torch.from_numpy(idx_loc.astype(np.float32) * 0.5 + rank)      # a weight that names its index and its source
        idx_tm, offs_tm, w_tm = ind(torch.from_numpy(l_loc), torch.from_numpy(idx_loc), wts)
        # expected: the global batch's bags of this rank's tables, table-major
        offs = c.offsets
        want_idx = np.concatenate([c.indices[offs[t * B]:offs[(t + 1) * B]] for t in plan.local_tables])
        want_len = np.concatenate([np.diff(offs[t * B:(t + 1) * B + 1]) for t in plan.local_tables])
        want_off = np.concatenate([[0], np.cumsum(want_len)])
        ok = np.array_equal(idx_tm.numpy(), want_idx) and np.array_equal(offs_tm.numpy(), want_off)
        if narrow:
            ok = ok and idx_tm.dtype == torch.int32 and offs_tm.dtype == torch.int32
        if weighted:
            Bl = B // world
            src = np.concatenate([np.repeat(np.arange(B) // Bl, np.diff(offs[t * B:(t + 1) * B + 1])) for t in plan.local_tables])
            ok = ok and np.array_equal(w_tm.numpy(), want_idx.astype(np.float32) * 0.5 + src)
        q.put((rank, bool(ok), ""))
        dist.destroy_process_group()
    except Exception as e:
        q.put((rank, False, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-800:]}"))


@pytest.mark.parametrize("weighted,narrow", [(False, False), (True, False), (False, True)])
def test_feature_major_input_dist_two_ranks(weighted, narrow):
    """Index all-to-all in front of the lookup: two CPU ranks, each with the feature-major request of its own
    samples, end up with the table-major request of the global batch for their own tables (also with the indices
    narrowed to int32 for the permutes and the exchange)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dist_main, args=(r, 2, port, weighted, q, narrow)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for pr in procs:
        pr.join(timeout=60)
        if pr.is_alive():
            pr.kill()
    assert all(ok for _, ok, _ in res), res


def test_feature_major_input_dist_one_rank():
    """world = 1: no exchange; the feature-major request is already table-major, offsets are the running sums."""
    from fbgemm_ascend_b200.sharded import FeatureMajorInputDist, ShardPlan
    c, dims, tys, order = _global_case()
    plan = ShardPlan(world=1, rank=0, dims=dims, feature_order=order, global_batch=c.B)

    def permute_fn(perm, lengths, values, weights, total):
        l, v, w = O.permute_2d_sparse_data(perm.numpy(), lengths.numpy(), values.numpy(), None)
        return torch.from_numpy(l), torch.from_numpy(v), None

    ind = FeatureMajorInputDist(plan, device=torch.device("cpu"), permute_fn=permute_fn,
                                cumsum_fn=lambda x: torch.from_numpy(O.complete_cumsum(x.numpy())))
    l_loc, idx_loc = _local_request(c, 0, 1)
    idx_tm, offs_tm, _ = ind(torch.from_numpy(l_loc), torch.from_numpy(idx_loc))
    assert np.array_equal(idx_tm.numpy(), c.indices) and np.array_equal(offs_tm.numpy(), c.offsets)


def test_slot_layout_of_the_peer_store_exchange():
    """The host logic of ``exchange="direct"`` without GPUs: every rank permutes its request by owner and "stores" owner
    r's part into slot `rank` of r's receive buffer (here: numpy arrays standing for the peers' memory); the second
    permute, over the slots' segments plus one segment of unused space per slot, must give the owner the table-major
    request of the global batch for its tables."""
    from fbgemm_ascend_b200.sharded import FeatureMajorInputDist, ShardPlan
    c, dims, tys, order = _global_case()
    world, B = 2, c.B
    Bl = B // world
    plans = [ShardPlan(world=world, rank=r, dims=dims, feature_order=order, global_batch=B) for r in range(world)]
    T_loc = len(plans[0].local_tables)
    cap = 16 * ((max(c.indices.size, 1) + 15) // 16)
    recv = [np.full((world, cap), -7, dtype=np.int64) for _ in range(world)]            # receive buffer of every owner
    len_recv = [np.zeros((world, T_loc, Bl), dtype=np.int64) for _ in range(world)]
    for s in range(world):                                                             # what rank s does in step 1
        l_loc, idx_loc = _local_request(c, s, world)
        by_owner = np.asarray(plans[s].exchanged_order, dtype=np.int32)
        l_by, v_by, _ = O.permute_2d_sparse_data(by_owner, l_loc, idx_loc, None)
        seg = l_by.reshape(world, -1).sum(1)
        start = np.concatenate([[0], np.cumsum(seg)])
        for r in range(world):
            recv[r][s, :seg[r]] = v_by[start[r]:start[r + 1]]                          # the peer store into slot s of owner r
            len_recv[r][s] = l_by[r * T_loc:(r + 1) * T_loc]                           # the lengths all-to-all
    offs = c.offsets
    for r in range(world):                                                             # what owner r does in step 3
        counts = torch.from_numpy(len_recv[r].reshape(world, -1).sum(1))
        ext = FeatureMajorInputDist.slot_segment_lengths(torch.from_numpy(len_recv[r]), counts, cap).numpy()
        perm = np.asarray(FeatureMajorInputDist.slot_permute_list(world, T_loc), dtype=np.int32)
        l_tm, v_tm, _ = O.permute_2d_sparse_data(perm, ext.reshape(world * (T_loc + 1), Bl), recv[r].reshape(-1), None)
        want_idx = np.concatenate([c.indices[offs[t * B]:offs[(t + 1) * B]] for t in plans[r].local_tables])
        want_len = np.concatenate([np.diff(offs[t * B:(t + 1) * B + 1]) for t in plans[r].local_tables])
        assert np.array_equal(v_tm, want_idx)
        assert np.array_equal(l_tm.reshape(-1), want_len)
