"""lengths -> offsets and the reordering of a jagged request by table.

CPU: the numpy restatements against hand-computed answers.  GPU: the operators against the
restatements on the grids of the reference's own tests
(bench/sparse/asynchronous_complete_cumsum_test/test_asynchronous_complete_cumsum.py:39-70,
bench/sparse/permute_sparse_data/test_permute2d_sparse_data.py:22-40,128-150,
test_permute1d_sparse_data.py, test_permute2d_sparse_data_input1d.py); all of it is bit-exact.
"""
import zlib

import numpy as np
import pytest

import oracle as O


# ---- restatements, pinned by hand -------------------------------------------------------------

def test_complete_cumsum_known_answer():
    assert O.complete_cumsum(np.array([3, 0, 5, 1], dtype=np.int64)).tolist() == [0, 3, 3, 8, 9]
    assert O.complete_cumsum(np.array([], dtype=np.int32)).tolist() == [0]
    big = O.complete_cumsum(np.array([2**31 - 1, 1], dtype=np.int32))
    assert big.dtype == np.int32 and big.tolist() == [0, 2**31 - 1, -2**31]   # wraps like the type


def test_permute_2d_known_answer():
    # 3 tables, batch 2; table t owns sum(lengths[t]) values: t0 -> [10, 11, 12], t1 -> [20], t2 -> [30, 31]
    lengths = np.array([[1, 2], [0, 1], [2, 0]], dtype=np.int32)
    values = np.array([10, 11, 12, 20, 30, 31], dtype=np.int64)
    weights = values.astype(np.float32) / 2
    permute = np.array([2, 0, 2, 1], dtype=np.int32)   # repeats allowed, 4 outputs from 3 inputs
    ol, ov, ow = O.permute_2d_sparse_data(permute, lengths, values, weights)
    assert ol.tolist() == [[2, 0], [1, 2], [2, 0], [0, 1]]
    assert ov.tolist() == [30, 31, 10, 11, 12, 30, 31, 20]
    assert np.array_equal(ow, ov.astype(np.float32) / 2)
    w2 = np.stack([weights, weights + 1], axis=1)
    assert np.array_equal(O.permute_2d_sparse_data(permute, lengths, values, w2)[2], np.stack([ow, ow + 1], axis=1))
    el, ev, ew = O.permute_2d_sparse_data(np.array([], dtype=np.int32), lengths, values, None)
    assert np.array_equal(el, lengths) and np.array_equal(ev, values) and ew is None


# ---- GPU operators ------------------------------------------------------------------------------

def _rng(*key):
    return np.random.default_rng(zlib.crc32(repr(key).encode()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("length", [0, 1, 10, 100, 1000, 1024, 2048, 2049, 8192, 8193, 16384, 16385, 20000, 1 << 20, (1 << 22) + 77])
@pytest.mark.parametrize("ns", ["fbgemm", "mxrec"])
def test_cumsum_ops(dtype, length, ns):
    import torch
    import fbgemm_ascend_b200  # noqa: F401

    x = _rng("cumsum", dtype.__name__, length).integers(0, 100, length).astype(dtype)
    t = torch.from_numpy(x).cuda()
    ops = getattr(torch.ops, ns)
    want = O.complete_cumsum(x)
    assert np.array_equal(ops.asynchronous_complete_cumsum(t).cpu().numpy(), want)
    assert np.array_equal(ops.asynchronous_inclusive_cumsum(t).cpu().numpy(), want[1:] if length else x)
    assert np.array_equal(ops.asynchronous_exclusive_cumsum(t).cpu().numpy(), want[:-1] if length else x)


@pytest.mark.gpu
def test_cumsum_wraps_and_rejects():
    import torch
    import fbgemm_ascend_b200  # noqa: F401
    from fbgemm_ascend_b200 import cabi

    x = np.full(5000, 2**30, dtype=np.int32)
    got = torch.ops.fbgemm.asynchronous_complete_cumsum(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got, O.complete_cumsum(x))
    with pytest.raises(RuntimeError, match="int32 or int64"):
        torch.ops.fbgemm.asynchronous_complete_cumsum(torch.zeros(4, device="cuda"))
    # the C entry point refuses to run a long input without its scratch
    t = torch.zeros(10000, dtype=torch.int64, device="cuda")
    out = torch.empty(10001, dtype=torch.int64, device="cuda")
    rc = cabi.lib().tbe_b200_complete_cumsum(t.data_ptr(), 10000, 64, out.data_ptr(), None, 0, None)
    assert rc != 0 and "scratch" in cabi.last_error()


@pytest.mark.gpu
def test_cumsum_large_and_signed():
    """16.8 M elements (2048 tiles looking back over one another) with negative entries, and int64 sums that wrap."""
    import torch
    import fbgemm_ascend_b200  # noqa: F401

    x = _rng("cumsum-large").integers(-50, 100, (1 << 24) + 5).astype(np.int64)
    got = torch.ops.fbgemm.asynchronous_complete_cumsum(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got, O.complete_cumsum(x))
    # a view that starts one element into its storage: not 16-byte aligned, staged element by element
    for dt in (np.int32, np.int64):
        z = _rng("cumsum-unaligned", dt.__name__).integers(0, 1000, 70_001).astype(dt)
        view = torch.from_numpy(z).cuda()[1:]
        assert view.data_ptr() % 16 != 0
        assert np.array_equal(torch.ops.fbgemm.asynchronous_complete_cumsum(view).cpu().numpy(), O.complete_cumsum(z[1:]))
    y = _rng("cumsum-wrap").integers(-2**62, 2**62, 100_000).astype(np.int64)
    got = torch.ops.fbgemm.asynchronous_complete_cumsum(torch.from_numpy(y).cuda()).cpu().numpy()
    with np.errstate(over="ignore"):
        assert np.array_equal(got, O.complete_cumsum(y))


_ALONE = """
import sys, numpy as np, torch
sys.path.insert(0, {root!r})
import fbgemm_ascend_b200, oracle as O
for dt in (np.int32, np.int64):
    for n in (8193, 50_000, 300_001):
        x = np.random.default_rng(n).integers(0, 100, n).astype(dt)
        got = torch.ops.fbgemm.asynchronous_complete_cumsum(torch.from_numpy(x).cuda()).cpu().numpy()
        assert np.array_equal(got, O.complete_cumsum(x)), (dt, n)
print("alone-ok")
"""


@pytest.mark.gpu
def test_cumsum_tile_whose_wait_runs_out_adds_up_its_prefix_itself():
    """With a poll limit of 0 no tile ever waits for the tiles in front of it: each one falls back to summing the
    input before it, and the result is the same."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TBE_B200_SCAN_POLLS="0")
    r = subprocess.run([sys.executable, "-c", _ALONE.format(root=root)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "alone-ok" in r.stdout, r.stdout[-500:] + r.stderr[-1500:]


@pytest.mark.gpu
@pytest.mark.parametrize("vname", ["int64", "int32", "float16"])
def test_permute_copy_to_several_destinations(vname):
    """The copy step with one output buffer per group of output tables (what folds the index all-to-all into the
    permute): every buffer holds its group's part of the plain permute's result, nothing is written behind it, and a
    buffer that is too small takes what fits and reports bit 2."""
    import torch
    import fbgemm_ascend_b200  # noqa: F401
    from fbgemm_ascend_b200 import cabi

    for T_in, groups, tpd, B, empty in ((12, 3, 4, 50, ()), (8, 8, 1, 7, (0, 3, 7)), (6, 2, 3, 1, (2, 3)), (10, 5, 2, 33, (1, 2, 9))):
        _check_copy_to_dests(vname, T_in, groups, tpd, B, empty)


def _check_copy_to_dests(vname, T_in, groups, tpd, B, empty):
    import torch
    from fbgemm_ascend_b200 import cabi

    rng = _rng("to-dests", vname, T_in, tpd, B)
    permute = rng.permutation(T_in).astype(np.int32)
    lengths = rng.integers(0, 10, (T_in, B)).astype(np.int64)
    lengths[list(empty)] = 0                      # whole tables without values, also at the edges of a destination
    total = int(lengths.sum())
    vdt = _torch_dtype(vname)
    values = torch.arange(total, dtype=torch.float32).to(vdt) if vdt.is_floating_point else torch.arange(total, dtype=vdt)
    want_len, want_val, _ = O.permute_2d_sparse_data(permute, lengths, _as_np(values), None)
    seg = want_len.sum(1)
    bounds = np.concatenate([[0], np.cumsum(seg)])
    dev = torch.device("cuda")
    perm_d, len_d, val_d = torch.from_numpy(permute).to(dev), torch.from_numpy(lengths).to(dev), values.to(dev)
    scratch = torch.empty(cabi.permute_2d_sparse_scratch_elems(T_in, T_in), dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out_len = cabi.permute_2d_sparse_offsets(perm_d, len_d, scratch, status)
    assert np.array_equal(out_len.cpu().numpy(), want_len)
    group_sizes = [int(bounds[(g + 1) * tpd] - bounds[g * tpd]) for g in range(groups)]
    for cap, overflow in ((max(group_sizes) + 8, False), (max(group_sizes) // 2, True)):
        pad = 64
        bufs = [torch.full((cap + pad,), 7, dtype=vdt, device=dev) for _ in range(groups)]
        bases = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
        status.zero_()
        cabi.permute_2d_sparse_copy_to_dests(perm_d, T_in, val_d, bases, tpd, cap, scratch, status)
        torch.cuda.synchronize()
        assert int(status.item()) == (2 if overflow else 0)
        for g in range(groups):
            part = want_val[bounds[g * tpd]:bounds[(g + 1) * tpd]][:cap]
            got = _as_np(bufs[g].cpu())
            assert np.array_equal(got[:part.size], part), (g, cap)
            assert np.all(got[part.size:] == _as_np(torch.full((1,), 7, dtype=vdt))[0]), (g, cap)


VTYPES = ["int64", "int32", "float32", "float16", "bfloat16"]
WTYPES = [None, "float32", "float16", "bfloat16", "float64", "int32", "int64"]


def _torch_dtype(name):
    import torch
    return getattr(torch, name)


def _make_request(rng, t_in, t_out, b, ltype, vname, wname, wcols, lo, hi):
    import torch
    permute = rng.integers(0, t_in, t_out).astype(np.int32)
    lengths = rng.integers(lo, hi, (t_in, b)).astype(ltype)
    total = int(lengths.sum())
    vdt = _torch_dtype(vname)
    values = torch.rand(total, generator=torch.Generator().manual_seed(int(rng.integers(1 << 30)))).to(vdt) if vdt.is_floating_point \
        else torch.arange(total, dtype=vdt)
    weights = None
    if wname is not None:
        wdt = _torch_dtype(wname)
        shape = (total,) if wcols == 1 else (total, wcols)
        n = total * wcols
        weights = (torch.arange(n, dtype=torch.float64) * 0.25).to(wdt).reshape(shape) if wdt.is_floating_point \
            else torch.arange(n, dtype=wdt).reshape(shape)
    return permute, lengths, values, weights


def _as_np(t):
    import torch
    if t is None:
        return None
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy()
    return t.cpu().numpy()


def _check_permute(op, permute, lengths, values, weights, with_sum, reshape=None):
    import torch
    ol, ov, ow = O.permute_2d_sparse_data(permute, lengths, _as_np(values), _as_np(weights))
    kw = {}
    if with_sum:
        kw["permuted_lengths_sum"] = int(lengths.astype(np.int64)[permute].sum()) if permute.size and lengths.size else 0
    args = [torch.from_numpy(permute).cuda(), torch.from_numpy(lengths if reshape is None else reshape(lengths)).cuda(), values.cuda()]
    gl, gv, gw = op(*args, None if weights is None else weights.cuda(), **kw)
    assert np.array_equal(_as_np(gl).reshape(ol.shape), ol)
    assert gv.dtype == values.dtype and np.array_equal(_as_np(gv), ov)
    if weights is None:
        assert gw is None
    else:
        assert gw.dtype == weights.dtype and gw.shape[1:] == weights.shape[1:] and np.array_equal(_as_np(gw), ow)


@pytest.mark.gpu
@pytest.mark.parametrize("vname", VTYPES)
@pytest.mark.parametrize("wname", WTYPES)
@pytest.mark.parametrize("ltype", [np.int64, np.int32])
@pytest.mark.parametrize("with_sum", [True, False])
def test_permute_2d_sparse_data_types(vname, wname, ltype, with_sum):
    import torch
    import fbgemm_ascend_b200  # noqa: F401

    rng = _rng("p2d", vname, wname, ltype.__name__, with_sum)
    t = int(rng.integers(2, 60))
    extra = int(rng.integers(0, t))                      # permute picks t outputs from t + extra inputs
    req = _make_request(rng, t + extra, t, 128, ltype, vname, wname, 1, 1, 10)
    ns = torch.ops.fbgemm if with_sum else torch.ops.mxrec
    _check_permute(ns.permute_2D_sparse_data, *req, with_sum)
    _check_permute(ns.permute_sparse_data, *req, with_sum)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 0, 128, 1, 10), (97, 40, 1024, 1, 10), (13, 0, 2048, 0, 4), (7, 3, 20480, 1, 10), (5, 0, 64, 100, 800),
                                   (300, 100, 128, 0, 3), (1, 0, 1, 0, 50)])
@pytest.mark.parametrize("wcols", [1, 3, 4])
def test_permute_2d_sparse_data_shapes(shape, wcols):
    import torch
    import fbgemm_ascend_b200  # noqa: F401

    t, extra, b, lo, hi = shape
    rng = _rng("p2d-shape", shape, wcols)
    req = _make_request(rng, t + extra, t, b, np.int32, "int64", "float32", wcols, lo, hi)
    _check_permute(torch.ops.fbgemm.permute_2D_sparse_data, *req, True)
    _check_permute(torch.ops.fbgemm.permute_2D_sparse_data, *req, False)


@pytest.mark.gpu
@pytest.mark.parametrize("vname", ["int64", "float16"])
@pytest.mark.parametrize("wname", [None, "float32"])
def test_permute_1d_and_input1d(vname, wname):
    import torch
    import fbgemm_ascend_b200  # noqa: F401

    rng = _rng("p1d", vname, wname)
    # 1-D: every "table" is one bag
    permute, lengths, values, weights = _make_request(rng, 500, 300, 1, np.int64, vname, wname, 1, 0, 20)
    _check_permute(torch.ops.mxrec.permute_1D_sparse_data, permute, lengths, values, weights, True, reshape=lambda a: a.reshape(-1))
    _check_permute(torch.ops.mxrec.permute_1D_sparse_data, permute, lengths, values, weights, False, reshape=lambda a: a.reshape(-1))
    # lengths given flat with the batch size as `stride`
    permute, lengths, values, weights = _make_request(rng, 20, 20, 256, np.int32, vname, wname, 1, 0, 6)
    op = lambda p, l, v, w, **kw: torch.ops.fbgemm.permute_2D_sparse_data_input1D(p, l, v, 256, w, **kw)
    _check_permute(op, permute, lengths, values, weights, True, reshape=lambda a: a.reshape(-1))


@pytest.mark.gpu
def test_permute_2d_empty_and_errors():
    import torch
    import fbgemm_ascend_b200  # noqa: F401

    lengths = torch.zeros((0, 4), dtype=torch.int32, device="cuda")
    values = torch.zeros(0, dtype=torch.int64, device="cuda")
    gl, gv, gw = torch.ops.fbgemm.permute_2D_sparse_data(torch.zeros(0, dtype=torch.int32, device="cuda"), lengths, values, None)
    assert gl.shape == (0, 4) and gv.numel() == 0 and gw is None
    # all bags empty
    lengths = torch.zeros((3, 8), dtype=torch.int64, device="cuda")
    gl, gv, gw = torch.ops.fbgemm.permute_2D_sparse_data(torch.tensor([2, 0], dtype=torch.int32, device="cuda"), lengths, values, None)
    assert gl.shape == (2, 8) and int(gl.sum()) == 0 and gv.numel() == 0
    with pytest.raises(RuntimeError, match="2D"):
        torch.ops.fbgemm.permute_2D_sparse_data(torch.zeros(1, dtype=torch.int32, device="cuda"), lengths.view(-1), values, None)
    with pytest.raises(RuntimeError, match="mismatch"):
        torch.ops.fbgemm.permute_2D_sparse_data(torch.zeros(1, dtype=torch.int32, device="cuda"), lengths, values,
                                                torch.zeros(3, device="cuda"))
    with pytest.raises(RuntimeError, match="non-negative"):
        torch.ops.fbgemm.permute_2D_sparse_data(torch.zeros(1, dtype=torch.int32, device="cuda"), lengths, values, None, -1)


@pytest.mark.gpu
def test_request_pipeline_feeds_the_lookup():
    """lengths -> permute by table -> offsets -> pooled lookup equals the lookup on the tables taken in that order."""
    import torch
    import fbgemm_ascend_b200  # noqa: F401
    from helpers import make_case, gpu_lookup, oracle_lookup, assert_close

    T, B = 3, 16
    case = make_case(np.random.default_rng(5), [O.INT8, O.INT4, O.INT8], [64, 32, 128], [500, 500, 500], B, [12, 12, 12],
                     index_dtype=np.int64)
    lengths = np.diff(case.offsets).reshape(T, B)
    # the request arrives with its tables in another order; permuting it back must reproduce the case
    order = np.array([2, 0, 1], dtype=np.int32)
    inv = np.argsort(order).astype(np.int32)
    seg = np.split(case.indices, np.cumsum(lengths.sum(axis=1))[:-1])
    shuffled_len = np.ascontiguousarray(lengths[order])
    shuffled_val = np.concatenate([seg[t] for t in order])
    gl, gv, _ = torch.ops.fbgemm.permute_2D_sparse_data(torch.from_numpy(inv).cuda(), torch.from_numpy(shuffled_len).cuda(),
                                                        torch.from_numpy(shuffled_val).cuda(), None, int(shuffled_val.size))
    offs = torch.ops.fbgemm.asynchronous_complete_cumsum(gl.view(-1))
    assert np.array_equal(offs.cpu().numpy(), case.offsets) and np.array_equal(gv.cpu().numpy(), case.indices)
    case.indices, case.offsets = gv.cpu().numpy(), offs.cpu().numpy()
    assert_close(gpu_lookup(case, O.SUM, O.FP32), oracle_lookup(case, O.SUM, O.FP32), O.FP32)
