"""permute_pooled_embs on the GPU: the reference's known-answer tests
(bench/pooled_embedding/permute_pooled_embs/permute_pooled_embedding_test.py:79-160,
permute_pooled_embedding_modules.py:45-80), its aligned / unaligned grids
(test_permute_pooled_embs.py:61-154) and bit-exact agreement with the CPU oracle."""
import random

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def lists(dims, perm, device="cuda"):
    off = np.concatenate([[0], np.cumsum(dims)]).astype(np.int64)
    inv_dims = [dims[p] for p in perm]
    inv_off = np.concatenate([[0], np.cumsum(inv_dims)]).astype(np.int64)
    inv_perm = np.zeros(len(perm), dtype=np.int64)
    for i, p in enumerate(perm):
        inv_perm[p] = i
    t = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int64)).to(device)
    return t(off), t(perm), t(inv_off), t(inv_perm)


@pytest.mark.parametrize("ns", ["fbgemm", "mxrec"])
def test_known_answer_permutation(ns):
    import fbgemm_ascend_b200  # noqa: F401
    off, perm, inv_off, inv_perm = lists([2, 3, 1, 4], [3, 0, 2, 1])
    x = torch.tensor([list(range(10))], dtype=torch.float32, device="cuda")
    y = getattr(torch.ops, ns).permute_pooled_embs(x, off, perm, inv_off, inv_perm)
    assert y.view(10).tolist() == [6, 7, 8, 9, 0, 1, 5, 2, 3, 4]


def test_docstring_example_and_module():
    from fbgemm_ascend_b200 import PermutePooledEmbeddings
    m = PermutePooledEmbeddings([4, 4, 8], [2, 0, 1], device="cuda")
    x = torch.arange(48, dtype=torch.float32, device="cuda").reshape(3, 16)
    y = m(x)
    want = torch.cat([x[:, 8:16], x[:, 0:4], x[:, 4:8]], 1)
    assert torch.equal(y, want)


def test_cat_reconstruction_and_autograd():
    from fbgemm_ascend_b200 import PermutePooledEmbeddings
    dims, order = [1, 2, 3, 4, 5], [2, 1, 3, 0, 4]
    parts = [torch.rand(7, d, device="cuda") for d in dims]
    x = torch.cat(parts, 1).requires_grad_(True)
    m = PermutePooledEmbeddings(dims, order, device="cuda")
    y = m(x)
    assert torch.allclose(y, torch.cat([parts[i] for i in order], 1))
    g = torch.rand_like(y)
    y.backward(g)
    # the gradient flows back through the inverse permutation
    inv = [order.index(i) for i in range(len(dims))]
    goff = np.concatenate([[0], np.cumsum([dims[i] for i in order])])
    want = torch.cat([g[:, goff[inv[i]]:goff[inv[i] + 1]] for i in range(len(dims))], 1)
    assert torch.equal(x.grad, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("aligned", [True, False])
@pytest.mark.parametrize("B", [1, 32, 333, 4096])
def test_random_dims_bit_exact(dtype, aligned, B):
    import fbgemm_ascend_b200  # noqa: F401
    rnd = random.Random(B * 3 + aligned)
    T = rnd.randint(1, 40)
    dims = [rnd.choice([16, 32, 64, 128, 256, 512, 1024]) if aligned else rnd.randint(1, 300) for _ in range(T)]
    if not aligned and T > 2:
        dims[1] = 0   # a zero-width feature must be skipped, not spin
    perm = list(range(T))
    rnd.shuffle(perm)
    off, p, inv_off, inv_p = lists(dims, perm)
    x = torch.randn(B, sum(dims), device="cuda").to(dtype)
    y = torch.ops.fbgemm.permute_pooled_embs(x, off, p, inv_off, inv_p)
    xb = x.view(torch.int16 if dtype != torch.float32 else torch.int32).cpu().numpy()
    want = O.permute_pooled_embs(xb, off.cpu().numpy(), np.asarray(perm), inv_off.cpu().numpy())
    got = y.view(torch.int16 if dtype != torch.float32 else torch.int32).cpu().numpy()
    assert np.array_equal(got, want)


def test_three_dim_input_and_validation_errors():
    import fbgemm_ascend_b200  # noqa: F401
    off, p, inv_off, inv_p = lists([8, 8], [1, 0])
    x = torch.randn(3, 5, 16, device="cuda")
    y = torch.ops.fbgemm.permute_pooled_embs(x, off, p, inv_off, inv_p)
    assert torch.equal(y, torch.cat([x[..., 8:], x[..., :8]], -1))
    with pytest.raises(RuntimeError, match="at least 2-D"):
        torch.ops.fbgemm.permute_pooled_embs(x[0, 0], off, p, inv_off, inv_p)
    with pytest.raises(RuntimeError, match="permute_list must be int64"):
        torch.ops.fbgemm.permute_pooled_embs(x, off, p.int(), inv_off, inv_p)
    with pytest.raises(RuntimeError, match="T\\+1 elements"):
        torch.ops.fbgemm.permute_pooled_embs(x, off[:-1], p, inv_off, inv_p)
    with pytest.raises(RuntimeError, match="float32, float16, or bfloat16"):
        torch.ops.fbgemm.permute_pooled_embs(x.double(), off, p, inv_off, inv_p)


def test_bad_permute_entry_sets_error_flag():
    from fbgemm_ascend_b200 import cabi
    off, p, inv_off, _ = lists([8, 8], [1, 0])
    p[0] = 5
    x = torch.randn(4, 16, device="cuda")
    out = torch.zeros_like(x)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.permute_pooled_embs(x, off, p, inv_off, out, flag)
    assert int(flag.item()) == 1
    assert torch.equal(out[:, 8:], x[:, :8])   # the valid feature was still copied


def test_config4_shape_involution():
    """Size-independent property at the sharded configuration's shape (fp16 [8192, 64*8*128]):
    permuting and then permuting back with the inverse lists is the identity."""
    import fbgemm_ascend_b200  # noqa: F401
    T = 512
    perm = list(range(T))
    random.Random(3).shuffle(perm)
    off, p, inv_off, inv_p = lists([128] * T, perm)
    x = torch.randn(8192, T * 128, device="cuda", dtype=torch.float16)
    y = torch.ops.fbgemm.permute_pooled_embs(x, off, p, inv_off, inv_p)
    z = torch.ops.fbgemm.permute_pooled_embs(y, inv_off, inv_p, off, p)
    assert torch.equal(z, x)
    assert torch.equal(y[:, :128], x[:, perm[0] * 128:(perm[0] + 1) * 128])
