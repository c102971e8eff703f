"""Size-independent properties of the oracle (test infrastructure checking itself): the Ulysses
re-layouts invert each other, sequence parallelism of any shape equals dense attention on the
gathered tensors, the online-softmax merge does not depend on the order of the blocks, and the
prologue's send layout is the head split of its single-rank form.  Seeded random shapes, float64."""
import itertools

import numpy as np
import pytest

from oracle import usp_oracle as O


def _rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("U,B,H,s,D", [(2, 1, 4, 6, 8), (4, 2, 8, 5, 4), (8, 1, 8, 3, 16), (1, 2, 3, 7, 4)])
def test_output_all_to_all_inverts_input_all_to_all(U, B, H, s, D):
    r = _rng(U * 100 + s)
    xs = [r.standard_normal((B, H, s, D)) for _ in range(U)]
    back = O.output_all_to_all(O.input_all_to_all(xs))
    for a, b in zip(xs, back):
        assert a.shape == b.shape and np.array_equal(a, b)
    if U > 1:
        # gathered sequence order is Ulysses-rank order; heads of peer p are [p*H/U, (p+1)*H/U)
        got = O.input_all_to_all(xs)
        for p in range(U):
            want = np.concatenate([x[:, p * H // U:(p + 1) * H // U] for x in xs], axis=2)
            assert np.array_equal(got[p], want)


@pytest.mark.parametrize("U,R", [(1, 1), (2, 1), (1, 3), (2, 2), (4, 2)])
@pytest.mark.parametrize("strategy", [None, "front", "rear"])
def test_usp_equals_dense_attention_on_the_gathered_sequence(U, R, strategy):
    P = U * R
    r = _rng(10 * U + R)
    B, H, D, s, sk, sj = 1, 4, 8, 5, 7, 3
    q = r.standard_normal((B, H, P * s, D))
    k = r.standard_normal((B, H, P * sk, D))
    v = r.standard_normal((B, H, P * sk, D))
    kw = {}
    if strategy:
        jq, jk, jv = (r.standard_normal((B, H, sj, D)) for _ in range(3))
        kw = dict(joint_query=jq, joint_key=jk, joint_value=jv, joint_strategy=strategy)
    outs = O.usp_from_global(q, k, v, U, R, **kw)
    if strategy:
        kk, vv = np.concatenate([k, jk], 2), np.concatenate([v, jv], 2)
    else:
        kk, vv = k, v
    img, _ = O.attention_dense(q, kk, vv)
    for g in range(P):
        want = img[:, :, g * s:(g + 1) * s]
        if strategy:
            txt, _ = O.attention_dense(jq, kk, vv)
            want = np.concatenate([want, txt], 2) if strategy == "rear" else np.concatenate([txt, want], 2)
        assert outs[g].shape == want.shape
        assert np.abs(outs[g] - want).max() < 1e-12, (U, R, strategy, g)


def test_merge_is_order_independent_and_matches_one_softmax():
    r = _rng(3)
    B, H, Sq, D, nblk, sk = 1, 2, 5, 4, 4, 6
    q = r.standard_normal((B, H, Sq, D))
    ks = [r.standard_normal((B, H, sk, D)) * 3 for _ in range(nblk)]
    vs = [r.standard_normal((B, H, sk, D)) for _ in range(nblk)]
    parts = [O.attention_dense(q, k, v) for k, v in zip(ks, vs)]
    want, want_lse = O.attention_dense(q, np.concatenate(ks, 2), np.concatenate(vs, 2))
    for order in itertools.permutations(range(nblk)):
        out = lse = None
        for i in order:
            out, lse = O.merge_out_lse(out, lse, *parts[i])
        assert np.abs(out - want).max() < 1e-12 and np.abs(lse - want_lse).max() < 1e-12


def test_merge_with_an_empty_block_keeps_the_other():
    """A block whose keys are all masked has lse = -inf and must not change the result."""
    r = _rng(4)
    out, lse = r.standard_normal((1, 1, 3, 4)), r.standard_normal((1, 1, 3))
    got, got_lse = O.merge_out_lse(out, lse, np.zeros_like(out), np.full_like(lse, -np.inf))
    assert np.allclose(got, out) and np.allclose(got_lse, lse)


@pytest.mark.parametrize("U", [1, 2, 4])
@pytest.mark.parametrize("per_head", [False, True])
def test_prologue_send_layout_is_the_head_split_of_the_single_rank_form(U, per_head):
    r = _rng(5 + U)
    B, s, H, D = 2, 6, 4, 8
    q, k, v = (r.standard_normal((B, s, H * D)) for _ in range(3))
    wq, wk = (1 + 0.1 * r.standard_normal(D if per_head else H * D) for _ in range(2))
    cos, sin = r.standard_normal((s, D)), r.standard_normal((s, D))
    one = O.attention_prologue(q, k, v, H, wq, wk, 1e-6, per_head, cos, sin, 1)
    many = O.attention_prologue(q, k, v, H, wq, wk, 1e-6, per_head, cos, sin, U)
    for a, b in zip(one, many):
        assert b.shape == (U, H // U, B, s, D)
        assert np.array_equal(a.reshape(H, B, s, D), b.reshape(H, B, s, D))
    # v passes through untouched; the norm leaves every group with unit mean square before the weight
    assert np.array_equal(one[2][0], v.reshape(B, s, H, D).transpose(2, 0, 1, 3))
    y = O.rms_norm(q, np.ones(D if per_head else H * D), 0.0, group=D if per_head else None)
    g = D if per_head else H * D
    assert np.allclose((y.reshape(B, s, -1, g) ** 2).mean(-1), 1.0)
    # a rotation keeps the norm of every pair when cos^2 + sin^2 = 1
    ang = r.standard_normal((s, D // 2))
    c, sn = np.repeat(np.cos(ang), 2, 1), np.repeat(np.sin(ang), 2, 1)
    x = r.standard_normal((B, s, H, D))
    rot = O.rope_interleaved(x, c[None, :, None, :], sn[None, :, None, :])
    assert np.allclose((rot.reshape(B, s, H, D // 2, 2) ** 2).sum(-1), (x.reshape(B, s, H, D // 2, 2) ** 2).sum(-1))
