"""The numpy oracle against fixtures produced by the unmodified reference
(tests/golden/make_golden.py).  This is what pins the oracle."""
import glob
import os

import numpy as np
import pytest

from oracle import usp_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
USP_FILES = sorted(glob.glob(os.path.join(HERE, "golden", "usp_*.npz")))


def _load(path):
    z = np.load(path)
    U, R, B, H, D, S, Sj, Sk = [int(x) for x in z["meta"]]
    strat = str(z["strategy"])
    return z, U, R, B, H, D, S, Sj, Sk, (None if strat == "none" else strat)


def test_fixture_inventory():
    assert len(USP_FILES) >= 14


@pytest.mark.parametrize("path", USP_FILES, ids=[os.path.basename(p)[4:-4] for p in USP_FILES])
def test_usp_matches_reference(path):
    z, U, R, B, H, D, S, Sj, Sk, strat = _load(path)
    kw = {}
    if strat:
        kw = dict(joint_query=z["jq"], joint_key=z["jk"], joint_value=z["jv"], joint_strategy=strat)
    if path.endswith("combined.npz"):
        kw["combine_qkv_a2a"] = True
    outs = O.usp_from_global(z["q"], z["k"], z["v"], U, R, **kw)
    ref = z["out"]
    assert ref.shape[0] == U * R
    for g in range(U * R):
        assert outs[g].shape == ref[g].shape
        np.testing.assert_allclose(outs[g], ref[g], atol=2e-5, rtol=1e-4)


def _bf16_round(a):
    """Round-to-nearest-even to bfloat16, in numpy (what ``tensor.to(torch.bfloat16)`` does)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


@pytest.mark.parametrize("path", USP_FILES, ids=[os.path.basename(p)[4:-4] for p in USP_FILES])
def test_usp_on_bf16_rounded_inputs_matches_reference(path):
    """``out_bf16`` is the reference's result for the inputs rounded to bf16 (arithmetic in fp32): the
    yardstick of the bf16 GPU tests.  The oracle on the same rounded inputs must reproduce it."""
    z, U, R, B, H, D, S, Sj, Sk, strat = _load(path)
    kw = {}
    if strat:
        kw = dict(joint_query=_bf16_round(z["jq"]), joint_key=_bf16_round(z["jk"]),
                  joint_value=_bf16_round(z["jv"]), joint_strategy=strat)
    outs = O.usp_from_global(_bf16_round(z["q"]), _bf16_round(z["k"]), _bf16_round(z["v"]), U, R, **kw)
    for g in range(U * R):
        np.testing.assert_allclose(outs[g], z["out_bf16"][g], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("path", USP_FILES, ids=[os.path.basename(p)[4:-4] for p in USP_FILES])
def test_usp_equals_dense_attention(path):
    """Layout-independent property: every rank's rows equal dense attention over all keys."""
    z, U, R, B, H, D, S, Sj, Sk, strat = _load(path)
    P = U * R
    q, k, v = z["q"], z["k"], z["v"]
    if strat:
        kfull = np.concatenate([k, z["jk"]], axis=2)
        vfull = np.concatenate([v, z["jv"]], axis=2)
    else:
        kfull, vfull = k, v
    for g in range(P):
        ql = np.array_split(q, P, axis=2)[g]
        if strat:
            ql = O.concat_joint(ql, z["jq"], strat)
        dense, _ = O.attention_dense(ql, kfull, vfull)
        np.testing.assert_allclose(z["out"][g], dense, atol=2e-5, rtol=1e-4)


def test_layout_identity_a2a(golden_dir):
    """a2a re-layouts with the collective replaced by an identity, as the reference's own
    test does (tests/layers/usp_test.py:268-307)."""
    z = np.load(os.path.join(golden_dir, "layout_identity_a2a.npz"))
    x = z["x"]
    b, h, s, d = x.shape
    U = 2
    # identity collective == every rank holds the same x and receives its own flat buffer
    y = np.ascontiguousarray(np.transpose(x, (1, 0, 2, 3)))
    y = y.reshape(U, h // U, b, -1, d).transpose(2, 1, 0, 3, 4).reshape(b, h // U, -1, d)
    np.testing.assert_array_equal(y, z["in_id"])
    y = np.ascontiguousarray(np.transpose(x, (2, 0, 1, 3)))
    y = y.reshape(U, s // U, b, -1, d).transpose(2, 0, 3, 1, 4).reshape(b, -1, s // U, d)
    np.testing.assert_array_equal(y, z["out_id"])


def test_combined_equals_separate():
    rng = np.random.default_rng(0)
    U = 2
    qs = [rng.standard_normal((2, 4, 6, 8)) for _ in range(U)]
    ks = [rng.standard_normal((2, 4, 6, 8)) for _ in range(U)]
    vs = [rng.standard_normal((2, 4, 6, 8)) for _ in range(U)]
    cq, ck, cv = O.combined_qkv_all_to_all(qs, ks, vs)
    for a, b in zip(cq, O.input_all_to_all(qs)):
        np.testing.assert_array_equal(a, b)
    for a, b in zip(ck, O.input_all_to_all(ks)):
        np.testing.assert_array_equal(a, b)
    for a, b in zip(cv, O.input_all_to_all(vs)):
        np.testing.assert_array_equal(a, b)


def test_output_a2a_inverts_input_a2a():
    rng = np.random.default_rng(1)
    U = 4
    xs = [rng.standard_normal((1, 8, 5, 4)) for _ in range(U)]
    back = O.output_all_to_all(O.input_all_to_all(xs))
    for a, b in zip(xs, back):
        np.testing.assert_array_equal(a, b)


def test_merge_is_exact_split_softmax():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((1, 2, 7, 8))
    k = rng.standard_normal((1, 2, 33, 8))
    v = rng.standard_normal((1, 2, 33, 8))
    full, lse_full = O.attention_dense(q, k, v)
    out = lse = None
    for lo, hi in ((0, 10), (10, 11), (11, 33)):
        bo, bl = O.attention_dense(q, k[:, :, lo:hi], v[:, :, lo:hi])
        out, lse = O.merge_out_lse(out, lse, bo, bl)
    np.testing.assert_allclose(out, full, atol=1e-12)
    np.testing.assert_allclose(lse, lse_full, atol=1e-12)


def _replay_cache(z, cache_type, U, slice_dim):
    c = O.KVCacheOracle(cache_type, U=U)
    ts = [int(x) for x in z["token_start"]]
    tn = [ts[i + 1] - ts[i] for i in range(len(ts) - 1)]
    k, v = c.update(z["k0"], z["v0"], slice_dim, 4, False, 0, ts, tn)
    np.testing.assert_array_equal(k, z["warm_k"])
    np.testing.assert_array_equal(v, z["warm_v"])
    for p in [int(x) for x in z["patch_order"]]:
        k, v = c.update(z[f"kp{p}"], z[f"vp{p}"], slice_dim, 4, True, p, ts, tn)
        np.testing.assert_array_equal(k, z[f"k_after{p}"])
        np.testing.assert_array_equal(v, z[f"v_after{p}"])


def test_kvcache_naive(golden_dir):
    _replay_cache(np.load(os.path.join(golden_dir, "kvcache_naive.npz")), "naive", 1, 2)


def test_kvcache_sp(golden_dir):
    z = np.load(os.path.join(golden_dir, "kvcache_sp.npz"))
    _replay_cache(z, "sp", int(z["U"]), 1)


def test_legacy_bshd_equals_usp():
    """The identity the reference asserts in tests/layers/usp_test.py:211-265: the BSHD layer
    equals USP on transposed tensors, with and without joint tensors."""
    rng = np.random.default_rng(3)
    U, R = 2, 2
    P = U * R
    B, H, S, D, Sj = 1, 4, 32, 8, 6
    q, k, v = (rng.standard_normal((B, H, S, D)) for _ in range(3))
    jq, jk, jv = (rng.standard_normal((B, H, Sj, D)) for _ in range(3))
    t = lambda x: np.transpose(x, (0, 2, 1, 3))
    for strat in (None, "rear", "front"):
        kw = dict(joint_query=jq, joint_key=jk, joint_value=jv, joint_strategy=strat) if strat else {}
        a = O.usp_from_global(q, k, v, U, R, **kw)
        kw2 = dict(joint_query=t(jq), joint_key=t(jk), joint_value=t(jv), joint_strategy=strat) if strat else {}
        b = O.long_context_attention_bshd(np.array_split(t(q), P, axis=1), np.array_split(t(k), P, axis=1),
                                          np.array_split(t(v), P, axis=1), U, R, **kw2)
        for g in range(P):
            np.testing.assert_allclose(t(b[g]), a[g], atol=1e-12)


def test_causal_ring_equals_dense_causal():
    """tests/core/test_ring_flash_attn.py:78-103: causal ring == causal dense on the global
    sequence (fp16 (1,128,4,32) there; float64 here)."""
    rng = np.random.default_rng(4)
    R = 2
    q, k, v = (rng.standard_normal((1, 128, 4, 32)) for _ in range(3))
    outs, _ = O.ring_flash_attn_bshd(np.array_split(q, R, axis=1), np.array_split(k, R, axis=1),
                                     np.array_split(v, R, axis=1), causal=True)
    t = lambda x: np.transpose(x, (0, 2, 1, 3))
    dense, _ = O.attention_dense(t(q), t(k), t(v), causal=True)
    np.testing.assert_allclose(np.concatenate(outs, axis=1), t(dense), atol=1e-12)


def test_usp_with_stale_kv_under_ulysses(golden_dir):
    """USP(attn_layer=...) with two PipeFusion patches and Ulysses degree 2 (usp.py:313-314 ->
    cache_manager.py:138-194): warm-up step, then a patch step that refreshes patch 1 only."""
    z = np.load(os.path.join(golden_dir, "uspkv_u2r1.npz"))
    U = int(z["U"])
    patches = [int(x) for x in z["patches"]]
    starts = [0]
    for n in patches:
        starts.append(starts[-1] + n)
    t = lambda x: np.transpose(x, (0, 2, 1, 3))
    caches = [O.KVCacheOracle("sp", U=U) for _ in range(U)]

    def step(q, k, v, patch_mode, patch_idx):
        sh = lambda x: np.array_split(x, U, axis=2)
        qs, ks, vs = O.input_all_to_all(sh(q)), O.input_all_to_all(sh(k)), O.input_all_to_all(sh(v))
        outs = []
        for r in range(U):
            kc, vc = caches[r].update(t(ks[r]), t(vs[r]), 1, len(patches), patch_mode, patch_idx, starts, patches)
            o, _ = O.attention_dense(qs[r], t(kc), t(vc))
            outs.append(o)
        return O.output_all_to_all(outs)

    out0 = step(z["q0"], z["k0"], z["v0"], False, 0)
    out1 = step(z["q1"], z["k1"], z["v1"], True, int(z["patch_idx"]))
    for r in range(U):
        np.testing.assert_allclose(out0[r], z["out0"][r], atol=2e-5, rtol=1e-4)
        np.testing.assert_allclose(out1[r], z["out1"][r], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("name", ["prologue_wan.npz", "prologue_per_head.npz"])
def test_attention_prologue_matches_reference(name):
    """Norm + rotary embedding + head split against the reference's own code path
    (torch.nn.RMSNorm and the rotary function of transformer_wan.py:108-120, see make_golden.py)."""
    z = np.load(os.path.join(HERE, "golden", name))
    H, per_head = int(z["heads"]), bool(z["per_head"])
    outs = O.attention_prologue(z["q"], z["k"], z["v"], H, z["wq"], z["wk"], float(z["eps"]), per_head,
                                z["cos"], z["sin"], U=1)
    for got, key in zip(outs, ("q_out", "k_out", "v_out")):
        assert np.abs(got[0].transpose(1, 0, 2, 3) - z[key]).max() < 2e-6, key
    # send layout for two peers: peer p holds heads [p*H/2, (p+1)*H/2)
    q2 = O.attention_prologue(z["q"], z["k"], z["v"], H, z["wq"], z["wk"], float(z["eps"]), per_head,
                              z["cos"], z["sin"], U=2)[0]
    for p in range(2):
        assert np.abs(q2[p].transpose(1, 0, 2, 3) - z["q_out"][:, p * H // 2:(p + 1) * H // 2]).max() < 2e-6


@pytest.mark.parametrize("name", ["prologue_wan.npz", "prologue_per_head.npz"])
def test_attention_prologue_rounding_points_match_the_reference_in_bf16(name):
    """`q_out_bf16` / `k_out_bf16` were produced by the reference's own norm modules and rotary function
    run in bf16.  The oracle with ``round_to="bf16"`` (one rounding after norm x weight, one after the
    rotation) reproduces them bit for bit: that is what pins where a 16-bit implementation may round."""
    z = np.load(os.path.join(HERE, "golden", name))
    r = lambda a: O.round_to_storage(a, "bf16")
    H, per_head = int(z["heads"]), bool(z["per_head"])
    qs, ks, _ = O.attention_prologue(r(z["q"]), r(z["k"]), r(z["v"]), H, r(z["wq"]), r(z["wk"]), float(z["eps"]),
                                     per_head, z["cos"], z["sin"], 1, round_to="bf16")
    np.testing.assert_array_equal(qs[0].transpose(1, 0, 2, 3), z["q_out_bf16"])
    np.testing.assert_array_equal(ks[0].transpose(1, 0, 2, 3), z["k_out_bf16"])


def test_round_to_storage_matches_torch():
    import torch

    x = np.random.default_rng(0).standard_normal(20000) * np.exp(np.random.default_rng(1).uniform(-8, 8, 20000))
    x = x.astype(np.float32).astype(np.float64)  # fp32 values: torch rounds a double by way of fp32
    t = torch.from_numpy(x).float()
    np.testing.assert_array_equal(O.round_to_storage(x, "bf16"), t.to(torch.bfloat16).double().numpy())
    np.testing.assert_array_equal(O.round_to_storage(x, "f16"), t.to(torch.float16).double().numpy())
    assert O.storage_ulp(1.0, "bf16") == 2.0 ** -7 and O.storage_ulp(5.0, "bf16") == 2.0 ** -5
    assert O.storage_ulp(1.0, "f16") == 2.0 ** -10


def test_model_boundary_shard_and_gather_match_reference(golden_dir):
    """`boundary_w4.npz`: the reference's `_chunk_and_pad_sequence` and `_gather_and_unpad` (on its real
    `GroupCoordinator.all_gather`) under 4 gloo ranks, sequence lengths 10, 13, 9 and 8."""
    z = np.load(os.path.join(golden_dir, "boundary_w4.npz"))
    W = int(z["world"])
    for name in z["names"]:
        x, dim, pad = z[f"{name}_x"], int(z[f"{name}_dim"]), int(z[f"{name}_pad"])
        chunks, got_pad = O.pad_and_shard_sequence(x, W, dim=dim)
        assert got_pad == pad
        np.testing.assert_array_equal(np.stack(chunks), z[f"{name}_chunks"])
        np.testing.assert_array_equal(O.gather_and_unpad(chunks, pad, dim=dim), z[f"{name}_gathered"])
        np.testing.assert_array_equal(z[f"{name}_gathered"], x)  # the round trip is the identity
