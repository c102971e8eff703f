"""xdit_qk_norm_rope_pack (RMSNorm(q, k) + rotary embedding + head split + Ulysses pack in one launch)
against the oracle, on the reference-generated fixtures and on seeded cases with the shapes of the
Wan and Flux layers.  The oracle rounds to the storage type where the reference's 16-bit modules do
(pinned bit-for-bit by the `*_out_bf16` fixtures), and the kernel is held to one spacing of that type per
element, with at least 99.5 % of the elements bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import usp_oracle as O
from tests.gpu_util import np64, rand
from tests.gpu_util import compare as compare_abs

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def compare(got, want, what, kind, pair_mag):
    """Element-wise bound in units of the storage type's spacing.  ``want`` is the oracle with its two
    storage roundings (after the norm, after the rotation), i.e. the values the reference's 16-bit
    modules produce; the kernel does the same arithmetic in fp32 instead of float64, so it can differ only
    where a value sits within fp32 noise of a rounding boundary.  Such a flip moves a normalised element
    by one spacing and a rotated element by at most one spacing of the larger element of its pair, which
    after the final rounding is at most one spacing of the binade above that magnitude
    (|out| <= sqrt(2) * max(|x1|, |x2|)).  So: every element within ONE such spacing, and all but a
    sliver bit-exact."""
    g = np64(got).reshape(-1)
    w = np.asarray(want, dtype=np.float64).reshape(-1)
    m = np.asarray(pair_mag, dtype=np.float64).reshape(-1)
    assert g.shape == w.shape == m.shape, (what, g.shape, w.shape, m.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite values"
    bound = O.storage_ulp(2.0 * np.maximum(m, np.abs(w)), kind)
    err = np.abs(g - w)
    worst = int(np.argmax(err / bound))
    assert (err <= bound).all(), f"{what}: |err| {err[worst]:.4g} > one spacing {bound[worst]:.4g} at want={w[worst]:.4g}"
    exact = float((err == 0).mean())
    assert exact >= 0.995, f"{what}: only {exact:.4f} of the elements are bit-exact"


def _pair_mag(x):
    """max(|x[2i]|, |x[2i+1]|) broadcast back to both elements of each interleaved pair."""
    a = np.abs(np.asarray(x, dtype=np.float64))
    p = np.maximum(a[..., 0::2], a[..., 1::2])
    return np.repeat(p, 2, axis=-1)


@pytest.fixture(scope="module")
def ops():
    from xdit_b200 import ops as _ops

    return _ops


def _run(ops, q, k, v, H, U, wq, wk, eps, per_head, cos, sin):
    B, s, HD = q.shape
    D = HD // H
    blk = (H // U) * B * s * D
    stride = 3 * blk + 64  # a gap between peers' blocks: the kernel must respect the stride
    send = torch.full((U * stride,), float("nan"), dtype=q.dtype, device=q.device)
    ops.qk_norm_rope_pack(q, k, v, H, send, send[blk:], send[2 * blk:], (stride, stride, stride), U,
                          norm_q_weight=wq, norm_k_weight=wk, eps=eps, norm_per_head=per_head, cos=cos, sin=sin)
    torch.cuda.synchronize()
    outs = []
    for i in range(3):
        outs.append(torch.stack([send[p * stride + i * blk:p * stride + (i + 1) * blk].view(H // U, B, s, D)
                                 for p in range(U)]))
    gaps = torch.stack([send[p * stride + 3 * blk:(p + 1) * stride] for p in range(U)])
    assert torch.isnan(gaps).all(), "wrote between the peers' blocks"
    return outs


def _kind(t):
    return "bf16" if t.dtype == torch.bfloat16 else "f16"


def _check(ops, q, k, v, H, U, wq, wk, eps, per_head, cos, sin, what):
    got = _run(ops, q, k, v, H, U, wq, wk, eps, per_head, cos, sin)
    n = lambda t: None if t is None else np64(t)
    kind = _kind(q)
    want = O.attention_prologue(np64(q), np64(k), np64(v), H, n(wq), n(wk), eps, per_head, n(cos), n(sin), U,
                                round_to=kind)
    # magnitude of each rotated element's pair before the rotation (the normalised, rounded values)
    pre = O.attention_prologue(np64(q), np64(k), np64(v), H, n(wq), n(wk), eps, per_head, None, None, U,
                               round_to=kind)
    for g, w, p, name in zip(got, want, pre, "qkv"):
        compare(g, w, f"{what} {name}", kind, _pair_mag(p))
    assert torch.equal(got[2].reshape(-1), _plain_v(v, H, U).reshape(-1)), "v must be copied bit for bit"


def _plain_v(v, H, U):
    B, s, HD = v.shape
    return v.view(B, s, H, HD // H).permute(2, 0, 1, 3).reshape(U, H // U, B, s, HD // H)


@pytest.mark.parametrize("name", ["prologue_wan.npz", "prologue_per_head.npz"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_reference_fixture(ops, name, dtype):
    z = np.load(os.path.join(HERE, "golden", name))
    put = lambda a, dt=dtype: torch.from_numpy(a).to(dt).cuda()
    H, per_head = int(z["heads"]), bool(z["per_head"])
    q, k, v, wq, wk = (put(z[n]) for n in ("q", "k", "v", "wq", "wk"))
    cos, sin = put(z["cos"], torch.float32), put(z["sin"], torch.float32)
    got = _run(ops, q, k, v, H, 1, wq, wk, float(z["eps"]), per_head, cos, sin)
    if dtype == torch.bfloat16:
        # q_out_bf16 / k_out_bf16: the reference's own modules and rotary function run in bf16
        pre = O.attention_prologue(np64(q), np64(k), np64(v), H, np64(wq), np64(wk), float(z["eps"]), per_head,
                                   None, None, 1, round_to="bf16")
        for g, key, p in zip(got, ("q_out_bf16", "k_out_bf16"), pre):
            compare(g[0].permute(1, 0, 2, 3), z[key], key, "bf16", _pair_mag(p[0].transpose(1, 0, 2, 3)))
    _check(ops, q, k, v, H, 2, wq, wk, float(z["eps"]), per_head, cos, sin, name)


@pytest.mark.parametrize("H,D,per_head,U", [(40, 128, False, 1), (40, 128, False, 8), (24, 128, True, 4),
                                            (16, 72, False, 2), (8, 64, True, 1), (2, 8, True, 2)])
def test_model_shapes(ops, H, D, per_head, U):
    B, s = 2, 300
    q, k, v = (rand((B, s, H * D), torch.bfloat16, i) for i in range(3))
    wq = (1 + 0.1 * rand((D if per_head else H * D,), torch.float32, 7)).to(torch.bfloat16)
    wk = (1 + 0.1 * rand((D if per_head else H * D,), torch.float32, 8)).to(torch.bfloat16)
    ang = rand((s, D // 2), torch.float32, 9) * 3
    cos, sin = torch.cos(ang).repeat_interleave(2, 1).contiguous(), torch.sin(ang).repeat_interleave(2, 1).contiguous()
    _check(ops, q, k, v, H, U, wq, wk, 1e-6, per_head, cos, sin, f"H{H} D{D} U{U}")


@pytest.mark.parametrize("H,D,per_head,U,s", [
    (1, 8, False, 1, 5), (4, 128, True, 2, 37), (12, 64, False, 3, 64), (12, 128, True, 1, 41), (16, 128, False, 4, 33),
    (20, 128, False, 5, 29), (48, 64, True, 2, 23), (32, 128, False, 1, 19), (48, 128, False, 3, 17),
    (64, 128, True, 8, 13), (2, 256, True, 1, 31), (9, 72, False, 3, 27), (32, 72, False, 2, 21), (64, 72, False, 1, 9),
    (40, 128, False, 2, 3)])
def test_every_row_width(ops, H, D, per_head, U, s):
    """One case per compiled width of the kernel (vectors per lane 1..32), head dims whose vectors do not line
    up with the lanes (72), and row counts that leave warps of the last CTA without a row."""
    B = 2
    q, k, v = (rand((B, s, H * D), torch.bfloat16, 30 + i) for i in range(3))
    wq = (1 + 0.1 * rand((D if per_head else H * D,), torch.float32, 7)).to(torch.bfloat16)
    wk = (1 + 0.1 * rand((D if per_head else H * D,), torch.float32, 8)).to(torch.bfloat16)
    ang = rand((s, D // 2), torch.float32, 9) * 3
    cos, sin = torch.cos(ang).repeat_interleave(2, 1).contiguous(), torch.sin(ang).repeat_interleave(2, 1).contiguous()
    _check(ops, q, k, v, H, U, wq, wk, 1e-6, per_head, cos, sin, f"H{H} D{D} U{U} s{s}")


def test_slices_of_a_fused_projection_and_optional_steps(ops):
    """q, k, v as column slices of one [B, s, 3*H*D] projection; norm or rotary embedding left out."""
    B, s, H, D = 1, 130, 12, 64
    qkv = rand((B, s, 3 * H * D), torch.float16, 3)
    q, k, v = qkv.split(H * D, dim=2)
    w = (1 + 0.1 * rand((H * D,), torch.float32, 4)).half()
    ang = rand((s, D // 2), torch.float32, 5)
    cos, sin = torch.cos(ang).repeat_interleave(2, 1).contiguous(), torch.sin(ang).repeat_interleave(2, 1).contiguous()
    _check(ops, q, k, v, H, 2, w, w, 1e-5, False, cos, sin, "fused qkv")
    _check(ops, q, k, v, H, 2, None, None, 1e-5, False, cos, sin, "rope only")
    _check(ops, q, k, v, H, 4, w, None, 1e-5, False, None, None, "norm of q only")
    got = _run(ops, q, k, v, H, 1, None, None, 1e-5, False, None, None)
    for g, x in zip(got, (q, k, v)):
        assert torch.equal(g.reshape(-1), _plain_v(x, H, 1).reshape(-1)), "plain head split must be exact"


def test_heads_tensors_feed_attention(ops):
    """qk_norm_rope_heads -> attention equals oracle prologue -> oracle attention."""
    from xdit_b200.prologue import qk_norm_rope_heads

    B, s, H, D = 1, 512, 4, 128
    q, k, v = (rand((B, s, H * D), torch.bfloat16, 20 + i) for i in range(3))
    wq = (1 + 0.1 * rand((H * D,), torch.float32, 1)).to(torch.bfloat16)
    ang = rand((s, D // 2), torch.float32, 2)
    cos, sin = torch.cos(ang).repeat_interleave(2, 1), torch.sin(ang).repeat_interleave(2, 1)
    qh, kh, vh = qk_norm_rope_heads(q, k, v, H, norm_q_weight=wq, norm_k_weight=wq,
                                    rotary_emb=(cos[None, :, None, :], sin[None, :, None, :]))
    out, _ = ops.attn_fwd(qh, kh, vh)
    qs, ks, vs = O.attention_prologue(np64(q), np64(k), np64(v), H, np64(wq), np64(wq), 1e-6, False, np64(cos),
                                      np64(sin), 1)
    want, _ = O.attention_dense(*(x[0].transpose(1, 0, 2, 3) for x in (qs, ks, vs)))
    compare_abs(out, want, "attention after the fused prologue")


def test_rejects_bad_arguments(ops):
    from xdit_b200._capi import XditError

    q = rand((1, 16, 4 * 12), torch.bfloat16, 0)  # D = 12 is not a multiple of 8
    dst = torch.empty(3 * q.numel(), dtype=q.dtype, device="cuda")
    with pytest.raises(XditError):
        ops.qk_norm_rope_pack(q, q, q, 4, dst, dst, dst, (0, 0, 0), 1)
    q = rand((1, 16, 2 * 24), torch.bfloat16, 0)  # per-head norm with D/8 = 3
    w = torch.ones(24, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(XditError):
        ops.qk_norm_rope_pack(q, q, q, 2, dst, dst, dst, (0, 0, 0), 1, norm_q_weight=w, norm_per_head=True)
    with pytest.raises(RuntimeError):
        ops.qk_norm_rope_pack(q.cpu(), q.cpu(), q.cpu(), 2, dst, dst, dst, (0, 0, 0), 1)
