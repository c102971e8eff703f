"""Attention kernels through the C ABI on a B200 against the oracle.

Tolerances (bf16/fp16): max-abs <= 2e-2 and cosine >= 0.9999 versus the oracle evaluated in
float64 on the same rounded inputs; fp32 (CUDA-core kernel): max-abs <= 2e-5.  LSE: 2e-3."""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import usp_oracle as O  # noqa: E402
from tests.gpu_util import compare, np64, oracle_attn, rand  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ops():
    from xdit_b200 import build, ops

    build.build()
    assert ops.query_caps()["supported"] == 1
    return ops


def _run(ops, q, k, v, k2=None, v2=None, **kw):
    out, lse = ops.attn_fwd(q, k, v, k2, v2, want_lse=True, **kw)
    torch.cuda.synchronize()
    ops.check_status()
    return out, lse


# ------------------------------------------------------------------ CUDA-core kernel
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Sq,Sk,D,causal", [
    (1, 2, 50, 50, 32, False), (2, 3, 33, 130, 4, False), (1, 2, 128, 128, 32, True),
    (1, 1, 1, 1, 8, False), (1, 2, 70, 200, 160, False), (1, 1, 97, 97, 72, True),
])
def test_generic_kernel(ops, dtype, B, H, Sq, Sk, D, causal):
    q, k, v = rand((B, H, Sq, D), dtype, 1), rand((B, H, Sk, D), dtype, 2), rand((B, H, Sk, D), dtype, 3)
    out, lse = _run(ops, q, k, v, causal=causal, force_generic=True)
    want, want_lse = oracle_attn(q, k, v, causal=causal)
    if dtype == torch.float32:
        compare(out, want, "out", max_abs=2e-5)
        compare(lse, want_lse, "lse", max_abs=2e-5, cos=0.0)
    else:
        compare(out, want, "out")
        compare(lse, want_lse, "lse", max_abs=2e-3, cos=0.0)


def test_generic_config1_fp32_joint(ops):
    """The Flux-shaped fp32 joint case as one dense call: 24 heads x 128, 4096 image + 512 joint keys; a
    4-head slice keeps the float64 oracle in seconds."""
    B, H, S, Sj, D = 1, 4, 4096, 512, 128
    q = rand((B, H, 600, D), torch.float32, 0)
    k, v = rand((B, H, S, D), torch.float32, 1), rand((B, H, S, D), torch.float32, 2)
    jk, jv = rand((B, H, Sj, D), torch.float32, 3), rand((B, H, Sj, D), torch.float32, 4)
    assert ops.attn_which(q, k, v, jk, jv) == 0
    out, lse = _run(ops, q, k, v, jk, jv)
    want, want_lse = oracle_attn(q, k, v, jk, jv)
    compare(out, want, "out", max_abs=2e-5)
    compare(lse, want_lse, "lse", max_abs=2e-5, cos=0.0)


# ------------------------------------------------------------------ tcgen05 kernel
SM100_SHAPES = [
    # B, H, Sq, Sk, D
    (1, 2, 256, 256, 128),      # exact tiles
    (1, 2, 128, 128, 128),      # one query tile, second tile of the CTA idle
    (2, 3, 300, 333, 128),      # ragged on both sides, batch > 1
    (1, 2, 64, 1, 128),         # a single key
    (1, 1, 1, 577, 128),        # a single query
    (1, 4, 515, 1200, 64),      # one-slab head_dim
    (1, 2, 200, 300, 72),       # PixArt head_dim: K padded to 80, V N = 80
    (1, 2, 128, 257, 32),       # head_dim of the reference's ring test
    (1, 2, 130, 190, 8),        # smallest head_dim of the TMA path
    (1, 3, 1030, 2050, 128),    # several CTAs per head, 17 key tiles
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Sq,Sk,D", SM100_SHAPES)
def test_sm100_kernel(ops, dtype, B, H, Sq, Sk, D):
    q, k, v = rand((B, H, Sq, D), dtype, 1), rand((B, H, Sk, D), dtype, 2), rand((B, H, Sk, D), dtype, 3)
    assert ops.attn_which(q, k, v) == 1
    out, lse = _run(ops, q, k, v)
    want, want_lse = oracle_attn(q, k, v)
    compare(lse, want_lse, "lse", max_abs=2e-3, cos=0.0)
    compare(out, want, "out")


def test_sm100_matches_generic_kernel(ops):
    q, k, v = (rand((1, 2, 333, 128), torch.bfloat16, i) for i in range(3))
    a, la = _run(ops, q, k, v)
    b, lb = _run(ops, q, k, v, force_generic=True)
    compare(a, np64(b), "tcgen05 vs CUDA-core", max_abs=1e-2)
    compare(la, np64(lb), "lse", max_abs=2e-3, cos=0.0)


def test_sm100_strided_views(ops):
    """[B,S,H,D] memory viewed as [B,H,S,D], as the processors pass it (transformer_flux.py:170-172)."""
    B, H, S, D = 2, 4, 300, 128
    q, k, v = (rand((B, S, H, D), torch.bfloat16, i).transpose(1, 2) for i in range(3))
    assert ops.attn_which(q, k, v) == 1
    out = torch.empty(B, S, H, D, dtype=torch.bfloat16, device="cuda").transpose(1, 2)
    _run(ops, q, k, v, out=out)
    compare(out, oracle_attn(q, k, v)[0], "out")


@pytest.mark.parametrize("D", [128, 64, 72])
def test_sm100_joint_second_source(ops, D):
    """Joint (text) K/V as a second source == torch.cat of usp.py:239-241, without the copy."""
    B, H, Sq, Sk, Sj = 1, 3, 260, 450, 77
    q, k, v = rand((B, H, Sq, D), torch.bfloat16, 1), rand((B, H, Sk, D), torch.bfloat16, 2), rand((B, H, Sk, D), torch.bfloat16, 3)
    jk_full, jv_full = rand((B, 2 * H, Sj, D), torch.bfloat16, 4), rand((B, 2 * H, Sj, D), torch.bfloat16, 5)
    jk, jv = jk_full[:, H:], jv_full[:, H:]  # head slice of a replicated tensor: a strided view
    out, lse = _run(ops, q, k, v, jk, jv)
    want, want_lse = oracle_attn(q, k, v, jk, jv)
    compare(lse, want_lse, "lse", max_abs=2e-3, cos=0.0)
    compare(out, want, "out")


@pytest.mark.parametrize("G,L", [(2, 576), (8, 72), (3, 100), (4, 64)])
def test_sm100_segmented_sequences(ops, G, L):
    """q/k/v as G segments (the receive buffer of a Ulysses all-to-all): equals attention over
    the concatenated rows, output written with the same segmentation."""
    B, H, D = 1, 2, 128
    def seg(seed, extra=0):
        buf = rand((G, H, B, L + extra, D), torch.bfloat16, seed)  # [peer][head][batch][rows][D]
        return buf.permute(2, 1, 0, 3, 4)[:, :, :, :L]
    q, k, v = seg(1), seg(2, 5), seg(3, 5)
    out_buf = torch.zeros(G, H, B, L, D, dtype=torch.bfloat16, device="cuda")
    out = out_buf.permute(2, 1, 0, 3, 4)
    assert ops.attn_which(q, k, v, out=out) == 1
    _, lse = _run(ops, q, k, v, out=out)
    want, want_lse = oracle_attn(q, k, v)
    compare(lse, want_lse, "lse", max_abs=2e-3, cos=0.0)
    compare(out.reshape(B, H, G * L, D), want, "out")


@pytest.mark.parametrize("force_generic", [False, True])
def test_ring_merge_in_epilogue(ops, force_generic):
    """Three key shards visited with acc_in/acc_out == one dense call (ring steps, usp.py:46-74)."""
    B, H, Sq, D = 1, 2, 300, 128
    q = rand((B, H, Sq, D), torch.bfloat16, 0)
    ks = [rand((B, H, n, D), torch.bfloat16, 10 + i) for i, n in enumerate((200, 333, 128))]
    vs = [rand((B, H, n, D), torch.bfloat16, 20 + i) for i, n in enumerate((200, 333, 128))]
    jk, jv = rand((B, H, 40, D), torch.bfloat16, 30), rand((B, H, 40, D), torch.bfloat16, 31)
    o_acc = torch.empty(B, H, Sq, D, dtype=torch.float32, device="cuda")
    lse_acc = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda")
    out = torch.empty_like(q)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda")
    for i in range(3):
        last = i == 2
        ops.attn_fwd(q, ks[i], vs[i], jk if last else None, jv if last else None, out=out if last else None,
                     lse=lse if last else None, o_acc=o_acc, lse_acc=lse_acc, acc_in=i > 0, acc_out=not last,
                     force_generic=force_generic)
    torch.cuda.synchronize()
    ops.check_status()
    want, want_lse = oracle_attn(q, torch.cat(ks + [jk], 2), torch.cat(vs + [jv], 2))
    compare(lse, want_lse, "lse", max_abs=2e-3, cos=0.0)
    compare(out, want, "out")


def test_large_magnitude_rows_rescale(ops):
    """Keys whose scores grow along the sequence force the lazy rescale path (max grows by > 2^8)."""
    B, H, Sq, Sk, D = 1, 1, 128, 1024, 128
    q = rand((B, H, Sq, D), torch.bfloat16, 0)
    k = rand((B, H, Sk, D), torch.bfloat16, 1)
    ramp = torch.linspace(0.2, 6.0, Sk, device="cuda").view(1, 1, Sk, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    v = rand((B, H, Sk, D), torch.bfloat16, 2)
    out, lse = _run(ops, q, k, v)
    want, want_lse = oracle_attn(q, k, v)
    compare(lse, want_lse, "lse", max_abs=5e-3, cos=0.0)
    compare(out, want, "out")


# ------------------------------------------------------------------ USP on one rank vs the reference fixture
def test_usp_single_rank_golden(ops):
    import xdit_b200

    xdit_b200.init_sequence_parallel(1, 1)
    z = np.load(os.path.join(HERE, "golden", "usp_u1r1_rear.npz"))
    q, k, v, jq, jk, jv = (torch.from_numpy(z[n]).cuda() for n in ("q", "k", "v", "jq", "jk", "jv"))
    out = xdit_b200.USP(q, k, v, joint_query=jq, joint_key=jk, joint_value=jv, joint_strategy="rear")
    torch.cuda.synchronize()
    compare(out, z["out"][0], "fp32 USP vs reference", max_abs=2e-5)
    b = lambda t: t.to(torch.bfloat16)
    out = xdit_b200.USP(b(q), b(k), b(v), joint_query=b(jq), joint_key=b(jk), joint_value=b(jv), joint_strategy="rear")
    torch.cuda.synchronize()
    ops.check_status()
    # held to what the reference returns for the same bf16-rounded inputs, at the stated tolerance
    compare(out, z["out_bf16"][0], "bf16 USP vs reference on bf16-rounded inputs")


def test_usp_errors(ops):
    import xdit_b200
    from xdit_b200.attention_backend import AttentionBackendType

    q = rand((1, 2, 16, 64), torch.bfloat16, 0)
    with pytest.raises(ValueError, match="Invalid joint_strategy"):
        xdit_b200.USP(q, q, q, joint_query=q, joint_key=q, joint_value=q, joint_strategy="middle")
    with pytest.raises(NotImplementedError, match="not registered"):
        xdit_b200.USP(q, q, q, backend=AttentionBackendType.AITER_FP8)
    with pytest.raises(NotImplementedError, match="masked"):
        xdit_b200.USP(q, q, q, attention_kwargs={"attn_mask": torch.ones(16, 16, device="cuda")})


# ------------------------------------------------------------------ full-size properties
def test_flux_shape_split_merge_property(ops):
    """Flux.1-dev attention shape (24 x 128, 4608 tokens): attention over all keys equals the fp32
    merge of attention over two key halves; and it is invariant to a permutation of the keys."""
    B, H, S, D = 1, 24, 4608, 128
    q, k, v = (rand((B, H, S, D), torch.bfloat16, i) for i in range(3))
    full, lse_full = _run(ops, q, k, v)
    o_acc = torch.empty(B, H, S, D, dtype=torch.float32, device="cuda")
    lse_acc = torch.empty(B, H, S, dtype=torch.float32, device="cuda")
    half = torch.empty_like(q)
    lse_half = torch.empty_like(lse_full)
    ops.attn_fwd(q, k[:, :, :2000], v[:, :, :2000], o_acc=o_acc, lse_acc=lse_acc, acc_out=True)
    ops.attn_fwd(q, k[:, :, 2000:], v[:, :, 2000:], out=half, lse=lse_half, o_acc=o_acc, lse_acc=lse_acc, acc_in=True)
    perm = torch.randperm(S, generator=torch.Generator().manual_seed(0)).cuda()
    permuted, _ = _run(ops, q, k[:, :, perm].contiguous(), v[:, :, perm].contiguous())
    torch.cuda.synchronize()
    ops.check_status()
    compare(half, np64(full), "split+merge vs full", max_abs=1e-2)
    compare(lse_half, np64(lse_full), "lse", max_abs=1e-3, cos=0.0)
    compare(permuted, np64(full), "key permutation", max_abs=1e-2)
    # one head against the oracle
    want, _ = oracle_attn(q[:, :1], k[:, :1], v[:, :1])
    compare(full[:, :1], want, "head 0 vs oracle")


def test_reference_test_shape_14867(ops):
    """tests/layers/usp_test.py:36: (1,24,14867,128) bf16, tolerance there 0.05 against sdpa_flash;
    here 4 heads against the oracle at the tolerance of this suite."""
    B, H, S, D = 1, 24, 14867, 128
    q, k, v = (rand((B, H, S, D), torch.bfloat16, i) for i in range(3))
    out, _ = _run(ops, q, k, v)
    for h in (0, 23):
        want, _ = oracle_attn(q[:, h:h + 1, :2048], k[:, h:h + 1], v[:, h:h + 1])
        compare(out[:, h:h + 1, :2048], want, f"head {h}")
    want, _ = oracle_attn(q[:, 5:6, -1500:], k[:, 5:6], v[:, 5:6])
    compare(out[:, 5:6, -1500:], want, "tail rows")


def test_wan_full_length_ring_split_property(ops):
    """Wan2.1 sequence length (75,600 tokens, head_dim 128), two heads: attention over all keys equals
    the epilogue-merged attention over four ring shards of 18,900 keys (the R4 split of the video
    configuration); selected query rows against the oracle over all 75,600 keys."""
    B, H, S, D, R = 1, 2, 75600, 128, 4
    q, k, v = (rand((B, H, S, D), torch.bfloat16, 40 + i) for i in range(3))
    full, lse_full = _run(ops, q, k, v)
    o_acc = torch.empty(B, H, S, D, dtype=torch.float32, device="cuda")
    lse_acc = torch.empty(B, H, S, dtype=torch.float32, device="cuda")
    ring = torch.empty_like(q)
    lse_ring = torch.empty_like(lse_full)
    sh = S // R
    for i in range(R):
        ks, vs = k[:, :, i * sh:(i + 1) * sh], v[:, :, i * sh:(i + 1) * sh]
        last = i == R - 1
        ops.attn_fwd(q, ks, vs, out=ring if last else None, lse=lse_ring if last else None, o_acc=o_acc,
                     lse_acc=lse_acc, acc_in=i > 0, acc_out=not last)
    torch.cuda.synchronize()
    ops.check_status()
    compare(ring, np64(full), "four ring shards vs one call", max_abs=1e-2)
    compare(lse_ring, np64(lse_full), "lse", max_abs=1e-3, cos=0.0)
    for rows in (slice(0, 96), slice(37777, 37777 + 96), slice(S - 96, S)):
        want, want_lse = oracle_attn(q[:, :, rows], k, v)
        compare(full[:, :, rows], want, f"rows {rows.start} vs oracle")
        assert np.abs(np64(lse_full[:, :, rows]) - want_lse).max() < 2e-3


def test_hunyuan_full_length_joint_rear_property(ops):
    """HunyuanVideo sequence length (118,800 image + 256 text tokens, joint "rear"), one head: the text
    keys as the kernel's second key/value source equal a concatenated key tensor; selected rows
    against the oracle."""
    B, H, S, Sj, D = 1, 1, 118800, 256, 128
    q, k, v = (rand((B, H, S, D), torch.bfloat16, 50 + i) for i in range(3))
    jk, jv = rand((B, H, Sj, D), torch.bfloat16, 60), rand((B, H, Sj, D), torch.bfloat16, 61)
    out2, _ = _run(ops, q, k, v, jk, jv)
    cat, _ = _run(ops, q, torch.cat([k, jk], 2), torch.cat([v, jv], 2))
    torch.cuda.synchronize()
    ops.check_status()
    compare(out2, np64(cat), "second source vs concatenated keys", max_abs=2e-3)
    rows = slice(59000, 59064)
    want, _ = oracle_attn(q[:, :, rows], k, v, jk, jv)
    compare(out2[:, :, rows], want, "rows vs oracle")


def test_cuda_graph_replay_matches_eager(ops):
    """A captured step (several USP calls) replays to the same bits as the eager calls."""
    import xdit_b200
    from xdit_b200.graph import GraphedStep

    xdit_b200.init_sequence_parallel(1, 1)
    ins = [tuple(rand((1, 4, 300, 128), torch.bfloat16, 10 * i + j) for j in range(3)) for i in range(3)]
    outs = []

    def step():
        outs.clear()
        for q, k, v in ins:
            outs.append(xdit_b200.USP(q, k, v))
        return outs

    step()
    torch.cuda.synchronize()
    eager = [o.clone() for o in outs]
    gs = GraphedStep(step, warmup=1)
    for q, _, _ in ins:
        q.mul_(1.0)  # inputs keep their addresses; replay reads whatever they hold now
    res = gs.replay()
    torch.cuda.synchronize()
    ops.check_status()
    for a, b in zip(res, eager):
        assert torch.equal(a, b)


def test_timed_out_wait_is_reported_by_the_next_call(ops):
    """The failure path of the tcgen05 kernel, without any fault: the loader leaves the first K/V
    stage un-armed (a barrier that nothing completes), the consumer's wait runs out after 2 ms, the
    launch drains and ends normally with the status words set.  The next launch does no work and the
    next call through the C ABI returns XDIT_E_KERNEL_TIMEOUT without the caller polling anything;
    after that the words are clear and the kernel computes again."""
    from xdit_b200 import _capi

    q, k, v = (rand((1, 2, 256, 128), torch.bfloat16, 40 + i) for i in range(3))
    assert ops.attn_which(q, k, v) == 1
    good, _ = _run(ops, q, k, v)
    sentinel = torch.full_like(q, 7.0)
    ops.attn_fwd(q, k, v, out=sentinel, _wait_limit_ns=2_000_000, _selftest_stall=True)
    torch.cuda.synchronize()  # the launch ended by itself: the context is alive
    st = ops._status(q.device)
    # both words carry a code (each CTA that gave up writes its own; the device word keeps the first)
    assert int(st.dev.item()) != 0 and int(st.host.item()) != 0
    assert torch.equal(sentinel, torch.full_like(q, 7.0))  # nothing was written
    with pytest.raises(_capi.XditError) as ei:
        ops.attn_fwd(q, k, v)
    assert ei.value.code == -6  # XDIT_E_KERNEL_TIMEOUT
    assert int(st.dev.item()) == 0 and int(st.host.item()) == 0  # cleared for a retry
    again, _ = _run(ops, q, k, v)
    assert torch.equal(again, good)


def test_launch_after_a_failure_is_a_no_op_until_cleared(ops):
    """While the device status word is set, launches exit at once (a failure must not cost one time
    limit per CTA); check_status() raises, clears, and the kernel runs again."""
    from xdit_b200 import _capi

    q, k, v = (rand((1, 1, 128, 64), torch.bfloat16, 50 + i) for i in range(3))
    st = ops._status(q.device)
    st.dev.fill_(123)  # as a timed-out CTA would leave it; the host word stays clear
    sentinel = torch.full_like(q, -3.0)
    ops.attn_fwd(q, k, v, out=sentinel)
    torch.cuda.synchronize()
    assert torch.equal(sentinel, torch.full_like(q, -3.0))
    with pytest.raises(_capi.XditError, match="code 123"):
        ops.check_status()
    out, _ = _run(ops, q, k, v)
    compare(out, oracle_attn(q, k, v)[0], "after clearing")


@pytest.mark.parametrize("Sk", [500, 2100])  # 2100 keys: the launch splits its keys and the merge kernel stores the rows
@pytest.mark.parametrize("D", [128, 64])
def test_segment_outputs_to_separate_bases(ops, D, Sk):
    """out_segments: the rows of query segment g go to a base address of their own, laid out
    [B, rows, H_total, D] with this call's heads at a column offset -- what the epilogue does when it stores
    every source rank's rows into that rank's result buffer.  Must equal the ordinary output bit for bit."""
    B, Hl, G, L, Htot, hoff = 1, 3, 4, 200, 12, 6
    q = rand((B, Hl, G, L, D), torch.bfloat16, 60)
    k, v = rand((B, Hl, Sk, D), torch.bfloat16, 61), rand((B, Hl, Sk, D), torch.bfloat16, 62)
    want, _ = _run(ops, q, k, v)  # [B, Hl, G, L, D]
    bufs = [torch.zeros(B, L, Htot, D, dtype=torch.bfloat16, device="cuda") for _ in range(G)]
    segs = [b.data_ptr() + hoff * D * 2 for b in bufs]
    ops.attn_fwd(q, k, v, out_segments=segs, out_strides=(L * Htot * D, D, Htot * D))
    torch.cuda.synchronize()
    ops.check_status()
    for g in range(G):
        got = bufs[g][:, :, hoff:hoff + Hl].permute(0, 2, 1, 3)  # [B, Hl, L, D]
        assert torch.equal(got, want[:, :, g]), g
        assert float(bufs[g][:, :, :hoff].abs().sum()) == 0 and float(bufs[g][:, :, hoff + Hl:].abs().sum()) == 0
    from xdit_b200 import _capi

    with pytest.raises(_capi.XditError):  # the CUDA-core kernel does not serve it
        ops.attn_fwd(q.float(), k.float(), v.float(), out_segments=segs, out_strides=(L * Htot * D, D, Htot * D))


@pytest.mark.parametrize("H,Sq,Sk,Sj,D,G", [(2, 1000, 2100, 0, 128, 1), (3, 300, 1537, 77, 128, 1),
                                             (2, 512, 4096, 0, 72, 1), (1, 256, 1100, 50, 64, 1),
                                             (2, 200, 2048, 0, 128, 3), (3, 4608, 4608, 0, 128, 1)])
def test_keys_split_over_ctas_equals_unsplit(ops, H, Sq, Sk, Sj, D, G):
    """A launch that would fill at most half of the SMs splits its keys over several CTAs per pair of query
    tiles and merges the partial results in a second kernel (the last case is a Flux layer's shard at Ulysses
    degree 8).  Same result as the unsplit kernel up to the rounding of the merge, same log-sum-exp, joint
    second source, ragged lengths, head_dim 64 / 72 and segmented queries included."""
    B = 1
    q = rand((B, H, G, Sq, D) if G > 1 else (B, H, Sq, D), torch.bfloat16, 70)
    k, v = rand((B, H, Sk, D), torch.bfloat16, 71), rand((B, H, Sk, D), torch.bfloat16, 72)
    k2 = v2 = None
    if Sj:
        k2, v2 = rand((B, H, Sj, D), torch.bfloat16, 73), rand((B, H, Sj, D), torch.bfloat16, 74)
    assert ops.attn_split_scratch_bytes(q, k, v, k2, v2) > 0
    try:
        ops.SPLIT_KEYS = False
        out0, lse0 = _run(ops, q, k, v, k2, v2)
    finally:
        ops.SPLIT_KEYS = True
    out1, lse1 = _run(ops, q, k, v, k2, v2)
    assert float((out1.float() - out0.float()).abs().max()) <= 8e-3
    assert float((lse1 - lse0).abs().max()) <= 1e-4
    if Sq * Sk <= 4_000_000:
        kk = k if k2 is None else torch.cat([k, k2], 2)
        vv = v if v2 is None else torch.cat([v, v2], 2)
        want, want_lse = oracle_attn(q.reshape(B, H, -1, D), kk, vv)
        compare(out1.reshape(B, H, -1, D), want, "out")
        compare(lse1.reshape(B, H, -1), want_lse, "lse", max_abs=2e-3, cos=0.0)
