"""xdit_attn_fwd_static_acc: the ring-step attention call that allocates nothing.

Some callers cannot hand the library freshly allocated device memory (a C serving loop with
fixed buffers, a plugin that must not touch its host framework's allocator).  For them the fp32
running accumulators of a ring sequence live in an array inside the library image.  This test
drives that entry point through the C ABI and checks it against the ordinary entry point
(caller-allocated accumulators) on two ring sequences in a row, because the array is shared by
all calls and keeps what the previous sequence left in it.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_util import compare, np64, oracle_attn, rand  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from xdit_b200 import build, ops

    build.build()
    assert ops.query_caps()["supported"] == 1
    return ops


def _ring_with_caller_buffers(ops, q, ks, vs, jk, jv):
    B, H, Sq, D = q.shape
    o_acc = torch.empty(B, H, Sq, D, dtype=torch.float32, device="cuda")
    lse_acc = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda")
    out = torch.empty_like(q)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda")
    n = len(ks)
    for i in range(n):
        last = i == n - 1
        ops.attn_fwd(q, ks[i], vs[i], jk if last else None, jv if last else None, out=out if last else None,
                     lse=lse if last else None, o_acc=o_acc, lse_acc=lse_acc, acc_in=i > 0, acc_out=not last)
    return out, lse


def _ring_without_allocation(ops, q, ks, vs, jk, jv, out, lse):
    n = len(ks)
    for i in range(n):
        last = i == n - 1
        ops.attn_fwd_static_acc(q, ks[i], vs[i], jk if last else None, jv if last else None,
                                out=out if last else None, lse=lse if last else None, acc_in=i > 0, acc_out=not last)


def test_static_accumulators_match_caller_accumulators_twice(ops):
    # two different ring sequences back to back: different shapes, so the second one reuses rows
    # of the shared array that still hold the first one's values
    cases = [((1, 3, 300, 128), (200, 333, 128), 40, 1), ((2, 2, 190, 64), (96, 260), 17, 2)]
    for (B, H, Sq, D), shards, Sj, seed in cases:
        q = rand((B, H, Sq, D), torch.bfloat16, seed)
        ks = [rand((B, H, n, D), torch.bfloat16, 10 * seed + i) for i, n in enumerate(shards)]
        vs = [rand((B, H, n, D), torch.bfloat16, 20 * seed + i) for i, n in enumerate(shards)]
        jk, jv = rand((B, H, Sj, D), torch.bfloat16, 30 * seed), rand((B, H, Sj, D), torch.bfloat16, 31 * seed)
        want, want_lse = _ring_with_caller_buffers(ops, q, ks, vs, jk, jv)
        out = torch.empty_like(q)
        lse = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda")
        # number of allocations made so far (a byte count would also move when the garbage collector
        # frees an unrelated tensor in between)
        count = lambda: torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        before = count()
        _ring_without_allocation(ops, q, ks, vs, jk, jv, out, lse)
        assert count() == before  # the wrapper itself allocated nothing
        torch.cuda.synchronize()
        ops.check_status()
        # same kernel, same arithmetic: the tolerance of the suite is far looser than what we see
        compare(out, np64(want), "static vs caller accumulators", max_abs=2e-2)
        compare(lse, np64(want_lse), "lse", max_abs=2e-3, cos=0.0)
        assert torch.equal(out, want) and torch.equal(lse, want_lse)
        # and both agree with the oracle over all keys
        ref, _ = oracle_attn(q, torch.cat(ks + [jk], 2), torch.cat(vs + [jv], 2))
        compare(out, ref, "vs oracle")


def test_static_accumulators_reject_oversize_and_misuse(ops):
    from xdit_b200 import _capi

    D = 128
    rows = _capi.XDIT_STATIC_ACC_FLOATS // (D + 1) + 64  # one step too large for the array
    q = torch.empty(1, 1, rows, D, dtype=torch.bfloat16, device="cuda")
    k = rand((1, 1, 64, D), torch.bfloat16, 0)
    with pytest.raises(_capi.XditError, match="exceeds the built-in scratch"):
        ops.attn_fwd_static_acc(q, k, k, acc_out=True)
    small = rand((1, 1, 64, D), torch.bfloat16, 1)
    with pytest.raises(_capi.XditError, match="neither acc_in nor acc_out"):
        ops.attn_fwd_static_acc(small, k, k, out=torch.empty_like(small))
    torch.cuda.synchronize()
    ops.check_status()
