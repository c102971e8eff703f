"""HBM-bound kernels through the C ABI on a GPU: Ulysses pack/unpack, stale-KV patch update,
merge.  Copies are bit-exact; the merge is checked against the oracle."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.gpu_util import np64, rand  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ops():
    from xdit_b200 import build, ops

    build.build()
    assert ops.query_caps()["supported"] == 1
    return ops


def _ref_pack(x, joint, front, U):
    if joint is not None:
        x = torch.cat([joint, x], 2) if front else torch.cat([x, joint], 2)
    return x.permute(1, 0, 2, 3).contiguous().reshape(-1)  # usp.py:105 (== peer-major blocks)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,H,s,D,U", [(1, 24, 576, 128, 8), (2, 4, 97, 72, 2), (1, 8, 33, 4, 4), (1, 2, 1, 128, 1)])
def test_pack_bit_exact(ops, dtype, B, H, s, D, U):
    x = rand((B, s, H, D), dtype, 1).transpose(1, 2)  # strided view, as the DiT processors pass
    send = torch.empty(B * H * s * D, dtype=dtype, device="cuda")
    ops.ulysses_pack([dict(src=x, dst=send, peer_stride=(H // U) * B * s * D)], U)
    assert torch.equal(send, _ref_pack(x, None, False, U))


@pytest.mark.parametrize("front", [False, True])
def test_pack_qkv_with_joint_one_launch(ops, front):
    B, H, s, sj, D, U = 1, 8, 130, 20, 64, 4
    q, k, v = (rand((B, H, s, D), torch.bfloat16, i) for i in range(3))
    jq = rand((B, H, sj, D), torch.bfloat16, 9)
    Hl = H // U
    qb, kb = Hl * B * (s + sj) * D, Hl * B * s * D
    stride = qb + 2 * kb
    send = torch.full((U * stride,), -7.0, dtype=torch.bfloat16, device="cuda")
    before = ops.launch_count
    ops.ulysses_pack([dict(src=q, joint=jq, front=front, dst=send, peer_stride=stride),
                      dict(src=k, dst=send[qb:], peer_stride=stride),
                      dict(src=v, dst=send[qb + kb:], peer_stride=stride)], U)
    assert ops.launch_count == before + 1
    blocks = send.view(U, stride)
    assert torch.equal(blocks[:, :qb].reshape(-1), _ref_pack(q, jq, front, U))
    assert torch.equal(blocks[:, qb:qb + kb].reshape(-1), _ref_pack(k, None, False, U))
    assert torch.equal(blocks[:, qb + kb:].reshape(-1), _ref_pack(v, None, False, U))


def test_reference_wire_layout_helpers(ops):
    """usp.py:96-150 with the collective replaced by an identity (tests/layers/usp_test.py:268-307)."""
    z = np.load(os.path.join(HERE, "golden", "layout_identity_a2a.npz"))
    x = torch.from_numpy(z["x"]).cuda()
    b, h, s, d = x.shape
    U = 2
    send = torch.empty(x.numel(), device="cuda")
    ops.ulysses_pack([dict(src=x, dst=send, peer_stride=x.numel() // U)], U)
    got = ops.ulysses_unpack_in(send, b, h // U, s, d, U)
    assert torch.equal(got.cpu(), torch.from_numpy(z["in_id"]))
    got = ops.ulysses_unpack_out(ops.ulysses_pack_out(x).reshape(-1), b, h, s // U, d, U)
    assert torch.equal(got.cpu(), torch.from_numpy(z["out_id"]))


def test_combined_equals_separate(ops, monkeypatch):
    """tests/layers/usp_test.py:268-307: _combined_qkv_all_to_all == 3 x _ft_c_input_all_to_all."""
    from xdit_b200 import usp

    monkeypatch.setattr(usp, "get_ulysses_parallel_world_size", lambda: 2)
    monkeypatch.setattr(usp, "_sdpa_all_to_all_single", lambda t, group=None: t)
    q, k, v = (rand((2, 4, 128, 64), torch.bfloat16, i) for i in range(3))
    cq, ck, cv = usp._combined_qkv_all_to_all(q, k, v)
    for a, b in zip((cq, ck, cv), (q, k, v)):
        assert torch.equal(a, usp._ft_c_input_all_to_all(b))


def _replay(ops, z, cache_type, U, slice_dim, monkeypatch):
    import xdit_b200
    from xdit_b200 import cache_manager, distributed

    rs = xdit_b200.initialize_runtime_state()
    ts = [int(x) for x in z["token_start"]]
    rs.set_patches([ts[i + 1] - ts[i] for i in range(len(ts) - 1)])
    monkeypatch.setattr(cache_manager, "get_ulysses_parallel_world_size", lambda: U)
    mgr = cache_manager.CacheManager()
    mgr.register_cache_entry("L", "attn", cache_type)
    rs.set_patched_mode(False)
    k, v = mgr.update_and_get_kv_cache([torch.from_numpy(z["k0"]).cuda(), torch.from_numpy(z["v0"]).cuda()],
                                       "L", slice_dim=slice_dim)
    assert torch.equal(k.cpu(), torch.from_numpy(z["warm_k"]))
    assert torch.equal(v.cpu(), torch.from_numpy(z["warm_v"]))
    rs.set_patched_mode(True)
    for p in [int(x) for x in z["patch_order"]]:
        rs.pipeline_patch_idx = p
        k, v = mgr.update_and_get_kv_cache([torch.from_numpy(z[f"kp{p}"]).cuda(), torch.from_numpy(z[f"vp{p}"]).cuda()],
                                           "L", slice_dim=slice_dim)
        assert torch.equal(k.cpu(), torch.from_numpy(z[f"k_after{p}"])), p
        assert torch.equal(v.cpu(), torch.from_numpy(z[f"v_after{p}"])), p
    distributed._RUNTIME = None


def test_kvcache_naive_golden(ops, monkeypatch):
    _replay(ops, np.load(os.path.join(HERE, "golden", "kvcache_naive.npz")), "naive_cache", 1, 2, monkeypatch)


def test_kvcache_sp_golden(ops, monkeypatch):
    z = np.load(os.path.join(HERE, "golden", "kvcache_sp.npz"))
    _replay(ops, z, "sequence_parallel_attn_cache", int(z["U"]), 1, monkeypatch)


def test_kv_patch_segments_and_bounds(ops):
    """Fresh rows arriving as U segments (post all-to-all view) land rank-major at U*start."""
    B, H, S, D, U, n = 1, 3, 64, 72, 2, 8
    kc = rand((B, H, S, D), torch.bfloat16, 0)
    vc = rand((B, H, S, D), torch.bfloat16, 1)
    k0, v0 = kc.clone(), vc.clone()
    kn = rand((B, H, U, n, D), torch.bfloat16, 2)
    vn = rand((B, H, U, n, D), torch.bfloat16, 3)
    ops.kv_patch_update(kc, vc, kn, vn, 16)
    k0[:, :, 16:16 + U * n] = kn.reshape(B, H, U * n, D)
    v0[:, :, 16:16 + U * n] = vn.reshape(B, H, U * n, D)
    assert torch.equal(kc, k0) and torch.equal(vc, v0)
    from xdit_b200._capi import XditError

    with pytest.raises(XditError):
        ops.kv_patch_update(kc, vc, kn, vn, S - 3)


def test_kv_patch_pixart_shape_roundtrip(ops):
    """PixArt-Sigma 2048^2 stage shape: [1,16,16384,72] caches, 8 patches of 2048 rows; writing every
    patch once reproduces the full fresh tensor (size-independent property)."""
    B, H, S, D, P = 1, 16, 16384, 72, 8
    kf, vf = rand((B, H, S, D), torch.bfloat16, 5), rand((B, H, S, D), torch.bfloat16, 6)
    kc = torch.zeros_like(kf)
    vc = torch.zeros_like(vf)
    n = S // P
    for p in (3, 0, 7, 1, 2, 6, 5, 4):
        ops.kv_patch_update(kc, vc, kf[:, :, p * n:(p + 1) * n], vf[:, :, p * n:(p + 1) * n], p * n)
    assert torch.equal(kc, kf) and torch.equal(vc, vf)


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 72), (torch.float16, 5)])
def test_merge_matches_oracle(ops, dtype, D):
    from oracle import usp_oracle as O

    rows = 1000
    oa = rand((rows, D), torch.float32, 0)
    la = rand((rows,), torch.float32, 1, scale=3.0)
    ob = rand((rows, D), dtype, 2)
    lb = rand((rows,), torch.float32, 3, scale=3.0)
    want_o, want_l = O.merge_out_lse(np64(oa).reshape(1, 1, rows, D), np64(la).reshape(1, 1, rows),
                                     np64(ob).reshape(1, 1, rows, D), np64(lb).reshape(1, 1, rows))
    final = torch.empty(rows, D, dtype=dtype, device="cuda")
    ops.merge_out_lse(oa, la, ob, lb, first=False, out_final=final)
    np.testing.assert_allclose(np64(oa), want_o.reshape(rows, D), atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(np64(la), want_l.reshape(rows), atol=2e-6, rtol=1e-5)
    assert torch.equal(final, oa.to(dtype))
    # first=True initialises the accumulators from the block
    ops.merge_out_lse(oa, la, ob, lb, first=True)
    assert torch.equal(oa, ob.float()) and torch.equal(la, lb)


@pytest.mark.parametrize("dtype,D,rows", [(torch.float32, 72, 150_000), (torch.bfloat16, 96, 120_000),
                                          (torch.bfloat16, 256, 70_000), (torch.float16, 40, 200_000)])
def test_merge_many_rows_whose_vectors_span_warps(ops, dtype, D, rows):
    """Rows of 18, 24, 64 or 10 vectors do not divide a warp, and the launch is several waves of a
    grid-stride loop: every row's lse must still be read by all of its lanes before it is rewritten.
    Checked against the oracle's merge on a sample of rows and against a torch restatement on all."""
    from oracle import usp_oracle as O

    oa = rand((rows, D), torch.float32, 10)
    la = rand((rows,), torch.float32, 11, scale=3.0)
    ob = rand((rows, D), dtype, 12)
    lb = rand((rows,), torch.float32, 13, scale=3.0)
    oa0, la0 = oa.clone(), la.clone()
    ops.merge_out_lse(oa, la, ob, lb, first=False)
    torch.cuda.synchronize()
    w = torch.sigmoid(lb.double() - la0.double())[:, None]
    want_all = oa0.double() - w * (oa0.double() - ob.double())
    assert (oa.double() - want_all).abs().max().item() <= 5e-6
    idx = torch.arange(0, rows, 997, device="cuda")
    want_o, want_l = O.merge_out_lse(np64(oa0[idx]).reshape(1, 1, -1, D), np64(la0[idx]).reshape(1, 1, -1),
                                     np64(ob[idx]).reshape(1, 1, -1, D), np64(lb[idx]).reshape(1, 1, -1))
    np.testing.assert_allclose(np64(oa[idx]), want_o.reshape(-1, D), atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(np64(la[idx]), want_l.reshape(-1), atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("U", [4, 8, 16])
@pytest.mark.parametrize("front", [False, True])
def test_pack_to_peer_bases_equals_pack_into_one_buffer(ops, front, U):
    """xdit_ulysses_pack_peers with every "peer" buffer on this GPU: peer p's blocks must hold what
    xdit_ulysses_pack puts at p * peer_stride of one send buffer (q with joint rows, k, v in one launch)."""
    B, H, s, sj, sk, D = 1, 16, 100, 20, 130, 64
    q = rand((B, s, H, D), torch.bfloat16, 1).transpose(1, 2)
    jq = rand((B, H, sj, D), torch.bfloat16, 2)
    k, v = rand((B, H, sk, D), torch.bfloat16, 3), rand((B, H, sk, D), torch.bfloat16, 4)
    Hl = H // U
    q_blk, kv_blk = Hl * B * (s + sj) * D, Hl * B * sk * D
    stride = q_blk + 2 * kv_blk
    send = torch.zeros(U * stride, dtype=torch.bfloat16, device="cuda")
    ops.ulysses_pack([dict(src=q, joint=jq, front=front, dst=send, peer_stride=stride),
                      dict(src=k, dst=send[q_blk:], peer_stride=stride),
                      dict(src=v, dst=send[q_blk + kv_blk:], peer_stride=stride)], U)
    me = 2  # this rank's slot inside every peer's receive buffer
    bufs = [torch.zeros(U * stride, dtype=torch.bfloat16, device="cuda") for _ in range(U)]
    base = me * stride
    ops.ulysses_pack_peers([dict(src=q, joint=jq, front=front, dst_offset=base),
                            dict(src=k, dst_offset=base + q_blk),
                            dict(src=v, dst_offset=base + q_blk + kv_blk)], U, [b.data_ptr() for b in bufs])
    torch.cuda.synchronize()
    for p in range(U):
        assert torch.equal(bufs[p][base:base + stride], send[p * stride:(p + 1) * stride]), p
        assert float(bufs[p][:base].abs().sum()) == 0 and float(bufs[p][base + stride:].abs().sum()) == 0


def test_peer_buffer_alloc_view_free(ops):
    ptr, handle, view = ops.peer_alloc(1 << 20, "cuda")
    assert len(handle) == 64 and view.numel() == 1 << 20 and view.data_ptr() == ptr
    t = view[:4096].view(torch.bfloat16)
    t.fill_(1.5)
    torch.cuda.synchronize()
    assert float(t.float().sum()) == 1.5 * 2048
    del t, view
    ops.peer_free(ptr)


def test_peer_barrier_passes_when_all_flags_arrived_and_reports_a_missing_rank(ops):
    """xdit_peer_barrier as rank 0 of 2 on one GPU.  The other rank's flag word is written by hand (no second
    kernel is ever made to wait for this one).  With the flag in place the barrier passes and bumps the epoch;
    with the flag missing -- a word that nothing sets -- the wait runs out after 1 ms, the status words carry
    400 + the missing rank, the context stays usable, and later barriers do not wait while the failure is
    pending."""
    from xdit_b200 import _capi

    mine = torch.zeros(64, dtype=torch.int32, device="cuda")    # this rank's flag array
    theirs = torch.zeros(64, dtype=torch.int32, device="cuda")  # stands for rank 1's array
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = [mine.data_ptr(), theirs.data_ptr()]
    mine[1] = 1  # rank 1 has arrived at barrier 1
    ops.peer_barrier(flags, mine.data_ptr(), epoch, 0, "cuda", wait_limit_ns=1_000_000)
    torch.cuda.synchronize()
    ops.check_status()
    assert int(epoch.item()) == 1 and int(mine[0].item()) == 1 and int(theirs[0].item()) == 1
    mine[1] = 5  # a peer that is ahead also satisfies the wait
    ops.peer_barrier(flags, mine.data_ptr(), epoch, 0, "cuda", wait_limit_ns=1_000_000)
    torch.cuda.synchronize()
    ops.check_status()
    assert int(epoch.item()) == 2 and int(theirs[0].item()) == 2
    mine[1] = 0  # rank 1 never arrives at barrier 3
    ops.peer_barrier(flags, mine.data_ptr(), epoch, 0, "cuda", wait_limit_ns=1_000_000)
    torch.cuda.synchronize()
    st = ops._status("cuda")
    assert int(st.dev.item()) == 401 and int(st.host.item()) == 401
    assert int(theirs[0].item()) == 3  # its own flag was still posted
    ops.peer_barrier(flags, mine.data_ptr(), epoch, 0, "cuda", wait_limit_ns=2_000_000_000)  # returns at once
    torch.cuda.synchronize()
    with pytest.raises(_capi.XditError, match="code 401"):
        ops.check_status()
    assert int(st.dev.item()) == 0 and int(st.host.item()) == 0
