"""Host-side orchestration of xdit_b200 (send-buffer layouts, strided receive views, all-to-all
and ring schedules) under gloo ranks on CPU.  The device kernels are replaced by the
oracle-backed stand-ins of tests/fake_ops.py, so what is checked here is the Python logic only;
the kernels themselves are checked on the GPU (tests marked gpu).  Expected values are the
outputs of the unmodified reference (tests/golden)."""
import pytest

import os

from tests.usp_worker import HERE, golden_files, run, run_flux_joint, run_kv, run_prologue


@pytest.mark.parametrize("mode", ["usp", "legacy", "compat", "yunchang", "usp_pipelined", "usp_peer"])
def test_world2_matches_reference(mode):
    run(2, golden_files(2), mode, 29720 + ["usp", "legacy", "compat", "yunchang", "usp_pipelined", "usp_peer"].index(mode))


@pytest.mark.parametrize("mode", ["usp", "legacy", "yunchang", "usp_pipelined", "usp_peer"])
def test_world4_matches_reference(mode):
    run(4, golden_files(4), mode, 29730 + ["usp", "legacy", "yunchang", "usp_pipelined", "usp_peer"].index(mode))


def _need_reference():
    """The reference's sources for this path: ``oracle/_ref`` (made by ``oracle/make_ref.py``) or a
    checkout named by ``XDIT_REFERENCE``."""
    from oracle import make_ref, ref_import

    if ref_import.root() is None and not make_ref.make(quiet=True):
        pytest.skip("the reference's sources are not here (oracle/make_ref.py makes oracle/_ref from a checkout)")


@pytest.mark.parametrize("world", [2, 4])
def test_reference_layer_runs_unmodified_on_the_shim(world):
    """The drop-in claim, exercised: the reference's own ``xFuserLongContextAttention.forward``
    (``hybrid/attn_layer.py:100-239``) and ``xdit_ring_flash_attn_forward`` (``ring/ring_flash_attn.py:27-148``)
    run unchanged on top of ``yunchang_compat.install()`` and reproduce the outputs of the reference's
    ``USP`` (the golden fixtures) -- the identity the reference asserts in ``tests/layers/usp_test.py:211-265``."""
    _need_reference()
    run(world, golden_files(world), "ref_layer", 29790 + world)


def test_yunchang_shim_serves_the_names_the_reference_imports():
    """xfuser/envs.py:346-352 and the other import sites listed in xdit_b200/yunchang_compat.py."""
    import sys

    from xdit_b200 import yunchang_compat

    assert "yunchang" not in sys.modules or getattr(sys.modules["yunchang"], "__xdit_b200_shim__", False)
    assert yunchang_compat.install()
    try:
        from yunchang import (LongContextAttention, LongContextAttentionQKVPacked, UlyssesAttention,  # noqa: F401
                              ring_flash_attn_func, set_seq_parallel_pg)
        from yunchang.comm.all_to_all import SeqAllToAll4D  # noqa: F401
        from yunchang.globals import HAS_SPARSE_SAGE_ATTENTION, PROCESS_GROUP
        from yunchang.kernels import AttnType, select_flash_attn_impl
        from yunchang.ring.ring_flash_attn import RingFlashAttnFunc, ring_flash_attn_backward  # noqa: F401
        from yunchang.ring.utils import RingComm, update_out_and_lse  # noqa: F401
        import xdit_b200

        assert PROCESS_GROUP is xdit_b200.PROCESS_GROUP and AttnType is xdit_b200.AttnType
        assert HAS_SPARSE_SAGE_ATTENTION is False
        assert AttnType.from_string("fa") is AttnType.FA
        with pytest.raises(NotImplementedError):
            select_flash_attn_impl(AttnType.FA, stage="bwd-only")
        with pytest.raises(NotImplementedError):
            ring_flash_attn_backward()
        layer = LongContextAttention(use_pack_qkv=True)
        assert layer.scatter_idx == 2 and layer.gather_idx == 1 and layer.use_pack_qkv
    finally:
        yunchang_compat.uninstall()
    assert "yunchang" not in sys.modules


def test_stale_kv_under_ulysses_matches_reference():
    """USP(attn_layer=...) with PipeFusion patches and Ulysses degree 2: the fresh rows reach the cache
    manager as two segments of the all-to-all receive buffer."""
    run_kv(2, os.path.join(HERE, "golden", "uspkv_u2r1.npz"), 29741)


@pytest.mark.parametrize("U,R", [(2, 1), (1, 2)])
def test_attention_from_projections_two_ranks(U, R):
    """The processor slice (norm, rotary embedding, head split, USP, head merge) against the oracle:
    Ulysses 2 takes the fused send-buffer path, ring 2 the [B,H,s,D] hand-over to USP."""
    run_prologue(2, U, R, 29745 + R)


def test_flux_joint_fp32_case_at_full_size_two_ranks():
    """Ulysses 2, 24 heads x 128, 4096 image + 512 joint text tokens (rear), fp32, seed 0: the host logic at
    the full shape (the stand-in attention is torch's fp32 CPU kernel here; the float64 oracle checks it)."""
    run_flux_joint(2, 29761, tol=2e-5)


@pytest.mark.parametrize("world", [2, 4])
def test_peer_store_exchange_in_bf16(world):
    """bf16 fixtures take the Ulysses exchange by stores into the peers' buffers (pack to per-peer bases, the
    attention's rows to per-segment bases) and the ring rotation through peer slots, with shared memory for
    the mapped buffers; compared with the reference's output for the bf16-rounded inputs."""
    run(world, golden_files(world), "usp_peer", 29790 + world, dtype_name="bfloat16", tol=2e-2)


def test_peer_buffers_grow_collectively():
    from tests.usp_worker import run_peer_growth

    run_peer_growth(2, 29797)


def test_kv_views_over_a_slot_of_a_larger_buffer():
    """The ring hands the view builder a slice of a peer-mapped buffer (slot 0 or 1): the views must address
    the slice, not the start of the storage it lives in."""
    import torch

    from xdit_b200.usp import _segmented_kv_views

    B, Hl, U, sk, D = 1, 2, 2, 5, 8
    kv_blk = Hl * B * sk * D
    stride = 2 * kv_blk
    flat = torch.arange(U * stride, dtype=torch.float32)
    k0, v0 = _segmented_kv_views(flat, B, Hl, U, sk, D, stride, 0, kv_blk)
    big = torch.full((3 * flat.numel() + 7,), -1.0)
    for off in (0, 7, flat.numel() + 7):
        slot = big[off:off + flat.numel()]
        slot.copy_(flat)
        k1, v1 = _segmented_kv_views(slot, B, Hl, U, sk, D, stride, 0, kv_blk)
        assert torch.equal(k1, k0) and torch.equal(v1, v0), off
        slot.fill_(-1.0)
