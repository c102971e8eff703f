#!/usr/bin/env python
"""Generate the golden fixtures in this directory by running the *unmodified* xDiT reference.

Run once, where a checkout of the reference is available; ``XDIT_REFERENCE`` names its root::

    XDIT_REFERENCE=<path to the xDiT checkout> python tests/golden/make_golden.py

The reference's ``xfuser/model_executor/layers/usp.py`` and
``xfuser/core/cache_manager/cache_manager.py`` are imported as they are.  Their heavy
package ``__init__`` files (which need ``diffusers``) are skipped by pre-seeding bare
namespace packages in ``sys.modules`` and a three-attribute ``diffusers`` stub.  Ranks are
gloo processes on CPU.  Ulysses groups are contiguous ranks and ring groups are strided by
the Ulysses degree (the yunchang convention the reference relies on,
``xfuser/core/distributed/parallel_state.py:494-512``).

Every case is written as one ``.npz`` holding the per-rank inputs and the per-rank outputs
``USP()`` returned, so that tests can replay the same inputs through the oracle and through
the CUDA path without the reference being present.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("XDIT_REFERENCE", "")
if not os.path.isdir(os.path.join(REF, "xfuser")):
    raise SystemExit("set XDIT_REFERENCE to the root of an xDiT checkout (the directory that holds xfuser/)")


# --------------------------------------------------------------------------------------
# importing the reference without its heavy __init__ files
# --------------------------------------------------------------------------------------
def _seed_namespace(name: str, path: str) -> None:
    mod = types.ModuleType(name)
    mod.__path__ = [path]
    sys.modules[name] = mod


def import_reference():
    """Return (usp, attention_backend, cache_manager, runtime_state) modules of the reference."""
    if "diffusers" not in sys.modules:
        stub = types.ModuleType("diffusers")
        stub.__version__ = "0.35.2"
        stub.DiffusionPipeline = object
        sys.modules["diffusers"] = stub
    if "xfuser" not in sys.modules:
        _seed_namespace("xfuser", os.path.join(REF, "xfuser"))
        _seed_namespace("xfuser.core", os.path.join(REF, "xfuser", "core"))
        _seed_namespace("xfuser.model_executor", os.path.join(REF, "xfuser", "model_executor"))
        _seed_namespace(
            "xfuser.model_executor.layers", os.path.join(REF, "xfuser", "model_executor", "layers")
        )
    usp = importlib.import_module("xfuser.model_executor.layers.usp")
    backend = importlib.import_module("xfuser.core.distributed.attention_backend")
    cache = importlib.import_module("xfuser.core.cache_manager.cache_manager")
    rts = importlib.import_module("xfuser.core.distributed.runtime_state")
    return usp, backend, cache, rts


class _FakeRuntimeConfig:
    use_spargeattn_head_balance = False


class FakeRuntimeState:
    """The fields of the reference's runtime state that the hot path reads."""

    def __init__(self, backend):
        self.attention_backend = backend
        self.runtime_config = _FakeRuntimeConfig()
        self.num_pipeline_patch = 1
        self.patch_mode = False
        self.pipeline_patch_idx = 0
        self.pp_patches_token_start_idx_local = [0]
        self.pp_patches_token_num = []


# --------------------------------------------------------------------------------------
# USP cases
# --------------------------------------------------------------------------------------
# name, U, R, B, H, D, S_global(image), Sj(joint text), strategy, Sk_global (None => = S)
USP_CASES = [
    ("u2r1_none", 2, 1, 1, 4, 32, 96, 0, None, None),
    ("u2r1_rear", 2, 1, 1, 4, 32, 96, 24, "rear", None),
    ("u2r1_front", 2, 1, 2, 4, 32, 64, 16, "front", None),
    ("u1r2_none", 1, 2, 1, 2, 32, 96, 0, None, None),
    ("u1r2_rear", 1, 2, 1, 2, 32, 96, 24, "rear", None),
    ("u1r2_front", 1, 2, 1, 2, 32, 96, 24, "front", None),
    ("u2r2_none", 2, 2, 1, 4, 16, 128, 0, None, None),
    ("u2r2_rear", 2, 2, 1, 4, 16, 128, 20, "rear", None),
    ("u2r2_front", 2, 2, 1, 4, 16, 128, 20, "front", None),
    ("u4r1_none", 4, 1, 1, 8, 16, 64, 0, None, None),
    ("u1r4_rear", 1, 4, 1, 2, 16, 128, 12, "rear", None),
    ("u2r1_cross", 2, 1, 1, 4, 32, 64, 0, None, 160),  # Sq != Sk
    ("u1r1_rear", 1, 1, 1, 2, 32, 50, 14, "rear", None),
    ("u2r1_combined", 2, 1, 1, 4, 32, 96, 0, None, None),  # combine_qkv_a2a=True
]


def _global_inputs(name, B, H, D, S, Sj, Sk):
    seed = abs(hash_name(name)) % (2**31)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S, D, generator=g)
    k = torch.randn(B, H, Sk, D, generator=g)
    v = torch.randn(B, H, Sk, D, generator=g)
    if Sj:
        jq = torch.randn(B, H, Sj, D, generator=g)
        jk = torch.randn(B, H, Sj, D, generator=g)
        jv = torch.randn(B, H, Sj, D, generator=g)
    else:
        jq = jk = jv = None
    return q, k, v, jq, jk, jv


def hash_name(name: str) -> int:
    h = 0
    for ch in name:
        h = (h * 131 + ord(ch)) & 0x7FFFFFFF
    return h


def _cpu_flash_lse(query, key, value, dropout_p, is_causal, attention_kwargs=None):
    """An (out, lse) CPU op for ring cases: the stock LSE-returning back-ends are CUDA-only."""
    out, lse = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(
        query, key, value, dropout_p=dropout_p, is_causal=is_causal
    )
    return out, lse


def _usp_worker(rank, world, port, cases, outdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    usp, backend, _cache, _rts = import_reference()
    backend.ATTENTION_FUNCTION_REGISTRY[backend.AttentionBackendType.SDPA_FLASH] = _cpu_flash_lse

    for (name, U, R, B, H, D, S, Sj, strat, Sk) in cases:
        P = U * R
        if P != world:
            continue
        Sk = S if Sk is None else Sk
        # groups: ulysses = contiguous ranks, ring = stride U
        uly_pg = ring_pg = None
        for r in range(R):
            ranks = list(range(r * U, (r + 1) * U))
            pg = dist.new_group(ranks, backend="gloo")
            if rank in ranks:
                uly_pg = pg
        for u in range(U):
            ranks = list(range(u, P, U))
            pg = dist.new_group(ranks, backend="gloo")
            if rank in ranks:
                ring_pg = pg
        uly_rank, ring_rank = rank % U, rank // U

        class PG:
            ULYSSES_PG = uly_pg
            RING_PG = ring_pg

        usp.PROCESS_GROUP = PG
        usp.get_ulysses_parallel_world_size = lambda U=U: U
        usp.get_ulysses_parallel_rank = lambda r=uly_rank: r
        usp.get_ring_parallel_world_size = lambda R=R: R
        usp.get_sequence_parallel_world_size = lambda P=P: P
        be = backend.AttentionBackendType.SDPA if R == 1 else backend.AttentionBackendType.SDPA_FLASH
        state = FakeRuntimeState(be)
        usp.get_runtime_state = lambda state=state: state

        q, k, v, jq, jk, jv = _global_inputs(name, B, H, D, S, Sj, Sk)
        # sequence shard of this SP rank (rank order = position in the sequence)
        ql = q.chunk(P, dim=2)[rank]
        kl = k.chunk(P, dim=2)[rank]
        vl = v.chunk(P, dim=2)[rank]
        kwargs = {}
        if strat:
            kwargs = dict(joint_query=jq, joint_key=jk, joint_value=jv, joint_strategy=strat)
        if name.endswith("combined"):
            kwargs["combine_qkv_a2a"] = True
        out = usp.USP(ql, kl, vl, **kwargs)
        gathered = [torch.empty_like(out) for _ in range(P)]
        dist.all_gather(gathered, out.contiguous())
        # the same call on inputs rounded to bf16 (arithmetic still fp32): what a bf16 implementation is
        # held to, so that input rounding does not eat into the tolerance
        rb = lambda t: t.to(torch.bfloat16).to(torch.float32) if torch.is_tensor(t) else t
        out_b = usp.USP(rb(ql), rb(kl), rb(vl), **{k_: rb(v_) for k_, v_ in kwargs.items()})
        gathered_b = [torch.empty_like(out_b) for _ in range(P)]
        dist.all_gather(gathered_b, out_b.contiguous())
        if rank == 0:
            arrays = dict(
                meta=np.array([U, R, B, H, D, S, Sj, Sk], dtype=np.int64),
                strategy=np.array(strat or "none"),
                q=q.numpy(), k=k.numpy(), v=v.numpy(),
                out=np.stack([g.numpy() for g in gathered]),
                out_bf16=np.stack([g.numpy() for g in gathered_b]),
            )
            if Sj:
                arrays.update(jq=jq.numpy(), jk=jk.numpy(), jv=jv.numpy())
            np.savez_compressed(os.path.join(outdir, f"usp_{name}.npz"), **arrays)
        dist.barrier()
    dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# helper-level cases (single process): a2a re-layouts with the collective made an identity,
# exactly the way the reference's own test does it (tests/layers/usp_test.py:270-271)
# --------------------------------------------------------------------------------------
def _layout_cases(outdir):
    from unittest import mock

    usp, _backend, _cache, _rts = import_reference()
    g = torch.Generator().manual_seed(7)
    x = torch.randn(2, 4, 12, 8, generator=g)
    q = torch.randn(2, 4, 12, 8, generator=g)
    k = torch.randn(2, 4, 12, 8, generator=g)
    v = torch.randn(2, 4, 12, 8, generator=g)
    with mock.patch.object(usp, "get_ulysses_parallel_world_size", lambda: 2), mock.patch.object(
        usp, "_sdpa_all_to_all_single", lambda t: t
    ):
        in_id = usp._ft_c_input_all_to_all(x)
        out_id = usp._ft_c_output_all_to_all(x)
        cq, ck, cv = usp._combined_qkv_all_to_all(q, k, v)
    np.savez_compressed(
        os.path.join(outdir, "layout_identity_a2a.npz"),
        x=x.numpy(), in_id=in_id.numpy(), out_id=out_id.numpy(),
        q=q.numpy(), k=k.numpy(), v=v.numpy(),
        cq=cq.contiguous().numpy(), ck=ck.contiguous().numpy(), cv=cv.contiguous().numpy(),
    )


# --------------------------------------------------------------------------------------
# PipeFusion stale-KV buffer cases (single process, fake runtime state)
# --------------------------------------------------------------------------------------
def _cache_cases(outdir):
    _usp, _backend, cache, rts = import_reference()
    import xfuser.core.distributed as xdist  # namespace stub or real package

    class State:
        num_pipeline_patch = 4
        patch_mode = False
        pipeline_patch_idx = 0
        pp_patches_token_num = [6, 6, 6, 6]
        pp_patches_token_start_idx_local = [0, 6, 12, 18, 24]

    state = State()
    rts.runtime_state_is_initialized = lambda: True
    rts.get_runtime_state = lambda: state
    cache.runtime_state_is_initialized = lambda: True

    g = torch.Generator().manual_seed(11)
    B, H, D = 1, 3, 8

    # naive cache, slice_dim=2, [B,H,S,D] (how the PixArt processor calls it,
    # xfuser/model_executor/layers/attention_processor.py:286-292)
    mgr = cache.CacheManager()
    layer = "L0"
    mgr.register_cache_entry(layer, "attn", "naive_cache")
    S = 24
    k0 = torch.randn(B, H, S, D, generator=g)
    v0 = torch.randn(B, H, S, D, generator=g)
    state.patch_mode = False
    ko, vo = mgr.update_and_get_kv_cache([k0, v0], layer, slice_dim=2, layer_type="attn")
    rec = dict(k0=k0.numpy(), v0=v0.numpy(), warm_k=ko.contiguous().numpy().copy(),
               warm_v=vo.contiguous().numpy().copy())
    state.patch_mode = True
    for p in [2, 0, 3]:
        state.pipeline_patch_idx = p
        kp = torch.randn(B, H, 6, D, generator=g)
        vp = torch.randn(B, H, 6, D, generator=g)
        ko, vo = mgr.update_and_get_kv_cache([kp, vp], layer, slice_dim=2, layer_type="attn")
        rec[f"kp{p}"] = kp.numpy()
        rec[f"vp{p}"] = vp.numpy()
        rec[f"k_after{p}"] = ko.contiguous().numpy().copy()
        rec[f"v_after{p}"] = vo.contiguous().numpy().copy()
    rec["patch_order"] = np.array([2, 0, 3])
    rec["token_start"] = np.array(state.pp_patches_token_start_idx_local)
    np.savez_compressed(os.path.join(outdir, "kvcache_naive.npz"), **rec)

    # sequence-parallel cache (U=2), slice_dim=1 on [B,S,H,D] as usp.py:191-203 calls it
    import xfuser.core.distributed as xd
    U = 2
    xd.get_ulysses_parallel_world_size = lambda: U
    xd.get_runtime_state = lambda: state
    mgr = cache.CacheManager()
    mgr.register_cache_entry(layer, "attn", "sequence_parallel_attn_cache")
    state.patch_mode = False
    state.pipeline_patch_idx = 0
    Sfull = U * 24
    k0 = torch.randn(B, Sfull, H, D, generator=g)
    v0 = torch.randn(B, Sfull, H, D, generator=g)
    ko, vo = mgr.update_and_get_kv_cache([k0, v0], layer, slice_dim=1, layer_type="attn")
    rec = dict(k0=k0.numpy(), v0=v0.numpy(), warm_k=ko.contiguous().numpy().copy(),
               warm_v=vo.contiguous().numpy().copy(), U=np.array(U))
    state.patch_mode = True
    for p in [1, 3, 0]:
        state.pipeline_patch_idx = p
        kp = torch.randn(B, U * 6, H, D, generator=g)
        vp = torch.randn(B, U * 6, H, D, generator=g)
        ko, vo = mgr.update_and_get_kv_cache([kp, vp], layer, slice_dim=1, layer_type="attn")
        rec[f"kp{p}"] = kp.numpy()
        rec[f"vp{p}"] = vp.numpy()
        rec[f"k_after{p}"] = ko.contiguous().numpy().copy()
        rec[f"v_after{p}"] = vo.contiguous().numpy().copy()
    rec["patch_order"] = np.array([1, 3, 0])
    rec["token_start"] = np.array(state.pp_patches_token_start_idx_local)
    rec["token_num"] = np.array(state.pp_patches_token_num)
    np.savez_compressed(os.path.join(outdir, "kvcache_sp.npz"), **rec)


# --------------------------------------------------------------------------------------
# USP with the PipeFusion stale-KV buffer under Ulysses (usp.py:313-314 -> cache_manager.py:138-194)
# --------------------------------------------------------------------------------------
def _usp_kvcache_worker(rank, world, port, outdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    usp, backend, cache, rts = import_reference()
    import xfuser.core.distributed as xd

    U, R, B, H, D = 2, 1, 1, 4, 16
    s_loc, patches = 32, [16, 16]
    pg = dist.new_group(list(range(world)), backend="gloo")

    class PG:
        ULYSSES_PG = pg
        RING_PG = None

    usp.PROCESS_GROUP = PG
    usp.get_ulysses_parallel_world_size = lambda: U
    usp.get_ulysses_parallel_rank = lambda: rank
    usp.get_ring_parallel_world_size = lambda: R
    usp.get_sequence_parallel_world_size = lambda: U * R
    state = FakeRuntimeState(backend.AttentionBackendType.SDPA)
    state.num_pipeline_patch = len(patches)
    state.pp_patches_token_num = patches
    state.pp_patches_token_start_idx_local = [0, 16, 32]
    usp.get_runtime_state = lambda: state
    xd.get_runtime_state = lambda: state
    xd.get_ulysses_parallel_world_size = lambda: U
    cache.runtime_state_is_initialized = lambda: True
    layer = "L"
    cache.get_cache_manager().register_cache_entry(layer, "attn", "sequence_parallel_attn_cache")

    g = torch.Generator().manual_seed(1234)
    mk = lambda n: torch.randn(B, H, U * n, D, generator=g)
    q0, k0, v0 = mk(s_loc), mk(s_loc), mk(s_loc)          # warm-up step: full local sequences
    q1, k1, v1 = mk(16), mk(16), mk(16)                   # patch step: fresh rows of patch 1
    sh = lambda t: t.chunk(U, dim=2)[rank]
    state.patch_mode = False
    out0 = usp.USP(sh(q0), sh(k0), sh(v0), attn_layer=layer)
    state.patch_mode = True
    state.pipeline_patch_idx = 1
    out1 = usp.USP(sh(q1), sh(k1), sh(v1), attn_layer=layer)
    # the same two steps on inputs rounded to bf16, with a second cache entry
    rb = lambda t: t.to(torch.bfloat16).to(torch.float32)
    layer_b = "Lb"
    cache.get_cache_manager().register_cache_entry(layer_b, "attn", "sequence_parallel_attn_cache")
    state.patch_mode = False
    state.pipeline_patch_idx = 0
    out0b = usp.USP(rb(sh(q0)), rb(sh(k0)), rb(sh(v0)), attn_layer=layer_b)
    state.patch_mode = True
    state.pipeline_patch_idx = 1
    out1b = usp.USP(rb(sh(q1)), rb(sh(k1)), rb(sh(v1)), attn_layer=layer_b)
    outs = []
    for o in (out0, out1, out0b, out1b):
        gathered = [torch.empty_like(o) for _ in range(world)]
        dist.all_gather(gathered, o.contiguous())
        outs.append(np.stack([x.numpy() for x in gathered]))
    if rank == 0:
        np.savez_compressed(os.path.join(outdir, "uspkv_u2r1.npz"), q0=q0.numpy(), k0=k0.numpy(), v0=v0.numpy(),
                            q1=q1.numpy(), k1=k1.numpy(), v1=v1.numpy(), out0=outs[0], out1=outs[1],
                            out0_bf16=outs[2], out1_bf16=outs[3],
                            patches=np.array(patches), patch_idx=np.array(1), U=np.array(U))
    dist.barrier()
    dist.destroy_process_group()


def _reference_wan_rope():
    """The rotary-embedding function the reference defines inline in its Wan attention processor
    (``xfuser/model_executor/models/transformers/transformer_wan.py:108-120``), taken from the file's
    syntax tree at generation time and executed as it is (importing the module would need diffusers)."""
    import ast

    path = os.path.join(REF, "xfuser", "model_executor", "models", "transformers", "transformer_wan.py")
    src = open(path).read()
    for node in ast.walk(ast.parse(src)):
        if isinstance(node, ast.FunctionDef) and node.name == "apply_rotary_emb":
            ns = {"torch": torch}
            exec(ast.get_source_segment(src, node), ns)
            return ns["apply_rotary_emb"]
    raise RuntimeError("apply_rotary_emb not found in the reference's Wan processor")


def _prologue_cases(outdir):
    """q/k/v projections -> what the processor hands to USP (``transformer_wan.py:97-122,143-147``):
    norm_q / norm_k (``torch.nn.RMSNorm``; the module objects are built by diffusers, which is absent,
    so they are constructed here with the same arguments: full hidden size, ``elementwise_affine``),
    unflatten to heads, the reference's own rotary function, transpose to [B, H, s, D].  The second case
    applies the norm per head, as the Flux processor does (``transformer_flux.py:117-122``)."""
    rope = _reference_wan_rope()
    g = torch.Generator().manual_seed(77)
    B, s, H, D = 2, 24, 4, 16
    eps = 1e-6
    q, k, v = (torch.randn(B, s, H * D, generator=g) for _ in range(3))
    pos = torch.arange(s, dtype=torch.float32)[:, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = (pos * inv[None, :]).repeat_interleave(2, dim=1)  # [s, D], each frequency twice
    # distinct even/odd entries as well, so that which column the reference reads is pinned
    cos = torch.cos(ang) + 0.01 * torch.randn(s, D, generator=g)
    sin = torch.sin(ang) + 0.01 * torch.randn(s, D, generator=g)
    fc, fs = cos[None, :, None, :], sin[None, :, None, :]
    for name, per_head in (("prologue_wan.npz", False), ("prologue_per_head.npz", True)):
        nq = torch.nn.RMSNorm(D if per_head else H * D, eps=eps, elementwise_affine=True)
        nk = torch.nn.RMSNorm(D if per_head else H * D, eps=eps, elementwise_affine=True)
        with torch.no_grad():
            nq.weight.copy_(1.0 + 0.1 * torch.randn(nq.weight.shape, generator=g))
            nk.weight.copy_(1.0 + 0.1 * torch.randn(nk.weight.shape, generator=g))
            if per_head:
                qq, kk = nq(q.unflatten(2, (H, -1))), nk(k.unflatten(2, (H, -1)))
            else:
                qq, kk = nq(q).unflatten(2, (H, -1)), nk(k).unflatten(2, (H, -1))
            vv = v.unflatten(2, (H, -1))
            qq, kk = rope(qq, fc, fs), rope(kk, fc, fs)
            outs = [t.transpose(1, 2).contiguous().numpy() for t in (qq, kk, vv)]
            # the same modules and the same rotary function run in bf16, the way the reference runs them in
            # a bf16 pipeline (16-bit activations and weights, fp32 cos/sin tables): pins where they round
            bf = torch.bfloat16
            import copy

            nq16, nk16 = copy.deepcopy(nq).to(bf), copy.deepcopy(nk).to(bf)
            q16, k16 = q.to(bf), k.to(bf)
            if per_head:
                qq16, kk16 = nq16(q16.unflatten(2, (H, -1))), nk16(k16.unflatten(2, (H, -1)))
            else:
                qq16, kk16 = nq16(q16).unflatten(2, (H, -1)), nk16(k16).unflatten(2, (H, -1))
            qq16, kk16 = rope(qq16, fc, fs), rope(kk16, fc, fs)
            assert qq16.dtype == bf
            outs16 = [t.transpose(1, 2).contiguous().float().numpy() for t in (qq16, kk16)]
        np.savez_compressed(os.path.join(outdir, name), q=q.numpy(), k=k.numpy(), v=v.numpy(), cos=cos.numpy(),
                            sin=sin.numpy(), wq=nq.weight.detach().numpy(), wk=nk.weight.detach().numpy(),
                            eps=np.array(eps), heads=np.array(H), per_head=np.array(int(per_head)),
                            q_out=outs[0], k_out=outs[1], v_out=outs[2], q_out_bf16=outs16[0], k_out_bf16=outs16[1])


def _reference_wan_methods(names):
    """Methods of the reference's Wan wrapper taken from the file's syntax tree (importing the module
    would need diffusers): ``xfuser/model_executor/models/transformers/transformer_wan.py:219-239``."""
    import ast

    path = os.path.join(REF, "xfuser", "model_executor", "models", "transformers", "transformer_wan.py")
    src = open(path).read()
    found = {}
    for node in ast.walk(ast.parse(src)):
        if isinstance(node, ast.FunctionDef) and node.name in names:
            found[node.name] = ast.get_source_segment(src, node)
    assert set(found) == set(names), found.keys()
    return found


def _boundary_worker(rank, world, port, outdir):
    """Model-boundary sharding as the reference does it: ``_chunk_and_pad_sequence`` at entry,
    ``_gather_and_unpad`` at exit on top of the real ``GroupCoordinator.all_gather`` (gloo ranks)."""
    import functools
    import textwrap
    import types as _types

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import_reference()
    gc = importlib.import_module("xfuser.core.distributed.group_coordinator")
    fake_group = _types.SimpleNamespace(world_size=world, device_group=dist.group.WORLD)
    fake_group.all_gather = functools.partial(gc.GroupCoordinator.all_gather, fake_group)
    srcs = _reference_wan_methods(["_chunk_and_pad_sequence", "_gather_and_unpad"])
    ns = {"torch": torch, "get_sp_group": lambda: fake_group}
    for body in srcs.values():
        exec(textwrap.dedent(body), ns)
    chunk_pad, gather_unpad = ns["_chunk_and_pad_sequence"], ns["_gather_and_unpad"]
    g = torch.Generator().manual_seed(99)
    rec = {}
    for name, shape, dim in (("a", (2, 10, 6), 1), ("b", (1, 13, 8), -2), ("c", (2, 3, 9, 4), 2), ("d", (1, 8, 16), 1)):
        x = torch.randn(*shape, generator=g)
        n = shape[dim]
        pad = (world - n % world) % world
        local = chunk_pad(None, x, rank, world, pad, dim)
        back = gather_unpad(None, local.contiguous() * 1.0, pad, dim)
        locs = [torch.empty_like(local.contiguous()) for _ in range(world)]
        dist.all_gather(locs, local.contiguous())
        if rank == 0:
            rec[f"{name}_x"] = x.numpy()
            rec[f"{name}_dim"] = np.array(dim)
            rec[f"{name}_pad"] = np.array(pad)
            rec[f"{name}_chunks"] = np.stack([t.numpy() for t in locs])
            rec[f"{name}_gathered"] = back.contiguous().numpy()
    if rank == 0:
        rec["world"] = np.array(world)
        rec["names"] = np.array(["a", "b", "c", "d"])
        np.savez_compressed(os.path.join(outdir, f"boundary_w{world}.npz"), **rec)
    dist.barrier()
    dist.destroy_process_group()


def main():
    outdir = HERE
    if "--prologue-only" in sys.argv:
        _prologue_cases(outdir)
        return
    if "--boundary-only" in sys.argv:
        mp.spawn(_boundary_worker, args=(4, 29631, outdir), nprocs=4, join=True)
        return
    port = 29611
    for world in (1, 2, 4):
        cases = [c for c in USP_CASES if c[1] * c[2] == world]
        if not cases:
            continue
        mp.spawn(_usp_worker, args=(world, port, cases, outdir), nprocs=world, join=True)
        port += 1
    mp.spawn(_usp_kvcache_worker, args=(2, port, outdir), nprocs=2, join=True)
    _layout_cases(outdir)
    _cache_cases(outdir)
    _prologue_cases(outdir)
    mp.spawn(_boundary_worker, args=(4, port + 1, outdir), nprocs=4, join=True)
    print("golden fixtures written to", outdir)


if __name__ == "__main__":
    main()
