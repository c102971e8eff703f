"""Per-rank body shared by the gloo (CPU, stand-in kernels) and NCCL (GPU, real kernels) USP tests:
replays the golden fixtures produced by the unmodified reference through xdit_b200."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def worker(rank, world, port, files, mode, errq, backend="gloo", dtype_name="float32", tol=5e-5):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        gpu = backend == "nccl"
        if gpu:
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
            torch.set_num_threads(1)
        import xdit_b200

        if gpu:
            from xdit_b200 import ops
        else:
            from tests import fake_ops

            fake_ops.install()
        dtype = getattr(torch, dtype_name)
        dev = torch.device("cuda", rank) if gpu else torch.device("cpu")
        put = lambda a: torch.from_numpy(a).to(dtype).to(dev)
        for path in files:
            z = np.load(path)
            U, R, B, H, D, S, Sj, Sk = [int(x) for x in z["meta"]]
            strat = str(z["strategy"])
            strat = None if strat == "none" else strat
            P = U * R
            xdit_b200.init_sequence_parallel(U, R, backend=backend)
            q, k, v = (put(z[n]) for n in ("q", "k", "v"))
            ql, kl, vl = (t.chunk(P, dim=2)[rank] for t in (q, k, v))
            kw = {}
            if strat:
                kw = dict(joint_query=put(z["jq"]), joint_key=put(z["jk"]), joint_value=put(z["jv"]),
                          joint_strategy=strat)
            if mode == "usp_peer":
                # both Ulysses exchanges by direct stores into the peers' buffers (CUDA IPC mappings); ring
                # fixtures rotate K/V by copy-engine transfers into the next rank's buffer
                from xdit_b200 import peer_exchange

                peer_exchange.enable(True)
                ql, kl, vl = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (ql, kl, vl))
                out = xdit_b200.USP(ql, kl, vl, **kw)
                out2 = xdit_b200.USP(ql, kl, vl, **kw)  # second call: other result slot, same receive buffer
                assert torch.equal(out, out2)
                if R > 1:
                    assert peer_exchange._exchanges, "the ring did not go through the peer buffers"
                peer_exchange.enable(False)
                out = out.clone()  # the result is a view of a peer buffer, which goes away next
                del out2
                peer_exchange.close_all()  # every rank: the buffers of this fixture's groups are released
            elif mode == "usp_pipelined":
                # the same call with the head-group pipeline forced on (it is size-gated in production)
                import xdit_b200.usp as _usp_mod

                _usp_mod.PIPELINE_MIN_BYTES = 0
                ql, kl, vl = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (ql, kl, vl))
                out = xdit_b200.USP(ql, kl, vl, **kw)
            elif mode == "usp":
                # transposed views, as the DiT processors pass them (transformer_flux.py:170-172)
                ql, kl, vl = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (ql, kl, vl))
                out = xdit_b200.USP(ql, kl, vl, **kw)
            elif mode == "compat":
                from xdit_b200.attention_backend import AttentionBackendType, register_attention_function

                if gpu:
                    from xdit_b200 import ops as _ops

                    def _custom(query, key, value, dropout_p, is_causal, attention_kwargs=None):
                        return _ops.attn_fwd(query, key, value, want_lse=True, force_generic=True)
                else:
                    def _custom(query, key, value, dropout_p, is_causal, attention_kwargs=None):
                        return fake_ops.attn_fwd(query, key, value, want_lse=True)

                register_attention_function(AttentionBackendType.SAGE)(_custom)
                out = xdit_b200.USP(ql, kl, vl, backend=AttentionBackendType.SAGE, combine_qkv_a2a=True, **kw)
            elif mode == "yunchang":
                out = _yunchang_shaped_forward(xdit_b200, ql, kl, vl, kw, strat, rank, U, R, dev)
            elif mode == "ref_layer":
                # the reference's OWN hybrid/attn_layer.py and ring/ring_flash_attn.py, unmodified, running on
                # the yunchang-shaped names this package serves (SeqAllToAll4D, RingComm, update_out_and_lse,
                # select_flash_attn_impl, RingFlashAttnFunc, LongContextAttention)
                from oracle import ref_import
                from xdit_b200 import yunchang_compat

                assert yunchang_compat.install()
                layer_mod, _ring_mod = ref_import.import_long_ctx_attention()
                assert layer_mod.__file__.startswith(ref_import.root())
                t = lambda x: x.transpose(1, 2)
                pack = not strat and ql.shape == kl.shape
                layer = layer_mod.xFuserLongContextAttention(use_pack_qkv=pack)
                assert layer.ring_pg is xdit_b200.PROCESS_GROUP.RING_PG
                assert layer.ulysses_pg is xdit_b200.PROCESS_GROUP.ULYSSES_PG
                kw2 = {}
                if strat:
                    kw2 = dict(joint_tensor_query=t(kw["joint_query"]), joint_tensor_key=t(kw["joint_key"]),
                               joint_tensor_value=t(kw["joint_value"]), joint_strategy=strat)
                out = t(layer(None, t(ql).contiguous(), t(kl).contiguous(), t(vl).contiguous(), **kw2))
            else:  # legacy [B,S,H,D] layer
                layer = xdit_b200.xFuserLongContextAttention()
                t = lambda x: x.transpose(1, 2)
                kw2 = {}
                if strat:
                    kw2 = dict(joint_tensor_query=t(kw["joint_query"]), joint_tensor_key=t(kw["joint_key"]),
                               joint_tensor_value=t(kw["joint_value"]), joint_strategy=strat)
                out = t(layer(None, t(ql), t(kl), t(vl), **kw2))
            if gpu:
                torch.cuda.synchronize()
                ops.check_status()
            # a bf16 run is held to what the reference returns for the same bf16-rounded inputs
            ref = torch.from_numpy(z["out_bf16" if dtype == torch.bfloat16 else "out"][rank]).double()
            assert tuple(out.shape) == tuple(ref.shape), (path, out.shape, ref.shape)
            got = out.detach().double().cpu()
            assert torch.isfinite(got).all(), (os.path.basename(path), mode, rank, "non-finite")
            err = (got - ref).abs().max().item()
            assert err < tol, (os.path.basename(path), mode, rank, err)
            cos = float((got * ref).sum() / (got.norm() * ref.norm() + 1e-30))
            assert cos >= 0.9999, (os.path.basename(path), mode, rank, "cosine", cos)
            dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # surface the failure in the parent
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def _yunchang_shaped_forward(xdit_b200, ql, kl, vl, kw, strat, rank, U, R, dev):
    """The [B,S,H,D] layer's forward spelled with the yunchang-named pieces, in the order of the
    reference's ``hybrid/attn_layer.py:136-236``: joint-Q concat, joint K/V head slice, SeqAllToAll4D
    (heads scattered, sequence gathered), ring function, inverse SeqAllToAll4D.  Also sends a token
    around the ring with RingComm and, without joint tensors, runs the shim's LongContextAttention."""
    from xdit_b200 import yunchang_compat

    assert yunchang_compat.install()
    from yunchang import LongContextAttention
    from yunchang.comm.all_to_all import SeqAllToAll4D
    from yunchang.globals import PROCESS_GROUP
    from yunchang.ring.utils import RingComm

    t = lambda x: x.transpose(1, 2)
    q, k, v = t(ql), t(kl), t(vl)
    u_rank = rank % U
    jk = jv = None
    if strat:
        jq, jk, jv = (t(kw[n]) for n in ("joint_query", "joint_key", "joint_value"))
        q = torch.cat([q, jq], 1) if strat == "rear" else torch.cat([jq, q], 1)
        hl = jk.shape[2] // U
        jk, jv = jk[:, :, u_rank * hl:(u_rank + 1) * hl], jv[:, :, u_rank * hl:(u_rank + 1) * hl]
    q2, k2, v2 = (SeqAllToAll4D.apply(PROCESS_GROUP.ULYSSES_PG, x, 2, 1) for x in (q, k, v))
    ctx = xdit_b200.xdit_ring_flash_attn_func(
        q2, k2, v2, group=PROCESS_GROUP.RING_PG, joint_tensor_key=jk, joint_tensor_value=jv,
        joint_strategy=strat or "none")
    out = t(SeqAllToAll4D.apply(PROCESS_GROUP.ULYSSES_PG, ctx, 1, 2))
    if R > 1:
        comm = RingComm(PROCESS_GROUP.RING_PG)
        token = torch.full((4,), float(rank), device=dev)
        got = comm.send_recv(token)
        comm.commit()
        comm.wait()
        prev = ((rank // U - 1) % R) * U + u_rank
        assert torch.equal(got.cpu(), torch.full((4,), float(prev))), (rank, got)
    if not strat:
        out_layer = t(LongContextAttention()(t(ql), t(kl), t(vl)))
        assert (out_layer.double() - out.double()).abs().max().item() < 1e-2
    return out


def flux_joint_worker(rank, world, port, errq, backend="gloo", dtype_name="float32", tol=5e-5):
    """USP at the Flux-shaped joint case at full size: Ulysses 2, B=1, 24 heads x 128, 4096 image tokens
    sharded + 512 text tokens replicated (joint, rear), N(0,1) from seed 0, softmax scale 128^-1/2.  Every
    rank's rows ``[image shard ; text]`` of two heads of each peer's head block are compared with the
    oracle's dense attention (float64) over all 4608 keys."""
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        gpu = backend == "nccl"
        if gpu:
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
            torch.set_num_threads(4)
        import xdit_b200
        from oracle import usp_oracle as O

        if not gpu:
            from tests import fake_ops

            fake_ops.install()
            fake_ops.FAST_FP32 = True
        dtype = getattr(torch, dtype_name)
        dev = torch.device("cuda", rank) if gpu else torch.device("cpu")
        xdit_b200.init_sequence_parallel(world, 1, backend=backend)
        B, H, D, S, Sj = 1, 24, 128, 4096, 512
        g = torch.Generator().manual_seed(0)
        q, k, v = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
        jq, jk, jv = (torch.randn(B, H, Sj, D, generator=g) for _ in range(3))
        cast = lambda t: t.to(dtype)
        put = lambda t: cast(t).to(dev)
        sh = lambda t: put(t.chunk(world, dim=2)[rank])
        out = xdit_b200.USP(sh(q), sh(k), sh(v), joint_query=put(jq), joint_key=put(jk), joint_value=put(jv),
                            joint_strategy="rear")
        if gpu:
            torch.cuda.synchronize()
            from xdit_b200 import ops

            ops.check_status()
        s = S // world
        assert tuple(out.shape) == (B, H, s + Sj, D)
        heads = [0, H // world - 1, H // world, H - 1]  # first and last head of each peer's block
        n64 = lambda t: cast(t).double().numpy()
        qrows = torch.cat([q.chunk(world, dim=2)[rank], jq], dim=2)
        want, _ = O.attention_dense(n64(qrows[:, heads]), n64(torch.cat([k, jk], 2)[:, heads]),
                                    n64(torch.cat([v, jv], 2)[:, heads]))
        got = out[:, heads].double().cpu().numpy()
        err = float(np.abs(got - want).max())
        cos = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
        assert err < tol and cos >= 0.9999, ("flux joint case", rank, err, cos)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def run_flux_joint(world, port, **kw):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=flux_joint_worker, args=(r, world, port, errq), kwargs=kw) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errs.append("a rank did not finish")
    assert not errs and all(p.exitcode == 0 for p in procs), "\n".join(errs)


def prologue_worker(rank, world, port, U, R, errq, backend="gloo", dtype_name="float32", tol=5e-5):
    """attention_from_projections under U x R ranks against the oracle: prologue on the global
    projections, dense attention, rows of this rank."""
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        gpu = backend == "nccl"
        if gpu:
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
            torch.set_num_threads(1)
        import xdit_b200
        from oracle import usp_oracle as O
        from xdit_b200.prologue import attention_from_projections

        if not gpu:
            from tests import fake_ops

            fake_ops.install()
        dtype = getattr(torch, dtype_name)
        dev = torch.device("cuda", rank) if gpu else torch.device("cpu")
        xdit_b200.init_sequence_parallel(U, R, backend=backend)
        B, S, H, D = 1, 64 * world, 4, 32
        g = torch.Generator().manual_seed(5)
        q, k, v = (torch.randn(B, S, H * D, generator=g).to(dtype) for _ in range(3))
        wq, wk = (1 + 0.1 * torch.randn(H * D, generator=g)).to(dtype), (1 + 0.1 * torch.randn(H * D, generator=g)).to(dtype)
        ang = torch.rand(S, D // 2, generator=g) * 6.28
        cos, sin = torch.cos(ang).repeat_interleave(2, 1), torch.sin(ang).repeat_interleave(2, 1)
        for per_head in (False, True):
            w_q, w_k = (wq[:D].contiguous(), wk[:D].contiguous()) if per_head else (wq, wk)
            n64 = lambda t: t.double().numpy()
            qs, ks, vs = O.attention_prologue(n64(q), n64(k), n64(v), H, n64(w_q), n64(w_k), 1e-6, per_head,
                                              n64(cos), n64(sin), 1)
            want, _ = O.attention_dense(*(x[0].transpose(1, 0, 2, 3) for x in (qs, ks, vs)))  # [B,H,S,D]
            want = want.transpose(0, 2, 1, 3).reshape(B, S, H * D)
            sl = slice(rank * (S // world), (rank + 1) * (S // world))
            put = lambda t: t.to(dev)
            got = attention_from_projections(
                put(q[:, sl]), put(k[:, sl]), put(v[:, sl]), H, norm_q_weight=put(w_q), norm_k_weight=put(w_k),
                eps=1e-6, norm_per_head=per_head, rotary_emb=(put(cos[sl])[None, :, None, :], put(sin[sl])[None, :, None, :]))
            if gpu:
                torch.cuda.synchronize()
                from xdit_b200 import ops

                ops.check_status()
            assert tuple(got.shape) == (B, S // world, H * D)
            err = (got.double().cpu() - torch.from_numpy(want[:, sl])).abs().max().item()
            assert err < tol, ("prologue", U, R, per_head, rank, err)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def run_prologue(world, U, R, port, **kw):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=prologue_worker, args=(r, world, port, U, R, errq), kwargs=kw) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errs.append("a rank did not finish")
    assert not errs and all(p.exitcode == 0 for p in procs), "\n".join(errs)


def kv_worker(rank, world, port, path, errq, backend="gloo", dtype_name="float32", tol=5e-5):
    """USP with the PipeFusion stale-KV buffer under Ulysses: warm-up step, then a patch step."""
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        gpu = backend == "nccl"
        if gpu:
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
            torch.set_num_threads(1)
        import xdit_b200

        if not gpu:
            from tests import fake_ops

            fake_ops.install()
        z = np.load(path)
        U = int(z["U"])
        dtype = getattr(torch, dtype_name)
        dev = torch.device("cuda", rank) if gpu else torch.device("cpu")
        put = lambda a: torch.from_numpy(a).to(dtype).to(dev).chunk(U, dim=2)[rank]
        xdit_b200.init_sequence_parallel(U, 1, backend=backend)
        rs = xdit_b200.initialize_runtime_state()
        rs.set_patches([int(x) for x in z["patches"]])
        layer = "L"
        xdit_b200.get_cache_manager().register_cache_entry(layer, "attn", "sequence_parallel_attn_cache")
        rs.set_patched_mode(False)
        out0 = xdit_b200.USP(put(z["q0"]), put(z["k0"]), put(z["v0"]), attn_layer=layer)
        rs.set_patched_mode(True)
        rs.pipeline_patch_idx = int(z["patch_idx"])
        out1 = xdit_b200.USP(put(z["q1"]), put(z["k1"]), put(z["v1"]), attn_layer=layer)
        if gpu:
            torch.cuda.synchronize()
            from xdit_b200 import ops

            ops.check_status()
        sfx = "_bf16" if dtype == torch.bfloat16 else ""
        for got, name in ((out0, "out0" + sfx), (out1, "out1" + sfx)):
            ref = torch.from_numpy(z[name][rank]).double()
            assert tuple(got.shape) == tuple(ref.shape), (name, got.shape, ref.shape)
            err = (got.detach().double().cpu() - ref).abs().max().item()
            assert err < tol, (name, rank, err)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def run_kv(world, path, port, **kw):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=kv_worker, args=(r, world, port, path, errq), kwargs=kw) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    assert not msgs, "\n".join(msgs)
    assert not alive, "ranks did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def run(world, files, mode, port, **kw):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=worker, args=(r, world, port, files, mode, errq), kwargs=kw) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    assert not msgs, "\n".join(msgs)
    assert not alive, "ranks did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]



def peer_growth_worker(rank, world, port, errq):
    """The peer buffers of one process group are re-allocated (collectively) when a later call needs more
    room; results of the small and the large call must equal the NCCL path's before and after the growth,
    for the Ulysses exchange by stores and for the ring rotation through peer slots."""
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.set_num_threads(1)
        import xdit_b200
        from tests import fake_ops
        from xdit_b200 import peer_exchange

        fake_ops.install()
        for U, R in ((world, 1), (1, world)):
            xdit_b200.init_sequence_parallel(U, R, backend="gloo")
            g = torch.Generator().manual_seed(5)
            data = {}
            for S in (64, 256):
                q, k, v = (torch.randn(1, 4, S, 16, generator=g).to(torch.bfloat16) for _ in range(3))
                data[S] = tuple(t.chunk(world, dim=2)[rank].contiguous() for t in (q, k, v))
            want = {S: xdit_b200.USP(*data[S]).clone() for S in data}
            peer_exchange.enable(True)
            sizes = []
            for S in (64, 256, 64, 256):  # the second call grows the buffers, the third runs in the grown ones
                got = xdit_b200.USP(*data[S]).clone()
                assert peer_exchange._exchanges, "the call did not go through the peer buffers"
                sizes.append(max(ex.out_bytes for ex in peer_exchange._exchanges.values()))
                err = float((got.float() - want[S].float()).abs().max())
                assert err <= 2e-2, (U, R, S, err)
            assert sizes[1] > sizes[0] and sizes[2] == sizes[1] == sizes[3], sizes
            peer_exchange.enable(False)
            peer_exchange.close_all()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def run_peer_growth(world, port):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=peer_growth_worker, args=(r, world, port, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    assert not msgs, "\n".join(msgs)
    assert not alive, "ranks did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]

def golden_files(world):
    import glob

    out = []
    for f in sorted(glob.glob(os.path.join(HERE, "golden", "usp_*.npz"))):
        m = np.load(f)["meta"]
        if int(m[0]) * int(m[1]) == world:
            out.append(f)
    return out
