"""Host-side orchestration of xdit_b200 (send-buffer layouts, strided receive views, all-to-all
and ring schedules, KV-cache bookkeeping) under gloo ranks on CPU.  The device kernels are
replaced by the oracle-backed stand-ins of tests/fake_ops.py, so what is checked here is the
Python logic only; the kernels themselves are checked on the GPU (tests marked gpu)."""
import glob
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
USP_FILES = sorted(glob.glob(os.path.join(HERE, "golden", "usp_*.npz")))


def _worker(rank, world, port, files, mode, errq):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.set_num_threads(1)
        import xdit_b200
        from tests import fake_ops

        fake_ops.install()
        for path in files:
            z = np.load(path)
            U, R, B, H, D, S, Sj, Sk = [int(x) for x in z["meta"]]
            strat = str(z["strategy"])
            strat = None if strat == "none" else strat
            P = U * R
            xdit_b200.init_sequence_parallel(U, R, backend="gloo")
            q, k, v = (torch.from_numpy(z[n]) for n in ("q", "k", "v"))
            ql, kl, vl = (t.chunk(P, dim=2)[rank] for t in (q, k, v))
            kw = {}
            if strat:
                kw = dict(joint_query=torch.from_numpy(z["jq"]), joint_key=torch.from_numpy(z["jk"]),
                          joint_value=torch.from_numpy(z["jv"]), joint_strategy=strat)
            if mode == "usp":
                # pass transposed views, as the DiT processors do (transformer_flux.py:170-172)
                ql, kl, vl = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (ql, kl, vl))
                out = xdit_b200.USP(ql, kl, vl, **kw)
            elif mode == "compat":
                from xdit_b200.attention_backend import AttentionBackendType, register_attention_function

                @register_attention_function(AttentionBackendType.SAGE)
                def _custom(query, key, value, dropout_p, is_causal, attention_kwargs=None):
                    return fake_ops.attn_fwd(query, key, value, want_lse=True)

                out = xdit_b200.USP(ql, kl, vl, backend=AttentionBackendType.SAGE, combine_qkv_a2a=True, **kw)
            else:  # legacy [B,S,H,D] layer
                layer = xdit_b200.xFuserLongContextAttention()
                t = lambda x: x.transpose(1, 2)
                kw2 = {}
                if strat:
                    kw2 = dict(joint_tensor_query=t(kw["joint_query"]), joint_tensor_key=t(kw["joint_key"]),
                               joint_tensor_value=t(kw["joint_value"]), joint_strategy=strat)
                out = t(layer(None, t(ql), t(kl), t(vl), **kw2))
            ref = torch.from_numpy(z["out"][rank])
            assert out.shape == ref.shape, (path, out.shape, ref.shape)
            err = (out.double() - ref.double()).abs().max().item()
            assert err < 5e-5, (os.path.basename(path), mode, rank, err)
            dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # surface the failure in the parent
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def _run(world, files, mode, port):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, files, mode, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def _files(world):
    out = []
    for f in USP_FILES:
        m = np.load(f)["meta"]
        if int(m[0]) * int(m[1]) == world:
            out.append(f)
    return out


@pytest.mark.parametrize("mode", ["usp", "legacy", "compat"])
def test_world2_matches_reference(mode):
    _run(2, _files(2), mode, 29720 + ["usp", "legacy", "compat"].index(mode))


@pytest.mark.parametrize("mode", ["usp", "legacy"])
def test_world4_matches_reference(mode):
    _run(4, _files(4), mode, 29730 + ["usp", "legacy"].index(mode))
