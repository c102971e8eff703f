"""Model-boundary sharding (zero-pad + shard at entry, gather + unpad at exit).

CPU: the host logic of ``xdit_b200.model_boundary`` under 4 gloo ranks with the kernels replaced by the
oracle-backed stand-ins, against the fixture produced by the reference's own functions.
GPU: the two kernels behind it, bit-exact against the oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from oracle import usp_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _worker(rank, world, port, errq):
    try:
        import sys

        sys.path.insert(0, ROOT)
        import torch.distributed as dist

        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from tests import fake_ops

        fake_ops.install()
        from xdit_b200 import model_boundary as mb

        z = np.load(os.path.join(HERE, "golden", f"boundary_w{world}.npz"))
        for name in z["names"]:
            x = torch.from_numpy(z[f"{name}_x"])
            dim, pad = int(z[f"{name}_dim"]), int(z[f"{name}_pad"])
            local, got_pad = mb.shard_sequence(x, dim=dim, rank=rank, world=world)
            assert got_pad == pad == mb.pad_amount(x.shape[dim], world)
            assert torch.equal(local, torch.from_numpy(z[f"{name}_chunks"][rank])), (name, rank)
            back = mb.gather_sequence(local, dim=dim, pad=pad, world=world)
            assert torch.equal(back, torch.from_numpy(z[f"{name}_gathered"])), (name, rank)
        # CFG gather along the batch axis: branch r holds value r
        y = torch.full((1, 5, 3), float(rank))
        full = mb.gather_cfg(y, None, world)
        assert full.shape == (world, 5, 3) and all(float(full[r, 0, 0]) == r for r in range(world))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # surface the failure in the parent
        import traceback

        errq.put(f"rank {rank}: {e}\n{traceback.format_exc()}")
        raise


def test_shard_and_gather_under_four_gloo_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 4, 29655, errq)) for r in range(4)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    assert not msgs and all(p.exitcode == 0 for p in procs), "\n".join(msgs)


def test_single_rank_is_a_view():
    from xdit_b200 import model_boundary as mb

    x = torch.randn(2, 7, 4)
    local, pad = mb.shard_sequence(x, dim=1, rank=0, world=1)
    assert local is x and pad == 0
    assert mb.gather_sequence(x, dim=1, pad=0, world=1) is x


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,S,C,W", [(1, 75600, 64, 8), (2, 4099, 3072, 8), (2, 10, 6, 4), (3, 1, 5, 2), (1, 4608, 64, 3)])
def test_shard_and_gather_kernels_bit_exact(dtype, B, S, C, W):
    """Wan (latent channels 64 after proj_out: 75,600 tokens), Flux-like with an odd length, and tiny
    ragged cases; every rank's shard and the gathered, unpadded tensor must equal the oracle's bit for bit."""
    from xdit_b200 import ops

    g = torch.Generator().manual_seed(B * 1000 + S)
    x = torch.randn(B, S, C, generator=g).to(dtype).cuda()
    xn = x.float().cpu().numpy()
    chunks, pad = O.pad_and_shard_sequence(xn, W, dim=1)
    s = chunks[0].shape[1]
    locals_ = []
    for r in range(W):
        got = ops.seq_shard_pad(x, r, W)
        assert got.shape == (B, s, C)
        assert np.array_equal(got.float().cpu().numpy(), chunks[r]), (r, "shard")
        locals_.append(got)
    # a strided source (a column slice of a wider tensor) gives the same rows
    wide = torch.randn(B, S, C + 8, generator=g).to(dtype).cuda()
    got = ops.seq_shard_pad(wide[:, :, :C], W - 1, W)
    want, _ = O.pad_and_shard_sequence(wide[:, :, :C].float().cpu().numpy(), W, dim=1)
    assert np.array_equal(got.float().cpu().numpy(), want[W - 1])
    recv = torch.stack(locals_)  # [W][B][s][C], what all_gather_into_tensor leaves
    back = ops.seq_gather_unpad(recv, B, s, C, W, W * s - pad)
    torch.cuda.synchronize()
    assert torch.equal(back, x)
    assert np.array_equal(back.float().cpu().numpy(), O.gather_and_unpad(chunks, pad, dim=1))


@pytest.mark.gpu
def test_boundary_rejects_bad_arguments():
    from xdit_b200 import _capi, ops

    x = torch.zeros(1, 8, 4, device="cuda")
    with pytest.raises(_capi.XditError):
        ops.seq_shard_pad(x, 4, 4)  # rank out of range
    with pytest.raises(_capi.XditError):
        ops.seq_gather_unpad(torch.zeros(2, 1, 4, 4, device="cuda"), 1, 4, 4, 2, 9)  # keeps more rows than exist
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.seq_shard_pad(x.cpu(), 0, 2)
