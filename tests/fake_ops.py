"""CPU stand-ins for ``xdit_b200.ops`` used ONLY by host-logic tests: they let the Python
orchestration (buffer layouts, strided views, all-to-all and ring schedules) run under gloo on
a machine without a GPU.  The arithmetic comes from the oracle.  Never imported by the package."""
import numpy as np
import torch

from oracle import usp_oracle as O


def _flat4(x):
    if x is None:
        return None
    if x.dim() == 5:
        B, H, G, L, D = x.shape
        return x.reshape(B, H, G * L, D)
    return x


def _np(x):
    return x.detach().to(torch.float64).numpy()


FAST_FP32 = False  # large shapes: torch's fp32 CPU attention instead of the float64 numpy one


def attn_fwd(q, k, v, k2=None, v2=None, *, out=None, lse=None, o_acc=None, lse_acc=None, acc_in=False,
             acc_out=False, causal=False, scale=None, force_generic=False, want_lse=False, out_segments=None,
             out_strides=None, **_):
    q4, k4, v4 = _flat4(q), _flat4(k), _flat4(v)
    if k2 is not None:
        k4 = torch.cat([k4, k2], dim=2)
        v4 = torch.cat([v4, v2], dim=2)
    if FAST_FP32 and not causal and scale is None:
        o, l = torch.ops.aten._scaled_dot_product_flash_attention_for_cpu(q4.float(), k4.float(), v4.float())
        o, l = o.double().numpy(), l.double().numpy()
    else:
        o, l = O.attention_dense(_np(q4), _np(k4), _np(v4), scale=scale, causal=causal)
    if acc_in:
        o, l = O.merge_out_lse(_np(o_acc), _np(lse_acc), o, l)
    if acc_out:
        o_acc.copy_(torch.from_numpy(o).to(o_acc.dtype))
        lse_acc.copy_(torch.from_numpy(l).to(lse_acc.dtype))
        return out, lse
    if out_segments is not None:
        # rows of query segment g go to the address out_segments[g] (a mapped peer buffer), laid out with the
        # given (batch, head, row) element strides
        B, H, G, L, D = q.shape if q.dim() == 5 else (q.shape[0], q.shape[1], 1, q.shape[2], q.shape[3])
        res = torch.from_numpy(o).to(q.dtype).reshape(B, H, G, L, D)
        es = q.element_size()
        for g in range(G):
            t, off = _find(int(out_segments[g]))
            typed = t[off:off + (t.numel() - off) // es * es].view(q.dtype)
            typed.as_strided((B, H, L, D), (*[int(x) for x in out_strides], 1)).copy_(res[:, :, g])
        return None, lse
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype)
    out.copy_(torch.from_numpy(o).to(q.dtype).reshape(out.shape))
    if lse is None and want_lse:
        lse = torch.empty(q4.shape[:3], dtype=torch.float32)
    if lse is not None:
        lse.copy_(torch.from_numpy(l).to(torch.float32))
    return out, lse


def ulysses_pack(items, U, head_group=None):
    g, G = head_group if head_group is not None else (0, 1)
    for it in items:
        src, joint, dst, stride = it["src"], it.get("joint"), it["dst"], it["peer_stride"]
        x = src
        if joint is not None:
            x = torch.cat([joint, src], 2) if it.get("front") else torch.cat([src, joint], 2)
        B, H, rows, D = x.shape
        Hl = H // U
        Hg = Hl // G
        blk = Hg * B * rows * D
        for p in range(U):
            part = x[:, p * Hl + g * Hg:p * Hl + (g + 1) * Hg].permute(1, 0, 2, 3).reshape(-1)
            dst[p * stride:p * stride + blk].copy_(part)


def ulysses_pack_peers(items, U, peer_base):
    """The pack with peer p's block stored at the address peer_base[p] + dst_offset elements."""
    for it in items:
        src, joint, off = it["src"], it.get("joint"), int(it["dst_offset"])
        x = src
        if joint is not None:
            x = torch.cat([joint, src], 2) if it.get("front") else torch.cat([src, joint], 2)
        B, H, rows, D = x.shape
        Hl = H // U
        es = x.element_size()
        for p in range(U):
            part = x[:, p * Hl:(p + 1) * Hl].permute(1, 0, 2, 3).reshape(-1).contiguous()
            t, boff = _find(int(peer_base[p]) + off * es)
            t[boff:boff + part.numel() * es].copy_(part.view(torch.uint8))


def ulysses_unpack_in(recv, B, Hl, s, D, U):
    return recv.reshape(U, Hl, B, s, D).permute(2, 1, 0, 3, 4).reshape(B, Hl, U * s, D).contiguous()


def ulysses_pack_out(x):
    return x.permute(2, 0, 1, 3).contiguous()


def ulysses_unpack_out(recv, B, Hl, s, D, U):
    return recv.reshape(U, s, B, Hl, D).permute(2, 0, 3, 1, 4).reshape(B, U * Hl, s, D).contiguous()


def kv_patch_update(k_cache, v_cache, k_new, v_new, row_start):
    kn, vn = _flat4(k_new), _flat4(v_new)
    n = kn.shape[2]
    if row_start < 0 or row_start + n > k_cache.shape[2]:
        raise RuntimeError("rows outside the cache")
    k_cache[:, :, row_start:row_start + n] = kn
    v_cache[:, :, row_start:row_start + n] = vn


def merge_out_lse(o_acc, lse_acc, out_b, lse_b, first, out_final=None):
    if first:
        o, l = _np(out_b), _np(lse_b)
    else:
        o, l = O.merge_out_lse(_np(o_acc), _np(lse_acc), _np(out_b), _np(lse_b))
    o_acc.copy_(torch.from_numpy(np.asarray(o)).to(o_acc.dtype))
    lse_acc.copy_(torch.from_numpy(np.asarray(l)).to(lse_acc.dtype))
    if out_final is not None:
        out_final.copy_(o_acc.to(out_final.dtype))


def qk_norm_rope_pack(q, k, v, heads, dst_q, dst_k, dst_v, peer_strides, U=1, *, norm_q_weight=None,
                      norm_k_weight=None, eps=1e-6, norm_per_head=False, cos=None, sin=None, dst_strides=None):
    n = lambda t: None if t is None else _np(t)
    outs = O.attention_prologue(_np(q), _np(k), _np(v), heads, n(norm_q_weight), n(norm_k_weight), eps,
                                norm_per_head, n(cos), n(sin), U)
    for i, (o, dst, stride) in enumerate(zip(outs, (dst_q, dst_k, dst_v), peer_strides)):
        st = dst_strides[i] if dst_strides is not None else None
        if st is not None and (st[0] or st[1]):
            # o[p]: [Hl, B, s, D] -> rows at dst + hip*stride_h + b*stride_b + row*D
            Hl, B, s, D = o[0].shape
            for p in range(U):
                view = dst[p * stride:].as_strided((Hl, B, s, D), (st[0], st[1], D, 1))
                view.copy_(torch.from_numpy(o[p]).to(dst.dtype))
            continue
        blk = o[0].size
        for p in range(U):
            dst[p * stride:p * stride + blk].copy_(torch.from_numpy(o[p].reshape(-1)).to(dst.dtype))


def seq_shard_pad(x, rank, world):
    chunks, _ = O.pad_and_shard_sequence(x.detach().numpy(), world, dim=1)
    return torch.from_numpy(np.ascontiguousarray(chunks[rank])).to(x.dtype)


def seq_gather_unpad(recv, B, s, Cn, world, keep):
    chunks = [recv[w].detach().numpy() for w in range(world)]
    return torch.from_numpy(np.ascontiguousarray(O.gather_and_unpad(chunks, world * s - keep, dim=1))).to(recv.dtype)


# ---- peer-mapped buffers: POSIX shared memory stands for CUDA IPC, addresses are this process's own --------
_shm = {}  # base address -> (SharedMemory, uint8 tensor over it, owner?)


def _find(addr):
    for base, (_, t, _) in _shm.items():
        if base <= addr < base + t.numel():
            return t, addr - base
    raise KeyError(f"address {addr:#x} is not inside a mapped peer buffer")


def peer_alloc(nbytes, device):
    from multiprocessing import shared_memory

    shm = shared_memory.SharedMemory(create=True, size=int(nbytes))
    t = torch.frombuffer(shm.buf, dtype=torch.uint8, count=int(nbytes))
    t.zero_()
    _shm[t.data_ptr()] = (shm, t, True)
    return t.data_ptr(), shm.name.encode().ljust(64, b"\0"), t


def peer_open(handle, device):
    from multiprocessing import shared_memory

    shm = shared_memory.SharedMemory(name=bytes(handle).rstrip(b"\0").decode())
    t = torch.frombuffer(shm.buf, dtype=torch.uint8, count=shm.size)
    _shm[t.data_ptr()] = (shm, t, False)
    return t.data_ptr()


def peer_close(ptr):
    shm, t, _ = _shm.pop(int(ptr))
    del t
    try:
        shm.close()
    except BufferError:  # a view handed out earlier is still alive: the mapping goes with the process
        pass


def peer_free(ptr):
    shm, t, _ = _shm.pop(int(ptr))
    del t
    try:
        shm.close()
    except BufferError:
        pass
    shm.unlink()


def peer_copy(dst_ptr, src, nbytes):
    t, off = _find(int(dst_ptr))
    t[off:off + nbytes].copy_(src.contiguous().view(torch.uint8).reshape(-1)[:nbytes])


def peer_barrier(peer_flags, local_flags, epoch, rank, device, wait_limit_ns=0):
    """The flag protocol of ``xdit_peer_barrier`` with host loads and stores: bump the epoch, store it into
    word ``rank`` of every rank's flag array, wait until every word of the own array has reached it."""
    import time

    e = int(epoch.item()) + 1
    epoch.fill_(e)
    for p in peer_flags:
        t, off = _find(int(p) + 4 * rank)
        t[off:off + 4].view(torch.int32)[0] = e
    mine, off = _find(int(local_flags))
    words = mine[off:off + 4 * len(peer_flags)].view(torch.int32)
    t0 = time.time()
    while int(words.min()) < e:
        if time.time() - t0 > 60:
            raise RuntimeError(f"peer barrier {e}: flags {words.tolist()} after 60 s")
        time.sleep(0.0005)


def install(monkeypatch_or_none=None):
    """Replace the CUDA wrappers of ``xdit_b200.ops`` with the CPU stand-ins above."""
    import xdit_b200.ops as ops

    names = ["attn_fwd", "ulysses_pack", "ulysses_unpack_in", "ulysses_pack_out", "ulysses_unpack_out",
             "kv_patch_update", "merge_out_lse", "qk_norm_rope_pack", "seq_shard_pad", "seq_gather_unpad",
             "peer_alloc", "peer_open", "peer_close", "peer_free", "peer_copy", "peer_barrier", "ulysses_pack_peers"]
    for n in names:
        if monkeypatch_or_none is not None:
            monkeypatch_or_none.setattr(ops, n, globals()[n])
        else:
            setattr(ops, n, globals()[n])
