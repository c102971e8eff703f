"""Unified Sequence Parallel attention with the call surface of
``xfuser/model_executor/layers/usp.py`` (``USP`` ``:247-361``, ``attention`` ``:364-392`` and the
helpers tests reach for), re-built around the sm_100a kernels of this package.

Data path of one ``USP`` call on rank ``g`` (Ulysses degree U, ring degree R):

1. ``xdit_ulysses_pack`` (one launch) writes q (+ joint text queries), k and v straight into
   the all-to-all send buffer, peer-major: block p = ``[H/U][B][rows][D]`` for heads of peer p.
2. One NCCL all-to-all (two when a ring follows, so that K/V stay one contiguous ring message).
   The receive buffer is *not* re-laid-out: source rank p's rows form segment p of a
   ``[B, H/U, U, rows, D]`` strided view that the attention kernel walks through TMA.
3. ``xdit_attn_fwd``: joint text K/V are a second key/value source (no ``torch.cat``); with a
   ring the partial results are merged in fp32 inside the kernel epilogue while the next K/V
   shard moves on NCCL's stream (double-buffered point-to-point exchange).
4. The kernel writes its output in the send layout of the return all-to-all; what comes back
   is ``[H][B][rows][D]``, returned as a ``[B,H,rows,D]`` view without a copy.

The result equals the reference's: rows ``[image shard ; joint text]`` ("rear") or
``[joint text ; image shard]`` ("front") of dense softmax attention over all keys.
"""
from __future__ import annotations

import functools
from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from .attention_backend import ATTENTION_FUNCTION_REGISTRY, AttentionBackendType, reject_masked
from .cache_manager import get_cache_manager
from .distributed import (
    PROCESS_GROUP,
    get_ring_parallel_world_size,
    get_runtime_state,
    get_sequence_parallel_world_size,
    get_ulysses_parallel_rank,
    get_ulysses_parallel_world_size,
)

__all__ = ["USP", "attention", "ring_attn"]


# --------------------------------------------------------------------------------------
# small mirrors of the reference helpers
# --------------------------------------------------------------------------------------
def _concat_joint_tensor(tensor, joint_tensor, joint_strategy, dim):
    """``usp.py:179-189``; used on the compatibility path only (the native path never copies)."""
    if joint_strategy == "rear":
        return torch.cat([tensor, joint_tensor], dim=dim)
    if joint_strategy == "front":
        return torch.cat([joint_tensor, tensor], dim=dim)
    raise ValueError(f"Invalid joint_strategy: {joint_strategy}")


def _preprocess_joint_tensors(joint_key, joint_value):
    """Keep this Ulysses rank's heads of the replicated joint K/V (``usp.py:153-177``); views."""
    U = get_ulysses_parallel_world_size()
    u = get_ulysses_parallel_rank()
    hp = joint_key.shape[1] // U
    return joint_key[:, hp * u:hp * (u + 1)], joint_value[:, hp * u:hp * (u + 1)]


def _get_attention_function(backend=None):
    attention_backend = backend if backend is not None else get_runtime_state().attention_backend
    func = ATTENTION_FUNCTION_REGISTRY.get(attention_backend, None)
    if func is None:
        raise NotImplementedError(f"Attention backend {attention_backend} not registered.")
    return func


def concat_joint_tensors_decorator(func):
    """``usp.py:218-245``: append joint K/V on ring step 0 ("front") or the last step ("rear").
    Wraps user-registered back-ends on the compatibility path."""

    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        query, key, value = args[0:3]
        is_causal = kwargs.get("is_causal")
        dropout_p = kwargs.get("dropout_p")
        joint_attn_kwargs = kwargs.get("joint_attn_kwargs", None)
        attention_kwargs = kwargs.get("attention_kwargs", None)
        if joint_attn_kwargs is not None:
            strategy = joint_attn_kwargs.get("joint_strategy", None)
            step = joint_attn_kwargs.get("step", 0)
            total = joint_attn_kwargs.get("total_steps", 1)
            if (strategy == "front" and step == 0) or (strategy == "rear" and step == total - 1):
                key = _concat_joint_tensor(key, joint_attn_kwargs["joint_key"], strategy, dim=2)
                value = _concat_joint_tensor(value, joint_attn_kwargs["joint_value"], strategy, dim=2)
            joint_attn_kwargs["step"] = step + 1
        return func(query, key, value, dropout_p=dropout_p, is_causal=is_causal, attention_kwargs=attention_kwargs)

    return wrapper


def _sdpa_all_to_all_single(x, group=None):
    """Equal-split all-to-all of ``x`` viewed flat over the Ulysses group (``usp.py:87-93``)."""
    flat = x.reshape(-1)
    out = torch.empty_like(flat)
    dist.all_to_all_single(out, flat, group=PROCESS_GROUP.ULYSSES_PG if group is None else group)
    return out.reshape(x.shape)


def _input_all_to_all(x, U, group=None):
    """Heads scattered, sequence gathered: [B,H,s,D] -> [B,H/U,U*s,D] over ``group``."""
    assert x.ndim == 4, "x must have 4 dimensions, got {}".format(x.ndim)
    b, h, s, d = x.shape
    assert h % U == 0, "h must be divisible by world_size, got {} and {}".format(h, U)
    send = torch.empty(h * b * s * d, dtype=x.dtype, device=x.device)
    ops.ulysses_pack([dict(src=x, dst=send, peer_stride=(h // U) * b * s * d)], U)
    recv = _sdpa_all_to_all_single(send, group)
    return ops.ulysses_unpack_in(recv, b, h // U, s, d, U)


def _output_all_to_all(x, U, group=None):
    """Sequence scattered, heads gathered: [B,H/U,S',D] -> [B,H,S'/U,D] over ``group``."""
    assert x.ndim == 4, "x must have 4 dimensions, got {}".format(x.ndim)
    b, h, s, d = x.shape
    assert s % U == 0, "s must be divisible by world_size, got {} and {}".format(s, U)
    send = ops.ulysses_pack_out(x)
    recv = _sdpa_all_to_all_single(send, group)
    return ops.ulysses_unpack_out(recv, b, h, s // U, d, U)


def _ft_c_input_all_to_all(x):
    """[B,H,s,D] -> [B,H/U,U*s,D] (``usp.py:96-108``), materialised."""
    U = get_ulysses_parallel_world_size()
    if U <= 1:
        return x
    return _input_all_to_all(x, U)


def _combined_qkv_all_to_all(q, k, v):
    """One collective for q, k and v of equal shape (``usp.py:111-135``), materialised."""
    U = get_ulysses_parallel_world_size()
    if U <= 1:
        return q, k, v
    assert q.ndim == 4, f"q must have 4 dimensions, got {q.ndim}"
    b, h, s, d = q.shape
    assert h % U == 0, f"h must be divisible by world_size, got {h} and {U}"
    blk = (h // U) * b * s * d
    send = torch.empty(3 * U * blk, dtype=q.dtype, device=q.device)
    ops.ulysses_pack([dict(src=t, dst=send[i * blk:], peer_stride=3 * blk) for i, t in enumerate((q, k, v))], U)
    recv = _sdpa_all_to_all_single(send)
    r5 = recv.view(U, 3, blk)
    outs = []
    for i in range(3):
        outs.append(ops.ulysses_unpack_in(r5[:, i].contiguous(), b, h // U, s, d, U))
    return tuple(outs)


def _ft_c_output_all_to_all(x):
    """[B,H/U,S',D] -> [B,H,S'/U,D] (``usp.py:138-150``), materialised."""
    U = get_ulysses_parallel_world_size()
    if U <= 1:
        return x
    return _output_all_to_all(x, U)


def _update_and_get_kv_cache(key, value, attn_layer):
    """``usp.py:191-203``: PipeFusion stale-KV update after the all-to-all.  ``key``/``value`` may be
    4-D or 5-D segmented views; returns full-sequence [B,H,S,D] caches."""
    return get_cache_manager().update_and_get_kv(key, value, attn_layer, "attn")


# --------------------------------------------------------------------------------------
# ring attention
# --------------------------------------------------------------------------------------
def _ring_neighbours(group):
    R = dist.get_world_size(group)
    r = dist.get_rank(group)
    nxt = dist.get_global_rank(group, (r + 1) % R)
    prv = dist.get_global_rank(group, (r - 1) % R)
    return R, r, nxt, prv


def _ring_native(q, kv_buf, kv_views, joint_k, joint_v, front, out, group, scale=None, causal=False, lse=None):
    """R-step ring with the fused kernel.  ``kv_buf`` is the flat buffer holding this rank's K and V,
    ``kv_views(buf) -> (k, v)`` builds the sequence views over such a buffer.  ``out`` receives the
    final rows.  At step i the K/V shard of ring rank (r - i) mod R is attended to while the
    shard for step i+1 is in flight (``usp.py:46-74``, ``ring_flash_attn.py:83-143``)."""
    R, rank, nxt, prv = _ring_neighbours(group)
    B, Hl, D = q.shape[0], q.shape[1], q.shape[-1]
    sq = q.shape[2] if q.dim() == 4 else q.shape[2] * q.shape[3]
    o_acc = torch.empty(B, Hl, sq, D, dtype=torch.float32, device=q.device)
    lse_acc = torch.empty(B, Hl, sq, dtype=torch.float32, device=q.device)
    if not causal and kv_buf.is_contiguous():
        from . import peer_exchange

        if peer_exchange.ring_enabled():
            return _ring_peer_copies(q, kv_buf, kv_views, joint_k, joint_v, front, out, group, scale, lse, o_acc,
                                     lse_acc)
    cur = kv_buf
    spare = torch.empty_like(kv_buf)
    # with a causal mask the shard of step i is visible only when i <= rank, and only step 0
    # carries the diagonal (ring_flash_attn.py:104,113)
    last_step = rank if causal else R - 1
    for i in range(R):
        reqs = None
        if i < R - 1:
            reqs = dist.batch_isend_irecv([
                dist.P2POp(dist.isend, cur, nxt, group),
                dist.P2POp(dist.irecv, spare, prv, group),
            ])
        if i <= last_step:
            k_i, v_i = kv_views(cur)
            use_joint = joint_k is not None and ((front and i == 0) or ((not front) and i == R - 1))
            last = i == last_step
            ops.attn_fwd(q, k_i, v_i, joint_k if use_joint else None, joint_v if use_joint else None,
                         out=out if last else None, lse=lse if last else None, o_acc=o_acc, lse_acc=lse_acc,
                         acc_in=i > 0, acc_out=not last, scale=scale, causal=causal and i == 0)
        if reqs is not None:
            for r in reqs:
                r.wait()
            cur, spare = spare, cur
    return out


def _ring_peer_copies(q, kv_buf, kv_views, joint_k, joint_v, front, out, group, scale, lse, o_acc, lse_acc):
    """The same ring with the K/V rotation done by the copy engines: at step i this rank's current block is
    copied into the next rank's spare slot (one ``cudaMemcpyAsync`` to peer-mapped memory on a side stream,
    ``xdit_peer_copy``) while the attention kernel, which wants every SM, works on it; the ranks meet in
    ``xdit_peer_barrier`` between steps.  NCCL's send/recv kernels are not involved, so no SM is taken from the
    attention kernel.  Slot (i+1) % 2 of the next rank is free at step i: that rank read it at step i-1 (and
    copied it on), and the barrier after step i-1 has passed; the barrier at the start covers the previous
    call's last reads."""
    from . import peer_exchange

    R = dist.get_world_size(group)
    rank = dist.get_rank(group)
    nbytes = kv_buf.numel() * kv_buf.element_size()
    ex = peer_exchange.get(group, 256, nbytes, q.device)
    nxt = (rank + 1) % R
    ts = _TwoStreams(q.device)
    ts.keep_for_side([kv_buf])
    ex.sync()
    cur = kv_buf
    for i in range(R):
        if i < R - 1:
            ts.side_waits_cur()  # the barrier that ended step i-1 (or opened the call) lies behind
            with ts.on(1):
                ops.peer_copy(ex.out_peers((i + 1) % 2)[nxt], cur, nbytes)
        k_i, v_i = kv_views(cur)
        use_joint = joint_k is not None and ((front and i == 0) or ((not front) and i == R - 1))
        last = i == R - 1
        ops.attn_fwd(q, k_i, v_i, joint_k if use_joint else None, joint_v if use_joint else None,
                     out=out if last else None, lse=lse if last else None, o_acc=o_acc, lse_acc=lse_acc,
                     acc_in=i > 0, acc_out=not last, scale=scale)
        if i < R - 1:
            ts.cur_waits_side()
            ex.sync()
            cur = ex.out_local((i + 1) % 2, kv_buf.dtype)[:kv_buf.numel()]
    return out


def _segmented_kv_views(buf, B, Hl, U, sk, D, kv_stride, k_off, kv_blk):
    """K and V as ``[B, Hl, U, sk, D]`` views of a flat exchange buffer whose U blocks lie ``kv_stride``
    elements apart, K at ``k_off`` and V ``kv_blk`` elements behind it inside a block.  ``buf`` may itself be
    a slice of a larger buffer (a ring slot): ``as_strided`` counts its offset from the start of the storage."""
    shape, strides = (B, Hl, U, sk, D), (sk * D, B * sk * D, kv_stride, D, 1)
    base = buf.storage_offset() + k_off
    return buf.as_strided(shape, strides, base), buf.as_strided(shape, strides, base + kv_blk)


def _pack_kv_flat(k, v):
    """Copy (possibly strided) k, v [B,H,S,D] into one flat buffer [k | v], each [B,H,S,D] contiguous."""
    B, H, S, D = k.shape
    n = B * H * S * D
    buf = torch.empty(2 * n, dtype=k.dtype, device=k.device)
    if B == 1:
        # [H][B][S][D] == [B][H][S][D] when B == 1: the pack kernel writes it in one launch
        ops.ulysses_pack([dict(src=k, dst=buf, peer_stride=n), dict(src=v, dst=buf[n:], peer_stride=n)], 1)
    else:
        buf[:n].view(B, H, S, D).copy_(k)
        buf[n:].view(B, H, S, D).copy_(v)

    def views(b, shape=(B, H, S, D), n=n):
        return b[:n].view(shape), b[n:].view(shape)

    return buf, views


def ring_attn(attention_function, query, key, value, dropout_p=0.0, is_causal=False, joint_attn_kwargs=None,
              attention_kwargs=None):
    """``usp.py:46-74``.  With the native back-end this is the fused ring; any other registered
    function is driven step by step and merged with ``xdit_merge_out_lse``."""
    group = PROCESS_GROUP.RING_PG
    R = get_ring_parallel_world_size()
    if is_causal:
        raise NotImplementedError("causal ring attention is offered by xdit_ring_flash_attn_func")
    jk = jv = None
    front = False
    if joint_attn_kwargs is not None:
        jk, jv = joint_attn_kwargs["joint_key"], joint_attn_kwargs["joint_value"]
        front = joint_attn_kwargs["joint_strategy"] == "front"
    if getattr(attention_function, "is_xdit_b200_native", False):
        if dropout_p:
            raise NotImplementedError("dropout is not implemented")
        reject_masked(attention_kwargs)
        out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        if R == 1 or group is None:
            ops.attn_fwd(query, key, value, jk, jv, out=out)
            return out
        buf, views = _pack_kv_flat(key, value)
        return _ring_native(query, buf, views, jk, jv, front, out, group)
    # compatibility path: user-registered (out, lse) function
    func = concat_joint_tensors_decorator(attention_function)
    if joint_attn_kwargs is not None:
        joint_attn_kwargs = dict(joint_attn_kwargs, step=0, total_steps=R)
    if R == 1 or group is None:
        out, _ = func(query, key, value, dropout_p=dropout_p, is_causal=False,
                      joint_attn_kwargs=joint_attn_kwargs, attention_kwargs=attention_kwargs)
        return out
    _, _, nxt, prv = _ring_neighbours(group)
    buf, views = _pack_kv_flat(key, value)
    spare = torch.empty_like(buf)
    B, H, S, D = query.shape
    o_acc = torch.empty(B, H, S, D, dtype=torch.float32, device=query.device)
    lse_acc = torch.empty(B, H, S, dtype=torch.float32, device=query.device)
    final = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    cur = buf
    for i in range(R):
        reqs = None
        if i < R - 1:
            reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, cur, nxt, group),
                                           dist.P2POp(dist.irecv, spare, prv, group)])
        k_i, v_i = views(cur)
        bo, bl = func(query, k_i, v_i, dropout_p=dropout_p, is_causal=False,
                      joint_attn_kwargs=joint_attn_kwargs, attention_kwargs=attention_kwargs)
        if bl is None:
            raise RuntimeError("ring attention needs a back-end that returns the log-sum-exp")
        ops.merge_out_lse(o_acc, lse_acc, bo.contiguous(), bl.contiguous().float(), first=i == 0,
                          out_final=final if i == R - 1 else None)
        if reqs is not None:
            for r in reqs:
                r.wait()
            cur, spare = spare, cur
    return final


# --------------------------------------------------------------------------------------
# USP
# --------------------------------------------------------------------------------------
def USP(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    joint_query: Optional[torch.Tensor] = None,
    joint_key: Optional[torch.Tensor] = None,
    joint_value: Optional[torch.Tensor] = None,
    joint_strategy: Optional[str] = None,
    attn_layer=None,
    combine_qkv_a2a: Optional[bool] = None,
    backend=None,
    attention_kwargs: Optional[dict] = None,
    head_balance_layer=None,
):
    """Same signature and result as the reference's ``USP`` (``usp.py:247-361``).

    Tensors are ``[B, H, S_local, D]`` with any strides (head_dim contiguous); returns
    ``[B, H, S_local (+ S_joint), D]`` in the input dtype.  ``combine_qkv_a2a`` is accepted for
    signature parity: q, k and v always share one pack launch and, without a ring, one
    collective.  ``head_balance_layer`` is a no-op for dense back-ends, as in the reference
    (``head_balance.py:80-90``).
    """
    func = _get_attention_function(backend)
    if not getattr(func, "is_xdit_b200_native", False):
        return _usp_compat(func, query, key, value, dropout_p, is_causal, joint_query, joint_key, joint_value,
                           joint_strategy, attn_layer, combine_qkv_a2a, attention_kwargs)
    if dropout_p:
        raise NotImplementedError("dropout is not implemented (the DiT callers always pass 0.0)")
    reject_masked(attention_kwargs)
    if torch.compiler.is_compiling() and not attn_layer:
        # under torch.compile the whole call is one opaque operator (no graph break at the ctypes calls)
        from . import compile_ops

        return compile_ops.usp(query, key, value, joint_query, joint_key, joint_value, joint_strategy or "",
                               bool(is_causal), 0.0)
    return usp_native(query, key, value, joint_query, joint_key, joint_value, joint_strategy, attn_layer,
                      is_causal, None, get_ulysses_parallel_world_size(), get_ring_parallel_world_size(),
                      get_ulysses_parallel_rank(), PROCESS_GROUP.ULYSSES_PG, PROCESS_GROUP.RING_PG)


# Ulysses exchanges of at least this many bytes per rank are pipelined by head groups (see
# _ulysses_pipelined); below it the extra collectives cost more than the overlap returns.
PIPELINE_MIN_BYTES = 32 << 20
_side_streams: dict = {}


def _all_to_all_chunks(out_chunks, in_chunks, group) -> None:
    """Equal-split all-to-all whose receive side is a list of separately placed chunks (the grouped
    send/recv form of NCCL).  gloo has no such collective: there (host-logic tests on CPU) it is one flat
    all-to-all and a copy."""
    if in_chunks[0].is_cuda:
        dist.all_to_all(out_chunks, in_chunks, group=group)
        return
    flat_in = torch.cat([c.reshape(-1) for c in in_chunks])
    flat_out = torch.empty_like(flat_in)
    dist.all_to_all_single(flat_out, flat_in, group=group)
    for dst, src in zip(out_chunks, flat_out.chunk(len(out_chunks))):
        dst.copy_(src.view_as(dst))


class _TwoStreams:
    """The current stream and one side stream of a CUDA device; on a CPU device (host-logic tests under
    gloo) every operation is a no-op and the work simply runs in program order."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        if self.cuda:
            key = device.index if device.index is not None else torch.cuda.current_device()
            side = _side_streams.get(key)
            if side is None:
                side = _side_streams[key] = torch.cuda.Stream(device)
            self.cur, self.side = torch.cuda.current_stream(device), side

    def on(self, which):
        import contextlib

        if not self.cuda or which == 0:
            return contextlib.nullcontext()
        return torch.cuda.stream(self.side)

    def side_waits_cur(self):
        if self.cuda:
            self.side.wait_stream(self.cur)

    def cur_waits_side(self):
        if self.cuda:
            self.cur.wait_stream(self.side)

    def mark_side(self):
        """An event at the current end of the side stream (None on CPU)."""
        if not self.cuda:
            return None
        ev = torch.cuda.Event()
        ev.record(self.side)
        return ev

    def cur_waits_mark(self, ev):
        if ev is not None:
            self.cur.wait_event(ev)

    def keep_for_side(self, tensors):
        if self.cuda:
            for t in tensors:  # used on both streams: keep the allocator from recycling them early
                t.record_stream(self.side)


def _ulysses_pipelined(query, key, value, jq, jk, jv, front, scale, U, uly):
    """Ulysses-only attention with the exchange hidden behind the arithmetic: every peer's heads are split
    into two groups; group 1 is packed and exchanged on a side stream while group 0 is attended to, and
    group 0's result travels back while group 1 is attended to (``usp.py:96-150`` does pack, collective,
    attention, collective strictly one after the other).  The two return exchanges write interleaved
    slices of one ``[H][B][rows][D]`` buffer, so the result is the same view as without pipelining."""
    B, H, s, D = query.shape
    sk = key.shape[2]
    sj = jq.shape[2] if jq is not None else 0
    sq = s + sj
    Hl = H // U
    Hg = Hl // 2
    dev, dt = query.device, query.dtype
    q_blk, kv_blk = Hg * B * sq * D, Hg * B * sk * D
    stride = q_blk + 2 * kv_blk
    ts = _TwoStreams(dev)
    out_recv = torch.empty(H * B * sq * D, dtype=dt, device=dev)
    out_chunks = out_recv.view(U, 2, q_blk)  # [peer][group][Hg*B*sq*D]
    ts.side_waits_cur()  # the inputs are ready for the side stream too
    recvs, sends, outs = [], [], []
    for g in (0, 1):
        with ts.on(g):
            send = torch.empty(U * stride, dtype=dt, device=dev)
            ops.ulysses_pack([
                dict(src=query, joint=jq, front=front, dst=send, peer_stride=stride),
                dict(src=key, dst=send[q_blk:], peer_stride=stride),
                dict(src=value, dst=send[q_blk + kv_blk:], peer_stride=stride),
            ], U, head_group=(g, 2))
            sends.append(send)
    for g in (0, 1):
        with ts.on(g):
            recv = torch.empty_like(sends[g])
            dist.all_to_all_single(recv, sends[g], group=uly)
            recvs.append(recv)
    arrived1 = ts.mark_side()  # group 1 has arrived once the side stream gets here
    for g in (0, 1):
        if g == 1:
            # only group 1's arrival is waited for: group 0's return exchange, queued on the side stream
            # after it, keeps running under this group's attention
            ts.cur_waits_mark(arrived1)
        recv = recvs[g]
        q5 = recv.as_strided((B, Hg, U, sq, D), (sq * D, B * sq * D, stride, D, 1), 0)
        shape, strides = (B, Hg, U, sk, D), (sk * D, B * sk * D, stride, D, 1)
        k5, v5 = recv.as_strided(shape, strides, q_blk), recv.as_strided(shape, strides, q_blk + kv_blk)
        out_send = torch.empty(U * q_blk, dtype=dt, device=dev)
        out5 = out_send.as_strided((B, Hg, U, sq, D), (sq * D, B * sq * D, q_blk, D, 1), 0)
        jkg = jk[:, g * Hg:(g + 1) * Hg] if jk is not None else None
        jvg = jv[:, g * Hg:(g + 1) * Hg] if jv is not None else None
        ops.attn_fwd(q5, k5, v5, jkg, jvg, out=out5, scale=scale)
        outs.append(out_send)
        if g == 0:
            ts.side_waits_cur()  # group 0's result exists; it travels back under group 1's attention
        with ts.on(1 - g):
            _all_to_all_chunks(list(out_chunks[:, g].unbind(0)), list(out_send.view(U, q_blk).unbind(0)), uly)
    ts.cur_waits_side()
    ts.keep_for_side(sends + recvs + outs + [out_recv])
    return out_recv.view(H, B, sq, D).permute(1, 0, 2, 3)


def _ulysses_peer_stores(query, key, value, jq, jk, jv, front, scale, U, u_rank, uly):
    """Ulysses-only attention with both exchanges done by the kernels themselves (``xdit_b200.peer_exchange``):
    the pack kernel stores every peer's block into that peer's receive buffer, the attention kernel's
    epilogue stores every source rank's rows into that rank's ``[B, rows, H, D]`` result buffer.  Two
    one-element all-reduces order the ranks.  Returns a ``[B, H, rows, D]`` view of the result buffer."""
    from . import peer_exchange

    B, H, s, D = query.shape
    sk = key.shape[2]
    sj = jq.shape[2] if jq is not None else 0
    sq = s + sj
    Hl = H // U
    dt, es = query.dtype, query.element_size()
    q_blk, kv_blk = Hl * B * sq * D, Hl * B * sk * D
    stride = q_blk + 2 * kv_blk
    ex = peer_exchange.get(uly, U * stride * es, B * sq * H * D * es, query.device)
    # input side: my block for peer p lands at element offset u_rank*stride of p's receive buffer
    base = u_rank * stride
    ops.ulysses_pack_peers([
        dict(src=query, joint=jq, front=front, dst_offset=base),
        dict(src=key, dst_offset=base + q_blk),
        dict(src=value, dst_offset=base + q_blk + kv_blk),
    ], U, ex.in_peers())
    ex.sync()
    recv = ex.in_local(dt)
    q5 = recv.as_strided((B, Hl, U, sq, D), (sq * D, B * sq * D, stride, D, 1), 0)
    shape, strides = (B, Hl, U, sk, D), (sk * D, B * sk * D, stride, D, 1)
    k5, v5 = recv.as_strided(shape, strides, q_blk), recv.as_strided(shape, strides, q_blk + kv_blk)
    # output side: the rows of query segment g (source rank g) go to rank g's [B, sq, H, D] buffer, into
    # the columns of this rank's heads
    slot = ex.next_out_slot()
    segs = [p + u_rank * Hl * D * es for p in ex.out_peers(slot)]
    ops.attn_fwd(q5, k5, v5, jk, jv, out_segments=segs, out_strides=(sq * H * D, D, H * D), scale=scale)
    ex.sync()
    out = ex.out_local(slot, dt)[:B * sq * H * D].view(B, sq, H, D)
    return out.permute(0, 2, 1, 3)


def usp_native(query, key, value, joint_query, joint_key, joint_value, joint_strategy, attn_layer, is_causal,
               scale, U, R, u_rank, uly, ring_pg, want_lse=False):
    """The fused data path described in the module docstring, for explicit groups and degrees.
    Returns the output, or ``(output, lse)`` with ``want_lse`` (Ulysses degree 1 only)."""
    if is_causal and U > 1:
        raise NotImplementedError("causal attention with a Ulysses all-to-all is not part of the DiT path")
    if query.ndim != 4:
        raise AssertionError("x must have 4 dimensions, got {}".format(query.ndim))
    B, H, s, D = query.shape
    sk = key.shape[2]
    if key.shape != value.shape:
        raise ValueError("key and value must have the same shape")

    jq = jk = jv = None
    front = False
    if joint_strategy:
        if joint_strategy not in ("front", "rear"):
            raise ValueError(f"Invalid joint_strategy: {joint_strategy}")
        if joint_query is None or joint_key is None or joint_value is None:
            raise ValueError("joint_query, joint_key and joint_value are required with a joint_strategy")
        front = joint_strategy == "front"
        jq = joint_query
        hp = joint_key.shape[1] // U
        jk, jv = joint_key[:, hp * u_rank:hp * (u_rank + 1)], joint_value[:, hp * u_rank:hp * (u_rank + 1)]
    sj = jq.shape[2] if jq is not None else 0
    sq = s + sj
    dev, dt = query.device, query.dtype

    if U > 1:
        assert H % U == 0, "h must be divisible by world_size, got {} and {}".format(H, U)
        Hl = H // U
        q_blk, kv_blk = Hl * B * sq * D, Hl * B * sk * D
        if (R == 1 and not attn_layer and not want_lse and not is_causal
                and dt in (torch.bfloat16, torch.float16) and D % 8 == 0 and D <= 128 and U <= 16):
            from . import peer_exchange

            if peer_exchange.enabled_for(U * (q_blk + 2 * kv_blk) * query.element_size()):
                return _ulysses_peer_stores(query, key, value, jq, jk, jv, front, scale, U, u_rank, uly)
        if (R == 1 and not attn_layer and not want_lse and not is_causal and Hl % 2 == 0
                and U * (q_blk + 2 * kv_blk) * query.element_size() >= PIPELINE_MIN_BYTES):
            return _ulysses_pipelined(query, key, value, jq, jk, jv, front, scale, U, uly)
        if R == 1:
            stride = q_blk + 2 * kv_blk
            send = torch.empty(U * stride, dtype=dt, device=dev)
            ops.ulysses_pack([
                dict(src=query, joint=jq, front=front, dst=send, peer_stride=stride),
                dict(src=key, dst=send[q_blk:], peer_stride=stride),
                dict(src=value, dst=send[q_blk + kv_blk:], peer_stride=stride),
            ], U)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=uly)
            q5 = recv.as_strided((B, Hl, U, sq, D), (sq * D, B * sq * D, stride, D, 1), 0)
            kv_recv, kv_stride, k_off = recv, stride, q_blk
        else:
            q_send = torch.empty(U * q_blk, dtype=dt, device=dev)
            kv_send = torch.empty(U * 2 * kv_blk, dtype=dt, device=dev)
            ops.ulysses_pack([
                dict(src=query, joint=jq, front=front, dst=q_send, peer_stride=q_blk),
                dict(src=key, dst=kv_send, peer_stride=2 * kv_blk),
                dict(src=value, dst=kv_send[kv_blk:], peer_stride=2 * kv_blk),
            ], U)
            q_recv = torch.empty_like(q_send)
            kv_recv = torch.empty_like(kv_send)
            dist.all_to_all_single(q_recv, q_send, group=uly)
            dist.all_to_all_single(kv_recv, kv_send, group=uly)
            q5 = q_recv.as_strided((B, Hl, U, sq, D), (sq * D, B * sq * D, q_blk, D, 1), 0)
            kv_stride, k_off = 2 * kv_blk, 0

        def kv_views(buf, kv_stride=kv_stride, k_off=k_off):
            return _segmented_kv_views(buf, B, Hl, U, sk, D, kv_stride, k_off, kv_blk)

        q_att = q5
        k_att, v_att = kv_views(kv_recv)
        out_send = torch.empty(U * q_blk, dtype=dt, device=dev)
        out_att = out_send.as_strided((B, Hl, U, sq, D), (sq * D, B * sq * D, q_blk, D, 1), 0)
    else:
        if jq is not None:
            q_att = torch.empty(B, H, sq, D, dtype=dt, device=dev)
            if B == 1:
                ops.ulysses_pack([dict(src=query, joint=jq, front=front, dst=q_att.view(-1), peer_stride=q_att.numel())], 1)
            else:
                q_att.copy_(_concat_joint_tensor(query, jq, joint_strategy, dim=2))
        else:
            q_att = query
        k_att, v_att = key, value
        kv_recv = kv_views = None
        out_att = torch.empty(B, H, sq, D, dtype=dt, device=dev)

    if attn_layer:
        k_att, v_att = _update_and_get_kv_cache(k_att, v_att, attn_layer)
        kv_recv = kv_views = None

    lse = None
    if want_lse:
        if U > 1:
            raise NotImplementedError("the log-sum-exp is returned for Ulysses degree 1 only")
        lse = torch.empty(B, H, sq, dtype=torch.float32, device=dev)
    if R == 1:
        ops.attn_fwd(q_att, k_att, v_att, jk, jv, out=out_att, lse=lse, causal=is_causal, scale=scale)
    else:
        if kv_recv is None or k_off != 0:
            buf, views = _pack_kv_flat(k_att if k_att.dim() == 4 else k_att.reshape(B, -1, k_att.shape[2] * k_att.shape[3], D),
                                       v_att if v_att.dim() == 4 else v_att.reshape(B, -1, v_att.shape[2] * v_att.shape[3], D))
        else:
            buf, views = kv_recv, kv_views
        _ring_native(q_att, buf, views, jk, jv, front, out_att, ring_pg, scale=scale, causal=is_causal, lse=lse)

    if U == 1:
        return (out_att, lse) if want_lse else out_att
    out_recv = torch.empty_like(out_send)
    dist.all_to_all_single(out_recv, out_send, group=uly)
    return out_recv.view(H, B, sq, D).permute(1, 0, 2, 3)


def _usp_compat(func, query, key, value, dropout_p, is_causal, joint_query, joint_key, joint_value,
                joint_strategy, attn_layer, combine_qkv_a2a, attention_kwargs):
    """The reference's sequence of steps, for a user-registered back-end function: materialised
    all-to-all re-layouts around ``func`` and a step-by-step ring."""
    joint_attn_kwargs = None
    if joint_strategy:
        query = _concat_joint_tensor(query, joint_query, joint_strategy, dim=2)
        jk, jv = _preprocess_joint_tensors(joint_key, joint_value)
        joint_attn_kwargs = {"joint_value": jv, "joint_key": jk, "joint_strategy": joint_strategy, "step": 0,
                             "total_steps": get_ring_parallel_world_size()}
    if get_ulysses_parallel_world_size() > 1:
        if combine_qkv_a2a and query.shape == key.shape == value.shape:
            query, key, value = _combined_qkv_all_to_all(query, key, value)
        else:
            query, key, value = (_ft_c_input_all_to_all(t) for t in (query, key, value))
    if attn_layer:
        key, value = _update_and_get_kv_cache(key, value, attn_layer)
    if get_ring_parallel_world_size() == 1:
        out, _ = concat_joint_tensors_decorator(func)(query, key, value, dropout_p=dropout_p, is_causal=is_causal,
                                                      joint_attn_kwargs=joint_attn_kwargs,
                                                      attention_kwargs=attention_kwargs)
    else:
        out = ring_attn(func, query, key, value, dropout_p=dropout_p, is_causal=is_causal,
                        joint_attn_kwargs=joint_attn_kwargs, attention_kwargs=attention_kwargs)
    if get_ulysses_parallel_world_size() > 1:
        out = _ft_c_output_all_to_all(out)
    return out


def attention(query, key, value, dropout_p: float = 0.0, is_causal: bool = False, backend=None,
              attention_kwargs=None, head_balance_layer=None):
    """Attention without any parallelism (``usp.py:364-392``), e.g. Wan's text cross-attention."""
    func = _get_attention_function(backend)
    out, _ = func(query, key, value, dropout_p=dropout_p, is_causal=is_causal, attention_kwargs=attention_kwargs)
    return out
