"""Tensor-level wrappers over the C-ABI kernels.

Tensors are ``torch`` CUDA tensors used as typed device pointers; all arithmetic happens in
``libxdit_b200.so``.  A *sequence* argument (q, k, v, fresh KV rows) is either a 4-D view
``[B, H, S, D]`` or a 5-D view ``[B, H, G, L, D]`` of ``G`` segments of ``L`` rows -- the shape a
Ulysses all-to-all receive buffer has, one segment per source rank.  Any strides are accepted
as long as the last axis is contiguous.

There is no CPU implementation: calling these with CPU tensors raises.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import torch

from . import _capi

_DTYPES = {torch.bfloat16: _capi.XDIT_BF16, torch.float16: _capi.XDIT_F16, torch.float32: _capi.XDIT_F32}
_status_bufs: dict = {}
launch_count = 0  # kernels launched through this module (read by the benchmark)


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "xdit_b200 kernels run on CUDA tensors only (sm_100a); got a tensor on "
                f"{t.device}. There is no CPU fallback."
            )


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _dtype(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _seq(t: Optional[torch.Tensor]) -> _capi.Seq:
    s = _capi.Seq()
    if t is None:
        return s
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        raise ValueError("the head_dim axis must be contiguous")
    s.ptr = t.data_ptr()
    if t.dim() == 4:
        s.stride_b, s.stride_h, s.stride_row = t.stride(0), t.stride(1), t.stride(2)
        s.stride_seg = 0
        s.nseg, s.seg_len = 1, t.shape[2]
    elif t.dim() == 5:
        s.stride_b, s.stride_h, s.stride_seg, s.stride_row = t.stride(0), t.stride(1), t.stride(2), t.stride(3)
        s.nseg, s.seg_len = t.shape[2], t.shape[3]
    else:
        raise ValueError(f"expected a 4-D or 5-D sequence tensor, got {t.dim()}-D")
    return s


class _Status:
    """Per-device pair of status words of the attention kernel: ``dev`` (int32 in device memory, read
    by every launch) and ``host`` (int32 in pinned, device-mapped host memory, written by a launch
    only when one of its bounded waits gave up, and read by the C entry point before it launches)."""

    def __init__(self, index: int):
        self.dev = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.index = index


def _device_index(device) -> int:
    device = torch.device(device) if device is not None else torch.device("cuda")
    return device.index if device.index is not None else torch.cuda.current_device()


def _status(device) -> _Status:
    key = _device_index(device)
    st = _status_bufs.get(key)
    if st is None:
        st = _status_bufs[key] = _Status(key)
    return st


def status_buffer(device) -> torch.Tensor:
    """Per-device int32 word the attention kernel sets when one of its bounded waits gives up."""
    return _status(device).dev


def clear_status(device=None) -> None:
    """Zero both status words of ``device`` (all devices when None), so that launches run again."""
    for st in (list(_status_bufs.values()) if device is None else [_status(device)]):
        st.dev.zero_()
        st.host.zero_()


def check_status(device=None) -> None:
    """Synchronise and raise if any attention kernel on ``device`` (the current device for a bare
    ``"cuda"``; every device used so far when None) reported a timed-out wait.  The words are cleared
    before the exception is raised, so that later launches run again.

    Product calls do not need this: a failure also lands in a host-visible word that the next
    ``xdit_attn_fwd`` call reads without synchronising, and that call raises
    ``XditError(XDIT_E_KERNEL_TIMEOUT)`` (see :func:`attn_fwd`).  This function is for the end of a
    run, where no next call follows."""
    sts = list(_status_bufs.values()) if device is None else [_status_bufs.get(_device_index(device))]
    for st in sts:
        if st is None:
            continue
        code = int(st.dev.item())  # synchronises the device
        code = code or int(st.host.item())
        if code:
            clear_status(torch.device("cuda", st.index))
            raise _capi.XditError(-6, "attention kernel", f"bounded wait gave up (code {code})")


def query_caps() -> dict:
    caps = _capi.Caps()
    _capi.check(_capi.load().xdit_query_caps(C.byref(caps)), "xdit_query_caps")
    return {name: getattr(caps, name) for name, _ in caps._fields_}


def _attn_params(q, k, v, k2, v2, out, lse, o_acc, lse_acc, acc_in, acc_out, causal, scale, force_generic):
    p = _capi.AttnParams()
    p.dtype = _dtype(q)
    p.B, p.H, p.D = q.shape[0], q.shape[1], q.shape[-1]
    p.q, p.k, p.v = _seq(q), _seq(k), _seq(v)
    p.k2, p.v2 = _seq(k2), _seq(v2)
    if out is not None:
        p.out = out.data_ptr()
        so = _seq(out)
        p.out_stride_b, p.out_stride_h, p.out_stride_seg, p.out_stride_row = (
            so.stride_b, so.stride_h, so.stride_seg, so.stride_row)
    p.lse = lse.data_ptr() if lse is not None else None
    p.o_acc = o_acc.data_ptr() if o_acc is not None else None
    p.lse_acc = lse_acc.data_ptr() if lse_acc is not None else None
    p.acc_in, p.acc_out, p.causal = int(bool(acc_in)), int(bool(acc_out)), int(bool(causal))
    p.softmax_scale = float(scale) if scale else 0.0
    p.force_generic = int(bool(force_generic))
    st = _status(q.device)
    p.status = st.dev.data_ptr()
    p.status_host = st.host.data_ptr()
    return p


# False: never hand out scratch, so that no call splits its keys (an A/B switch for measurements)
SPLIT_KEYS = True
_split_scratch = {}  # device index -> uint8 tensor reused by every call that splits its keys over CTAs


def _give_split_scratch(p, q) -> None:
    """Hand ``xdit_attn_fwd`` the scratch it wants for splitting a small launch's keys over several CTAs
    (``xdit_attn_split_scratch_bytes``; nothing for most calls).  The buffer is kept per device and grows on
    demand, but never while a stream is being captured: a call whose first run is a captured one simply is
    not split.  One buffer per device: calls that split must not run at the same time on two streams of one
    device (nothing in this package does that; a caller who does sets ``SPLIT_KEYS = False`` or passes scratch
    of its own through the C ABI)."""
    with torch.cuda.device(q.device):
        need = int(_capi.load().xdit_attn_split_scratch_bytes(C.byref(p)))
    if need <= 0:
        return
    key = q.device.index if q.device.index is not None else torch.cuda.current_device()
    buf = _split_scratch.get(key)
    if buf is None or buf.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            if buf is None:
                return
        else:
            buf = _split_scratch[key] = torch.empty(need, dtype=torch.uint8, device=q.device)
    p.split_scratch = buf.data_ptr()
    p.split_scratch_bytes = buf.numel()


def attn_split_scratch_bytes(q, k, v, k2=None, v2=None) -> int:
    """Scratch the library wants for splitting this call's keys over several CTAs (0: it would not split);
    ``attn_fwd`` provides it by itself, this is for callers of the C ABI and for tests."""
    _require_cuda(q, k, v, k2, v2)
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    p = _attn_params(q, k, v, k2, v2, out, None, None, None, False, False, False, None, False)
    with torch.cuda.device(q.device):
        return int(_capi.load().xdit_attn_split_scratch_bytes(C.byref(p)))


def _launch_attn(fn, p, q, where):
    """Call an attention entry point; a timeout reported by an earlier launch surfaces here, and the
    status words are cleared so that the caller may retry."""
    with torch.cuda.device(q.device):
        rc = fn(C.byref(p), _stream(q))
    if rc == -6:  # XDIT_E_KERNEL_TIMEOUT
        msg = _capi.load().xdit_last_error_string()
        torch.cuda.synchronize(q.device)
        clear_status(q.device)
        raise _capi.XditError(rc, where, msg.decode() if msg else "")
    _capi.check(rc, where)


def attn_fwd(q, k, v, k2=None, v2=None, *, out=None, lse=None, o_acc=None, lse_acc=None,
             acc_in=False, acc_out=False, causal=False, scale=None, force_generic=False,
             want_lse=False, out_segments=None, out_strides=None, _wait_limit_ns=0, _selftest_stall=False):
    """Dense softmax attention forward (C-ABI ``xdit_attn_fwd``).

    Returns ``(out, lse)``.  ``out`` is allocated like ``q`` (contiguous, same dims) unless given;
    ``lse`` ([B,H,Sq] fp32) is produced when ``want_lse`` or when a buffer is passed.  With
    ``acc_out`` the result goes to the fp32 accumulators instead and ``out`` may stay ``None``.

    ``out_segments`` (a list of ``q``'s segment count device addresses, possibly in peer GPUs' memory) with
    ``out_strides = (batch, head, row)`` in elements sends the rows of every query segment to a base of its
    own instead of one ``out`` tensor; nothing is returned for ``out`` then.

    Raises ``XditError`` (code ``XDIT_E_KERNEL_TIMEOUT``) when an earlier launch on this device gave
    up one of its bounded waits: that launch's output is invalid, nothing new was launched, and the
    status words have been cleared so that the caller can retry.
    """
    global launch_count
    _require_cuda(q, k, v, k2, v2, out, lse, o_acc, lse_acc)
    for t in (k, v, k2, v2):
        if t is not None and t.dtype != q.dtype:
            raise TypeError("q, k, v (and joint k, v) must share one dtype")
    sq = q.shape[2] if q.dim() == 4 else q.shape[2] * q.shape[3]
    if out is None and not acc_out and out_segments is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    if lse is None and want_lse and not acc_out:
        lse = torch.empty(q.shape[0], q.shape[1], sq, dtype=torch.float32, device=q.device)
    p = _attn_params(q, k, v, k2, v2, out, lse, o_acc, lse_acc, acc_in, acc_out, causal, scale, force_generic)
    p.wait_limit_ns = int(_wait_limit_ns)
    p.selftest_stall = int(bool(_selftest_stall))
    if out_segments is not None:
        nseg = q.shape[2] if q.dim() == 5 else 1
        if len(out_segments) != nseg or out_strides is None:
            raise ValueError("out_segments needs one address per query segment and out_strides=(batch, head, row)")
        seg_arr = (C.c_void_p * nseg)(*[int(x) for x in out_segments])
        p.out_segments = C.cast(seg_arr, C.POINTER(C.c_void_p))
        p.out = None
        p.out_stride_b, p.out_stride_h, p.out_stride_row = (int(x) for x in out_strides)
        p.out_stride_seg = 0
    if not acc_in and not acc_out and not force_generic and not _selftest_stall and SPLIT_KEYS:
        _give_split_scratch(p, q)
    _launch_attn(_capi.load().xdit_attn_fwd, p, q, "xdit_attn_fwd")
    launch_count += 1
    return out, lse


def attn_fwd_static_acc(q, k, v, k2=None, v2=None, *, out=None, lse=None, acc_in=False, acc_out=False,
                        scale=None, force_generic=False):
    """One ring step through ``xdit_attn_fwd_static_acc``: like :func:`attn_fwd` with ``o_acc`` /
    ``lse_acc``, but the fp32 running accumulators live in a fixed array inside the library, so
    this wrapper allocates no device memory apart from the per-device status words (4 bytes of device
    memory and 4 bytes of pinned host memory, created by the first attention call of any kind on the
    device).  ``out`` (and ``lse`` if wanted) must be passed for the last step (``acc_out=False``).  One sequence at a time per device; sizes beyond the built-in
    array raise ``XditError``."""
    global launch_count
    _require_cuda(q, k, v, k2, v2, out, lse)
    if not acc_out and out is None:
        raise ValueError("the last step (acc_out=False) needs an output tensor: this entry point allocates nothing")
    p = _attn_params(q, k, v, k2, v2, out, lse, None, None, acc_in, acc_out, False, scale, force_generic)
    _launch_attn(_capi.load().xdit_attn_fwd_static_acc, p, q, "xdit_attn_fwd_static_acc")
    launch_count += 1
    return out, lse


def attn_which(q, k, v, k2=None, v2=None, *, out=None, causal=False, acc=False) -> int:
    """1 when the tcgen05 kernel would serve this call, 0 for the CUDA-core kernel."""
    dummy = q if out is None else out
    acc_buf = q if acc else None
    p = _attn_params(q, k, v, k2, v2, dummy, None, acc_buf, acc_buf, acc, False, causal, None, False)
    return _capi.load().xdit_attn_which(C.byref(p))


def ulysses_pack(items: Sequence[dict], U: int, head_group=None) -> None:
    """Pack up to four tensors into all-to-all send buffers with one launch (``xdit_ulysses_pack``).

    Each item: ``src`` [B,H,s,D]; optional ``joint`` [B,H,sj,D] and ``front`` (bool); ``dst`` a
    1-D tensor positioned at this tensor's slot inside peer 0's block; ``peer_stride`` the
    distance in elements between two peers' blocks of that buffer.

    ``head_group=(g, G)`` packs only group ``g`` of ``G`` equal groups of every peer's heads: peer p's
    block then holds heads ``[p*H/U + g*H/(U*G), +H/(U*G))``.
    """
    global launch_count
    n = len(items)
    if not 1 <= n <= _capi.XDIT_MAX_PACK_JOBS:
        raise ValueError(f"1..{_capi.XDIT_MAX_PACK_JOBS} tensors per pack call")
    jobs = (_capi.PackJob * n)()
    ref = items[0]["src"]
    B, H, _, D = ref.shape
    g, G = head_group if head_group is not None else (0, 1)
    if H % (U * G):
        raise ValueError("heads must divide into U peers x G groups")
    Hl, Hg = H // U, H // (U * G)
    es = ref.element_size()
    for j, it in zip(jobs, items):
        src, joint, dst = it["src"], it.get("joint"), it["dst"]
        _require_cuda(src, joint, dst)
        if src.dtype != ref.dtype or src.shape[0] != B or src.shape[1] != H or src.shape[3] != D:
            raise ValueError("tensors packed together must agree in dtype, B, H and D")
        if src.stride(3) != 1 and D != 1:
            raise ValueError("the head_dim axis must be contiguous")
        j.src = src.data_ptr() + g * Hg * src.stride(1) * es
        j.src_stride_b, j.src_stride_h, j.src_stride_row = src.stride(0), src.stride(1), src.stride(2)
        j.src_stride_peer = Hl * src.stride(1) if G > 1 else 0
        j.s = src.shape[2]
        if joint is not None:
            if joint.stride(3) != 1 and D != 1:
                raise ValueError("the head_dim axis must be contiguous")
            j.joint = joint.data_ptr() + g * Hg * joint.stride(1) * es
            j.joint_stride_b, j.joint_stride_h, j.joint_stride_row = joint.stride(0), joint.stride(1), joint.stride(2)
            j.joint_stride_peer = Hl * joint.stride(1) if G > 1 else 0
            j.s_joint = joint.shape[2]
            j.joint_front = int(bool(it.get("front", False)))
        j.dst = dst.data_ptr()
        j.dst_peer_stride = int(it["peer_stride"])
    with torch.cuda.device(ref.device):
        _capi.check(_capi.load().xdit_ulysses_pack(jobs, n, _dtype(ref), B, U * Hg, D, U, _stream(ref)),
                    "xdit_ulysses_pack")
    launch_count += 1


def ulysses_pack_peers(items: Sequence[dict], U: int, peer_base: Sequence[int]) -> None:
    """Like :func:`ulysses_pack`, but peer p's block of item j is stored at ``peer_base[p] + dst_offset_j``
    (``dst_offset`` in elements, an item key): the peers' receive buffers are written directly, over NVLink
    for the other ranks (``xdit_ulysses_pack_peers``).  ``peer_base``: ``U`` device addresses."""
    global launch_count
    n = len(items)
    if not 1 <= n <= _capi.XDIT_MAX_PACK_JOBS:
        raise ValueError(f"1..{_capi.XDIT_MAX_PACK_JOBS} tensors per pack call")
    if len(peer_base) != U:
        raise ValueError("one base address per peer")
    jobs = (_capi.PackJob * n)()
    offs = (C.c_int64 * n)()
    ref = items[0]["src"]
    B, H, _, D = ref.shape
    for i, (j, it) in enumerate(zip(jobs, items)):
        src, joint = it["src"], it.get("joint")
        _require_cuda(src, joint)
        if src.dtype != ref.dtype or src.shape[0] != B or src.shape[1] != H or src.shape[3] != D:
            raise ValueError("tensors packed together must agree in dtype, B, H and D")
        if src.stride(3) != 1 and D != 1:
            raise ValueError("the head_dim axis must be contiguous")
        j.src = src.data_ptr()
        j.src_stride_b, j.src_stride_h, j.src_stride_row = src.stride(0), src.stride(1), src.stride(2)
        j.s = src.shape[2]
        if joint is not None:
            j.joint = joint.data_ptr()
            j.joint_stride_b, j.joint_stride_h, j.joint_stride_row = joint.stride(0), joint.stride(1), joint.stride(2)
            j.s_joint = joint.shape[2]
            j.joint_front = int(bool(it.get("front", False)))
        offs[i] = int(it["dst_offset"])
    bases = (C.c_void_p * U)(*[int(x) for x in peer_base])
    with torch.cuda.device(ref.device):
        _capi.check(_capi.load().xdit_ulysses_pack_peers(jobs, n, _dtype(ref), B, H, D, U,
                                                         C.cast(bases, C.POINTER(C.c_void_p)), offs, _stream(ref)),
                    "xdit_ulysses_pack_peers")
    launch_count += 1


class _DeviceMemory:
    """A raw device allocation presented through the CUDA array interface, so that torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def peer_alloc(nbytes: int, device) -> tuple:
    """``(address, handle, uint8 tensor over it)`` of a buffer other processes of this node can map
    (``xdit_peer_alloc``: cudaMalloc + an IPC handle).  Set-up path; free with :func:`peer_free`."""
    ptr = C.c_void_p()
    handle = C.create_string_buffer(_capi.XDIT_PEER_HANDLE_BYTES)
    with torch.cuda.device(device):
        _capi.check(_capi.load().xdit_peer_alloc(int(nbytes), C.byref(ptr), handle), "xdit_peer_alloc")
        view = torch.as_tensor(_DeviceMemory(ptr.value, int(nbytes)), device=torch.device(device))
    return ptr.value, handle.raw, view


def peer_open(handle: bytes, device) -> int:
    """Map a peer's buffer from its handle; returns the local address (``xdit_peer_open``)."""
    ptr = C.c_void_p()
    with torch.cuda.device(device):
        _capi.check(_capi.load().xdit_peer_open(handle, C.byref(ptr)), "xdit_peer_open")
    return ptr.value


def peer_close(ptr: int) -> None:
    _capi.check(_capi.load().xdit_peer_close(C.c_void_p(ptr)), "xdit_peer_close")


def peer_free(ptr: int) -> None:
    _capi.check(_capi.load().xdit_peer_free(C.c_void_p(ptr)), "xdit_peer_free")


def peer_barrier(peer_flags: Sequence[int], local_flags: int, epoch: torch.Tensor, rank: int, device,
                 wait_limit_ns: int = 0) -> None:
    """Flag barrier over peer-mapped memory on the current stream (``xdit_peer_barrier``).  A wait that runs
    out is reported like an attention kernel's: through the device's status words."""
    global launch_count
    U = len(peer_flags)
    arr = (C.c_void_p * U)(*[int(x) for x in peer_flags])
    st = _status(device)
    with torch.cuda.device(device):
        _capi.check(_capi.load().xdit_peer_barrier(C.cast(arr, C.POINTER(C.c_void_p)), C.c_void_p(int(local_flags)),
                                                   C.c_void_p(epoch.data_ptr()), U, int(rank), int(wait_limit_ns),
                                                   C.c_void_p(st.dev.data_ptr()), C.c_void_p(st.host.data_ptr()),
                                                   torch.cuda.current_stream(torch.device(device)).cuda_stream),
                    "xdit_peer_barrier")
    launch_count += 1


def peer_copy(dst_ptr: int, src: torch.Tensor, nbytes: int) -> None:
    """One copy-engine transfer of the first ``nbytes`` bytes of ``src`` (contiguous, on this GPU) to the device
    address ``dst_ptr`` -- possibly a peer's buffer (``peer_open``) -- on the current stream (``xdit_peer_copy``)."""
    _require_cuda(src)
    if not src.is_contiguous() or nbytes > src.numel() * src.element_size():
        raise ValueError("peer_copy needs a contiguous source of at least nbytes bytes")
    with torch.cuda.device(src.device):
        _capi.check(_capi.load().xdit_peer_copy(C.c_void_p(int(dst_ptr)), C.c_void_p(src.data_ptr()), int(nbytes),
                                                _stream(src)), "xdit_peer_copy")


def ulysses_pack_out(x: torch.Tensor) -> torch.Tensor:
    """[B,Hl,S,D] -> [S,B,Hl,D] contiguous (the reference's output-side wire layout)."""
    global launch_count
    _require_cuda(x)
    B, Hl, S, D = x.shape
    dst = torch.empty(S, B, Hl, D, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().xdit_ulysses_pack_out(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2),
                                                       dst.data_ptr(), _dtype(x), B, Hl, S, D, _stream(x)),
                    "xdit_ulysses_pack_out")
    launch_count += 1
    return dst


def ulysses_unpack_out(recv: torch.Tensor, B: int, Hl: int, s: int, D: int, U: int) -> torch.Tensor:
    """recv [U][s][B][Hl][D] -> [B, U*Hl, s, D] contiguous."""
    global launch_count
    _require_cuda(recv)
    dst = torch.empty(B, U * Hl, s, D, dtype=recv.dtype, device=recv.device)
    with torch.cuda.device(recv.device):
        _capi.check(_capi.load().xdit_ulysses_unpack_out(recv.data_ptr(), dst.data_ptr(), _dtype(recv), B, Hl, s,
                                                         D, U, _stream(recv)), "xdit_ulysses_unpack_out")
    launch_count += 1
    return dst


def ulysses_unpack_in(recv: torch.Tensor, B: int, Hl: int, s: int, D: int, U: int) -> torch.Tensor:
    """recv [U][Hl][B][s][D] -> [B, Hl, U*s, D] contiguous."""
    global launch_count
    _require_cuda(recv)
    dst = torch.empty(B, Hl, U * s, D, dtype=recv.dtype, device=recv.device)
    with torch.cuda.device(recv.device):
        _capi.check(_capi.load().xdit_ulysses_unpack_in(recv.data_ptr(), dst.data_ptr(), _dtype(recv), B, Hl, s,
                                                        D, U, _stream(recv)), "xdit_ulysses_unpack_in")
    launch_count += 1
    return dst


def kv_patch_update(k_cache: torch.Tensor, v_cache: torch.Tensor, k_new: torch.Tensor,
                    v_new: torch.Tensor, row_start: int) -> None:
    """Overwrite cache rows [row_start, row_start + n) of [B,H,S,D] caches (``xdit_kv_patch_update``)."""
    global launch_count
    _require_cuda(k_cache, v_cache, k_new, v_new)
    if k_cache.stride() != v_cache.stride() or k_cache.shape != v_cache.shape:
        raise ValueError("K and V caches must share shape and strides")
    p = _capi.KvPatchParams()
    p.dtype = _dtype(k_cache)
    p.B, p.H, p.D = k_cache.shape[0], k_cache.shape[1], k_cache.shape[3]
    p.k_cache, p.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    p.cache_stride_b, p.cache_stride_h, p.cache_stride_row = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    p.cache_rows = k_cache.shape[2]
    p.k_new, p.v_new = _seq(k_new), _seq(v_new)
    p.row_start = int(row_start)
    with torch.cuda.device(k_cache.device):
        _capi.check(_capi.load().xdit_kv_patch_update(C.byref(p), _stream(k_cache)), "xdit_kv_patch_update")
    launch_count += 1


def seq_shard_pad(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows of ``x`` [B, S, C] owned by sequence-parallel rank ``rank`` of ``world`` after zero-padding S
    to a multiple of ``world``: a new contiguous [B, ceil(S/world), C] tensor (``xdit_seq_shard_pad``)."""
    global launch_count
    _require_cuda(x)
    if x.dim() != 3 or (x.stride(2) != 1 and x.shape[2] != 1):
        raise ValueError("expected [B, S, C] with a contiguous last axis")
    B, S, Cn = x.shape
    s = (S + world - 1) // world
    dst = torch.empty(B, s, Cn, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().xdit_seq_shard_pad(x.data_ptr(), x.stride(0), x.stride(1), dst.data_ptr(), _dtype(x),
                                                    B, S, Cn, world, rank, _stream(x)), "xdit_seq_shard_pad")
    launch_count += 1
    return dst


def seq_gather_unpad(recv: torch.Tensor, B: int, s: int, Cn: int, world: int, keep: int) -> torch.Tensor:
    """``recv`` [world][B][s][C] (an all-gather's output) -> [B, keep, C] contiguous, the gathered sequence
    without its ``world*s - keep`` padding rows (``xdit_seq_gather_unpad``)."""
    global launch_count
    _require_cuda(recv)
    dst = torch.empty(B, keep, Cn, dtype=recv.dtype, device=recv.device)
    with torch.cuda.device(recv.device):
        _capi.check(_capi.load().xdit_seq_gather_unpad(recv.data_ptr(), dst.data_ptr(), _dtype(recv), world, B, s, Cn,
                                                       keep, _stream(recv)), "xdit_seq_gather_unpad")
    launch_count += 1
    return dst


def merge_out_lse(o_acc: torch.Tensor, lse_acc: torch.Tensor, out_b: torch.Tensor, lse_b: torch.Tensor,
                  first: bool, out_final: Optional[torch.Tensor] = None) -> None:
    """In-place online-softmax merge of (out_b, lse_b) into fp32 (o_acc, lse_acc)."""
    global launch_count
    _require_cuda(o_acc, lse_acc, out_b, lse_b, out_final)
    if not (o_acc.is_contiguous() and lse_acc.is_contiguous() and out_b.is_contiguous() and lse_b.is_contiguous()):
        raise ValueError("merge_out_lse needs contiguous tensors")
    D = out_b.shape[-1]
    rows = out_b.numel() // D
    with torch.cuda.device(o_acc.device):
        _capi.check(_capi.load().xdit_merge_out_lse(
            o_acc.data_ptr(), lse_acc.data_ptr(), out_b.data_ptr(), lse_b.data_ptr(),
            out_final.data_ptr() if out_final is not None else None, _dtype(out_b), rows, D, int(bool(first)),
            _stream(o_acc)), "xdit_merge_out_lse")
    launch_count += 1


def qk_norm_rope_pack(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, dst_q: torch.Tensor,
                      dst_k: torch.Tensor, dst_v: torch.Tensor, peer_strides: Sequence[int], U: int = 1, *,
                      norm_q_weight: Optional[torch.Tensor] = None, norm_k_weight: Optional[torch.Tensor] = None,
                      eps: float = 1e-6, norm_per_head: bool = False, cos: Optional[torch.Tensor] = None,
                      sin: Optional[torch.Tensor] = None, dst_strides: Optional[Sequence] = None) -> None:
    """RMSNorm(q, k) + rotary embedding + head split + Ulysses pack in one launch (``xdit_qk_norm_rope_pack``).

    ``q, k, v``: projections ``[B, s, heads*D]`` (any batch/row strides, e.g. column slices of a fused
    qkv projection).  ``dst_*``: 1-D tensors positioned at the tensor's slot inside peer 0's block of
    the send buffer, ``peer_strides`` the distance in elements between two peers' blocks.  ``cos, sin``:
    fp32 ``[s, D]``.  ``dst_strides``: optional ``[(head_stride, batch_stride)] * 3`` in elements (``None`` or
    zeros: the packed ``[H/U][B][s][D]`` layout), e.g. to write k and v straight into ``[B,H,S,D]`` buffers.
    """
    global launch_count
    _require_cuda(q, k, v, dst_q, dst_k, dst_v, norm_q_weight, norm_k_weight, cos, sin)
    B, s, HD = q.shape
    if HD % heads or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k and v must be [B, s, heads*D] of one shape")
    if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1:
        raise ValueError("the hidden axis must be contiguous")
    D = HD // heads
    for w in (norm_q_weight, norm_k_weight):
        if w is not None and (w.dtype != q.dtype or not w.is_contiguous() or w.numel() != (D if norm_per_head else HD)):
            raise ValueError("norm weights must be contiguous, in the tensors' dtype, [D] per head or [heads*D]")
    if (cos is None) != (sin is None):
        raise ValueError("cos and sin go together")
    if cos is not None:
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != (s, D) or sin.shape != (s, D):
            raise ValueError("cos and sin must be fp32 [s, D]")
        if cos.stride(1) != 1 or sin.stride(1) != 1 or cos.stride(0) != sin.stride(0):
            raise ValueError("cos and sin need contiguous rows of equal stride")
    p = _capi.PrologueParams(
        dtype=_dtype(q), B=B, H=heads, D=D, s=s, U=U, norm_per_head=int(bool(norm_per_head)), eps=float(eps),
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(),
        q_stride_b=q.stride(0), q_stride_row=q.stride(1), k_stride_b=k.stride(0), k_stride_row=k.stride(1),
        v_stride_b=v.stride(0), v_stride_row=v.stride(1),
        norm_q_weight=norm_q_weight.data_ptr() if norm_q_weight is not None else None,
        norm_k_weight=norm_k_weight.data_ptr() if norm_k_weight is not None else None,
        cos=cos.data_ptr() if cos is not None else None, sin=sin.data_ptr() if sin is not None else None,
        cos_sin_stride_row=cos.stride(0) if cos is not None else 0,
        dst_q=dst_q.data_ptr(), dst_k=dst_k.data_ptr(), dst_v=dst_v.data_ptr(),
        dst_q_peer_stride=int(peer_strides[0]), dst_k_peer_stride=int(peer_strides[1]),
        dst_v_peer_stride=int(peer_strides[2]))
    if dst_strides is not None:
        for i, st in enumerate(dst_strides):
            if st is not None:
                p.dst_stride_h[i], p.dst_stride_b[i] = int(st[0]), int(st[1])
    with torch.cuda.device(q.device):
        _capi.check(_capi.load().xdit_qk_norm_rope_pack(C.byref(p), _stream(q)), "xdit_qk_norm_rope_pack")
    launch_count += 1


def default_scale(D: int) -> float:
    return 1.0 / math.sqrt(D)
