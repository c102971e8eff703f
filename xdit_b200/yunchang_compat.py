"""A ``yunchang``-shaped module tree served by this package.

The reference builds its ``[B, S, H, D]`` attention layer and its ring function on the un-vendored
yunchang package (``setup.py:34``, ``yunchang>=0.6.0``) and gates sequence parallelism on being able
to import five names from it (``xfuser/envs.py:342-360``).  ``install()`` registers modules under
``sys.modules`` that carry exactly the names the reference imports, each implemented here on top of
the sm_100a kernels, so that the reference's wrappers import and run without the third-party package:

===============================  ==========================================================
``yunchang``                     ``set_seq_parallel_pg, ring_flash_attn_func, UlyssesAttention,
                                 LongContextAttention, LongContextAttentionQKVPacked``
                                 (``envs.py:346-352``, ``parallel_state.py:495``,
                                 ``hybrid/attn_layer.py:10``)
``yunchang.globals``             ``PROCESS_GROUP, HAS_SPARSE_SAGE_ATTENTION``
                                 (``usp.py:11``, ``attn_layer.py:17``)
``yunchang.kernels``             ``AttnType, select_flash_attn_impl``
                                 (``attention_processor.py:59``, ``ring_flash_attn.py:13``)
``yunchang.comm.all_to_all``     ``SeqAllToAll4D`` (``attn_layer.py:16``)
``yunchang.ring.utils``          ``RingComm, update_out_and_lse`` (``ring_flash_attn.py:11``)
``yunchang.ring.ring_flash_attn``  ``RingFlashAttnFunc, ring_flash_attn_backward``
                                 (``ring_flash_attn.py:12,214``), ``ring_flash_attn_forward``
                                 (``usp_legacy.py:9``)
``yunchang.ring.ring_pytorch_attn``  ``ring_pytorch_attn_func`` (``usp_legacy.py:10``)
``yunchang.ring.ring_npu_flash_attn``, ``update_npu_out``  names only (``ring_npu_flash_attn.py:11-13``);
                                 they raise when called
===============================  ==========================================================

None of this is yunchang's code: the semantics are the ones the reference's call sites rely on
(tensor layouts, argument order, return values).  Forward only; backward entry points raise.
A real yunchang that is already imported is left alone unless ``install(force=True)``.
"""
from __future__ import annotations

import math
import sys
import types
from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from . import usp as _usp
from .distributed import PROCESS_GROUP, set_seq_parallel_pg
from .long_ctx_attention import AttnType, _DENSE_TYPES, _group_info, xdit_ring_flash_attn_func

HAS_SPARSE_SAGE_ATTENTION = False


# ------------------------------------------------------------------------------------------
# yunchang.comm.all_to_all
# ------------------------------------------------------------------------------------------
class SeqAllToAll4D:
    """``SeqAllToAll4D.apply(group, x, scatter_idx, gather_idx, use_sync=False)`` on
    ``[B, S, H, D]`` tensors (``hybrid/attn_layer.py:183-202, 232-236``): scatter heads / gather
    sequence (2, 1) before attention and the inverse (1, 2) after it.  Forward only."""

    @staticmethod
    def apply(group, x: torch.Tensor, scatter_idx: int = 2, gather_idx: int = 1, use_sync: bool = False):
        U, _ = _group_info(group)
        if U <= 1:
            return x
        xt = x.transpose(1, 2)  # [B, H, S, D] view
        if scatter_idx == 2 and gather_idx == 1:
            y = _usp._input_all_to_all(xt, U, group)
        elif scatter_idx == 1 and gather_idx == 2:
            y = _usp._output_all_to_all(xt, U, group)
        else:
            raise NotImplementedError("SeqAllToAll4D: (scatter_idx, gather_idx) must be (2, 1) or (1, 2)")
        if use_sync:
            torch.cuda.current_stream(x.device).synchronize()
        return y.transpose(1, 2)


# ------------------------------------------------------------------------------------------
# yunchang.ring.utils
# ------------------------------------------------------------------------------------------
class RingComm:
    """Neighbour exchange helper of the legacy ring loop (``ring_flash_attn.py:52,84-87,140-143``):
    ``send_recv`` queues a send to the next rank and a receive from the previous one, ``commit``
    posts everything queued as one batch, ``wait`` completes it."""

    def __init__(self, process_group):
        self._group = process_group
        self._ops = []
        self._reqs = None
        self.rank = dist.get_rank(process_group)
        self.world_size = dist.get_world_size(process_group)
        self.send_rank = (self.rank + 1) % self.world_size
        self.recv_rank = (self.rank - 1) % self.world_size
        if process_group is not None:
            self.send_rank = dist.get_global_rank(process_group, self.send_rank)
            self.recv_rank = dist.get_global_rank(process_group, self.recv_rank)

    def send_recv(self, to_send: torch.Tensor, recv_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
        res = torch.empty_like(to_send) if recv_tensor is None else recv_tensor
        self._ops.append(dist.P2POp(dist.isend, to_send, self.send_rank, group=self._group))
        self._ops.append(dist.P2POp(dist.irecv, res, self.recv_rank, group=self._group))
        return res

    def commit(self):
        if self._reqs is not None:
            raise RuntimeError("commit called twice")
        self._reqs = dist.batch_isend_irecv(self._ops)

    def wait(self):
        if self._reqs is None:
            raise RuntimeError("wait called before commit")
        for r in self._reqs:
            r.wait()
        self._reqs = None
        self._ops = []


def update_out_and_lse(out, lse, block_out, block_lse, slice_=None):
    """Online-softmax merge of one ring step (``ring_flash_attn.py:138``).

    ``block_out`` is ``[B, S, H, D]`` in the compute dtype, ``block_lse`` ``[B, H, S]`` fp32.  The
    running pair is ``out`` ``[B, S, H, D]`` fp32 and ``lse`` ``[B, S, H, 1]`` fp32; pass ``None`` for
    both on the first step.  Returns the updated pair (updated in place after the first step).
    """
    if slice_ is not None:
        raise NotImplementedError("update_out_and_lse: slice_ is only used by the zig-zag variants")
    B, S, H, D = block_out.shape
    first = out is None
    if first:
        out = torch.empty(B, S, H, D, dtype=torch.float32, device=block_out.device)
        lse = torch.empty(B, S, H, 1, dtype=torch.float32, device=block_out.device)
    # one row per (b, s, h): the block's lse is brought to that row order
    lse_rows = block_lse.transpose(1, 2).contiguous()
    ops.merge_out_lse(out, lse.view(B, S, H), block_out.contiguous(), lse_rows, first)
    return out, lse


# ------------------------------------------------------------------------------------------
# yunchang.kernels
# ------------------------------------------------------------------------------------------
def select_flash_attn_impl(impl_type=AttnType.FA, stage: str = "fwd-only", attn_processor=None):
    """Return the dense kernel as a ``[B, S, H, D]`` function with the flash-attn forward calling
    convention used at ``ring_flash_attn.py:106-136``: ``fn(q, k, v, dropout_p=..., softmax_scale=...,
    causal=..., window_size=..., softcap=..., alibi_slopes=..., return_softmax=...) -> (out, lse)``."""
    if stage != "fwd-only":
        raise NotImplementedError("select_flash_attn_impl: only the forward stage exists (inference path)")
    if impl_type not in _DENSE_TYPES:
        raise NotImplementedError(f"attn_type {impl_type} is not a dense bf16/fp16 type")

    def fwd(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=None,
            alibi_slopes=None, return_softmax=False, **unused):
        if dropout_p:
            raise NotImplementedError("dropout is not implemented")
        if alibi_slopes is not None or tuple(window_size) != (-1, -1) or softcap:
            raise NotImplementedError("alibi, sliding windows and softcap are not part of the dense path")
        if softmax_scale is None:
            softmax_scale = 1.0 / math.sqrt(q.size(-1))
        B, S, H, D = q.shape
        if causal and k.shape[1] != S:
            # flash-attn aligns a causal mask to the bottom-right corner, the kernel here (like torch
            # SDPA) to the top-left; the two agree only for equal lengths, which is all the ring uses
            raise NotImplementedError("causal attention with Sq != Sk: the flash-attn (bottom-right) mask "
                                      "alignment is not implemented")
        out = torch.empty(B, S, H, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
        ops.attn_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), out=out.transpose(1, 2), lse=lse,
                     causal=causal, scale=softmax_scale)
        return out, lse

    return fwd


# ------------------------------------------------------------------------------------------
# yunchang (top level) and yunchang.ring.ring_flash_attn
# ------------------------------------------------------------------------------------------
def ring_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                         alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None,
                         attn_type=AttnType.FA, attn_processor=None):
    """Plain ring attention on ``[B, S_local, H, D]`` (no joint tensors, no KV cache)."""
    return xdit_ring_flash_attn_func(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                                     deterministic, return_attn_probs, group, attn_type, attn_processor)


class RingFlashAttnFunc(torch.autograd.Function):
    """The autograd function the reference subclasses (``ring_flash_attn.py:151``: it overrides
    ``forward`` / ``backward`` and calls ``.apply`` with its own argument list, which only works on a
    real ``torch.autograd.Function``).  Applied directly it is plain ring attention.  Forward only."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes, deterministic,
                return_softmax, group, attn_type=AttnType.FA, attn_processor=None):
        return ring_flash_attn_func(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                                    deterministic, return_softmax, group, attn_type, attn_processor)

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("the attention backward pass is not part of this inference path")


def ring_flash_attn_forward(process_group, q, k, v, softmax_scale, dropout_p=0, causal=True, window_size=(-1, -1),
                            alibi_slopes=None, deterministic=False, attn_type=AttnType.FA, attn_processor=None):
    """``(out, lse)`` form of the ring function (imported by ``xfuser/model_executor/layers/usp_legacy.py:9``)."""
    out, lse, _ = xdit_ring_flash_attn_func(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                                            deterministic, True, process_group, attn_type, attn_processor)
    return out, lse


def ring_pytorch_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                           alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None):
    """The "pure torch" ring of yunchang (``usp_legacy.py:10,42``): the same ring on the same kernel here."""
    return xdit_ring_flash_attn_func(q, k, v, dropout_p, softmax_scale, causal, window_size, alibi_slopes,
                                     deterministic, return_attn_probs, group)


def ring_flash_attn_backward(*args, **kwargs):
    raise NotImplementedError("the attention backward pass is not part of this inference path")


# Ascend-NPU names that ``xfuser/core/long_ctx_attention/ring/ring_npu_flash_attn.py:11-13,173`` imports
# whenever a GPU is present; they have to exist for that package to import, and raise when used.
def update_npu_out(*args, **kwargs):
    raise NotImplementedError("Ascend NPU attention is not part of this package")


class RingNpuFlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, *args, **kwargs):
        raise NotImplementedError("Ascend NPU attention is not part of this package")

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("Ascend NPU attention is not part of this package")


def ring_npu_flash_attn_backward(*args, **kwargs):
    raise NotImplementedError("Ascend NPU attention is not part of this package")


class LongContextAttention(torch.nn.Module):
    """Base class shape the reference's layer derives from (``hybrid/attn_layer.py:33-97``): holds
    ``ring_pg, ulysses_pg, scatter_idx, gather_idx, use_pack_qkv, use_sync, attn_type,
    attn_processor`` and, called directly, runs Ulysses x ring attention on ``[B, S_local, H, D]``."""

    def __init__(self, scatter_idx: int = 2, gather_idx: int = 1, ring_impl_type: str = "basic",
                 use_pack_qkv: bool = False, use_sync: bool = False, attn_type: AttnType = AttnType.FA,
                 attn_processor: Optional[torch.nn.Module] = None) -> None:
        super().__init__()
        self.ring_pg = PROCESS_GROUP.RING_PG
        self.ulysses_pg = PROCESS_GROUP.ULYSSES_PG
        self.scatter_idx = scatter_idx
        self.gather_idx = gather_idx
        self.use_pack_qkv = use_pack_qkv
        self.use_sync = use_sync
        self.attn_type = attn_type
        self.attn_processor = attn_processor
        self.ring_impl_type = ring_impl_type
        self.ring_attn_fn = ring_flash_attn_func

    def forward(self, query, key, value, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False, *args):
        if dropout_p or alibi_slopes is not None or tuple(window_size) != (-1, -1) or softcap:
            raise NotImplementedError("dropout, alibi, sliding windows and softcap are not part of the dense path")
        U, u_rank = _group_info(self.ulysses_pg)
        R, _ = _group_info(self.ring_pg)
        t = lambda x: x.transpose(1, 2)
        out = _usp.usp_native(t(query), t(key), t(value), None, None, None, None, None, causal, softmax_scale,
                              U, R, u_rank, self.ulysses_pg, self.ring_pg)
        return out.transpose(1, 2)


class LongContextAttentionQKVPacked(LongContextAttention):
    """Same layer fed with one ``[B, S_local, 3, H, D]`` tensor."""

    def forward(self, qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                alibi_slopes=None, deterministic=False, return_attn_probs=False, *args):
        q, k, v = qkv.unbind(2)
        return super().forward(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                               deterministic, return_attn_probs)


class UlyssesAttention(torch.nn.Module):
    """Ulysses-only attention on ``[B, S_local, H, D]`` over ``sequence_process_group``."""

    def __init__(self, sequence_process_group=None, scatter_idx: int = 2, gather_idx: int = 1,
                 attn_type: AttnType = AttnType.FA) -> None:
        super().__init__()
        self.spg = sequence_process_group
        self.scatter_idx = scatter_idx
        self.gather_idx = gather_idx
        self.attn_type = attn_type

    def forward(self, query, key, value, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False, *args):
        if dropout_p or alibi_slopes is not None or tuple(window_size) != (-1, -1) or softcap:
            raise NotImplementedError("dropout, alibi, sliding windows and softcap are not part of the dense path")
        pg = self.spg if self.spg is not None else PROCESS_GROUP.ULYSSES_PG
        U, u_rank = _group_info(pg)
        t = lambda x: x.transpose(1, 2)
        out = _usp.usp_native(t(query), t(key), t(value), None, None, None, None, None, causal, softmax_scale,
                              U, 1, u_rank, pg, None)
        return out.transpose(1, 2)


_TREE = {
    "yunchang": dict(set_seq_parallel_pg=set_seq_parallel_pg, ring_flash_attn_func=ring_flash_attn_func,
                     UlyssesAttention=UlyssesAttention, LongContextAttention=LongContextAttention,
                     LongContextAttentionQKVPacked=LongContextAttentionQKVPacked, __version__="0.6.0+xdit_b200"),
    "yunchang.globals": dict(PROCESS_GROUP=PROCESS_GROUP, HAS_SPARSE_SAGE_ATTENTION=HAS_SPARSE_SAGE_ATTENTION,
                             set_seq_parallel_pg=set_seq_parallel_pg),
    "yunchang.kernels": dict(AttnType=AttnType, select_flash_attn_impl=select_flash_attn_impl),
    "yunchang.comm": dict(SeqAllToAll4D=SeqAllToAll4D),
    "yunchang.comm.all_to_all": dict(SeqAllToAll4D=SeqAllToAll4D),
    "yunchang.ring": dict(ring_flash_attn_func=ring_flash_attn_func, RingFlashAttnFunc=RingFlashAttnFunc),
    "yunchang.ring.utils": dict(RingComm=RingComm, update_out_and_lse=update_out_and_lse,
                                update_npu_out=update_npu_out),
    "yunchang.ring.ring_flash_attn": dict(RingFlashAttnFunc=RingFlashAttnFunc,
                                          ring_flash_attn_func=ring_flash_attn_func,
                                          ring_flash_attn_forward=ring_flash_attn_forward,
                                          ring_flash_attn_backward=ring_flash_attn_backward),
    "yunchang.ring.ring_pytorch_attn": dict(ring_pytorch_attn_func=ring_pytorch_attn_func),
    "yunchang.ring.ring_npu_flash_attn": dict(RingNpuFlashAttnFunc=RingNpuFlashAttnFunc,
                                              ring_npu_flash_attn_backward=ring_npu_flash_attn_backward),
}


def install(force: bool = False) -> bool:
    """Register the module tree above under ``sys.modules``.  Returns False (and changes nothing) when
    a ``yunchang`` that is not this shim is already imported and ``force`` is not set."""
    present = sys.modules.get("yunchang")
    if present is not None and not getattr(present, "__xdit_b200_shim__", False) and not force:
        return False
    mods = {}
    for name, names in _TREE.items():
        m = types.ModuleType(name, f"{name} names served by xdit_b200.yunchang_compat")
        m.__dict__.update(names)
        m.__xdit_b200_shim__ = True
        if name in ("yunchang", "yunchang.comm", "yunchang.ring"):
            m.__path__ = []  # packages: sub-modules below are importable by dotted name
        mods[name] = m
    for name, m in mods.items():
        parent, _, leaf = name.rpartition(".")
        if parent:
            setattr(mods[parent], leaf, m)
    sys.modules.update(mods)
    return True


def uninstall() -> None:
    """Remove the shim's modules (a real yunchang is left alone)."""
    for name in list(sys.modules):
        if (name == "yunchang" or name.startswith("yunchang.")) and getattr(sys.modules[name],
                                                                            "__xdit_b200_shim__", False):
            del sys.modules[name]
