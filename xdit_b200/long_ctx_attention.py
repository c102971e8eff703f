"""The ``[B, S, H, D]``-layout attention layer and ring function of
``xfuser/core/long_ctx_attention`` (``hybrid/attn_layer.py:33-239``,
``ring/ring_flash_attn.py:27-312``), which the reference builds on the un-vendored yunchang
package.  Here they are thin adapters: tensors are viewed as ``[B, H, S, D]`` (a transpose
view, no copy) and handed to the same fused data path as ``USP``.

Names the reference imports from yunchang and that callers touch are provided with the same
spelling: ``AttnType`` (a plain enum: every member maps to the one sm_100a kernel),
``ring_pg`` / ``ulysses_pg`` attributes, ``scatter_idx`` / ``gather_idx`` / ``use_pack_qkv``.
"""
from __future__ import annotations

import math
from enum import Enum
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from . import usp as _usp
from .distributed import PROCESS_GROUP


class AttnType(Enum):
    AITER = "aiter"
    FA = "fa"
    FA3 = "fa3"
    FLASHINFER = "flashinfer"
    TORCH = "torch"
    SAGE_AUTO = "sage_auto"
    SAGE_FP16 = "sage_fp16"
    SAGE_FP16_TRITON = "sage_fp16_triton"
    SAGE_FP8 = "sage_fp8"
    SAGE_FP8_SM90 = "sage_fp8_sm90"
    SPARSE_SAGE = "sparse_sage"
    NPU = "npu"

    @classmethod
    def from_string(cls, s: str):
        for member in cls:
            if member.value == s:
                return member
        raise ValueError(f"'{s}' is not a valid {cls.__name__}")


_DENSE_TYPES = (AttnType.FA, AttnType.FA3, AttnType.TORCH, AttnType.FLASHINFER, AttnType.AITER)


def _group_info(pg):
    if pg is None:
        return 1, 0
    return dist.get_world_size(pg), dist.get_rank(pg)


def xdit_ring_flash_attn_func(
    q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), alibi_slopes=None,
    deterministic=False, return_attn_probs=False, group=None, attn_type=AttnType.FA, attn_processor=None,
    attn_layer=None, joint_tensor_key=None, joint_tensor_value=None, joint_strategy="none",
    q_descale=None, k_descale=None, v_descale=None,
):
    """Ring attention over ``group`` on ``[B, S_local, H, D]`` tensors
    (``ring/ring_flash_attn.py:248-312`` -> ``:27-148``).  Returns ``out`` or, with
    ``return_attn_probs``, ``(out, lse[B,H,S], None)``."""
    if dropout_p:
        raise NotImplementedError("dropout is not implemented")
    assert alibi_slopes is None
    if tuple(window_size) != (-1, -1):
        raise NotImplementedError("sliding-window attention is not part of the dense path")
    if q_descale is not None or k_descale is not None or v_descale is not None:
        raise NotImplementedError("fp8 descale factors belong to the fp8 back-ends")
    if attn_type not in _DENSE_TYPES:
        raise NotImplementedError(f"attn_type {attn_type} is not a dense bf16/fp16 type")
    is_joint = False
    if joint_tensor_key is not None and joint_tensor_value is not None:
        if joint_strategy not in ("front", "rear"):
            raise ValueError(
                f"joint_strategy: {joint_strategy} not supprted. supported joint strategy: ['front', 'rear']")
        is_joint = True
    elif joint_tensor_key is None and joint_tensor_value is None:
        pass
    else:
        raise ValueError("joint_tensor_key and joint_tensor_value should be None or not None simultaneously.")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.size(-1))
    R, _ = _group_info(group)
    t = lambda x: x.transpose(1, 2)
    kw = {}
    if is_joint:
        # joint K/V arrive already head-sliced for this Ulysses rank; there are no joint queries here
        kw = dict(jk=t(joint_tensor_key), jv=t(joint_tensor_value), front=joint_strategy == "front")
    out, lse = _ring_bhsd(t(q), t(k), t(v), softmax_scale, causal, group, R, attn_layer, **kw)
    out = t(out)
    return (out, lse, None) if return_attn_probs else out


def _ring_bhsd(q, k, v, scale, causal, group, R, attn_layer, jk=None, jv=None, front=False):
    from . import ops

    B, H, S, D = q.shape
    if causal and k.shape[2] != S:
        # the legacy ring only ever masks the diagonal block of equal shards (ring_flash_attn.py:104,113);
        # for unequal lengths flash-attn's bottom-right alignment would differ from this kernel's top-left
        raise NotImplementedError("causal ring attention needs equal query and key shard lengths")
    if attn_layer is not None:
        k, v = _usp._update_and_get_kv_cache(k, v, attn_layer)
    out = torch.empty(B, H, S, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    if R == 1:
        ops.attn_fwd(q, k, v, jk, jv, out=out, lse=lse, causal=causal, scale=scale)
        return out, lse
    buf, views = _usp._pack_kv_flat(k, v)
    _usp._ring_native(q, buf, views, jk, jv, front, out, group, scale=scale, causal=causal, lse=lse)
    return out, lse


class xFuserLongContextAttention(torch.nn.Module):
    """Hybrid Ulysses x ring attention layer on ``[B, S_local, H, D]`` tensors."""

    ring_impl_type_supported_kv_cache = ["basic"]

    def __init__(self, scatter_idx: int = 2, gather_idx: int = 1, ring_impl_type: str = "basic",
                 use_pack_qkv: bool = False, use_kv_cache: bool = False, use_sync: bool = False,
                 attn_type: Optional[AttnType] = None, attn_processor: Optional[torch.nn.Module] = None,
                 q_descale=None, k_descale=None, v_descale=None) -> None:
        super().__init__()
        if attn_type is None:
            attn_type = AttnType.FA
        if scatter_idx != 2 or gather_idx != 1:
            raise NotImplementedError("only scatter_idx=2 (heads), gather_idx=1 (sequence) is implemented")
        if ring_impl_type != "basic":
            if use_kv_cache:
                raise RuntimeError(f"ring_impl_type: {ring_impl_type} do not support SP kv cache.")
            raise NotImplementedError(f"ring_impl_type {ring_impl_type}: only 'basic' is implemented")
        if q_descale is not None or k_descale is not None or v_descale is not None:
            raise NotImplementedError("fp8 descale factors belong to the fp8 back-ends")
        self.ring_pg = PROCESS_GROUP.RING_PG
        self.ulysses_pg = PROCESS_GROUP.ULYSSES_PG
        self.scatter_idx = scatter_idx
        self.gather_idx = gather_idx
        self.use_pack_qkv = use_pack_qkv
        self.use_sync = use_sync
        self.attn_type = attn_type
        self.use_kv_cache = use_kv_cache
        self.attn_processor = attn_processor
        self.ring_attn_fn = xdit_ring_flash_attn_func

    def forward(self, attn, query: Tensor, key: Tensor, value: Tensor, *, joint_tensor_query=None,
                joint_tensor_key=None, joint_tensor_value=None, dropout_p=0.0, softmax_scale=None, causal=False,
                window_size=(-1, -1), alibi_slopes=None, deterministic=False, return_attn_probs=False,
                joint_strategy="none") -> Tensor:
        """``hybrid/attn_layer.py:100-239``.  ``query/key/value`` are ``[B, S_local, H, D]``; the joint
        tensors ``[B, S_joint, H, D]`` replicated on every rank.  Returns ``[B, S_local (+S_joint), H, D]``."""
        if dropout_p:
            raise NotImplementedError("dropout is not implemented")
        if tuple(window_size) != (-1, -1) or alibi_slopes is not None:
            raise NotImplementedError("sliding-window / alibi attention is not part of the dense path")
        if self.attn_type not in _DENSE_TYPES:
            raise NotImplementedError(f"attn_type {self.attn_type} is not a dense bf16/fp16 type")
        given = [x is not None for x in (joint_tensor_query, joint_tensor_key, joint_tensor_value)]
        strategy = None
        if all(given):
            if joint_strategy not in ("front", "rear"):
                raise ValueError(
                    f"joint_strategy: {joint_strategy} not supprted. supported joint strategy: ['front', 'rear']")
            strategy = joint_strategy
        elif any(given):
            raise ValueError(
                "joint_tensor_query, joint_tensor_key, and joint_tensor_value should be None or not None simultaneously.")
        t = lambda x: None if x is None else x.transpose(1, 2)
        if (torch.compiler.is_compiling() and not self.use_kv_cache and self.ulysses_pg is PROCESS_GROUP.ULYSSES_PG
                and self.ring_pg is PROCESS_GROUP.RING_PG):
            # under torch.compile the call is one opaque operator (the reference disables compilation of
            # this method altogether, hybrid/attn_layer.py:99)
            from . import compile_ops

            return compile_ops.usp(t(query), t(key), t(value), t(joint_tensor_query), t(joint_tensor_key),
                                   t(joint_tensor_value), strategy or "", bool(causal),
                                   float(softmax_scale) if softmax_scale else 0.0).transpose(1, 2)
        U, u_rank = _group_info(self.ulysses_pg)
        R, _ = _group_info(self.ring_pg)
        out = _usp.usp_native(
            t(query), t(key), t(value), t(joint_tensor_query), t(joint_tensor_key), t(joint_tensor_value), strategy,
            attn if self.use_kv_cache else None, causal, softmax_scale, U, R, u_rank, self.ulysses_pg, self.ring_pg)
        return out.transpose(1, 2)


class xFuserSanaLinearLongContextAttention(xFuserLongContextAttention):
    """Sana's linear attention uses different arithmetic (``ring_flash_attn.py:314-405``) and is
    outside the dense softmax path."""

    def forward(self, *args, **kwargs):
        raise NotImplementedError("Sana linear attention is not part of the dense softmax path")
