"""Attention back-end registry with the reference's contract
(``xfuser/core/distributed/attention_backend.py:23, 429-463``):

    func(query, key, value, dropout_p, is_causal, attention_kwargs=None) -> (out[B,H,Sq,D], lse[B,H,Sq] | None)

The enum keeps the reference's member names so that ``--attention_backend`` strings and
``RuntimeState.set_attention_backend`` calls keep working.  Every dense bf16/fp16 member is
served by the one sm_100a kernel of this package; there is no library dispatch.  Members whose
numerics differ (fp8, fp4, sparse, AMD, Ascend) stay unregistered, which surfaces as the same
``NotImplementedError`` the reference raises for an unregistered back-end (``usp.py:205-216``).
"""
from __future__ import annotations

from enum import Enum

import torch

from . import ops

ATTENTION_FUNCTION_REGISTRY = {}


class AttentionBackendType(Enum):
    SDPA = "SDPA"
    SDPA_MATH = "SDPA with Math backend"
    SDPA_EFFICIENT = "SDPA with memory-efficient backend"
    SDPA_FLASH = "SDPA with FLASH backend"
    FLASH = "Flash Attention V2"
    CUDNN = "cuDNN"
    FLASH_3 = "Flash Attention V3"
    FLASH_3_FP8 = "Flash Attention v3 FP8"
    NVTE_FP8 = "NVTE FP8"
    FLASH_4 = "Flash Attention V4"
    FLASH_4_FP4 = "Flash Attention V4 FP4"
    SAGE = "Sage Attention"
    FLEX_BLOCK_ATTN = "Flex Block Attention"
    AITER = "AITER"
    AITER_FP8 = "AITER FP8"
    AITER_MLA = "AITER MLA"
    AITER_SAGE = "AITER Sage"
    AITER_SPARSE_SAGE = "AITER Sparse Sage"
    AITER_SAGE_V2 = "AITER Sage V2"
    AITER_SPARSE_SAGE_V2 = "AITER Sparse Sage V2"
    AITER_SPARGE = "AITER Sparge"
    AITER_SPARGE_V2 = "AITER Sparge V2"
    FLEX_BLOCK_SPARGE = "Flex Block Sparge"
    AITER_FLYDSL = "AITER FlyDSL"
    NPU = "NPU"
    B200 = "B200 tcgen05"  # not in the reference: the kernel of this package under its own name


def register_attention_function(backend_type):
    """Decorator registering ``func`` under ``backend_type`` (``attention_backend.py:456-463``)."""

    def decorator(func):
        ATTENTION_FUNCTION_REGISTRY[backend_type] = func
        return func

    return decorator


_UNSUPPORTED_KWARGS = ("attn_mask", "indices_k", "cu_seqlens_k", "max_seqlen_k")


def reject_masked(attention_kwargs) -> None:
    """Masked / variable-length calls are outside the dense path this package implements."""
    if attention_kwargs:
        for key in _UNSUPPORTED_KWARGS:
            if attention_kwargs.get(key) is not None:
                raise NotImplementedError(
                    f"attention_kwargs[{key!r}] selects masked/varlen attention, which the dense "
                    "sm_100a kernel does not implement; keep such calls on the reference's stock back-ends"
                )


def b200_attn_call(query, key, value, dropout_p=0.0, is_causal=False, attention_kwargs=None):
    """Dense attention on the sm_100a kernel; returns ``(out, lse)`` with lse [B,H,Sq] fp32."""
    if dropout_p:
        raise NotImplementedError("dropout is not implemented (the DiT callers always pass 0.0)")
    reject_masked(attention_kwargs)
    if torch.compiler.is_compiling():
        from . import compile_ops

        return compile_ops.attn(query, key, value, None, None, bool(is_causal), 0.0)
    return ops.attn_fwd(query, key, value, causal=is_causal, want_lse=True)


b200_attn_call.is_xdit_b200_native = True

for _member in (
    AttentionBackendType.B200,
    AttentionBackendType.SDPA,
    AttentionBackendType.SDPA_MATH,
    AttentionBackendType.SDPA_EFFICIENT,
    AttentionBackendType.SDPA_FLASH,
    AttentionBackendType.FLASH,
    AttentionBackendType.CUDNN,
    AttentionBackendType.FLASH_3,
    AttentionBackendType.FLASH_4,
):
    ATTENTION_FUNCTION_REGISTRY[_member] = b200_attn_call
