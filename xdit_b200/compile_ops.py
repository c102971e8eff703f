"""``torch.library`` custom operators over the attention path, so that ``torch.compile`` traces a DiT
block around ``USP`` / ``xFuserLongContextAttention`` as one opaque node instead of breaking the graph at
the ctypes calls (the reference wraps its own non-traceable kernels the same way,
``xfuser/core/distributed/attention_backend.py:383-399``).

* ``xdit_b200::attn``  -- one dense attention call, ``(q, k, v[, joint k, v]) -> (out, lse)``;
* ``xdit_b200::usp``   -- a whole ``USP`` call under the current sequence-parallel state (pack, collectives,
  attention, return exchange), ``(q, k, v[, joint q, k, v]) -> out``.

Both are functional (they allocate their results) and carry shape-only "fake" implementations for
tracing.  ``xdit_b200.USP`` and the ``[B,S,H,D]`` layer route through them while Dynamo is tracing and
call the kernels directly otherwise.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch.library import custom_op, register_fake

from . import ops


@custom_op("xdit_b200::attn", mutates_args=())
def attn(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, joint_key: Optional[torch.Tensor],
         joint_value: Optional[torch.Tensor], is_causal: bool, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    out, lse = ops.attn_fwd(query, key, value, joint_key, joint_value, causal=is_causal,
                            scale=scale if scale > 0 else None, want_lse=True)
    return out, lse


@register_fake("xdit_b200::attn")
def _attn_fake(query, key, value, joint_key, joint_value, is_causal, scale):
    B, H, Sq, D = query.shape
    return (torch.empty((B, H, Sq, D), dtype=query.dtype, device=query.device),
            torch.empty((B, H, Sq), dtype=torch.float32, device=query.device))


@custom_op("xdit_b200::usp", mutates_args=())
def usp(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, joint_query: Optional[torch.Tensor],
        joint_key: Optional[torch.Tensor], joint_value: Optional[torch.Tensor], joint_strategy: str,
        is_causal: bool, scale: float) -> torch.Tensor:
    from . import usp as _usp
    from .distributed import (PROCESS_GROUP, get_ring_parallel_world_size, get_ulysses_parallel_rank,
                              get_ulysses_parallel_world_size)

    out = _usp.usp_native(query, key, value, joint_query, joint_key, joint_value, joint_strategy or None, None,
                          is_causal, scale if scale > 0 else None, get_ulysses_parallel_world_size(),
                          get_ring_parallel_world_size(),
                          get_ulysses_parallel_rank(), PROCESS_GROUP.ULYSSES_PG, PROCESS_GROUP.RING_PG)
    # a custom operator may not return a view of an input; the data path never does, but the result can
    # be a permuted view of a fresh buffer, which is fine
    return out


@register_fake("xdit_b200::usp")
def _usp_fake(query, key, value, joint_query, joint_key, joint_value, joint_strategy, is_causal, scale):
    B, H, s, D = query.shape
    sj = joint_query.shape[2] if joint_query is not None else 0
    return torch.empty((B, H, s + sj, D), dtype=query.dtype, device=query.device)
