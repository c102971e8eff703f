"""The slice of a DiT attention processor that sits between the q/k/v projections and the output
projection, as one call: RMSNorm(q, k) + rotary embedding + head split + Ulysses pack in a single
kernel, the all-to-all, the attention kernel on the receive buffer, the output all-to-all and the
head merge.

It stands for these lines of the reference's processors::

    query = attn.norm_q(query); key = attn.norm_k(key)            # transformer_wan.py:99-100
    query = query.unflatten(2, (attn.heads, -1)) ...               # :102-104
    query = apply_rotary_emb(query, *rotary_emb) ...               # :106-122
    hidden_states = USP(query.transpose(1, 2), ...).transpose(1, 2)  # :143-150
    hidden_states = hidden_states.flatten(2, 3)                    # :151

(the same steps with a per-head norm in ``transformer_flux.py:113-147,170-219``).  The norm modules
and Flux's rotary helper come from diffusers, which the reference does not vendor: the norm is
``torch.nn.RMSNorm`` semantics, the rotary embedding is the interleaved-pair form that the Wan
processor defines inline.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import ops
from . import usp as _usp
from .distributed import (PROCESS_GROUP, get_ring_parallel_world_size, get_ulysses_parallel_rank,
                          get_ulysses_parallel_world_size)


def qk_norm_rope_heads(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, heads: int, *,
                       norm_q_weight: Optional[torch.Tensor] = None, norm_k_weight: Optional[torch.Tensor] = None,
                       eps: float = 1e-6, norm_per_head: bool = False,
                       rotary_emb: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Projections ``[B, s, heads*D]`` -> normalised, rotated ``q, k`` and ``v`` as ``[B, heads, s, D]``
    tensors (what the processor passes to ``USP``).  One launch; for ``B > 1`` the results are
    ``[heads, B, s, D]`` buffers viewed with the batch axis first."""
    B, s, HD = query.shape
    D = HD // heads
    cos, sin = _cos_sin(rotary_emb, s, D)
    n = heads * B * s * D
    buf = torch.empty(3 * n, dtype=query.dtype, device=query.device)
    ops.qk_norm_rope_pack(query, key, value, heads, buf, buf[n:], buf[2 * n:], (n, n, n), 1,
                          norm_q_weight=norm_q_weight, norm_k_weight=norm_k_weight, eps=eps,
                          norm_per_head=norm_per_head, cos=cos, sin=sin)
    return tuple(buf[i * n:(i + 1) * n].view(heads, B, s, D).permute(1, 0, 2, 3) for i in range(3))


def _cos_sin(rotary_emb, s, D):
    if rotary_emb is None:
        return None, None
    cos, sin = rotary_emb
    # the processors carry [1, s, 1, D] tables (transformer_wan.py:108-120); [s, D] is accepted as well
    cos = cos.reshape(s, D) if cos.numel() == s * D else cos
    sin = sin.reshape(s, D) if sin.numel() == s * D else sin
    if cos.shape != (s, D) or sin.shape != (s, D):
        raise ValueError("rotary_emb must hold cos and sin tables of s x D elements")
    return cos.float().contiguous(), sin.float().contiguous()


def attention_from_projections(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, heads: int, *,
                               norm_q_weight: Optional[torch.Tensor] = None,
                               norm_k_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                               norm_per_head: bool = False,
                               rotary_emb: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                               softmax_scale: Optional[float] = None,
                               out_proj_weight: Optional[torch.Tensor] = None,
                               out_proj_bias: Optional[torch.Tensor] = None, attn_layer=None) -> torch.Tensor:
    """Self-attention of one DiT layer from its q/k/v projections ``[B, s_local, heads*D]`` to the
    tensor the output projection takes, ``[B, s_local, heads*D]``, under the current sequence-parallel
    degrees.  With a Ulysses degree ``U > 1`` and no ring the prologue kernel writes straight into the
    all-to-all send buffer; otherwise it produces ``[B, heads, s, D]`` tensors for ``USP``'s data path.

    With ``out_proj_weight`` (``[hidden, heads*D]``, optional bias) the layer's output projection
    (``attn.to_out[0]``, ``transformer_wan.py:152``, ``transformer_flux.py:210-219``) is applied as well and
    ``[B, s_local, hidden]`` is returned: the attention kernel writes its rows head-merged, so the
    projection reads them where they lie.

    ``attn_layer`` (PipeFusion, no sequence parallelism): the layer's stale-KV buffers are the attention's
    keys and values, and the prologue kernel writes the fresh K and V rows of the current patch straight
    into them -- no separate patch-update pass (``attention_processor.py:286-292`` ->
    ``cache_manager.py:103-135``)."""
    if attn_layer is not None:
        out = _attention_with_stale_kv(query, key, value, heads, norm_q_weight, norm_k_weight, eps, norm_per_head,
                                       rotary_emb, softmax_scale, attn_layer)
        if out_proj_weight is not None:
            out = torch.nn.functional.linear(out, out_proj_weight, out_proj_bias)
        return out
    out = _attention_from_projections(query, key, value, heads, norm_q_weight, norm_k_weight, eps, norm_per_head,
                                      rotary_emb, softmax_scale)
    if out_proj_weight is not None:
        out = torch.nn.functional.linear(out, out_proj_weight, out_proj_bias)
    return out


def _attention_with_stale_kv(query, key, value, heads, norm_q_weight, norm_k_weight, eps, norm_per_head, rotary_emb,
                             softmax_scale, attn_layer):
    from .cache_manager import get_cache_manager

    if get_ulysses_parallel_world_size() * get_ring_parallel_world_size() != 1:
        raise NotImplementedError("the fused stale-KV path serves PipeFusion without sequence parallelism; "
                                  "use USP(..., attn_layer=...) otherwise")
    B, n, HD = query.shape
    D = HD // heads
    kc, vc, start = get_cache_manager().rows_for_producer(attn_layer, B, heads, n, D, query.dtype, query.device)
    S = kc.shape[2]
    cos, sin = _cos_sin(rotary_emb, n, D)
    q_buf = torch.empty(heads * B * n * D, dtype=query.dtype, device=query.device)
    # q in the packed [H][B][n][D] layout; k and v rows at [start, start + n) of the [B,H,S,D] buffers
    ops.qk_norm_rope_pack(query, key, value, heads, q_buf, kc.view(-1)[start * D:], vc.view(-1)[start * D:],
                          (q_buf.numel(), 0, 0), 1, norm_q_weight=norm_q_weight, norm_k_weight=norm_k_weight, eps=eps,
                          norm_per_head=norm_per_head, cos=cos, sin=sin,
                          dst_strides=[None, (S * D, heads * S * D), (S * D, heads * S * D)])
    q4 = q_buf.view(heads, B, n, D).permute(1, 0, 2, 3)
    out = torch.empty(B, n, heads, D, dtype=query.dtype, device=query.device)
    ops.attn_fwd(q4, kc, vc, out=out.permute(0, 2, 1, 3), scale=softmax_scale)
    return out.view(B, n, HD)


def _attention_from_projections(query, key, value, heads, norm_q_weight, norm_k_weight, eps, norm_per_head,
                                rotary_emb, softmax_scale):
    B, s, HD = query.shape
    if HD % heads:
        raise ValueError("hidden size must be divisible by the number of heads")
    D = HD // heads
    U, R = get_ulysses_parallel_world_size(), get_ring_parallel_world_size()
    if U == 1 and R == 1:
        # one GPU: the attention kernel writes its rows straight into [B, s, heads, D], which is the
        # head-merged tensor the output projection takes
        q, k, v = qk_norm_rope_heads(query, key, value, heads, norm_q_weight=norm_q_weight,
                                     norm_k_weight=norm_k_weight, eps=eps, norm_per_head=norm_per_head,
                                     rotary_emb=rotary_emb)
        out = torch.empty(B, s, heads, D, dtype=query.dtype, device=query.device)
        ops.attn_fwd(q, k, v, out=out.permute(0, 2, 1, 3), scale=softmax_scale)
        return out.view(B, s, HD)
    if U == 1 or R > 1:
        q, k, v = qk_norm_rope_heads(query, key, value, heads, norm_q_weight=norm_q_weight,
                                     norm_k_weight=norm_k_weight, eps=eps, norm_per_head=norm_per_head,
                                     rotary_emb=rotary_emb)
        out = _usp.usp_native(q, k, v, None, None, None, None, None, False, softmax_scale, U, R,
                              get_ulysses_parallel_rank(), PROCESS_GROUP.ULYSSES_PG, PROCESS_GROUP.RING_PG)
        # [B, heads, s, D] -> [B, s, heads*D]
        return out.permute(0, 2, 1, 3).reshape(B, s, HD)
    assert heads % U == 0, "h must be divisible by world_size, got {} and {}".format(heads, U)
    Hl = heads // U
    cos, sin = _cos_sin(rotary_emb, s, D)
    blk = Hl * B * s * D
    stride = 3 * blk
    send = torch.empty(U * stride, dtype=query.dtype, device=query.device)
    ops.qk_norm_rope_pack(query, key, value, heads, send, send[blk:], send[2 * blk:], (stride, stride, stride), U,
                          norm_q_weight=norm_q_weight, norm_k_weight=norm_k_weight, eps=eps,
                          norm_per_head=norm_per_head, cos=cos, sin=sin)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=PROCESS_GROUP.ULYSSES_PG)
    shape, strides = (B, Hl, U, s, D), (s * D, B * s * D, stride, D, 1)
    q5 = recv.as_strided(shape, strides, 0)
    k5 = recv.as_strided(shape, strides, blk)
    v5 = recv.as_strided(shape, strides, 2 * blk)
    out_send = torch.empty(U * blk, dtype=query.dtype, device=query.device)
    out5 = out_send.as_strided(shape, (s * D, B * s * D, blk, D, 1), 0)
    ops.attn_fwd(q5, k5, v5, out=out5, scale=softmax_scale)
    out_recv = torch.empty_like(out_send)
    dist.all_to_all_single(out_recv, out_send, group=PROCESS_GROUP.ULYSSES_PG)
    # received [heads][B][s][D] -> [B, s, heads*D]
    return out_recv.view(heads, B, s, D).permute(1, 2, 0, 3).reshape(B, s, HD)
