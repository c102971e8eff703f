"""Sequence and CFG sharding at the boundary of a DiT forward pass: the steps the reference's model
wrappers run once per forward around the transformer blocks.

* entry -- pad the token axis with zeros up to a multiple of the sequence-parallel degree and keep this
  rank's chunk: ``_chunk_and_pad_sequence`` (``xfuser/model_executor/models/transformers/
  transformer_wan.py:219-234``), ``_pad_to_sp_divisible`` + ``torch.chunk`` (``transformer_flux.py:279-284,
  307-309``).  The padded tokens are real tokens to the blocks (they are projected and attended to, not
  masked); that is the reference's behaviour and is kept.
* exit -- gather the shards along the token axis and drop the padding: ``_gather_and_unpad``
  (``transformer_wan.py:236-239``), ``get_sp_group().all_gather(sample, dim=-2)`` followed by
  ``sample[:, :-padding_length]`` (``transformer_flux.py:333-336``), on top of
  ``GroupCoordinator.all_gather`` (``xfuser/core/distributed/group_coordinator.py:221-262``); and the
  classifier-free-guidance gather along the batch axis (``transformer_flux.py:334``).

The reference builds the padded tensor with ``torch.cat`` (a copy of the whole sequence on every rank)
and re-lays the gathered tensor out with ``movedim`` + ``reshape`` (another full copy) before slicing the
padding off.  Here each side is one pass over the bytes that are kept: ``xdit_seq_shard_pad`` writes only
the local rows (zeros where the sequence has ended), the collective is one ``all_gather_into_tensor``, and
``xdit_seq_gather_unpad`` writes ``[B, S, C]`` without the padding -- or nothing at all when the gathered
buffer already is that tensor (batch 1 and no padding).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import ops
from .distributed import get_sequence_parallel_rank, get_sequence_parallel_world_size

_SP_GROUP = None  # process group spanning the U*R ranks of one sequence-parallel block (None: default group)


def set_sequence_parallel_group(group) -> None:
    """The group the token-axis gather runs over (``get_sp_group().device_group`` in the reference).
    ``None`` selects the default group, which is right when every rank belongs to one SP block."""
    global _SP_GROUP
    _SP_GROUP = group


def _to_3d(x: torch.Tensor, dim: int) -> Tuple[torch.Tensor, Tuple[int, ...], int]:
    """View ``x`` as [B, S, C] with S the axis ``dim`` (leading axes folded into B, trailing into C)."""
    if dim < 0:
        dim += x.dim()
    if not 0 <= dim < x.dim():
        raise AssertionError(f"Invalid dim ({dim}) for input tensor with shape {tuple(x.shape)}")
    lead = 1
    for n in x.shape[:dim]:
        lead *= n
    trail = 1
    for n in x.shape[dim + 1:]:
        trail *= n
    return x.reshape(lead, x.shape[dim], trail), tuple(x.shape), dim


def pad_amount(seq_len: int, world: Optional[int] = None) -> int:
    """Zero rows needed to make ``seq_len`` a multiple of the sequence-parallel degree."""
    world = get_sequence_parallel_world_size() if world is None else world
    return (world - seq_len % world) % world


def shard_sequence(x: torch.Tensor, dim: int = 1, rank: Optional[int] = None, world: Optional[int] = None
                   ) -> Tuple[torch.Tensor, int]:
    """This rank's chunk of ``x`` along ``dim`` after zero-padding that axis to a multiple of the
    sequence-parallel degree.  Returns ``(chunk, pad_amount)``; the chunk is a new contiguous tensor."""
    world = get_sequence_parallel_world_size() if world is None else world
    rank = get_sequence_parallel_rank() if rank is None else rank
    x3, shape, dim = _to_3d(x, dim)
    pad = pad_amount(shape[dim], world)
    if world == 1:
        return x, 0
    local = ops.seq_shard_pad(x3, rank, world)
    return local.view(shape[:dim] + (local.shape[1],) + shape[dim + 1:]), pad


def gather_sequence(x: torch.Tensor, dim: int = -2, pad: int = 0, group=None, world: Optional[int] = None
                    ) -> torch.Tensor:
    """All ranks' chunks joined along ``dim`` (rank order), the last ``pad`` rows dropped."""
    world = (get_sequence_parallel_world_size() if world is None else world)
    if world == 1:
        if pad:
            d = dim if dim >= 0 else dim + x.dim()
            return x.narrow(d, 0, x.shape[d] - pad)
        return x
    group = _SP_GROUP if group is None else group
    x3, shape, dim = _to_3d(x.contiguous(), dim)
    B, s, C = x3.shape
    recv = torch.empty(world, B, s, C, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(recv.view(world * B, s, C), x3, group=group)
    keep = world * s - pad
    if B == 1 and pad == 0:
        out3 = recv.view(1, world * s, C)  # [W][1][s][C] already is [1][W*s][C]
    else:
        out3 = ops.seq_gather_unpad(recv, B, s, C, world, keep)
    return out3.view(shape[:dim] + (keep,) + shape[dim + 1:])


def gather_cfg(x: torch.Tensor, group, world: int, dim: int = 0) -> torch.Tensor:
    """Classifier-free-guidance branches joined along the batch axis
    (``get_cfg_group().all_gather(sample, dim=0)``): the collective's output is the result."""
    if world == 1:
        return x
    if dim != 0:
        return gather_sequence(x, dim=dim, pad=0, group=group, world=world)
    x = x.contiguous()
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out
