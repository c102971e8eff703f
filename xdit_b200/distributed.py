"""Sequence-parallel process groups and the slice of runtime state the USP hot path reads.

Mirrors the getters of ``xfuser/core/distributed/parallel_state.py:73-101`` and the fields of
``xfuser/core/distributed/runtime_state.py`` that the path consults (``attention_backend``,
PipeFusion patch bookkeeping ``:556-566, 731-745``), plus the two names the reference takes
from yunchang: ``set_seq_parallel_pg`` and ``PROCESS_GROUP`` (``parallel_state.py:494-512``,
``usp.py:11``).  Everything else in those files (DP/CFG/PP/TP groups, config validation) is
host bookkeeping outside this path.

Rank layout: SP rank ``g = ring_rank * U + ulysses_rank``; a Ulysses group is ``U`` contiguous
ranks, a ring group is ``R`` ranks strided by ``U``.
"""
from __future__ import annotations

from typing import List, Optional

import torch.distributed as dist


class _ProcessGroups:
    """Holder with the attribute names of ``yunchang.globals.PROCESS_GROUP``."""

    ULYSSES_PG = None
    RING_PG = None


PROCESS_GROUP = _ProcessGroups()

_ULYSSES_WORLD = 1
_RING_WORLD = 1
_SP_RANK = 0


def set_seq_parallel_pg(sp_ulysses_degree: int, sp_ring_degree: int, rank: int, world_size: int,
                        use_ulysses_low: bool = True, backend: Optional[str] = None) -> None:
    """Create the Ulysses and ring groups for every SP block of ``U*R`` consecutive ranks.

    Same call shape as yunchang's function.  Must be called by all ranks of the default group.
    ``use_ulysses_low=True`` makes Ulysses groups contiguous and ring groups strided.
    """
    global _ULYSSES_WORLD, _RING_WORLD, _SP_RANK
    U, R = int(sp_ulysses_degree), int(sp_ring_degree)
    P = U * R
    if U < 1 or R < 1:
        raise ValueError("degrees must be >= 1")
    if world_size % P != 0:
        raise ValueError(f"world_size {world_size} is not divisible by ulysses*ring = {P}")
    PROCESS_GROUP.ULYSSES_PG = None
    PROCESS_GROUP.RING_PG = None
    for block in range(world_size // P):
        off = block * P
        if use_ulysses_low:
            uly = [[off + r * U + u for u in range(U)] for r in range(R)]
            ring = [[off + r * U + u for r in range(R)] for u in range(U)]
        else:
            ring = [[off + u * R + r for r in range(R)] for u in range(U)]
            uly = [[off + u * R + r for u in range(U)] for r in range(R)]
        for ranks in uly:
            pg = dist.new_group(ranks, backend=backend)
            if rank in ranks:
                PROCESS_GROUP.ULYSSES_PG = pg
        for ranks in ring:
            pg = dist.new_group(ranks, backend=backend)
            if rank in ranks:
                PROCESS_GROUP.RING_PG = pg
    _ULYSSES_WORLD, _RING_WORLD = U, R
    _SP_RANK = rank % P


def init_sequence_parallel(ulysses_degree: int = 1, ring_degree: int = 1, backend: Optional[str] = None) -> None:
    """Convenience: build the groups over the default process group (or no group when P == 1)."""
    global _ULYSSES_WORLD, _RING_WORLD, _SP_RANK
    if ulysses_degree * ring_degree == 1:
        PROCESS_GROUP.ULYSSES_PG = None
        PROCESS_GROUP.RING_PG = None
        _ULYSSES_WORLD = _RING_WORLD = 1
        _SP_RANK = 0
        return
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialised before sequence parallelism")
    set_seq_parallel_pg(ulysses_degree, ring_degree, dist.get_rank(), dist.get_world_size(), backend=backend)


def get_ulysses_parallel_world_size() -> int:
    return _ULYSSES_WORLD


def get_ring_parallel_world_size() -> int:
    return _RING_WORLD


def get_sequence_parallel_world_size() -> int:
    return _ULYSSES_WORLD * _RING_WORLD


def get_sequence_parallel_rank() -> int:
    return _SP_RANK


def get_ulysses_parallel_rank() -> int:
    return _SP_RANK % _ULYSSES_WORLD


def get_ring_parallel_rank() -> int:
    return _SP_RANK // _ULYSSES_WORLD


# --------------------------------------------------------------------------------------
# runtime state
# --------------------------------------------------------------------------------------
class _RuntimeConfig:
    use_spargeattn_head_balance = False


class RuntimeState:
    """Fields of the reference's ``RuntimeState`` / ``DiTRuntimeState`` that the hot path reads."""

    def __init__(self):
        from .attention_backend import AttentionBackendType

        self.attention_backend = AttentionBackendType.B200
        self.runtime_config = _RuntimeConfig()
        self.num_pipeline_patch = 1
        self.patch_mode = False
        self.pipeline_patch_idx = 0
        self.pp_patches_token_start_idx_local: List[int] = [0]
        self.pp_patches_token_num: List[int] = []
        self.split_text_embed_in_sp = False

    # runtime_state.py:113-131
    def set_attention_backend(self, backend) -> None:
        from .attention_backend import ATTENTION_FUNCTION_REGISTRY, AttentionBackendType

        if isinstance(backend, str):
            key = backend.upper()
            if key not in AttentionBackendType.__members__:
                raise ValueError(f"Invalid attention backend: {backend}")
            backend = AttentionBackendType[key]
        if backend not in ATTENTION_FUNCTION_REGISTRY:
            raise NotImplementedError(f"Attention backend {backend} not registered.")
        self.attention_backend = backend

    def set_patches(self, token_num: List[int]) -> None:
        """Install the per-patch token counts of the local stage (``_calc_patches_metadata``)."""
        self.pp_patches_token_num = list(token_num)
        starts = [0]
        for n in token_num:
            starts.append(starts[-1] + n)
        self.pp_patches_token_start_idx_local = starts
        self.num_pipeline_patch = max(1, len(token_num))
        self.pipeline_patch_idx = 0

    # runtime_state.py:556-566
    def set_patched_mode(self, patch_mode: bool) -> None:
        self.patch_mode = patch_mode
        self.pipeline_patch_idx = 0

    def next_patch(self) -> None:
        if self.patch_mode:
            self.pipeline_patch_idx += 1
            if self.pipeline_patch_idx == self.num_pipeline_patch:
                self.pipeline_patch_idx = 0
        else:
            self.pipeline_patch_idx = 0


_RUNTIME: Optional[RuntimeState] = None


def initialize_runtime_state() -> RuntimeState:
    global _RUNTIME
    _RUNTIME = RuntimeState()
    return _RUNTIME


def runtime_state_is_initialized() -> bool:
    return _RUNTIME is not None


def get_runtime_state() -> RuntimeState:
    global _RUNTIME
    if _RUNTIME is None:
        _RUNTIME = RuntimeState()
    return _RUNTIME
