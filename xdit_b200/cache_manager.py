"""PipeFusion stale-KV buffers, same interface as the reference's ``CacheManager``
(``xfuser/core/cache_manager/cache_manager.py:38-101``).

The reference keeps one ``[K || V]`` tensor per attention layer, rebuilt with ``torch.cat`` on
every call, patched by slice-assignment and split again with ``torch.chunk`` -- after which its
callers make both halves contiguous (``usp.py:201-202``).  Here each layer owns a persistent K
cache and a persistent V cache already in attention layout ``[B, H, S, D]``; one kernel launch
(``xdit_kv_patch_update``) writes the fresh rows of both, and the caches themselves are handed to
the attention kernel.  Returned tensors are views of the caches in the caller's axis order.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Union

import torch

from . import ops
from .distributed import get_runtime_state, get_ulysses_parallel_world_size, runtime_state_is_initialized


class CacheEntry:
    def __init__(self, cache_type: str):
        self.cache_type = cache_type
        self.k: Optional[torch.Tensor] = None  # [B, H, S, D]
        self.v: Optional[torch.Tensor] = None

    @property
    def tensors(self):
        return [self.k, self.v]


class CacheManager:
    supported_layer = ["attn"]
    supported_cache_type = ["naive_cache", "sequence_parallel_attn_cache"]

    def __init__(self):
        self.cache: Dict[Tuple[str, Any], CacheEntry] = {}

    def register_cache_entry(self, layer, layer_type: str, cache_type: str = "naive_cache"):
        if layer_type not in self.supported_layer:
            raise ValueError(
                f"Layer type: {layer_type} is not supported. Supported layer type: {self.supported_layer}")
        if cache_type not in self.supported_cache_type:
            raise ValueError(
                f"Cache type: {cache_type} is not supported. Supported cache type: {self.supported_cache_type}")
        self.cache[layer_type, layer] = CacheEntry(cache_type)

    # ------------------------------------------------------------------ reference-shaped entry
    def update_and_get_kv_cache(self, new_kv: Union[torch.Tensor, List[torch.Tensor]], layer: Any,
                                slice_dim: int = 1, layer_type: str = "attn", custom_get_kv=None, **kwargs):
        """``new_kv`` is ``[k, v]`` (or one tensor with K and V concatenated on the last axis) with the
        token axis at ``slice_dim`` (1: ``[B,S,H,D]``, 2: ``[B,H,S,D]``).  Returns full-sequence
        ``(k, v)`` in the same axis order (one concatenated tensor if one was passed)."""
        if custom_get_kv is not None:
            return custom_get_kv(self, new_kv, layer, slice_dim, layer_type, **kwargs)
        return_list = isinstance(new_kv, (list, tuple))
        if return_list:
            k, v = new_kv
        else:
            k, v = torch.chunk(new_kv, 2, dim=-1)
        if k.dim() != 4:
            raise ValueError("KV tensors must be 4-D")
        if slice_dim < 0:
            slice_dim += 4
        if slice_dim not in (1, 2):
            raise ValueError(f"'dim' argument {slice_dim} is not a token axis of a 4-D KV tensor")
        if slice_dim == 1:
            k, v = k.transpose(1, 2), v.transpose(1, 2)
        ko, vo = self.update_and_get_kv(k, v, layer, layer_type)
        if slice_dim == 1:
            ko, vo = ko.transpose(1, 2), vo.transpose(1, 2)
        if return_list:
            return ko, vo
        return torch.cat([ko, vo], dim=-1)

    # ------------------------------------------------------------------ native entry
    def update_and_get_kv(self, k: torch.Tensor, v: torch.Tensor, layer: Any, layer_type: str = "attn"):
        """``k``/``v``: fresh rows as ``[B,H,n,D]`` or, after a Ulysses all-to-all, ``[B,H,U,n,D]``
        (one segment per source rank).  Returns the full ``[B,H,S,D]`` K and V for attention."""
        entry = self.cache[layer_type, layer]
        segs = k.shape[2] if k.dim() == 5 else 1
        n_new = k.shape[-2] * segs
        state_ready = runtime_state_is_initialized()
        num_patch = get_runtime_state().num_pipeline_patch if state_ready else 1
        patch_mode = get_runtime_state().patch_mode if state_ready else False

        if entry.cache_type == "naive_cache":
            # cache_manager.py:103-135
            if num_patch == 1 or not patch_mode:
                return self._store_all(entry, k, v, n_new)
            rs = get_runtime_state()
            start = rs.pp_patches_token_start_idx_local[rs.pipeline_patch_idx]
            end = rs.pp_patches_token_start_idx_local[rs.pipeline_patch_idx + 1]
            return self._patch(entry, k, v, start, end, n_new)

        # sequence_parallel_attn_cache, cache_manager.py:138-194
        U = get_ulysses_parallel_world_size()
        if num_patch == 1:
            return self._as_4d(k), self._as_4d(v)  # returned untouched, nothing is stored
        if not patch_mode:
            # per-rank chunks split per patch and re-joined rank-major == the incoming order
            return self._store_all(entry, k, v, n_new)
        rs = get_runtime_state()
        start = U * rs.pp_patches_token_start_idx_local[rs.pipeline_patch_idx]
        end = U * rs.pp_patches_token_start_idx_local[rs.pipeline_patch_idx + 1]
        return self._patch(entry, k, v, start, end, n_new)

    def rows_for_producer(self, layer: Any, B: int, H: int, n_new: int, D: int, dtype, device,
                          layer_type: str = "attn"):
        """For a caller that produces the fresh K/V rows itself (the fused attention prologue): make sure
        the layer's buffers exist and say where the ``n_new`` rows belong.  Returns ``(k_cache, v_cache,
        row_start)``; the caller writes rows ``[row_start, row_start + n_new)`` of both and then attends to
        the whole buffers.  Same bookkeeping as ``update_and_get_kv`` for a ``naive_cache`` entry
        (``cache_manager.py:103-135``); Ulysses-sharded entries go through ``update_and_get_kv``."""
        entry = self.cache[layer_type, layer]
        if entry.cache_type != "naive_cache":
            raise NotImplementedError("rows_for_producer serves naive_cache entries (no sequence parallelism)")
        state_ready = runtime_state_is_initialized()
        num_patch = get_runtime_state().num_pipeline_patch if state_ready else 1
        patch_mode = get_runtime_state().patch_mode if state_ready else False
        if num_patch == 1 or not patch_mode:
            if entry.k is None or entry.k.shape != (B, H, n_new, D) or entry.k.dtype != dtype \
                    or entry.k.device != device:
                entry.k = torch.empty(B, H, n_new, D, dtype=dtype, device=device)
                entry.v = torch.empty(B, H, n_new, D, dtype=dtype, device=device)
            return entry.k, entry.v, 0
        rs = get_runtime_state()
        start = rs.pp_patches_token_start_idx_local[rs.pipeline_patch_idx]
        end = rs.pp_patches_token_start_idx_local[rs.pipeline_patch_idx + 1]
        if entry.k is None:
            raise RuntimeError("KV cache updated in patch mode before a full-sequence (warm-up) step filled it")
        if end - start != n_new:
            raise RuntimeError(
                f"The expanded size of the tensor ({end - start}) must match the existing size ({n_new})")
        return entry.k, entry.v, start

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _as_4d(x: torch.Tensor) -> torch.Tensor:
        if x.dim() == 4:
            return x
        B, H, G, L, D = x.shape
        return x.reshape(B, H, G * L, D)

    def _store_all(self, entry: CacheEntry, k, v, n_new):
        B, H, D = k.shape[0], k.shape[1], k.shape[-1]
        if entry.k is None or entry.k.shape != (B, H, n_new, D) or entry.k.dtype != k.dtype \
                or entry.k.device != k.device:
            entry.k = torch.empty(B, H, n_new, D, dtype=k.dtype, device=k.device)
            entry.v = torch.empty(B, H, n_new, D, dtype=v.dtype, device=v.device)
        ops.kv_patch_update(entry.k, entry.v, k, v, 0)
        return entry.k, entry.v

    def _patch(self, entry: CacheEntry, k, v, start, end, n_new):
        if entry.k is None:
            raise RuntimeError("KV cache updated in patch mode before a full-sequence (warm-up) step filled it")
        if end - start != n_new:
            raise RuntimeError(
                f"The expanded size of the tensor ({end - start}) must match the existing size ({n_new})")
        ops.kv_patch_update(entry.k, entry.v, k, v, start)
        return entry.k, entry.v


_CACHE_MGR = CacheManager()


def get_cache_manager() -> CacheManager:
    return _CACHE_MGR
