"""xdit_b200: B200 (sm_100a) implementation of xDiT's Unified-Sequence-Parallel attention path.

Public surface (same names as the reference modules they stand in for):

* ``xdit_b200.usp``                 -- ``USP``, ``attention``, ``ring_attn``  (xfuser/model_executor/layers/usp.py)
* ``xdit_b200.long_ctx_attention``  -- ``xFuserLongContextAttention``, ``xdit_ring_flash_attn_func``, ``AttnType``
* ``xdit_b200.attention_backend``   -- ``AttentionBackendType``, ``ATTENTION_FUNCTION_REGISTRY``, ``register_attention_function``
* ``xdit_b200.cache_manager``       -- ``get_cache_manager`` (PipeFusion stale-KV buffers)
* ``xdit_b200.distributed``         -- sequence-parallel groups and the runtime state the path reads
* ``xdit_b200.ops``                 -- tensor-level wrappers over the C ABI declared in ``include/xdit_b200.h``

All arithmetic runs in ``libxdit_b200.so`` (built in-tree by ``python -m xdit_b200.build``).
"""
from .attention_backend import ATTENTION_FUNCTION_REGISTRY, AttentionBackendType, register_attention_function
from .cache_manager import get_cache_manager
from .distributed import (
    PROCESS_GROUP,
    get_ring_parallel_rank,
    get_ring_parallel_world_size,
    get_runtime_state,
    get_sequence_parallel_rank,
    get_sequence_parallel_world_size,
    get_ulysses_parallel_rank,
    get_ulysses_parallel_world_size,
    init_sequence_parallel,
    initialize_runtime_state,
    set_seq_parallel_pg,
)
from .long_ctx_attention import AttnType, xFuserLongContextAttention, xdit_ring_flash_attn_func
from .usp import USP, attention, ring_attn

__version__ = "0.1.0"
