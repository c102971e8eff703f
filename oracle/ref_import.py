"""Import the reference's own modules for the USP attention path from ``oracle/_ref`` (or from a
checkout named by ``XDIT_REFERENCE``), unmodified.

Test infrastructure, not product code: used by the tests that replay the reference next to this
package and by the benchmark's CPU-baseline legs.  The reference's package ``__init__`` files pull in
diffusers and every model wrapper; they are skipped by pre-seeding bare namespace packages in
``sys.modules`` plus a three-attribute ``diffusers`` stub, the recipe that produced the golden
fixtures (``tests/golden/make_golden.py``).
"""
from __future__ import annotations

import importlib
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
_NAMESPACES = ["xfuser", "xfuser.core", "xfuser.model_executor", "xfuser.model_executor.layers"]


def root() -> str | None:
    """Directory that holds the reference's ``xfuser`` package, or None."""
    for cand in (os.path.join(HERE, "_ref"), os.environ.get("XDIT_REFERENCE", "")):
        if cand and os.path.exists(os.path.join(cand, "xfuser", "model_executor", "layers", "usp.py")):
            return cand
    return None


def seed_namespaces(ref_root: str) -> None:
    if "diffusers" not in sys.modules:
        stub = types.ModuleType("diffusers")
        stub.__version__ = "0.35.2"
        stub.DiffusionPipeline = object
        sys.modules["diffusers"] = stub
    # With a GPU present the reference's usp.py takes PROCESS_GROUP from the (un-vendored, absent) yunchang
    # package at import time (usp.py:10-13); configure_usp() replaces that attribute anyway, so a bare
    # holder is enough for the import.  A yunchang that is already importable is left alone.
    if "yunchang" not in sys.modules:
        try:
            importlib.import_module("yunchang.globals")
        except ImportError:
            pkg, glob = types.ModuleType("yunchang"), types.ModuleType("yunchang.globals")
            pkg.__path__ = []
            glob.PROCESS_GROUP = type("PROCESS_GROUP", (), {"ULYSSES_PG": None, "RING_PG": None})
            pkg.globals = glob
            pkg.__xdit_b200_shim__ = glob.__xdit_b200_shim__ = True  # may be replaced by the package's own shim
            sys.modules["yunchang"], sys.modules["yunchang.globals"] = pkg, glob
    for name in _NAMESPACES:
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = [os.path.join(ref_root, *name.split("."))]
            sys.modules[name] = mod


def import_usp():
    """(usp, attention_backend, cache_manager, runtime_state) modules of the reference."""
    ref_root = root()
    if ref_root is None:
        raise ImportError("the reference sources are not available (run oracle/make_ref.py)")
    seed_namespaces(ref_root)
    usp = importlib.import_module("xfuser.model_executor.layers.usp")
    backend = importlib.import_module("xfuser.core.distributed.attention_backend")
    cache = importlib.import_module("xfuser.core.cache_manager.cache_manager")
    rts = importlib.import_module("xfuser.core.distributed.runtime_state")
    return usp, backend, cache, rts


def import_long_ctx_attention():
    """(attn_layer, ring_flash_attn) modules of the reference's ``[B,S,H,D]`` layer.  They take the
    yunchang names only when ``torch.cuda.is_available()`` says so at import time
    (``hybrid/attn_layer.py:9-21``, ``ring/ring_flash_attn.py:10-18``), so that query is answered
    with True for the duration of the import; a ``yunchang`` module tree must be importable."""
    import torch

    ref_root = root()
    if ref_root is None:
        raise ImportError("the reference sources are not available (run oracle/make_ref.py)")
    import_usp()  # envs, logger and the distributed package import first, seeing the real device state
    real = torch.cuda.is_available
    torch.cuda.is_available = lambda: True
    try:
        layer = importlib.import_module("xfuser.core.long_ctx_attention.hybrid.attn_layer")
        ring = importlib.import_module("xfuser.core.long_ctx_attention.ring.ring_flash_attn")
    finally:
        torch.cuda.is_available = real
    return layer, ring


class FakeRuntimeState:
    """The fields of the reference's runtime state that the hot path reads."""

    class _Cfg:
        use_spargeattn_head_balance = False

    def __init__(self, backend):
        self.attention_backend = backend
        self.runtime_config = self._Cfg()
        self.num_pipeline_patch = 1
        self.patch_mode = False
        self.pipeline_patch_idx = 0
        self.pp_patches_token_start_idx_local = [0]
        self.pp_patches_token_num = []


def configure_usp(usp, backend_mod, U, R, uly_rank, uly_pg, ring_pg, backend_member=None):
    """Point the reference's ``usp`` module at explicit groups and degrees (it reads them through
    module-level getters that normally come from its global parallel state)."""

    class PG:
        ULYSSES_PG = uly_pg
        RING_PG = ring_pg

    usp.PROCESS_GROUP = PG
    usp.get_ulysses_parallel_world_size = lambda: U
    usp.get_ulysses_parallel_rank = lambda: uly_rank
    usp.get_ring_parallel_world_size = lambda: R
    usp.get_sequence_parallel_world_size = lambda: U * R
    if backend_member is None:
        backend_member = (backend_mod.AttentionBackendType.SDPA if R == 1
                          else backend_mod.AttentionBackendType.SDPA_FLASH)
    state = FakeRuntimeState(backend_member)
    usp.get_runtime_state = lambda: state
    return state
