#!/usr/bin/env python
"""Place the reference's own Python sources for the USP attention path under ``oracle/_ref/``.

Test infrastructure, not product code.  The reference (xDiT) is pure Python, so "building" it for
this path means copying the files that the path imports out of a checkout, unmodified, into a
directory that is kept out of version control (``oracle/_ref/`` is git-ignored) but travels with the
working tree to wherever the tests and the benchmark's CPU baseline run::

    XDIT_REFERENCE=<root of an xDiT checkout> python oracle/make_ref.py

The list is the import closure of ``xfuser/model_executor/layers/usp.py`` and
``xfuser/core/cache_manager/cache_manager.py`` when their heavy package ``__init__`` files are
skipped (see ``oracle/ref_import.py``), plus the ``[B,S,H,D]`` layer and ring function under
``xfuser/core/long_ctx_attention``.  Nothing is edited; a missing file is an error.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

FILES = [
    "xfuser/envs.py",
    "xfuser/logger.py",
    "xfuser/config/__init__.py",
    "xfuser/config/args.py",
    "xfuser/config/config.py",
    "xfuser/core/cache_manager/__init__.py",
    "xfuser/core/cache_manager/cache_manager.py",
    "xfuser/core/distributed/__init__.py",
    "xfuser/core/distributed/attention_backend.py",
    "xfuser/core/distributed/attention_schedule.py",
    "xfuser/core/distributed/group_coordinator.py",
    "xfuser/core/distributed/parallel_state.py",
    "xfuser/core/distributed/runtime_state.py",
    "xfuser/core/distributed/sharding.py",
    "xfuser/core/distributed/ssta.py",
    "xfuser/core/distributed/utils.py",
    "xfuser/core/sparge_attention/__init__.py",
    "xfuser/core/sparge_attention/block_mask.py",
    "xfuser/core/sparge_attention/gilbert.py",
    "xfuser/core/sparge_attention/head_balance.py",
    "xfuser/core/sparge_attention/sparge.py",
    "xfuser/model_executor/layers/usp.py",
    "xfuser/core/long_ctx_attention/__init__.py",
    "xfuser/core/long_ctx_attention/hybrid/__init__.py",
    "xfuser/core/long_ctx_attention/hybrid/attn_layer.py",
    "xfuser/core/long_ctx_attention/ring/__init__.py",
    "xfuser/core/long_ctx_attention/ring/ring_flash_attn.py",
    "xfuser/core/long_ctx_attention/ring/ring_npu_flash_attn.py",
]


def reference_root() -> str:
    """``XDIT_REFERENCE``, else a directory ``reference`` beside this repository."""
    return os.environ.get("XDIT_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def available() -> bool:
    return all(os.path.exists(os.path.join(DEST, f)) for f in FILES)


def make(src_root: str | None = None, quiet: bool = False) -> bool:
    """Copy the listed files from ``src_root`` into ``oracle/_ref``.  Returns False (and does
    nothing) when no checkout is given or it does not hold an ``xfuser`` package."""
    src_root = src_root or reference_root()
    if not src_root or not os.path.isdir(os.path.join(src_root, "xfuser")):
        return False
    for rel in FILES:
        src = os.path.join(src_root, rel)
        if not os.path.exists(src):
            raise FileNotFoundError(f"{src}: the reference checkout lacks a file of the USP path")
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    if not quiet:
        print(f"{len(FILES)} reference files copied to {DEST}")
    return True


if __name__ == "__main__":
    if not make():
        sys.exit("set XDIT_REFERENCE to the root of an xDiT checkout (the directory that holds xfuser/)")
