"""Host-side orchestration of xdit_b200 (send-buffer layouts, strided receive views, all-to-all
and ring schedules) under gloo ranks on CPU.  The device kernels are replaced by the
oracle-backed stand-ins of tests/fake_ops.py, so what is checked here is the Python logic only;
the kernels themselves are checked on the GPU (tests marked gpu).  Expected values are the
outputs of the unmodified reference (tests/golden)."""
import pytest

import os

from tests.usp_worker import HERE, golden_files, run, run_kv


@pytest.mark.parametrize("mode", ["usp", "legacy", "compat"])
def test_world2_matches_reference(mode):
    run(2, golden_files(2), mode, 29720 + ["usp", "legacy", "compat"].index(mode))


@pytest.mark.parametrize("mode", ["usp", "legacy"])
def test_world4_matches_reference(mode):
    run(4, golden_files(4), mode, 29730 + ["usp", "legacy"].index(mode))


def test_stale_kv_under_ulysses_matches_reference():
    """USP(attn_layer=...) with PipeFusion patches and Ulysses degree 2: the fresh rows reach the cache
    manager as two segments of the all-to-all receive buffer."""
    run_kv(2, os.path.join(HERE, "golden", "uspkv_u2r1.npz"), 29741)
