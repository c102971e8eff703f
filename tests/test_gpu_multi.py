"""USP on 2 and 4 GPUs over NCCL against the outputs of the unmodified reference (tests/golden).
fp32 inputs take the CUDA-core kernel (tight tolerance); bf16 inputs take the tcgen05 kernel
(tolerance 3e-2 because the fixtures were computed from unrounded fp32 inputs)."""
import pytest
import torch

import os

from tests.usp_worker import HERE, golden_files, run, run_kv, run_prologue

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("mode,dtype,tol", [("usp", "float32", 5e-5), ("usp", "bfloat16", 3e-2),
                                            ("legacy", "bfloat16", 3e-2), ("compat", "float32", 5e-5),
                                            ("yunchang", "bfloat16", 3e-2)])
def test_two_gpus(mode, dtype, tol):
    _need(2)
    run(2, golden_files(2), mode, 29750, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("mode,dtype,tol", [("usp", "float32", 5e-5), ("usp", "bfloat16", 3e-2),
                                            ("yunchang", "float32", 5e-5)])
def test_four_gpus(mode, dtype, tol):
    _need(4)
    run(4, golden_files(4), mode, 29760, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
def test_stale_kv_under_ulysses_two_gpus(dtype, tol):
    _need(2)
    run_kv(2, os.path.join(HERE, "golden", "uspkv_u2r1.npz"), 29770, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("U,R", [(2, 1), (1, 2)])
def test_attention_from_projections_two_gpus(U, R):
    """The processor slice with the fused prologue kernel: Ulysses 2 writes the projections straight into
    the all-to-all send buffer, ring 2 hands [B,H,s,D] tensors to the ring path."""
    _need(2)
    run_prologue(2, U, R, 29780 + R, backend="nccl", dtype_name="bfloat16", tol=3e-2)
