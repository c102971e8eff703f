"""USP on 2 and 4 GPUs over NCCL against the outputs of the unmodified reference (tests/golden).
fp32 inputs take the CUDA-core kernel (tight tolerance); bf16 inputs take the tcgen05 kernel
(tolerance 3e-2 because the fixtures were computed from unrounded fp32 inputs)."""
import pytest
import torch

from tests.usp_worker import golden_files, run

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("mode,dtype,tol", [("usp", "float32", 5e-5), ("usp", "bfloat16", 3e-2),
                                            ("legacy", "bfloat16", 3e-2), ("compat", "float32", 5e-5)])
def test_two_gpus(mode, dtype, tol):
    _need(2)
    run(2, golden_files(2), mode, 29750, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("mode,dtype,tol", [("usp", "float32", 5e-5), ("usp", "bfloat16", 3e-2)])
def test_four_gpus(mode, dtype, tol):
    _need(4)
    run(4, golden_files(4), mode, 29760, backend="nccl", dtype_name=dtype, tol=tol)
