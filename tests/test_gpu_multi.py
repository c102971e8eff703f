"""USP on 1, 2 and 4 GPUs over NCCL against the outputs of the unmodified reference (tests/golden).
fp32 inputs take the CUDA-core kernel (tight tolerance); bf16 inputs take the tcgen05 kernel and are
compared, at max-abs 2e-2, with the fixture's `out_bf16`: what the reference returns for the same
inputs after rounding them to bf16."""
import pytest
import torch

import os

from tests.usp_worker import HERE, golden_files, run, run_flux_joint, run_kv, run_prologue

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _need_reference():
    from oracle import make_ref, ref_import

    if ref_import.root() is None and not make_ref.make(quiet=True):
        pytest.skip("the reference's sources are not here (oracle/make_ref.py makes oracle/_ref from a checkout)")


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 2e-2)])
def test_reference_layer_on_the_shim_one_gpu(dtype, tol):
    """The reference's own xFuserLongContextAttention.forward and ring function, unmodified, on top of
    the yunchang-shaped names of this package, with the real kernels (one rank: no collectives run, but
    every call site of the layer does)."""
    _need_reference()
    run(1, golden_files(1), "ref_layer", 29748, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 2e-2)])
def test_reference_layer_on_the_shim_multi_gpu(world, dtype, tol):
    _need(world)
    _need_reference()
    run(world, golden_files(world), "ref_layer", 29790 + world, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("mode,dtype,tol", [("usp", "float32", 5e-5), ("usp", "bfloat16", 2e-2),
                                            ("legacy", "bfloat16", 2e-2), ("compat", "float32", 5e-5),
                                            ("yunchang", "bfloat16", 2e-2), ("usp_pipelined", "bfloat16", 2e-2),
                                            ("usp_pipelined", "float32", 5e-5), ("usp_peer", "bfloat16", 2e-2),
                                            ("usp_peer", "float32", 5e-5)])
def test_two_gpus(mode, dtype, tol):
    _need(2)
    run(2, golden_files(2), mode, 29750, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("mode,dtype,tol", [("usp", "float32", 5e-5), ("usp", "bfloat16", 2e-2),
                                            ("yunchang", "float32", 5e-5), ("usp_pipelined", "bfloat16", 2e-2),
                                            ("usp_peer", "bfloat16", 2e-2), ("usp_peer", "float32", 5e-5)])
def test_four_gpus(mode, dtype, tol):
    _need(4)
    run(4, golden_files(4), mode, 29760, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 2e-2)])
def test_stale_kv_under_ulysses_two_gpus(dtype, tol):
    _need(2)
    run_kv(2, os.path.join(HERE, "golden", "uspkv_u2r1.npz"), 29770, backend="nccl", dtype_name=dtype, tol=tol)


@pytest.mark.parametrize("U,R", [(2, 1), (1, 2)])
def test_attention_from_projections_two_gpus(U, R):
    """The processor slice with the fused prologue kernel: Ulysses 2 writes the projections straight into
    the all-to-all send buffer, ring 2 hands [B,H,s,D] tensors to the ring path."""
    _need(2)
    run_prologue(2, U, R, 29780 + R, backend="nccl", dtype_name="bfloat16", tol=2e-2)


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 2e-2)])
def test_flux_joint_case_at_full_size_two_gpus(dtype, tol):
    """Ulysses 2 over NCCL at the full Flux-shaped joint case: 24 heads x 128, 4096 image + 512 joint text
    tokens (rear), seed 0; fp32 (CUDA-core kernel) and bf16 (tcgen05 kernel) against the float64 oracle."""
    _need(2)
    run_flux_joint(2, 29762, backend="nccl", dtype_name=dtype, tol=tol)
