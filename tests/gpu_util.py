"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import usp_oracle as O

TOL_MAX_ABS = 2e-2   # bf16/fp16 outputs vs the oracle on the same (rounded) inputs
TOL_COS = 0.9999


def rand(shape, dtype, seed, device="cuda", scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(device)


def np64(x):
    return x.detach().float().cpu().double().numpy()


def flat4(x):
    if x.dim() == 5:
        B, H, G, L, D = x.shape
        return x.reshape(B, H, G * L, D)
    return x


def oracle_attn(q, k, v, k2=None, v2=None, causal=False, scale=None):
    kk, vv = np64(flat4(k)), np64(flat4(v))
    if k2 is not None:
        kk = np.concatenate([kk, np64(k2)], axis=2)
        vv = np.concatenate([vv, np64(v2)], axis=2)
    return O.attention_dense(np64(flat4(q)), kk, vv, scale=scale, causal=causal)


def compare(got, want, what="", max_abs=TOL_MAX_ABS, cos=TOL_COS):
    g = np64(got).reshape(-1)
    w = np.asarray(want, dtype=np.float64).reshape(-1)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite values in the result"
    err = np.abs(g - w).max()
    c = float(g @ w / (np.linalg.norm(g) * np.linalg.norm(w) + 1e-30))
    assert err <= max_abs, f"{what}: max-abs error {err:.4g} > {max_abs}"
    assert c >= cos, f"{what}: cosine {c:.6f} < {cos}"
    return err, c
