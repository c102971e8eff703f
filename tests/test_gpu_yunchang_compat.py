"""The yunchang-named single-GPU pieces (xdit_b200/yunchang_compat.py) against the oracle: the
[B,S,H,D] flash-attn-style forward returned by select_flash_attn_impl and the ring-step merge
update_out_and_lse, used the way the reference's legacy ring loop uses them
(xfuser/core/long_ctx_attention/ring/ring_flash_attn.py:104-143)."""
import numpy as np
import pytest
import torch

from oracle import usp_oracle as O
from tests.gpu_util import compare, np64, rand

pytestmark = pytest.mark.gpu


@pytest.fixture()
def yc():
    from xdit_b200 import yunchang_compat

    assert yunchang_compat.install()
    yield yunchang_compat
    yunchang_compat.uninstall()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_ring_loop_spelled_with_yunchang_names(yc, dtype):
    from yunchang.kernels import AttnType, select_flash_attn_impl
    from yunchang.ring.utils import update_out_and_lse

    B, S, H, D, steps = 1, 333, 3, 128, 3
    q = rand((B, S, H, D), dtype, 1)
    ks = [rand((B, S, H, D), dtype, 10 + i) for i in range(steps)]
    vs = [rand((B, S, H, D), dtype, 20 + i) for i in range(steps)]
    fn = select_flash_attn_impl(AttnType.FA, stage="fwd-only")
    out = lse = None
    for k, v in zip(ks, vs):
        block_out, block_lse = fn(q, k, v, dropout_p=0.0, softmax_scale=D ** -0.5, causal=False,
                                  window_size=(-1, -1), softcap=None, alibi_slopes=None, return_softmax=False)
        assert block_out.shape == (B, S, H, D) and block_lse.shape == (B, H, S)
        out, lse = update_out_and_lse(out, lse, block_out, block_lse)
    assert out.dtype == torch.float32 and lse.shape == (B, S, H, 1)
    t = lambda x: np64(x).transpose(0, 2, 1, 3)
    want, want_lse = O.attention_dense(t(q), np.concatenate([t(k) for k in ks], 2),
                                       np.concatenate([t(v) for v in vs], 2))
    compare(out.transpose(1, 2), want, "merged ring steps")
    got_lse = np64(lse.squeeze(-1).transpose(1, 2))
    assert np.abs(got_lse - want_lse).max() < 2e-2
