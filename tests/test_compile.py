"""torch.compile traces a processor-shaped module around USP without a graph break: the attention path
is one custom operator (xdit_b200::usp / xdit_b200::attn) with a shape-only fake implementation."""
import pytest
import torch


class _Block(torch.nn.Module):
    """q/k/v projections -> heads -> USP -> head merge -> output projection, as the reference's
    processors are laid out (transformer_wan.py:97-160)."""

    def __init__(self, hidden, heads):
        super().__init__()
        self.heads = heads
        self.q, self.k, self.v, self.o = (torch.nn.Linear(hidden, hidden, bias=False) for _ in range(4))

    def forward(self, x):
        import xdit_b200

        B, s, hid = x.shape
        q, k, v = (p(x).unflatten(2, (self.heads, -1)).transpose(1, 2) for p in (self.q, self.k, self.v))
        a = xdit_b200.USP(q, k, v)
        return x + self.o(a.transpose(1, 2).flatten(2, 3))


def _check(block, x, backend):
    import torch._dynamo as dynamo

    want = block(x)
    dynamo.reset()
    compiled = torch.compile(block, fullgraph=True, backend=backend)  # fullgraph: any graph break raises
    got = compiled(x)
    assert torch.allclose(got.float(), want.float(), atol=1e-5, rtol=1e-5)
    explanation = dynamo.explain(block)(x)
    assert explanation.graph_break_count == 0, explanation.break_reasons
    assert "xdit_b200.usp" in str(explanation.graphs[0].graph) or "xdit_b200::usp" in str(explanation.graphs[0].graph)


def test_usp_block_compiles_without_graph_break_on_cpu(monkeypatch):
    """Host-side check with the kernels replaced by the oracle-backed stand-ins."""
    import xdit_b200
    from tests import fake_ops

    fake_ops.install(monkeypatch)
    xdit_b200.init_sequence_parallel(1, 1)
    torch.manual_seed(0)
    block = _Block(64, 4)
    with torch.no_grad():
        _check(block, torch.randn(1, 24, 64), "eager")


@pytest.mark.gpu
def test_usp_block_compiles_without_graph_break_on_gpu():
    import xdit_b200
    from xdit_b200 import ops

    xdit_b200.init_sequence_parallel(1, 1)
    torch.manual_seed(0)
    block = _Block(512, 4).cuda().to(torch.bfloat16)
    with torch.no_grad():
        _check(block, torch.randn(1, 300, 512, device="cuda", dtype=torch.bfloat16), "aot_eager")
    torch.cuda.synchronize()
    ops.check_status()
