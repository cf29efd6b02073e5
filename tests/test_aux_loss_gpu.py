"""GPU parity of the auxiliary load-balancing loss (forward and gradient) against its CPU oracle; the oracle itself
is checked against torch autograd of the same formula in tests/test_aux_loss_oracle.py."""

import numpy as np
import pytest
import torch

from oracle import aux_loss_oracle as orc

pytestmark = pytest.mark.gpu

# relative to the largest magnitude of the reference tensor; the loss is an fp32 scalar of order top_k
TOL = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T,E,K", [(1, 1, 1), (7, 8, 2), (300, 64, 8), (1000, 128, 8), (513, 72, 4), (40, 1000, 32),
                                   (5000, 256, 1)])
def test_load_balancing_loss_matches_oracle(dtype, T, E, K):
    from xma.functional import load_balancing_loss

    rng = np.random.RandomState(T + E)
    bias = np.log(1.0 / np.arange(1, E + 1) ** 1.2)  # a skewed router
    logits = torch.from_numpy((rng.standard_normal((T, E)) + bias[rng.permutation(E)]).astype(np.float32)).to(dtype)
    ref_loss, _ = orc.loss(logits.float().numpy(), K)
    ref_grad = orc.grad(logits.float().numpy(), K, d_loss=0.7)

    x = logits.cuda().requires_grad_()
    out = load_balancing_loss(x, K)
    assert out.dtype == torch.float32 and out.dim() == 0
    (out * 0.7).backward()
    assert abs(float(out.detach()) - ref_loss) <= 1e-4 * max(1.0, abs(ref_loss)), (float(out.detach()), ref_loss)
    got = x.grad.double().cpu().numpy()
    scale = max(float(np.abs(ref_grad).max()), 1e-30)
    assert np.isfinite(got).all()
    assert float(np.abs(got - ref_grad).max()) / scale <= TOL[dtype]


def test_uniform_router_gives_top_k_and_compiles():
    from xma.functional import load_balancing_loss

    logits = torch.zeros(64, 16, device="cuda")
    assert abs(float(load_balancing_loss(logits, 4)) - 4.0) < 1e-5  # ties go to the lowest ids; P is uniform
    x = torch.randn(200, 32, device="cuda", dtype=torch.bfloat16)
    eager = load_balancing_loss(x, 2)
    compiled = torch.compile(load_balancing_loss, fullgraph=True)(x, 2)
    assert torch.equal(eager, compiled)


def test_loss_consumes_the_layers_router_logits():
    """End to end: the logits `MoE.forward` returns feed the loss, and its gradient reaches the gate weight."""
    from xma.functional import load_balancing_loss
    from xma.layers import MoE, SwiGLU

    torch.manual_seed(0)
    moe = MoE(8, 2, 64, 128, SwiGLU(), True, False, 0.02).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(100, 64, device="cuda", dtype=torch.bfloat16)
    y, logits = moe(x)
    aux = load_balancing_loss(logits, 2)
    (y.float().mean() + 0.01 * aux).backward()
    ref, _ = orc.loss(logits.detach().float().cpu().numpy(), 2)
    assert abs(float(aux) - ref) <= 1e-3 * ref
    assert torch.isfinite(moe.gate.weight.grad.float()).all() and float(moe.gate.weight.grad.abs().max()) > 0
