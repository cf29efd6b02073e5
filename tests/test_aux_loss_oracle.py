"""The auxiliary-loss oracle against torch autograd of the same formula (CPU). The reference has no such loss, so
this is the oracle's only pin: an independent evaluation of the published definition."""

import numpy as np
import pytest
import torch

from oracle import aux_loss_oracle as orc


@pytest.mark.parametrize("T,E,K", [(9, 4, 2), (64, 16, 4), (200, 72, 8)])
def test_oracle_matches_torch_autograd(T, E, K):
    rng = np.random.RandomState(E)
    logits = rng.standard_normal((T, E))
    x = torch.from_numpy(logits).requires_grad_()
    p = torch.softmax(x, dim=-1)
    selected = torch.sort(x.detach(), dim=-1, descending=True, stable=True).indices[:, :K]
    f = torch.bincount(selected.reshape(-1), minlength=E).double() / T
    loss = E * (f * p.mean(0)).sum()
    loss.backward()
    ref_loss, ref_f = orc.loss(logits, K)
    assert abs(ref_loss - float(loss)) < 1e-12
    np.testing.assert_allclose(ref_f, f.numpy(), rtol=0, atol=0)
    np.testing.assert_allclose(orc.grad(logits, K), x.grad.numpy(), rtol=1e-10, atol=1e-14)
    assert np.array_equal(orc.select(logits, K), selected.numpy())


def test_uniform_router():
    loss, f = orc.loss(np.zeros((32, 8)), 2)
    assert abs(loss - 2.0) < 1e-12 and f[:2].tolist() == [1.0, 1.0] and f[2:].sum() == 0
