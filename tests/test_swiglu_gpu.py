"""GPU parity of swiglu / swiglu_packed (forward and gradients) against the CPU oracle, on the
reference's own test distribution: integer-valued inputs in [-8, 8), sizes 2^i + j and 50 odd ones
(tests/functional/swiglu_test.py:24-97, swiglu_packed_test.py:21-51)."""

import os
import random

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# absolute tolerances of the reference tests (rtol 0); bf16 uses torch's assert_close defaults there
FWD_ATOL = {torch.float32: 7e-5, torch.float16: 1e-3}
GRAD_ATOL = {torch.float32: 4.6e-5, torch.float16: 5e-4}


def _sizes():
    rng = random.Random(0)
    sizes = set()
    for i in range(0, 13, 2):
        for j in (0, 1, 7):
            sizes.add((2**i + j, 2**i + j))
    for _ in range(6):
        sizes.add((3000 + rng.randint(-1000, 1000), 3000 + rng.randint(-1000, 1000)))
    sizes.add((4100, 3700))
    return sorted(sizes)


def _close(got, ref, dtype, table):
    got, ref = got.detach().cpu(), ref.detach().cpu()
    if dtype in table:
        torch.testing.assert_close(got, ref, rtol=0, atol=table[dtype])
    else:
        torch.testing.assert_close(got, ref)  # bf16 defaults: rtol 1.6e-2, atol 1e-5


@pytest.mark.parametrize("name", list(gi.SWIGLU_CASES))
def test_swiglu_golden(name):
    from xma.functional import swiglu, swiglu_packed

    gold = np.load(os.path.join(GOLDEN, "swiglu.npz"))
    g, u = gi.swiglu_inputs(name)
    gd, ud = g.cuda().requires_grad_(), u.cuda().requires_grad_()
    y = swiglu(gd, ud)
    y.mean().backward()
    np.testing.assert_allclose(y.detach().cpu().numpy(), gold[name + ".y"], rtol=0, atol=7e-5)
    np.testing.assert_allclose(gd.grad.cpu().numpy(), gold[name + ".dg"], rtol=0, atol=4.6e-5)
    np.testing.assert_allclose(ud.grad.cpu().numpy(), gold[name + ".du"], rtol=1e-5, atol=1e-6)
    rows, cols = g.shape
    x = torch.stack([g, u], dim=-1).reshape(rows, 2 * cols).cuda().requires_grad_()
    yp = swiglu_packed(x)
    yp.mean().backward()
    np.testing.assert_allclose(yp.detach().cpu().numpy(), gold[name + ".packed_y"], rtol=0, atol=7e-5)
    np.testing.assert_allclose(x.grad.cpu().numpy(), gold[name + ".packed_dx"], rtol=0, atol=4.6e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_swiglu_size_grid(dtype):
    from xma.functional import swiglu, swiglu_packed

    for size in _sizes():
        rng = np.random.RandomState(size[0])
        g = torch.from_numpy(rng.randint(-8, 8, size=size).astype(np.float32)).to(dtype)
        u = torch.from_numpy(rng.randint(-8, 8, size=size).astype(np.float32)).to(dtype)
        gd, ud = g.cuda().requires_grad_(), u.cuda().requires_grad_()
        y = swiglu(gd, ud)
        _close(y, orc.swiglu(g, u), dtype, FWD_ATOL)
        y.mean().backward()
        dy = torch.full(size, 1.0 / (size[0] * size[1]), dtype=dtype)
        dg, du = orc.swiglu_backward(g, u, dy)
        _close(gd.grad, dg, dtype, GRAD_ATOL)
        _close(ud.grad, du, dtype, GRAD_ATOL)

        cols = size[1] + (size[1] % 2)
        x = torch.from_numpy(rng.randint(-8, 8, size=(size[0], cols)).astype(np.float32)).to(dtype)
        xd = x.cuda().requires_grad_()
        yp = swiglu_packed(xd)
        _close(yp, orc.swiglu_packed(x), dtype, FWD_ATOL)
        yp.mean().backward()
        dyp = torch.full(yp.shape, 1.0 / yp.numel(), dtype=dtype)
        _close(xd.grad, orc.swiglu_packed_backward(x, dyp), dtype, GRAD_ATOL)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_strided_halves_and_nd(dtype):
    """`swiglu(*h.chunk(2, -1))`: the halves are row-strided views and are read in place."""
    from xma.functional import swiglu

    h = torch.randn(3, 50, 256, dtype=dtype, device="cuda", requires_grad=True)
    g, u = h.chunk(2, dim=-1)
    y = swiglu(g, u)
    assert y.shape == (3, 50, 128)
    y.sum().backward()
    hc = h.detach().cpu()
    gc, uc = hc.chunk(2, dim=-1)
    _close(y, orc.swiglu(gc, uc), dtype, FWD_ATOL)
    dg, du = orc.swiglu_backward(gc, uc, torch.ones_like(gc))
    _close(h.grad, torch.cat([dg, du], dim=-1), dtype, {torch.float32: 1e-5})
    with pytest.raises(AssertionError):
        swiglu(g, u[..., :-1])
