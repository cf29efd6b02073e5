"""GPU parity of fused_residual_add_rmsnorm (forward and gradients) against the CPU oracle and the stored
outputs of the reference's torch path, on the grid of the reference's own test
(tests/functional/fused_residual_add_rmsnorm_test.py:27-103: 400 rows x sizes 2^i + j, with and without weight,
multiplier None / 0.9, memory_efficient on / off, eager and compiled; output combined as 2 y + 3 residual)."""

import os

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import rmsnorm_oracle as rn

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
EPS = 1e-5

# fp32: absolute tolerances of the reference test (rtol 0; 7.7e-5 for the weight gradient there, over 400 rows of
# N(0,1) data; here the sum is compared relative to its scale). 16-bit: relative to the tensor's largest magnitude.
REL = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


def _close(got, ref, dtype, what):
    got = got.detach().double().cpu().numpy()
    scale = max(float(np.abs(ref).max()), 1e-30)
    err = float(np.abs(got - ref).max()) / scale
    assert np.isfinite(got).all(), what
    assert err <= REL[dtype], f"{what}: max rel err {err:.3e}"


@pytest.mark.parametrize("name", list(gi.RMSNORM_CASES))
def test_rmsnorm_golden(name):
    from xma.functional import fused_residual_add_rmsnorm

    gold = np.load(os.path.join(GOLDEN, "rmsnorm.npz"))
    inp = gi.rmsnorm_inputs(name)
    dev = lambda t: None if t is None else t.cuda().requires_grad_()
    x, r, w = dev(inp["x"]), dev(inp["residual"]), dev(inp["weight"])
    y, xr = fused_residual_add_rmsnorm(x, r, w, gi.RMSNORM_EPS, inp["multiplier"])
    loss = (y * inp["dy"].cuda()).sum()
    if xr is not None:
        loss = loss + (xr * inp["dxr"].cuda()).sum()
    loss.backward()
    np.testing.assert_allclose(y.detach().cpu().numpy(), gold[name + ".y"], rtol=2e-5, atol=4e-6)
    np.testing.assert_allclose(x.grad.cpu().numpy(), gold[name + ".dx"], rtol=2e-5, atol=1e-5)
    if r is not None:
        np.testing.assert_allclose(xr.detach().cpu().numpy(), gold[name + ".xr"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(r.grad.cpu().numpy(), gold[name + ".dr"], rtol=2e-5, atol=1e-5)
    else:
        assert xr is None
    if w is not None:
        np.testing.assert_allclose(w.grad.cpu().numpy(), gold[name + ".dw"], rtol=2e-5, atol=5e-5)


def _sizes():
    sizes = set()
    for i in range(0, 15, 2):
        for j in (0, 1, 3):
            sizes.add(2**i + j)
    sizes.update([3, 24, 576, 2049, 3000, 4096, 5000, 20000])
    return sorted(sizes)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("memory_efficient", [False, True])
@pytest.mark.parametrize("has_weight", [False, True])
@pytest.mark.parametrize("multiplier", [None, 0.9])
def test_rmsnorm_size_grid(dtype, memory_efficient, has_weight, multiplier):
    from xma.functional import fused_residual_add_rmsnorm

    rows = 400 if dtype == torch.float32 else 77
    for cols in _sizes():
        if dtype != torch.float32 and cols not in (1, 3, 24, 64, 257, 576, 2049, 4096, 5000, 20000):
            continue
        rng = np.random.RandomState(cols)
        mk = lambda *s: torch.from_numpy(rng.standard_normal(s).astype(np.float32)).to(dtype)
        x, r = mk(rows, cols), mk(rows, cols)
        w = (1.0 + 0.1 * mk(cols).float()).to(dtype) if has_weight else None
        xd, rd = x.cuda().requires_grad_(), r.cuda().requires_grad_()
        wd = None if w is None else w.cuda().requires_grad_()
        y, xr = fused_residual_add_rmsnorm(xd, rd, wd, EPS, multiplier, memory_efficient)
        (y * 2 + xr * 3).sum().backward()
        torch.cuda.synchronize()

        np_ = lambda t: None if t is None else t.double().numpy()
        # the kernel rounds the new residual stream to the storage type before normalising it; give the oracle
        # that rounded stream so that both sides normalise the same numbers
        xr_ref = np_(xr.detach().cpu())
        exact_y, exact_xr, _ = rn.forward(np_(x), np_(r), np_(w), EPS, multiplier)
        _close(xr, exact_xr, dtype, f"xr cols={cols}")
        ref_y, _, _ = rn.forward(xr_ref, None, np_(w), EPS, None)
        _close(y, ref_y, dtype, f"y cols={cols}")
        dy, dxr = np.full((rows, cols), 2.0), np.full((rows, cols), 3.0)
        dv, _, dw = rn.backward(xr_ref, None, np_(w), EPS, None, dy, dxr)
        m = 1.0 if multiplier is None else multiplier
        _close(xd.grad, dv * m, dtype, f"dx cols={cols}")
        _close(rd.grad, dv, dtype, f"dr cols={cols}")
        if has_weight:
            _close(wd.grad, dw, dtype, f"dw cols={cols}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [64, 520, 2048, 4096, 8192])
@pytest.mark.parametrize("has_residual,has_weight,memory_efficient", [(True, True, False), (False, True, True),
                                                                      (True, False, False)])
def test_rmsnorm_many_rows(dtype, cols, has_residual, has_weight, memory_efficient):
    """More rows than CTAs of the backward kernel, so that each CTA walks several rows through its staged
    pipeline (rows requested ahead, stages reused); random gradients for both outputs."""
    from xma.functional import fused_residual_add_rmsnorm

    rows = 3001
    rng = np.random.RandomState(cols + rows)
    mk = lambda *s: torch.from_numpy(rng.standard_normal(s).astype(np.float32)).to(dtype)
    x = mk(rows, cols)
    r = mk(rows, cols) if has_residual else None
    w = (1.0 + 0.1 * mk(cols).float()).to(dtype) if has_weight else None
    dy = mk(rows, cols)
    dxr = mk(rows, cols) if has_residual else None
    dev = lambda t: None if t is None else t.cuda().requires_grad_()
    xd, rd, wd = dev(x), dev(r), dev(w)
    y, xr = fused_residual_add_rmsnorm(xd, rd, wd, EPS, None, memory_efficient)
    loss = (y * dy.cuda()).sum()
    if has_residual:
        loss = loss + (xr * dxr.cuda()).sum()
    loss.backward()
    torch.cuda.synchronize()

    np_ = lambda t: None if t is None else t.double().numpy()
    stream = np_(xr.detach().cpu()) if has_residual else np_(x)
    ref_y, _, _ = rn.forward(stream, None, np_(w), EPS, None)
    _close(y, ref_y, dtype, "y")
    dv, _, dw = rn.backward(stream, None, np_(w), EPS, None, np_(dy), np_(dxr))
    _close(xd.grad, dv, dtype, "dx")
    if has_residual:
        _close(rd.grad, dv, dtype, "dr")
    if has_weight:
        # a sum over 3001 rows of products rounded to the storage type only at the end: fp32 accumulation
        _close(wd.grad, dw, dtype, "dw")


def test_rmsnorm_without_residual_and_unused_outputs():
    """No residual: the second result is None; with a multiplier the gradient is that of the function computed.
    A residual stream nobody reads contributes no gradient (d(xr) absent, not zeros read from memory)."""
    from xma.functional import fused_residual_add_rmsnorm

    rng = np.random.RandomState(3)
    x = torch.from_numpy(rng.standard_normal((50, 300)).astype(np.float32))
    w = torch.from_numpy((1 + 0.1 * rng.standard_normal(300)).astype(np.float32))
    dy = rng.standard_normal((50, 300))
    for multiplier in (None, 0.5):
        xd, wd = x.cuda().requires_grad_(), w.cuda().requires_grad_()
        y, xr = fused_residual_add_rmsnorm(xd, None, wd, EPS, multiplier)
        assert xr is None
        (y * torch.from_numpy(dy).float().cuda()).sum().backward()
        ref_y, _, _ = rn.forward(x.numpy(), None, w.numpy(), EPS, multiplier)
        dx, _, dw = rn.backward(x.numpy(), None, w.numpy(), EPS, multiplier, dy, None)
        _close(y, ref_y, torch.float32, "y")
        _close(xd.grad, dx, torch.float32, "dx")
        _close(wd.grad, dw, torch.float32, "dw")
    r = torch.from_numpy(rng.standard_normal((50, 300)).astype(np.float32))
    xd, rd = x.cuda().requires_grad_(), r.cuda().requires_grad_()
    y, xr = fused_residual_add_rmsnorm(xd, rd, None, None)  # eps None -> machine epsilon of the dtype
    y.sum().backward()
    eps = float(torch.finfo(torch.float32).eps)
    dx, dr, _ = rn.backward(x.numpy(), r.numpy(), None, eps, None, np.ones((50, 300)), None)
    _close(xd.grad, dx, torch.float32, "dx")
    _close(rd.grad, dr, torch.float32, "dr")


def test_rmsnorm_compiled_matches_eager():
    from xma.functional import fused_residual_add_rmsnorm

    fn = torch.compile(fused_residual_add_rmsnorm, fullgraph=True)
    torch.manual_seed(0)
    x = torch.randn(64, 515, device="cuda", dtype=torch.bfloat16)
    r, w = torch.randn_like(x), torch.randn(515, device="cuda", dtype=torch.bfloat16)
    outs = []
    for f in (fused_residual_add_rmsnorm, fn):
        xd, rd, wd = (t.clone().requires_grad_() for t in (x, r, w))
        y, xr = f(xd, rd, wd, EPS, 0.9)
        (y * 2 + xr * 3).sum().backward()
        outs.append((y, xr, xd.grad, rd.grad, wd.grad))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_rmsnorm_rejects_bad_arguments():
    from xma import KernelBackend
    from xma.functional import fused_residual_add_rmsnorm

    x = torch.randn(4, 8, device="cuda")
    with pytest.raises(AssertionError):
        fused_residual_add_rmsnorm(x, None, torch.ones(7, device="cuda"), EPS)
    with pytest.raises(AssertionError):
        fused_residual_add_rmsnorm(x, None, torch.ones(8, device="cuda", dtype=torch.bfloat16), EPS)
    with pytest.raises(ValueError):
        fused_residual_add_rmsnorm(x, None, None, EPS, kernel_backend=KernelBackend.triton)
    with pytest.raises(RuntimeError):
        fused_residual_add_rmsnorm(x.cpu(), None, None, EPS)
