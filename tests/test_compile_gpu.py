"""`torch.compile(fullgraph=True)` over the hot-path entry points, as the reference tests do for every op
(tests/functional/continuous_count_test.py:25, tests/layers/moe_test.py:104-105): the custom ops are
opaque, mutate-out nodes, so the compiled callables must give the same bits as eager."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_compiled_continuous_count_and_swiglu():
    from xma.functional import continuous_count, swiglu, swiglu_packed

    ids = torch.randint(0, 72, (5000,), device="cuda", dtype=torch.int32)
    fn = torch.compile(continuous_count, fullgraph=True)
    assert torch.equal(fn(ids, 72).view(torch.int32), continuous_count(ids, 72).view(torch.int32))

    g = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    u = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y_ref = swiglu(g, u)
    y_ref.sum().backward()
    ref = (y_ref.detach().clone(), g.grad.clone(), u.grad.clone())
    g.grad = u.grad = None
    y = torch.compile(swiglu, fullgraph=True)(g, u)
    y.sum().backward()
    assert torch.equal(y, ref[0]) and torch.equal(g.grad, ref[1]) and torch.equal(u.grad, ref[2])

    x = torch.randn(32, 128, device="cuda", dtype=torch.float16)
    assert torch.equal(torch.compile(swiglu_packed, fullgraph=True)(x), swiglu_packed(x))


@pytest.mark.parametrize("fused", [True, False])
def test_compiled_moe_matches_eager(fused):
    import torch.nn as nn

    from xma.layers import MoE, SwiGLU

    torch.manual_seed(0)
    act = SwiGLU() if fused else nn.GLU()
    moe = MoE(8, 2, 128, 256, act, True, False, 0.02).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(70, 128, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(70, 128, device="cuda", dtype=torch.bfloat16)

    def run(module):
        moe.zero_grad()
        xin = x.clone().requires_grad_()
        y, logits = module(xin)
        y.backward(dy)
        return y.detach(), logits.detach(), xin.grad, moe.c_fc.weight.grad.clone(), moe.c_proj.weight.grad.clone(), \
            moe.gate.weight.grad.clone()

    eager = run(moe)
    compiled = run(torch.compile(moe, fullgraph=True))
    for a, b in zip(eager, compiled):
        if fused:
            assert torch.equal(a, b)  # only opaque custom ops between the inputs and the outputs
        else:
            # the user activation (nn.GLU) is compiled by inductor, which may round differently from eager
            torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-3)
