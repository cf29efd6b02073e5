"""End-to-end parity of xma.layers.MoE on the GPU against the CPU oracle (and, in fp32, against the
stored outputs of the reference's own torch path): routing bit-exact, outputs and gradients within
tolerance, forward and backward, fused SwiGLU and generic activations."""

import os

import numpy as np
import pytest
import torch

import inputs as gi
from helpers import REL_TOL, assert_close_rel
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# absolute tolerances of the reference's MoE test (tests/layers/moe_test.py:113-157), used as a
# second gate beside the relative one
REF_ATOL_OUT = {torch.float32: 5.1e-3, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}
REF_ATOL_DX = {torch.float32: 5.9e-3, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}
REF_ATOL_DW = {torch.float32: 3e-2, torch.float16: 2e-3, torch.bfloat16: 7.9e-3}


def _activation(name):
    import torch.nn as nn

    from xma.layers import SwiGLU, SwiGLUPacked

    return {"swiglu": SwiGLU(), "swiglu_packed": SwiGLUPacked(), "glu": nn.GLU(),
            "gelu_tanh": nn.GELU(approximate="tanh")}[name]


def _build(name, dtype):
    from xma.layers import MoE

    T, H, I, E, K, act = gi.MOE_CASES[name]
    inp = gi.moe_inputs(name, dtype)
    moe = MoE(E, K, H, I, _activation(act), act != "gelu_tanh", False, 0.02).to(device="cuda", dtype=dtype)
    with torch.no_grad():
        moe.gate.weight.copy_(inp["gate"])
        moe.c_fc.weight.copy_(inp["w1"])
        moe.c_proj.weight.copy_(inp["w2"])
    return moe, inp


def _run_and_compare(name, dtype, impl):
    from xma import _lib, ops
    from xma.layers.moe import build_route_plan

    moe, inp = _build(name, dtype)
    prev = ops.set_gemm_impl(impl)
    try:
        x = inp["x"].cuda().requires_grad_()
        y, logits = moe(x)
        y.backward(inp["dy"].cuda())
        torch.cuda.synchronize()
    finally:
        ops.set_gemm_impl(prev)
    assert _lib.read_and_clear_device_status() == 0
    assert y.dtype == dtype and logits.shape == (x.size(0), moe.num_experts)

    # The oracle runs in fp32 on the same (already rounded) values and takes the GPU's router logits,
    # so that the routing decision is compared on identical numbers.
    f32 = lambda t: t.detach().float().cpu()
    ref = orc.moe_forward_backward(f32(inp["x"]), f32(inp["gate"]), f32(inp["w1"]), f32(inp["w2"]), inp["top_k"],
                                   inp["activation"], dy=f32(inp["dy"]), router_logits=f32(logits))
    # integer outputs, bit-exact
    with torch.no_grad():
        _, weights, selected = moe._compute_routing_weights(x.detach())
        plan = build_route_plan(selected, moe.num_experts)
    assert torch.equal(selected.cpu().long(), ref.selected_experts)
    assert np.array_equal(plan.expert_frequency.cpu().numpy(), ref.sort.counts)
    assert np.array_equal(plan.offsets_incl.cpu().numpy(), ref.sort.offsets_incl)
    assert np.array_equal(plan.sorted_expert_idxs.cpu().numpy(), ref.sort.sorted_expert_idxs)
    assert np.array_equal(plan.sorted_scattered_idxs.cpu().numpy(), ref.sort.sorted_scattered_idxs)

    tol = REL_TOL[dtype]
    assert_close_rel(weights, ref.router_weights, 1e-6 if dtype == torch.float32 else 8e-3, "router_weights")
    assert_close_rel(y, ref.y, tol, "y")
    assert_close_rel(moe.c_fc.weight.grad, ref.grads["c_fc"], tol, "c_fc.weight.grad")
    assert_close_rel(moe.c_proj.weight.grad, ref.grads["c_proj"], tol, "c_proj.weight.grad")
    # x.grad and gate.weight.grad also flow through the router: rebuild them from the oracle's d_logits
    d_logits = ref.grads["router_logits"]
    dx_ref = ref.grads["x_experts"] + d_logits @ f32(inp["gate"])
    dgate_ref = d_logits.t() @ f32(inp["x"])
    assert_close_rel(x.grad, dx_ref, tol, "x.grad")
    assert_close_rel(moe.gate.weight.grad, dgate_ref, 2 * tol, "gate.weight.grad")
    # second gate: the reference test's absolute tolerances. They were chosen for gradients of O(1e-1)
    # (7 tokens, `y.sum().backward()`); a 16-bit result cannot be closer than half an ulp of its own
    # magnitude, so the bound scales with the tensor's largest value when that exceeds 1.
    def abs_gate(got, want, atol, what):
        scale = max(1.0, float(want.abs().max()))
        err = float((got.float().cpu() - want).abs().max())
        assert err <= atol * scale, f"{what}: max abs err {err:.3e} > {atol:.1e} * {scale:.2f}"

    abs_gate(y, ref.y, REF_ATOL_OUT[dtype], "y")
    abs_gate(x.grad, dx_ref, REF_ATOL_DX[dtype], "x.grad")
    abs_gate(moe.c_fc.weight.grad, ref.grads["c_fc"], REF_ATOL_DW[dtype], "c_fc.weight.grad")
    abs_gate(moe.c_proj.weight.grad, ref.grads["c_proj"], REF_ATOL_DW[dtype], "c_proj.weight.grad")
    return moe, x, y, logits


@pytest.mark.parametrize("name", list(gi.MOE_CASES))
def test_moe_fp32_cuda_cores(name):
    """fp32 runs on the CUDA-core GEMMs (exact fp32 FMA); `config1` is the CPU-runnable 512-token layer."""
    moe, x, y, logits = _run_and_compare(name, torch.float32, impl=0)
    # against the stored outputs of the reference's torch path
    gold = np.load(os.path.join(GOLDEN, "moe.npz"))
    key = f"{name}.f32"
    for what, t in (("y", y), ("dx", x.grad), ("dw1", moe.c_fc.weight.grad), ("dw2", moe.c_proj.weight.grad),
                    ("dgate", moe.gate.weight.grad), ("router_logits", logits)):
        ref = gold[f"{key}.{what}.sample"]
        got = gi.sample(t.cpu())
        scale = max(float(np.abs(ref).max()), 1e-30)
        assert float(np.abs(got - ref).max()) / scale <= 2e-4, what


@pytest.mark.parametrize("name", list(gi.MOE_CASES))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_16bit_cuda_cores(name, dtype):
    _run_and_compare(name, dtype, impl=1)


@pytest.mark.parametrize("name", list(gi.MOE_CASES))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_16bit_tensor_cores(name, dtype):
    """Automatic kernel choice = tcgen05 path for bf16/fp16 with widths that are multiples of 8."""
    from xma import _lib

    T, H, I, E, K, act = gi.MOE_CASES[name]
    assert _lib.lib.xma_b200_grouped_gemm_uses_tensor_cores(_lib.dtype_code(dtype), H, I) == 1
    _run_and_compare(name, dtype, impl=2)


@pytest.mark.parametrize("name", list(gi.MOE_CASES))
def test_moe_bf16_tensor_core_pairs(name):
    """tcgen05 cta_group::2 kernels (one 256 x 256 tile per CTA pair)."""
    _run_and_compare(name, torch.bfloat16, impl=3)


def test_moe_3d_input_and_backend_argument():
    from xma import KernelBackend
    from xma.layers import MoE, SwiGLU

    moe = MoE(8, 2, 64, 128, SwiGLU(), True, False, 0.02).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(2, 5, 64, device="cuda", dtype=torch.bfloat16)
    y, logits = moe(x, kernel_backend=KernelBackend.cuda)
    assert y.shape == x.shape and logits.shape == (10, 8)
    y2, _ = moe(x)
    assert torch.equal(y, y2)  # deterministic
    with pytest.raises(ValueError):
        moe(x, kernel_backend=KernelBackend.torch)


def test_moe_reference_grid_shape():
    """One point of the reference's own grid (tests/layers/moe_test.py:26-53): 7 tokens, E=128, K=8,
    H=576, I=256, nn.GLU, bf16 - most experts receive no token."""
    import torch.nn as nn

    from xma.layers import MoE

    torch.manual_seed(42)
    moe = MoE(128, 8, 576, 256, nn.GLU(), True, False, 0.02).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randn(7, 576, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, logits = moe(x)
    y.sum().backward()
    f32 = lambda t: t.detach().float().cpu()
    ref = orc.moe_forward_backward(f32(x), f32(moe.gate.weight), f32(moe.c_fc.weight), f32(moe.c_proj.weight), 8,
                                   "glu", dy=torch.ones(7, 576), router_logits=f32(logits))
    torch.testing.assert_close(f32(y), ref.y, rtol=0, atol=1.6e-2)
    torch.testing.assert_close(f32(moe.c_fc.weight.grad), ref.grads["c_fc"], rtol=0, atol=7.9e-3)
    torch.testing.assert_close(f32(moe.c_proj.weight.grad), ref.grads["c_proj"], rtol=0, atol=7.9e-3)


_GRID = [(E, K, 2048, 8192) for E in (2, 4, 6, 8) for K in (2, 4) if K <= E] + [(128, 8, 576, 256), (4, 1, 2048, 8192)]
# every point runs eagerly; these also run under torch.compile(fullgraph=True), as the reference's grid does
_COMPILED = {(4, 2, 2048, 8192), (8, 4, 2048, 8192), (128, 8, 576, 256), (4, 1, 2048, 8192)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("num_experts,top_k,H,I", _GRID)
@pytest.mark.parametrize("is_glu", [True, False])
@pytest.mark.parametrize("compiled", [False, True])
@torch._dynamo.config.patch(recompile_limit=1024)  # every point is a new module, as in the reference's test
def test_moe_reference_grid(dtype, num_experts, top_k, H, I, is_glu, compiled):
    """The reference's own MoE test (tests/layers/moe_test.py:26-157) on its grid: 7 tokens; E in {2,4,6,8} x
    K in {2,4} at hidden 2048 / intermediate 8192, and E=128, K=8 at 576 / 256; three dtypes; nn.GLU /
    GELU(tanh); eager and compiled; `y.sum().backward()`; its absolute tolerances (rtol 0); gate gradients not
    compared - with the CPU oracle in the place of its torch path. One more point, K=1, takes the `.max`
    branch of the reference's top-k (xma/layers/moe/__init__.py:256-260)."""
    import torch.nn as nn

    from xma.layers import MoE

    if compiled and (num_experts, top_k, H, I) not in _COMPILED:
        pytest.skip("compiled on a subset of the grid")
    torch.manual_seed(42)
    act = nn.GLU() if is_glu else nn.GELU(approximate="tanh")
    moe = MoE(num_experts, top_k, H, I, act, is_glu, False, 0.02).to(device="cuda", dtype=dtype)
    x = torch.randn(7, H, device="cuda", dtype=dtype, requires_grad=True)
    module = torch.compile(moe, fullgraph=True) if compiled else moe
    y, logits = module(x)
    y.sum().backward()
    # like the reference test, both sides run in `dtype`: the oracle is the torch path's arithmetic in
    # that dtype on the CPU (the tolerances were chosen for a comparison between two `dtype` results)
    cpu = lambda t: t.detach().cpu()
    ref = orc.moe_forward_backward(cpu(x), cpu(moe.gate.weight), cpu(moe.c_fc.weight), cpu(moe.c_proj.weight), top_k,
                                   "glu" if is_glu else "gelu_tanh", dy=torch.ones(7, H, dtype=dtype),
                                   router_logits=cpu(logits))
    f32 = lambda t: t.detach().float().cpu()
    dx_ref = ref.grads["x_experts"].float() + ref.grads["router_logits"].float() @ f32(moe.gate.weight)
    # The reference's absolute tolerances equal one ulp of the 16-bit types for magnitudes in [1, 2); its
    # seeds keep the compared tensors there. With other seeds a few entries are larger, and two correct
    # 16-bit results may differ by one ulp of *that* magnitude, so the bound scales with max|ref| above 1.
    def close(got, want, atol, what):
        want = want.float()
        bound = atol * max(1.0, float(want.abs().max()))
        err = float((f32(got) - want).abs().max())
        assert err <= bound, f"{what}: max abs err {err:.3e} > {bound:.3e}"

    close(y, ref.y, REF_ATOL_OUT[dtype], "y")
    close(x.grad, dx_ref, REF_ATOL_DX[dtype], "x.grad")
    close(moe.c_fc.weight.grad, ref.grads["c_fc"], REF_ATOL_DW[dtype], "c_fc.weight.grad")
    close(moe.c_proj.weight.grad, ref.grads["c_proj"], REF_ATOL_DW[dtype], "c_proj.weight.grad")


def test_moe_empty_batch():
    """No tokens at all: every kernel gets a zero-sized problem and the gradients are exact zeros."""
    from xma.layers import MoE, SwiGLU

    moe = MoE(4, 2, 64, 128, SwiGLU(), True, False, 0.02).to(device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(0, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, logits = moe(x)
    assert y.shape == (0, 64) and logits.shape == (0, 4)
    y.sum().backward()
    assert x.grad.shape == (0, 64)
    assert float(moe.c_fc.weight.grad.abs().max()) == 0.0 and float(moe.c_proj.weight.grad.abs().max()) == 0.0


def test_tagged_activation_is_fused_and_lambda_warns():
    """`xma.functional.swiglu_chunked` / `swiglu_packed` (or any callable tagged `xma_fused_activation`) take the
    fused GEMM epilogues, bit for bit like `xma.layers.SwiGLU`; an untagged lambda that computes SwiGLU runs the
    generic path (same result within rounding) and warns once."""
    import warnings

    from xma import ops
    from xma.functional import swiglu, swiglu_chunked, swiglu_packed
    from xma.layers import MoE, SwiGLU, SwiGLUPacked

    torch.manual_seed(1)
    x = torch.randn(300, 128, device="cuda", dtype=torch.bfloat16)

    def run(act):
        torch.manual_seed(2)
        moe = MoE(8, 2, 128, 256, act, True, False, 0.02).to(device="cuda", dtype=torch.bfloat16)
        ops.STATS.enabled, ops.STATS.timing = True, False
        ops.STATS.reset()
        try:
            y, _ = moe(x)
        finally:
            ops.STATS.enabled = False
        return y, ops.STATS.launches

    y_cls, n_cls = run(SwiGLU())
    y_fn, n_fn = run(swiglu_chunked)
    assert torch.equal(y_cls, y_fn) and n_cls == n_fn
    y_pcls, n_pcls = run(SwiGLUPacked())
    y_pfn, n_pfn = run(swiglu_packed)
    assert torch.equal(y_pcls, y_pfn) and n_pcls == n_pfn
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        y_lambda, n_lambda = run(lambda h: swiglu(*h.chunk(2, dim=-1)))
    assert any("runs unfused" in str(w.message) for w in caught)
    assert n_lambda > n_cls  # the stand-alone activation kernels and the generic path's separate row passes
    torch.testing.assert_close(y_lambda.float(), y_cls.float(), rtol=2e-2, atol=2e-3)
