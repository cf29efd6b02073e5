"""Generates tests/golden/*.npz by running the REFERENCE's own torch path on CPU.

Usage (in a container that has the reference tree):  python tests/golden/make_golden.py <path-to-reference-checkout>
The reference package is loaded under the alias `xma_ref` (this repository's package is also called
`xma`). Two harness-side adjustments, neither touching reference code:
  * `MoE._compute_experts` calls `continuous_count` without forwarding `kernel_backend`
    (xma/layers/moe/__init__.py:211), which on a CPU-only host resolves to a backend that raises; the
    name is rebound to the same function with `kernel_backend=torch`.
  * `Tensor.sort` is made stable for the duration of the call, so the permutation is the canonical
    one (the reference's outputs change only at rounding level, its integer outputs not at all).
  * `Tensor.topk` is replaced, for the duration of the call, by "stable descending sort, first k":
    the same values as torch.topk and the same indices on rows without ties; on rows with ties
    (frequent for bf16 logits) torch leaves the choice unspecified and this picks the lowest index.
    The unpatched torch.topk result is stored beside it (`selected_topk`) so the tests can check
    that the two agree on every tie-free row and select equal values on the others.
Large tensors are stored as an evenly strided sample plus sum and sum of absolute values.
"""

from __future__ import annotations

import functools
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import inputs as gi  # noqa: E402


def load_reference(root: str):
    pkg = os.path.join(root, "xma")
    spec = importlib.util.spec_from_file_location("xma_ref", os.path.join(pkg, "__init__.py"),
                                                  submodule_search_locations=[pkg])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["xma_ref"] = mod
    spec.loader.exec_module(mod)
    import xma_ref.layers.moe as ref_moe
    from xma_ref.functional import continuous_count

    ref_moe.continuous_count = functools.partial(continuous_count, kernel_backend=mod.KernelBackend.torch)
    return mod


class canonical_ties:
    def __enter__(self):
        self._sort, self._topk = torch.Tensor.sort, torch.Tensor.topk
        orig = self._sort

        def sort(t, *args, **kwargs):
            kwargs["stable"] = True
            return orig(t, *args, **kwargs)

        def topk(t, k, dim=-1, **kwargs):
            values, indices = orig(t, dim=dim, descending=True, stable=True)
            return values.narrow(dim, 0, k), indices.narrow(dim, 0, k)

        torch.Tensor.sort, torch.Tensor.topk = sort, topk

    def __exit__(self, *exc):
        torch.Tensor.sort, torch.Tensor.topk = self._sort, self._topk


def summarize(prefix: str, t: torch.Tensor, out: dict) -> None:
    out[prefix + ".sample"] = gi.sample(t)
    tf = t.detach().double()
    out[prefix + ".sum"] = np.array(tf.sum().item())
    out[prefix + ".abssum"] = np.array(tf.abs().sum().item())
    out[prefix + ".shape"] = np.array(t.shape, dtype=np.int64)


def main(root: str, only: str | None = None) -> None:
    ref = load_reference(root)
    from xma_ref.functional import continuous_count, swiglu, swiglu_packed
    from xma_ref.layers import MoE

    KB = ref.KernelBackend.torch
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // 2))

    if only in (None, "rmsnorm"):
        # ---- fused_residual_add_rmsnorm (forward and gradients for given upstream gradients) ----------
        from xma_ref.functional import fused_residual_add_rmsnorm

        out = {}
        for name in gi.RMSNORM_CASES:
            inp = gi.rmsnorm_inputs(name)
            x = inp["x"].clone().requires_grad_()
            r = None if inp["residual"] is None else inp["residual"].clone().requires_grad_()
            w = None if inp["weight"] is None else inp["weight"].clone().requires_grad_()
            y, xr = fused_residual_add_rmsnorm(x, r, w, gi.RMSNORM_EPS, inp["multiplier"], kernel_backend=KB)
            loss = (y * inp["dy"]).sum()
            if xr is not None:
                loss = loss + (xr * inp["dxr"]).sum()
            loss.backward()
            out[name + ".y"], out[name + ".dx"] = y.detach().numpy(), x.grad.numpy()
            if xr is not None:
                out[name + ".xr"], out[name + ".dr"] = xr.detach().numpy(), r.grad.numpy()
            if w is not None:
                out[name + ".dw"] = w.grad.numpy()
        np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), **out)
    if only == "rmsnorm":
        return

    # ---- pack_sequence / unpack_sequence (outputs and gradients, both padding sides) ----------
    from xma_ref.functional import pack_sequence, unpack_sequence

    out = {}
    for name in gi.PACK_CASES:
        inp = gi.pack_inputs(name)
        cu = torch.tensor(inp["cu_seqlens"], dtype=torch.int32)
        B, S = len(inp["cu_seqlens"]) - 1, inp["seq_len"]
        for side in ("left", "right"):
            x = inp["x"].clone().requires_grad_()
            (y,) = pack_sequence([x], cu, inp["cu_seqlens"][-1], side, kernel_backend=KB)
            (y * inp["dpacked"]).sum().backward()
            out[f"{name}.{side}.pack"], out[f"{name}.{side}.pack_dx"] = y.detach().numpy(), x.grad.numpy()
            p = inp["p"].clone().requires_grad_()
            (z,) = unpack_sequence([p], cu, B, S, side, kernel_backend=KB)
            (z * inp["dpadded"]).sum().backward()
            out[f"{name}.{side}.unpack"], out[f"{name}.{side}.unpack_dx"] = z.detach().numpy(), p.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "sequence_packing.npz"), **out)
    if only == "sequence_packing":
        return

    # ---- continuous_count -------------------------------------------------------------------
    out = {}
    for name in gi.COUNT_CASES:
        ids, bins = gi.count_inputs(name)
        out[name] = continuous_count(torch.from_numpy(ids), bins, kernel_backend=KB).to(torch.int64).numpy()
    np.savez_compressed(os.path.join(HERE, "continuous_count.npz"), **out)

    # ---- swiglu / swiglu_packed (forward and gradients of .mean()) -----------------------------
    out = {}
    for name in gi.SWIGLU_CASES:
        g, u = gi.swiglu_inputs(name)
        g.requires_grad_(), u.requires_grad_()
        y = swiglu(g, u, kernel_backend=KB)
        y.mean().backward()
        out[name + ".y"], out[name + ".dg"], out[name + ".du"] = y.detach().numpy(), g.grad.numpy(), u.grad.numpy()
        rows, cols = g.shape
        x = torch.stack([g.detach(), u.detach()], dim=-1).reshape(rows, 2 * cols).clone().requires_grad_()
        yp = swiglu_packed(x, kernel_backend=KB)
        yp.mean().backward()
        out[name + ".packed_y"], out[name + ".packed_dx"] = yp.detach().numpy(), x.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "swiglu.npz"), **out)

    # ---- MoE fwd + bwd through the reference torch path ---------------------------------------
    acts = {
        "swiglu": lambda h: swiglu(*h.chunk(2, dim=-1), kernel_backend=KB),
        "swiglu_packed": lambda h: swiglu_packed(h, kernel_backend=KB),
        "glu": torch.nn.GLU(),
        "gelu_tanh": torch.nn.GELU(approximate="tanh"),
    }
    out = {}
    for name, (T, H, I, E, K, act) in gi.MOE_CASES.items():
        for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            inp = gi.moe_inputs(name, dtype)
            moe = MoE(num_experts=E, num_experts_per_tok=K, hidden_size=H, intermediate_size=I,
                      activation_function=acts[act], is_glu=(act != "gelu_tanh"), add_bias=False, std=0.02).to(dtype)
            with torch.no_grad():
                moe.gate.weight.copy_(inp["gate"])
                moe.c_fc.weight.copy_(inp["w1"])
                moe.c_proj.weight.copy_(inp["w2"])
            x = inp["x"].clone().requires_grad_()
            with canonical_ties():
                y, logits = moe(x, kernel_backend=KB)
                _, weights, selected = moe._compute_routing_weights(x.detach())
                y.backward(inp["dy"])
            with torch.no_grad():
                out[f"{name}.{tag}.selected_topk"] = moe._compute_routing_weights(x.detach())[2].numpy().astype(np.int64)
            key = f"{name}.{tag}"
            summarize(key + ".y", y, out)
            summarize(key + ".router_logits", logits, out)
            summarize(key + ".router_weights", weights, out)
            summarize(key + ".dx", x.grad, out)
            summarize(key + ".dgate", moe.gate.weight.grad, out)
            summarize(key + ".dw1", moe.c_fc.weight.grad, out)
            summarize(key + ".dw2", moe.c_proj.weight.grad, out)
            sel = selected.reshape(-1)
            out[key + ".selected"] = selected.numpy().astype(np.int64)
            sorted_e, sorted_s = sel.sort(stable=True)
            out[key + ".sorted_expert_idxs.sample"] = gi.sample(sorted_e)
            out[key + ".sorted_scattered_idxs.sample"] = gi.sample(sorted_s)
            out[key + ".expert_frequency"] = continuous_count(sorted_e, E, kernel_backend=KB).to(torch.int64).numpy()
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)
    print("wrote golden files to", HERE)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: make_golden.py <path-to-reference-checkout> [rmsnorm | sequence_packing]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
