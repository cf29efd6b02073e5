"""Parity of `xma.layers.MoE` at the layer shapes that `bench.py` times, with the automatic kernel choice:

  c2  16384 tokens, hidden 4096, intermediate 14336, 8 experts, top-2 (every expert above 2048 rows: more than
      one raster group per expert, reductions of 14336 and 28672, CTA-pair kernels);
  c3  32768 tokens, hidden 2048, intermediate 1024, 64 experts, top-8, Zipf(1.2)-skewed loads;
  c4  16384 tokens, hidden 4096, intermediate 1536, 128 experts, top-8 (about 1024 +- 32 rows per expert).

Inputs and weights come from `bench.py`'s own generators, so what is checked here is what is timed there.
Checked against the CPU oracle: routing decisions and every table of the counting sort bit for bit over all
tokens; `y` and `x.grad` of a seeded sample of tokens (a token's row depends on no other token); the weight
gradients of the heaviest, the lightest non-empty and (when there is one) an empty expert on a strided
subset of the intermediate features, each from all rows of that expert. Tolerance: max |err| / max |ref|
<= 2e-2 against the fp32 oracle (bf16 kernels, fp32 accumulation)."""

import argparse

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _bench():
    import bench

    args = argparse.Namespace(gpus=1, transport="peer", ep_chunks=None, fused_return=True)
    return bench, bench.Bench(args)


@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_layer_parity_at_benchmark_shape(name):
    from oracle import moe_oracle as orc
    from xma import _lib, ops
    from xma.layers.moe import _TopKSoftmax, build_route_plan

    bench, b = _bench()
    w = bench.WORKLOADS[name]
    E, K, I = w["experts"], w["top_k"], w["inter"]
    assert ops.GEMM_IMPL == _lib.IMPL_AUTO
    layer, moe, x, dy = bench.build_workload(b, name)
    results = bench.make_step(layer)(x, dy)
    torch.cuda.synchronize()
    assert _lib.read_and_clear_device_status() == 0
    y, dx, logits = results
    assert torch.isfinite(y.float()).all() and torch.isfinite(dx.float()).all()

    # (a) + (b): routing of every token, y and x.grad of 256 sampled tokens
    weights = bench.gather_expert_weights(b, layer, moe)
    report = bench.parity_check(results, weights, x, dy, K, sample_tokens=256, tol=TOL)
    assert report["routing_bit_exact"] and report["counts_bit_exact"], report
    assert report["y_max_rel_err"] <= TOL and report["dx_max_rel_err"] <= TOL, report

    # (a) continued: every table of the counting sort
    logits_cpu = logits.detach().cpu()
    ref_weights, ref_selected = orc.route(logits_cpu, K)
    with torch.no_grad():
        rw, selected = _TopKSoftmax.apply(logits.detach(), K)
        plan = build_route_plan(selected, E)
    srt = orc.count_sort(ref_selected.numpy(), E)
    used = int(srt.pad_offsets[-1])
    assert np.array_equal(plan.expert_frequency.cpu().numpy(), srt.counts)
    assert np.array_equal(plan.offsets_incl.cpu().numpy(), srt.offsets_incl)
    assert np.array_equal(plan.sorted_expert_idxs.cpu().numpy(), srt.sorted_expert_idxs)
    assert np.array_equal(plan.sorted_scattered_idxs.cpu().numpy(), srt.sorted_scattered_idxs)
    assert np.array_equal(plan.pad_offsets.cpu().numpy(), srt.pad_offsets)
    assert np.array_equal(plan.tile_prefix.cpu().numpy(), srt.tile_prefix)
    assert np.array_equal(plan.row_src.cpu().numpy()[:used], srt.row_src)
    # routing weights are floating point: softmax over the selected logits in fp32, rounded once to the
    # storage type; the device's exp may differ from the host's in the last place, i.e. one bf16 step (2^-8 relative)
    torch.testing.assert_close(rw.float().cpu(), ref_weights.float(), rtol=2.0 ** -7, atol=1e-7)

    # (c) weight gradients of single experts, all of their rows, a strided subset of the intermediate features
    counts = srt.counts.astype(np.int64)
    nonempty = np.nonzero(counts)[0]
    picks = {int(nonempty[np.argmax(counts[nonempty])]), int(nonempty[np.argmin(counts[nonempty])])}
    cols = torch.unique(torch.cat([torch.arange(0, I, max(1, I // 96)), torch.arange(I - 8, I)]))
    w1, w2, _ = weights
    perm = torch.from_numpy(srt.sorted_scattered_idxs.astype(np.int64))
    gates = ref_weights.flatten()[perm].float()
    x_cpu, dy_cpu = x.cpu(), dy.cpu()
    ends = srt.offsets_incl.astype(np.int64)
    g1, g2 = moe.c_fc.weight.grad, moe.c_proj.weight.grad
    for e in sorted(picks):
        rows = perm[ends[e] - counts[e]: ends[e]]
        tokens = rows // K
        d_o = dy_cpu[tokens].float() * gates[ends[e] - counts[e]: ends[e]].unsqueeze(-1)
        ref1, ref2 = orc.expert_weight_grads_slice(x_cpu[tokens], d_o, w1[e], w2[e], cols)
        got1 = g1[e][torch.cat([cols, cols + I]).to(g1.device)].float().cpu()
        got2 = g2[e][:, cols.to(g2.device)].float().cpu()
        err1 = float((got1 - ref1).abs().max() / ref1.abs().max().clamp_min(1e-30))
        err2 = float((got2 - ref2).abs().max() / ref2.abs().max().clamp_min(1e-30))
        assert err1 <= TOL, f"{name}: c_fc.weight.grad[{e}] ({counts[e]} rows) max rel err {err1:.3e}"
        assert err2 <= TOL, f"{name}: c_proj.weight.grad[{e}] ({counts[e]} rows) max rel err {err2:.3e}"
    for e in np.nonzero(counts == 0)[0][:2]:
        assert float(g1[int(e)].abs().max()) == 0.0 and float(g2[int(e)].abs().max()) == 0.0
    # the largest expert of the dense layer must exceed one raster group (16 row tiles), or this test would
    # not cover the tile order that the benchmark runs
    if name == "c2":
        assert counts.max() > 2048


def test_automatic_choice_takes_cta_pairs_for_large_experts():
    """The shapes above must reach the kernels they are meant to cover: CTA pairs for every GEMM of the dense
    layer, the CUDA-core kernels for fp32."""
    from xma import _lib

    q = _lib.lib.xma_b200_grouped_gemm_choice
    tile_cap = 32768 // 128 + 8
    for kd, n, wl, epi in [(4096, 28672, _lib.W_NK, _lib.EPI_SWIGLU), (14336, 4096, _lib.W_NK, _lib.EPI_PLAIN),
                           (4096, 14336, _lib.W_KN, _lib.EPI_DSWIGLU), (28672, 4096, _lib.W_KN, _lib.EPI_PLAIN)]:
        assert q(0, _lib.BF16, 8, tile_cap, kd, n, wl, epi, 0) == _lib.IMPL_TC_PAIR
    assert q(1, _lib.BF16, 8, tile_cap, 28672, 4096, 0, 0, 0) == _lib.IMPL_TC_PAIR
    assert q(0, _lib.BF16, 8, 8 + 7, 4096, 4096, _lib.W_NK, _lib.EPI_PLAIN, 0) == _lib.IMPL_TC  # small experts
    assert q(0, _lib.F32, 8, tile_cap, 4096, 4096, _lib.W_NK, _lib.EPI_PLAIN, 0) == _lib.IMPL_SIMT
