"""Pins the CPU oracle to outputs of the reference's own torch path (tests/golden/*.npz, written by
tests/golden/make_golden.py). No GPU involved."""

import os

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import moe_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def golden_moe():
    return np.load(os.path.join(GOLDEN, "moe.npz"))


@pytest.mark.parametrize("name", list(gi.COUNT_CASES))
def test_continuous_count_matches_reference(name):
    gold = np.load(os.path.join(GOLDEN, "continuous_count.npz"))
    ids, bins = gi.count_inputs(name)
    got = orc.continuous_count(ids, bins)
    assert got.dtype == np.uint32
    assert np.array_equal(got.astype(np.int64), gold[name])


def test_continuous_count_ignores_out_of_range_and_bins_1():
    ids = np.array([0, 5, -1, 72, 71, 5], dtype=np.int64)
    got = orc.continuous_count(ids, 72)
    assert got.sum() == 4 and got[5] == 2 and got[71] == 1
    assert orc.continuous_count(ids, 1).tolist() == [6]


@pytest.mark.parametrize("name", list(gi.SWIGLU_CASES))
def test_swiglu_matches_reference(name):
    gold = np.load(os.path.join(GOLDEN, "swiglu.npz"))
    g, u = gi.swiglu_inputs(name)
    y = orc.swiglu(g, u)
    np.testing.assert_allclose(y.numpy(), gold[name + ".y"], rtol=1e-6, atol=1e-6)
    dy = torch.full_like(y, 1.0 / y.numel())
    dg, du = orc.swiglu_backward(g, u, dy)
    np.testing.assert_allclose(dg.numpy(), gold[name + ".dg"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(du.numpy(), gold[name + ".du"], rtol=1e-5, atol=1e-7)
    rows, cols = g.shape
    x = torch.stack([g, u], dim=-1).reshape(rows, 2 * cols)
    np.testing.assert_allclose(orc.swiglu_packed(x).numpy(), gold[name + ".packed_y"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(orc.swiglu_packed_backward(x, dy).numpy(), gold[name + ".packed_dx"], rtol=1e-5,
                               atol=1e-7)


def _check(gold, key, t, rtol, atol):
    ref = gold[key + ".sample"]
    got = gi.sample(t)
    assert list(gold[key + ".shape"]) == list(t.shape), key
    scale = max(float(np.abs(ref).max()), 1e-30)
    err = float(np.abs(got - ref).max())
    assert err <= atol + rtol * scale, f"{key}: max abs err {err:.3e} vs scale {scale:.3e}"
    # whole-tensor checksums, so that elements outside the sample are pinned too
    total = float(gold[key + ".abssum"])
    assert abs(float(t.double().abs().sum()) - total) <= (atol * t.numel() + 10 * rtol * total), key


@pytest.mark.parametrize("name", list(gi.MOE_CASES))
@pytest.mark.parametrize("tag,dtype,rtol", [("f32", torch.float32, 2e-5), ("bf16", torch.bfloat16, 3e-2)])
def test_moe_matches_reference(golden_moe, name, tag, dtype, rtol):
    inp = gi.moe_inputs(name, dtype)
    res = orc.moe_forward_backward(inp["x"], inp["gate"], inp["w1"], inp["w2"], inp["top_k"], inp["activation"],
                                   dy=inp["dy"])
    key = f"{name}.{tag}"
    # integer outputs: exact
    assert np.array_equal(res.selected_experts.numpy(), golden_moe[key + ".selected"])
    # against the unpatched torch.topk: identical on rows whose logits have no tie among the top
    # k+1 values, and the same selected values everywhere
    lg = res.router_logits.float()
    topk = torch.from_numpy(golden_moe[key + ".selected_topk"])
    srt = torch.sort(lg, dim=-1, descending=True).values[:, : inp["top_k"] + 1]
    tie_free = (srt[:, 1:] != srt[:, :-1]).all(-1)
    assert torch.equal(res.selected_experts[tie_free], topk[tie_free])
    assert torch.equal(torch.gather(lg, 1, res.selected_experts), torch.gather(lg, 1, topk))
    assert np.array_equal(res.sort.counts.astype(np.int64), golden_moe[key + ".expert_frequency"])
    assert np.array_equal(gi.sample(torch.from_numpy(res.sort.sorted_expert_idxs)),
                          golden_moe[key + ".sorted_expert_idxs.sample"])
    assert np.array_equal(gi.sample(torch.from_numpy(res.sort.sorted_scattered_idxs)),
                          golden_moe[key + ".sorted_scattered_idxs.sample"])
    # floating-point outputs: relative to the tensor's largest magnitude
    _check(golden_moe, key + ".router_logits", res.router_logits, rtol, 0)
    _check(golden_moe, key + ".router_weights", res.router_weights, rtol, 0)
    _check(golden_moe, key + ".y", res.y, rtol, 0)
    _check(golden_moe, key + ".dx", res.grads["x"], rtol, 0)
    _check(golden_moe, key + ".dgate", res.grads["gate"], rtol, 0)
    _check(golden_moe, key + ".dw1", res.grads["c_fc"], rtol, 0)
    _check(golden_moe, key + ".dw2", res.grads["c_proj"], rtol, 0)


def test_count_sort_tables():
    ids = np.array([3, 1, 3, 0, 1, 3, 3], dtype=np.int64)
    s = orc.count_sort(ids, 5)
    assert s.counts.tolist() == [1, 2, 0, 4, 0]
    assert s.offsets_incl.tolist() == [1, 3, 3, 7, 7]
    assert s.sorted_expert_idxs.tolist() == [0, 1, 1, 3, 3, 3, 3]
    assert s.sorted_scattered_idxs.tolist() == [3, 1, 4, 0, 2, 5, 6]
    assert s.pad_offsets.tolist() == [0, 128, 256, 256, 384, 384]
    assert s.tile_prefix.tolist() == [0, 1, 2, 2, 3, 3]
    assert s.tile_expert.tolist() == [0, 1, 3]
    assert s.row_src[:2].tolist() == [3, -1] and s.row_src[128:131].tolist() == [1, 4, -1]
    assert s.row_src[256:261].tolist() == [0, 2, 5, 6, -1]


def test_route_tie_rule():
    logits = torch.tensor([[1.0, 3.0, 3.0, 3.0, 0.0], [2.0, 2.0, 2.0, 2.0, 2.0]])
    w, sel = orc.route(logits, 2)
    assert sel.tolist() == [[1, 2], [0, 1]]
    assert torch.allclose(w, torch.full((2, 2), 0.5))


@pytest.mark.parametrize("name", list(gi.RMSNORM_CASES))
def test_rmsnorm_oracle_matches_reference(name):
    """fused_residual_add_rmsnorm: the float64 restatement against the reference's fp32 torch path."""
    from oracle import rmsnorm_oracle as rn

    gold = np.load(os.path.join(GOLDEN, "rmsnorm.npz"))
    inp = gi.rmsnorm_inputs(name)
    np_ = lambda t: None if t is None else t.numpy()
    x, r, w = np_(inp["x"]), np_(inp["residual"]), np_(inp["weight"])
    y, xr, _ = rn.forward(x, r, w, gi.RMSNORM_EPS, inp["multiplier"])
    dx, dr, dw = rn.backward(x, r, w, gi.RMSNORM_EPS, inp["multiplier"], np_(inp["dy"]), np_(inp["dxr"]))
    np.testing.assert_allclose(y, gold[name + ".y"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(dx, gold[name + ".dx"], rtol=2e-5, atol=5e-6)
    if r is not None:
        np.testing.assert_allclose(xr, gold[name + ".xr"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(dr, gold[name + ".dr"], rtol=2e-5, atol=5e-6)
    if w is not None:
        np.testing.assert_allclose(dw, gold[name + ".dw"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("side", ["left", "right"])
@pytest.mark.parametrize("name", list(gi.PACK_CASES))
def test_sequence_packing_oracle_matches_reference(name, side):
    """pack_sequence / unpack_sequence and their gradients: bit for bit against the reference's torch path."""
    from oracle import sequence_packing_oracle as sp

    gold = np.load(os.path.join(GOLDEN, "sequence_packing.npz"))
    inp = gi.pack_inputs(name)
    cu, S = inp["cu_seqlens"], inp["seq_len"]
    key = f"{name}.{side}."
    assert np.array_equal(sp.pack(inp["x"].numpy(), cu, side), gold[key + "pack"])
    assert np.array_equal(sp.pack_backward(inp["dpacked"].numpy(), cu, S, side), gold[key + "pack_dx"])
    assert np.array_equal(sp.unpack(inp["p"].numpy(), cu, S, side), gold[key + "unpack"])
    assert np.array_equal(sp.unpack_backward(inp["dpadded"].numpy(), cu, side), gold[key + "unpack_dx"])


def test_sequence_packing_oracle_round_trips():
    """Size-independent properties of the restatement on random ragged batches: unpacking what was packed gives the
    input with its padding zeroed, packing what was unpacked gives the packed input back, and the two padding sides
    differ only in where a sequence sits in its row."""
    from oracle import sequence_packing_oracle as sp

    rng = np.random.RandomState(11)
    for _ in range(25):
        B, S = int(rng.randint(1, 7)), int(rng.randint(1, 12))
        lens = rng.randint(0, S + 1, size=B)
        cu = [0] + np.cumsum(lens).tolist()
        trailing = tuple(rng.randint(1, 4, size=int(rng.randint(0, 3))).tolist())
        x = rng.standard_normal((B, S, *trailing)).astype(np.float32)
        p = rng.standard_normal((cu[-1], *trailing)).astype(np.float32)
        for side in ("left", "right"):
            packed = sp.pack(x, cu, side)
            assert packed.shape == (cu[-1], *trailing)
            back = sp.unpack(packed, cu, S, side)
            pos = np.arange(S)[None, :]
            valid = (pos >= S - lens[:, None]) if side == "left" else (pos < lens[:, None])
            mask = valid.reshape(B, S, *([1] * len(trailing)))
            assert np.array_equal(back, np.where(mask, x, 0))
            assert np.array_equal(sp.pack(sp.unpack(p, cu, S, side), cu, side), p)
        left, right = sp.unpack(p, cu, S, "left"), sp.unpack(p, cu, S, "right")
        for b in range(B):
            assert np.array_equal(left[b, S - lens[b]:], right[b, :lens[b]])
