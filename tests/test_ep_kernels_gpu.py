"""Kernels of the expert-parallel peer transport on one GPU: the "ranks" are ordinary buffers of the
same device, addressed through the same pointer tables the multi-process layer builds, and every
result is compared bit for bit with a numpy restatement of the layout rules."""

import numpy as np
import pytest
import torch

from xma import ops

pytestmark = pytest.mark.gpu

PAD = 128


def _layout(cm: np.ndarray, rank: int):
    """numpy statement of what ep_plan computes for `rank` from the [W, E] count matrix."""
    W, E = cm.shape
    el = E // W
    total = cm.sum(0)
    before = cm[:rank].sum(0)
    send_delta = np.zeros(E, np.int64)
    my_run = 0
    tables = None
    for w in range(W):
        pad = tiles = 0
        counts, pad_off, tile_prefix, tile_expert, pad_slots = [], [], [], [], []
        for j in range(el):
            e = w * el + j
            send_delta[e] = pad + before[e] - my_run
            my_run += cm[rank, e]
            t = -(-int(total[e]) // PAD)
            counts.append(int(total[e]))
            pad_off.append(pad)
            tile_prefix.append(tiles)
            tile_expert += [j] * t
            pad_slots += list(range(pad + int(total[e]), pad + t * PAD))
            tiles += t
            pad += t * PAD
        if w == rank:
            tables = dict(counts=counts, pad_offsets=pad_off + [pad], tile_prefix=tile_prefix + [tiles],
                          tile_expert=tile_expert, pad_slots=pad_slots, rows=pad)
    return send_delta, tables


@pytest.mark.parametrize("world,experts", [(1, 4), (2, 8), (4, 8), (8, 8), (8, 128)])
def test_ep_plan_matches_numpy(world, experts):
    rng = np.random.RandomState(world * 100 + experts)
    cm = rng.randint(0, 400, size=(world, experts)).astype(np.int32)
    cm[rng.rand(world, experts) < 0.2] = 0  # experts without rows from some ranks
    dev = torch.device("cuda")
    cm_dev = torch.from_numpy(cm).to(dev)
    el = experts // world
    for rank in range(world):
        send_delta, t = _layout(cm.astype(np.int64), rank)
        tile_cap = t["rows"] // PAD + el
        meta = torch.full((t["rows"] + PAD,), 7, dtype=torch.int32, device=dev)
        out = dict(
            send_delta=torch.empty(experts, dtype=torch.int32, device=dev),
            counts=torch.empty(el, dtype=torch.int32, device=dev),
            pad_offsets=torch.empty(el + 1, dtype=torch.int32, device=dev),
            tile_prefix=torch.empty(el + 1, dtype=torch.int32, device=dev),
            tile_expert=torch.full((tile_cap,), -5, dtype=torch.int32, device=dev),
        )
        ops.ep_plan_(cm_dev, rank, out["send_delta"], out["counts"], out["pad_offsets"], out["tile_prefix"],
                     out["tile_expert"], meta)
        torch.cuda.synchronize()
        assert np.array_equal(out["send_delta"].cpu().numpy(), send_delta)
        for k in ("counts", "pad_offsets", "tile_prefix"):
            assert np.array_equal(out[k].cpu().numpy(), np.array(t[k])), k
        n_tiles = len(t["tile_expert"])
        assert np.array_equal(out["tile_expert"].cpu().numpy()[:n_tiles], np.array(t["tile_expert"]))
        m = meta.cpu().numpy()
        expect = np.full_like(m, 7)
        expect[t["pad_slots"]] = -1
        assert np.array_equal(m, expect)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [2, 4])
def test_dispatch_copy_return_round_trip(world, dtype):
    """Every rank dispatches its routed rows; every owner copies what it got and returns it: each
    home buffer must then hold, slot by slot, the (weighted) token rows that were sent."""
    E, K, H = 8, 2, 64
    el = E // world
    dev = torch.device("cuda")
    rng = np.random.RandomState(3)
    tokens = [90 + 17 * r for r in range(world)]
    sel = [np.stack([rng.permutation(E)[:K] for _ in range(t)]).astype(np.int32) for t in tokens]
    cm = np.stack([np.bincount(s.reshape(-1), minlength=E) for s in sel]).astype(np.int32)
    cm_dev = torch.from_numpy(cm).to(dev)
    rows_cap = max(_layout(cm.astype(np.int64), r)[1]["rows"] for r in range(world)) + PAD
    home_cap = max(tokens) * K

    recv = [torch.full((rows_cap, H), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    meta = [torch.full((rows_cap,), 7, dtype=torch.int32, device=dev) for _ in range(world)]
    home = [torch.full((home_cap, H), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    table = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    recv_table, meta_table, home_table = table(recv), table(meta), table(home)

    xs, coeffs, plans = [], [], []
    for r in range(world):
        send_delta, t = _layout(cm.astype(np.int64), r)
        out = dict(
            send_delta=torch.empty(E, dtype=torch.int32, device=dev),
            counts=torch.empty(el, dtype=torch.int32, device=dev),
            pad_offsets=torch.empty(el + 1, dtype=torch.int32, device=dev),
            tile_prefix=torch.empty(el + 1, dtype=torch.int32, device=dev),
            tile_expert=torch.empty(t["rows"] // PAD + el, dtype=torch.int32, device=dev),
        )
        ops.ep_plan_(cm_dev, r, out["send_delta"], out["counts"], out["pad_offsets"], out["tile_prefix"],
                     out["tile_expert"], meta[r])
        plans.append((out, t))
        flat = sel[r].reshape(-1)
        order = np.argsort(flat, kind="stable").astype(np.int32)
        x = torch.from_numpy(rng.standard_normal((tokens[r], H)).astype(np.float32)).to(dev, dtype)
        c = torch.from_numpy(rng.uniform(0.5, 1.5, tokens[r] * K).astype(np.float32)).to(dev, dtype)
        xs.append(x)
        coeffs.append(c)
        ops.ep_dispatch_(x, torch.from_numpy(flat[order]).to(dev), torch.from_numpy(order).to(dev), c, K,
                         out["send_delta"], world, r, recv_table, meta_table, rows_cap)
    torch.cuda.synchronize()

    for r in range(world):
        out, t = plans[r]
        rows = t["rows"]
        m = meta[r].cpu().numpy()[:rows]
        valid = np.ones(rows, bool)
        valid[t["pad_slots"]] = False
        assert (m[valid] >= 0).all() and (m[~valid] == -1).all()
        # rows of one expert come ordered by source rank
        for j in range(el):
            lo = t["pad_offsets"][j]
            src = m[lo : lo + t["counts"][j]] >> 24
            assert (np.diff(src) >= 0).all()
        private = torch.full((rows, H), float("nan"), dtype=dtype, device=dev)
        ops.ep_copy_rows_(recv[r], meta[r], private)
        assert not torch.isnan(private).any()
        assert (private[torch.from_numpy(~valid).to(dev)] == 0).all()
        ops.ep_copy_rows_(recv[r][:rows], meta[r], recv[r][:rows])  # in place: pad rows only
        assert torch.equal(recv[r][:rows], private)
        ops.ep_return_(private, meta[r], world, home_table, home_cap)
    torch.cuda.synchronize()

    for r in range(world):
        q = torch.arange(tokens[r] * K, device=dev)
        expect = (xs[r][q // K].float() * coeffs[r].float()[:, None]).to(dtype)
        assert torch.equal(home[r][: tokens[r] * K], expect)
