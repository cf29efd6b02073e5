"""GPU parity of the row-movement kernels (gather into expert order, weighted combine, its backward)."""

import numpy as np
import pytest
import torch

from helpers import assert_close_rel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,K,H", [(7, 2, 64), (300, 8, 576), (1000, 4, 2048)])
def test_gather_combine(dtype, T, K, H):
    from xma import ops

    rng = np.random.RandomState(T + K)
    x = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(dtype).cuda()
    R = T * K
    rows = R + 256
    row_src = np.full(rows, -1, dtype=np.int32)
    pos = np.sort(rng.choice(rows, size=R, replace=False))
    perm = rng.permutation(R).astype(np.int32)
    row_src[pos] = perm
    row_src_d = torch.from_numpy(row_src).cuda()
    coeff = torch.from_numpy(rng.standard_normal(R).astype(np.float32)).to(dtype).cuda()

    out = torch.full((rows, H), 7.0, dtype=dtype, device="cuda")
    ops.gather_rows_(x, row_src_d, None, K, None, out)
    ref = torch.zeros(rows, H, dtype=dtype, device="cuda")
    ref[torch.from_numpy(pos).cuda()] = x[torch.from_numpy(perm // K).long().cuda()]
    assert torch.equal(out, ref)

    out2 = torch.full((rows, H), 7.0, dtype=dtype, device="cuda")
    ops.gather_rows_(x, row_src_d, coeff, K, None, out2)
    ref2 = torch.zeros(rows, H, dtype=torch.float32, device="cuda")
    idx = torch.from_numpy(perm).long().cuda()
    ref2[torch.from_numpy(pos).cuda()] = x[idx // K].float() * coeff[idx].float().unsqueeze(-1)
    assert torch.equal(out2, ref2.to(dtype))

    # rows_in_use limits the rows that are touched
    lim = torch.tensor([128], dtype=torch.int32, device="cuda")
    out3 = torch.full((rows, H), 7.0, dtype=dtype, device="cuda")
    ops.gather_rows_(x, row_src_d, None, K, lim, out3)
    assert torch.equal(out3[:128], ref[:128]) and bool((out3[128:] == 7.0).all())

    ys = torch.from_numpy(rng.standard_normal((R, H)).astype(np.float32)).to(dtype).cuda()
    w = torch.from_numpy(rng.random_sample((T, K)).astype(np.float32)).to(dtype).cuda()
    y = torch.empty(T, H, dtype=dtype, device="cuda")
    ops.combine_rows_(ys, w, K, y)
    y_ref = (ys.double().view(T, K, H) * w.double().unsqueeze(-1)).sum(1)
    tol = 1e-6 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1e-2)
    assert_close_rel(y, y_ref, tol, "combine")
    ops.combine_rows_(ys, None, K, y)
    assert_close_rel(y, ys.double().view(T, K, H).sum(1), tol, "combine (plain sum)")

    dy = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(dtype).cuda()
    dw = torch.empty(T, K, dtype=dtype, device="cuda")
    ops.combine_bwd_(ys, dy, K, dw)
    dw_ref = (ys.double().view(T, K, H) * dy.double().unsqueeze(1)).sum(-1)
    assert_close_rel(dw, dw_ref, 1e-5 if dtype == torch.float32 else tol, "combine backward")

    # rows kept in another order and addressed through an index (the expert-parallel layer combines
    # straight from expert-sorted rows)
    order = torch.from_numpy(rng.permutation(R).astype(np.int32)).cuda()  # flat index f lives in row order[f]
    shuffled = torch.empty_like(ys)
    shuffled[order.long()] = ys
    y2 = torch.empty(T, H, dtype=dtype, device="cuda")
    ops.combine_rows_(shuffled, w, K, y2, order)
    ops.combine_rows_(ys, w, K, y)
    assert torch.equal(y2, y)
    dw2 = torch.empty(T, K, dtype=dtype, device="cuda")
    ops.combine_bwd_(shuffled, dy, K, dw2, order)
    assert torch.equal(dw2, dw)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,K,H,E", [(7, 2, 64, 4), (300, 8, 576, 128), (1000, 4, 2048, 6), (513, 16, 4096, 8),
                                     (40, 1, 128, 3)])
def test_spread_rows_matches_gather_and_combine_bwd(dtype, T, K, H, E):
    """The token-major scatter, on a real routing decision: same grouped rows (bit for bit) as gather_rows,
    pad rows zero, and - fused - the same d_router_weights as combine_bwd within the rounding of the sum order."""
    from xma import ops
    from xma.layers.moe import build_route_plan

    rng = np.random.RandomState(T * K + E)
    selected = torch.from_numpy(np.stack([rng.permutation(E)[:K] if K <= E else rng.randint(0, E, K)
                                          for _ in range(T)]).astype(np.int32)).cuda()
    plan = build_route_plan(selected, E)
    # the inverse map: row_dst[row_src[p]] == p for every real row, and every flat index has a row
    row_src = plan.row_src.cpu().numpy()
    row_dst = plan.row_dst.cpu().numpy()
    real = np.nonzero(row_src >= 0)[0]
    assert len(real) == T * K and np.array_equal(row_dst[row_src[real]], real)

    mk = lambda *s: torch.from_numpy(rng.standard_normal(s).astype(np.float32)).to(dtype).cuda()
    x, coeff, ys = mk(T, H), mk(T, K), mk(T * K, H)
    rows = plan.row_src.numel()
    used = int(plan.pad_offsets[-1])
    for cf in (None, coeff.view(-1)):
        want = torch.full((rows, H), 7.0, dtype=dtype, device="cuda")
        ops.gather_rows_(x, plan.row_src, cf, K, plan.pad_offsets[E:], want)
        got = torch.full((rows, H), 7.0, dtype=dtype, device="cuda")
        ops.spread_rows_(x, plan.row_dst, cf, None, None, K, plan.counts, plan.pad_offsets, got)
        assert torch.equal(got[:used], want[:used])
        assert bool((got[used:] == 7.0).all())  # rows behind the last expert are not touched
        dw = torch.full((T, K), 7.0, dtype=dtype, device="cuda")
        got2 = torch.full((rows, H), 7.0, dtype=dtype, device="cuda")
        ops.spread_rows_(x, plan.row_dst, cf, ys, dw, K, plan.counts, plan.pad_offsets, got2)
        assert torch.equal(got2[:used], want[:used])
        dw_ref = (ys.double().view(T, K, H) * x.double().unsqueeze(1)).sum(-1)
        tol = 1e-5 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1e-2)
        assert_close_rel(dw, dw_ref, tol, "fused combine backward")
