"""GPU parity of the expert grouped GEMMs: every operand layout and epilogue, on the CUDA-core
kernels (all dtypes) and on the tcgen05 kernels (bf16 / fp16), against fp64 torch matmuls on the
same values. Ragged experts, empty experts and widths that are not multiples of the tile."""

import numpy as np
import pytest
import torch

from helpers import REL_TOL, assert_close_rel
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

SIMT, TC, TC_PAIR = 1, 2, 3
IMPLS = [pytest.param(SIMT, torch.float32, id="cudacore-f32"), pytest.param(SIMT, torch.bfloat16, id="cudacore-bf16"),
         pytest.param(TC, torch.bfloat16, id="tcgen05-bf16"), pytest.param(TC, torch.float16, id="tcgen05-f16"),
         pytest.param(TC_PAIR, torch.bfloat16, id="pair-bf16"), pytest.param(TC_PAIR, torch.float16, id="pair-f16"),
         pytest.param(0, torch.bfloat16, id="auto-bf16")]


def _plan(counts, E):
    from xma.layers.moe import build_route_plan

    ids = np.repeat(np.arange(E, dtype=np.int32), counts)
    np.random.RandomState(0).shuffle(ids)
    return build_route_plan(torch.from_numpy(ids).cuda().view(-1, 1), E), ids


def _grouped(plan, R, width, dtype, seed):
    """Random grouped buffer whose pad rows are zero (as the gather kernel leaves them)."""
    rng = np.random.RandomState(seed)
    full = torch.from_numpy(rng.standard_normal((R, width)).astype(np.float32)).to(dtype).cuda()
    buf = torch.zeros(plan.row_cap, width, dtype=dtype, device="cuda")
    src = plan.row_src.long()
    valid = src >= 0
    buf[valid] = full[src[valid]]
    return buf, full


CASES = [
    # counts per expert, Kd, N
    ([5, 0, 130, 1], 64, 256),
    ([128, 256, 3], 192, 512),
    ([300, 7, 0, 0, 129, 64], 576, 264),
    ([1000, 24], 1024, 2048),
    # experts above 2048 rows: more than one raster group of 16 row tiles (8 tile pairs), odd tile and pair counts
    ([2049, 300], 128, 512),
    ([4097, 16384], 192, 768),
]


@pytest.mark.parametrize("impl,dtype", IMPLS)
@pytest.mark.parametrize("counts,kd,n", CASES)
def test_rows_gemm_plain_both_layouts(impl, dtype, counts, kd, n):
    from xma import _lib, ops

    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    a, a_full = _grouped(plan, R, kd, dtype, seed=1)
    rng = np.random.RandomState(2)
    w = torch.from_numpy((rng.standard_normal((E, n, kd)) * 0.05).astype(np.float32)).to(dtype).cuda()
    src = plan.row_src.long().cpu()
    tol = REL_TOL[dtype]

    # expected, per grouped row
    exp = torch.zeros(plan.row_cap, n, dtype=torch.float64)
    pad = plan.pad_offsets.cpu().tolist()
    for e in range(E):
        r0, c = pad[e], counts[e]
        if c:
            exp[r0 : r0 + c] = a[r0 : r0 + c].double().cpu() @ w[e].double().cpu().t()

    # weight stored [E, n, kd], grouped output
    out = torch.full((plan.row_cap, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, w, _lib.W_NK, out, None, None, plan.tile_expert, plan.tile_prefix, kd, n,
                           _lib.EPI_PLAIN, impl)
    used = pad[-1]
    assert_close_rel(out[:used].cpu(), exp[:used], tol, "grouped out")

    # same product, rows scattered to flat order through row_src
    ys = torch.full((R, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, w, _lib.W_NK, ys, None, plan.row_src, plan.tile_expert, plan.tile_prefix, kd, n,
                           _lib.EPI_PLAIN, impl)
    valid = src[:used] >= 0
    exp_scat = torch.zeros(R, n, dtype=torch.float64)
    exp_scat[src[:used][valid]] = exp[:used][valid]
    assert_close_rel(ys.cpu(), exp_scat, tol, "scattered out")

    # weight stored [E, kd, n]: out = a @ w_e
    wt = w.transpose(1, 2).contiguous()
    out2 = torch.full((plan.row_cap, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, wt, _lib.W_KN, out2, None, None, plan.tile_expert, plan.tile_prefix, kd, n,
                           _lib.EPI_PLAIN, impl)
    assert_close_rel(out2[:used].cpu(), exp[:used], tol, "kn layout")
    assert _lib.read_and_clear_device_status() == 0


@pytest.mark.parametrize("impl,dtype", IMPLS)
@pytest.mark.parametrize("counts,kd,inter", [([5, 0, 130, 1], 64, 128), ([300, 7, 0, 129], 192, 200),
                                             ([700, 100], 512, 1024), ([4097, 2049], 128, 384)])
def test_rows_gemm_swiglu_epilogues(impl, dtype, counts, kd, inter):
    from xma import _lib, ops

    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    used = int(plan.pad_offsets[-1])
    a, _ = _grouped(plan, R, kd, dtype, seed=3)
    rng = np.random.RandomState(4)
    w1 = torch.from_numpy((rng.standard_normal((E, 2 * inter, kd)) * 0.05).astype(np.float32)).to(dtype).cuda()
    gu = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
    act = torch.full((plan.row_cap, inter), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, w1, _lib.W_NK, act, gu, None, plan.tile_expert, plan.tile_prefix, kd, 2 * inter,
                           _lib.EPI_SWIGLU, impl)
    pad = plan.pad_offsets.cpu().tolist()
    exp_gu = torch.zeros(plan.row_cap, 2 * inter, dtype=torch.float64)
    for e in range(E):
        r0, c = pad[e], counts[e]
        if c:
            exp_gu[r0 : r0 + c] = a[r0 : r0 + c].double().cpu() @ w1[e].double().cpu().t()
    tol = REL_TOL[dtype]
    assert_close_rel(gu[:used].cpu(), exp_gu[:used], tol, "gate|up")
    g, u = gu[:used].cpu().float().chunk(2, dim=-1)
    exp_act = u.double() * g.double() * torch.sigmoid(g.double())  # from the stored (rounded) halves
    assert_close_rel(act[:used].cpu(), exp_act, 2e-6 if dtype == torch.float32 else tol / 2, "activation")

    # backward epilogue: d(activation) = dys @ W2_e with W2 stored [E, H, I]
    H = kd
    dys, _ = _grouped(plan, R, H, dtype, seed=5)
    w2 = torch.from_numpy((rng.standard_normal((E, H, inter)) * 0.05).astype(np.float32)).to(dtype).cuda()
    dgu = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(dys, w2, _lib.W_KN, dgu, gu, None, plan.tile_expert, plan.tile_prefix, H, inter,
                           _lib.EPI_DSWIGLU, impl)
    d_act = torch.zeros(plan.row_cap, inter, dtype=torch.float64)
    for e in range(E):
        r0, c = pad[e], counts[e]
        if c:
            d_act[r0 : r0 + c] = dys[r0 : r0 + c].double().cpu() @ w2[e].double().cpu()
    gd, ud = g.double(), u.double()
    s = torch.sigmoid(gd)
    exp_dg = d_act[:used] * ud * s * (1 + gd * (1 - s))
    exp_du = d_act[:used] * gd * s
    assert_close_rel(dgu[:used, :inter].cpu(), exp_dg, 2 * tol, "d gate")
    assert_close_rel(dgu[:used, inter:].cpu(), exp_du, 2 * tol, "d up")
    assert _lib.read_and_clear_device_status() == 0


@pytest.mark.parametrize("impl,dtype", IMPLS)
@pytest.mark.parametrize("counts,m,n", [([5, 0, 130, 1], 64, 256), ([300, 7, 0, 129], 136, 264),
                                        ([1000, 24, 64], 512, 384),
                                        # more row tiles than one group of 8 (tiles or tile pairs), ragged last group
                                        ([300, 0, 70], 2432, 264), ([4097, 2049], 256, 512)])
def test_dw_gemm(impl, dtype, counts, m, n):
    from xma import _lib, ops

    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    x, _ = _grouped(plan, R, m, dtype, seed=6)
    y, _ = _grouped(plan, R, n, dtype, seed=7)
    dw = torch.full((E, m, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_dw_(x, y, plan.counts, plan.pad_offsets, dw, impl)
    pad = plan.pad_offsets.cpu().tolist()
    exp = torch.zeros(E, m, n, dtype=torch.float64)
    for e in range(E):
        r0, c = pad[e], counts[e]
        if c:
            exp[e] = x[r0 : r0 + c].double().cpu().t() @ y[r0 : r0 + c].double().cpu()
    assert_close_rel(dw.cpu(), exp, REL_TOL[dtype], "dW")
    for e in range(E):
        if counts[e] == 0:
            assert bool((dw[e] == 0).all()), "experts without rows must get exactly zero"
    assert _lib.read_and_clear_device_status() == 0


def test_dw_gemm_ticket_order_matches_fixed_stride():
    """The CTA-pair weight-gradient kernel hands its tiles out heaviest expert first by an atomic ticket; the
    order in which tiles are computed changes no arithmetic, so the result equals the fixed-stride version bit
    for bit. Many experts with a skewed load: a few heavy ones, many light ones, several without rows."""
    from xma import _lib, ops

    rng = np.random.RandomState(5)
    E = 70
    counts = [int(c) for c in rng.zipf(1.3, size=E).clip(max=3000)]
    for e in (3, 17, 40, 69):
        counts[e] = 0
    counts[11], counts[50] = 5000, 2300
    R = int(sum(counts))
    m, n, dtype = 520, 776, torch.bfloat16
    plan, _ = _plan(counts, E)
    x, _ = _grouped(plan, R, m, dtype, seed=8)
    y, _ = _grouped(plan, R, n, dtype, seed=9)
    out = {}
    for dynamic in (1, 0, 1):
        previous = _lib.lib.xma_b200_tuning_set(_lib.TUNE_DW_DYNAMIC, dynamic)
        try:
            dw = torch.full((E, m, n), float("nan"), dtype=dtype, device="cuda")
            ops.grouped_gemm_dw_(x, y, plan.counts, plan.pad_offsets, dw, TC_PAIR)
            torch.cuda.synchronize()
        finally:
            _lib.lib.xma_b200_tuning_set(_lib.TUNE_DW_DYNAMIC, previous)
        assert _lib.read_and_clear_device_status() == 0
        assert torch.isfinite(dw.float()).all()
        out.setdefault(dynamic, dw)
        assert torch.equal(dw, out[dynamic])  # the second ticket run repeats the first
    assert torch.equal(out[1], out[0])
    pad = plan.pad_offsets.cpu().tolist()
    for e in (11, 50, 0, 3):
        r0, c = pad[e], counts[e]
        exp = x[r0 : r0 + c].double().cpu().t() @ y[r0 : r0 + c].double().cpu() if c else torch.zeros(m, n).double()
        assert_close_rel(out[1][e].cpu(), exp, REL_TOL[dtype], f"dW[{e}]")


@pytest.mark.parametrize("counts,kd,inter", [([1100, 1025, 1280, 2049, 1024, 1153], 256, 320),
                                             ([4097, 4096, 0, 4225], 192, 128)])
def test_automatic_choice_splits_odd_last_tiles_off(counts, kd, inter):
    """With experts of eight and more 128-row tiles the automatic choice takes the CTA-pair kernel; an expert with an
    odd number of tiles then has its last tile computed by the one-CTA kernel in a second launch instead of as half
    of a 256-row pair tile. Same arithmetic per output element: every epilogue gives the bits of the single launch."""
    from xma import _lib, ops

    dtype = torch.bfloat16
    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    used = int(plan.pad_offsets[-1])
    assert any(((c + 127) // 128) % 2 for c in counts)
    assert _lib.lib.xma_b200_grouped_gemm_choice(0, _lib.BF16, E, plan.tile_expert.numel(), kd, 2 * inter, _lib.W_NK,
                                                 _lib.EPI_SWIGLU, 0) == TC_PAIR
    a, _ = _grouped(plan, R, kd, dtype, seed=3)
    dys, _ = _grouped(plan, R, kd, dtype, seed=5)
    rng = np.random.RandomState(4)
    mk = lambda *s: torch.from_numpy((rng.standard_normal(s) * 0.05).astype(np.float32)).to(dtype).cuda()
    w1, w2, wp = mk(E, 2 * inter, kd), mk(E, kd, inter), mk(E, inter, kd)
    got = {}
    for split in (2, 0):
        previous = _lib.lib.xma_b200_tuning_set(_lib.TUNE_ODD_TAIL, split)
        try:
            nan = lambda width: torch.full((plan.row_cap, width), float("nan"), dtype=dtype, device="cuda")
            gu, act, dgu, plain, scattered = nan(2 * inter), nan(inter), nan(2 * inter), nan(inter), nan(inter)
            ops.grouped_gemm_rows_(a, w1, _lib.W_NK, act, gu, None, plan.tile_expert, plan.tile_prefix, kd, 2 * inter,
                                   _lib.EPI_SWIGLU, 0)
            ops.grouped_gemm_rows_(dys, w2, _lib.W_KN, dgu, gu, None, plan.tile_expert, plan.tile_prefix, kd, inter,
                                   _lib.EPI_DSWIGLU, 0)
            ops.grouped_gemm_rows_(a, wp, _lib.W_NK, plain, None, None, plan.tile_expert, plan.tile_prefix, kd, inter,
                                   _lib.EPI_PLAIN, 0)
            ops.grouped_gemm_rows_(a, wp, _lib.W_NK, scattered, None, plan.row_src, plan.tile_expert,
                                   plan.tile_prefix, kd, inter, _lib.EPI_PLAIN, 0)
            torch.cuda.synchronize()
        finally:
            _lib.lib.xma_b200_tuning_set(_lib.TUNE_ODD_TAIL, previous)
        assert _lib.read_and_clear_device_status() == 0
        got[split] = (gu[:used], act[:used], dgu[:used], plain[:used], scattered[:R])
    for x, y, what in zip(got[2], got[0], ("gate|up", "activation", "d gate|d up", "plain", "scattered")):
        assert torch.isfinite(x.float()).all(), what
        assert torch.equal(x, y), what
    pad = plan.pad_offsets.cpu().tolist()
    e = max(range(E), key=lambda i: counts[i] % 256 if ((counts[i] + 127) // 128) % 2 else -1)  # an odd expert
    r0, c = pad[e], counts[e]
    exp = a[r0 : r0 + c].double().cpu() @ wp[e].double().cpu().t()
    assert_close_rel(got[2][3][r0 : r0 + c].cpu(), exp, REL_TOL[dtype], "plain, rows of an odd expert")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,kd,inter", [([700, 0, 100, 1], 512, 1024), ([4097, 2049], 4096, 96),
                                             ([300, 129], 192, 288)])
def test_staged_swiglu_epilogues_match_row_per_thread_epilogues(dtype, counts, kd, inter):
    """The CTA-pair kernel moves the tiles of its SwiGLU epilogues through shared memory by TMA (activation width a
    multiple of 32); the arithmetic is that of the epilogues that read and write one row per thread, so the results
    are the same bit for bit - forward (gate|up and activation), backward into a separate buffer and backward in
    place over gate|up. Switch values: 0 = one row per thread, 7 = staged, the forward also for long reductions."""
    from xma import _lib, ops

    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    used = int(plan.pad_offsets[-1])
    a, _ = _grouped(plan, R, kd, dtype, seed=3)
    dys, _ = _grouped(plan, R, kd, dtype, seed=5)
    rng = np.random.RandomState(4)
    w1 = torch.from_numpy((rng.standard_normal((E, 2 * inter, kd)) * 0.05).astype(np.float32)).to(dtype).cuda()
    w2 = torch.from_numpy((rng.standard_normal((E, kd, inter)) * 0.05).astype(np.float32)).to(dtype).cuda()
    got = {}
    for staged in (7, 0):
        previous = _lib.lib.xma_b200_tuning_set(_lib.TUNE_DSWIGLU_STAGED, staged)
        try:
            gu = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
            act = torch.full((plan.row_cap, inter), float("nan"), dtype=dtype, device="cuda")
            ops.grouped_gemm_rows_(a, w1, _lib.W_NK, act, gu, None, plan.tile_expert, plan.tile_prefix, kd, 2 * inter,
                                   _lib.EPI_SWIGLU, TC_PAIR)
            dgu = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
            ops.grouped_gemm_rows_(dys, w2, _lib.W_KN, dgu, gu, None, plan.tile_expert, plan.tile_prefix, kd, inter,
                                   _lib.EPI_DSWIGLU, TC_PAIR)
            in_place = gu.clone()
            ops.grouped_gemm_rows_(dys, w2, _lib.W_KN, in_place, in_place, None, plan.tile_expert, plan.tile_prefix,
                                   kd, inter, _lib.EPI_DSWIGLU, TC_PAIR)
            # the interleaved layout (gate, up, gate, up, ... along the columns)
            gu_p = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
            act_p = torch.full((plan.row_cap, inter), float("nan"), dtype=dtype, device="cuda")
            ops.grouped_gemm_rows_(a, w1, _lib.W_NK, act_p, gu_p, None, plan.tile_expert, plan.tile_prefix, kd,
                                   2 * inter, _lib.EPI_SWIGLU_PACKED, TC_PAIR)
            dgu_p = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
            ops.grouped_gemm_rows_(dys, w2, _lib.W_KN, dgu_p, gu_p, None, plan.tile_expert, plan.tile_prefix, kd, inter,
                                   _lib.EPI_DSWIGLU_PACKED, TC_PAIR)
            torch.cuda.synchronize()
        finally:
            _lib.lib.xma_b200_tuning_set(_lib.TUNE_DSWIGLU_STAGED, previous)
        assert _lib.read_and_clear_device_status() == 0
        got[staged] = (gu[:used], act[:used], dgu[:used], in_place[:used], dgu_p[:used])
    for x, y, what in zip(got[7], got[0], ("gate|up", "activation", "d gate|d up", "d gate|d up in place",
                                           "d gate, d up interleaved")):
        assert torch.isfinite(x.float()).all(), what
        assert torch.equal(x, y), what
    assert torch.equal(got[7][2], got[7][3])


@pytest.mark.parametrize("impl,dtype", [pytest.param(TC, torch.bfloat16, id="tcgen05-bf16"),
                                        pytest.param(TC_PAIR, torch.bfloat16, id="pair-bf16"),
                                        pytest.param(TC_PAIR, torch.float16, id="pair-f16")])
@pytest.mark.parametrize("counts,kd,inter", [([5, 0, 130, 1], 64, 128), ([300, 7, 0, 129], 192, 200),
                                             ([700, 100], 512, 1024)])
def test_rows_gemm_packed_swiglu_epilogues(impl, dtype, counts, kd, inter):
    """Epilogues 3 / 4: gate and up interleaved along the columns (the swiglu_packed layout)."""
    from xma import _lib, ops

    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    used = int(plan.pad_offsets[-1])
    a, _ = _grouped(plan, R, kd, dtype, seed=8)
    rng = np.random.RandomState(9)
    w1 = torch.from_numpy((rng.standard_normal((E, 2 * inter, kd)) * 0.05).astype(np.float32)).to(dtype).cuda()
    gu = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
    act = torch.full((plan.row_cap, inter), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, w1, _lib.W_NK, act, gu, None, plan.tile_expert, plan.tile_prefix, kd, 2 * inter,
                           _lib.EPI_SWIGLU_PACKED, impl)
    pad = plan.pad_offsets.cpu().tolist()
    exp_gu = torch.zeros(plan.row_cap, 2 * inter, dtype=torch.float64)
    for e in range(E):
        r0, c = pad[e], counts[e]
        if c:
            exp_gu[r0 : r0 + c] = a[r0 : r0 + c].double().cpu() @ w1[e].double().cpu().t()
    tol = REL_TOL[dtype]
    assert_close_rel(gu[:used].cpu(), exp_gu[:used], tol, "gate/up interleaved")
    stored = gu[:used].cpu().double()
    g, u = stored[:, 0::2], stored[:, 1::2]
    assert_close_rel(act[:used].cpu(), u * g * torch.sigmoid(g), tol / 2, "activation")

    H = kd
    dys, _ = _grouped(plan, R, H, dtype, seed=10)
    w2 = torch.from_numpy((rng.standard_normal((E, H, inter)) * 0.05).astype(np.float32)).to(dtype).cuda()
    dgu = torch.full((plan.row_cap, 2 * inter), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(dys, w2, _lib.W_KN, dgu, gu, None, plan.tile_expert, plan.tile_prefix, H, inter,
                           _lib.EPI_DSWIGLU_PACKED, impl)
    d_act = torch.zeros(plan.row_cap, inter, dtype=torch.float64)
    for e in range(E):
        r0, c = pad[e], counts[e]
        if c:
            d_act[r0 : r0 + c] = dys[r0 : r0 + c].double().cpu() @ w2[e].double().cpu()
    s = torch.sigmoid(g)
    assert_close_rel(dgu[:used, 0::2].cpu(), d_act[:used] * u * s * (1 + g * (1 - s)), 2 * tol, "d gate")
    assert_close_rel(dgu[:used, 1::2].cpu(), d_act[:used] * g * s, 2 * tol, "d up")
    assert _lib.read_and_clear_device_status() == 0
    # the CUDA-core kernels do not have these epilogues
    with pytest.raises(RuntimeError):
        ops.grouped_gemm_rows_(a, w1, _lib.W_NK, act, gu, None, plan.tile_expert, plan.tile_prefix, kd, 2 * inter,
                               _lib.EPI_SWIGLU_PACKED, SIMT)


@pytest.mark.parametrize("impl,dtype", [pytest.param(SIMT, torch.float32, id="cudacore-f32"),
                                        pytest.param(TC, torch.bfloat16, id="tcgen05-bf16"),
                                        pytest.param(TC_PAIR, torch.bfloat16, id="pair-bf16"),
                                        pytest.param(0, torch.float16, id="auto-f16")])
@pytest.mark.parametrize("counts,kd,n", [([5, 0, 130, 1], 64, 256), ([300, 7, 0, 0, 129, 64], 576, 264),
                                         ([1000, 24], 256, 1032), ([2300, 1100], 128, 512)])
@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_rows_gemm_peer_output_matches_scattered_output(impl, dtype, counts, kd, n, layout):
    """out_peers: every output row is stored into the buffer that its row_map word names
    ((buffer << 24) | row). The buffers here are tensors of the same device; the values must be bit-equal to
    the same GEMM without the table, whatever the epilogue does to coalesce the stores."""
    from xma import _lib, ops

    E, R = len(counts), int(sum(counts))
    plan, _ = _plan(counts, E)
    a, _ = _grouped(plan, R, kd, dtype, seed=4)
    rng = np.random.RandomState(6)
    shape = (E, n, kd) if layout == "nk" else (E, kd, n)
    w = torch.from_numpy((rng.standard_normal(shape) * 0.05).astype(np.float32)).to(dtype).cuda()
    wl = _lib.W_NK if layout == "nk" else _lib.W_KN

    ref = torch.full((plan.row_cap, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, w, wl, ref, None, None, plan.tile_expert, plan.tile_prefix, kd, n, _lib.EPI_PLAIN, impl)

    buffers = 3
    src = plan.row_src.cpu().numpy()
    valid = np.nonzero(src >= 0)[0]
    owner = rng.randint(0, buffers, size=valid.size)
    slot = np.empty(valid.size, np.int64)
    for b in range(buffers):
        idx = np.nonzero(owner == b)[0]
        slot[idx] = rng.permutation(idx.size)
    row_map = np.full(src.shape, -1, np.int32)
    row_map[valid] = (owner << 24) | slot
    cap = int(max((owner == b).sum() for b in range(buffers))) + 1
    outs = [torch.full((cap, n), float("nan"), dtype=dtype, device="cuda") for _ in range(buffers)]
    table = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device="cuda")
    # a few words that name a buffer outside the table or a row outside the buffers: their rows must be
    # skipped (nothing stored anywhere) and status bit 1 raised
    bad = rng.choice(valid.size, size=min(5, valid.size), replace=False)
    bad_words = row_map.copy()
    bad_words[valid[bad[0::2]]] = (buffers << 24) | 0            # buffer index == number of buffers
    bad_words[valid[bad[1::2]]] = (owner[bad[1::2]] << 24) | cap  # row == rows of the buffer
    ops.grouped_gemm_rows_(a, w, wl, outs[0], None, torch.from_numpy(bad_words).cuda(), plan.tile_expert,
                           plan.tile_prefix, kd, n, _lib.EPI_PLAIN, impl, table, cap)
    torch.cuda.synchronize()
    assert _lib.read_and_clear_device_status(torch.device("cuda")) == _lib.DEV_ID_OUT_OF_RANGE
    for i in bad:
        assert torch.isnan(outs[int(owner[i])][int(slot[i])]).all(), "a row with a bad word was stored"
    for o in outs:
        o.fill_(float("nan"))

    ops.grouped_gemm_rows_(a, w, wl, outs[0], None, torch.from_numpy(row_map).cuda(), plan.tile_expert,
                           plan.tile_prefix, kd, n, _lib.EPI_PLAIN, impl, table, cap)
    torch.cuda.synchronize()
    assert _lib.read_and_clear_device_status(torch.device("cuda")) == 0
    for b in range(buffers):
        idx = np.nonzero(owner == b)[0]
        got = outs[b][torch.from_numpy(slot[idx]).cuda()]
        want = ref[torch.from_numpy(valid[idx]).cuda()]
        assert torch.equal(got, want), (b, layout)
        untouched = np.setdiff1d(np.arange(cap), slot[idx])
        assert torch.isnan(outs[b][torch.from_numpy(untouched).cuda()]).all()


@pytest.mark.parametrize("impl", [TC, TC_PAIR])
def test_gemms_on_expert_slices_match_the_whole(impl):
    """The expert-parallel layer runs its experts group by group: weights `w[a:b]`, `tile_prefix[a:b+1]`,
    `counts[a:b]`, `pad_offsets[a:b+1]` are slices of the layer's tables, the row buffers stay whole. Two calls
    on two slices must write exactly what one call on all experts writes."""
    from xma import _lib, ops

    counts = [700, 0, 129, 2100, 64, 300]
    E, R, kd, n, dtype = len(counts), int(sum(counts)), 192, 512, torch.bfloat16
    plan, _ = _plan(counts, E)
    a, _ = _grouped(plan, R, kd, dtype, seed=11)
    y, _ = _grouped(plan, R, n, dtype, seed=12)
    rng = np.random.RandomState(13)
    w = torch.from_numpy((rng.standard_normal((E, n, kd)) * 0.05).astype(np.float32)).to(dtype).cuda()

    whole = torch.full((plan.row_cap, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_rows_(a, w, _lib.W_NK, whole, None, None, plan.tile_expert, plan.tile_prefix, kd, n,
                           _lib.EPI_PLAIN, impl)
    dw_whole = torch.full((E, kd, n), float("nan"), dtype=dtype, device="cuda")
    ops.grouped_gemm_dw_(a, y, plan.counts, plan.pad_offsets, dw_whole, impl)

    parts = torch.full((plan.row_cap, n), float("nan"), dtype=dtype, device="cuda")
    dw_parts = torch.full((E, kd, n), float("nan"), dtype=dtype, device="cuda")
    for lo, hi in ((0, 2), (2, 4), (4, 6)):
        ops.grouped_gemm_rows_(a, w[lo:hi], _lib.W_NK, parts, None, None, plan.tile_expert,
                               plan.tile_prefix[lo:hi + 1], kd, n, _lib.EPI_PLAIN, impl)
        ops.grouped_gemm_dw_(a, y, plan.counts[lo:hi], plan.pad_offsets[lo:hi + 1], dw_parts[lo:hi], impl)
    torch.cuda.synchronize()
    assert _lib.read_and_clear_device_status() == 0
    used = int(plan.pad_offsets[-1])
    assert torch.equal(parts[:used], whole[:used])
    assert torch.equal(dw_parts, dw_whole)
