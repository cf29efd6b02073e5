"""GPU parity of the routing kernels against the CPU oracle: continuous_count, top-k + softmax
(forward and backward) and the stable counting sort with its tables. Integer outputs bit-exact."""

import os

import numpy as np
import pytest
import torch

import inputs as gi
from helpers import assert_close_rel, sizes_1d, zipf_ids
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(autouse=True)
def _status_clean():
    from xma import _lib

    yield
    assert _lib.read_and_clear_device_status() == 0


# ---- continuous_count ---------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(gi.COUNT_CASES))
@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_continuous_count_golden(name, dtype):
    from xma.functional import continuous_count

    gold = np.load(os.path.join(GOLDEN, "continuous_count.npz"))
    ids, bins = gi.count_inputs(name)
    got = continuous_count(torch.from_numpy(ids).to(dtype).cuda(), bins)
    assert got.dtype == torch.uint32 and got.shape == (bins,)
    assert np.array_equal(got.cpu().numpy().astype(np.int64), gold[name])


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_continuous_count_reference_size_list(dtype):
    """Sizes and id range of the reference's test (tests/functional/continuous_count_test.py:18-41)."""
    from xma.functional import continuous_count

    rng = np.random.RandomState(42)
    for n in sizes_1d():
        ids = rng.randint(0, 72, size=n)
        got = continuous_count(torch.from_numpy(ids).to(dtype).cuda(), 72)
        assert np.array_equal(got.cpu().numpy(), orc.continuous_count(ids, 72)), n


def test_continuous_count_edge_cases():
    from xma import KernelBackend, _lib
    from xma.functional import continuous_count

    empty = continuous_count(torch.zeros(0, dtype=torch.int32, device="cuda"), 5)
    assert empty.cpu().tolist() == [0] * 5
    assert continuous_count(torch.zeros(9, dtype=torch.int64, device="cuda"), 1).cpu().tolist() == [9]
    # a view that does not start on a 16-byte boundary
    rng = np.random.RandomState(3)
    ids = rng.randint(0, 16, size=10007).astype(np.int32)
    dev = torch.from_numpy(ids).cuda()
    for off in (1, 2, 3):
        got = continuous_count(dev[off:], 16, kernel_backend=KernelBackend.cuda)
        assert np.array_equal(got.cpu().numpy(), orc.continuous_count(ids[off:], 16))
    # many bins (counters do not fit in shared memory) and sorted input (worst-case contention)
    big = rng.randint(0, 50000, size=200000).astype(np.int64)
    got = continuous_count(torch.from_numpy(big).cuda(), 50000)
    assert np.array_equal(got.cpu().numpy(), orc.continuous_count(big, 50000))
    srt = np.sort(rng.randint(0, 8, size=100000)).astype(np.int64)
    got = continuous_count(torch.from_numpy(srt).cuda(), 8)
    assert np.array_equal(got.cpu().numpy(), orc.continuous_count(srt, 8))
    # out-of-range ids are ignored and flagged
    bad = np.array([0, 3, -1, 4, 7, 3], dtype=np.int64)
    got = continuous_count(torch.from_numpy(bad).cuda(), 4)
    assert got.cpu().tolist() == [1, 0, 0, 2]
    assert _lib.read_and_clear_device_status() == _lib.DEV_ID_OUT_OF_RANGE
    with pytest.raises(ValueError):
        continuous_count(dev, 16, kernel_backend=KernelBackend.triton)


@pytest.mark.parametrize("dist", ["uniform", "zipf"])
def test_continuous_count_full_size(dist):
    """The routing microbench at full size: 64 Mi int32 ids over 256 bins, uniform and Zipf(1.1)."""
    from xma.functional import continuous_count

    n = 1 << 26
    if dist == "uniform":
        ids = np.random.RandomState(0).randint(0, 256, size=n).astype(np.int32)
    else:
        ids = zipf_ids(n, 256, 1.1, seed=1)
    got = continuous_count(torch.from_numpy(ids).cuda(), 256)
    assert np.array_equal(got.cpu().numpy(), orc.continuous_count(ids, 256))


# ---- top-k + softmax ---------------------------------------------------------------------------
def _logits(T, E, dtype, ties, seed):
    rng = np.random.RandomState(seed)
    if ties:  # few distinct values -> ties at and inside the top-k boundary on most rows
        a = rng.randint(-3, 4, size=(T, E)).astype(np.float32) * 0.5
    else:
        a = rng.standard_normal((T, E)).astype(np.float32)
    return torch.from_numpy(a).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("E,K", [(2, 1), (2, 2), (8, 2), (6, 4), (64, 8), (72, 3), (128, 8), (256, 8), (1000, 32)])
@pytest.mark.parametrize("ties", [False, True])
def test_topk_softmax(dtype, E, K, ties):
    from xma import ops

    T = 517
    logits = _logits(T, E, dtype, ties, seed=E * 31 + K)
    w_ref, sel_ref = orc.route(logits, K)
    dev = logits.cuda()
    w = torch.empty(T, K, dtype=dtype, device="cuda")
    sel = torch.empty(T, K, dtype=torch.int32, device="cuda")
    ops.route_topk_softmax_(dev, K, w, sel)
    assert torch.equal(sel.cpu().long(), sel_ref)
    assert_close_rel(w.cpu().float(), w_ref.float(), 1e-6 if dtype == torch.float32 else 8e-3, "router weights")
    sel64 = torch.empty(T, K, dtype=torch.int64, device="cuda")
    ops.route_topk_softmax_(dev, K, w, sel64)
    assert torch.equal(sel64.cpu(), sel_ref)

    dw = torch.from_numpy(np.random.RandomState(5).standard_normal((T, K)).astype(np.float32)).to(dtype)
    dl_ref = orc.route_backward(logits, sel_ref, dw)
    dl = torch.full((T, E), float("nan"), dtype=dtype, device="cuda")
    ops.route_topk_softmax_bwd_(dev, sel, dw.cuda(), dl)
    assert_close_rel(dl.cpu().float(), dl_ref.float(), 1e-5 if dtype == torch.float32 else 1e-2, "d_logits")


def test_topk_nan_and_inf():
    from xma import ops

    logits = torch.tensor([[0.0, float("nan"), 2.0, float("inf")], [float("-inf"), -1.0, float("-inf"), -2.0]])
    _, sel_ref = orc.route(logits, 2)
    w = torch.empty(2, 2, device="cuda")
    sel = torch.empty(2, 2, dtype=torch.int32, device="cuda")
    ops.route_topk_softmax_(logits.cuda(), 2, w, sel)
    assert torch.equal(sel.cpu().long(), sel_ref)


# ---- counting sort -------------------------------------------------------------------------------
def _check_sort(ids: np.ndarray, E: int, dtype=torch.int32):
    from xma.layers.moe import build_route_plan

    plan = build_route_plan(torch.from_numpy(ids).to(dtype).cuda().view(-1, 1), E)
    ref = orc.count_sort(ids, E)
    assert np.array_equal(plan.expert_frequency.cpu().numpy(), ref.counts)
    assert np.array_equal(plan.offsets_incl.cpu().numpy(), ref.offsets_incl)
    assert np.array_equal(plan.pad_offsets.cpu().numpy(), ref.pad_offsets)
    assert np.array_equal(plan.tile_prefix.cpu().numpy(), ref.tile_prefix)
    used = int(ref.tile_prefix[-1])
    assert np.array_equal(plan.tile_expert.cpu().numpy()[:used], ref.tile_expert)
    assert np.array_equal(plan.sorted_expert_idxs.cpu().numpy(), ref.sorted_expert_idxs)
    assert np.array_equal(plan.sorted_scattered_idxs.cpu().numpy(), ref.sorted_scattered_idxs)
    rows = int(ref.pad_offsets[-1])
    assert np.array_equal(plan.row_src.cpu().numpy()[:rows], ref.row_src)
    return plan


@pytest.mark.parametrize("n,E", [(1, 1), (7, 2), (14, 16), (1024, 8), (4096, 8), (4097, 72), (12293, 64),
                                 (70001, 256), (300000, 1024), (262144, 64)])
def test_count_sort_matches_oracle(n, E):
    ids = np.random.RandomState(n + E).randint(0, E, size=n).astype(np.int32)
    _check_sort(ids, E)


def test_count_sort_skew_empty_experts_and_int64():
    rng = np.random.RandomState(9)
    ids = zipf_ids(50000, 64, 1.2, seed=2)
    _check_sort(ids, 64)
    ids = rng.choice([1, 5, 6], size=9000).astype(np.int32)  # most experts receive nothing
    _check_sort(ids, 8)
    _check_sort(np.sort(ids), 8)
    _check_sort(ids[::-1].copy(), 8)
    _check_sort(rng.randint(0, 128, size=20000).astype(np.int64), 128, dtype=torch.int64)
    _check_sort(np.zeros(0, dtype=np.int32), 4)


def test_count_sort_is_deterministic():
    ids = np.random.RandomState(1).randint(0, 32, size=100000).astype(np.int32)
    a = _check_sort(ids, 32)
    b = _check_sort(ids, 32)
    assert torch.equal(a.sorted_scattered_idxs, b.sorted_scattered_idxs)


@pytest.mark.parametrize("dist", ["uniform", "zipf"])
def test_count_sort_full_size_properties(dist):
    """64 Mi ids over 256 bins: counts equal bincount, output sorted, a permutation, and stable."""
    from xma.layers.moe import build_route_plan

    n = 1 << 26
    ids = (np.random.RandomState(0).randint(0, 256, size=n).astype(np.int32) if dist == "uniform"
           else zipf_ids(n, 256, 1.1, seed=1))
    dev = torch.from_numpy(ids).cuda()
    plan = build_route_plan(dev.view(-1, 1), 256)
    assert np.array_equal(plan.expert_frequency.cpu().numpy(), orc.continuous_count(ids, 256))
    se, ss = plan.sorted_expert_idxs, plan.sorted_scattered_idxs
    assert bool((se[1:] >= se[:-1]).all())
    assert torch.equal(dev[ss.long()], se)  # row p really holds expert se[p]
    same = se[1:] == se[:-1]
    assert bool((ss[1:][same] > ss[:-1][same]).all())  # stable: ties by flat index
    seen = torch.zeros(n, dtype=torch.int8, device="cuda")
    seen[ss.long()] = 1
    assert int(seen.sum(dtype=torch.int64)) == n  # every flat index exactly once
    # checksum of checksums against the CPU oracle on the first million sorted rows
    ref = orc.count_sort(ids, 256)
    assert np.array_equal(ss[: 1 << 20].cpu().numpy(), ref.sorted_scattered_idxs[: 1 << 20])
    assert int(ss.sum(dtype=torch.int64)) == n * (n - 1) // 2


def test_check_device_status_raises_once_and_clears():
    """`xma.check_device_status()` surfaces what the kernels flagged asynchronously: an id outside the bins is
    skipped by the kernel (the counts are those of the valid ids) and reported by the next check, which also clears
    the word."""
    import xma
    from xma.functional import continuous_count

    xma.check_device_status()  # clean slate
    ids = torch.tensor([0, 1, 7, 3, 1], dtype=torch.int32, device="cuda")
    counts = continuous_count(ids, 4)
    assert counts.cpu().tolist() == [1, 2, 0, 1]
    with pytest.raises(RuntimeError, match="out of range"):
        xma.check_device_status()
    xma.check_device_status()  # cleared by the check that raised
