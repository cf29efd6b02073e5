"""The scratch-free counting sort, called through the C ABI.

`xma_b200_count_sort_static` exists for callers that must not allocate device memory while they run
(an inference engine that reserved its whole budget up front, a plug-in that lives between other
allocators): it keeps the sort's scratch (per-tile counts, look-back words) in a fixed array inside the library. This test
drives it exactly as such a caller would - raw pointers, no scratch argument - twice in a row on the
same device, so the second call meets whatever the first one left in the shared array, and requires
the same bits as the regular entry point, which gets a fresh caller-owned scratch buffer each time.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(n, E, tile_cap):
    i32 = dict(dtype=torch.int32, device="cuda")
    return dict(
        counts=torch.full((E,), -7, **i32), offsets=torch.full((E,), -7, **i32),
        pad_offsets=torch.full((E + 1,), -7, **i32), tile_prefix=torch.full((E + 1,), -7, **i32),
        tile_expert=torch.full((tile_cap,), -7, **i32), sorted_expert=torch.full((max(n, 1),), -7, **i32),
        sorted_scattered=torch.full((max(n, 1),), -7, **i32), row_src=torch.full((tile_cap * 128,), -7, **i32),
    )


def _call(lib, ids, E, static, check_no_allocation=False):
    from xma import _lib

    n = ids.numel()
    tile_cap = int(lib.xma_b200_tile_capacity(n, E))
    o = _outputs(n, E, tile_cap)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if check_no_allocation:
        torch.cuda.synchronize()
        free_before, pool_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    stream = torch.cuda.current_stream().cuda_stream
    head = (ids.data_ptr(), _lib.I32, n, E, o["counts"].data_ptr(), o["offsets"].data_ptr(),
            o["pad_offsets"].data_ptr(), o["tile_prefix"].data_ptr(), o["tile_expert"].data_ptr(), tile_cap,
            o["sorted_expert"].data_ptr(), o["sorted_scattered"].data_ptr(), o["row_src"].data_ptr(), tile_cap * 128)
    if static:
        rc = lib.xma_b200_count_sort_static(*head, status.data_ptr(), stream)
    else:
        need = int(lib.xma_b200_count_sort_scratch_bytes(n, E))
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = lib.xma_b200_count_sort(*head, None, scratch.data_ptr(), need, status.data_ptr(), stream)
    assert rc == 0, _lib.error_string(rc)
    torch.cuda.synchronize()
    if check_no_allocation:
        # outputs were allocated before the call: neither the driver's free memory nor torch's pool may move
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_allocated() == pool_before
    assert int(status.item()) == 0
    used_tiles = int(o["tile_prefix"][-1])
    used_rows = int(o["pad_offsets"][-1])
    o["tile_expert"] = o["tile_expert"][:used_tiles]
    o["row_src"] = o["row_src"][:used_rows]
    return o


def test_static_scratch_sort_matches_regular_entry_point_twice():
    from xma import _lib

    lib = _lib.lib
    limit = int(lib.xma_b200_count_sort_static_scratch_limit())
    assert limit == 256 + 256 * 256 * 8
    rng = np.random.RandomState(123)
    # first call: many tiles and experts (fills most of the array); second: fewer of both, so any
    # state left behind by the first call would be read as look-back status if it were not cleared
    # (the first static call on a device may load the module, a driver-side allocation; from the second on the
    # call must leave the device's free memory and torch's pool exactly as they were)
    for call, (n, E) in enumerate(((900_001, 256), (70_003, 40))):
        assert int(lib.xma_b200_count_sort_scratch_bytes(n, E)) <= limit
        ids = torch.from_numpy(rng.randint(0, E, size=n).astype(np.int32)).cuda()
        got = _call(lib, ids, E, static=True, check_no_allocation=call > 0)
        want = _call(lib, ids, E, static=False)
        for key in want:
            assert torch.equal(got[key], want[key]), (n, E, key)
        # and both are the stable sort
        order = torch.sort(ids.long(), stable=True).indices.int()
        assert torch.equal(got["sorted_scattered"], order)


def test_static_scratch_sort_rejects_oversized_problems():
    from xma import _lib

    lib = _lib.lib
    n, E = 1 << 22, 1024  # needs far more scratch than the fixed array holds
    assert int(lib.xma_b200_count_sort_scratch_bytes(n, E)) > int(lib.xma_b200_count_sort_static_scratch_limit())
    ids = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.xma_b200_count_sort_static(ids.data_ptr(), _lib.I32, n, E, None, None, None, None, None, 0, None, None,
                                        None, 0, None, None)
    assert rc == -8 and "exceeds" in _lib.error_string(rc)
