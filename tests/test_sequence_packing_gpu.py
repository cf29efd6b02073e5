"""GPU parity of pack_sequence / unpack_sequence (results and gradients, bit for bit) against the CPU oracle and the
stored outputs of the reference's torch path, on the grid of the reference's own test
(tests/functional/pack_sequence_test.py:20-130: padded [7, 1000, i, j] / packed [691, i, j] for seven (i, j), cumulative
lengths 0, 70, 170, 295, 393, 412, 515, 691 as uint32, fp32 / fp16 / bf16, both padding sides, eager and compiled)."""

import os

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import sequence_packing_oracle as sp

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF_CU = [0, 70, 170, 295, 393, 412, 515, 691]
REF_TRAILING = [(14, 16), (12, 14), (12, 21), (9, 7), (1, 1), (11, 11), (19, 19)]


def _bits(t: torch.Tensor) -> np.ndarray:
    """Exact comparison regardless of dtype: the raw bytes."""
    flat = t.detach().contiguous().cpu().reshape(-1)
    return flat.view(torch.uint8).numpy() if flat.numel() else np.zeros(0, np.uint8)


def _same(got: torch.Tensor, want: np.ndarray, like: torch.Tensor, what: str) -> None:
    want_t = torch.from_numpy(np.ascontiguousarray(want)).to(like.dtype)
    assert tuple(got.shape) == tuple(want_t.shape), (what, got.shape, want_t.shape)
    assert np.array_equal(_bits(got), _bits(want_t)), what


def _rand(shape, dtype, seed):
    rng = np.random.RandomState(seed)
    return torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dtype)


@pytest.mark.parametrize("side", ["left", "right"])
@pytest.mark.parametrize("name", list(gi.PACK_CASES))
def test_sequence_packing_golden(name, side):
    from xma.functional import pack_sequence, unpack_sequence

    gold = np.load(os.path.join(GOLDEN, "sequence_packing.npz"))
    inp = gi.pack_inputs(name)
    cu = torch.tensor(inp["cu_seqlens"], dtype=torch.int32, device="cuda")
    B, S, T = len(inp["cu_seqlens"]) - 1, inp["seq_len"], inp["cu_seqlens"][-1]
    key = f"{name}.{side}."
    x = inp["x"].cuda().requires_grad_()
    (y,) = pack_sequence([x], cu, T, side)
    (y * inp["dpacked"].cuda()).sum().backward()
    _same(y, gold[key + "pack"], y, "pack")
    _same(x.grad, gold[key + "pack_dx"], y, "pack_dx")
    p = inp["p"].cuda().requires_grad_()
    (z,) = unpack_sequence([p], cu, B, S, side)
    (z * inp["dpadded"].cuda()).sum().backward()
    _same(z, gold[key + "unpack"], z, "unpack")
    _same(p.grad, gold[key + "unpack_dx"], z, "unpack_dx")


@pytest.mark.parametrize("compiled", [False, True])
@pytest.mark.parametrize("side", ["left", "right"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@torch._dynamo.config.patch(recompile_limit=1024)
def test_sequence_packing_reference_grid(dtype, side, compiled):
    from xma import KernelBackend
    from xma.functional import pack_sequence, unpack_sequence

    pack_fn = torch.compile(pack_sequence, fullgraph=True) if compiled else pack_sequence
    unpack_fn = torch.compile(unpack_sequence, fullgraph=True) if compiled else unpack_sequence
    cu = torch.tensor(REF_CU, device="cuda", dtype=torch.uint32)
    B, S, T = len(REF_CU) - 1, 1000, REF_CU[-1]
    for n, trailing in enumerate(REF_TRAILING):
        x = _rand((B, S, *trailing), dtype, n)
        xd = x.cuda().requires_grad_()
        (y,) = pack_fn([xd], cu_seqlens=cu, total_tokens=T, padding_side=side, kernel_backend=KernelBackend.cuda)
        y.sum().backward()
        _same(y, sp.pack(x.float().numpy(), REF_CU, side), y, f"pack {trailing}")
        _same(xd.grad, sp.pack_backward(np.ones((T, *trailing), np.float32), REF_CU, S, side), y, f"pack dx {trailing}")

        p = _rand((T, *trailing), dtype, 100 + n)
        pd = p.cuda().requires_grad_()
        (z,) = unpack_fn([pd], cu_seqlens=cu, batch_size=B, sequence_length=S, padding_side=side,
                         kernel_backend=KernelBackend.cuda)
        z.sum().backward()
        _same(z, sp.unpack(p.float().numpy(), REF_CU, S, side), z, f"unpack {trailing}")
        _same(pd.grad, sp.unpack_backward(np.ones((B, S, *trailing), np.float32), REF_CU, side), z,
              f"unpack dx {trailing}")


@pytest.mark.parametrize("cu_dtype", [torch.int32, torch.uint32, torch.int64])
@pytest.mark.parametrize("side", ["left", "right"])
def test_sequence_packing_edges(cu_dtype, side):
    """Empty and full sequences, one sequence, nothing at all, several tensors per call, byte-sized and odd rows
    (copy units of 16, 8, 4, 2 and 1 bytes), a packed buffer longer than the sequences (zeros behind them)."""
    from xma.functional import pack_sequence, unpack_sequence

    cases = [
        ([0, 0, 6, 6, 6, 12, 12], 6, (8,), torch.float32),      # empty and full sequences, 32-byte rows
        ([0, 5], 9, (3,), torch.float32),                        # one sequence, 12-byte rows
        ([0, 2, 9], 7, (5,), torch.bfloat16),                    # 10-byte rows
        ([0, 2, 9], 7, (3,), torch.uint8),                       # 3-byte rows
        ([0, 4, 4, 5], 4, (2, 2), torch.float16),                # 8-byte rows
        ([0, 0, 0], 3, (4,), torch.float32),                     # no tokens at all
    ]
    for cu_list, S, trailing, dtype in cases:
        cu = torch.tensor(cu_list, device="cuda", dtype=cu_dtype)
        B, T = len(cu_list) - 1, cu_list[-1]
        rng = np.random.RandomState(S + T)
        mk = lambda *s: torch.from_numpy(rng.randint(1, 100, size=s).astype(np.float32)).to(dtype)
        x1, x2 = mk(B, S, *trailing), mk(B, S, 2)
        y1, y2 = pack_sequence([x1.cuda(), x2.cuda()], cu, T, side)
        _same(y1, sp.pack(x1.float().numpy(), cu_list, side), y1, f"pack {cu_list}")
        _same(y2, sp.pack(x2.float().numpy(), cu_list, side), y2, f"pack second {cu_list}")
        p = mk(T, *trailing)
        (z,) = unpack_sequence([p.cuda()], cu, B, S, side)
        _same(z, sp.unpack(p.float().numpy(), cu_list, S, side), z, f"unpack {cu_list}")
        # round trip: what was packed comes back, zeros elsewhere
        (back,) = unpack_sequence([y1], cu, B, S, side)
        _same(back, sp.unpack(sp.pack(x1.float().numpy(), cu_list, side), cu_list, S, side), back, "round trip")
        # a packed buffer with room behind the last sequence: zeros there
        (longer,) = pack_sequence([x1.cuda()], cu, T + 3, side)
        want = np.concatenate([sp.pack(x1.float().numpy(), cu_list, side), np.zeros((3, *trailing), np.float32)])
        _same(longer, want, longer, "tail")


def test_sequence_packing_large_round_trip():
    """Sizes of a training batch (8 x 4096 tokens of 4096 bf16 values, ragged lengths): pack then unpack returns the
    input with its padding zeroed; unpack then pack is the identity on the packed tokens."""
    from xma.functional import pack_sequence, unpack_sequence

    B, S, H = 8, 4096, 4096
    rng = np.random.RandomState(5)
    lens = rng.randint(1, S + 1, size=B)
    lens[3], lens[5] = S, 0
    cu_list = [0] + np.cumsum(lens).tolist()
    cu = torch.tensor(cu_list, device="cuda", dtype=torch.int32)
    T = cu_list[-1]
    x = torch.randn(B, S, H, device="cuda", dtype=torch.bfloat16)
    for side in ("left", "right"):
        (y,) = pack_sequence([x], cu, T, side)
        (z,) = unpack_sequence([y], cu, B, S, side)
        pos = torch.arange(S, device="cuda")[None, :]
        n = torch.tensor(lens, device="cuda")[:, None]
        valid = (pos >= S - n) if side == "left" else (pos < n)
        assert torch.equal(z, torch.where(valid[..., None], x, torch.zeros_like(x)))
        (y2,) = pack_sequence([z], cu, T, side)
        assert torch.equal(y2, y)
        for b in (0, 3, 7):
            seg = x[b, S - lens[b]:] if side == "left" else x[b, :lens[b]]
            assert torch.equal(y[cu_list[b]:cu_list[b + 1]], seg)


def test_sequence_packing_rejects_and_flags():
    from xma import KernelBackend, check_device_status
    from xma.functional import pack_sequence, unpack_sequence

    x = torch.zeros(2, 4, 3, device="cuda")
    cu = torch.tensor([0, 2, 5], device="cuda", dtype=torch.int32)
    with pytest.raises(ValueError):
        pack_sequence([x], cu, 5, "left", kernel_backend=KernelBackend.torch)
    with pytest.raises(AssertionError):
        pack_sequence([x], cu, 5, "middle")
    with pytest.raises(AssertionError):
        pack_sequence(x, cu, 5)
    with pytest.raises(AssertionError):
        unpack_sequence([torch.zeros(5, 3, device="cuda")], cu, 3, 4)
    # a sequence longer than the padded length is skipped and reported, not written out of bounds
    check_device_status()
    bad = torch.tensor([0, 5, 6], device="cuda", dtype=torch.int32)
    (z,) = unpack_sequence([torch.ones(6, 3, device="cuda")], bad, 2, 4, "right")
    assert float(z[0].abs().sum()) == 0.0 and float(z[1].sum()) == 3.0
    with pytest.raises(RuntimeError):
        check_device_status()
