"""Host-side logic of the expert-parallel layer on two CPU ranks (gloo): split sizes, the count
exchange, and the variable-size row exchange with its backward. The expert kernels themselves are
CUDA-only and are covered by the GPU tests; here the rows carry recognisable values instead."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "accelerated-model-architectures_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from xma.distributed import _AllToAllRows, exchange_counts, split_sizes

        E, H = 6, 4
        e_local = E // world
        # rank 0 routes 1,2,3 | 0,4,1 rows to experts 0..5; rank 1 routes 2,0,1 | 3,3,0
        counts = torch.tensor([[1, 2, 3, 0, 4, 1], [2, 0, 1, 3, 3, 0]][rank], dtype=torch.int32)
        send = split_sizes(counts, world)
        assert send == [[6, 5], [3, 6]][rank]
        recv_counts = exchange_counts(counts, dist.group.WORLD)
        expect = [[[1, 2, 3], [2, 0, 1]], [[0, 4, 1], [3, 3, 0]]][rank]
        assert recv_counts.tolist() == expect
        recv = recv_counts.sum(1).tolist()

        # rows sorted by expert; value = 1000 * source rank + 10 * expert + index within the expert
        rows = []
        for e in range(E):
            for i in range(int(counts[e])):
                rows.append(torch.full((H,), 1000.0 * rank + 10 * e + i))
        rows = torch.stack(rows).requires_grad_()
        got = _AllToAllRows.apply(rows, send, recv, dist.group.WORLD)
        assert got.shape == (sum(recv), H)
        want = []
        for src in range(world):
            for e in range(e_local):
                ge = rank * e_local + e
                for i in range(expect[src][e]):
                    want.append(1000.0 * src + 10 * ge + i)
        assert got[:, 0].tolist() == want

        # the experts here multiply a row by (global expert id + 1); send back and check the gradient path
        scale = torch.tensor([(int(v) % 1000) // 10 + 1 for v in want], dtype=torch.float32).unsqueeze(1)
        back = _AllToAllRows.apply(got * scale, recv, send, dist.group.WORLD)
        assert back.shape == rows.shape
        own_scale = torch.tensor([e + 1 for e in range(E) for _ in range(int(counts[e]))], dtype=torch.float32)
        assert torch.equal(back.detach(), rows.detach() * own_scale.unsqueeze(1))
        back.sum().backward()
        assert torch.equal(rows.grad, own_scale.unsqueeze(1).expand(-1, H))
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_expert_parallel_plumbing_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a gloo rank did not finish in time")
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: "ok", 1: "ok"}
