"""Host-side logic of the expert-parallel layer on two CPU ranks (gloo): split sizes, the count
exchange, and the variable-size row exchange with its backward. The expert kernels themselves are
CUDA-only and are covered by the GPU tests; here the rows carry recognisable values instead.
A second test drives the peer transport's buffer mapping and growth logic with the CUDA calls faked,
including a mapping that fails on one rank only."""

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


def _peer_worker(rank: int, world: int, port: int, results) -> None:
    """Host logic of the peer transport with the CUDA calls replaced by fakes: buffer mapping that
    fails on one rank must raise on every rank (nobody is left waiting in a collective), and the
    exchange buffers grow by the same collective decision on every rank."""
    import ctypes
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "accelerated-model-architectures_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from xma import distributed as ep

        log = []

        class FakeBlock:
            fail_on: int | None = None

            def __init__(self, nbytes, device):
                if FakeBlock.fail_on == rank:
                    raise RuntimeError("allocation refused (injected)")
                self.nbytes, self.ptr = nbytes, 0x1000 * (rank + 1)
                self.tensor = torch.zeros(nbytes, dtype=torch.uint8)

            def export(self):
                return bytes([rank]) * 64

            def free(self):
                log.append(("free", self.nbytes))
                self.tensor, self.ptr = None, 0

        class FakeLib:
            open_fails_on: int | None = None

            @staticmethod
            def xma_b200_exchange_open(handle, out_ref):
                if FakeLib.open_fails_on == rank:
                    return -7
                ctypes.cast(out_ref, ctypes.POINTER(ctypes.c_void_p))[0] = 0x9000 + handle[0]
                return 0

            @staticmethod
            def xma_b200_exchange_close(address):
                log.append(("close", address))
                return 0

        def fake_check(rc, name):
            if rc != 0:
                raise RuntimeError(f"{name} failed with status {rc}")

        class _NoDeviceGuard:
            def __init__(self, device):
                pass

            def __enter__(self):
                return self

            def __exit__(self, *exc):
                return False

        ep._DeviceBlock, ep.lib, ep.check = FakeBlock, FakeLib, fake_check
        torch.cuda.device = _NoDeviceGuard
        torch.cuda.synchronize = lambda *a, **k: None
        link = ep.PeerLink(dist.group.WORLD)
        cpu = torch.device("cpu")

        # 1. everything works: own address for this rank, mapped addresses for the others
        block, addresses, mapped = link.share(256, cpu)
        assert addresses[rank] == 0x1000 * (rank + 1)
        assert [a for r, a in enumerate(addresses) if r != rank] == [0x9000 + r for r in range(world) if r != rank]
        assert mapped == [a for r, a in enumerate(addresses) if r != rank]
        link.release(block, mapped)
        assert ("free", 256) in log and ("close", mapped[0]) in log

        # 2. allocation fails on rank 1 only, 3. mapping fails on rank 0 only: both ranks raise
        for attr, holder, bad in (("fail_on", FakeBlock, 1), ("open_fails_on", FakeLib, 0)):
            setattr(holder, attr, bad)
            try:
                link.share(256, cpu)
                raised = False
            except RuntimeError as exc:
                raised = "could not map" in str(exc)
            setattr(holder, attr, None)
            assert raised, (attr, rank)
            dist.barrier()  # nobody is stuck in a collective

        # 4. exchange buffers: capacity with head-room, regrown only when a need exceeds it
        ex = ep._Exchange(link, cpu, torch.float32, hidden=8, fused_return=False)
        ex.ensure(300, 200)
        assert (ex.recv_cap, ex.home_cap) == (384, 256)
        assert ex.recv_rows.shape == (384, 8) and ex.recv_meta.shape == (384,) and ex.home_rows.shape == (256, 8)
        assert ex.recv_table.tolist()[rank] == 0x1000 * (rank + 1)
        held = list(ex._held)
        ex.ensure(384, 256)
        assert ex._held == held  # fits: nothing reallocated
        ex.ensure(385, 10)
        assert ex.recv_cap == 512 and ex.home_cap == 256 and ex._held != held
        # 5. the expert groups of the pipelined exchange: contiguous groups of this rank's experts with their padded
        #    row ranges, at most one group per expert, one group when nothing is known about the rows per expert
        ep.ops.ep_plan_ = lambda *args, **kwargs: None
        counts = torch.zeros(world, 4 * world, dtype=torch.int32)
        padded = [128, 256, 128, 512]
        route = ep._PeerRoute(counts, rank, 1024, ex, local_padded=padded, parts=2)
        assert route.parts == [(0, 2, 0, 384), (2, 4, 384, 1024)]
        assert (route.e_local, route.tile_expert.numel(), route.send_delta.numel()) == (4, 1024 // 128 + 4, 4 * world)
        route = ep._PeerRoute(counts, rank, 1024, ex, local_padded=padded, parts=9)
        assert route.parts == [(0, 1, 0, 128), (1, 2, 128, 384), (2, 3, 384, 512), (3, 4, 512, 1024)]
        assert ep._PeerRoute(counts, rank, 1024, ex, local_padded=padded, parts=1).parts == [(0, 4, 0, 1024)]
        assert ep._PeerRoute(counts, rank, 1024, ex, local_padded=None, parts=3).parts == [(0, 4, 0, 1024)]
        ex.close()
        assert ex._held == [] and ex.recv_rows is None
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_peer_transport_host_logic_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, results)) for r in range(world)]
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
