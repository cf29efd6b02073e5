"""Expert-parallel MoE on 2 GPUs (NCCL) against the single-device CPU oracle run on the
concatenation of both ranks' tokens: per-rank outputs and input gradients, expert weight gradients
on the owning rank, and the router gradient after the usual data-parallel sum."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

E, K, H, I, T = 8, 2, 64, 128, 150


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _global_inputs(world):
    rng = np.random.RandomState(11)
    mk = lambda *s, scale=1.0: torch.from_numpy((rng.standard_normal(s) * scale).astype(np.float32)).bfloat16()
    return dict(x=mk(world * T, H), dy=mk(world * T, H), gate=mk(E, H, scale=0.02), w1=mk(E, 2 * I, H, scale=0.02),
                w2=mk(E, H, I, scale=0.02))


def _worker(rank: int, world: int, port: int, results, chunks: int) -> None:
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "accelerated-model-architectures_b200"), os.path.join(root, "tests")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import moe_oracle as orc
        from helpers import max_rel_err
        from xma import _lib
        from xma.distributed import ExpertParallelMoE
        from xma.layers import MoE, SwiGLU

        g = _global_inputs(world)
        e_local = E // world
        moe = MoE(e_local, K, H, I, SwiGLU(), True, False, 0.02).to(device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            moe.c_fc.weight.copy_(g["w1"][rank * e_local : (rank + 1) * e_local])
            moe.c_proj.weight.copy_(g["w2"][rank * e_local : (rank + 1) * e_local])
        layer = ExpertParallelMoE(moe, g["gate"].to(dev), overlap_chunks=chunks)
        x = g["x"][rank * T : (rank + 1) * T].to(dev).requires_grad_()
        y, logits = layer(x)
        y.backward(g["dy"][rank * T : (rank + 1) * T].to(dev))
        torch.cuda.synchronize()
        assert _lib.read_and_clear_device_status(dev) == 0

        all_logits = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(all_logits, logits.detach().contiguous())
        gate_grad = layer.gate_weight.grad.clone()
        dist.all_reduce(gate_grad)

        f32 = lambda t: t.detach().float().cpu()
        ref = orc.moe_forward_backward(f32(g["x"]), f32(g["gate"]), f32(g["w1"]), f32(g["w2"]), K, "swiglu",
                                       dy=f32(g["dy"]), router_logits=f32(torch.cat(all_logits)))
        sl = slice(rank * T, (rank + 1) * T)
        d_logits = ref.grads["router_logits"]
        dx_ref = ref.grads["x_experts"] + d_logits @ f32(g["gate"])
        errs = {
            "y": max_rel_err(y, ref.y[sl]),
            "dx": max_rel_err(x.grad, dx_ref[sl]),
            "dw1": max_rel_err(moe.c_fc.weight.grad, ref.grads["c_fc"][rank * e_local : (rank + 1) * e_local]),
            "dw2": max_rel_err(moe.c_proj.weight.grad, ref.grads["c_proj"][rank * e_local : (rank + 1) * e_local]),
            "dgate": max_rel_err(gate_grad, d_logits.t() @ f32(g["x"])),
        }
        results[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("chunks", [1, 2])
def test_expert_parallel_matches_single_device_oracle(chunks):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results, chunks)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a rank did not finish in time")
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(world):
        for name, err in results[rank].items():
            assert err <= (4e-2 if name == "dgate" else 2e-2), (rank, name, err)
