"""One rank of the expert-parallel tests (spawned as a child process by tests/test_ep_gpu.py).

The rank runs `ExpertParallelMoE` on its own tokens and compares with the single-device CPU oracle
run on the concatenation of every rank's tokens: per-rank outputs and input gradients, expert weight
gradients on the owning rank, and the router gradient after the usual data-parallel sum.

Two set-ups:
  * one GPU per rank, NCCL (the real thing);
  * every rank on GPU 0, gloo: the peer transport's exchange buffers are still mapped across
    processes, and the barrier between the phases is a host barrier after a stream synchronise, so
    no kernel of one rank ever waits for a kernel of another.
"""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

E, K, H, I = 8, 2, 64, 128


def tokens_of(rank: int, base: int, step: int) -> int:
    """Ragged on purpose: ranks and steps have different token counts."""
    return base - 13 * rank + 120 * step


def global_inputs(world: int, base: int, step: int, dtype: torch.dtype):
    rng = np.random.RandomState(11 + step)
    total = sum(tokens_of(r, base, step) for r in range(world))
    mk = lambda *s, scale=1.0: torch.from_numpy((rng.standard_normal(s) * scale).astype(np.float32)).to(dtype)
    wrng = np.random.RandomState(5)
    wk = lambda *s: torch.from_numpy((wrng.standard_normal(s) * 0.02).astype(np.float32)).to(dtype)
    return dict(x=mk(total, H), dy=mk(total, H), gate=wk(E, H), w1=wk(E, 2 * I, H), w2=wk(E, H, I))


def run_rank(rank: int, world: int, port: int, results, cfg: dict) -> None:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "accelerated-model-architectures_b200"), os.path.join(root, "tests")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    shared_gpu = cfg["shared_gpu"]
    dev = torch.device("cuda", 0 if shared_gpu else rank)
    torch.cuda.set_device(dev)
    if shared_gpu:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import moe_oracle as orc
        from helpers import max_rel_err
        from xma import _lib
        from xma.distributed import ExpertParallelMoE, PeerLink
        from xma.layers import MoE, SwiGLU

        class HostSyncLink(PeerLink):
            """Ranks that share one GPU: collectives on the host, barrier = stream sync + host barrier."""

            def all_gather_counts(self, counts):
                mine = counts.cpu()
                outs = [torch.empty_like(mine) for _ in range(self.world)]
                dist.all_gather(outs, mine, group=self.group)
                return torch.stack(outs).to(counts.device)

            def barrier(self):
                torch.cuda.current_stream().synchronize()
                dist.barrier(group=self.group)

        dtype = getattr(torch, cfg["dtype"])
        transport, base = cfg["transport"], cfg["tokens"]
        e_local = E // world
        g0 = global_inputs(world, base, 0, dtype)
        moe = MoE(e_local, K, H, I, SwiGLU(), True, False, 0.02).to(device=dev, dtype=dtype)
        with torch.no_grad():
            moe.c_fc.weight.copy_(g0["w1"][rank * e_local : (rank + 1) * e_local])
            moe.c_proj.weight.copy_(g0["w2"][rank * e_local : (rank + 1) * e_local])
        link = HostSyncLink(dist.group.WORLD) if (shared_gpu and transport == "peer") else None
        layer = ExpertParallelMoE(moe, g0["gate"].to(dev), overlap_chunks=cfg["chunks"], transport=transport,
                                  link=link, fused_return=cfg.get("fused_return", True),
                                  private_copies=cfg.get("private_copies", False),
                                  pipeline_parts=cfg.get("parts"))

        errs = {}
        for step in range(cfg["steps"]):
            g = global_inputs(world, base, step, dtype)
            sizes = [tokens_of(r, base, step) for r in range(world)]
            lo = sum(sizes[:rank])
            sl = slice(lo, lo + sizes[rank])
            for p in layer.parameters():
                p.grad = None
            x = g["x"][sl].to(dev).requires_grad_()
            y, logits = layer(x)
            y.backward(g["dy"][sl].to(dev))
            torch.cuda.synchronize()
            assert _lib.read_and_clear_device_status(dev) == 0

            # the oracle routes from the logits the GPUs produced (rounding of the gate GEMM aside)
            mine = logits.detach().float().cpu()
            gathered = [torch.empty(sizes[r], E) for r in range(world)]
            gate_grad = layer.gate_weight.grad.detach().float().cpu()
            if shared_gpu:
                _gather_ragged(gathered, mine, rank, world)
                dist.all_reduce(gate_grad)
            else:
                _gather_ragged(gathered, mine, rank, world, device=dev)
                gg = gate_grad.to(dev)
                dist.all_reduce(gg)
                gate_grad = gg.cpu()

            f32 = lambda t: t.detach().float().cpu()
            ref = orc.moe_forward_backward(f32(g["x"]), f32(g["gate"]), f32(g["w1"]), f32(g["w2"]), K, "swiglu",
                                           dy=f32(g["dy"]), router_logits=torch.cat(gathered))
            d_logits = ref.grads["router_logits"]
            dx_ref = ref.grads["x_experts"] + d_logits @ f32(g["gate"])
            own = slice(rank * e_local, (rank + 1) * e_local)
            errs[step] = {
                "y": max_rel_err(y, ref.y[sl]),
                "dx": max_rel_err(x.grad, dx_ref[sl]),
                "dw1": max_rel_err(moe.c_fc.weight.grad, ref.grads["c_fc"][own]),
                "dw2": max_rel_err(moe.c_proj.weight.grad, ref.grads["c_proj"][own]),
                "dgate": max_rel_err(gate_grad, d_logits.t() @ f32(g["x"])),
            }
        if transport == "peer":
            layer.close()
        results[rank] = errs
    finally:
        dist.destroy_process_group()


def _gather_ragged(outs, mine, rank, world, device=None):
    """all_gather of tensors whose first dimension differs per rank (broadcast from each owner)."""
    for r in range(world):
        buf = mine.clone() if r == rank else outs[r]
        if device is not None:
            buf = buf.to(device)
        dist.broadcast(buf, src=r)
        outs[r] = buf.cpu()
