"""MoE forward+backward throughput on B200 (tokens/s), one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c1] [--impl reference]

N = 1 runs the Mixtral-shaped layer of BASELINE.json configs[1] (16384 tokens, hidden 4096,
intermediate 14336, 8 experts, top-2, bf16) through `xma.layers.MoE`. For N > 1 the script is
launched by torchrun, one rank per GPU, and runs the same per-GPU workload expert-parallel
(experts sharded over ranks, NCCL all-to-all dispatch/combine): weak scaling.
A step = one forward + backward of the layer on one batch of seeded synthetic inputs.

`value`  : tokens/s with inputs resident in HBM (CUDA events around exactly K steps, max over ranks)
`e2e`    : the same metric with the step's inputs copied from pinned host memory and its results
           copied back inside the timed region
`roofline`: the dominant kernel family against the measured cuBLAS bf16 peak (MEASURED_PEAKS.json)
`cpu_baseline`: the CPU oracle (restatement of the reference's torch path) on a bounded sample
`--impl reference`: the reference's CPU implementation of the path = the oracle port (the reference
           is a Python package that cannot travel to the GPU box), on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "accelerated-model-architectures_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

# name -> tokens per GPU, hidden, intermediate, experts (global), top_k
WORKLOADS = {
    "c1": dict(tokens=512, hidden=256, inter=512, experts=8, top_k=2, dtype="f32",
               desc="configs[0] tiny fp32"),
    "c2": dict(tokens=16384, hidden=4096, inter=14336, experts=8, top_k=2, dtype="bf16",
               desc="configs[1] Mixtral-shaped: 4x4096 tokens, 8 experts top-2, SwiGLU"),
    "c2e2": dict(tokens=4096, hidden=4096, inter=14336, experts=2, top_k=2, dtype="bf16",
                 desc="profiling slice of configs[1]: same per-expert GEMM shapes (4096 rows/expert), 2 experts"),
    "c3": dict(tokens=32768, hidden=2048, inter=1024, experts=64, top_k=8, dtype="bf16",
               desc="configs[2] fine-grained: 64 experts top-8, Zipf(1.2)-skewed load"),
    "c4": dict(tokens=16384, hidden=4096, inter=1536, experts=128, top_k=8, dtype="bf16",
               desc="configs[3] expert-parallel: 128 experts top-8, uniform random logits"),
}
PEAK_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
METRIC = "moe_fwd_bwd_tokens_per_s"


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(PEAK_FALLBACK), "fallback"


def expert_flops(w: dict, tokens: int) -> float:
    """Algorithmic FLOPs of the expert GEMMs, forward + backward: 18 * R * H * I (R = tokens * top_k)."""
    return 18.0 * tokens * w["top_k"] * w["hidden"] * w["inter"]


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append((time.time(), line.strip()))

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def mark_begin(self) -> None:
        self.t_begin = time.time()

    def mark_end(self) -> None:
        self.t_end = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t0 = getattr(self, "t_begin", 0.0)
        t1 = getattr(self, "t_end", float("inf")) + 0.05
        for stamp, line in self.lines:
            if not (t0 <= stamp <= t1):
                continue  # keep the samples taken while the timed region ran
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # samples taken under load: the upper half of the observed clocks is not assumed; use all
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------------
def make_layer(w: dict, device: torch.device, dtype: torch.dtype, seed: int, local_experts: tuple[int, int] | None):
    """Random-init layer of the named shape. Weights ~ N(0, 0.02) (gate included: with N(0,1) inputs
    this gives near-uniform expert loads); the Zipf workload adds a per-expert logit bias through an
    extra constant input feature folded into the gate weight's last column."""
    from xma.layers import MoE, SwiGLU

    torch.manual_seed(seed)
    e0, e1 = local_experts if local_experts else (0, w["experts"])
    with torch.device(device):
        moe = MoE(e1 - e0, w["top_k"], w["hidden"], w["inter"], SwiGLU(), True, False, 0.02)
    moe = moe.to(dtype)
    # the router always sees every expert
    gen = torch.Generator(device="cpu").manual_seed(1234)
    gate = torch.randn(w["experts"], w["hidden"], generator=gen) * 0.02
    if w is WORKLOADS["c3"]:
        ranks = torch.randperm(w["experts"], generator=gen).float() + 1.0
        bias = -1.2 * torch.log(ranks)
        gate[:, -1] = bias  # paired with x[:, -1] = 1
    if w is WORKLOADS["c4"]:
        gate.zero_()  # logits come from uniform random features instead (see make_inputs)
    return moe, gate.to(device=device, dtype=dtype)


def make_inputs(w: dict, device: torch.device, dtype: torch.dtype, seed: int, pinned: bool):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    T, H = w["tokens"], w["hidden"]
    x = torch.randn(T, H, generator=gen)
    if w is WORKLOADS["c3"]:
        x[:, -1] = 1.0
    dy = torch.randn(T, H, generator=gen)
    x, dy = x.to(dtype), dy.to(dtype)
    if pinned:
        return x.pin_memory(), dy.pin_memory()
    return x.to(device), dy.to(device)


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's torch path
# ---------------------------------------------------------------------------------------------------
def cpu_step_tokens_per_s(w: dict, sample_tokens: int, steps: int, warmup: int) -> tuple[float, float, int]:
    """Times the oracle's forward+backward on `sample_tokens` tokens of the workload (same shapes per
    expert, same dtype) with all host threads. Returns (tokens/s, seconds per step, threads)."""
    from oracle import moe_oracle as orc

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    dtype = torch.float32 if w["dtype"] == "f32" else torch.bfloat16
    gen = torch.Generator().manual_seed(0)
    E, H, I, K = w["experts"], w["hidden"], w["inter"], w["top_k"]
    x = torch.randn(sample_tokens, H, generator=gen).to(dtype)
    dy = torch.randn(sample_tokens, H, generator=gen).to(dtype)
    gate = (torch.randn(E, H, generator=gen) * 0.02).to(dtype)
    w1 = torch.empty(E, 2 * I, H, dtype=dtype).normal_(0, 0.02, generator=gen)
    w2 = torch.empty(E, H, I, dtype=dtype).normal_(0, 0.02, generator=gen)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        orc.moe_forward_backward(x, gate, w1, w2, K, "swiglu", dy=dy)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return sample_tokens / sec, sec, threads


def cpu_sample_tokens(w: dict) -> int:
    # about 10-30 s of CPU work in total (a 16-core host sustains roughly 1.5-2 TFLOP/s bf16 on this path)
    target_flops = 2.0e13
    per_token = expert_flops(w, 1)
    return int(max(64, min(w["tokens"], 2 ** int(np.log2(max(target_flops / per_token, 64))))))


def run_reference_arm(args, w: dict, name: str) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = cpu_sample_tokens(w)
    value, sec, threads = cpu_step_tokens_per_s(w, sample, max(1, args.steps), max(0, min(args.warmup, 1)))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": f"{name}: {w['desc']}", "tokens_per_step_sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{sample} of {w['tokens']} tokens per step, full expert shapes, "
                                   "oracle/moe_oracle.py (CPU restatement of the reference torch path)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# configs[4]: routing microbench (HBM-bound kernels only)
# ---------------------------------------------------------------------------------------------------
def zipf_ids(n: int, bins: int, s: float, seed: int) -> np.ndarray:
    rng = np.random.RandomState(seed)
    p = 1.0 / np.arange(1, bins + 1) ** s
    cdf = np.cumsum(p / p.sum())
    ranks = np.searchsorted(cdf, rng.random_sample(n), side="right").clip(0, bins - 1)
    return rng.permutation(bins)[ranks].astype(np.int32)


def run_routing_microbench(args) -> None:
    """continuous_count, the counting sort and the row permute of BASELINE configs[4]: 64 Mi int32 ids
    over 256 bins (uniform and Zipf(1.1)) and rows of 2048 bf16. The 64 Mi x 2048 token buffer of the
    config is 256 GiB and does not fit a B200, so the permute moves the first `rows` rows (8 Mi =
    32 GiB in + 32 GiB out) with the sort permutation of the first `rows` ids; GB/s does not depend on
    the row count at this size."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from xma import ops
    from xma.functional import continuous_count
    from xma.layers.moe import build_route_plan

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks.get("hbm_gbs", PEAK_FALLBACK["hbm_gbs"]))
    n, bins, width = 1 << 26, 256, 2048
    rows = 1 << 23
    steps, warm = max(args.steps, 5), max(args.warmup, 3)

    def timed(fn) -> float:
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    out = {}
    for dist_name, ids_np in (("uniform", np.random.RandomState(0).randint(0, bins, size=n).astype(np.int32)),
                              ("zipf1.1", zipf_ids(n, bins, 1.1, 1))):
        ids = torch.from_numpy(ids_np).to(device)
        ms = timed(lambda: continuous_count(ids, bins))
        out[f"continuous_count_{dist_name}"] = {"ms": ms, "gbs": n * 4 / ms / 1e6, "frac": n * 4 / ms / 1e6 / hbm,
                                               "bytes": n * 4}
        ms = timed(lambda: build_route_plan(ids.view(-1, 1), bins))
        # algorithmic bytes: ids read by the histogram and by the scatter pass (8 B/id), sorted ids,
        # permutation and padded row map written (12 B/id)
        out[f"count_sort_{dist_name}"] = {"ms": ms, "gbs": n * 20 / ms / 1e6, "frac": n * 20 / ms / 1e6 / hbm,
                                         "bytes": n * 20}
        if dist_name == "uniform":
            plan = build_route_plan(ids[:rows].view(-1, 1), bins)
    src = torch.randn(rows, width, device=device, dtype=torch.bfloat16)
    dst = torch.empty(plan.row_cap, width, device=device, dtype=torch.bfloat16)
    ms = timed(lambda: ops.gather_rows_(src, plan.row_src, None, 1, plan.rows_in_use, dst))
    moved = rows * width * 2 * 2 + rows * 4
    out["permute_rows_2048_bf16"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / ms / 1e6 / hbm,
                                     "bytes": moved, "rows": rows}
    del dst
    w8 = torch.rand(rows // 8, 8, device=device, dtype=torch.bfloat16)
    y = torch.empty(rows // 8, width, device=device, dtype=torch.bfloat16)
    ms = timed(lambda: ops.combine_rows_(src, w8, 8, y))
    moved = rows * width * 2 + (rows // 8) * width * 2
    out["combine_rows_top8_2048_bf16"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / ms / 1e6 / hbm,
                                          "bytes": moved}
    best = out["permute_rows_2048_bf16"]
    print(json.dumps({
        "metric": "routing_hbm_gb_per_s", "value": best["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": best["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int32/bf16", "data": "synthetic",
        "config": {"workload": "c5: configs[4] routing microbench, 64 Mi ids over 256 bins; permute of 8 Mi x 2048 bf16 rows",
                   "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": "gather_rows_kernel", "achieved": best["gbs"], "peak": hbm,
                     "unit": "GB/s", "frac": best["frac"], "peak_source": f"{peak_kind} copy bandwidth",
                     "traffic": None},
        "kernels": out,
    }), flush=True)


def run_ep_microbench(args) -> None:
    """Kernels of the expert-parallel peer transport on ONE GPU, with the shapes one rank of configs[1] sees
    at 4 ranks (2 local experts, 32768 received rows of 4096 bf16, I = 14336): the "ranks" are buffers of
    the same device addressed through the same pointer tables, so the figures are HBM figures (what the
    kernels cost before NVLink enters) and the kernels can be captured by ncu, which a multi-rank run cannot."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from xma import _lib, ops
    from xma.layers.moe import build_route_plan

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks.get("hbm_gbs", PEAK_FALLBACK["hbm_gbs"]))
    W, E, K, H, I, T = 4, 8, 2, 4096, 14336, 16384
    el, R, dt = E // W, T * K, torch.bfloat16
    steps, warm = max(args.steps, 1), max(args.warmup, 1)

    def timed(fn) -> float:
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    gen = torch.Generator(device="cpu").manual_seed(0)
    sel = torch.stack([torch.randperm(E, generator=gen)[:K] for _ in range(T)]).to(torch.int32).to(device)
    plan = build_route_plan(sel, E)
    cm = plan.counts.view(1, E).repeat(W, 1).contiguous()  # every virtual rank routes like this one
    host = cm.cpu().numpy().astype(np.int64)
    padded = ((host.sum(0) + 127) // 128 * 128).reshape(W, el).sum(1)
    cap, rows0 = int(padded.max()) + el * 128, int(padded[0])
    recv = [torch.zeros(cap, H, dtype=dt, device=device) for _ in range(W)]
    meta = [torch.full((cap,), -1, dtype=torch.int32, device=device) for _ in range(W)]
    home = [torch.empty(R, H, dtype=dt, device=device) for _ in range(W)]
    table = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=device)
    recv_table, meta_table, home_table = table(recv), table(meta), table(home)
    x = torch.randn(T, H, device=device, dtype=dt)

    def plan_rank(r: int):
        t = dict(send_delta=torch.empty(E, dtype=torch.int32, device=device),
                 counts=torch.empty(el, dtype=torch.int32, device=device),
                 pad_offsets=torch.empty(el + 1, dtype=torch.int32, device=device),
                 tile_prefix=torch.empty(el + 1, dtype=torch.int32, device=device),
                 tile_expert=torch.empty(int(padded[r]) // 128 + el, dtype=torch.int32, device=device))
        ops.ep_plan_(cm, r, t["send_delta"], t["counts"], t["pad_offsets"], t["tile_prefix"], t["tile_expert"], meta[r])
        return t

    tables = [plan_rank(r) for r in range(W)]
    dispatch = lambda r: ops.ep_dispatch_(x, plan.sorted_expert_idxs, plan.sorted_scattered_idxs, None, K,
                                          tables[r]["send_delta"], W, r, recv_table, meta_table, cap)
    for r in range(1, W):
        dispatch(r)
    out = {}
    row_bytes = H * 2
    ms = timed(lambda: plan_rank(0))
    out["ep_plan"] = {"ms": ms}
    ms = timed(lambda: dispatch(0))
    moved = R * (2 * row_bytes + 12)
    out["ep_dispatch"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / ms / 1e6 / hbm, "bytes": moved}
    t0 = tables[0]
    alloc = t0["tile_expert"].numel() * 128
    xs = torch.empty(alloc, H, dtype=dt, device=device)
    ms = timed(lambda: ops.ep_copy_rows_(recv[0], meta[0], xs[:rows0]))
    moved = rows0 * (2 * row_bytes + 4)
    out["ep_copy_rows"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / ms / 1e6 / hbm, "bytes": moved}
    ms = timed(lambda: ops.ep_return_(xs[:rows0], meta[0], W, home_table, R))
    out["ep_return"] = {"ms": ms, "gbs": moved / ms / 1e6, "frac": moved / ms / 1e6 / hbm, "bytes": moved}

    act = torch.randn(alloc, I, device=device, dtype=dt)
    w2 = torch.randn(el, H, I, device=device, dtype=dt) * 0.02
    ys = torch.empty(alloc, H, dtype=dt, device=device)
    flops = 2.0 * rows0 * I * H
    ms = timed(lambda: ops.grouped_gemm_rows_(act, w2, _lib.W_NK, ys, None, None, t0["tile_expert"], t0["tile_prefix"],
                                              I, H, _lib.EPI_PLAIN, 0))
    out["gemm_down_plain"] = {"ms": ms, "tflops": flops / ms / 1e9}
    ms = timed(lambda: ops.grouped_gemm_rows_(act, w2, _lib.W_NK, home[0], None, meta[0], t0["tile_expert"],
                                              t0["tile_prefix"], I, H, _lib.EPI_PLAIN, 0, home_table, R))
    out["gemm_down_rows_to_ranks"] = {"ms": ms, "tflops": flops / ms / 1e9}
    _lib.raise_on_device_status(device)
    best = out["ep_dispatch"]
    print(json.dumps({
        "metric": "ep_row_exchange_hbm_gb_per_s", "value": best["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": best["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"ep: peer-transport kernels of configs[1] at {W} ranks, ranks emulated as buffers of one GPU",
                   "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": "ep_dispatch_kernel", "achieved": best["gbs"], "peak": hbm,
                     "unit": "GB/s", "frac": best["frac"], "peak_source": f"{peak_kind} copy bandwidth", "traffic": None},
        "kernels": out,
    }), flush=True)


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c5", "ep"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--transport", choices=["peer", "nccl"], default="peer",
                    help="row exchange of the expert-parallel layer: stores into peer memory, or NCCL all-to-all")
    ap.add_argument("--unfused-return", dest="fused_return", action="store_false",
                    help="peer transport: return rows with a separate row kernel instead of the GEMM epilogues")
    ap.add_argument("--ep-chunks", type=int, default=None,
                    help="micro-batches per step in the expert-parallel layer (overlap of all-to-all and GEMM)")
    args = ap.parse_args()
    if args.workload == "c5":
        run_routing_microbench(args)
        return
    if args.workload == "ep":
        run_ep_microbench(args)
        return
    w = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, w, args.workload)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 kernels are the only implementation (no CPU path)")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    from xma import _lib, ops

    dtype = torch.float32 if w["dtype"] == "f32" else torch.bfloat16
    E = w["experts"]
    if E % world:
        raise SystemExit(f"{E} experts do not shard over {world} ranks")
    local = (rank * E // world, (rank + 1) * E // world)
    moe, gate = make_layer(w, device, dtype, seed=100 + rank, local_experts=local if world > 1 else None)
    if world > 1:
        from xma.distributed import ExpertParallelMoE, PeerLink

        if args.transport == "peer":
            # the peer transport needs the ranks to map each other's memory; where the node does not allow
            # that, every rank learns it here (share() fails collectively) and the run uses NCCL all-to-all
            try:
                probe = PeerLink(dist.group.WORLD)
                probe.release(*probe.share(1 << 20, device)[::2])
            except RuntimeError as exc:
                if rank == 0:
                    print(f"peer transport unavailable ({exc}); using NCCL all-to-all", file=sys.stderr)
                args.transport = "nccl"
        layer = ExpertParallelMoE(moe, gate, world_group=dist.group.WORLD, overlap_chunks=args.ep_chunks,
                                  transport=args.transport, fused_return=args.fused_return)
    else:
        with torch.no_grad():
            moe.gate.weight.copy_(gate)
        layer = moe
    x_dev, dy_dev = make_inputs(w, device, dtype, seed=rank, pinned=False)
    if w is WORKLOADS["c4"]:
        # uniform random router logits: bypass the gate projection by making it an identity on E features
        gen = torch.Generator(device="cpu").manual_seed(77 + rank)
        x_dev[:, :E] = torch.rand(w["tokens"], E, generator=gen).to(device=device, dtype=dtype)
        with torch.no_grad():
            g = torch.zeros(E, w["hidden"], device=device, dtype=dtype)
            g[:, :E] = torch.eye(E, device=device, dtype=dtype)
            (layer.gate_weight if world > 1 else moe.gate.weight).copy_(g)

    params = list(layer.parameters())

    def step(x: torch.Tensor, dy: torch.Tensor):
        for p in params:
            p.grad = None
        xin = x.detach().requires_grad_()
        y, _ = layer(xin)
        y.backward(dy)
        return y, xin.grad

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing --------------------------------------------------------------
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    sampler.start()  # nvidia-smi needs a moment to come up; samples are filtered to the timed region
    for _ in range(max(args.warmup, 3)):
        step(x_dev, dy_dev)
    barrier()
    _lib.raise_on_device_status(device)

    ops.STATS.enabled, ops.STATS.timing = True, True
    ops.STATS.reset()
    barrier()
    sampler.mark_begin()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        step(x_dev, dy_dev)
    t_end.record()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop()
    ms_total = max_over_ranks(t_start.elapsed_time(t_end))
    launches = ops.STATS.launches
    kernel_ms = ops.STATS.elapsed_ms()
    ops.STATS.enabled = ops.STATS.timing = False
    _lib.raise_on_device_status(device)
    ms_per_step = ms_total / args.steps
    tokens_per_step = w["tokens"] * world
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- end to end: pinned host inputs in, results out, every step ------------------------------
    x_pin, dy_pin = make_inputs(w, device, dtype, seed=rank, pinned=True)
    if w is WORKLOADS["c4"]:
        x_pin.copy_(x_dev.cpu())
    y_host = torch.empty_like(x_pin).pin_memory()
    dx_host = torch.empty_like(x_pin).pin_memory()

    # Every step's inputs come from pinned host memory and its results go back to pinned host memory.
    # The copies run on their own streams so that the upload of step s+1 and the download of step s-1
    # overlap the kernels of step s (double-buffered device inputs); all of it is inside the timed region.
    main_stream = torch.cuda.current_stream()
    h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
    x_buf = [torch.empty_like(x_dev) for _ in range(2)]
    dy_buf = [torch.empty_like(dy_dev) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def upload(s: int) -> None:
        b = s & 1
        h2d.wait_event(consumed[b])  # the step that last read this buffer pair has finished
        with torch.cuda.stream(h2d):
            x_buf[b].copy_(x_pin, non_blocking=True)
            dy_buf[b].copy_(dy_pin, non_blocking=True)
            uploaded[b].record(h2d)

    def e2e_run(steps: int) -> None:
        for ev in consumed:
            ev.record(main_stream)
        upload(0)
        for s in range(steps):
            b = s & 1
            if s + 1 < steps:
                upload(s + 1)
            main_stream.wait_event(uploaded[b])
            y, dx = step(x_buf[b], dy_buf[b])
            consumed[b].record(main_stream)
            d2h.wait_event(consumed[b])
            with torch.cuda.stream(d2h):
                y_host.copy_(y, non_blocking=True)
                dx_host.copy_(dx, non_blocking=True)
            y.record_stream(d2h)
            dx.record_stream(d2h)
        main_stream.wait_stream(d2h)

    e2e_run(4)  # the caching allocator settles (tensors held for the downloads change its working set)
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    e2e_run(args.steps)
    e_end.record()
    barrier()
    e2e_ms = max_over_ranks(e_start.elapsed_time(e_end)) / args.steps
    e2e_value = tokens_per_step / (e2e_ms * 1e-3)
    bytes_in = (x_pin.numel() + dy_pin.numel()) * x_pin.element_size()
    bytes_out = (y_host.numel() + dx_host.numel()) * y_host.element_size()

    # ---- roofline of the dominant kernel family ----------------------------------------------------
    peaks, peak_kind = measured_peaks()
    T_local = w["tokens"] * (world if world > 1 else 1) // world  # tokens routed through this rank on average
    R = T_local * w["top_k"]
    H, I = w["hidden"], w["inter"]
    gemm_flops = {  # algorithmic FLOPs per launch
        "gemm_up_swiglu": 2.0 * R * H * 2 * I, "gemm_down": 2.0 * R * I * H, "gemm_dact_dswiglu": 2.0 * R * H * I,
        "gemm_dx": 2.0 * R * 2 * I * H, "gemm_dw1": 2.0 * R * 2 * I * H, "gemm_dw2": 2.0 * R * H * I,
    }
    per_kernel = {}
    for name, times in kernel_ms.items():
        per_kernel[name] = {"launches": len(times), "ms_total": sum(times), "ms_avg": sum(times) / len(times)}
        if name in gemm_flops:
            per_kernel[name]["tflops"] = gemm_flops[name] / (per_kernel[name]["ms_avg"] * 1e-3) / 1e12
    # One entry per kernel function; the dominant one (largest share of the timed region) gets the roofline.
    kernel_functions = {
        "rows_gemm_tc2_kernel<T, W_NK, SwiGLU> (up projection, CTA pairs)": ["gemm_up_swiglu"],
        "rows_gemm_tc_kernel<T, W_NK, plain> (down projection)": ["gemm_down"],
        "rows_gemm_tc2_kernel<T, W_KN, dSwiGLU> (d activation, CTA pairs)": ["gemm_dact_dswiglu"],
        "rows_gemm_tc_kernel<T, W_KN, plain> (d input)": ["gemm_dx"],
        "dw_gemm_tc2_kernel<T> (dW1 and dW2, CTA pairs)": ["gemm_dw1", "gemm_dw2"],
    }
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures of the
    # 2-expert slice `c2e2` summarised in profiles/ncu_grouped_gemm_tcgen05_c2e2.md; traffic grows in
    # proportion to the number of experts at fixed rows per expert, so configs[1] moves experts/2 times this
    # on one GPU (expert-parallel ranks see other rows per expert: no figure there). The dominant kernel is the
    # weight-gradient GEMM; the four rows-GEMM entries were captured with the older tile order (an expert's row
    # tiles innermost) and are upper bounds for the grouped order.
    ncu_traffic_c2e2 = {"gemm_up_swiglu": 1.435e9, "gemm_down": 1.279e9, "gemm_dact_dswiglu": 1.784e9,
                        "gemm_dx": 2.500e9, "gemm_dw1": 1.524e9, "gemm_dw2": 0.782e9}
    peak = float(peaks.get("bf16_tflops_sustained", PEAK_FALLBACK["bf16_tflops_sustained"]))
    groups = {}
    for fn, tags in kernel_functions.items():
        tags = [t for t in tags if t in per_kernel]
        if not tags:
            continue
        ms = sum(per_kernel[t]["ms_total"] for t in tags)
        n_launch = sum(per_kernel[t]["launches"] for t in tags)
        flops = sum(gemm_flops[t] * per_kernel[t]["launches"] for t in tags)
        groups[fn] = {"ms_total": ms, "launches": n_launch, "tflops": flops / (ms * 1e-3) / 1e12,
                      "share_of_step": ms / (ms_per_step * args.steps), "tags": tags}
    roofline = None
    all_gemms = None
    if groups:
        fn = max(groups, key=lambda k: groups[k]["ms_total"])
        g = groups[fn]
        traffic = None
        if world == 1 and args.workload in ("c2", "c2e2") and all(t in ncu_traffic_c2e2 for t in g["tags"]):
            scale = E / 2.0
            traffic = scale * sum(ncu_traffic_c2e2[t] for t in g["tags"]) / len(g["tags"])
        roofline = {
            "bound": "tensor", "kernel": fn, "achieved": g["tflops"], "peak": peak, "unit": "TFLOP/s",
            "frac": g["tflops"] / peak, "peak_source": f"{peak_kind} cuBLAS bf16 sustained (kernel timed inside a long step)",
            "traffic": traffic, "launches_per_step": g["launches"] // args.steps,
            "ms_per_launch": g["ms_total"] / g["launches"], "share_of_step": g["share_of_step"],
            "frac_of_nominal_2250": g["tflops"] / 2250.0,
        }
        gemm_ms = sum(g["ms_total"] for g in groups.values())
        achieved = sum(gemm_flops.values()) * args.steps / (gemm_ms * 1e-3) / 1e12
        all_gemms = {"tflops": achieved, "frac": achieved / peak, "frac_of_nominal_2250": achieved / 2250.0,
                     "share_of_step": gemm_ms / (ms_per_step * args.steps),
                     "by_kernel": {k: {"tflops": v["tflops"], "share_of_step": v["share_of_step"]}
                                   for k, v in groups.items()}}
    step_tflops = expert_flops(w, tokens_per_step // world) / (ms_per_step * 1e-3) / 1e12

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        sample = cpu_sample_tokens(w)
        v, sec, threads = cpu_step_tokens_per_s(w, sample, 1, 1)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{sample} of {w['tokens']} tokens, full expert shapes, {sec:.1f} s per step, "
                         "oracle/moe_oracle.py on the host cores"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "tokens_per_gpu": w["tokens"],
                       "hidden": H, "intermediate": I, "experts": E, "top_k": w["top_k"],
                       "parallelism": "single GPU" if world == 1 else
                       f"expert-parallel ep{world}, "
                       + (("dispatch kernel + GEMM epilogues" if args.fused_return else "dispatch and return kernels")
                          + " storing rows into peer memory over NVLink"
                          if args.transport == "peer" else "NCCL all-to-all")
                       + f", {layer.overlap_chunks} micro-batch(es) per step",
                       "l2_policy": "inputs_exceed_l2 (weights + activations >> 126 MB)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out},
            "gpu_launches": launches,
            "roofline": roofline,
            "all_grouped_gemms": all_gemms,
            "step_tflops_per_gpu": step_tflops,
            "kernels": per_kernel,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        if world > 1 and args.transport == "peer":
            layer.close()  # collective: unmap the other ranks' exchange buffers before anyone frees them
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
