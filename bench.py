"""MoE forward+backward throughput on B200 (tokens/s), one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c1] [--impl reference]

N = 1 runs the Mixtral-shaped layer (16384 tokens, hidden 4096, intermediate 14336, 8 experts,
top-2, SwiGLU, bf16) through `xma.layers.MoE`. For N > 1 the script is
launched by torchrun, one rank per GPU, and runs the same per-GPU workload expert-parallel
(experts sharded over ranks, NCCL all-to-all dispatch/combine): weak scaling.
A step = one forward + backward of the layer on one batch of seeded synthetic inputs.

After the headline workload the same process times the fine-grained skewed layer (64 experts top-8,
N = 1 only) and the 128-expert top-8 layer (at the same N) with fewer steps and reports them under
`configs2` / `configs3`, and checks the headline layer's results against the CPU oracle
(`parity_check`, outside every timed region).

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
               desc="tiny fp32 layer"),
    "c2": dict(tokens=16384, hidden=4096, inter=14336, experts=8, top_k=2, dtype="bf16",
               desc="Mixtral-shaped: 4x4096 tokens, 8 experts top-2, SwiGLU"),
    "c2e2": dict(tokens=4096, hidden=4096, inter=14336, experts=2, top_k=2, dtype="bf16",
                 desc="profiling slice of c2: same per-expert GEMM shapes (4096 rows/expert), 2 experts"),
    "c3": dict(tokens=32768, hidden=2048, inter=1024, experts=64, top_k=8, dtype="bf16",
               desc="fine-grained: 64 experts top-8, Zipf(1.2)-skewed load"),
    "c4": dict(tokens=16384, hidden=4096, inter=1536, experts=128, top_k=8, dtype="bf16",
               desc="expert-parallel shape: 128 experts top-8, uniform random logits"),
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
    steps, warm = max(1, args.steps), max(0, min(args.warmup, 1))  # one warm-up step is all a CPU arm needs
    value, sec, threads = cpu_step_tokens_per_s(w, sample, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "warmup_requested": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": f"{name}: {w['desc']}", "tokens_per_step_sample": sample,
                   "note": f"each step runs {sample} of the workload's {w['tokens']} tokens through the full expert "
                           "shapes; tokens/s is per token, so the sample size does not enter it"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{sample} of {w['tokens']} tokens per step, full expert shapes, "
                                   "oracle/moe_oracle.py (CPU restatement of the reference torch path)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# routing microbench (HBM-bound kernels only)
# ---------------------------------------------------------------------------------------------------
def zipf_ids(n: int, bins: int, s: float, seed: int) -> np.ndarray:
    rng = np.random.RandomState(seed)
    p = 1.0 / np.arange(1, bins + 1) ** s
    cdf = np.cumsum(p / p.sum())
    ranks = np.searchsorted(cdf, rng.random_sample(n), side="right").clip(0, bins - 1)
    return rng.permutation(bins)[ranks].astype(np.int32)


def run_routing_microbench(args) -> None:
    """continuous_count, the counting sort and the row permute of the routing microbench: 64 Mi int32 ids
    over 256 bins (uniform and Zipf(1.1)) and rows of 2048 bf16. A 64 Mi x 2048 token buffer would be
    256 GiB and does not fit a B200, so the permute moves the first `rows` rows (8 Mi =
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
    n, bins, width = 1 << args.ids_log2, 256, 2048
    rows = min(1 << 23, n)
    steps, warm = max(args.steps, 5 if not args.ids_only else 1), max(args.warmup, 3 if not args.ids_only else 1)

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
    if args.ids_only:  # the id kernels alone (a small, short run for a profiler capture)
        print(json.dumps({"metric": "routing_hbm_gb_per_s", "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warm,
                          "config": {"workload": f"c5 ids only: {n} ids over {bins} bins"}, "kernels": out}), flush=True)
        return
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
        "config": {"workload": f"c5: routing microbench, {n} ids over 256 bins; permute of {rows} x 2048 bf16 rows",
                   "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": "gather_rows_kernel", "achieved": best["gbs"], "peak": hbm,
                     "unit": "GB/s", "frac": best["frac"], "peak_source": f"{peak_kind} copy bandwidth",
                     "traffic": None},
        "kernels": out,
    }), flush=True)


def run_ep_microbench(args) -> None:
    """Kernels of the expert-parallel peer transport on ONE GPU, with the shapes one rank of workload c2 sees
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
        "config": {"workload": f"ep: peer-transport kernels of workload c2 at {W} ranks, ranks emulated as buffers of one GPU",
                   "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": "ep_dispatch_kernel", "achieved": best["gbs"], "peak": hbm,
                     "unit": "GB/s", "frac": best["frac"], "peak_source": f"{peak_kind} copy bandwidth", "traffic": None},
        "kernels": out,
    }), flush=True)


# ---------------------------------------------------------------------------------------------------
# stand-alone swiglu / swiglu_packed (HBM-bound)
# ---------------------------------------------------------------------------------------------------
def run_swiglu_microbench(args) -> None:
    """`swiglu` and `swiglu_packed`, forward and backward, on the shape of the reference's own throughput
    scripts (tools/throughput_swiglu.py:31-32,61-75 and tools/throughput_swiglu_packed.py:26-27,48-62):
    B = 16 * 4096 rows, H = 4096 columns, fp32 / fp16 / bf16, algorithmic bytes 3 * B * H * itemsize forward and
    5 * B * H * itemsize backward, against the measured copy bandwidth."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from xma.functional import swiglu, swiglu_packed

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks.get("hbm_gbs", PEAK_FALLBACK["hbm_gbs"]))
    B, H = int(args.rmsnorm_rows), 4096
    full = B == 16 * 4096
    steps, warm = (max(args.steps, 20), max(args.warmup, 5)) if full else (args.steps, args.warmup)
    wanted = [t.strip() for t in args.rmsnorm_dtypes.split(",") if t.strip()]

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
    for dtype, tag in ((torch.float32, "f32"), (torch.float16, "f16"), (torch.bfloat16, "bf16")):
        item = torch.empty((), dtype=dtype).element_size()
        g = torch.randn(B, H, device=device, dtype=dtype, requires_grad=True)
        u = torch.randn(B, H, device=device, dtype=dtype, requires_grad=True)
        dy = torch.randn(B, H, device=device, dtype=dtype)
        ms = timed(lambda: swiglu(g.detach(), u.detach()))
        out[f"swiglu_fwd_{tag}"] = {"ms": ms, "gbs": 3 * B * H * item / ms / 1e6}
        z = swiglu(g, u)
        ms = timed(lambda: torch.autograd.grad(z, (g, u), grad_outputs=dy, retain_graph=True))
        out[f"swiglu_bwd_{tag}"] = {"ms": ms, "gbs": 5 * B * H * item / ms / 1e6}
        del z
        # gate and up as the two halves of one [B, 2H] buffer (the layout `chunk(2, -1)` hands over)
        gu = torch.randn(B, 2 * H, device=device, dtype=dtype)
        ms = timed(lambda: swiglu(*gu.chunk(2, dim=-1)))
        out[f"swiglu_fwd_chunked_{tag}"] = {"ms": ms, "gbs": 3 * B * H * item / ms / 1e6}
        xp = gu.requires_grad_()
        ms = timed(lambda: swiglu_packed(xp.detach()))
        out[f"swiglu_packed_fwd_{tag}"] = {"ms": ms, "gbs": 3 * B * H * item / ms / 1e6}
        zp = swiglu_packed(xp)
        ms = timed(lambda: torch.autograd.grad(zp, (xp,), grad_outputs=dy, retain_graph=True))
        out[f"swiglu_packed_bwd_{tag}"] = {"ms": ms, "gbs": 5 * B * H * item / ms / 1e6}
        del zp, xp, gu, g, u, dy
    for v in out.values():
        v["frac"] = v["gbs"] / hbm
    worst = min(out, key=lambda k: out[k]["frac"])
    head = out["swiglu_bwd_bf16"]
    print(json.dumps({
        "metric": "swiglu_hbm_gb_per_s", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"swiglu: stand-alone swiglu / swiglu_packed, {B} x {H}, fp32/fp16/bf16, forward and backward",
                   "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": "swiglu_bwd_kernel<bf16>", "achieved": head["gbs"], "peak": hbm,
                     "unit": "GB/s", "frac": head["frac"], "peak_source": f"{peak_kind} copy bandwidth",
                     "traffic": None},
        "lowest": {"kernel": worst, **out[worst]},
        "kernels": out,
    }), flush=True)


# ---------------------------------------------------------------------------------------------------
# fused_residual_add_rmsnorm (HBM-bound)
# ---------------------------------------------------------------------------------------------------
def run_rmsnorm_microbench(args) -> None:
    """`fused_residual_add_rmsnorm` forward and backward on [16 * 4096, 4096] (the activation shape in front of the
    dense-expert layer), fp32 / fp16 / bf16, with weight, residual and multiplier. Algorithmic bytes: forward reads
    x and the residual and writes y and the new residual stream (4 * B * H * itemsize); backward reads the stream,
    dy and d(stream) and writes dx and d(residual) (5 * B * H * itemsize); weight and row statistics are noise."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from xma.functional import fused_residual_add_rmsnorm

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks.get("hbm_gbs", PEAK_FALLBACK["hbm_gbs"]))
    B, H = int(args.rmsnorm_rows), 4096
    full = B == 16 * 4096
    steps, warm = (max(args.steps, 20), max(args.warmup, 5)) if full else (args.steps, args.warmup)
    wanted = [t.strip() for t in args.rmsnorm_dtypes.split(",") if t.strip()]

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
    for dtype, tag in ((torch.float32, "f32"), (torch.float16, "f16"), (torch.bfloat16, "bf16")):
        if tag not in wanted:
            continue
        item = torch.empty((), dtype=dtype).element_size()
        x = torch.randn(B, H, device=device, dtype=dtype, requires_grad=True)
        r = torch.randn(B, H, device=device, dtype=dtype, requires_grad=True)
        w = torch.randn(H, device=device, dtype=dtype, requires_grad=True)
        dy, dxr = torch.randn(B, H, device=device, dtype=dtype), torch.randn(B, H, device=device, dtype=dtype)
        ms = timed(lambda: fused_residual_add_rmsnorm(x.detach(), r.detach(), w.detach(), 1e-5, 0.9))
        out[f"rmsnorm_fwd_{tag}"] = {"ms": ms, "gbs": 4 * B * H * item / ms / 1e6}
        y, xr = fused_residual_add_rmsnorm(x, r, w, 1e-5, 0.9)
        ms = timed(lambda: torch.autograd.grad((y, xr), (x, r, w), grad_outputs=(dy, dxr), retain_graph=True))
        out[f"rmsnorm_bwd_{tag}"] = {"ms": ms, "gbs": 5 * B * H * item / ms / 1e6}
        del y, xr, x, r, w, dy, dxr
    for v in out.values():
        v["frac"] = v["gbs"] / hbm
    worst = min(out, key=lambda k: out[k]["frac"])
    head_name = "rmsnorm_fwd_bf16" if "rmsnorm_fwd_bf16" in out else sorted(out)[0]
    head = out[head_name]
    print(json.dumps({
        "metric": "rmsnorm_hbm_gb_per_s", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"rmsnorm: fused_residual_add_rmsnorm, {B} x {H}, fp32/fp16/bf16, forward and backward "
                               "(backward includes the sum of the weight-gradient partial rows)",
                   "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": head_name, "achieved": head["gbs"], "peak": hbm,
                     "unit": "GB/s", "frac": head["frac"], "peak_source": f"{peak_kind} copy bandwidth",
                     "traffic": None},
        "lowest": {"kernel": worst, **out[worst]},
        "kernels": out,
    }), flush=True)


# ---------------------------------------------------------------------------------------------------
# pack_sequence / unpack_sequence (HBM-bound)
# ---------------------------------------------------------------------------------------------------
def run_packing_microbench(args) -> None:
    """`pack_sequence` and `unpack_sequence` on a ragged training batch: 16 sequences padded to 4096 tokens of
    4096 bf16 values (512 MiB padded), seeded lengths uniform in [1024, 4096], both padding sides. Algorithmic bytes:
    pack reads and writes the valid tokens (2 * T * row bytes); unpack reads the valid tokens and writes the whole
    padded batch ((T + B * S) * row bytes)."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    from xma.functional import pack_sequence, unpack_sequence

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks.get("hbm_gbs", PEAK_FALLBACK["hbm_gbs"]))
    B, S, H = 16, 4096, 4096
    steps, warm = max(args.steps, 20), max(args.warmup, 5)
    rng = np.random.RandomState(0)
    lens = rng.randint(1024, S + 1, size=B)
    cu_list = [0] + np.cumsum(lens).tolist()
    T = cu_list[-1]
    cu = torch.tensor(cu_list, device=device, dtype=torch.int32)
    x = torch.randn(B, S, H, device=device, dtype=torch.bfloat16)
    p = torch.randn(T, H, device=device, dtype=torch.bfloat16)
    row = H * 2

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
    for side in ("left", "right"):
        ms = timed(lambda: pack_sequence([x], cu, T, side))
        out[f"pack_{side}"] = {"ms": ms, "gbs": 2 * T * row / ms / 1e6}
        ms = timed(lambda: unpack_sequence([p], cu, B, S, side))
        out[f"unpack_{side}"] = {"ms": ms, "gbs": (T + B * S) * row / ms / 1e6}
    for v in out.values():
        v["frac"] = v["gbs"] / hbm
    worst = min(out, key=lambda k: out[k]["frac"])
    head = out["pack_left"]
    print(json.dumps({
        "metric": "pack_sequence_hbm_gb_per_s", "value": head["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": warm, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bytes", "data": "synthetic",
        "config": {"workload": f"packing: pack_sequence / unpack_sequence, {B} x {S} x {H} bf16 padded, {T} valid "
                               "tokens, both padding sides", "l2_policy": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm", "kernel": "sequence_packing_kernel<uint4, int, pack>", "achieved": head["gbs"],
                     "peak": hbm, "unit": "GB/s", "frac": head["frac"], "peak_source": f"{peak_kind} copy bandwidth",
                     "traffic": None},
        "lowest": {"kernel": worst, **out[worst]},
        "kernels": out,
    }), flush=True)


# ---------------------------------------------------------------------------------------------------
# DRAM traffic table (ncu) and kernel names
# ---------------------------------------------------------------------------------------------------
KERNEL_SOURCES = ("grouped_gemm_sm100.cu", "grouped_gemm_sm100_2cta.cu", "sm100_common.cuh", "gemm_api.cu")
TRAFFIC_TABLE = os.path.join(ROOT, "profiles", "dram_traffic_grouped_gemm_c2e2.md")


def kernel_source_digest() -> str:
    """sha256 over the grouped-GEMM kernel sources: a traffic table names the digest it was captured with."""
    import hashlib

    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        with open(os.path.join(ROOT, "accelerated-model-architectures_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def load_traffic_table() -> tuple[dict | None, str]:
    """-> ({tag: DRAM bytes per launch on the 2-expert slice}, note). The table is a text summary of an ncu
    capture (`dram__bytes_read.sum + dram__bytes_write.sum` per launch); it is used only while the kernel
    sources still have the digest the capture was taken with, otherwise the traffic is reported as null."""
    if not os.path.exists(TRAFFIC_TABLE):
        return None, "no ncu traffic table in profiles/"
    digest, rows = None, {}
    with open(TRAFFIC_TABLE) as f:
        for line in f:
            parts = [c.strip() for c in line.strip().strip("|").split("|")]
            if line.startswith("kernel-source-digest:"):
                digest = line.split(":", 1)[1].strip()
            elif len(parts) >= 2 and parts[0].startswith("gemm_"):
                try:
                    rows[parts[0]] = float(parts[1])
                except ValueError:
                    pass
    if digest != kernel_source_digest():
        return None, f"ncu traffic table is older than the kernel sources (table {digest}, sources {kernel_source_digest()})"
    return rows, "profiles/dram_traffic_grouped_gemm_c2e2.md (ncu, 2-expert slice, scaled by experts / 2)"


_IMPL_NAMES = {1: "CUDA cores", 2: "tcgen05, one CTA per 128x256 tile", 3: "tcgen05, CTA pairs, 256x256 tiles"}


def gemm_kernel_names(w: dict, rows_per_rank: int, local_experts: int, peer: bool, dtype: torch.dtype) -> dict:
    """tag -> the kernel function the automatic choice launches for this workload (asked of the library)."""
    from xma import _lib

    H, I = w["hidden"], w["inter"]
    code = _lib.dtype_code(dtype)
    tile_cap = rows_per_rank // _lib.ROW_PAD + local_experts
    q = _lib.lib.xma_b200_grouped_gemm_choice
    rows = lambda kd, n, wl, epi, p=0: q(0, code, local_experts, tile_cap, kd, n, wl, epi, p)
    dw = lambda m, n: q(1, code, local_experts, tile_cap, m, n, 0, 0, 0)
    fam = {2: "rows_gemm_tc_kernel", 3: "rows_gemm_tc2_kernel", 1: "rows_gemm_simt_kernel"}
    famw = {2: "dw_gemm_tc_kernel", 3: "dw_gemm_tc2_kernel", 1: "dw_gemm_simt_kernel"}
    choice = {
        "gemm_up_swiglu": (fam, rows(H, 2 * I, _lib.W_NK, _lib.EPI_SWIGLU), "<T, W_NK, SwiGLU>"),
        "gemm_down": (fam, rows(I, H, _lib.W_NK, _lib.EPI_PLAIN, int(peer)), "<T, W_NK, plain%s>" % (" to peers" if peer else "")),
        "gemm_dact_dswiglu": (fam, rows(H, I, _lib.W_KN, _lib.EPI_DSWIGLU), "<T, W_KN, dSwiGLU>"),
        "gemm_dx": (fam, rows(2 * I, H, _lib.W_KN, _lib.EPI_PLAIN, int(peer)), "<T, W_KN, plain%s>" % (" to peers" if peer else "")),
        "gemm_dw1": (famw, dw(2 * I, H), "<T>"),
        "gemm_dw2": (famw, dw(H, I), "<T>"),
    }
    return {tag: f"{f[impl]}{targs} ({_IMPL_NAMES[impl]})" for tag, (f, impl, targs) in choice.items()}


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
class Bench:
    """One process of the GPU arm: device, process group, and the helpers every workload shares."""

    def __init__(self, args) -> None:
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torchrun --nproc-per-node {args.gpus}")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist
        self.transport = args.transport

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        if self.dist is None:
            return ms
        t = torch.tensor([ms], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gpu_index(self) -> int:
        if "CUDA_VISIBLE_DEVICES" not in os.environ:
            return self.local_rank
        return int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[self.local_rank])


def build_workload(b: Bench, name: str):
    """-> (layer, local MoE, x, dy) on the device, for this rank."""
    w = WORKLOADS[name]
    args, rank, world, device = b.args, b.rank, b.world, b.device
    dtype = torch.float32 if w["dtype"] == "f32" else torch.bfloat16
    E = w["experts"]
    if E % world:
        raise SystemExit(f"{E} experts do not shard over {world} ranks")
    local = (rank * E // world, (rank + 1) * E // world)
    moe, gate = make_layer(w, device, dtype, seed=100 + rank, local_experts=local if world > 1 else None)
    if world > 1:
        from xma.distributed import ExpertParallelMoE, PeerLink

        if b.transport == "peer":
            # the peer transport needs the ranks to map each other's memory; where the node does not allow
            # that, every rank learns it here (share() fails collectively) and the run uses NCCL all-to-all
            try:
                probe = PeerLink(b.dist.group.WORLD)
                probe.release(*probe.share(1 << 20, device)[::2])
            except RuntimeError as exc:
                if rank == 0:
                    print(f"peer transport unavailable ({exc}); using NCCL all-to-all", file=sys.stderr)
                b.transport = "nccl"
        layer = ExpertParallelMoE(moe, gate, world_group=b.dist.group.WORLD, overlap_chunks=args.ep_chunks,
                                  transport=b.transport, fused_return=args.fused_return,
                                  private_copies=args.private_copies, pipeline_parts=args.ep_parts)
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
    return layer, moe, x_dev, dy_dev


def make_step(layer):
    params = list(layer.parameters())

    def step(x: torch.Tensor, dy: torch.Tensor):
        for p in params:
            p.grad = None
        xin = x.detach().requires_grad_()
        y, logits = layer(xin)
        y.backward(dy)
        return y, xin.grad, logits

    return step


def release_layer(b: Bench, layer) -> None:
    if b.world > 1 and b.transport == "peer":
        layer.close()  # collective: unmap the other ranks' exchange buffers before anyone frees them


def time_device_resident(b: Bench, name: str, layer, x_dev, dy_dev, steps: int, warmup: int, sampler=None) -> dict:
    """W warm-up steps, then exactly K steps between CUDA events with a barrier + synchronize on both sides;
    the time is the maximum over the ranks. Per-op CUDA events on the launching stream give the kernel table."""
    from xma import _lib, ops

    w = WORKLOADS[name]
    step = make_step(layer)
    for _ in range(max(warmup, 3)):
        step(x_dev, dy_dev)
    b.barrier()
    _lib.raise_on_device_status(b.device)
    ops.STATS.enabled, ops.STATS.timing = True, True
    ops.STATS.reset()
    b.barrier()
    if sampler:
        sampler.mark_begin()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(steps):
        step(x_dev, dy_dev)
    t_end.record()
    b.barrier()
    if sampler:
        sampler.mark_end()
    ms_total = b.max_over_ranks(t_start.elapsed_time(t_end))
    launches = ops.STATS.launches
    kernel_ms = ops.STATS.elapsed_ms()
    ops.STATS.enabled = ops.STATS.timing = False
    _lib.raise_on_device_status(b.device)
    ms_per_step = ms_total / steps
    R = w["tokens"] * w["top_k"]  # routed rows through this rank's experts on average
    H, I = w["hidden"], w["inter"]
    gemm_flops = {  # algorithmic FLOPs per launch
        "gemm_up_swiglu": 2.0 * R * H * 2 * I, "gemm_down": 2.0 * R * I * H, "gemm_dact_dswiglu": 2.0 * R * H * I,
        "gemm_dx": 2.0 * R * 2 * I * H, "gemm_dw1": 2.0 * R * 2 * I * H, "gemm_dw2": 2.0 * R * H * I,
    }
    per_kernel = {}
    for tag, times in kernel_ms.items():
        per_kernel[tag] = {"launches": len(times), "ms_total": sum(times), "ms_avg": sum(times) / len(times)}
        if tag in gemm_flops:
            per_kernel[tag]["tflops"] = gemm_flops[tag] / (per_kernel[tag]["ms_avg"] * 1e-3) / 1e12
    gemm_ms = sum(v["ms_total"] for t, v in per_kernel.items() if t in gemm_flops)
    return {"ms_per_step": ms_per_step, "steps": steps, "launches": launches, "per_kernel": per_kernel,
            "gemm_flops": gemm_flops, "gemm_ms_per_step": gemm_ms / steps,
            "tokens_per_s": w["tokens"] * b.world / (ms_per_step * 1e-3),
            "step_tflops_per_gpu": expert_flops(w, w["tokens"]) / (ms_per_step * 1e-3) / 1e12}


def time_end_to_end(b: Bench, name: str, layer, x_dev, dy_dev, steps: int) -> dict:
    """The same step with its inputs copied from pinned host memory and its results copied back to pinned host
    memory inside the timed region. The copies run on their own streams so that the upload of step s+1 and the
    download of step s-1 overlap the kernels of step s (double-buffered device inputs). The copy streams carry
    their own CUDA events, which give the achieved host->device and device->host rates of this rank."""
    w = WORKLOADS[name]
    step = make_step(layer)
    x_pin, dy_pin = x_dev.cpu().pin_memory(), dy_dev.cpu().pin_memory()
    y_host = torch.empty_like(x_pin).pin_memory()
    dx_host = torch.empty_like(x_pin).pin_memory()
    main_stream = torch.cuda.current_stream()
    h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
    x_buf = [torch.empty_like(x_dev) for _ in range(2)]
    dy_buf = [torch.empty_like(dy_dev) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_events: list = []
    step_ticks: list = []

    def upload(s: int) -> None:
        k = s & 1
        h2d.wait_event(consumed[k])  # the step that last read this buffer pair has finished
        with torch.cuda.stream(h2d):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(h2d)
            x_buf[k].copy_(x_pin, non_blocking=True)
            dy_buf[k].copy_(dy_pin, non_blocking=True)
            e1.record(h2d)
            uploaded[k].record(h2d)
            copy_events.append(("h2d", e0, e1))

    def run(n: int) -> None:
        for ev in consumed:
            ev.record(main_stream)
        upload(0)
        for s in range(n):
            k = s & 1
            if s + 1 < n:
                upload(s + 1)
            main_stream.wait_event(uploaded[k])
            y, dx, _ = step(x_buf[k], dy_buf[k])
            consumed[k].record(main_stream)
            tick = torch.cuda.Event(enable_timing=True)
            tick.record(main_stream)
            step_ticks.append(tick)
            d2h.wait_event(consumed[k])
            with torch.cuda.stream(d2h):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(d2h)
                y_host.copy_(y, non_blocking=True)
                dx_host.copy_(dx, non_blocking=True)
                e1.record(d2h)
                copy_events.append(("d2h", e0, e1))
            y.record_stream(d2h)
            dx.record_stream(d2h)
        main_stream.wait_stream(d2h)

    run(4)  # the caching allocator settles (tensors held for the downloads change its working set)
    b.barrier()
    copy_events.clear()
    step_ticks.clear()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    run(steps)
    e_end.record()
    b.barrier()
    e2e_ms = b.max_over_ranks(e_start.elapsed_time(e_end)) / steps
    bytes_in = (x_pin.numel() + dy_pin.numel()) * x_pin.element_size()
    bytes_out = (y_host.numel() + dx_host.numel()) * y_host.element_size()
    rate = {}
    for kind, nbytes in (("h2d", bytes_in), ("d2h", bytes_out)):
        ms = [a.elapsed_time(c) for k, a, c in copy_events if k == kind]
        # slowest rank decides: report the minimum rate over the ranks
        gbs = nbytes / (statistics.median(ms) * 1e-3) / 1e9 if ms else 0.0
        rate[kind] = -b.max_over_ranks(-gbs)
    ends = [e_start.elapsed_time(t) for t in step_ticks]
    return {"value": w["tokens"] * b.world / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
            "step_end_ms_rank0": [round(t, 2) for t in ends],
            "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out,
            "h2d_gb_per_s_per_rank_min": rate["h2d"], "d2h_gb_per_s_per_rank_min": rate["d2h"],
            "copy_overlap": "upload of step s+1 and download of step s-1 run on their own streams under step s"}


def gather_expert_weights(b: Bench, layer, moe):
    """Every rank's expert weights and the router weight on rank 0's host (the parity check needs all experts)."""
    w1, w2 = moe.c_fc.weight.detach(), moe.c_proj.weight.detach()
    gate = (layer.gate_weight if b.world > 1 else moe.gate.weight).detach()
    if b.world > 1:
        full1 = torch.empty((b.world,) + tuple(w1.shape), dtype=w1.dtype, device=w1.device)
        full2 = torch.empty((b.world,) + tuple(w2.shape), dtype=w2.dtype, device=w2.device)
        b.dist.all_gather_into_tensor(full1, w1.contiguous())
        b.dist.all_gather_into_tensor(full2, w2.contiguous())
        w1, w2 = full1.flatten(0, 1), full2.flatten(0, 1)
    if b.rank != 0:
        return None
    return w1.cpu(), w2.cpu(), gate.cpu()


def parity_check(results, weights_cpu, x: torch.Tensor, dy: torch.Tensor, top_k: int, sample_tokens: int = 64,
                 tol: float = 2e-2) -> dict:
    """`results` = (y, x.grad, router_logits) of one forward + backward of the layer on (x, dy), checked against
    the CPU oracle (test infrastructure, never on the timed path):
      routing   : selected experts of EVERY token bit-equal to the oracle's top-k of the layer's own router
                  logits (ties: lowest expert index first), and the per-expert counts bit-equal to a bincount;
      y, x.grad : for a seeded sample of tokens, against the fp32 oracle run on those tokens with all expert
                  weights (a token's output and input gradient depend on its own row only); max |err| / max |ref|.
    `weights_cpu` = (c_fc [E, 2I, H], c_proj [E, H, I], gate [E, H]) on the host, all experts."""
    from oracle import moe_oracle as orc
    from xma.layers.moe import _TopKSoftmax

    w1, w2, gate = weights_cpu
    E = gate.size(0)
    y, dx, logits = results
    torch.cuda.synchronize()
    with torch.no_grad():
        _, selected = _TopKSoftmax.apply(logits.detach(), top_k)
    logits_cpu = logits.detach().cpu()
    _, ref_selected = orc.route(logits_cpu, top_k)
    routing_ok = bool(torch.equal(selected.cpu().long(), ref_selected))
    counts = torch.bincount(selected.flatten().long(), minlength=E).cpu().numpy()
    counts_ok = bool((counts == orc.continuous_count(ref_selected.numpy(), E)).all())

    T = x.size(0)
    gen = torch.Generator().manual_seed(4321)
    pick = torch.unique(torch.cat([torch.tensor([0, T - 1]), torch.randint(0, T, (sample_tokens,), generator=gen)]))
    f32 = lambda t: t.detach().float().cpu()
    ref = orc.moe_forward_backward(f32(x[pick.to(x.device)]), gate.float(), w1.float(), w2.float(), top_k, "swiglu",
                                   dy=f32(dy[pick.to(x.device)]), router_logits=logits_cpu[pick].float())
    dx_ref = ref.grads["x_experts"] + ref.grads["router_logits"] @ gate.float()

    def rel(got, want):
        return float((f32(got) - want).abs().max() / want.abs().max().clamp_min(1e-30))

    err_y, err_dx = rel(y[pick.to(x.device)], ref.y), rel(dx[pick.to(x.device)], dx_ref)
    return {"routing_bit_exact": routing_ok, "counts_bit_exact": counts_ok, "tokens_routed": T,
            "sample_tokens": int(pick.numel()), "y_max_rel_err": err_y, "dx_max_rel_err": err_dx, "tolerance": tol,
            "ok": routing_ok and counts_ok and err_y <= tol and err_dx <= tol}


def secondary_workload(b: Bench, name: str, steps: int) -> dict:
    """A shorter timed run of another layer shape in the same process, reported as an extra key of the line."""
    layer, moe, x_dev, dy_dev = build_workload(b, name)
    r = time_device_resident(b, name, layer, x_dev, dy_dev, steps, 3)
    w = WORKLOADS[name]
    peaks, _ = measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", PEAK_FALLBACK["bf16_tflops_sustained"]))
    gemm_tflops = sum(r["gemm_flops"].values()) / (r["gemm_ms_per_step"] * 1e-3) / 1e12 if r["gemm_ms_per_step"] else None
    out = {"workload": f"{name}: {w['desc']}", "n_gpus": b.world, "steps": steps, "warmup": 3,
           "ms_per_step": r["ms_per_step"], "tokens_per_s": r["tokens_per_s"],
           "step_tflops_per_gpu": r["step_tflops_per_gpu"], "step_frac_of_measured_sustained": r["step_tflops_per_gpu"] / peak,
           "grouped_gemms_tflops": gemm_tflops, "share_outside_gemms": 1.0 - r["gemm_ms_per_step"] / r["ms_per_step"],
           "efficiency_inputs": {"tokens_per_gpu": w["tokens"], "ms_per_step": r["ms_per_step"], "n_gpus": b.world},
           "kernels_ms_avg": {k: round(v["ms_avg"], 4) for k, v in r["per_kernel"].items()}}
    if b.world == 1:
        out["parity_check"] = parity_check(make_step(layer)(x_dev, dy_dev), gather_expert_weights(b, layer, moe),
                                           x_dev, dy_dev, w["top_k"], 32)
    release_layer(b, layer)
    del layer, moe, x_dev, dy_dev
    torch.cuda.empty_cache()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c5", "ep", "swiglu", "rmsnorm", "packing"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--ids-log2", type=int, default=26, help="workload c5: log2 of the number of ids (default 64 Mi)")
    ap.add_argument("--rmsnorm-rows", type=int, default=16 * 4096,
                    help="workload rmsnorm: rows of the [rows, 4096] activation (default 65536; a profiler capture "
                         "takes fewer)")
    ap.add_argument("--rmsnorm-dtypes", default="f32,f16,bf16", help="workload rmsnorm: which of f32,f16,bf16 to run")
    ap.add_argument("--ids-only", action="store_true",
                    help="workload c5: histogram and counting sort only, no row permute (small profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the secondary workloads (configs2 / configs3) and the parity check")
    ap.add_argument("--transport", choices=["peer", "nccl"], default="peer",
                    help="row exchange of the expert-parallel layer: stores into peer memory, or NCCL all-to-all")
    ap.add_argument("--ep-parts", type=int, default=None,
                    help="peer transport: expert groups of the pipelined exchange (default: the layer's choice)")
    ap.add_argument("--private-copies", action="store_true",
                    help="peer transport: copy the rows the backward needs out of the exchange buffers")
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
    if args.workload == "rmsnorm":
        return run_rmsnorm_microbench(args)
    if args.workload == "packing":
        return run_packing_microbench(args)
    if args.workload == "swiglu":
        run_swiglu_microbench(args)
        return
    w = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, w, args.workload)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 kernels are the only implementation (no CPU path)")

    b = Bench(args)
    rank, world = b.rank, b.world
    dtype = torch.float32 if w["dtype"] == "f32" else torch.bfloat16
    E = w["experts"]
    layer, moe, x_dev, dy_dev = build_workload(b, args.workload)

    # ---- device-resident timing --------------------------------------------------------------
    sampler = ClockSampler(b.gpu_index())
    sampler.start()  # nvidia-smi needs a moment to come up; samples are filtered to the timed region
    r = time_device_resident(b, args.workload, layer, x_dev, dy_dev, args.steps, args.warmup, sampler)
    clocks = sampler.stop()
    ms_per_step, per_kernel, gemm_flops = r["ms_per_step"], r["per_kernel"], r["gemm_flops"]

    # ---- end to end: pinned host inputs in, results out, every step ------------------------------
    e2e = time_end_to_end(b, args.workload, layer, x_dev, dy_dev, args.steps)

    # ---- roofline of the dominant kernel function ----------------------------------------------------
    peaks, peak_kind = measured_peaks()
    H, I = w["hidden"], w["inter"]
    peer = world > 1 and b.transport == "peer" and args.fused_return
    names = gemm_kernel_names(w, w["tokens"] * w["top_k"], E // world, peer, dtype)
    # tags launched by the same kernel function are one entry; the one with the largest share gets the roofline
    functions: dict = {}
    for tag, fn in names.items():
        if tag in per_kernel:
            functions.setdefault(fn, []).append(tag)
    traffic_rows, traffic_note = load_traffic_table()
    peak = float(peaks.get("bf16_tflops_sustained", PEAK_FALLBACK["bf16_tflops_sustained"]))
    sm_mhz = clocks.get("sm_mhz")
    groups = {}
    for fn, tags in functions.items():
        ms = sum(per_kernel[t]["ms_total"] for t in tags)
        n_launch = sum(per_kernel[t]["launches"] for t in tags)
        flops = sum(gemm_flops[t] * per_kernel[t]["launches"] for t in tags)
        groups[fn] = {"ms_total": ms, "launches": n_launch, "tflops": flops / (ms * 1e-3) / 1e12,
                      "share_of_step": ms / (ms_per_step * args.steps), "tags": tags}
    roofline = all_gemms = None
    if groups:
        fn = max(groups, key=lambda k: groups[k]["ms_total"])
        g = groups[fn]
        traffic = None
        if traffic_rows is None:
            traffic_source = traffic_note
        elif world != 1 or args.workload not in ("c2", "c2e2"):
            traffic_source = "the ncu table covers the one-GPU c2 / c2e2 shapes only"
        elif not all(t in traffic_rows for t in g["tags"]):
            traffic_source = "the ncu table has no row for this kernel"
        else:
            traffic = (E / 2.0) * sum(traffic_rows[t] for t in g["tags"]) / len(g["tags"])
            traffic_source = traffic_note
        roofline = {
            "bound": "tensor", "kernel": fn, "achieved": g["tflops"], "peak": peak, "unit": "TFLOP/s",
            "frac": g["tflops"] / peak, "peak_source": f"{peak_kind} cuBLAS bf16 sustained (kernel timed inside a long step)",
            "traffic": traffic, "traffic_source": traffic_source, "launches_per_step": g["launches"] // args.steps,
            "ms_per_launch": g["ms_total"] / g["launches"], "share_of_step": g["share_of_step"],
            "frac_of_nominal_2250": g["tflops"] / 2250.0,
            # time x clock compares boxes whose clocks under the power cap differ
            "ms_per_launch_x_sm_ghz": (g["ms_total"] / g["launches"]) * sm_mhz / 1e3 if sm_mhz else None,
        }
        gemm_ms = sum(g["ms_total"] for g in groups.values())
        achieved = sum(gemm_flops.values()) * args.steps / (gemm_ms * 1e-3) / 1e12
        all_gemms = {"tflops": achieved, "frac": achieved / peak, "frac_of_nominal_2250": achieved / 2250.0,
                     "share_of_step": gemm_ms / (ms_per_step * args.steps),
                     "by_kernel": {k: {"tflops": v["tflops"], "share_of_step": v["share_of_step"]}
                                   for k, v in groups.items()}}

    # ---- parity of the timed layer against the CPU oracle (outside every timed region) ------------------
    parity = None
    if not args.no_extra:
        results = make_step(layer)(x_dev, dy_dev)  # every rank: the expert-parallel step is collective
        weights = gather_expert_weights(b, layer, moe)
        if rank == 0:
            parity = parity_check(results, weights, x_dev, dy_dev, w["top_k"])
        del results, weights

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        sample = cpu_sample_tokens(w)
        v, sec, threads = cpu_step_tokens_per_s(w, sample, 1, 1)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{sample} of {w['tokens']} tokens, full expert shapes, {sec:.1f} s per step, "
                         "oracle/moe_oracle.py on the host cores"}

    parallelism = "single GPU" if world == 1 else (
        f"expert-parallel ep{world}, "
        + (("dispatch kernel + GEMM epilogues" if args.fused_return else "dispatch and return kernels")
           + " storing rows into peer memory over NVLink" if b.transport == "peer" else "NCCL all-to-all")
        + f", {layer.overlap_chunks} micro-batch(es) per step")
    release_layer(b, layer)
    del layer, moe, x_dev, dy_dev
    torch.cuda.empty_cache()

    # ---- the other layer shapes, shorter runs in the same process ---------------------------------------
    extra = {}
    if not args.no_extra and args.workload == "c2":
        few = max(3, min(args.steps, 5))
        if world == 1:
            extra["configs2"] = secondary_workload(b, "c3", few)
        extra["configs3"] = secondary_workload(b, "c4", few)

    if rank == 0:
        line = {
            "metric": METRIC, "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "tokens_per_gpu": w["tokens"],
                       "hidden": H, "intermediate": I, "experts": E, "top_k": w["top_k"], "parallelism": parallelism,
                       "l2_policy": "inputs_exceed_l2 (weights + activations >> 126 MB)"},
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": r["launches"],
            "roofline": roofline,
            "all_grouped_gemms": all_gemms,
            "step_tflops_per_gpu": r["step_tflops_per_gpu"],
            "step_ms_x_sm_ghz": ms_per_step * sm_mhz / 1e3 if sm_mhz else None,
            "kernels": per_kernel,
            "parity_check": parity,
            "cpu_baseline": cpu,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    if b.dist is not None:
        b.dist.destroy_process_group()


if __name__ == "__main__":
    main()
