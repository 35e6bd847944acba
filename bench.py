"""Benchmark of the per-layer MoE FFN block.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

A step is one pass of the block over one batch of synthetic tokens through one layer's weights
(for the stack workloads: one pass over all layers).  Layers rotate every step over `--layers`
resident layers so that weights come from HBM, not from L2.  `value` is tokens per second per
layer over all ranks with inputs resident on the device; `e2e` is the same through the host-buffer
entry point, copies included.

Which workload runs when none is named:
  * launched as one plain process: `decode64` (64 tokens, Zipf-skewed routing, one layer per step)
    is the line's `value`; the line's `also` object carries, measured in the same process, the
    one-token decode step, the 2048-token prefill chunk and the 40-layer 16384-token stack on this
    one GPU (the base of the expert-parallel curve);
  * launched by torch.distributed.run (WORLD_SIZE in the environment, any N including 1): the
    40-layer, 16384-token expert-parallel prefill stack, experts sharded over the N ranks, rows and
    results exchanged over peer memory (NVLink) -- strong scaling, the same global batch at every N.

The timed region is `--steps` steps, repeated back to back until it is at least 0.5 s long (the
line's `timed_repeats`); `ms_per_step` is the mean over all of them.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s/layer"
MIN_TIMED_SECONDS = 0.5
BF16_PEAK_TFLOPS_FALLBACK = 1590.0

E, K, H, I = 256, 8, 2048, 512

# name -> (tokens, bucket width, zipf skew).  Geometry 256 experts / top-8 / 2048 / 512.
WORKLOADS = {
    "decode1": (1, 16, False),      # one sequence, one token: the latency case
    "decode3": (3, 16, True),       # three concurrent sequences
    "decode64": (64, 16, True),     # 64 concurrent sequences (default)
    "decode16": (16, 16, True),     # widths in between, for choosing kernel thresholds
    "decode32": (32, 16, True),
    # the MoE half of Forward::body: --stack-layers layers chained (l_out -> next residual) in ONE graph
    "decode64_stack": (64, 16, True),
    # the LM head of the same model (hidden 2048 -> vocab 248,320, Q8_0, 540 MB): run_head() below
    "lm_head1": (1, 0, False),
    "lm_head8": (8, 0, False),
    "prefill2048": (2048, 32, True),  # one prefill chunk, bf16 rows in
    # the 40-layer prefill stack, experts sharded over the ranks (strong scaling): run_ep() below
    "ep_prefill_stack": (16384, 64, True),
    # the dense 27B block (hidden 5120 / intermediate 17408, Q6_K): run_dense() below; under torchrun
    # the intermediate dimension is sharded over the ranks (tensor parallel)
    "dense1": (1, 64, False),
    "dense64": (64, 64, False),
    "dense4096": (4096, 64, False),
}

# DRAM bytes (read + write) of the dominant kernel per launch from an ncu capture of the same workload
# (dram__bytes_read.sum + dram__bytes_write.sum); the line says where each figure came from
NCU_TRAFFIC = {
    "decode64": (332.9e6 + 5.9e6, "ncu capture of k_gateup_rows at decode64, one launch, constant recorded in bench.py"),
    "prefill2048": (468.3e6 + 18.1e6, "ncu capture of k_prefill_gemm<GATEUP> at prefill2048, one launch, constant recorded in bench.py"),
}

Q6K_MATRIX = (512 * 2048 // 256) * 210   # one [512][2048] or [2048][512] matrix, 860,160 B
Q8_0_MATRIX = (512 * 2048 // 32) * 34    # 1,114,112 B
ROUTER_BYTES = 256 * 2048 * 4
VEC_BYTES = 2 * 2048 * 4                 # post-norm weight + shared-gate vector


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, BF16_PEAK_TFLOPS_FALLBACK, "fallback (no MEASURED_PEAKS.json)"


def matrix_bytes(quant: str) -> int:
    return Q8_0_MATRIX if quant == "q8_0" else Q6K_MATRIX


def layer_algorithmic_bytes(distinct: float, tokens: int, args) -> float:
    """Weights of the experts actually routed + shared expert + router + vectors + x in, ffn_out, l_out."""
    routed = 2 * matrix_bytes(args.routed_quant) + matrix_bytes(args.routed_down_quant)
    shared = 3 * matrix_bytes(args.shared_quant)
    return distinct * routed + shared + ROUTER_BYTES + VEC_BYTES + tokens * 3 * 2048 * 4


def gateup_algorithmic_bytes(distinct: float, tokens: int, args) -> float:
    """What the gate/up launch must move: gate and up of the routed experts and of the shared one,
    the f16 activations in, the f16 intermediates out."""
    return (distinct * 2 * matrix_bytes(args.routed_quant) + 2 * matrix_bytes(args.shared_quant)
            + tokens * 2048 * 2 + tokens * 9 * 512 * 2)


def quant_label(args) -> str:
    r, d = args.routed_quant.upper(), args.routed_down_quant.upper()
    return f"{r} gate/up/down" if r == d else f"{r} gate/up, {d} down"


def moe_config(workload: str, args, world: int) -> dict:
    """The workload as both arms print it: static facts only, so the two lines' `config` are equal."""
    tokens, block_size, zipf = WORKLOADS[workload]
    return {"workload": workload, "tokens": tokens, "experts": E, "top_k": K, "hidden": H, "intermediate": I,
            "quant": quant_label(args), "shared_expert_quant": args.shared_quant.upper(), "bucket": block_size,
            "routing": "Zipf(1.1)-skewed" if zipf else "unskewed", "resident_layers": args.layers,
            "l2": "layers rotate every step; one layer's routed weights (660 MB) exceed the 126 MB L2",
            "parallelism": f"replicas x{world}"}


def ep_config(args, world: int) -> dict:
    return {"workload": "ep_prefill_stack", "tokens": args.ep_tokens, "layers": args.ep_layers, "experts": E,
            "top_k": K, "hidden": H, "intermediate": I, "quant": "Q6_K routed experts",
            "shared_expert_quant": "Q8_0", "bucket": 64, "routing": "Zipf(1.1)-skewed",
            "l2": "every layer has its own weights; a pass streams all of them (26.6 GB over all ranks)",
            "parallelism": f"ep{world} ({E // world} experts/rank), " +
                           ("peer-memory (NVLink) dispatch + combine, device-side counts and flags"
                            if args.ep_peer_memory else "NCCL all-to-all-v dispatch + combine")}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.mark = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def begin_region(self):
        """Samples from here on are the ones reported (the sampler itself starts before warm-up,
        since nvidia-smi needs a moment to deliver its first line)."""
        self.mark = len(self.rows)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = self.rows[self.mark:] or self.rows
        sm = [float(r[0]) for r in rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


class Timer:
    """CUDA-event timing of a region of steps on the current stream, barrier and synchronise on both
    sides, the maximum over ranks; regions shorter than MIN_TIMED_SECONDS are repeated back to back."""

    def __init__(self, torch, dist, world):
        self.torch, self.dist, self.world = torch, dist, world
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def _max(self, v: float) -> float:
        if self.world > 1:
            t = self.torch.tensor([v], device="cuda")
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            v = float(t.item())
        return v

    def region(self, fn, steps: int, repeats: int = 1) -> float:
        """Milliseconds per step over `repeats` x `steps` steps."""
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(repeats):
            for i in range(steps):
                fn(i)
        e1.record(self.stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (steps * repeats)
        self.barrier()
        return self._max(ms)

    def timed(self, fn, steps: int, min_seconds: float = MIN_TIMED_SECONDS):
        """(ms per step, repeats): first `steps` steps once; if that took under `min_seconds`, the
        reported figure comes from a second region of as many repeats as fill it."""
        ms = self.region(fn, steps)
        total = ms * steps * 1e-3
        if total >= min_seconds:
            return ms, 1
        repeats = max(2, int(math.ceil(min_seconds / max(total, 1e-6))))
        return self.region(fn, steps, repeats), repeats


def host_layer_from_device(w):
    """The oracle's view of a device layer (bytes copied back to the host)."""
    from oracle import xabe_oracle as oracle
    n = lambda t: t.detach().cpu().numpy()
    return oracle.Layer(num_experts=256, top_k=8, hidden=2048, inter=512, post_norm=n(w.post_norm),
                        router=n(w.router), router_bias=None if w.router_bias is None else n(w.router_bias),
                        gate_exps=n(w.gate_exps.bytes), gate_quant=int(w.gate_exps.quant),
                        up_exps=n(w.up_exps.bytes), up_quant=int(w.up_exps.quant),
                        down_exps=n(w.down_exps.bytes), down_quant=int(w.down_exps.quant),
                        shared_gate_inp=n(w.shared_gate_inp), shared_gate=n(w.shared_gate.bytes),
                        shared_gate_quant=int(w.shared_gate.quant), shared_up=n(w.shared_up.bytes),
                        shared_up_quant=int(w.shared_up.quant), shared_down=n(w.shared_down.bytes),
                        shared_down_quant=int(w.shared_down.quant))


def time_cpu_oracle(layer, x, steps: int, warmup: int, budget_s: float):
    """Times the CPU oracle (every host thread) on a bounded sample of the batch.  Returns
    (tokens/s, sample tokens, steps timed, threads, ms per step)."""
    from oracle import xabe_oracle as oracle
    threads = oracle.max_threads()
    sample = x.shape[0]
    t0 = time.perf_counter()
    oracle.moe_block_forward(layer, x[:sample], dev_order=False, threads=threads)
    once = time.perf_counter() - t0
    # shrink the per-step sample until warmup + steps fit the budget
    while sample > 1 and once * (steps + warmup) > budget_s:
        sample = max(1, sample // 2)
        t0 = time.perf_counter()
        oracle.moe_block_forward(layer, x[:sample], dev_order=False, threads=threads)
        once = time.perf_counter() - t0
    for _ in range(max(0, warmup - 1)):
        oracle.moe_block_forward(layer, x[:sample], dev_order=False, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.moe_block_forward(layer, x[:sample], dev_order=False, threads=threads)
    dt = time.perf_counter() - t0
    return sample * steps / dt, sample, steps, threads, dt / steps * 1e3


def _quant_code(name: str) -> int:
    return 1 if name == "q8_0" else 0


def run_reference(args, workload: str) -> dict:
    """`--impl reference`: the CPU oracle (the port of the reference's scalar path) on the host cores,
    every host thread, on a bounded sample of the same workload per step."""
    from llmxabe_b200 import synth
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import oracle_layer
    from oracle import xabe_oracle as oracle
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if workload.startswith("lm_head"):
        tokens = WORKLOADS[workload][0]
        # gemv over dequantised rows on a bounded sample of the vocabulary, scaled to all 248,320 rows
        rows, hidden, vocab = 16384, 2048, 248_320
        wb = synth.q8_0_bytes(rows * hidden, 0, 0, 3)
        x = synth.activations(tokens, hidden, seed=0, layer=901)
        threads = oracle.max_threads()
        for _ in range(max(args.warmup, 1)):
            oracle.lm_head(oracle.Q8_0, wb, rows, hidden, x, threads=threads)
        steps = max(1, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(steps):
            oracle.lm_head(oracle.Q8_0, wb, rows, hidden, x, threads=threads)
        per_pass = (time.perf_counter() - t0) / steps * (vocab / rows)
        tps = tokens / per_pass
        return {
            "impl": "reference", "metric": "lm_head_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": per_pass * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": head_config(workload),
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": f"{rows} of {vocab} vocabulary rows per step, scaled to the whole vocabulary"},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
    if workload == "ep_prefill_stack":
        # one layer of the stack (Q6_K experts, Q8_0 shared expert) on a sample of the 16384 tokens; the
        # metric is per layer, so tokens/s over one layer is the stack's figure
        L = synth.moe_layer(seed=0, layer=0, shared_quant=synth.Q8_0, zipf=True)
        config, scaling, tokens = ep_config(args, world), "strong", args.ep_tokens
    elif workload.startswith("dense"):
        tokens = WORKLOADS[workload][0]
        hidden, inter = 5120, 17408
        post_norm, gate, up, down = synth.dense_layer(seed=0, hidden=hidden, inter=inter, quant=0)
        sample = min(tokens, 16)
        x = synth.activations(sample, hidden, seed=0, layer=902)
        threads = oracle.max_threads()
        oracle.dense_block_forward(post_norm, 1e-6, gate, 0, up, 0, down, 0, hidden, inter, x, dev_order=False,
                                   threads=threads)
        steps = max(1, min(args.steps, 3))
        t0 = time.perf_counter()
        for _ in range(steps):
            oracle.dense_block_forward(post_norm, 1e-6, gate, 0, up, 0, down, 0, hidden, inter, x,
                                       dev_order=False, threads=threads)
        ms = (time.perf_counter() - t0) / steps * 1e3
        tps = sample / (ms * 1e-3)
        return {
            "impl": "reference", "metric": "dense_layer_tokens_per_s", "value": tps, "unit": UNIT,
            "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dense_config(workload, args, world),
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{sample} of {tokens} tokens per step, one layer, dequantisation included"},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
    else:
        tokens, _, zipf = WORKLOADS[workload]
        L = synth.moe_layer(seed=0, layer=0, zipf=zipf, routed_quant=_quant_code(args.routed_quant),
                            down_quant=_quant_code(args.routed_down_quant),
                            shared_quant=_quant_code(args.shared_quant))
        config, scaling = moe_config(workload, args, world), "weak"
    layer = oracle_layer(oracle, L)
    x = synth.activations(min(tokens, 256), 2048, seed=0, layer=900)
    tps, sample, steps, threads, ms = time_cpu_oracle(layer, x, max(1, min(args.steps, 20)), min(args.warmup, 2),
                                                      budget_s=120.0)
    return {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": ms, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} of {tokens} tokens per step, one layer, OpenMP over tokens/experts"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def measure_moe(args, workload: str, *, full: bool, sampler: ClockSampler | None = None) -> dict:
    """One single-layer MoE workload on this rank's GPU (replicas under torchrun).  `full` adds the
    eager timing, the repeat distribution and the calibration row (the main line); without it only
    the graph-replayed step, its stage profile and the host-buffer step are measured."""
    import torch
    import torch.distributed as dist

    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry, kernel_launch_count

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    tokens, block_size, zipf = WORKLOADS[workload]
    g = MoeGeometry.qwen3_6(block_size, tokens)
    block = MoeBlock(g)
    for key, value in args.tune:
        block.moe.set_tuning(key, value)
    layers = [synth.moe_layer_on_device(seed=rank, layer=i, zipf=zipf, routed_quant=_quant_code(args.routed_quant),
                                        down_quant=_quant_code(args.routed_down_quant),
                                        shared_quant=_quant_code(args.shared_quant)) for i in range(args.layers)]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4242 + rank)
    bf16_in = tokens >= 512   # a prefill chunk arrives as bf16 rows from the layers before it
    xs = [torch.randn(tokens, H, device="cuda", generator=gen) for _ in range(args.layers)]
    if bf16_in:
        xs = [x.to(torch.bfloat16) for x in xs]
    ffn = torch.empty(tokens, H, device="cuda")
    lout = torch.empty(tokens, H, device="cuda")
    hx = [x.float().cpu().pin_memory() for x in xs]
    hout = torch.empty(tokens, H).pin_memory()
    stream = torch.cuda.current_stream()
    tm = Timer(torch, dist, world)
    steps = args.steps

    def step(i):
        block.forward(layers[i % args.layers], xs[i % args.layers], tokens, ffn, lout)

    def step_host(i):
        block.forward_host(layers[i % args.layers], hx[i % args.layers], tokens, None, hout)
        stream.synchronize()  # the caller reads the result every step

    # warm-up: at least W steps and at least 0.3 s, so clocks are up (the reference warms by duration,
    # crates/xabe-engine/src/bin/bench_dense_ffn.rs:57-65)
    t0 = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t0 < 0.3:
        step(i)
        i += 1
    torch.cuda.synchronize()
    # distinct experts each resident layer's batch routes (the "unique" denominator of the byte count)
    distinct, busiest = [], 0
    for li in range(args.layers):
        step(li)
        torch.cuda.synchronize()
        ids = block.buffers().topk_ids[:tokens]
        distinct.append(int(torch.unique(ids).numel()))
        busiest = max(busiest, int(torch.bincount(ids.reshape(-1).long(), minlength=E).max().item()))
    d_mean = sum(distinct) / len(distinct)

    # Steps are replayed from a CUDA graph, as the reference's decode bodies are
    # (crates/xabe-engine/src/forward.rs:2059,3145): one graph holds one step per resident layer.
    graph, launches_per_step = None, None
    if args.graph:
        block.publish_tokens(tokens)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = kernel_launch_count()
        with torch.cuda.graph(graph):
            for i in range(args.layers):
                step(i)
        launches_per_step = (kernel_launch_count() - n0) / args.layers
        torch.cuda.synchronize()
    else:
        n0 = kernel_launch_count()
        step(0)
        launches_per_step = kernel_launch_count() - n0

    def replay(i):
        if i % args.layers == 0:
            graph.replay()

    steps_g = (steps + args.layers - 1) // args.layers * args.layers
    fn, n = (replay, steps_g) if graph is not None else (step, steps)
    for i in range(args.layers * 3):
        fn(i)
    if sampler is not None:
        sampler.begin_region()
    ms, repeats = tm.timed(fn, n)
    clocks = sampler.stop() if sampler is not None else None
    out = {"tokens": tokens, "ms": ms, "repeats": repeats, "steps_timed": n, "d_mean": d_mean, "busiest": busiest,
           "launches_per_step": launches_per_step, "clocks": clocks, "graph": graph is not None,
           "bf16_in": bf16_in}
    if full:
        out["ms_eager"], _ = tm.timed(step, steps, min_seconds=0.1)
        reps = sorted(tm.region(fn, n, repeats) for _ in range(5))
        out["reps"] = {"median": reps[len(reps) // 2], "min": reps[0], "max": reps[-1], "n": len(reps)}
        # calibration row: a pure streaming read of one resident layer's expert weights
        from llmxabe_b200.moe import stream_read
        sink = torch.zeros(1, dtype=torch.int32, device="cuda")
        cal_bytes = sum(int(t.bytes.numel()) for t in (layers[0].gate_exps, layers[0].up_exps, layers[0].down_exps))

        def cal_step(i):
            w = layers[i % args.layers]
            for t in (w.gate_exps.bytes, w.up_exps.bytes, w.down_exps.bytes):
                stream_read(t, sink)
        for i in range(3):
            cal_step(i)
        cal_ms, _ = tm.timed(cal_step, 20, min_seconds=0.1)
        out["calibration"] = {"what": "pure 128-bit streaming read of one layer's routed expert weights, no arithmetic",
                              "bytes": cal_bytes, "ms": cal_ms, "gbs": cal_bytes / (cal_ms * 1e-3) / 1e9}
    # the same step with per-stage CUDA events, for the dominant kernel's duration
    block.moe.stage_profile(True)
    tm.region(step, 8)
    block.moe.stage_times()   # the first calls after the graph replays run at eager-launch pace: not recorded
    tm.region(step, min(max(steps, 100), 256))
    stage_ms, calls = block.moe.stage_times()
    block.moe.stage_profile(False)
    out["stage_ms"] = {k: v / max(calls, 1) for k, v in stage_ms.items()}
    # The caller replays its host-buffer step from a CUDA graph too (one graph per resident layer:
    # pinned H2D copy, the block's launches, D2H copy) and reads the result after every step.
    for i in range(3):
        step_host(i)
    if args.graph:
        torch.cuda.synchronize()
        host_graphs = []
        for li in range(args.layers):
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph):
                block.forward_host(layers[li], hx[li], tokens, None, hout)
            host_graphs.append(gph)
        torch.cuda.synchronize()

        def step_host_graph(i):
            host_graphs[i % args.layers].replay()
            stream.synchronize()  # the caller reads the result every step
        for i in range(3):
            step_host_graph(i)
        out["ms_e2e"], _ = tm.timed(step_host_graph, steps, min_seconds=0.25)
    else:
        out["ms_e2e"], _ = tm.timed(step_host, steps, min_seconds=0.25)
    out["status"] = block.moe.device_status()
    out["layer0"], out["x0"] = layers[0], xs[0]
    return out


def moe_rooflines(args, workload: str, m: dict) -> dict:
    """The roofline objects of one measured MoE workload: `roofline` for its dominant kernel (the
    gate/up launch), `layer_roofline` for the whole step against HBM, and for prefill widths the
    step's tensor-pipe figure as well."""
    hbm, tflops, src = measured_peaks()
    tokens = m["tokens"]
    gateup_ms = m["stage_ms"]["gate_up"]
    gu_bytes = gateup_algorithmic_bytes(m["d_mean"], tokens, args)
    achieved = gu_bytes / (gateup_ms * 1e-3) / 1e9 if gateup_ms > 0 else 0.0
    layer_bytes = layer_algorithmic_bytes(m["d_mean"], tokens, args)
    traffic, traffic_src = NCU_TRAFFIC.get(workload, (None, None))
    if (args.shared_quant, args.routed_quant, args.routed_down_quant) != ("q6_k", "q6_k", "q6_k"):
        traffic, traffic_src = None, None
    kernel = ("k_prefill_gemm<GATEUP>" if tokens >= 512 else "k_gateup_rows" if tokens >= 16
              else "k_expert_stream<GATEUP>")
    out = {
        "roofline": {"bound": "hbm", "kernel": f"gate/up + SwiGLU launch ({kernel})", "achieved": achieved,
                     "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "traffic": traffic,
                     "traffic_source": traffic_src, "peak_source": src,
                     "algorithmic_bytes_per_launch": gu_bytes, "ms_per_launch": gateup_ms},
        "layer_roofline": {"bound": "hbm", "algorithmic_bytes": layer_bytes,
                           "achieved_gbs": layer_bytes / (m["ms"] * 1e-3) / 1e9,
                           "frac": layer_bytes / (m["ms"] * 1e-3) / 1e9 / hbm},
    }
    if tokens >= 512:
        # routed + shared GEMM flops only, the reference's accounting
        # (crates/xabe-engine/src/bin/bench_moe_mma.rs:236-244)
        flops = 2.0 * tokens * (K + 1) * 3 * H * I
        gu_flops = 2.0 * tokens * (K + 1) * 2 * H * I
        out["tensor_roofline"] = {
            "bound": "tensor", "flops_per_step": flops, "achieved": flops / (m["ms"] * 1e-3) / 1e12,
            "peak": tflops, "unit": "TFLOP/s", "frac": flops / (m["ms"] * 1e-3) / 1e12 / tflops,
            "gate_up_launch_frac": gu_flops / (gateup_ms * 1e-3) / 1e12 / tflops if gateup_ms > 0 else None,
            "peak_source": src + ", burst"}
    return out


def moe_entry(args, workload: str, m: dict) -> dict:
    """The short form of a workload for the main line's `also` object."""
    tokens = m["tokens"]
    e = {"config": moe_config(workload, args, 1), "value": tokens / (m["ms"] * 1e-3), "unit": UNIT,
         "ms_per_step": m["ms"], "timed_repeats": m["repeats"], "steps": m["steps_timed"],
         "e2e": {"value": tokens / (m["ms_e2e"] * 1e-3), "unit": UNIT, "ms_per_step": m["ms_e2e"],
                 "h2d_bytes_per_step": tokens * H * 4, "d2h_bytes_per_step": tokens * H * 4},
         "gpu_launches_per_step": m["launches_per_step"], "stage_ms": m["stage_ms"],
         "distinct_experts_mean": m["d_mean"], "busiest_expert_tokens": m["busiest"],
         "device_status": m["status"]}
    e.update(moe_rooflines(args, workload, m))
    return e


def run_ours(args, workload: str) -> dict:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sampler = ClockSampler(local_rank)
    sampler.start()   # before warm-up: nvidia-smi takes a moment to deliver its first sample
    m = measure_moe(args, workload, full=True, sampler=sampler)
    tokens, ms = m["tokens"], m["ms"]
    out = {
        "metric": METRIC, "value": world * tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "timed_repeats": m["repeats"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("f16 activations x Q6_K/Q8_0 weights dequantised to f16 (tcgen05), fp32 accumulate" if tokens >= 512
                  else "f16 activations x exact Q6_K/Q8_0 codes, fp32 scales+accumulate"),
        "data": "synthetic", "config": moe_config(workload, args, world),
        "workload_stats": {"distinct_experts_mean": m["d_mean"], "busiest_expert_tokens": m["busiest"],
                           "activations_in": "bf16" if m["bf16_in"] else "f32"},
        "e2e": {"value": world * tokens / (m["ms_e2e"] * 1e-3), "unit": UNIT, "ms_per_step": m["ms_e2e"],
                "h2d_bytes_per_step": tokens * H * 4, "d2h_bytes_per_step": tokens * H * 4},
        "gpu_launches": int(round(m["launches_per_step"] * m["steps_timed"] * m["repeats"])),
        "gpu_launches_per_step": m["launches_per_step"],
        "ms_per_step_eager": m["ms_eager"], "cuda_graph": m["graph"], "clocks": m["clocks"],
        "stage_ms": m["stage_ms"], "ms_per_step_repeats": m["reps"], "calibration": m["calibration"],
        "device_status": m["status"],
    }
    out.update(moe_rooflines(args, workload, m))
    if rank == 0 and world == 1 and not args.no_cpu:
        layer = host_layer_from_device(m["layer0"])
        x_host = m["x0"].float().cpu().numpy()
        tps, sample, steps, threads, cms = time_cpu_oracle(layer, x_host[:256], 3, 1, budget_s=30.0)
        out["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                               "sample": f"{sample} of {tokens} tokens x {steps} passes over layer 0 "
                                         f"({cms:.0f} ms per pass)"}
        # the same code on one thread (the reference's scalar path is single-threaded), a smaller sample
        from oracle import xabe_oracle as oracle
        n1 = min(4, tokens)
        oracle.moe_block_forward(layer, x_host[:n1], dev_order=False, threads=1)
        t0 = time.perf_counter()
        oracle.moe_block_forward(layer, x_host[:n1], dev_order=False, threads=1)
        out["cpu_baseline"]["single_thread"] = {"value": n1 / (time.perf_counter() - t0), "unit": UNIT,
                                                "sample": f"{n1} tokens, one pass, dequantisation included"}
    del m
    torch.cuda.empty_cache()
    if args.also and world == 1:
        also = {}
        for name in args.also_workloads:
            if name == workload:
                continue
            try:
                if name == "ep_prefill_stack":
                    e = run_ep(args, init_dist=False)
                    also[name] = {k: e[k] for k in ("config", "value", "unit", "ms_per_step", "steps", "scaling",
                                                    "roofline", "e2e", "phase_ms_per_layer_rank0", "device_status",
                                                    "gpu_launches_per_step")}
                else:
                    mm = measure_moe(args, name, full=False)
                    also[name] = moe_entry(args, name, mm)
                    del mm
            except Exception as exc:  # the main line stands even if a side measurement fails
                also[name] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.empty_cache()
        out["also"] = also
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_stack(args) -> dict:
    """`--stack-layers` MoE layers of the 64-token decode geometry driven as the reference's Forward::body drives
    them (crates/xabe-engine/src/forward.rs:3497-3618): one handle, each layer's l_out the next layer's
    residual, the whole pass one CUDA graph, the token count a device scalar.  A step = one pass over the
    stack; `value` stays per layer (tokens x layers / time) so it compares with the one-layer workloads."""
    import torch

    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeGeometry, kernel_launch_count
    from llmxabe_b200.stack import MoeStack

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("decode64_stack is a one-GPU workload")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(0)
    sampler = ClockSampler(0)
    sampler.start()
    tokens, block_size, zipf = WORKLOADS[args.workload]
    n_layers = args.stack_layers
    layers = [synth.moe_layer_on_device(seed=0, layer=i, zipf=zipf, routed_quant=_quant_code(args.routed_quant),
                                        down_quant=_quant_code(args.routed_down_quant),
                                        shared_quant=_quant_code(args.shared_quant)) for i in range(n_layers)]
    stack = MoeStack(MoeGeometry.qwen3_6(block_size, tokens), layers)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4242)
    x = torch.randn(tokens, H, device="cuda", generator=gen)
    hx = x.cpu().pin_memory()
    hout = torch.empty(tokens, H).pin_memory()
    stream = torch.cuda.current_stream()
    distinct = []
    stack.run(x, on_waypoint=lambda i, h: distinct.append(
        int(torch.unique(stack.block.buffers().topk_ids[:tokens]).numel())))
    torch.cuda.synchronize()
    d_mean = sum(distinct) / len(distinct)
    n0 = kernel_launch_count()
    stack.capture()
    launches_per_pass = (kernel_launch_count() - n0) // 2   # capture() runs the pass twice (warm-up + capture)

    def step(_i):
        stack.replay()

    def step_host(_i):  # the step's input from pinned host memory, its result back to the host
        stack.hidden_in[:tokens].copy_(hx, non_blocking=True)
        stack.replay()
        hout.copy_(stack.hidden_out[:tokens], non_blocking=True)
        stream.synchronize()

    tm = Timer(torch, None, 1)
    t0 = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t0 < 0.3:
        step(i)
        i += 1
    steps = max(3, min(args.steps, 50))
    sampler.begin_region()
    ms, repeats = tm.timed(step, steps)
    clocks = sampler.stop()
    for i in range(3):
        step_host(i)
    ms_e2e, _ = tm.timed(step_host, steps, min_seconds=0.25)
    status = stack.block.moe.device_status()
    hbm, _, peak_src = measured_peaks()
    layer_bytes = layer_algorithmic_bytes(d_mean, tokens, args)
    achieved = n_layers * layer_bytes / (ms * 1e-3) / 1e9
    cfg = moe_config("decode64_stack", args, 1)
    cfg.update({"layers": n_layers, "resident_layers": n_layers,
                "l2": f"every layer has its own weights ({n_layers * layer_bytes / 1e9:.1f} GB per pass, L2 126 MB)",
                "parallelism": "one GPU"})
    return {
        "metric": METRIC, "value": tokens * n_layers / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "timed_repeats": repeats, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 activations x exact Q6_K/Q8_0 codes, fp32 scales+accumulate", "data": "synthetic",
        "config": cfg,
        "workload_stats": {"distinct_experts_mean": d_mean, "stack_passes_per_s": 1e3 / ms,
                           "stack_tokens_per_s": tokens * 1e3 / ms},
        "e2e": {"value": tokens * n_layers / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": tokens * H * 4, "d2h_bytes_per_step": tokens * H * 4},
        "gpu_launches": launches_per_pass * steps * repeats, "gpu_launches_per_step": launches_per_pass,
        "cuda_graph": True, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "whole stack pass (all launches of all layers, one graph)",
                     "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "traffic": None,
                     "traffic_source": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": n_layers * layer_bytes, "ms_per_launch": ms},
        "device_status": status,
    }


def head_config(workload: str) -> dict:
    return {"workload": workload, "tokens": WORKLOADS[workload][0], "hidden": 2048, "vocab": 248_320,
            "quant": "Q8_0", "l2": "three resident copies of the head rotate; one copy is 540 MB (L2 126 MB)",
            "parallelism": "one GPU"}


def run_head(args) -> dict:
    """The LM head at the real geometry (crates/xabe-cuda/src/kernels/lm_head.rs:1318-1324): one pass over
    the 540 MB Q8_0 tensor serves up to eight tokens.  Three resident copies of the head rotate, and
    one copy alone is four times the L2.  A step = logits for the batch (+ argmax and the 4-byte
    read-back of each token id in the end-to-end figure, which is what a sampler reads)."""
    import torch

    from llmxabe_b200.lm_head import HeadFormat, HeadTensor, LmHeadGeometry, LmHeadKernels

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("the lm_head workloads are one-GPU workloads")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the LM head has no CPU fallback")
    torch.cuda.set_device(0)
    sampler = ClockSampler(0)
    sampler.start()
    tokens = WORKLOADS[args.workload][0]
    g = LmHeadGeometry.qwen3_6(tokens)
    head = LmHeadKernels(g)
    n_bytes = g.weight_bytes_for(HeadFormat.Q8_0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(777)
    copies = []
    for _ in range(3):
        raw = torch.randint(0, 256, (n_bytes,), dtype=torch.uint8, device="cuda", generator=gen).view(-1, 34)
        # the block scale: fp16(|N(0,1)| * 2e-4 * 4.6), as the synthetic Q8_0 tensors of the MoE workloads
        d = (torch.randn(raw.shape[0], device="cuda", generator=gen).abs() * (2e-4 * 4.6)).to(torch.float16)
        raw[:, 0:2] = d.view(torch.uint8).view(-1, 2)
        copies.append(HeadTensor(raw.view(-1), HeadFormat.Q8_0))
    x = torch.randn(tokens, g.hidden, device="cuda", generator=gen)
    logits = torch.empty(tokens, g.vocab, device="cuda")
    ids = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    hx = x.cpu().pin_memory()
    hids = torch.zeros(tokens, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream()

    def step(i):
        head.forward(copies[i % 3], x, tokens, logits)

    def step_host(i):
        x.copy_(hx, non_blocking=True)
        head.forward(copies[i % 3], x, tokens, logits)
        head.argmax(logits, tokens, ids)
        hids.copy_(ids, non_blocking=True)
        stream.synchronize()

    tm = Timer(torch, None, 1)
    t0 = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t0 < 0.3:
        step(i)
        i += 1
    sampler.begin_region()
    ms, repeats = tm.timed(step, args.steps)
    clocks = sampler.stop()
    for i in range(3):
        step_host(i)
    ms_e2e, _ = tm.timed(step_host, args.steps, min_seconds=0.25)
    status = head.device_status()
    hbm, _, peak_src = measured_peaks()
    alg_bytes = g.weight_bytes_read(tokens) + tokens * (g.hidden + g.vocab) * 4
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": "lm_head_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "timed_repeats": repeats,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "exact Q8_0 codes x fp32 activations as two f16 parts, fp32 scales+accumulate",
        "data": "synthetic", "config": head_config(args.workload),
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": tokens * g.hidden * 4, "d2h_bytes_per_step": tokens * 4},
        "gpu_launches": 2 * args.steps * repeats, "gpu_launches_per_step": 2, "cuda_graph": False, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "k_head_rows<Q8_0>", "achieved": achieved, "peak": hbm,
                     "unit": "GB/s", "frac": achieved / hbm, "traffic": None, "traffic_source": None,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": ms},
        "device_status": status,
    }
    if not args.no_cpu:
        from oracle import xabe_oracle as oracle
        rows = 16384  # a bounded sample of the vocabulary, every host thread
        wb = copies[0].bytes[: rows * 2176].cpu().numpy()
        xn = x.cpu().numpy()
        threads = oracle.max_threads()
        oracle.lm_head(oracle.Q8_0, wb, rows, g.hidden, xn, threads=threads)
        t0 = time.perf_counter()
        reps = 0
        while reps < 3 or time.perf_counter() - t0 < 5.0:
            oracle.lm_head(oracle.Q8_0, wb, rows, g.hidden, xn, threads=threads)
            reps += 1
        per_pass = (time.perf_counter() - t0) / reps * (g.vocab / rows)
        out["cpu_baseline"] = {"value": tokens / per_pass, "unit": "tokens/s", "cores": threads, "kind": "port",
                               "sample": f"{rows} of {g.vocab} vocabulary rows x {tokens} tokens, {reps} passes, "
                                         f"scaled to the whole vocabulary ({per_pass * 1e3:.0f} ms per pass)"}
    return out


def run_ep(args, init_dist: bool = True) -> dict:
    """The 40-layer prefill stack (Q6_K experts, Q8_0 shared expert), `--ep-tokens` tokens, experts
    sharded over the ranks, rows and results exchanged over peer memory (or NCCL all-to-alls with
    --ep-nccl).  Strong scaling: the global batch is fixed, each rank owns tokens/N tokens and 256/N
    experts of every layer.  A step = one pass over all layers."""
    import torch
    import torch.distributed as dist

    from llmxabe_b200 import synth
    from llmxabe_b200.ep import CudaEpBackend, EpMoeBlock
    from llmxabe_b200.moe import MoeGeometry, QuantTensor, kernel_launch_count

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1 and init_dist:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sampler = ClockSampler(local_rank)
    sampler.start()
    tokens, n_layers = args.ep_tokens, args.ep_layers
    per, epr = tokens // world, E // world
    g = MoeGeometry(E, K, H, I, 64, per)
    max_rows = tokens * K if world == 1 else min(tokens * K, int(tokens * K / world * 3) + 1024)
    layers = []
    for li in range(n_layers):
        # replicated tensors share one seed on every rank; the expert stacks are this rank's own
        front = synth.moe_layer_on_device(seed=7, layer=li, num_experts=1, top_k=1, routed_quant=synth.Q6K,
                                          shared_quant=synth.Q8_0, zipf=False)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(7000 + li)
        front.router = torch.randn(E, H, device="cuda", generator=gen) * 0.02
        front.router_bias = torch.from_numpy(synth.zipf_bias(E, 7, li)).cuda()
        gen.manual_seed(900000 + li * 64 + rank)
        n = epr * I * H
        local = [QuantTensor(synth._device_quant_bytes(torch, synth.Q6K, n, gen, "cuda"), front.gate_exps.quant)
                 for _ in range(3)]
        layers.append((front, local))
    if args.ep_peer_memory:
        from llmxabe_b200.ep import PeerMemoryEpBackend
        backend = PeerMemoryEpBackend(g, epr, rank, world, layers[0][0], *layers[0][1],
                                      fused_return=not args.ep_separate_return)
    else:
        backend = CudaEpBackend(g, epr, max_rows, layers[0][0], *layers[0][1])
    for key, value in args.tune:
        backend.front_k.set_tuning(key, value)
        backend.back_k.set_tuning(key, value)
    blk = EpMoeBlock(backend, E, K, rank, world, overlap_shared=args.ep_overlap)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(31 + rank)
    x0 = torch.randn(per, H, device="cuda", generator=gen)
    hx = x0.cpu().pin_memory()
    hout = torch.empty(per, H).pin_memory()
    bufs = [torch.empty(per, H, device="cuda") for _ in range(2)]
    ffn = torch.empty(per, H, device="cuda")
    stream = torch.cuda.current_stream()
    xin = torch.empty_like(x0)

    def step(_i, src=x0):
        h = src
        for li, (front, local) in enumerate(layers):
            backend.set_layer(front, *local)
            out = bufs[li & 1]
            blk.forward(h, per, ffn, out)
            h = out
        return h

    def step_host(i):   # this rank's rows from pinned host memory, its final hidden state back
        xin.copy_(hx, non_blocking=True)
        h = step(i, xin)
        hout.copy_(h, non_blocking=True)
        stream.synchronize()

    tm = Timer(torch, dist, world)
    for i in range(max(min(args.warmup, 3), 1)):
        step(i)
    n0 = kernel_launch_count()
    step(0)
    launches_per_step = kernel_launch_count() - n0
    steps = max(1, min(args.steps, 10))
    sampler.begin_region()
    ms, repeats = tm.timed(step, steps)
    clocks = sampler.stop()
    step_host(0)
    ms_e2e, _ = tm.timed(step_host, max(1, min(steps, 3)), min_seconds=0.0)
    rows = sum(blk.last_plan.recv_counts) if blk.last_plan is not None else 0  # not known on the host with peer memory
    # one more, untimed, pass with per-phase events (per layer, this rank)
    blk.enable_phase_timing()
    step(0)
    phases = {k: v / n_layers for k, v in blk.phase_times_ms().items()}
    blk._events = None
    if world > 1:
        t = torch.tensor([float(rows)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rows = int(t[0].item())
    status = backend.front_k.device_status() | backend.back_k.device_status()
    _, tflops, peak_src = measured_peaks()
    flops = 2.0 * tokens * (K + 1) * 3 * H * I * n_layers
    out = {
        "metric": METRIC, "value": tokens * n_layers / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": steps, "warmup": max(min(args.warmup, 3), 1), "ms_per_step": ms, "timed_repeats": repeats,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 x f16 -> f32 (tcgen05), weights dequantised to f16", "data": "synthetic",
        "config": ep_config(args, world),
        "workload_stats": {"max_rows_received_by_a_rank_last_layer": rows},
        "e2e": {"value": tokens * n_layers / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": per * H * 4, "d2h_bytes_per_step": per * H * 4},
        "clocks": clocks, "device_status": status, "phase_ms_per_layer_rank0": phases,
        "roofline": {"bound": "tensor", "kernel": "whole stack pass per GPU (routed + shared GEMM flops only)",
                     "achieved": flops / (ms * 1e-3) / 1e12 / world, "unit": "TFLOP/s", "peak": tflops,
                     "frac": flops / (ms * 1e-3) / 1e12 / world / tflops, "traffic": None, "traffic_source": None,
                     "peak_source": peak_src + ", burst"},
        "gpu_launches": launches_per_step * steps * repeats, "gpu_launches_per_step": launches_per_step,
        "cuda_graph": False,
    }
    if args.ep_peer_memory:
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        for b in backend._shared.values():
            b.release()
    if world > 1 and init_dist:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else {}


def dense_config(workload: str, args, world: int) -> dict:
    return {"workload": workload, "tokens": WORKLOADS[workload][0], "hidden": 5120, "intermediate": 17408,
            "quant": "Q6_K", "resident_layers": max(args.layers, 2),
            "parallelism": f"tp{world} (intermediate split in whole 256-element units), NCCL all-reduce",
            "l2": "layers rotate every step; one layer is 219 MB (> 126 MB L2)"}


def run_dense(args) -> dict:
    """The dense SwiGLU block of the 27B sibling, Q6_K.  One rank: DenseFfnBlock.
    Several ranks: the intermediate dimension sharded (llmxabe_b200.tp), one all-reduce per layer;
    strong scaling (the token batch is the same on every rank)."""
    import torch
    import torch.distributed as dist

    from llmxabe_b200 import synth
    from llmxabe_b200.moe import QuantTensor, kernel_launch_count
    from llmxabe_b200.tp import CudaTpBackend, TpDenseFfnBlock

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sampler = ClockSampler(local_rank)
    sampler.start()
    HD, ID = 5120, 17408
    tokens = WORKLOADS[args.workload][0]
    n_layers = max(args.layers, 2)
    blocks = []
    for li in range(n_layers):
        gen = torch.Generator(device="cuda")
        gen.manual_seed(4000 + li)           # every rank generates the full matrices and keeps its shard
        full = [QuantTensor(synth._device_quant_bytes(torch, synth.Q6K, HD * ID, gen, "cuda"), synth.Q6K)
                for _ in range(3)]
        backend = CudaTpBackend(HD, ID, tokens, rank, world, torch.ones(HD, device="cuda"), *full)
        if world > 1:
            backend.gate = QuantTensor(backend.gate.bytes.clone(), synth.Q6K)
            backend.up = QuantTensor(backend.up.bytes.clone(), synth.Q6K)
        else:
            backend.down = full[2]
        del full
        for key, value in args.tune:
            backend.k.set_tuning(key, value)
        blocks.append(TpDenseFfnBlock(backend, rank, world))
    torch.cuda.empty_cache()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    x0 = torch.randn(tokens, HD, device="cuda", generator=gen)
    bufs = [torch.empty(tokens, HD, device="cuda") for _ in range(2)]
    ffn = torch.empty(tokens, HD, device="cuda")
    stream = torch.cuda.current_stream()

    def step(i):
        blocks[i % n_layers].forward(x0, tokens, ffn, bufs[i & 1])

    tm = Timer(torch, dist, world)
    for i in range(max(args.warmup, 3)):
        step(i)
    n0 = kernel_launch_count()
    step(0)
    launches_per_step = kernel_launch_count() - n0
    # Decode widths on one GPU: the steps are replayed from a CUDA graph (one step per resident layer), as
    # the MoE decode steps are and as the reference's decode bodies are (crates/xabe-engine/src/forward.rs:2059)
    graph = None
    if args.graph and world == 1 and tokens <= 64:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n_layers):
                step(i)
        torch.cuda.synchronize()

    def replay(i):
        if i % n_layers == 0:
            graph.replay()

    steps_g = (args.steps + n_layers - 1) // n_layers * n_layers
    fn, n_timed = (replay, steps_g) if graph is not None else (step, args.steps)
    for i in range(n_layers * 3):
        fn(i)
    sampler.begin_region()
    ms, repeats = tm.timed(fn, n_timed)
    clocks = sampler.stop()
    status = 0
    for b in blocks:
        status |= b.backend.k.device_status()
    # end to end: host rows in, host rows out
    hx = torch.randn(tokens, HD).pin_memory()
    hout = torch.empty(tokens, HD).pin_memory()
    dx = torch.empty(tokens, HD, device="cuda")

    def step_host(i):
        dx.copy_(hx, non_blocking=True)
        blocks[i % n_layers].forward(dx, tokens, ffn, bufs[0])
        hout.copy_(bufs[0], non_blocking=True)
        stream.synchronize()
    step_host(0)
    e2e_ms, _ = tm.timed(step_host, max(3, min(args.steps, 20)), min_seconds=0.25)
    hbm, tflops, peak_src = measured_peaks()
    weight_bytes = 3 * (HD * ID // 256) * 210
    alg_bytes = weight_bytes // world + tokens * HD * 4 * 3
    flops = 2.0 * tokens * 3 * HD * ID
    hbm_bound = tokens <= 256
    roof = ({"bound": "hbm", "kernel": "whole layer per rank (norm, gate/up, down, residual)",
             "achieved": alg_bytes / (ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
             "frac": alg_bytes / (ms * 1e-3) / 1e9 / hbm, "traffic": None, "traffic_source": None,
             "peak_source": peak_src, "algorithmic_bytes_per_launch": alg_bytes}
            if hbm_bound else
            {"bound": "tensor", "kernel": "whole layer per rank", "achieved": flops / world / (ms * 1e-3) / 1e12,
             "peak": tflops, "unit": "TFLOP/s", "frac": flops / world / (ms * 1e-3) / 1e12 / tflops, "traffic": None,
             "traffic_source": None, "peak_source": peak_src + ", burst"})
    out = {
        "metric": "dense_layer_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "timed_repeats": repeats,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 activations x Q6_K weights (exact codes at decode widths, f16 weights on tcgen05 at prefill widths), fp32 accumulate",
        "data": "synthetic", "config": dense_config(args.workload, args, world),
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": tokens * HD * 4, "d2h_bytes_per_step": tokens * HD * 4},
        "gpu_launches": launches_per_step * n_timed * repeats, "gpu_launches_per_step": launches_per_step,
        "cuda_graph": graph is not None, "steps_timed": n_timed, "clocks": clocks, "roofline": roof,
        "device_status": status,
    }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="default: decode64 as one plain process, ep_prefill_stack under torch.distributed.run")
    ap.add_argument("--layers", type=int, default=4, help="distinct resident layers the steps rotate over")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--no-also", dest="also", action="store_false",
                    help="skip the side measurements the default line carries in `also`")
    ap.add_argument("--also-workloads", default="decode1,prefill2048,ep_prefill_stack",
                    type=lambda s: [w for w in s.split(",") if w])
    ap.add_argument("--shared-quant", default="q6_k", choices=["q6_k", "q8_0"],
                    help="format of the shared expert in the MoE workloads (the shipped file's is Q8_0)")
    ap.add_argument("--routed-quant", default="q6_k", choices=["q6_k", "q8_0"],
                    help="format of the routed gate/up stacks (Q8_0 in the shipped file's last block)")
    ap.add_argument("--routed-down-quant", default=None, choices=["q6_k", "q8_0"],
                    help="format of the routed down stack (the shipped file's is Q8_0); default: as --routed-quant")
    ap.add_argument("--stack-layers", type=int, default=40, help="layers of the decode64_stack workload")
    ap.add_argument("--ep-tokens", type=int, default=16384)
    ap.add_argument("--ep-layers", type=int, default=40)
    ap.add_argument("--ep-separate-return", action="store_true",
                    help="peer-memory exchange with the result rows pushed by a kernel of their own after the "
                         "down projection instead of by its epilogue (for comparison)")
    ap.add_argument("--ep-nccl", dest="ep_peer_memory", action="store_false",
                    help="exchange rows and results with NCCL all-to-alls instead of peer stores over NVLink")
    ap.add_argument("--ep-no-overlap", dest="ep_overlap", action="store_false",
                    help="run the shared expert on the main stream instead of beside the exchange")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time eager launches instead of CUDA-graph replay")
    ap.add_argument("--tune", default=[], type=lambda s: [(kv.split("=")[0], int(kv.split("=")[1])) for kv in s.split(",") if kv],
                    help="per-handle launch-shape switches of the single-layer MoE workloads, e.g. fused_decode=0,pdl=1")
    args = ap.parse_args()
    if args.routed_down_quant is None:
        args.routed_down_quant = args.routed_quant
    under_torchrun = "WORLD_SIZE" in os.environ and "RANK" in os.environ
    default_workload = args.workload is None
    workload = args.workload or ("ep_prefill_stack" if under_torchrun else "decode64")
    args.workload = workload
    if not default_workload:
        args.also = False
    # Libraries write to stdout too (NCCL prints its version line there when NCCL_DEBUG asks for it):
    # while the workload runs, file descriptor 1 points at stderr, and it is put back for the one JSON line.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(obj), flush=True)

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        emit(run_reference(args, workload))
        return
    if workload == "ep_prefill_stack":
        out = run_ep(args)
    elif workload.startswith("dense"):
        out = run_dense(args)
    elif workload == "decode64_stack":
        out = run_stack(args)
    elif workload.startswith("lm_head"):
        out = run_head(args)
    else:
        out = run_ours(args, workload)
    if out:
        emit(out)


if __name__ == "__main__":
    main()
