"""Benchmark of the per-layer MoE FFN block.

    python bench.py --gpus N --steps K --warmup W [--workload decode64] [--impl reference]

A step is one pass of the block over one batch of synthetic tokens through one
layer's weights.  Layers rotate every step over `--layers` resident layers so
that weights come from HBM, not from L2.  `value` is tokens per second per
layer over all ranks (inputs resident); `e2e` is the same through the
host-buffer entry point, copies included.  At N > 1 every rank is a replica
with its own layers and its own batch (weak scaling, no data-path collective),
the reference's own multi-GPU model.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s/layer"

# name -> (tokens, bucket width, zipf skew).  Geometry 256 experts / top-8 / 2048 / 512, Q6_K everywhere.
WORKLOADS = {
    "decode1": (1, 16, False),      # BASELINE config 0
    "decode3": (3, 16, True),       # BASELINE config 1, three sequences
    "decode64": (64, 16, True),     # BASELINE config 1, 64 tokens  (default)
    "decode16": (16, 16, True),     # widths between the configs, for choosing kernel thresholds
    "decode32": (32, 16, True),
    # the MoE half of Forward::body: --stack-layers layers chained (l_out -> next residual) in ONE graph
    "decode64_stack": (64, 16, True),
    # the LM head of the same model (hidden 2048 -> vocab 248,320, Q8_0, 540 MB): run_head() below
    "lm_head1": (1, 0, False),
    "lm_head8": (8, 0, False),
    "prefill2048": (2048, 32, True),  # BASELINE config 2
    # BASELINE config 3 (expert-parallel stack, strong scaling): run_ep() below; tokens/layers from --ep-*
    "ep_prefill_stack": (16384, 64, True),
    # BASELINE config 4 (dense 27B block, hidden 5120 / intermediate 17408, Q6_K): run_dense() below;
    # under torchrun the intermediate dimension is sharded over the ranks (tensor parallel)
    "dense1": (1, 64, False),
    "dense64": (64, 64, False),
    "dense4096": (4096, 64, False),
}

# DRAM bytes (read + write) of the dominant kernel per launch, from the ncu captures summarised under
# profiles/ (k_gateup_rows_decode64.md, k_prefill_gemm_prefill2048.md); none taken for the others
NCU_TRAFFIC_BYTES = {"decode64": 329.3e6 + 4.3e6, "prefill2048": 467.0e6 + 16.5e6}

Q6K_EXPERT_BYTES = 3 * (512 * 2048 // 256) * 210   # 2,580,480
ROUTER_BYTES = 256 * 2048 * 4
VEC_BYTES = 2 * 2048 * 4                           # post-norm weight + shared-gate vector


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (no MEASURED_PEAKS.json)"


Q8_0_EXPERT_BYTES = 3 * (512 * 2048 // 32) * 34    # 3,342,336


def layer_algorithmic_bytes(distinct: int, tokens: int, shared_q8: bool = False) -> int:
    """Weights of the experts actually routed + shared expert + router + vectors + x in, ffn_out, l_out."""
    shared = Q8_0_EXPERT_BYTES if shared_q8 else Q6K_EXPERT_BYTES
    return distinct * Q6K_EXPERT_BYTES + shared + ROUTER_BYTES + VEC_BYTES + tokens * 3 * 2048 * 4


def gateup_algorithmic_bytes(distinct: int, tokens: int, shared_q8: bool = False) -> int:
    """What the gate/up launch must move: gate and up of the routed experts and of the shared one,
    the f16 activations in, the f16 intermediates out."""
    per = 2 * (512 * 2048 // 256) * 210
    shared = 2 * (512 * 2048 // 32) * 34 if shared_q8 else per
    return distinct * per + shared + tokens * 2048 * 2 + tokens * 9 * 512 * 2


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

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

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


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
    (tokens/s, sample tokens, steps timed, threads)."""
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


def run_reference(args) -> dict:
    """`--impl reference`: the CPU oracle (the port of the reference's scalar path) on the host cores."""
    tokens, block_size, zipf = WORKLOADS[args.workload]
    from llmxabe_b200 import synth
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import oracle_layer
    from oracle import xabe_oracle as oracle
    if args.workload.startswith("lm_head"):
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
            "config": {"workload": args.workload, "tokens": tokens, "hidden": hidden, "vocab": vocab, "quant": "Q8_0"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": f"{rows} of {vocab} vocabulary rows per step, scaled to the whole vocabulary"},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
    L = synth.moe_layer(seed=0, layer=0, zipf=zipf)
    layer = oracle_layer(oracle, L)
    x = synth.activations(tokens, 2048, seed=0, layer=900)
    tps, sample, steps, threads, ms = time_cpu_oracle(layer, x, args.steps, args.warmup, budget_s=150.0)
    return {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "experts": 256, "top_k": 8, "hidden": 2048,
                   "intermediate": 512, "quant": "Q6_K"},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} of {tokens} tokens per step, one layer, OpenMP over tokens/experts"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeBlock, MoeGeometry

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    tokens, block_size, zipf = WORKLOADS[args.workload]
    H = 2048
    g = MoeGeometry.qwen3_6(block_size, tokens)
    block = MoeBlock(g)
    shared_q = synth.Q8_0 if args.shared_quant == "q8_0" else synth.Q6K
    layers = [synth.moe_layer_on_device(seed=rank, layer=i, zipf=zipf, shared_quant=shared_q) for i in range(args.layers)]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4242 + rank)
    xs = [torch.randn(tokens, H, device="cuda", generator=gen) for _ in range(args.layers)]
    ffn = torch.empty(tokens, H, device="cuda")
    lout = torch.empty(tokens, H, device="cuda")
    hx = [x.cpu().pin_memory() for x in xs]
    hout = torch.empty(tokens, H).pin_memory()
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(i):
        block.forward(layers[i % args.layers], xs[i % args.layers], tokens, ffn, lout)

    def step_host(i):
        block.forward_host(layers[i % args.layers], hx[i % args.layers], tokens, None, hout)
        stream.synchronize()  # the caller reads the result every step

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        barrier()
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # warm-up: at least W steps and at least 0.3 s, so clocks are up (the reference warms by duration,
    # crates/xabe-engine/src/bin/bench_dense_ffn.rs:57-65)
    t0 = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t0 < 0.3:
        step(i)
        i += 1
    torch.cuda.synchronize()
    # distinct experts each resident layer's batch routes (the "unique" denominator of the byte count)
    distinct = []
    for li in range(args.layers):
        step(li)
        torch.cuda.synchronize()
        distinct.append(int(torch.unique(block.buffers().topk_ids[:tokens]).numel()))
    d_mean = sum(distinct) / len(distinct)

    # Decode steps are replayed from a CUDA graph, as the reference's decode bodies are
    # (crates/xabe-engine/src/forward.rs:2059,3145): one graph holds one step per resident layer.
    graph = None
    if args.graph:
        block.publish_tokens(tokens)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(args.layers):
                step(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.layers):
                step(i)
        torch.cuda.synchronize()

    def replay(i):
        if i % args.layers == 0:
            graph.replay()

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_eager = timed(step, args.steps)
    if graph is not None:
        steps_g = (args.steps + args.layers - 1) // args.layers * args.layers
        for i in range(args.layers * 3):
            replay(i)
        ms = timed(replay, steps_g)
    else:
        ms = ms_eager
    clocks = sampler.stop()
    # distribution over repeats of the timed region (median and best), same method
    reps = []
    for _ in range(5):
        reps.append(timed(replay, steps_g) if graph is not None else timed(step, args.steps))
    reps.sort()
    # calibration row: a pure streaming read of one resident layer's expert weights
    from llmxabe_b200.moe import stream_read
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    w0 = layers[0]
    cal_tensors = [w0.gate_exps.bytes, w0.up_exps.bytes, w0.down_exps.bytes]
    cal_bytes = sum(int(t.numel()) for t in cal_tensors)

    def cal_step(i):
        w = layers[i % args.layers]
        for t in (w.gate_exps.bytes, w.up_exps.bytes, w.down_exps.bytes):
            stream_read(t, sink)
    for i in range(3):
        cal_step(i)
    cal_ms = timed(cal_step, max(8, min(args.steps, 40)))
    # the same region again with per-stage CUDA events, for the dominant kernel's duration
    block.moe.stage_profile(True)
    timed(step, min(args.steps, 256))
    stage_ms, calls = block.moe.stage_times()
    block.moe.stage_profile(False)
    for i in range(3):
        step_host(i)
    # The caller replays its host-buffer step from a CUDA graph too (one graph per resident layer:
    # pinned H2D copy, the block's launches, D2H copy) and reads the result after every step.
    host_graphs = None
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
        ms_e2e = timed(step_host_graph, args.steps)
    else:
        ms_e2e = timed(step_host, args.steps)
    status = block.moe.device_status()

    launches_per_step = 7 if tokens * 8 <= 2048 and tokens > 8 else (6 if tokens <= 8 else 11)
    peak, peak_src = measured_peaks()
    gateup_ms = stage_ms["gate_up"] / max(calls, 1)
    gu_bytes = gateup_algorithmic_bytes(d_mean, tokens, args.shared_quant == "q8_0")
    achieved = gu_bytes / (gateup_ms * 1e-3) / 1e9 if gateup_ms > 0 else 0.0
    layer_bytes = layer_algorithmic_bytes(d_mean, tokens, args.shared_quant == "q8_0")
    out = {
        "metric": METRIC, "value": world * tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations x exact Q6_K codes, fp32 scales+accumulate",
        "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_rank": tokens, "experts": 256, "top_k": 8,
                   "hidden": 2048, "intermediate": 512, "quant": "Q6_K", "shared_expert_quant": args.shared_quant,
                   "bucket": block_size,
                   "resident_layers": args.layers, "distinct_experts_mean": d_mean,
                   "l2": f"layers rotate every step; each touches {layer_bytes / 1e6:.0f} MB of weights "
                         f"(> 126 MB L2) out of {args.layers} resident layers",
                   "parallelism": f"replicas x{world}"},
        "e2e": {"value": world * tokens / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": tokens * H * 4, "d2h_bytes_per_step": tokens * H * 4},
        "gpu_launches": launches_per_step * args.steps, "ms_per_step_eager": ms_eager, "cuda_graph": graph is not None,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "gate/up + SwiGLU launch (k_expert_stream<GATEUP> below 16 tokens, k_gateup_rows from 16, k_prefill_gemm<GATEUP> from 512)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                     "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": gu_bytes, "ms_per_launch": gateup_ms},
        "layer_roofline": {"algorithmic_bytes": layer_bytes, "achieved_gbs": layer_bytes / (ms * 1e-3) / 1e9,
                           "frac": layer_bytes / (ms * 1e-3) / 1e9 / peak},
        "stage_ms": {k: v / max(calls, 1) for k, v in stage_ms.items()},
        "ms_per_step_repeats": {"median": reps[len(reps) // 2], "min": reps[0], "max": reps[-1], "n": len(reps)},
        "calibration": {"what": "pure 128-bit streaming read of one layer's routed expert weights, no arithmetic",
                        "bytes": cal_bytes, "ms": cal_ms, "gbs": cal_bytes / (cal_ms * 1e-3) / 1e9},
        "device_status": status,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        layer = host_layer_from_device(layers[0])
        tps, sample, steps, threads, cms = time_cpu_oracle(layer, xs[0].cpu().numpy(), 3, 1, budget_s=30.0)
        out["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                               "sample": f"{sample} of {tokens} tokens x {steps} passes over layer 0 "
                                         f"({cms:.0f} ms per pass)"}
        # the same code on one thread (the reference's scalar path is single-threaded), a smaller sample
        from oracle import xabe_oracle as oracle
        n1 = min(4, tokens)
        x1 = xs[0][:n1].cpu().numpy()
        oracle.moe_block_forward(layer, x1, dev_order=False, threads=1)
        t0 = time.perf_counter()
        oracle.moe_block_forward(layer, x1, dev_order=False, threads=1)
        out["cpu_baseline"]["single_thread"] = {"value": n1 / (time.perf_counter() - t0), "unit": UNIT,
                                                "sample": f"{n1} tokens, one pass, dequantisation included"}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_stack(args) -> dict:
    """`--stack-layers` MoE layers of config 1's geometry driven as the reference's Forward::body drives
    them (crates/xabe-engine/src/forward.rs:3497-3618): one handle, each layer's l_out the next layer's
    residual, the whole pass one CUDA graph, the token count a device scalar.  A step = one pass over the
    stack; `value` stays per layer (tokens x layers / time) so it compares with the one-layer workloads."""
    import torch

    from llmxabe_b200 import synth
    from llmxabe_b200.moe import MoeGeometry
    from llmxabe_b200.stack import MoeStack

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("decode64_stack is a one-GPU workload")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(0)
    tokens, block_size, zipf = WORKLOADS[args.workload]
    H, n_layers = 2048, args.stack_layers
    shared_q = synth.Q8_0 if args.shared_quant == "q8_0" else synth.Q6K
    layers = [synth.moe_layer_on_device(seed=0, layer=i, zipf=zipf, shared_quant=shared_q) for i in range(n_layers)]
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
    stack.capture()

    def step(_i):
        stack.replay()

    def step_host(_i):  # the step's input from pinned host memory, its result back to the host
        stack.hidden_in[:tokens].copy_(hx, non_blocking=True)
        stack.replay()
        hout.copy_(stack.hidden_out[:tokens], non_blocking=True)
        stream.synchronize()

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    t0 = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t0 < 0.3:
        step(i)
        i += 1
    steps = max(3, min(args.steps, 50))
    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(step, steps)
    clocks = sampler.stop()
    for i in range(3):
        step_host(i)
    ms_e2e = timed(step_host, steps)
    status = stack.block.moe.device_status()
    peak, peak_src = measured_peaks()
    layer_bytes = layer_algorithmic_bytes(d_mean, tokens, args.shared_quant == "q8_0")
    achieved = n_layers * layer_bytes / (ms * 1e-3) / 1e9
    return {
        "metric": METRIC, "value": tokens * n_layers / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 activations x exact Q6_K codes, fp32 scales+accumulate",
        "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_rank": tokens, "layers": n_layers, "experts": 256,
                   "top_k": 8, "hidden": 2048, "intermediate": 512, "quant": "Q6_K",
                   "shared_expert_quant": args.shared_quant, "bucket": block_size,
                   "distinct_experts_mean": d_mean, "stack_passes_per_s": 1e3 / ms,
                   "stack_tokens_per_s": tokens * 1e3 / ms,
                   "l2": f"every layer has its own weights ({n_layers * layer_bytes / 1e9:.1f} GB per pass, L2 126 MB)",
                   "parallelism": "one GPU"},
        "e2e": {"value": tokens * n_layers / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": tokens * H * 4, "d2h_bytes_per_step": tokens * H * 4},
        "gpu_launches": 7 * n_layers * steps, "cuda_graph": True, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "whole stack pass (all launches of all layers, one graph)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": n_layers * layer_bytes,
                     "ms_per_launch": ms},
        "device_status": status,
    }


def run_head(args) -> dict:
    """The LM head at the real geometry (crates/xabe-cuda/src/kernels/lm_head.rs:1318-1324): one pass over
    the 540 MB Q8_0 tensor serves up to eight tokens.  Three resident copies of the head rotate, and
    one copy alone is four times the L2.  A step = logits for the batch (+ argmax and the 4-byte
    read-back of each token id in the end-to-end figure, which is what a sampler reads)."""
    import numpy as np
    import torch

    from llmxabe_b200 import synth
    from llmxabe_b200.lm_head import HeadFormat, HeadTensor, LmHeadGeometry, LmHeadKernels

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("the lm_head workloads are one-GPU workloads")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the LM head has no CPU fallback")
    torch.cuda.set_device(0)
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

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    t0 = time.perf_counter()
    i = 0
    while i < max(args.warmup, 3) or time.perf_counter() - t0 < 0.3:
        step(i)
        i += 1
    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(step, args.steps)
    clocks = sampler.stop()
    for i in range(3):
        step_host(i)
    ms_e2e = timed(step_host, args.steps)
    status = head.device_status()
    peak, peak_src = measured_peaks()
    alg_bytes = g.weight_bytes_read(tokens) + tokens * (g.hidden + g.vocab) * 4
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": "lm_head_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "exact Q8_0 codes x fp32 activations as two f16 parts, fp32 scales+accumulate",
        "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "hidden": g.hidden, "vocab": g.vocab,
                   "quant": "Q8_0", "weight_bytes": n_bytes,
                   "l2": "three resident copies of the head rotate; one copy is 540 MB (L2 126 MB)",
                   "parallelism": "one GPU"},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": tokens * g.hidden * 4, "d2h_bytes_per_step": tokens * 4},
        "gpu_launches": 2 * args.steps, "cuda_graph": False, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "k_head_rows<Q8_0>", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": alg_bytes, "ms_per_launch": ms},
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


def run_ep(args) -> dict:
    """BASELINE config 3: a stack of MoE layers (Q6_K experts, Q8_0 shared expert), `--ep-tokens` tokens,
    experts sharded over the ranks with NCCL all-to-all dispatch/combine.  Strong scaling: the global
    batch is fixed, each rank owns tokens/N tokens and 256/N experts of every layer."""
    import torch
    import torch.distributed as dist

    from llmxabe_b200 import synth
    from llmxabe_b200.ep import CudaEpBackend, EpMoeBlock
    from llmxabe_b200.moe import MoeGeometry, QuantTensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    E, K, H, I = 256, 8, 2048, 512
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
        backend = PeerMemoryEpBackend(g, epr, rank, world, layers[0][0], *layers[0][1])
    else:
        backend = CudaEpBackend(g, epr, max_rows, layers[0][0], *layers[0][1])
    blk = EpMoeBlock(backend, E, K, rank, world)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(31 + rank)
    x0 = torch.randn(per, H, device="cuda", generator=gen)
    bufs = [torch.empty(per, H, device="cuda") for _ in range(2)]
    ffn = torch.empty(per, H, device="cuda")

    def step(_i):
        h = x0
        for li, (front, local) in enumerate(layers):
            backend.set_layer(front, *local)
            out = bufs[li & 1]
            blk.forward(h, per, ffn, out)
            h = out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 1)):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    barrier()
    clocks = sampler.stop()
    rows = sum(blk.last_plan.recv_counts) if blk.last_plan is not None else 0  # not known on the host with peer memory
    # one more, untimed, pass with per-phase events (per layer, this rank)
    blk.enable_phase_timing()
    step(0)
    phases = {k: v / n_layers for k, v in blk.phase_times_ms().items()}
    blk._events = None
    if world > 1:
        t = torch.tensor([ms, float(rows)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, rows = float(t[0].item()), int(t[1].item())
    status = backend.front_k.device_status() | backend.back_k.device_status()
    flops = 2.0 * tokens * (K + 1) * 3 * H * I * n_layers
    out = {
        "metric": METRIC, "value": tokens * n_layers / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 x f16 -> f32 (tcgen05), weights dequantised to f16",
        "data": "synthetic",
        "config": {"workload": "ep_prefill_stack", "tokens_global": tokens, "layers": n_layers, "experts": E,
                   "top_k": K, "hidden": H, "intermediate": I, "quant": "Q6_K experts, Q8_0 shared",
                   "parallelism": f"ep{world} ({epr} experts/rank), " +
                                  ("peer-memory (NVLink) dispatch + combine, device-side counts and flags"
                                   if args.ep_peer_memory else "NCCL all-to-all-v dispatch + combine"),
                   "max_rows_received_by_a_rank_last_layer": rows,
                   "l2": "every layer has its own weights; a pass streams all of them"},
        "clocks": clocks, "device_status": status, "phase_ms_per_layer_rank0": phases,
        "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12 / world, "unit": "TFLOP/s per GPU",
                     "peak": 1628.8, "frac": flops / (ms * 1e-3) / 1e12 / world / 1628.8, "traffic": None},
        "gpu_launches": None,
    }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_dense(args) -> dict:
    """BASELINE config 4: the dense SwiGLU block of the 27B sibling, Q6_K.  One rank: DenseFfnBlock.
    Several ranks: the intermediate dimension sharded (llmxabe_b200.tp), one all-reduce per layer;
    strong scaling (the token batch is the same on every rank)."""
    import torch
    import torch.distributed as dist

    from llmxabe_b200 import synth
    from llmxabe_b200.moe import QuantTensor
    from llmxabe_b200.tp import CudaTpBackend, TpDenseFfnBlock, shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    H, I = 5120, 17408
    tokens = WORKLOADS[args.workload][0]
    n_layers = max(args.layers, 2)
    i0, i1 = shard_bounds(I, rank, world)
    blocks = []
    for li in range(n_layers):
        gen = torch.Generator(device="cuda")
        gen.manual_seed(4000 + li)           # every rank generates the full matrices and keeps its shard
        full = [QuantTensor(synth._device_quant_bytes(torch, synth.Q6K, H * I, gen, "cuda"), synth.Q6K)
                for _ in range(3)]
        backend = CudaTpBackend(H, I, tokens, rank, world, torch.ones(H, device="cuda"), *full)
        if world > 1:
            backend.gate = QuantTensor(backend.gate.bytes.clone(), synth.Q6K)
            backend.up = QuantTensor(backend.up.bytes.clone(), synth.Q6K)
        else:
            backend.down = full[2]
        del full
        blocks.append(TpDenseFfnBlock(backend, rank, world))
    torch.cuda.empty_cache()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    x0 = torch.randn(tokens, H, device="cuda", generator=gen)
    bufs = [torch.empty(tokens, H, device="cuda") for _ in range(2)]
    ffn = torch.empty(tokens, H, device="cuda")

    def step(i):
        blocks[i % n_layers].forward(x0, tokens, ffn, bufs[i & 1])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    barrier()
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0].item())
    status = 0
    for b in blocks:
        status |= b.backend.k.device_status()
    # end to end: host rows in, host rows out
    hx = torch.randn(tokens, H).pin_memory()
    hout = torch.empty(tokens, H).pin_memory()
    dx = torch.empty(tokens, H, device="cuda")
    barrier()
    e0.record()
    e2e_steps = max(3, min(args.steps, 20))
    for i in range(e2e_steps):
        dx.copy_(hx, non_blocking=True)
        blocks[i % n_layers].forward(dx, tokens, ffn, bufs[0])
        hout.copy_(bufs[0], non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0].item())
    peak, peak_src = measured_peaks()
    weight_bytes = 3 * (H * I // 256) * 210
    alg_bytes = weight_bytes // world + tokens * H * 4 * 3
    flops = 2.0 * tokens * 3 * H * I
    hbm_bound = tokens <= 256
    roof = ({"bound": "hbm", "achieved": alg_bytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
             "frac": alg_bytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
             "algorithmic_bytes_per_launch": alg_bytes, "note": "whole layer per rank (norm, gate/up, down, residual)"}
            if hbm_bound else
            {"bound": "tensor", "achieved": flops / world / (ms * 1e-3) / 1e12, "peak": 1628.8, "unit": "TFLOP/s",
             "frac": flops / world / (ms * 1e-3) / 1e12 / 1628.8, "traffic": None,
             "peak_source": "measured (MEASURED_PEAKS.json, burst)", "note": "whole layer per rank"})
    out = {
        "metric": "dense_layer_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 x f16 -> f32 (tcgen05), Q6_K weights dequantised to f16 on the fly", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "hidden": H, "intermediate": I, "quant": "Q6_K",
                   "resident_layers": n_layers,
                   "parallelism": f"tp{world} (intermediate {i1 - i0} of {I} per rank), NCCL all-reduce",
                   "l2": f"layers rotate every step; a layer's shard is {weight_bytes // world >> 20} MiB (> 126 MB L2)"
                         if weight_bytes // world > 126 << 20 else "layers rotate every step"},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": tokens * H * 4, "d2h_bytes_per_step": tokens * H * 4},
        "gpu_launches": args.steps * 5, "clocks": clocks, "roofline": roof, "device_status": status,
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
    ap.add_argument("--workload", default="decode64", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=4, help="distinct resident layers the steps rotate over")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--shared-quant", default="q6_k", choices=["q6_k", "q8_0"],
                    help="format of the shared expert in the MoE workloads (the shipped file's is Q8_0)")
    ap.add_argument("--stack-layers", type=int, default=40, help="layers of the decode64_stack workload")
    ap.add_argument("--ep-tokens", type=int, default=16384)
    ap.add_argument("--ep-layers", type=int, default=40)
    ap.add_argument("--ep-nccl", dest="ep_peer_memory", action="store_false",
                    help="exchange rows and results with NCCL all-to-alls instead of peer stores over NVLink")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time eager launches instead of CUDA-graph replay")
    args = ap.parse_args()
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
        emit(run_reference(args))
        return
    if args.workload == "ep_prefill_stack":
        out = run_ep(args)
    elif args.workload.startswith("dense"):
        out = run_dense(args)
    elif args.workload == "decode64_stack":
        out = run_stack(args)
    elif args.workload.startswith("lm_head"):
        out = run_head(args)
    else:
        out = run_ours(args)
    if out:
        emit(out)


if __name__ == "__main__":
    main()
