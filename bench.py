"""Benchmark of the routed-expert MoE layer (affine 4-bit group-64 experts) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows T]

Workload: BASELINE config 2 - one layer, hidden 2048, 128 experts of width 768, top-8 - at 64-token decode (the
headline line), with 1-, 4- and 16-token decode, the 2048-token prompt and the EXL3 layer (config 3) beside it under
"sweep"; `--gpus N` (torchrun) times the expert-parallel step, `--config c4` the large skewed layer.  One step = one pass of
the whole layer (router, top-k, plan, gate/up + SiLU-gate, down, combine) over one batch of seeded synthetic tokens.
Two independent weight copies (340 MB each, together far beyond the 126 MB L2) alternate step by step.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the reference's path (oracle/) on
the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

TRAFFIC_GATE_UP_C2_64 = 225054208 + 4798464      # bytes, from the committed ncu capture of the same launch
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
SMI_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense bf16 TFLOP/s, which) from MEASURED_PEAKS.json, else the pool's earlier measurement."""

    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the timed region runs."""

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def layer_bytes(shape, rows: int, distinct: int) -> dict:
    """Algorithmic bytes of one layer call: packed weights of the distinct experts touched + router rows + the tokens
    in and out; intermediates (logits, plan, act, y) are not counted."""

    d, ni = shape.dims, shape.width
    per_matrix = ni * d // 2 + ni * (d // 64) * 4
    ne = shape.experts + (1 if shape.shared else 0)
    return {"gate_up": distinct * 2 * per_matrix + rows * d * 2, "down": distinct * per_matrix,
            "layer": distinct * 3 * per_matrix + ne * d * 2 + 2 * rows * d * 2}


def cpu_baseline(shape, rows: int, steps: int, warmup: int):
    """The CPU restatement of the reference's path (oracle/cpu_moe.c, OpenMP over all host cores) on the same
    synthetic workload; returns (tokens/s, seconds a step, cores)."""

    import numpy as np
    import torch

    from oracle import cpu
    from tensorfold_b200 import synthetic

    def b16(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    def tri(m):
        return m[0].numpy().view(np.uint32), b16(m[1]), b16(m[2])

    gate, up, down = (tri(m) for m in synthetic.affine_layer(shape, "cpu"))
    x = b16(synthetic.activations(shape, rows, "cpu"))
    rt = b16(synthetic.router_rows(shape, "cpu"))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        cpu.moe_layer(x, rt, shape.experts, shape.top_k, shape.shared, gate, up, down, 64, True)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return rows / sec, sec, cpu.threads()


def run_reference(args) -> None:
    """--impl reference: the reference's CPU path (restated in oracle/) on the host cores; rank 0 only."""

    if int(os.environ.get("RANK", "0")) != 0:
        return
    from tensorfold_b200 import synthetic

    shape, rows = synthetic.C2, args.rows
    value, sec, cores = cpu_baseline(shape, rows, args.steps, args.warmup)
    sample = f"{rows}-token batch of the c2 layer a step, all experts' math on the host ({cores} threads)"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(shape, rows, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(shape, rows: int, gpus: int, config: str = "c2") -> dict:
    if config == "c5":
        return {"workload": f"BASELINE config 5: 8 MoE layers with bf16 residual adds, {rows * gpus} tokens over the "
                            f"ranks, hidden {shape.dims}, {shape.experts} experts x FFN {shape.width}, "
                            f"top-{shape.top_k}, EXL3 experts at a seeded 2..8 bits a tensor (3inst)",
                "rows_per_gpu": rows, "l2": "the 8 layers' weights of a rank (15 GB / ranks) cycle every step",
                "parallelism": f"ep{gpus}" if gpus > 1 else "single"}
    what = (f"BASELINE config 4: one MoE layer, {rows * gpus} tokens over the ranks, Zipf-skewed router, one replicated "
            "shared expert," if config == "c4" else f"BASELINE config 2: one MoE layer, {rows}-token decode,")
    return {"workload": f"{what} hidden {shape.dims}, {shape.experts} "
                        f"experts x FFN {shape.width}, top-{shape.top_k}, MLX affine 4-bit g64 (fp16 scales)",
            "rows_per_gpu": rows, "l2": "two 340 MB weight copies alternate (inputs larger than the 126 MB L2)",
            "parallelism": f"ep{gpus}" if gpus > 1 else "single"}


def time_graphs(torch, graphs, steps: int, warmup: int) -> float:
    """Milliseconds a step: `steps` replays alternating over `graphs`, CUDA events on the current stream."""

    for i in range(warmup):
        graphs[i % len(graphs)].replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        graphs[i % len(graphs)].replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def bench_rows(torch, shape, layers, rows: int, steps: int, warmup: int, hbm: float, prefill: bool = False,
               tflops: float = 0.0):
    """Device-resident timing of the whole layer at `rows` tokens plus the gate/up kernel alone."""

    from tensorfold_b200 import experts, moe, synthetic

    dev = layers[0].router.device
    runners = [moe.Runner(m, rows, prefill=prefill, device=dev) for m in layers]
    x = synthetic.activations(shape, rows, dev)
    for r in runners:
        r.x.copy_(x)
    ms = time_graphs(torch, [r.graph for r in runners], steps, warmup)
    distinct = int(runners[0].buf.plan.counts[1])
    nbytes = layer_bytes(shape, rows, distinct)
    # the dominant kernel alone: gate/up over the plan the layer just made, 4 launches a weight copy in one graph
    reps = 4
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.graph(g, stream=side):
        for _ in range(reps):
            for r in runners:
                experts.gate_up(r.x, r.layer.experts, r.buf.plan, r.buf.act.view(-1, shape.width), rows)
    kms = time_graphs(torch, [g], max(3, steps // 4), 3) / (reps * len(runners))
    gbs = nbytes["gate_up"] / (kms * 1e-3) / 1e9
    extra = {}
    if prefill:
        pairs = rows * runners[0].buf.slots
        flops_gu, flops_all = pairs * 2 * 2 * shape.dims * shape.width, pairs * 3 * 2 * shape.dims * shape.width
        extra = {"form": "prefill (tcgen05)", "gate_up_tflops": flops_gu / (kms * 1e-3) / 1e12,
                 "gate_up_frac_of_bf16_peak": flops_gu / (kms * 1e-3) / 1e12 / tflops if tflops else None,
                 "layer_tflops": flops_all / (ms * 1e-3) / 1e12,
                 "layer_frac_of_bf16_peak": flops_all / (ms * 1e-3) / 1e12 / tflops if tflops else None}
    return {**extra, "rows": rows, "ms_per_step": ms, "tokens_per_s": rows / (ms * 1e-3), "distinct_experts": distinct,
            "layer_bytes": nbytes["layer"], "layer_gbs": nbytes["layer"] / (ms * 1e-3) / 1e9,
            "layer_frac_of_hbm": nbytes["layer"] / (ms * 1e-3) / 1e9 / hbm,
            "gate_up_us": kms * 1e3, "gate_up_bytes": nbytes["gate_up"], "gate_up_gbs": gbs,
            "launches_per_step": runners[0].launches}, runners


def bench_exl3(torch, rows_list, steps: int, warmup: int, hbm: float):
    """Config 3: the same layer shape with EXL3 experts at 4.00 bits a weight (3inst), router and selection included;
    two weight copies alternate.  Bytes = trellis + suh/svh of the distinct experts + router rows + tokens."""

    from tensorfold_b200 import moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape, dev = synthetic.C3, torch.device("cuda", torch.cuda.current_device())
    router = synthetic.router_rows(shape, dev)
    layers = [x3.prepare(*synthetic.exl3_layer(shape, dev, 4, copy=c), x3.CB_3INST, device=dev) for c in range(2)]

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    results = []
    for rows in rows_list:
        x = synthetic.activations(shape, rows, dev)
        graphs, bufs = [], []
        for ex in layers:
            buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
            scratch = x3.Scratch(ex, rows, shape.top_k, device=dev)
            out = torch.empty((rows, shape.dims), dtype=torch.float32, device=dev)

            def step(ex=ex, buf=buf, scratch=scratch, out=out):
                moe.router(x, router, buf.logits)
                moe.select_rows(buf.logits, buf, shape.top_k, shape.experts)
                x3.routed(x, buf.pick, buf.wts, ex, scratch, out, rows)

            step()
            torch.cuda.synchronize()
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                step()
            graphs.append(g)
            bufs.append((buf, scratch))
        ms = time_graphs(torch, graphs, steps, warmup)
        distinct = int(bufs[0][1].count[0])
        per_expert = 3 * shape.dims * shape.width // 2 + 2 * (2 * shape.dims + 2 * shape.width) + 2 * (shape.dims + shape.width)
        nbytes = distinct * per_expert + shape.experts * shape.dims * 2 + rows * shape.dims * (2 + 4)
        results.append({"form": "exl3 4.00 bpw (config 3)", "rows": rows, "ms_per_step": ms,
                        "tokens_per_s": rows / (ms * 1e-3), "distinct_experts": distinct, "layer_bytes": nbytes,
                        "layer_gbs": nbytes / (ms * 1e-3) / 1e9, "layer_frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm,
                        "launches_per_step": 8})
    return results


def bench_e2e(torch, runners, shape, rows: int, steps: int, warmup: int):
    """The same step through the public API with HOST buffers: pinned tokens in, layer, result back, every step."""

    from tensorfold_b200 import synthetic

    x_host = synthetic.activations(shape, rows, "cpu").pin_memory()
    out_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    for r in runners:
        r.bind_host(x_host, out_host)                           # the copies become nodes of the step's graph
    for i in range(warmup):
        runners[i % len(runners)].replay_host()
        torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        runners[i % len(runners)].replay_host()
        torch.cuda.current_stream().synchronize()               # the caller reads the result before the next step
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    nbytes = rows * shape.dims * 2
    return {"value": rows / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "h2d_bytes_per_step": nbytes,
            "d2h_bytes_per_step": nbytes}


def ep_rows(args, shape, world: int) -> int:
    """Rows a rank: config 2 keeps `--rows` a GPU (weak scaling); config 4 splits its 256 tokens over the ranks."""

    return 256 // world if args.config == "c4" else args.rows


def hot_pairs(args) -> int:
    """Pairs from which a rank's expert runs through the prompt-form kernel (off unless asked for: at config 4's sizes
    one prompt-form item is a 70 us serial chain on 16 CTAs, which costs more than the decode items it replaces)."""

    return max(args.hot_pairs, 0)


def ep_copies(args, world: int) -> int:
    """Independent weight copies a rank rotates so that a step's weights never sit in the 126 MB L2."""

    return 2 if args.config == "c4" else 2 * world          # a config-4 slice is 5.4 GB / world


COLLECTIVE = {
    "tokens": "NCCL all-gather of the tokens, reduce-scatter of fp32 per-token partial sums",
    "rows": "NCCL all-gather of the tokens, reduce-scatter of fp32 per-pair rows (exact)",
    "peer": "own kernels over NVLink peer memory: pull of the tokens, push of fp32 per-token partial sums, two flag "
            "barriers (no collective library on the step)",
}


def bench_ep(torch, dist, args, shape, dev, rank: int, world: int):
    """Expert-parallel step: this rank's `rows` tokens through the layer whose experts are sharded over the ranks
    (NCCL all-to-all dispatch and return).  Each rank keeps 2 * world copies of its expert slice and rotates them, so a
    step's weights (a slice is 340 / world MB) never sit in L2.  Returns (ms a step by CUDA events, launches a step)."""

    from tensorfold_b200 import ep, experts, moe, synthetic

    rows, per = ep_rows(args, shape, world), shape.experts // world
    router = synthetic.router_rows(shape, dev)
    bias = synthetic.zipf_bias(shape, 1.1, dev) if args.config == "c4" else None
    copies, graphs = [], []
    for copy in range(ep_copies(args, world)):
        gate, up, down = synthetic.affine_layer(shape, dev, torch.float16 if args.scales == "fp16" else torch.bfloat16,
                                                copy=copy)

        def cut(which):
            return experts.make([tuple(t[which].contiguous() for t in gate), tuple(t[which].contiguous() for t in up)],
                                tuple(t[which].contiguous() for t in down), 64)

        local = cut(slice(rank * per, (rank + 1) * per))
        if args.ep_reduce == "peer":
            shared = cut(slice(shape.experts, shape.experts + 1)) if shape.shared else None
            layer, why = None, ""
            try:
                layer = ep.PeerExpertParallel(router, local, shape.experts, shape.top_k, rows, shared_experts=shared,
                                              logit_bias=bias, hot_pairs=hot_pairs(args))
            except Exception as err:                       # e.g. peer mappings refused on this machine
                why = repr(err)
            failed = torch.tensor([0 if layer is not None else 1], device=dev)
            dist.all_reduce(failed, op=dist.ReduceOp.MAX)
            if int(failed.item()) and copy == 0 and args.config == "c2":
                # said loudly and recorded in the line: the same data flow through NCCL, still this library's kernels
                print(f"[bench] rank {rank}: peer windows unavailable ({why or 'on another rank'}); "
                      "falling back to --ep-reduce tokens", file=sys.stderr)
                args.ep_reduce = "tokens"
                copies.append(ep.GatheredExpertParallel(router, local, shape.experts, shape.top_k, rows,
                                                        reduce="tokens"))
            elif int(failed.item()):
                raise SystemExit(f"peer windows unavailable: {why or 'on another rank'}")
            else:
                copies.append(layer)
        else:
            copies.append(ep.GatheredExpertParallel(router, local, shape.experts, shape.top_k, rows,
                                                    reduce=args.ep_reduce))
        del gate, up, down
    x = synthetic.activations(shape, rows, dev, index=100 + rank)
    side = torch.cuda.Stream(dev)
    if args.ep_reduce == "peer":                           # the tokens live in each copy's window; nothing to stage
        inputs = [layer.tokens for layer in copies]
        for t in inputs:
            t.copy_(x)
        steps = [layer.forward for layer in copies]
    else:
        inputs = [x] * len(copies)
        steps = [(lambda layer=layer: layer.forward(x)) for layer in copies]
    for step in steps:                                     # warm up eagerly (NCCL set-up), then capture the step
        step()
    torch.cuda.synchronize()
    dist.barrier()
    for step in steps:
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            step()
        graphs.append(g)
    torch.cuda.synchronize()
    dist.barrier()
    for i in range(args.warmup):
        graphs[i % len(graphs)].replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(args.steps):
        graphs[i % len(graphs)].replay()
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = a.elapsed_time(b) / args.steps
    # end to end: pinned host tokens in, result back, every step
    x_host = x.cpu().pin_memory()
    out_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()
    dist.barrier()
    host_graphs = []
    for step, inp, layer in zip(steps, inputs, copies):    # the same step with its host transfers inside the graph
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            if args.ep_reduce == "peer":                   # kernels read the pinned rows and store the pinned result
                layer.forward(x_host, out_host)
            else:
                inp.copy_(x_host, non_blocking=True)
                step()
                out_host.copy_(layer.out, non_blocking=True)
        host_graphs.append(g)
    torch.cuda.synchronize()
    dist.barrier()
    for i in range(min(args.warmup, len(host_graphs))):
        host_graphs[i].replay()
    torch.cuda.synchronize()
    dist.barrier()
    a.record()
    for i in range(args.steps):
        host_graphs[i % len(host_graphs)].replay()
        torch.cuda.current_stream().synchronize()
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    e2e_ms = a.elapsed_time(b) / args.steps
    # this rank's algorithmic bytes a step: its touched experts' packed weights, the router rows, its tokens in and out
    layer = copies[0]
    nbytes = router.numel() * 2 + 2 * rows * shape.dims * 2
    if args.ep_reduce == "peer":
        w = layer.win
        mine = w.pick_all[:, :shape.top_k].reshape(-1)
        mine = mine[(mine >= w.lo) & (mine < w.lo + w.per_rank)]
        nbytes += int(torch.unique(mine).numel()) * local.bytes_per_expert()
        if shape.shared:
            nbytes += local.bytes_per_expert()
    else:
        nbytes += per * local.bytes_per_expert()
    return ms, e2e_ms, layer.launches, nbytes


def bench_c5(torch, dist, args, dev, rank: int, world: int):
    """Config 5 on the expert-parallel EXL3 path: 8 layers (hidden 4096, 160 experts x FFN 1536, top-8, a seeded width
    of 2..8 bits a tensor), 128 tokens split over the ranks, `h = bf16(h + moe(h))` between layers; one step = the
    8-layer stack in one CUDA graph.  A rank holds only its experts (1.9 GB over the 8 layers at 8 ranks, so no layer's
    weights survive in L2 from step to step).  Returns (ms a step, ms end to end, launches, rank-0 bytes, rows)."""

    import random

    from tensorfold_b200 import ep, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape, layers_n, tokens = synthetic.C5, 8, 128
    rows, per = tokens // world, shape.experts // world
    rng = random.Random(5005)
    widths = {(li, e, m): rng.choice((2, 3, 4, 5, 6, 7, 8)) for li in range(layers_n) for e in range(shape.experts)
              for m in range(3)}                                  # every rank draws all widths in the same order
    router = synthetic.router_rows(shape, dev)
    layers = []
    for li in range(layers_n):
        base = 1000 * shape.config + 10 + 1000003 * li
        gate, up, down = [], [], []
        for e in range(rank * per, (rank + 1) * per):
            gate.append(synthetic.exl3_matrix(base + 3 * e, shape.dims, shape.width, widths[(li, e, 0)], dev))
            up.append(synthetic.exl3_matrix(base + 3 * e + 1, shape.dims, shape.width, widths[(li, e, 1)], dev))
            down.append(synthetic.exl3_matrix(base + 3 * e + 2, shape.width, shape.dims, widths[(li, e, 2)], dev))
        ex = x3.prepare(gate, up, down, x3.CB_3INST, device=dev)
        layers.append(ep.PeerExl3ExpertParallel(router, ex, shape.experts, shape.top_k, rows))
    x = synthetic.activations(shape, rows, dev, index=100 + rank)
    h_out = torch.zeros_like(x)

    def step(src):
        h = src
        for li, layer in enumerate(layers):
            y = layer.forward(h)                                  # fp32 [rows, D]
            if li == 0:
                h = layer.tokens                                  # the staged rows (src may be pinned host memory)
            h = (h.float() + y).to(torch.bfloat16)                # the residual add between layers
        h_out.copy_(h)

    step(x)
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step(x)
    x_host = x.cpu().pin_memory()
    out_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    side.wait_stream(torch.cuda.current_stream())
    host_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(host_graph, stream=side):
        step(x_host)
        out_host.copy_(h_out, non_blocking=True)
    torch.cuda.synchronize()
    dist.barrier()

    def timed(g, sync_each):
        for _ in range(args.warmup):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            g.replay()
            if sync_each:
                torch.cuda.current_stream().synchronize()
        b.record()
        torch.cuda.synchronize()
        dist.barrier()
        return a.elapsed_time(b) / args.steps

    ms, e2e_ms = timed(graph, False), timed(host_graph, True)
    nbytes = layers_n * (router.numel() * 2) + 2 * rows * shape.dims * 2
    for layer in layers:
        w = layer.win
        mine = w.pick_all.reshape(-1)
        mine = torch.unique(mine[(mine >= w.lo) & (mine < w.lo + w.per_rank)]) - w.lo
        nbytes += layer.local.nbytes_read(mine.cpu().tolist())
    launches = sum(layer.launches for layer in layers) + 3 * layers_n + 1
    return ms, e2e_ms, launches, nbytes, rows


def run_ours(args) -> None:
    import torch

    from tensorfold_b200 import _lib, experts, moe, synthetic

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU fallback (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ep_path = world > 1 or args.config in ("c4", "c5")   # configs 4 and 5 always run the expert-parallel code
    if ep_path:
        import torch.distributed as dist

        if world == 1:                                 # not under torchrun: a group of one
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
        else:
            dist.init_process_group("nccl", device_id=dev)
    hbm, tflops, which = peaks()
    _lib.set_pdl(bool(args.pdl))
    if args.exl3_only:
        print(json.dumps({"sweep": bench_exl3(torch, (1, 64), args.steps, args.warmup, hbm)}))
        return
    shape, rows = (synthetic.C4 if args.config == "c4" else synthetic.C5 if args.config == "c5" else synthetic.C2), \
        args.rows
    if args.config == "c5" and args.ep_reduce != "peer":
        raise SystemExit("--config c5 runs the peer-memory form")
    if args.config == "c4":
        if args.ep_reduce != "peer":
            raise SystemExit("--config c4 runs the peer-memory form")
        rows = ep_rows(args, shape, world)
    layers = []
    for copy in range(0 if ep_path else 2):
        gate, up, down = synthetic.affine_layer(shape, dev, torch.float16 if args.scales == "fp16" else torch.bfloat16,
                                                 copy=copy)
        layers.append(moe.Routed(synthetic.router_rows(shape, dev), experts.make([gate, up], down, 64), shape.top_k,
                                 shared=shape.shared))
        del gate, up, down
    torch.cuda.synchronize()

    if ep_path:
        if shape.experts % world:
            raise SystemExit(f"{shape.experts} experts do not shard over {world} ranks")
        del layers
        with ClockSampler(local) as clocks:
            if args.config == "c5":
                ms, e2e_ms, launches, rank_bytes, rows = bench_c5(torch, dist, args, dev, rank, world)
            else:
                ms, e2e_ms, launches, rank_bytes = bench_ep(torch, dist, args, shape, dev, rank, world)
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
        status = _lib.kernel_status()
        if status != 0:
            raise SystemExit(f"a kernel recorded device status {status}")
        if rank == 0:
            nbytes = rows * shape.dims * 2 * world
            line = {"metric": METRIC, "value": world * rows / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                    "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                    "scaling": "weak" if args.config == "c2" else "strong", "vs_baseline": None,
                    "dtype": "f16" if args.config == "c5" else "bf16", "data": "synthetic",
                    "config": {**workload_config(shape, rows, world, args.config),
                               **({} if args.config == "c5" else {
                                   "l2": f"each rank rotates {ep_copies(args, world)} copies of its "
                                         f"{shape.experts // world}-expert slice (inputs larger than the 126 MB L2)"}),
                               "collective": COLLECTIVE[args.ep_reduce] + "; the step is one CUDA graph",
                               "hot_pairs": hot_pairs(args)},
                    "clocks": clocks.summary(),
                    "e2e": {"value": world * rows / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                            "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes},
                    "gpu_launches": launches * args.steps,
                    "roofline": {"bound": "hbm", "kernel": "the whole expert-parallel step on one GPU (rank 0)",
                                 "achieved": rank_bytes / (ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                                 "frac": rank_bytes / (ms * 1e-3) / 1e9 / hbm, "peak_source": f"of {which}",
                                 "traffic": None, "bytes_per_step": rank_bytes,
                                 "note": "algorithmic bytes of rank 0's step (its touched experts' packed weights, "
                                         "router rows, tokens in and out) over the step time; the per-kernel roofline "
                                         "with ncu traffic is the 1-GPU line's"},
                    "cpu_baseline": None}
            print(json.dumps(line))
        dist.barrier()
        dist.destroy_process_group()
        return
    with ClockSampler(local) as clocks:
        torch.cuda.synchronize()
        head, runners = bench_rows(torch, shape, layers, rows, args.steps, args.warmup, hbm, args.form == "prefill",
                                   tflops)
        torch.cuda.synchronize()
    e2e = bench_e2e(torch, runners, shape, rows, args.steps, args.warmup)
    status = _lib.kernel_status()
    if status != 0:
        raise SystemExit(f"a kernel recorded device status {status}")
    ms = head["ms_per_step"]
    sweep = []
    if world == 1 and not args.no_sweep:
        del runners
        for t_rows, pre in ((1, False), (4, False), (16, False), (2048, True)):
            res, rr = bench_rows(torch, shape, layers, t_rows, max(5, args.steps // 2), args.warmup, hbm, pre, tflops)
            res.setdefault("form", "decode")
            sweep.append(res)
            del rr
        del layers
        torch.cuda.empty_cache()
        sweep += bench_exl3(torch, (1, 64), max(5, args.steps // 2), args.warmup, hbm)
    if rank != 0:
        return
    value = world * rows / (ms * 1e-3)
    cpu = None
    if not args.no_cpu:
        passes = 100                                      # about 10 s of host work at 0.1 s a pass
        v, sec, cores = cpu_baseline(shape, rows, passes, 2)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{passes} timed passes (2 warm-up) of the same {rows}-token layer call, {sec:.3f} s a pass"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(shape, rows, world),
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": head["launches_per_step"] * args.steps,
            "roofline": {"bound": "hbm", "kernel": "decode_kernel<M=2, SwiGLU> (gate/up)",
                         "achieved": head["gate_up_gbs"], "peak": hbm, "unit": "GB/s",
                         "frac": head["gate_up_gbs"] / hbm, "peak_source": f"of {which}",
                         "traffic": TRAFFIC_GATE_UP_C2_64 if (rows, args.form) == (64, "decode") else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this "
                                           "workload (profiles/decode_kernel_c2_64tokens.md)",
                         "bytes_per_launch": head["gate_up_bytes"], "us_per_launch": head["gate_up_us"]},
            "layer": {k: head[k] for k in ("distinct_experts", "layer_bytes", "layer_gbs", "layer_frac_of_hbm")},
            "cpu_baseline": cpu, "sweep": sweep}
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=64, help="tokens a step on each GPU")
    ap.add_argument("--scales", default="fp16", choices=["fp16", "bf16"], help="dtype of the affine scales and biases")
    ap.add_argument("--pdl", type=int, default=1, help="1: programmatic dependent launch between the layer's kernels")
    ap.add_argument("--form", default="decode", choices=["decode", "prefill"],
                    help="arithmetic form of the headline run (the sweep always uses decode at 1 and prefill at 2048)")
    ap.add_argument("--exl3-only", action="store_true",
                    help="run only the EXL3 (config 3) lines of the sweep and print them (a profiling aid)")
    ap.add_argument("--ep-reduce", default="peer", choices=["tokens", "rows", "peer"],
                    help="multi-GPU exchanges: own kernels over NVLink peer memory (default), or NCCL with per-token "
                         "partial sums / exact per-pair rows")
    ap.add_argument("--config", default="c2", choices=["c2", "c4", "c5"],
                    help="c2: the headline layer (default); c4: the 256-expert layer with a shared expert and skewed "
                         "routing, 256 tokens split over the ranks; c5: the 8-layer mixed-width EXL3 stack, 128 tokens "
                         "split over the ranks")
    ap.add_argument("--hot-pairs", type=int, default=-1,
                    help="expert-parallel peer form: experts with at least this many pairs use the prompt-form kernel "
                         "(default 0: never)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sweep", action="store_true", help="skip the 1-, 4-, 16- and 2048-token lines")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        args.steps = min(args.steps, 400)                        # a bounded CPU sample: a pass takes ~0.3 s
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
