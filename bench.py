"""Benchmark of the routed-expert MoE layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows T] [--config c2|c4|c5]

Headline workload: BASELINE config 2 - one layer, hidden 2048, 128 experts of width 768, top-8, MLX affine 4-bit
group-64 experts - at 64-token decode.  One step = one pass of the whole layer (router, top-k, plan, gate/up +
SiLU-gate, down, combine) over one batch of seeded synthetic tokens.  Beside it, in the same JSON line:

* "sweep": 1-, 4- and 16-token decode, the 2048-token prompt (tcgen05 form) and the EXL3 layer of config 3;
* "c4": BASELINE config 4 (hidden 6144, 256 experts x FFN 2048 + a shared expert, Zipf-skewed router, 256 tokens
  split over the ranks - strong scaling) and "c5": BASELINE config 5 (8 EXL3 layers of mixed width, 1..512 tokens
  split over the ranks), both on the expert-parallel path at the run's rank count;
* with `--gpus N` (torchrun) the headline is the expert-parallel step at 64 tokens a rank (weak scaling), and
  "ep_check" records that every rank's output was compared with the one-GPU layer before the clock started.

Timing: K steps between two CUDA events, repeated until at least 300 steps were timed; the median repeat is reported
(every repeat times exactly K steps).  Weights and inputs rotate so that a step's weights are read from DRAM.
Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference's path (oracle/) on
all host cores instead.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
SMI_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
C5_TOKENS = (1, 8, 32, 128, 512)
C5_LAYERS = 8
TOL = 1e-2                                         # relative L2 of a layer output against the one-GPU layer


def peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense bf16 TFLOP/s, which) from MEASURED_PEAKS.json, else the pool's earlier measurement."""

    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, "fallback"


def kernel_source_sha() -> str:
    """Hash of the decode kernel's sources: an ncu capture is quoted only while the kernel it measured is unchanged."""

    h = hashlib.sha256()
    for name in ("common.cuh", "experts_decode.cu"):
        h.update((ROOT / "tensorfold_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def captured_traffic() -> tuple[int | None, str]:
    """DRAM bytes of one gate/up launch of the headline workload from the committed ncu summary, or None when that
    summary was taken from other kernel sources than the ones in this tree."""

    path = ROOT / "profiles" / "decode_kernel_c2_64tokens.md"
    if not path.exists():
        return None, "no ncu summary committed"
    text = path.read_text()
    nbytes = re.search(r"traffic_bytes_per_launch:\s*(\d+)", text)
    sha = re.search(r"kernel_source_sha:\s*([0-9a-f]+)", text)
    if not nbytes or not sha:
        return None, "the ncu summary carries no traffic record"
    if sha.group(1) != kernel_source_sha():
        return None, "the committed ncu capture measured other kernel sources than this tree's (stale)"
    return int(nbytes.group(1)), ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload "
                                  "(profiles/decode_kernel_c2_64tokens.md, same kernel sources)")


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


# ---- CPU legs (the only code here that touches oracle/) --------------------------------------------------------------

def cpu_baseline(shape, rows: int, steps: int, warmup: int, threads: int | None = None):
    """The CPU restatement of the reference's path (oracle/cpu_moe.c, OpenMP) on the same synthetic workload with
    `threads` host threads (all cores unless given); returns (tokens/s, seconds a step, threads used)."""

    import numpy as np
    import torch

    from oracle import cpu
    from tensorfold_b200 import synthetic

    cpu.set_threads(threads or os.cpu_count() or 1)      # torchrun exports OMP_NUM_THREADS=1: set it explicitly

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


def cpu_baseline_exl3(rows: int, steps: int, threads: int | None = None):
    """The EXL3 layer of config 3 (4.00 bits a weight) through oracle/cpu_exl3.c on the host cores: the routed experts
    of `rows` seeded tokens (routing by the oracle's router and top-k).  Returns (tokens/s, seconds a step, threads)."""

    import numpy as np
    import torch

    from oracle import cpu
    from tensorfold_b200 import synthetic

    cpu.set_threads(threads or os.cpu_count() or 1)
    shape = synthetic.C3
    x = synthetic.activations(shape, rows, "cpu")
    rt = synthetic.router_rows(shape, "cpu")

    def b16(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    logits = cpu.router_logits(b16(x), b16(rt))
    pick, wts = cpu.topk_rows(logits, shape.experts, shape.top_k, False)
    used = sorted(set(pick.reshape(-1).tolist()))
    base = 1000 * shape.config + 10
    mats = [[None] * shape.experts for _ in range(3)]
    for e in used:                                          # only the experts the rows use are generated
        for m, (k, n) in enumerate(((shape.dims, shape.width), (shape.dims, shape.width), (shape.width, shape.dims))):
            t, suh, svh = synthetic.exl3_matrix(base + 3 * e + m, k, n, 4, "cpu")
            mats[m][e] = (t.numpy(), suh.numpy(), svh.numpy())
    xf = x.float().numpy()
    times = []
    for i in range(1 + steps):
        t0 = time.perf_counter()
        cpu.exl3_routed(xf, pick, wts, mats[0], mats[1], mats[2], 0, shape.dims, shape.width)
        if i >= 1:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return rows / sec, sec, cpu.threads()


def run_reference(args) -> None:
    """--impl reference: the reference's CPU path (restated in oracle/) on all host cores; rank 0 only."""

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
        batch = f"{rows} tokens" if rows else "batches of " + ", ".join(str(t) for t in C5_TOKENS) + " tokens"
        return {"workload": f"BASELINE config 5: {C5_LAYERS} MoE layers with bf16 residual adds, {batch} over the "
                            f"ranks, hidden {shape.dims}, {shape.experts} experts x FFN {shape.width}, "
                            f"top-{shape.top_k}, EXL3 experts at a seeded 2..8 bits a tensor (3inst)",
                "tokens": rows, "l2": "16 seeded token batches rotate, so the experts (and weights) change every step",
                "parallelism": f"ep{gpus}" if gpus > 1 else "single"}
    what = (f"BASELINE config 4: one MoE layer, {rows * gpus} tokens over the ranks, Zipf-skewed router, one replicated "
            "shared expert," if config == "c4" else f"BASELINE config 2: one MoE layer, {rows}-token decode,")
    return {"workload": f"{what} hidden {shape.dims}, {shape.experts} "
                        f"experts x FFN {shape.width}, top-{shape.top_k}, MLX affine 4-bit g64 (fp16 scales)",
            "rows_per_gpu": rows, "l2": "two 340 MB weight copies alternate (inputs larger than the 126 MB L2)",
            "parallelism": f"ep{gpus}" if gpus > 1 else "single"}


# ---- timing ---------------------------------------------------------------------------------------------------------

def repeats_for(steps: int) -> int:
    """Repeats of `steps` timed steps so that at least 300 steps are timed in all (3 .. 25 repeats)."""

    return max(3, min(25, math.ceil(300 / max(steps, 1))))


def timed(torch, replay, steps: int, warmup: int, repeats: int, dist=None, sync_each: bool = False):
    """`repeats` measurements, each of exactly `steps` calls `replay(i)` between two CUDA events on the current stream
    (device time; with `dist` a barrier before each and the max over ranks of each).  Returns (median ms a step, all)."""

    n = 0
    for _ in range(warmup):
        replay(n)
        n += 1
    torch.cuda.synchronize()
    out = []
    for _ in range(repeats):
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            replay(n)
            n += 1
            if sync_each:
                torch.cuda.current_stream().synchronize()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / steps)
    if dist is not None and dist.get_world_size() > 1:
        t = torch.tensor(out, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out = t.tolist()
    return statistics.median(out), out


def spread(all_ms) -> dict:
    return {"repeats": len(all_ms), "ms_min": min(all_ms), "ms_max": max(all_ms)}


def rel_l2(torch, got, want) -> float:
    return float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-30))


# ---- one GPU --------------------------------------------------------------------------------------------------------

def bench_rows(torch, shape, layers, rows: int, steps: int, warmup: int, hbm: float, prefill: bool = False,
               tflops: float = 0.0):
    """Device-resident timing of the whole layer at `rows` tokens plus the gate/up kernel alone.  Enough runners
    (weight copy x seeded token batch) rotate that the weights a step reads were not read by the steps just before
    it: a few tokens touch only a few experts, so their batches - and with them the experts - change every step."""

    from tensorfold_b200 import _lib, experts, moe, synthetic

    dev = layers[0].router.device
    per_expert = layers[0].experts.bytes_per_expert()
    touched = min(shape.experts, rows * shape.top_k) * per_expert
    n_inputs = 1 if prefill else max(1, min(16, math.ceil(400e6 / (touched * len(layers)))))
    runners = []
    for i in range(n_inputs):
        for m in layers:
            r = moe.Runner(m, rows, prefill=prefill, device=dev)
            r.x.copy_(synthetic.activations(shape, rows, dev, index=i))
            runners.append(r)
    # the timed mode (CUDA graph + programmatic dependent launch) against ordinary eager launches, once
    was = _lib.set_pdl(False)
    eager = moe.run(runners[0].x, runners[0].layer, prefill=prefill).clone()
    _lib.set_pdl(was)
    if not torch.equal(runners[0].replay(), eager):
        raise SystemExit(f"graph replay of the {rows}-token layer differs from the eager layer")
    ms, all_ms = timed(torch, lambda i: runners[i % len(runners)].graph.replay(), steps, warmup, repeats_for(steps))
    distinct = statistics.mean(int(r.buf.plan.counts[1]) for r in runners)
    nbytes = {k: 0 for k in ("gate_up", "down", "layer")}
    for r in runners:
        for k, v in layer_bytes(shape, rows, int(r.buf.plan.counts[1])).items():
            nbytes[k] += v / len(runners)
    # the dominant kernel alone: gate/up over the plans the layers just made, one graph over every runner
    reps = max(1, 8 // len(runners))
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.graph(g, stream=side):
        for _ in range(reps):
            for r in runners:
                experts.gate_up(r.x, r.layer.experts, r.buf.plan, r.buf.act.view(-1, shape.width), rows)
    kms, _ = timed(torch, lambda i: g.replay(), max(3, steps // 4), 3, 5)
    kms /= reps * len(runners)
    gbs = nbytes["gate_up"] / (kms * 1e-3) / 1e9
    extra = {}
    if prefill:
        pairs = rows * runners[0].buf.slots
        flops_gu, flops_all = pairs * 2 * 2 * shape.dims * shape.width, pairs * 3 * 2 * shape.dims * shape.width
        extra = {"form": "prefill (tcgen05)", "gate_up_tflops": flops_gu / (kms * 1e-3) / 1e12,
                 "gate_up_frac_of_bf16_peak": flops_gu / (kms * 1e-3) / 1e12 / tflops if tflops else None,
                 "layer_tflops": flops_all / (ms * 1e-3) / 1e12,
                 "layer_frac_of_bf16_peak": flops_all / (ms * 1e-3) / 1e12 / tflops if tflops else None}
    return {**extra, "rows": rows, "ms_per_step": ms, **spread(all_ms), "tokens_per_s": rows / (ms * 1e-3),
            "distinct_experts": distinct, "rotation": f"{len(layers)} weight copies x {n_inputs} token batches",
            "layer_bytes": nbytes["layer"], "layer_gbs": nbytes["layer"] / (ms * 1e-3) / 1e9,
            "layer_frac_of_hbm": nbytes["layer"] / (ms * 1e-3) / 1e9 / hbm,
            "gate_up_us": kms * 1e3, "gate_up_bytes": nbytes["gate_up"], "gate_up_gbs": gbs,
            "gate_up_frac_of_hbm": gbs / hbm, "launches_per_step": runners[0].launches}, runners


def bench_exl3(torch, rows_list, steps: int, warmup: int, hbm: float):
    """Config 3: the same layer shape with EXL3 experts at 4.00 bits a weight (3inst), router and selection included;
    two weight copies x enough seeded token batches rotate that a step's trellises come from DRAM.
    Bytes = trellis + suh/svh of the distinct experts + router rows + tokens."""

    from tensorfold_b200 import moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape, dev = synthetic.C3, torch.device("cuda", torch.cuda.current_device())
    router = synthetic.router_rows(shape, dev)
    layers = [x3.prepare(*synthetic.exl3_layer(shape, dev, 4, copy=c), x3.CB_3INST, device=dev) for c in range(2)]
    per_expert = 3 * shape.dims * shape.width // 2 + 2 * (2 * shape.dims + 2 * shape.width) + 2 * (shape.dims + shape.width)

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    results = []
    for rows in rows_list:
        touched = min(shape.experts, rows * shape.top_k) * per_expert
        n_inputs = max(1, min(16, math.ceil(400e6 / (touched * len(layers)))))
        graphs, counts, keep = [], [], []
        for i in range(n_inputs):
            x = synthetic.activations(shape, rows, dev, index=i)
            for ex in layers:
                buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
                scratch = x3.Scratch(ex, rows, shape.top_k, device=dev)
                out = torch.empty((rows, shape.dims), dtype=torch.float32, device=dev)

                def step(x=x, ex=ex, buf=buf, scratch=scratch, out=out):
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
                counts.append(scratch.count)
                keep.append((x, buf, scratch, out))
        ms, all_ms = timed(torch, lambda i: graphs[i % len(graphs)].replay(), steps, warmup, repeats_for(steps))
        distinct = statistics.mean(int(c[0]) for c in counts)
        nbytes = distinct * per_expert + shape.experts * shape.dims * 2 + rows * shape.dims * (2 + 4)
        results.append({"form": "exl3 4.00 bpw (config 3)", "rows": rows, "ms_per_step": ms, **spread(all_ms),
                        "tokens_per_s": rows / (ms * 1e-3), "distinct_experts": distinct,
                        "rotation": f"{len(layers)} weight copies x {n_inputs} token batches", "layer_bytes": nbytes,
                        "layer_gbs": nbytes / (ms * 1e-3) / 1e9, "layer_frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm,
                        "launches_per_step": x3.LAUNCHES_PER_CALL + 2})
        del graphs, keep
    return results


def bench_reference_cuda(torch, rows_list, steps: int, warmup: int):
    """The reference's OWN CUDA kernels for the grouped experts (its experts.cu / experts_prefill.cu / experts_pack.cu
    compiled unmodified for sm_100 by oracle/build_ref_cuda.py) beside this library's, on this GPU, with the same
    method: plan + gate/up + down of config 2's layer (bf16 scales, the reference's convention) in a CUDA graph, two
    weight copies alternating.  Router, top-k and combine are left out on both sides (the reference's are Triton
    kernels of its Python package, which does not travel).  None when the module was never built."""

    from oracle import build_ref_cuda
    from tensorfold_b200 import experts, moe, synthetic

    ref = build_ref_cuda.load()
    if ref is None:
        return None
    shape, dev = synthetic.C2, torch.device("cuda", torch.cuda.current_device())
    kg_up, nb_up, kg_dn, nb_dn = shape.dims // 64, shape.width // 32, shape.width // 64, shape.dims // 32
    ours, theirs = [], []
    for copy in range(2):
        gate, up, down = synthetic.affine_layer(shape, dev, torch.bfloat16, copy=copy)

        def ref_pack(m):
            e, n, k8 = m[0].shape
            out = torch.empty((e, n // 32, k8 * 8 // 64, 288), dtype=torch.int32, device=dev)
            ref.pack(m[0].contiguous(), m[1].contiguous(), m[2].contiguous(), 64, out)
            return out

        theirs.append((torch.stack([ref_pack(gate), ref_pack(up)], dim=3).contiguous(),
                       ref_pack(down).unsqueeze(3).contiguous()))
        ours.append(experts.make([gate, up], down, 64))
        del gate, up, down
    router = synthetic.router_rows(shape, dev)
    layer = moe.Routed(router, ours[0], shape.top_k, shared=False)
    out = []
    for rows in rows_list:
        prefill = rows >= 1024
        x = synthetic.activations(shape, rows, dev)
        buf = moe.MoEBuffers(rows, moe._Shape(layer), dev, shared=False, prefill=prefill)
        moe.router(x, router, buf.logits[:rows])
        moe.select_rows(buf.logits[:rows], buf, shape.top_k, shape.experts)
        picks, pairs = buf.pick[:rows].contiguous(), rows * shape.top_k
        tile = 64 if prefill else 16
        r_members = torch.zeros((pairs,), dtype=torch.int32, device=dev)
        r_items = torch.zeros((min(pairs, shape.experts) + pairs // 16, 3), dtype=torch.int32, device=dev)
        r_counts = torch.zeros((2,), dtype=torch.int32, device=dev)
        r_rank = torch.zeros((pairs,), dtype=torch.int32, device=dev)
        r_hist = torch.zeros((-(-pairs // 1024) * shape.experts,), dtype=torch.int32, device=dev)
        r_items_n = min(pairs, shape.experts) + pairs // tile
        act = torch.zeros((pairs, shape.width), dtype=torch.bfloat16, device=dev)
        y = torch.zeros((pairs, shape.dims), dtype=torch.bfloat16 if prefill else torch.float32, device=dev)
        plan = experts.Plan(rows, shape.top_k, shape.experts, dev, prefill=prefill)

        def step_ref(w):
            ref.plan(picks, pairs, shape.experts, tile, r_members, r_items, r_counts, r_rank, r_hist)
            if prefill:
                ref.prefill(64, 2, x, shape.top_k, w[0], kg_up, nb_up, r_items, r_counts, r_members, act, shape.width,
                            0.0, r_items_n)
                ref.prefill(64, 3, act, 0, w[1], kg_dn, nb_dn, r_items, r_counts, r_members, y, shape.dims, 0.0,
                            r_items_n)
            else:
                ref.run(64, 2, x, shape.top_k, w[0], kg_up, nb_up, r_items, r_counts, r_members, act, shape.width, 0.0,
                        r_items_n * nb_up)
                ref.run(64, 0, act, 0, w[1], kg_dn, nb_dn, r_items, r_counts, r_members, y, shape.dims, 0.0,
                        r_items_n * nb_dn)

        def step_ours(ex):
            experts.route(picks, plan)
            experts.gate_up(x, ex, plan, act, rows)
            experts.down(act, ex, plan, y, rows)

        times = {}
        for name, step, sets in (("reference", step_ref, theirs), ("ours", step_ours, ours)):
            graphs = []
            for w in sets:
                step(w)
                torch.cuda.synchronize()
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream())
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step(w)
                graphs.append(g)
            ms, _ = timed(torch, lambda i: graphs[i % len(graphs)].replay(), steps, warmup, 5)
            times[name] = ms * 1e3
        out.append({"rows": rows, "form": "prefill" if prefill else "decode",
                    "reference_kernels_us": times["reference"], "these_kernels_us": times["ours"],
                    "speedup": times["reference"] / times["ours"]})
    del ours, theirs
    torch.cuda.empty_cache()
    return {"what": "plan + gate/up + down of config 2's layer with bf16 scales, CUDA graph, two weight copies; the "
                    "reference's experts.cu / experts_prefill.cu compiled unmodified for sm_100 against this library",
            "lines": out, "exl3": bench_reference_exl3(torch, (1, 64), steps, warmup)}


def bench_reference_exl3(torch, rows_list, steps: int, warmup: int):
    """The reference's own EXL3 expert kernels (its exl3/experts*.cu compiled unmodified for sm_100) beside this
    library's on config 3's layer (4.00 bits a weight): the whole ``routed`` call with the weighted combine, in a CUDA
    graph, two weight copies alternating, the same picks on both sides.  None when the module was never built."""

    from oracle import build_ref_cuda
    from oracle import ref_exl3 as drive
    from tensorfold_b200 import moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    ext = build_ref_cuda.load("exl3")
    if ext is None:
        return None
    shape, dev = synthetic.C3, torch.device("cuda", torch.cuda.current_device())
    router = synthetic.router_rows(shape, dev)
    layers = [x3.prepare(*synthetic.exl3_layer(shape, dev, 4, copy=c), x3.CB_3INST, device=dev) for c in range(2)]

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    out = []
    for rows in rows_list:
        x = synthetic.activations(shape, rows, dev)
        buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
        moe.router(x, router, buf.logits[:rows])
        moe.select_rows(buf.logits[:rows], buf, shape.top_k, shape.experts)
        pick, wts = buf.pick[:rows].contiguous(), buf.wts[:rows].contiguous()
        res = torch.zeros((rows, shape.dims), dtype=torch.float32, device=dev)
        times = {}
        for name in ("reference", "ours"):
            graphs, keep = [], []
            for ex in layers:
                s = drive.Scratch(ex, rows, shape.top_k, dev) if name == "reference" else x3.Scratch(ex, rows, shape.top_k,
                                                                                                   device=dev)
                step = ((lambda ex=ex, s=s: drive.routed(ext, x, pick, wts, ex, s, res)) if name == "reference" else
                        (lambda ex=ex, s=s: x3.routed(x, pick, wts, ex, s, res, rows)))
                step()
                torch.cuda.synchronize()
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream())
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step()
                graphs.append(g)
                keep.append(s)
            ms, _ = timed(torch, lambda i: graphs[i % len(graphs)].replay(), steps, warmup, 5)
            times[name] = ms * 1e3
        out.append({"rows": rows, "reference_kernels_us": times["reference"], "these_kernels_us": times["ours"],
                    "speedup": times["reference"] / times["ours"]})
    return {"what": "the routed EXL3 call (grouping, rotations, both projections, weighted combine) of config 3's "
                    "layer at 4.00 bits a weight, CUDA graph, two weight copies", "lines": out}


def bench_e2e(torch, runners, shape, rows: int, steps: int, warmup: int):
    """The same step through the public API with HOST buffers: pinned tokens in, layer, result back, every step."""

    from tensorfold_b200 import synthetic

    x_host = synthetic.activations(shape, rows, "cpu").pin_memory()
    out_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    for r in runners:
        r.bind_host(x_host, out_host)                           # the copies become nodes of the step's graph
    ms, all_ms = timed(torch, lambda i: runners[i % len(runners)].replay_host(), steps, warmup, repeats_for(steps),
                       sync_each=True)                          # the caller reads the result before the next step
    nbytes = rows * shape.dims * 2
    return {"value": rows / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, **spread(all_ms),
            "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}


# ---- expert parallelism ---------------------------------------------------------------------------------------------

COLLECTIVE = {
    "tokens": "NCCL all-gather of the tokens, reduce-scatter of fp32 per-token partial sums",
    "rows": "NCCL all-gather of the tokens, reduce-scatter of fp32 per-pair rows (exact)",
    "peer": "own kernels over NVLink peer memory: pull of the tokens, push of fp32 per-token partial sums, two flag "
            "barriers (no collective library on the step)",
}


C4_HOT_PAIRS = 32        # config 4: a rank's experts with at least this many pairs go through the prompt-form kernel


def hot_pairs_for(config: str, asked: int) -> int:
    """`--hot-pairs` when given; else the split plan for config 4's skewed routing (measured: 1643 -> 1424 us on one
    GPU, 599 -> 503 us on four) and the plain plan for config 2's uniform routing."""

    return asked if asked >= 0 else (C4_HOT_PAIRS if config == "c4" else 0)


def ep_rows(config: str, rows: int, world: int) -> int:
    """Rows a rank: config 2 keeps `--rows` a GPU (weak scaling); config 4 splits its 256 tokens over the ranks."""

    return 256 // world if config == "c4" else rows


def ep_copies(config: str, world: int) -> int:
    """Independent weight copies a rank rotates so that a step's weights never sit in the 126 MB L2."""

    return 2 if config == "c4" else 2 * world              # a config-4 slice is 5.4 GB / world


def all_ok(torch, dist, ok: bool, value: float):
    """(every rank's ok, the largest value over the ranks)."""

    t = torch.tensor([0.0 if ok else 1.0, value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t[0].item() == 0.0, t[1].item()


def one_gpu_layer(torch, x, router, full, shape, bias):
    """The plain one-GPU layer on `x` (the same kernels, no exchange): (out bf16, pick)."""

    from tensorfold_b200 import experts, moe

    layer = moe.Routed(router, full, shape.top_k, shared=shape.shared)
    rows = x.shape[0]
    buf = moe.MoEBuffers(rows, moe._Shape(layer), x.device, shared=shape.shared)
    moe.router(x, router, buf.logits[:rows])
    if bias is not None:
        buf.logits[:rows, :shape.experts] += bias
    moe.select(buf.logits[:rows], buf, shape.top_k, shape.experts)
    experts.gate_up(x, full, buf.plan, buf.act.view(-1, full.width), rows)
    experts.down(buf.act.view(-1, full.width), full, buf.plan, buf.y.view(-1, full.dims), rows)
    return moe.combine(buf.y[:rows], buf.wts[:rows]), buf.pick[:rows].clone()


def bench_rank_slice(torch, args, config: str, shape, dev, hbm: float) -> dict:
    """One GPU doing what rank `--slice-rank` of an `--as-rank-of N` group does between its two exchanges, for profiling
    that regime under ncu (never wrap a multi-rank run in ncu): the rank's E / N experts, the tokens of all ranks routed
    over all experts (config 2: 64 a rank; config 4: its 256 tokens, Zipf-skewed), the plan over the rank's expert
    window (`--hot-pairs`: the split plan), gate/up and down.  The slice's weight copies rotate so every step reads
    DRAM.  Times the expert launches together and gate/up alone."""

    from tensorfold_b200 import _lib, experts, moe, synthetic

    n, r = args.as_rank_of, args.slice_rank
    rows = 256 if config == "c4" else (args.rows or 64) * n
    per = shape.experts // n
    router = synthetic.router_rows(shape, dev)
    x = synthetic.activations(shape, rows, dev, index=100)

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
    moe.router(x, router[:shape.experts], buf.logits)
    if config == "c4":
        buf.logits.add_(synthetic.zipf_bias(shape, 1.1, dev))
    moe.select_rows(buf.logits, buf, shape.top_k, shape.experts)
    pick = buf.pick.contiguous()
    wide = rows * shape.top_k >= 24 * shape.experts              # the expert-parallel step's own rule for items of 16
    hot = hot_pairs_for(config, args.hot_pairs)
    plan = experts.Plan(rows, shape.top_k, per, dev, decode_tile=experts.WIDE_TILE if wide else experts.TILE, hot=hot)
    plan.tile = plan.decode_tile
    st = torch.cuda.current_stream(dev).cuda_stream
    if hot:
        experts.route_split(pick, plan, r * per)
    else:
        _lib.call("tfb_plan_window", pick.data_ptr(), rows * shape.top_k, r * per, per, plan.tile,
                  plan.members.data_ptr(), plan.items.data_ptr(), plan.counts.data_ptr(), st)
    torch.cuda.synchronize()
    mine = pick[(pick >= r * per) & (pick < (r + 1) * per)] - r * per
    counts = torch.bincount(mine.long(), minlength=per)
    slices = []
    for copy in range(2 if config == "c4" else 2 * n):            # as a rank of the group does
        gate, up, down = synthetic.affine_layer(shape, dev, torch.float16 if args.scales == "fp16" else torch.bfloat16,
                                                copy=copy)
        cut = slice(r * per, (r + 1) * per)
        slices.append(experts.make([tuple(t[cut].contiguous() for t in gate), tuple(t[cut].contiguous() for t in up)],
                                   tuple(t[cut].contiguous() for t in down), 64))
        del gate, up, down
    act = torch.zeros((rows * shape.top_k, shape.width), dtype=torch.bfloat16, device=dev)
    y = torch.zeros((rows * shape.top_k, shape.dims), dtype=torch.float32, device=dev)

    def graph_of(body):
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            body()
        return g

    def both():
        for ex in slices:
            experts.gate_up(x, ex, plan, act, rows)
            experts.down(act, ex, plan, y, rows)

    def first():
        for ex in slices:
            experts.gate_up(x, ex, plan, act, rows)

    both()
    torch.cuda.synchronize()
    g_both, g_first = graph_of(both), graph_of(first)
    k = len(slices)
    ms_both, _ = timed(torch, lambda i: g_both.replay(), max(args.steps // k, 3), args.warmup, 5)
    ms_first, _ = timed(torch, lambda i: g_first.replay(), max(args.steps // k, 3), args.warmup, 5)
    nbytes = int((counts > 0).sum()) * slices[0].bytes_per_expert()
    return {"as_rank_of": n, "rank": r, "config": config, "experts": per, "experts_in_use": int((counts > 0).sum()),
            "tokens": rows, "pairs_in_window": int(counts.sum()), "most_pairs_an_expert": int(counts.max()),
            "items_of": plan.tile, "hot_pairs": hot, "weight_copies": k, "slice_bytes": nbytes,
            "gate_up_plus_down_us": ms_both / k * 1e3, "gate_up_us": ms_first / k * 1e3,
            "frac_of_hbm": nbytes / (ms_both / k * 1e-3) / 1e9 / hbm,
            "gate_up_frac_of_hbm": nbytes * 2 / 3 / (ms_first / k * 1e-3) / 1e9 / hbm}


def bench_rank_slice_c5(torch, args, dev, hbm: float) -> dict:
    """`--as-rank-of N --config c5`: one GPU running the routed EXL3 call of rank `--slice-rank` of an N-rank group for
    layer 0 of config 5 (its 160 / N experts at their seeded mixed widths, the `--rows` tokens (128 unless given) of all
    ranks routed over all experts, the selections renumbered to the rank's window), for profiling under ncu.
    `--one-width B` gives every tensor B bits instead (the comparison that shows what the mix of widths costs)."""

    from tensorfold_b200 import _lib, moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape = synthetic.C5
    n, r, rows = args.as_rank_of, args.slice_rank, args.rows or 128
    per = shape.experts // n
    widths = c5_widths()
    if args.one_width:
        widths = {key: args.one_width for key in widths}
    mine = list(range(r * per, (r + 1) * per))
    g, u, d = c5_experts(torch, dev, 0, mine, widths)
    ex = x3.prepare(g, u, d, x3.CB_3INST, device=dev)
    router = synthetic.router_rows(shape, dev)
    x = synthetic.activations(shape, rows, dev, index=100)

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
    moe.router(x, router, buf.logits)
    moe.select_rows(buf.logits, buf, shape.top_k, shape.experts)
    pick = torch.zeros((rows, shape.top_k), dtype=torch.int32, device=dev)
    wts = torch.zeros((rows, shape.top_k), dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    _lib.call("tfb_window_picks", buf.pick.data_ptr(), buf.wts.data_ptr(), r * per, per, pick.data_ptr(), wts.data_ptr(),
              rows * shape.top_k, st)
    scratch = x3.Scratch(ex, rows, shape.top_k, device=dev)
    scratch.y.zero_()
    out = torch.zeros((rows, shape.dims), dtype=torch.float32, device=dev)

    def call():
        x3.routed(x, pick, wts, ex, scratch, out, rows, share=per / shape.experts)

    call()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        call()
    ms, _ = timed(torch, lambda i: graph.replay(), max(args.steps, 3), args.warmup, 5)
    in_window = int((pick < per).sum())
    nbytes = ex.nbytes_read(sorted(set(pick[pick < per].tolist())))
    return {"as_rank_of": n, "rank": r, "config": "c5", "experts": per, "tokens": rows, "pairs_in_window": in_window,
            "widths": f"{args.one_width} bits every tensor" if args.one_width else "seeded 2..8 bits a tensor",
            "trellis_bytes": nbytes, "routed_call_us": ms * 1e3, "frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm}


def bench_ep(torch, dist, args, config: str, shape, dev, rank: int, world: int) -> dict:
    """Expert-parallel step of the affine layer: this rank's rows through the layer whose experts are sharded over the
    ranks.  Each rank keeps several copies of its expert slice and rotates them, so a step's weights never sit in L2.
    Before the clock starts every rank compares its output with the one-GPU layer on the same rows ("ep_check")."""

    from tensorfold_b200 import _lib, ep, experts, synthetic

    rows, per = ep_rows(config, args.rows, world), shape.experts // world
    reduce = args.ep_reduce
    router = synthetic.router_rows(shape, dev)
    bias = synthetic.zipf_bias(shape, 1.1, dev) if config == "c4" else None
    x = synthetic.activations(shape, rows, dev, index=100 + rank)
    copies, graphs, check = [], [], None
    for copy in range(ep_copies(config, world)):
        gate, up, down = synthetic.affine_layer(shape, dev, torch.float16 if args.scales == "fp16" else torch.bfloat16,
                                                copy=copy)

        def cut(which):
            return experts.make([tuple(t[which].contiguous() for t in gate), tuple(t[which].contiguous() for t in up)],
                                tuple(t[which].contiguous() for t in down), 64)

        local = cut(slice(rank * per, (rank + 1) * per))
        if reduce == "peer":
            shared = cut(slice(shape.experts, shape.experts + 1)) if shape.shared else None
            layer = ep.PeerExpertParallel(router, local, shape.experts, shape.top_k, rows, shared_experts=shared,
                                          logit_bias=bias, hot_pairs=hot_pairs_for(config, args.hot_pairs))
        else:
            layer = ep.GatheredExpertParallel(router, local, shape.experts, shape.top_k, rows, reduce=reduce)
        copies.append(layer)
        if copy == 0:
            # correctness before speed: this rank's rows through the expert-parallel step and through the whole layer
            # on this GPU alone (every rank holds all experts of copy 0 for the moment)
            full = experts.make([gate, up], down, 64)
            got = layer.forward(x).clone()
            want, pick = one_gpu_layer(torch, x, router, full, shape, bias)
            mine = layer.win.pick_mine if reduce == "peer" else layer.buf.pick[rank * rows:(rank + 1) * rows]
            same = bool(torch.equal(mine[:, :pick.shape[1]], pick))
            err = rel_l2(torch, got, want)
            torch.cuda.synchronize()
            status = _lib.kernel_status()
            ok, worst = all_ok(torch, dist, same and err <= TOL and status == 0, err)
            check = {"picks_equal": ok or same, "rel_l2": worst, "tolerance": TOL, "rows_per_rank": rows,
                     "against": "the one-GPU layer (same kernels, all experts on one GPU) on each rank's own rows",
                     "passed": ok}
            if not ok:
                raise SystemExit(f"expert-parallel output differs from the one-GPU layer on rank {rank}: picks equal "
                                 f"{same}, rel-L2 {err:.3e}, device status {_lib.describe_status(status)}")
            del full, got, want
        del gate, up, down
    side = torch.cuda.Stream(dev)
    if reduce == "peer":                                       # the tokens live in each copy's window; nothing to stage
        for layer in copies:
            layer.tokens.copy_(x)
        steps = [layer.forward for layer in copies]
    else:
        steps = [(lambda layer=layer: layer.forward(x)) for layer in copies]
    for step in steps:                                         # warm up eagerly (NCCL set-up), then capture the step
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
    k = args.steps if config == "c2" else min(args.steps, 20)
    ms, all_ms = timed(torch, lambda i: graphs[i % len(graphs)].replay(), k, args.warmup,
                       repeats_for(k) if config == "c2" else 5, dist)
    # end to end: pinned host tokens in, result back, every step
    x_host = x.cpu().pin_memory()
    out_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()
    dist.barrier()
    host_graphs = []
    for step, layer in zip(steps, copies):                     # the same step with its host transfers inside the graph
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            if reduce == "peer":                               # kernels read the pinned rows and store the pinned result
                layer.forward(x_host, out_host)
            else:
                x.copy_(x_host, non_blocking=True)
                step()
                out_host.copy_(layer.out, non_blocking=True)
        host_graphs.append(g)
    torch.cuda.synchronize()
    dist.barrier()
    e2e_ms, e2e_all = timed(torch, lambda i: host_graphs[i % len(host_graphs)].replay(), k, min(args.warmup, 4),
                            repeats_for(k) if config == "c2" else 5, dist, sync_each=True)
    torch.cuda.synchronize()
    status = _lib.kernel_status()
    if status != 0:
        raise SystemExit(f"a kernel recorded a failure on rank {rank}: {_lib.describe_status(status)}")
    # this rank's algorithmic bytes a step: its touched experts' packed weights, the router rows, its tokens in and out
    layer = copies[0]
    nbytes = router.numel() * 2 + 2 * rows * shape.dims * 2
    pairs = 0
    if reduce == "peer":
        w = layer.win
        mine = w.pick_all[:, :shape.top_k].reshape(-1)
        mine = mine[(mine >= w.lo) & (mine < w.lo + w.per_rank)]
        pairs = int(mine.numel())
        nbytes += int(torch.unique(mine).numel()) * local.bytes_per_expert()
        if shape.shared:
            nbytes += local.bytes_per_expert()
    else:
        nbytes += per * local.bytes_per_expert()
    per_rank = torch.zeros((world, 2), device=dev, dtype=torch.float64)
    per_rank[rank, 0], per_rank[rank, 1] = nbytes, pairs
    dist.all_reduce(per_rank)
    return {"ms": ms, "all_ms": all_ms, "e2e_ms": e2e_ms, "e2e_all": e2e_all, "launches": layer.launches, "rows": rows,
            "rank_bytes": [int(v) for v in per_rank[:, 0].tolist()], "rank_pairs": [int(v) for v in per_rank[:, 1].tolist()],
            "check": check, "steps": k, "reduce": reduce,
            "hot_pairs": hot_pairs_for(config, args.hot_pairs) if reduce == "peer" else 0}


def c5_widths() -> dict:
    """Config 5's seeded width (2..8 bits) of every (layer, expert, matrix); every rank draws them in the same order."""

    import random

    from tensorfold_b200 import synthetic

    rng = random.Random(5005)
    return {(li, e, m): rng.choice((2, 3, 4, 5, 6, 7, 8)) for li in range(C5_LAYERS)
            for e in range(synthetic.C5.experts) for m in range(3)}


def c5_experts(torch, dev, li: int, ids, widths):
    """The EXL3 experts `ids` of layer `li` (per-expert triples for gate, up, down)."""

    from tensorfold_b200 import synthetic

    shape = synthetic.C5
    base = 1000 * shape.config + 10 + 1000003 * li
    gate, up, down = [], [], []
    for e in ids:
        gate.append(synthetic.exl3_matrix(base + 3 * e, shape.dims, shape.width, widths[(li, e, 0)], dev))
        up.append(synthetic.exl3_matrix(base + 3 * e + 1, shape.dims, shape.width, widths[(li, e, 1)], dev))
        down.append(synthetic.exl3_matrix(base + 3 * e + 2, shape.width, shape.dims, widths[(li, e, 2)], dev))
    return gate, up, down


def bench_c5(torch, dist, args, dev, rank: int, world: int, hbm: float) -> dict:
    """Config 5 on the expert-parallel EXL3 path: 8 layers (hidden 4096, 160 experts x FFN 1536, top-8, a seeded width
    of 2..8 bits a tensor), `h = bf16(h + moe(h))` between layers, at 1, 8, 32, 128 and 512 tokens split over the ranks
    (a batch smaller than the rank count leaves the last ranks without a token; they still serve their experts).
    One step = the 8-layer stack in one CUDA graph; 16 seeded token batches rotate (a small copy in front of the graph)
    so the experts change every step.  Before timing, every layer of the stack is compared with the one-GPU layer on
    the same input ("ep_check")."""

    from tensorfold_b200 import _lib, ep, moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape = synthetic.C5
    per = shape.experts // world
    widths = c5_widths()
    router = synthetic.router_rows(shape, dev)
    mine = list(range(rank * per, (rank + 1) * per))
    local = [x3.prepare(*c5_experts(torch, dev, li, mine, widths), x3.CB_3INST, device=dev) for li in range(C5_LAYERS)]

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    def build(tokens):
        rows = max(1, math.ceil(tokens / world))
        active = max(0, min(rows, tokens - rank * rows))
        layers = [ep.PeerExl3ExpertParallel(router, ex, shape.experts, shape.top_k, rows, rows_active=active)
                  for ex in local]
        return rows, active, layers

    def stack(layers, src, h_out, each=None):
        """The 8 layers with h = bf16(h + layer(h)) between them.  Timed form (no `each`): the kernel that adds the
        ranks' shares also adds the residual row and rounds.  Checked form: the layer's fp32 output is handed to
        `each`, the residual add is torch's - the same arithmetic, and the two forms' results are compared below."""

        h = src
        for li, layer in enumerate(layers):
            if each is None:
                h = layer.forward(h, residual=True)               # bf16 [rows, D]
                continue
            y = layer.forward(h)                                  # fp32 [rows, D]
            if li == 0:
                h = layer.tokens                                  # the staged rows (src may be pinned host memory)
            each(li, h, y)
            h = (h.float() + y).to(torch.bfloat16)                # the residual add between layers
        h_out.copy_(h)

    # ---- correctness first: 32 tokens, every layer against the one-GPU layer on the same input ----
    rows, active, layers = build(32)
    x = torch.zeros((rows, shape.dims), dtype=torch.bfloat16, device=dev)
    x[:active] = synthetic.activations(shape, rows, dev, index=100 + rank)[:active]
    worst, same = 0.0, True

    def compare(li, h, y):
        nonlocal worst, same
        if active == 0:
            return
        full = x3.prepare(*c5_experts(torch, dev, li, range(shape.experts), widths), x3.CB_3INST, device=dev)
        buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
        moe.router(h[:active], router, buf.logits[:active])
        moe.select_rows(buf.logits[:active], buf, shape.top_k, shape.experts)
        want = x3.routed(h[:active], buf.pick[:active].contiguous(), buf.wts[:active].contiguous(), full,
                         x3.Scratch(full, active, shape.top_k, device=dev), None, active)
        same = same and bool(torch.equal(layers[li].win.pick_mine[:active], buf.pick[:active]))
        worst = max(worst, rel_l2(torch, y[:active], want))
        del full

    h_chk, h_fused = torch.zeros_like(x), torch.zeros_like(x)
    stack(layers, x, h_chk, compare)
    stack(layers, x, h_fused)                                     # the timed form: residual inside the last kernel
    torch.cuda.synchronize()
    status = _lib.kernel_status()
    same = same and bool(torch.equal(h_fused[:active], h_chk[:active]))
    ok, worst_all = all_ok(torch, dist, same and worst <= TOL and status == 0, worst)
    check = {"picks_equal": ok or same, "rel_l2": worst_all, "tolerance": TOL, "tokens": 32, "layers": C5_LAYERS,
             "against": "the one-GPU EXL3 layer on the same layer input, every layer of the stack", "passed": ok}
    if not ok:
        raise SystemExit(f"config 5: expert-parallel stack differs from the one-GPU layers on rank {rank}: picks "
                         f"equal {same}, rel-L2 {worst:.3e}, device status {_lib.describe_status(status)}")
    del layers
    # ---- the sweep ----
    lines = []
    for tokens in C5_TOKENS:
        rows, active, layers = build(tokens)
        batches = []
        for i in range(16):
            xb = torch.zeros((rows, shape.dims), dtype=torch.bfloat16, device=dev)
            xb[:active] = synthetic.activations(shape, rows, dev, index=200 + 16 * rank + i)[:active]
            batches.append(xb)
        x_in, h_out = batches[0].clone(), torch.zeros_like(batches[0])
        stack(layers, x_in, h_out)
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            stack(layers, x_in, h_out)
        x_host = [b.cpu().pin_memory() for b in batches[:4]]
        x_pin = torch.empty_like(x_host[0]).pin_memory()
        out_host = torch.empty((rows, shape.dims), dtype=torch.bfloat16).pin_memory()
        side.wait_stream(torch.cuda.current_stream())
        host_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(host_graph, stream=side):
            stack(layers, x_pin, h_out)
            out_host.copy_(h_out, non_blocking=True)
        torch.cuda.synchronize()
        dist.barrier()

        def step(i):
            x_in.copy_(batches[i % len(batches)], non_blocking=True)
            graph.replay()

        def host_step(i):
            x_pin.copy_(x_host[i % len(x_host)])                  # the caller fills its pinned buffer
            host_graph.replay()

        k = min(args.steps, 10)
        ms, all_ms = timed(torch, step, k, 3, 5, dist)
        e2e_ms, _ = timed(torch, host_step, k, 2, 3, dist, sync_each=True)
        # bytes of the last step on this rank: trellises and scales of the experts its layers touched
        nbytes = C5_LAYERS * router.numel() * 2 + 2 * active * shape.dims * 2
        for layer in layers:
            w = layer.win
            sel = w.pick_all.reshape(-1)
            sel = torch.unique(sel[(sel >= w.lo) & (sel < w.lo + w.per_rank)]) - w.lo
            nbytes += layer.local.nbytes_read(sel.cpu().tolist())
        per_rank = torch.zeros((world,), device=dev, dtype=torch.float64)
        per_rank[rank] = nbytes
        dist.all_reduce(per_rank)
        rb = [int(v) for v in per_rank.tolist()]
        launches = sum(layer.launches + 1 for layer in layers) + 2    # each layer stages its rows; two copies a step
        lines.append({"tokens": tokens, "rows_per_rank": rows, "ms_per_step": ms, **spread(all_ms),
                      "tokens_per_s": tokens / (ms * 1e-3), "e2e_ms_per_step": e2e_ms,
                      "e2e_tokens_per_s": tokens / (e2e_ms * 1e-3), "steps": k, "launches_per_step": launches,
                      "rank_bytes_max": max(rb), "rank_bytes_sum": sum(rb),
                      "slowest_rank_frac_of_hbm": max(rb) / (ms * 1e-3) / 1e9 / hbm,
                      "all_ranks_frac_of_hbm": sum(rb) / world / (ms * 1e-3) / 1e9 / hbm})
        status = _lib.kernel_status()
        if status != 0:
            raise SystemExit(f"config 5: a kernel recorded a failure on rank {rank}: {_lib.describe_status(status)}")
        del layers, graph, host_graph
        torch.cuda.empty_cache()
    return {"config": workload_config(shape, 0, world, "c5") | {"tokens": list(C5_TOKENS)}, "dtype": "f16",
            "scaling": "strong", "n_gpus": world, "sweep": lines, "ep_check": check}


def ep_summary(res: dict, shape, config: str, world: int, hbm: float, which: str) -> dict:
    """The fields of one expert-parallel affine run (configs 2 and 4) that go into the JSON line."""

    ms, rows = res["ms"], res["rows"]
    rb = res["rank_bytes"]
    return {"config": {**workload_config(shape, rows, world, config),
                       "l2": f"each rank rotates {ep_copies(config, world)} copies of its {shape.experts // world}-expert "
                             "slice (inputs larger than the 126 MB L2)",
                       "collective": COLLECTIVE[res["reduce"]] + "; the step is one CUDA graph",
                       "hot_pairs": res.get("hot_pairs", 0)},
            "scaling": "weak" if config == "c2" else "strong", "n_gpus": world, "steps": res["steps"],
            "ms_per_step": ms, **spread(res["all_ms"]), "tokens_per_s": world * rows / (ms * 1e-3),
            "e2e_ms_per_step": res["e2e_ms"], "e2e_tokens_per_s": world * rows / (res["e2e_ms"] * 1e-3),
            "launches_per_step": res["launches"], "rank_bytes": rb, "rank_pairs": res["rank_pairs"],
            "pairs_per_rank_min": min(res["rank_pairs"]), "pairs_per_rank_max": max(res["rank_pairs"]),
            "rank0_frac_of_hbm": rb[0] / (ms * 1e-3) / 1e9 / hbm,
            "slowest_rank_frac_of_hbm": max(rb) / (ms * 1e-3) / 1e9 / hbm,
            "all_ranks_frac_of_hbm": sum(rb) / world / (ms * 1e-3) / 1e9 / hbm, "peak_source": f"of {which}",
            "ep_check": res["check"]}


def guarded(name: str, fn, torch, dist) -> dict:
    """Run one of the extra workloads; a failure becomes an "error" entry instead of losing the headline line."""

    try:
        return fn()
    except (Exception, SystemExit) as err:                     # noqa: BLE001
        print(f"[bench] {name} failed: {err!r}", file=sys.stderr)
        return {"error": repr(err)}


def run_ours(args) -> None:
    import torch

    from tensorfold_b200 import _lib, experts, moe, synthetic

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU fallback (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import datetime

    import torch.distributed as dist

    if world == 1:                                     # not under torchrun: a group of one
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev, timeout=datetime.timedelta(seconds=180))
    else:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    hbm, tflops, which = peaks()
    _lib.set_pdl(bool(args.pdl))
    if args.exl3_only:
        print(json.dumps({"sweep": bench_exl3(torch, args.exl3_rows, args.steps, args.warmup, hbm)}))
        dist.destroy_process_group()
        return
    if args.as_rank_of:
        shape = {"c2": synthetic.C2, "c4": synthetic.C4, "c5": synthetic.C5}[args.config]
        if world != 1 or shape.experts % args.as_rank_of or not 0 <= args.slice_rank < args.as_rank_of:
            raise SystemExit("--as-rank-of N runs on one GPU, N a divisor of the expert count")
        if args.config == "c5":
            print(json.dumps(bench_rank_slice_c5(torch, args, dev, hbm)))
        else:
            print(json.dumps(bench_rank_slice(torch, args, args.config, shape, dev, hbm)))
        dist.destroy_process_group()
        return
    shapes = {"c2": synthetic.C2, "c4": synthetic.C4, "c5": synthetic.C5}
    if args.config != "c2" and args.ep_reduce != "peer":
        raise SystemExit(f"--config {args.config} runs the peer-memory form")
    for s in shapes.values():
        if s.experts % world:
            raise SystemExit(f"{s.experts} experts do not shard over {world} ranks")

    extras = {}

    def run_extras():
        if args.no_extra:
            return
        torch.cuda.empty_cache()
        extras["c4"] = guarded("config 4", lambda: ep_summary(
            bench_ep(torch, dist, args, "c4", synthetic.C4, dev, rank, world), synthetic.C4, "c4", world, hbm, which),
            torch, dist)
        torch.cuda.empty_cache()
        extras["c5"] = guarded("config 5", lambda: bench_c5(torch, dist, args, dev, rank, world, hbm), torch, dist)
        torch.cuda.empty_cache()

    if world > 1 or args.config in ("c4", "c5"):
        # ---- the expert-parallel path is the headline ----
        with ClockSampler(local) as clocks:
            if args.config == "c5":
                c5 = bench_c5(torch, dist, args, dev, rank, world, hbm)
            else:
                res = bench_ep(torch, dist, args, args.config, shapes[args.config], dev, rank, world)
        if args.config == "c2":
            run_extras()
        if rank == 0:
            if args.config == "c5":
                top = next(l for l in c5["sweep"] if l["tokens"] == 128)
                line = {"metric": METRIC, "value": top["tokens_per_s"], "unit": UNIT, "n_gpus": world,
                        "steps": top["steps"], "warmup": 3, "ms_per_step": top["ms_per_step"],
                        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                        "data": "synthetic", "config": workload_config(synthetic.C5, 128, world, "c5"),
                        "clocks": clocks.summary(),
                        "e2e": {"value": top["e2e_tokens_per_s"], "unit": UNIT, "ms_per_step": top["e2e_ms_per_step"],
                                "h2d_bytes_per_step": 128 * synthetic.C5.dims * 2,
                                "d2h_bytes_per_step": 128 * synthetic.C5.dims * 2},
                        "gpu_launches": top["launches_per_step"] * top["steps"],
                        "roofline": {"bound": "hbm", "kernel": "the 8-layer expert-parallel EXL3 step (slowest rank)",
                                     "achieved": top["rank_bytes_max"] / (top["ms_per_step"] * 1e-3) / 1e9,
                                     "peak": hbm, "unit": "GB/s", "frac": top["slowest_rank_frac_of_hbm"],
                                     "peak_source": f"of {which}", "traffic": None},
                        "cpu_baseline": None, "ep_check": c5["ep_check"], "c5": c5}
            else:
                shape = shapes[args.config]
                s = ep_summary(res, shape, args.config, world, hbm, which)
                nbytes = res["rows"] * shape.dims * 2 * world
                line = {"metric": METRIC, "value": s["tokens_per_s"], "unit": UNIT, "n_gpus": world,
                        "steps": res["steps"], "warmup": args.warmup, "ms_per_step": res["ms"],
                        **spread(res["all_ms"]), "higher_is_better": True, "scaling": s["scaling"],
                        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                        "config": s["config"], "clocks": clocks.summary(),
                        "e2e": {"value": s["e2e_tokens_per_s"], "unit": UNIT, "ms_per_step": res["e2e_ms"],
                                "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes},
                        "gpu_launches": res["launches"] * res["steps"],
                        "roofline": {"bound": "hbm", "kernel": "the whole expert-parallel step on one GPU (rank 0)",
                                     "achieved": res["rank_bytes"][0] / (res["ms"] * 1e-3) / 1e9, "peak": hbm,
                                     "unit": "GB/s", "frac": s["rank0_frac_of_hbm"], "peak_source": f"of {which}",
                                     "traffic": None, "bytes_per_step": res["rank_bytes"][0],
                                     "slowest_rank_frac": s["slowest_rank_frac_of_hbm"],
                                     "note": "algorithmic bytes of rank 0's step (its touched experts' packed weights, "
                                             "router rows, tokens in and out) over the step time; the per-kernel "
                                             "roofline with ncu traffic is the 1-GPU line's"},
                        "rank_pairs": res["rank_pairs"], "cpu_baseline": None, "ep_check": res["check"], **extras}
            print(json.dumps(line))
        dist.barrier()
        dist.destroy_process_group()
        return

    # ---- one GPU: the headline layer, its sweep, then configs 4 and 5 on the expert-parallel code with one rank ----
    shape, rows = synthetic.C2, args.rows
    layers = []
    for copy in range(2):
        gate, up, down = synthetic.affine_layer(shape, dev, torch.float16 if args.scales == "fp16" else torch.bfloat16,
                                                 copy=copy)
        layers.append(moe.Routed(synthetic.router_rows(shape, dev), experts.make([gate, up], down, 64), shape.top_k,
                                 shared=shape.shared))
        del gate, up, down
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        torch.cuda.synchronize()
        head, runners = bench_rows(torch, shape, layers, rows, args.steps, args.warmup, hbm, args.form == "prefill",
                                   tflops)
        torch.cuda.synchronize()
    e2e = bench_e2e(torch, runners, shape, rows, args.steps, args.warmup)
    status = _lib.kernel_status()
    if status != 0:
        raise SystemExit(f"a kernel recorded a failure: {_lib.describe_status(status)}")
    ms = head["ms_per_step"]
    sweep = []
    if not args.no_sweep:
        del runners
        for t_rows, pre in ((1, False), (4, False), (16, False), (2048, True)):
            res, rr = bench_rows(torch, shape, layers, t_rows, max(5, args.steps // 2), args.warmup, hbm, pre, tflops)
            res.setdefault("form", "decode")
            sweep.append(res)
            del rr
        del layers
        torch.cuda.empty_cache()
        sweep += bench_exl3(torch, (1, 64), max(5, args.steps // 2), args.warmup, hbm)
    else:
        del layers
    ref_cuda = None if args.no_sweep else guarded("reference kernels", lambda: bench_reference_cuda(
        torch, (1, 64, 2048), max(5, args.steps // 4), 3), torch, dist)
    torch.cuda.empty_cache()
    run_extras()
    value = rows / (ms * 1e-3)
    cpu = cpu_1 = cpu_x3 = None
    if not args.no_cpu:
        passes = 100                                      # about 10 s of host work at 0.1 s a pass
        v, sec, cores = cpu_baseline(shape, rows, passes, 2)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{passes} timed passes (2 warm-up) of the same {rows}-token layer call, {sec:.3f} s a pass"}
        v1, sec1, _ = cpu_baseline(shape, rows, 4, 1, threads=1)
        cpu_1 = {"value": v1, "unit": UNIT, "cores": 1, "kind": "port",
                 "sample": f"4 timed passes (1 warm-up) of the same {rows}-token layer call, {sec1:.3f} s a pass"}
        vx, secx, cx = cpu_baseline_exl3(rows, 3)
        cpu_x3 = {"value": vx, "unit": UNIT, "cores": cx, "kind": "port",
                  "sample": f"3 timed passes (1 warm-up) of the routed EXL3 experts of config 3 (4.00 bpw) on {rows} "
                            f"tokens, {secx:.3f} s a pass"}
    traffic, traffic_source = captured_traffic() if (rows, args.form) == (64, "decode") else (None, "not captured")
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, **{k: head[k] for k in ("repeats", "ms_min", "ms_max")},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(shape, rows, world),
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": head["launches_per_step"] * args.steps,
            "roofline": {"bound": "hbm", "kernel": "decode_kernel<M=2, SwiGLU> (gate/up)",
                         "achieved": head["gate_up_gbs"], "peak": hbm, "unit": "GB/s",
                         "frac": head["gate_up_gbs"] / hbm, "peak_source": f"of {which}",
                         "traffic": traffic, "traffic_source": traffic_source,
                         "bytes_per_launch": head["gate_up_bytes"], "us_per_launch": head["gate_up_us"]},
            "layer": {k: head[k] for k in ("distinct_experts", "layer_bytes", "layer_gbs", "layer_frac_of_hbm")},
            "cpu_baseline": cpu, "cpu_baseline_1_thread": cpu_1, "cpu_baseline_exl3": cpu_x3, "reference_cuda": ref_cuda, "sweep": sweep, **extras}
    print(json.dumps(line))
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=None, help="tokens a step on each GPU (64 unless given)")
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
                    help="c2: the headline layer, with configs 4 and 5 beside it under \"c4\" / \"c5\" (default); c4: "
                         "only the 256-expert layer with a shared expert and skewed routing, 256 tokens split over the "
                         "ranks; c5: only the 8-layer mixed-width EXL3 stack, 1..512 tokens split over the ranks")
    ap.add_argument("--hot-pairs", type=int, default=-1,
                    help="expert-parallel peer form: experts with at least this many pairs use the prompt-form kernel "
                         "(default: 32 for config 4, never for config 2)")
    ap.add_argument("--as-rank-of", type=int, default=0,
                    help="one GPU runs the expert launches of one rank of an N-rank config-2 group (for profiling)")
    ap.add_argument("--slice-rank", type=int, default=0, help="which rank's expert window --as-rank-of runs")
    ap.add_argument("--one-width", type=int, default=0, choices=[0, 2, 3, 4, 5, 6, 7, 8],
                    help="--as-rank-of with --config c5: every tensor at this many bits instead of the seeded mix")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-sweep", action="store_true", help="skip the 1-, 4-, 16- and 2048-token and EXL3 lines")
    ap.add_argument("--no-extra", action="store_true", help="skip configs 4 and 5")
    args = ap.parse_args()
    args.exl3_rows = (1, 64) if args.rows is None else (args.rows,)
    args.rows = 64 if args.rows is None else args.rows
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        args.steps = min(args.steps, 400)                        # a bounded CPU sample: a pass takes ~0.1 s
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
