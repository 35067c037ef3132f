"""Benchmark of the FP8 fused-MoE layer (DeepSeek-V3 shape) on B200.

    python bench.py --gpus N --steps K --warmup W [--tokens T] [--impl reference]

One step = one layer call over a batch of T tokens per GPU (routing -> sort -> quant -> gate_up ->
down -> combine).  Prints ONE JSON line.  ``value`` is tokens/s with inputs resident in HBM;
``e2e`` is the same through the reference-facing op (``deepseek_v2_fp8_moe``, router GEMM
included) from pinned HOST buffers with both copies timed; ``roofline`` describes the dominant
kernel (the gate_up grouped GEMM); ``cpu_baseline`` is the reference's CPU implementation of the
path timed on a bounded sample.  The same line also carries, as sub-records: ``sustained`` (two
seconds of back-to-back steps with the clocks seen), ``sweep`` (other token counts as CUDA-graph
replays), ``models`` (the Mixtral-8x7B and Qwen3-30B-A3B widths) and ``mxfp4`` (MXFP4 weights with
MXFP8 activations at 8192 tokens).
N > 1: expert parallelism, each rank holds n_routed/N routed experts + the shared expert and its
own T tokens (weak scaling); dispatch and combine are NCCL all-to-alls; before anything is timed
rank 0 checks tokens of its own against the CPU oracle (``parity``; a failed gate exits non-zero).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import statistics
import subprocess
import sys
import tempfile
import time
import types

import torch

ROOT = pathlib.Path(__file__).resolve().parent
# DRAM bytes the gate_up grouped GEMM moves per algorithmic byte, from ncu captures of smaller cases
# of the same kernels (dram__bytes_read.sum + dram__bytes_write.sum over the launch's algorithmic bytes)
TRAFFIC_PER_ALGORITHMIC_BYTE = {"prefill": 1.068, "decode": 1.01}
sys.path.insert(0, str(ROOT))

from aklr_b200 import workloads as wl  # noqa: E402

METRIC = "fp8_fused_moe_tokens_per_s"
UNIT = "tokens/s"
SEED = 2024
FALLBACK_HBM_GBS = 6650.0
STAGES = ["route", "sort", "quant", "gate_up", "down", "combine"]
# token counts each configuration is quoted on
SWEEP_TOKENS = {"deepseek_v3": (1, 64, 256, 16384), "mixtral": (1, 16, 64, 256, 1024, 4096), "qwen3": (1, 32, 256, 2048, 8192)}
# Tokens per step of the CPU legs.  The sample is a slice of the workload BY EXPERTS: every one of its tokens is routed
# (through the reference's own routing, by a correction bias that lifts eight routed experts of four groups) to the same
# eight routed experts plus the shared one, so each of the nine experts decodes its weights once for 143 rows -- the
# 4096-token batch's rows per expert (4096 x 9 / 257).  Time per token is then the full batch's, in seconds not hours.
CPU_SAMPLE_TOKENS = 143


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense FP8 TFLOP/s taken as twice the measured bf16 burst, 'measured' | 'fallback')."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            peaks = json.loads(path.read_text())
            return float(peaks["hbm_gbs"]), 2.0 * float(peaks["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, 2.0 * 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi sampled every 50 ms, started before the warm-up so that it is already running;
    only samples stamped between begin() and stop() -- the timed region -- count."""

    FIELDS = (
        "timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.t0 = time.time()
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(gpu_index)],
                stdout=self.file,
                stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None

    def begin(self) -> None:
        self.t0 = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t1 = time.time()
        time.sleep(0.1)  # let the sample in flight land
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        import datetime

        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((stamp, float(parts[1]), float(parts[2]), parts[5:9]))
            except ValueError:
                continue
        os.unlink(self.file.name)
        inside = [r for r in rows if self.t0 <= r[0] <= t1] or rows  # a region shorter than the period: all samples
        sm, sm_max, reasons = [r[1] for r in inside], [r[2] for r in inside], set()
        for r in inside:
            for name, flag in zip(names, r[3]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(sm_max) if sm_max else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def bind_near_gpu(local_rank: int) -> str:
    """Run this process on the CPUs the driver reports as closest to its GPU, BEFORE pinned host buffers are
    allocated: with eight ranks on one box, buffers that land on the other socket halve the copy bandwidth of the
    end-to-end leg.  Reads the GPU's CPU set through NVML and changes only this process's scheduler affinity."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return "unchanged (the GPU's CPU set is outside this process's)"
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} CPUs near GPU {local_rank}"
    except Exception as e:  # noqa: BLE001 -- no NVML, no permission: the copies still work, only slower
        return f"unchanged ({type(e).__name__})"


def routing_of(cfg):
    from aklr_b200.moe import Routing

    return Routing(cfg.topk, cfg.scoring, cfg.n_shared, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor)


# --------------------------------------------------------------------------------------------------
# The reference's CPU implementation of the path (cpu_baseline leg and the --impl reference arm)
# --------------------------------------------------------------------------------------------------
class HostExperts:
    """One field (0: w1, 1: w1_scale, 2: w2, 3: w2_scale) of the layer's experts on the host, indexable by
    expert like the stacked tensor; an expert is drawn on first use (outside timing)."""

    def __init__(self, cfg, seed, which, cache):
        self.cfg, self.seed, self.which, self.cache = cfg, seed, which, cache

    def prefetch(self, experts):
        draw_on = "cuda" if torch.cuda.is_available() else "cpu"
        for e in experts:
            if e not in self.cache:
                self.cache[e] = tuple(t.cpu() for t in wl.one_expert_weights(self.cfg, self.seed, e, draw_on))

    def __getitem__(self, e):
        self.prefetch([e])
        return self.cache[e][self.which]


class CpuPath:
    """The layer on the host cores: the reference's own ``deepseek_v2_fp8_moe_reference`` where its package
    can be imported (an install under baseline/_ref travels with the repository), else the restatement
    under oracle/ (the same arithmetic function by function)."""

    def __init__(self, cfg):
        from oracle import moe_oracle as orc

        self.cfg, self.orc = cfg, orc
        if hasattr(os, "sched_setaffinity"):  # the GPU legs may have narrowed this process to the CPUs near its GPU
            os.sched_setaffinity(0, range(os.cpu_count() or 1))
        self.cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        torch.set_num_threads(self.cores)
        cache: dict = {}
        self.host = [HostExperts(cfg, SEED, i, cache) for i in range(4)]
        self.router_w = wl.router_weight(cfg, SEED)
        self.kind, self.reference, self.fp8_linear = "port", None, None
        ref_dir = ROOT / "baseline" / "_ref"
        if (ref_dir / "aklr").is_dir():
            sys.path.insert(0, str(ref_dir))
            try:
                from aklr.plugins.sglang.models.deepseek_v2 import reference as ref_module

                self.reference = ref_module.deepseek_v2_fp8_moe_reference
                self.fp8_linear = ref_module._fp8_linear
                self.kind = "reference"
            except Exception as e:  # the port below is the same arithmetic
                print(f"bench: the reference package under {ref_dir} did not import ({e!r}); timing the port", file=sys.stderr)
            finally:
                sys.path.remove(str(ref_dir))
        self.point = types.SimpleNamespace(
            dtypes={"hidden_states": "bfloat16", "router_weight": "bfloat16", "correction_bias": "bfloat16", "w1": "float8_e4m3fn",
                    "w1_scale": "float32", "w2": "float8_e4m3fn", "w2_scale": "float32"},
            attrs={"topk": cfg.topk, "num_expert_group": cfg.num_expert_group, "topk_group": cfg.topk_group, "renormalize": cfg.renormalize},
            axes={"n_routed": cfg.n_routed},
        )

    def experts_hit(self, hidden, bias):
        logits = self.orc.router_logits(hidden, self.router_w)
        ids, _ = self.orc.grouped_sigmoid_topk(logits, bias.float(), self.cfg.topk, self.cfg.num_expert_group, self.cfg.topk_group,
                                               self.cfg.renormalize, self.cfg.routed_scaling_factor)
        return sorted(set(ids.flatten().tolist()) | set(range(self.cfg.n_routed, self.cfg.n_experts)))

    def step(self, hidden, bias):
        c = self.cfg
        if self.reference is not None:
            args = dict(hidden_states=hidden, router_weight=self.router_w, correction_bias=bias, w1=self.host[0], w1_scale=self.host[1],
                        w2=self.host[2], w2_scale=self.host[3], routed_scaling_factor=c.routed_scaling_factor)
            return self.reference(self.point, args)
        return self.orc.deepseek_v2_fp8_moe(hidden, self.router_w, bias, self.host[0], self.host[1], self.host[2], self.host[3], c.topk,
                                            c.num_expert_group, c.topk_group, c.renormalize, c.routed_scaling_factor)

    def slice_bias(self, bias, step):
        """The correction bias with eight routed experts (two in each of four groups, others every step) lifted far above
        the sigmoid scores: the reference's grouped top-k then sends every token to exactly those."""
        c = self.cfg
        if c.scoring != "sigmoid" or c.num_expert_group < 4 or c.topk != 8:
            return bias  # other routings: the sample's tokens spread over the experts as they fall
        per_group = c.n_routed // c.num_expert_group
        lifted = bias.clone().float()
        step %= 4  # four sets of experts in turn: 36 experts (1.6 GB) in host memory however many steps run
        for g in range(4):
            group = (2 * g + step) % c.num_expert_group
            for k in range(2):
                lifted[group * per_group + (3 + 7 * step + 13 * k) % per_group] += 100.0
        return lifted.to(bias.dtype)

    def time_steps(self, sample_tokens, steps, warmup):
        """(tokens/s, seconds in the timed steps): ``steps`` calls on ``sample_tokens`` tokens each."""
        batches = []
        for s in range(steps + warmup):
            hidden, _, bias = wl.router_inputs(self.cfg, sample_tokens, SEED + 1000 + s)
            bias = self.slice_bias(bias, s)
            self.host[0].prefetch(self.experts_hit(hidden, bias))
            batches.append((hidden, bias))
        for hidden, bias in batches[:warmup]:
            self.step(hidden, bias)
        t0 = time.perf_counter()
        for hidden, bias in batches[warmup:]:
            self.step(hidden, bias)
        elapsed = time.perf_counter() - t0
        return sample_tokens * steps / elapsed, elapsed

    def full_batch_estimate(self, n_tokens):
        """Tokens/s the same code would reach on the whole batch, where every expert is decoded once for
        about 128 rows instead of once for one or two: (time of one expert's MLP on 1 row) x experts +
        (extra time per row, from the MLP on 128 rows) x the other routes.  An estimate, labelled as one."""
        c, orc = self.cfg, self.orc
        e = c.n_routed  # the shared expert: drawn for every sample already
        w1, s1, w2, s2 = (h[e] for h in self.host)
        rows = wl.normal(SEED, "estimate", (128, c.hidden), 1.0, dtype=torch.bfloat16).float()

        def mlp(x):
            if self.fp8_linear is not None:
                gate, up = self.fp8_linear(x, w1.float(), s1).chunk(2, dim=-1)
                return self.fp8_linear(torch.nn.functional.silu(gate) * up, w2.float(), s2)
            gate, up = (orc.fp8_input(x) @ orc.dequant_block_weight(w1, s1).T).chunk(2, dim=-1)
            return orc.fp8_input(torch.nn.functional.silu(gate) * up) @ orc.dequant_block_weight(w2, s2).T

        def best_of(x, n=3):
            times = []
            for _ in range(n):
                t0 = time.perf_counter()
                mlp(x)
                times.append(time.perf_counter() - t0)
            return min(times)

        t_one, t_block = best_of(rows[:1]), best_of(rows)
        per_row = max(t_block - t_one, 0.0) / 127
        routes = n_tokens * c.routes_per_token
        seconds = c.n_experts * t_one + max(routes - c.n_experts, 0) * per_row
        return {
            "value": n_tokens / seconds,
            "unit": UNIT,
            "seconds_per_step": seconds,
            "method": f"{c.n_experts} experts x {t_one * 1e3:.0f} ms (one expert's MLP on 1 row, weights decoded) + "
                      f"{routes - c.n_experts} further routes x {per_row * 1e6:.0f} us (from the MLP on 128 rows); an estimate, not a measurement",
        }


def cpu_record(cpu: CpuPath, value, elapsed, steps, sample) -> dict:
    return {
        "value": value,
        "unit": UNIT,
        "cores": cpu.cores,
        "kind": cpu.kind,
        "sample": f"{steps} steps of {sample} tokens ({elapsed:.1f} s timed), router GEMM and routing included, expert weights "
                  "already in host memory; a slice of the batch by experts: the step's tokens all route to the same 8 routed "
                  "experts + the shared one, so each expert decodes once for the full batch's ~143 rows per expert",
    }


def run_reference_arm(args, cfg):
    """The reference's CPU implementation of the path on this box's host cores, on a bounded sample of
    the workload per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = CpuPath(cfg)
    value, elapsed = cpu.time_steps(CPU_SAMPLE_TOKENS, args.steps, args.warmup)
    record = cpu_record(cpu, value, elapsed, args.steps, CPU_SAMPLE_TOKENS)
    record["full_batch_estimate"] = cpu.full_batch_estimate(args.tokens)
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": workload_config(cfg, args),
        "cpu_baseline": record,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, args):
    return {
        "workload": f"{'deepseek_v3' if cfg.name.startswith('deepseek_v3') else cfg.name} fp8 fused-moe layer, {args.tokens} tokens per GPU per step",
        "hidden": cfg.hidden,
        "moe_intermediate": cfg.inter,
        "routed_experts": cfg.n_routed,
        "shared_experts": cfg.n_shared,
        "topk": cfg.topk,
        "routing": "sigmoid + correction bias, 8 groups / top-4 groups / top-8, x2.5" if cfg.scoring == "sigmoid" else f"softmax top-{cfg.topk}",
        "weights": "fp8 e4m3, 128x128 fp32 block scales, N(0,0.02)" + (", tile-contiguous layout" if getattr(args, "tiled_weights", False) else ""),
        "activations": "bf16 N(0,1), 1x128 fp8 groups",
        "tokens_per_gpu": args.tokens,
        "parallelism": f"ep{args.gpus}" if args.gpus > 1 else "single gpu",
        "l2": "inputs larger than L2: every step streams all expert weights hit (GBs vs 126 MB); batches rotate",
    }


# --------------------------------------------------------------------------------------------------
# GPU arm, one GPU
# --------------------------------------------------------------------------------------------------
def distinct_experts(ids: torch.Tensor) -> int:
    return int(torch.unique(ids).numel())


def device_ids(cfg, logits, bias):
    """Routing ids of a batch computed by the routing kernel itself (for experts-hit counts)."""
    from aklr_b200.moe import route

    return route(logits, bias, routing_of(cfg))[0]


def read_stage_ms(lib, calls, first=0, stride=1):
    from aklr_b200 import _lib

    stage_ms = [0.0] * 6
    buf = (ctypes.c_float * 6)()
    for i in range(calls):
        _lib.check(lib.aklr_profile_read(first + stride * i, buf))
        for j in range(6):
            stage_ms[j] += buf[j] / calls
    return stage_ms


def graph_sweep(cfg, tokens_list, weights, bias, device, peak_hbm, peak_fp8, layer_call, block_m=0):
    """Each token count as one CUDA graph of 8 layer calls on rotating batches, replayed (the reference's
    measurement protocol): at small counts the host cannot issue the launches as fast as they run."""
    from aklr_b200.moe import Workspace, _config

    routing = routing_of(cfg)
    rows = []
    for tokens in tokens_list:
        batches = [wl.router_inputs(cfg, tokens, SEED + 50 + b, device)[:2] for b in range(8)]
        out = torch.empty((tokens, cfg.hidden), dtype=torch.bfloat16, device=device)
        ws = Workspace(_config(tokens, cfg.hidden, cfg.inter, cfg.n_routed, routing, batches[0][1], bias, block_m), device)
        for hidden, logits in batches:  # every batch once outside a capture
            layer_call(hidden, logits, bias, *weights, routing, out=out, workspace=ws, block_m=block_m)
        ws.check_status()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for hidden, logits in batches:
                layer_call(hidden, logits, bias, *weights, routing, out=out, workspace=ws, block_m=block_m)
        for _ in range(3):
            graph.replay()
        replays = 2 if tokens >= 1024 else 8
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / (replays * 8)
        hit = sum(distinct_experts(device_ids(cfg, logits, bias)) for _, logits in batches) / 8
        flops, nbytes = wl.roofline_work(cfg, tokens, hit)
        t_hbm, t_tensor = nbytes / (peak_hbm * 1e9), flops / (peak_fp8 * 1e12)
        rows.append({
            "tokens": tokens, "us_per_call": ms * 1e3, "tokens_per_s": tokens / (ms * 1e-3), "experts_hit": hit,
            "bound": "hbm" if t_hbm > t_tensor else "tensor", "frac_of_hbm_roofline": t_hbm / (ms * 1e-3),
            "tflops": flops / (ms * 1e-3) / 1e12, "frac_of_fp8_peak": flops / (ms * 1e-3) / 1e12 / peak_fp8, "block_m": ws.layout.block_m,
        })
        del graph, ws, out, batches
    return rows


def bench_mxfp4_record(cfg, tokens, steps, warmup, device, lib, peak_hbm, peak_fp8):
    """Configuration 5 on one GPU: the same layer with MXFP4 expert weights and MXFP8 activations."""
    from aklr_b200.moe import Workspace, _config, fused_moe_mxfp4

    routing = routing_of(cfg)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, SEED, device)
    bias = wl.router_inputs(cfg, 1, SEED + 1, device)[2]
    batches = [wl.router_inputs(cfg, tokens, SEED + 1 + b, device)[:2] for b in range(4)]
    out = torch.empty((tokens, cfg.hidden), dtype=torch.bfloat16, device=device)
    ws = Workspace(_config(tokens, cfg.hidden, cfg.inter, cfg.n_routed, routing, batches[0][1], bias, 128), device)

    def step(i):
        hidden, logits = batches[i % 4]
        fused_moe_mxfp4(hidden, logits, bias, w1, s1, w2, s2, routing, out=out, workspace=ws)

    for i in range(warmup):
        step(i)
    ws.check_status()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    lib.aklr_profile_begin(steps)
    start.record()
    for i in range(steps):
        step(warmup + i)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    stage_ms = read_stage_ms(lib, steps)
    lib.aklr_profile_begin(0)
    hit = distinct_experts(ws.topk_ids())
    h, inter = cfg.hidden, cfg.inter
    weight_bytes = hit * (3 * h * inter // 2 + 3 * h * inter // 32)
    flops = tokens * cfg.routes_per_token * cfg.flops_per_route
    return {
        "workload": f"deepseek_v3 widths, mxfp4 weights (e2m1 + e8m0 per 32) x mxfp8 activations, {tokens} tokens",
        "tokens": tokens, "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
        "frac_of_fp8_peak": flops / (ms * 1e-3) / 1e12 / peak_fp8,
        "frac_of_hbm_roofline": weight_bytes / (peak_hbm * 1e9) / (ms * 1e-3),
        "gate_up_tflops": 2 * flops / 3 / (stage_ms[3] * 1e-3) / 1e12 if stage_ms[3] > 0 else None,
        "down_tflops": flops / 3 / (stage_ms[4] * 1e-3) / 1e12 if stage_ms[4] > 0 else None,
        "stage_ms": dict(zip(STAGES, stage_ms)),
        "parity": "tests/test_gpu_full_width.py checks this shape against the oracle",
    }


# ---------------------------------------------------------------------------------------------------------
# The workloads the reference records timings for (its kernel JSONs: AMD MI355X, CUDA-graph replay, L2 flushed
# before every call, median microseconds per call), run here the same way through the same op functions.
# Shapes and the recorded microseconds are copied from those files; inputs are seeded synthetic tensors of the
# contracts' distributions.  Context, not a target: another machine, and TP8-sliced widths.
# ---------------------------------------------------------------------------------------------------------
PUBLISHED = [
    # (op, shape, {tokens: recorded microseconds})
    ("deepseek_v2_fp8_moe", dict(hidden=7168, inter=256, n_routed=256, topk=8, groups=8, topk_group=4),
     {1: 17.4, 8: 61.0, 64: 198.0, 256: 258.0, 1024: 358.0, 4096: 607.0, 16384: 1810.0}),
    ("minimax_m2_fp8_moe", dict(hidden=3072, inter=384, n_routed=256, topk=8), {1: 14.1, 256: 177.0, 4096: 349.0, 16384: 1050.0}),
    ("qwen2_moe_fp8_router_experts", dict(hidden=2048, inter=128, n_routed=512, topk=10), {1: 13.0, 256: 96.0, 16384: 533.0}),
    ("deepseek_v2_mxfp4_moe", dict(hidden=6144, inter=256, n_routed=256, topk=8), {1: 18.3, 256: 127.0, 4096: 349.0}),
    ("fused_moe mxfp4", dict(hidden=6144, inter=256, n_routed=257, topk=9), {1: 10.9, 64: 96.6, 4096: 240.0}),
    ("fused_moe mxfp4 interleave, 48 of 384 experts held", dict(hidden=7168, inter=3072, n_routed=48, topk=6, global_experts=384), {2048: 313.0}),
    ("per_group_quant_fp8", dict(hidden=7168), {448: 4.77, 2048: 9.43, 16384: 55.2}),
    ("per_group_quant_mxfp8", dict(hidden=7168), {16384: 51.1}),
]


def _published_call(name, shape, tokens, device, seed):
    """(callable running the op once, number of rotating input sets it was built with)."""
    from aklr_b200 import ops

    h = shape["hidden"]
    n_sets = 4
    xs = [wl.normal(seed + i, "hidden", (tokens, h), 1.0, device, torch.bfloat16) for i in range(n_sets)]
    if name.startswith("per_group_quant"):
        op = ops.per_group_quant_fp8 if name.endswith("fp8") and "mx" not in name else ops.per_group_quant_mxfp8
        return lambda i: op(x=xs[i % n_sets])
    cfg = wl.MoEConfig(name, hidden=h, inter=shape["inter"], n_routed=shape["n_routed"], topk=shape["topk"],
                       scoring="sigmoid" if "deepseek" in name or "minimax" in name else "softmax",
                       n_shared=1 if ("deepseek" in name or "qwen2" in name) else 0)
    mx = "mxfp4" in name
    w1, s1, w2, s2 = (wl.mx_expert_weights if mx else wl.expert_weights)(cfg, seed, device)
    weights = dict(w1=w1, w1_scale=s1, w2=w2, w2_scale=s2)
    if name.startswith("fused_moe"):
        n_global = shape.get("global_experts", cfg.n_routed)
        g = torch.Generator(device="cpu").manual_seed(seed)
        sets = []
        for i in range(n_sets):
            ids = torch.stack([torch.randperm(n_global, generator=g)[: cfg.topk] for _ in range(tokens)]).to(torch.int32).to(device)
            wts = torch.rand(tokens, cfg.topk, generator=g).to(device)
            sets.append((ids, wts))
        extra = {}
        if n_global != cfg.n_routed:  # this rank holds a slice: the mask, a count of rows received, the clamped SwiGLU
            mask = torch.zeros(n_global, dtype=torch.int32)
            mask[96 : 96 + cfg.n_routed] = 1
            extra = dict(expert_mask=mask.to(device), num_local_tokens=torch.tensor([tokens], dtype=torch.int32, device=device),
                         gate_mode="interleave", swiglu_limit=7.0)
        return lambda i: ops.fused_moe(xs[i % n_sets], w1, w2, sets[i % n_sets][1], sets[i % n_sets][0], activation="silu",
                                       quant_type="per_1x32", w1_scale=s1, w2_scale=s2, **extra)
    if name == "deepseek_v2_fp8_moe" or name == "deepseek_v2_mxfp4_moe":
        rw = (wl.router_weight(cfg, seed, device).float() * 40).to(torch.bfloat16)
        fp8 = not mx
        bias = wl.normal(seed, "bias", (cfg.n_routed,), 0.05, device, torch.bfloat16 if fp8 else torch.float32) + (0.0 if fp8 else 8.0)
        op = ops.deepseek_v2_fp8_moe if fp8 else ops.deepseek_v2_mxfp4_moe
        groups = (shape["groups"], shape["topk_group"]) if fp8 else (1, 1)
        return lambda i: op(hidden_states=xs[i % n_sets], router_weight=rw, correction_bias=bias, **weights, topk=cfg.topk,
                            num_expert_group=groups[0], topk_group=groups[1], renormalize=True, scoring_func="sigmoid",
                            routed_scaling_factor=2.5)
    if name == "minimax_m2_fp8_moe":
        rw = wl.normal(seed, "router", (cfg.n_routed, h), 3.0 / h**0.5, device)
        bias = 8.0 + wl.normal(seed, "bias", (cfg.n_routed,), 0.02, device)
        return lambda i: ops.minimax_m2_fp8_moe(hidden_states=xs[i % n_sets], router_weight=rw, correction_bias=bias, **weights, topk=cfg.topk)
    if name == "qwen2_moe_fp8_router_experts":
        rw = (wl.router_weight(cfg, seed, device).float() * 30).to(torch.bfloat16)
        gate = wl.normal(seed, "shared_gate", (1, h), 2.0 / h**0.5, device, torch.bfloat16)
        return lambda i: ops.qwen2_moe_fp8_router_experts(hidden_states=xs[i % n_sets], router_weight=rw, shared_gate_weight=gate,
                                                          **weights, topk=cfg.topk)
    raise ValueError(name)


def bench_published(device) -> dict:
    """Microseconds per call of every workload in PUBLISHED: a CUDA graph of 8 calls on rotating inputs, each
    preceded by a write over a 256 MB buffer (the L2 flush of the reference's protocol), replayed; the same graph
    without the calls is timed and subtracted."""
    from aklr_b200 import ops

    ops.init()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    calls_per_graph = 8

    def graph_ms(body):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(calls_per_graph):
                flush.zero_()
                body(i)
        for _ in range(2):
            graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(4):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / (4 * calls_per_graph)

    flush_ms = graph_ms(lambda i: None)
    rows = []
    for name, shape, recorded in PUBLISHED:
        for tokens, ref_us in recorded.items():
            call = _published_call(name, shape, tokens, device, SEED + 900)
            for i in range(4):  # every input set once outside a capture (the ops warm each shape up)
                out = call(i)
                if not isinstance(out, (torch.Tensor, tuple)):
                    raise RuntimeError(f"{name} at {tokens} tokens was not served: {out}")
            torch.cuda.synchronize()
            us = (graph_ms(call) - flush_ms) * 1e3
            rows.append({"op": name, "shape": shape, "tokens": tokens, "us_per_call": us, "reference_us_mi355x": ref_us,
                         "ratio": ref_us / us})
            del call
            torch.cuda.empty_cache()
    return {"protocol": "CUDA-graph replay of 8 calls on rotating inputs, 256 MB written before each call (its time, "
                        f"{flush_ms * 1e3:.1f} us, subtracted); through the op functions, router GEMM included where the op has one",
            "rows": rows}


def bench_emulated_ep(args, cfg, device) -> dict:
    """Expert parallelism with ``--emulate-ep`` ranks emulated in ONE process on one GPU (phase by phase, the
    exchanges as device copies): the dispatch and combine kernels at the benchmark's sizes where a profiler can
    see them (a multi-rank command is never run under one).  Times the whole emulated step; not a bench value."""
    from aklr_b200.ep import ExpertParallelMoE, run_in_process

    world, T = args.emulate_ep, args.tokens
    routing = routing_of(cfg)
    w1, s1, w2, s2 = wl.expert_weights(cfg, SEED, device)
    bias = wl.router_inputs(cfg, 1, SEED + 1, device)[2]
    n_local = cfg.n_routed // world
    layers, inputs = [], []
    for r in range(world):
        mine = list(range(r * n_local, (r + 1) * n_local)) + list(range(cfg.n_routed, cfg.n_experts))
        layers.append(ExpertParallelMoE(routing, w1[mine].contiguous(), s1[mine].contiguous(), w2[mine].contiguous(),
                                        s2[mine].contiguous(), r, world))
        hidden, logits, _ = wl.router_inputs(cfg, T, SEED + 10 + r, device)
        inputs.append((hidden, logits, bias))
    del w1, s1, w2, s2
    torch.cuda.empty_cache()
    for _ in range(args.warmup):
        run_in_process(layers, inputs)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        run_in_process(layers, inputs)
    stop.record()
    torch.cuda.synchronize()
    return {"emulated_ranks": world, "tokens_per_rank": T, "ms_per_emulated_step_all_ranks": start.elapsed_time(stop) / args.steps,
            "note": "all ranks' phases one after the other on one GPU: for profiler captures of the dispatch / combine kernels"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU per step")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="skip the sub-records (sustained, sweep, models, mxfp4, e2e, cpu): profiling captures")
    ap.add_argument("--sweep-tokens", default="", help="token counts of the sweep sub-record, comma-separated (default: the configuration's)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--routed-experts", type=int, default=0, help="shrink the layer to this many routed experts (profiling captures only)")
    ap.add_argument("--block-m", type=int, default=0, help="force the tokens-per-block of the grouped GEMMs")
    ap.add_argument("--variant", type=int, default=0, help="aklr_moe_config.variant bits for the headline leg")
    ap.add_argument("--format", default="fp8", choices=["fp8", "mxfp4"], help="mxfp4: only the MXFP4 record, as the line's value")
    ap.add_argument("--model", default="deepseek_v3", choices=["deepseek_v3", "mixtral", "qwen3"],
                    help="widths of the headline leg (profiling captures of the other configurations; with --headline-only)")
    ap.add_argument("--emulate-ep", type=int, default=0, help="this many expert-parallel ranks emulated in one process on one GPU (profiling captures)")
    ap.add_argument("--tiled-weights", action="store_true", help="expert weights in the tile-contiguous layout (aklr_b200.layouts)")
    ap.add_argument("--published", action="store_true", help="only the workloads the reference records timings for, one JSON object")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    cfg = wl.CONFIGS[args.model]
    if args.model != "deepseek_v3" and not args.headline_only:
        raise SystemExit("--model other than deepseek_v3 times the headline leg alone: add --headline-only")
    if args.routed_experts:
        import dataclasses

        cfg = dataclasses.replace(cfg, name=f"deepseek_v3_{args.routed_experts}e", n_routed=args.routed_experts)

    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    args.cpu_affinity = bind_near_gpu(local_rank)
    if args.published:
        print(json.dumps(bench_published(device)))
        return
    if args.emulate_ep:
        print(json.dumps(bench_emulated_ep(args, cfg, device)))
        return
    saved_stdout = None
    if world > 1:
        import torch.distributed as dist

        # NCCL may print a version banner on stdout at its first collective: keep stdout for the JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=device)

    from aklr_b200 import _lib
    from aklr_b200.csrc.build import build

    build()
    lib = _lib.load()

    if world > 1:
        line = bench_ep(args, cfg, rank, world, device, lib)
        dist.destroy_process_group()
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        if line is not None:
            print(line, flush=True)
        return
    print(json.dumps(bench_one_gpu(args, cfg, device, local_rank, lib)), flush=True)


def bench_one_gpu(args, cfg, device, local_rank, lib) -> dict:
    from aklr_b200 import _lib, ops
    from aklr_b200.moe import Workspace, _config, fused_moe_fp8

    routing = routing_of(cfg)
    T = args.tokens
    peak, peak_fp8, peak_kind = measured_peaks()
    if args.format == "mxfp4":
        sampler = ClockSampler(local_rank)
        sampler.begin()
        launches0 = lib.aklr_kernel_launch_count()
        record = bench_mxfp4_record(cfg, T, args.steps, args.warmup, device, lib, peak, peak_fp8)
        config = workload_config(cfg, args)
        config["workload"] = record["workload"]
        config["weights"], config["activations"] = "mxfp4: e2m1 + e8m0 per 32 along K, N(0,0.02)", "bf16 N(0,1), quantised to MXFP8"
        return {"metric": METRIC.replace("fp8", "mxfp4"), "value": record["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": record["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "mxfp4 x mxfp8", "data": "synthetic", "config": config, "clocks": sampler.stop(), "e2e": None,
                "gpu_launches": int(lib.aklr_kernel_launch_count() - launches0),
                "roofline": {"bound": "tensor", "achieved": record["tflops"], "peak": peak_fp8, "peak_kind": f"2 x bf16 burst, of {peak_kind}",
                             "unit": "TFLOP/s", "frac": record["frac_of_fp8_peak"], "traffic": None, "detail": record},
                "cpu_baseline": None}

    w1, s1, w2, s2 = wl.expert_weights(cfg, SEED, device)
    if args.tiled_weights:  # the load-time layout variant: same results, every TMA box one contiguous 16 KB run
        from aklr_b200 import layouts

        w1, w2 = layouts.to_b200_tiled(w1), layouts.to_b200_tiled(w2)
        torch.cuda.empty_cache()
    router_w = wl.router_weight(cfg, SEED, device)
    n_batches = 4
    batches = []
    for b in range(n_batches):
        hidden, logits, bias = wl.router_inputs(cfg, T, SEED + 1 + b, device)
        batches.append((hidden, logits))
    bias = wl.router_inputs(cfg, 1, SEED + 1, device)[2]
    out = torch.empty((T, cfg.hidden), dtype=torch.bfloat16, device=device)
    ws = Workspace(_config(T, cfg.hidden, cfg.inter, cfg.n_routed, routing, batches[0][1], bias, args.block_m, variant=args.variant), device)

    def step(i):
        hidden, logits = batches[i % n_batches]
        fused_moe_fp8(hidden, logits, bias, w1, s1, w2, s2, routing, out=out, workspace=ws, block_m=args.block_m, variant=args.variant)

    sampler = ClockSampler(local_rank)
    for i in range(args.warmup):
        step(i)
    ws.check_status()
    torch.cuda.synchronize()

    # ---- timed region: K steps, CUDA events on the launching stream, clocks sampled meanwhile ----
    lib.aklr_profile_begin(args.steps)
    launches0 = lib.aklr_kernel_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.begin()
    start.record()
    for i in range(args.steps):
        step(args.warmup + i)
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    launches = lib.aklr_kernel_launch_count() - launches0
    ms_per_step = start.elapsed_time(stop) / args.steps
    ws.check_status()
    stage_ms = read_stage_ms(lib, args.steps)
    lib.aklr_profile_begin(0)

    # ---- roofline of the dominant kernel (gate_up grouped GEMM): algorithmic bytes / its time ----
    experts_hit = distinct_experts(ws.topk_ids())
    routes = T * cfg.routes_per_token
    h, i_dim = cfg.hidden, cfg.inter
    gate_up_bytes = experts_hit * (2 * i_dim * h + 4 * (2 * i_dim // 128) * (h // 128)) + routes * h + routes * (h // 128) * 4 + routes * i_dim
    down_bytes = experts_hit * (h * i_dim + 4 * (h // 128) * (i_dim // 128)) + routes * i_dim + routes * h * 2
    achieved = gate_up_bytes / (stage_ms[3] * 1e-3) / 1e9
    flops, layer_bytes = wl.roofline_work(cfg, T, experts_hit)
    token_major = ws.layout.block_m == 128
    # DRAM bytes of this launch: the ratio measured by ncu on a smaller case of the same kernel times
    # this launch's algorithmic bytes (the traffic grows with the weights streamed)
    traffic_ratio = TRAFFIC_PER_ALGORITHMIC_BYTE["prefill" if token_major else "decode"]
    roofline = {
        "kernel": ("grouped_gemm_prefill_kernel<gate_up>" if token_major else "grouped_gemm_kernel<gate_up>")
        + " (tcgen05 FP8, SiLU*mul + requant epilogue)",
        "bound": "hbm",
        "achieved": achieved,
        "peak": peak,
        "peak_kind": f"of {peak_kind}",
        "unit": "GB/s",
        "frac": achieved / peak,
        "traffic": gate_up_bytes * traffic_ratio,
        "traffic_source": f"ncu capture of a smaller case of the same kernel: {traffic_ratio:.3f} x algorithmic bytes",
        "block_m": ws.layout.block_m,
        "algorithmic_bytes_per_launch": gate_up_bytes,
        "ms_per_launch": stage_ms[3],
        "tflops": routes * 4 * h * i_dim / (stage_ms[3] * 1e-3) / 1e12,
        "stage_ms": dict(zip(STAGES, stage_ms)),
        "down": {
            "achieved": down_bytes / (stage_ms[4] * 1e-3) / 1e9,
            "frac": down_bytes / (stage_ms[4] * 1e-3) / 1e9 / peak,
            "tflops": routes * 2 * h * i_dim / (stage_ms[4] * 1e-3) / 1e12,
        },
        "layer": {
            "algorithmic_bytes": layer_bytes,
            "flops": flops,
            "hbm_time_ms": layer_bytes / (peak * 1e9) * 1e3,
            "frac_of_hbm_roofline": layer_bytes / (peak * 1e9) * 1e3 / ms_per_step,
            "experts_hit": experts_hit,
        },
    }
    line = {
        "metric": METRIC,
        "value": T / (ms_per_step * 1e-3),
        "unit": UNIT,
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": workload_config(cfg, args),
        "clocks": clocks,
        "e2e": None,
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": None,
    }
    if args.headline_only:
        return line

    if not args.no_e2e:
        # ---- end to end through the op API from pinned host buffers --------------------------------
        # Three streams, two buffers each way: step i's H2D overlaps step i-1's compute and step
        # i-2's D2H, as a serving loop would run it.  Every step still copies its own inputs in and
        # its own result out inside the timed region.
        host_hidden = [b[0].cpu().pin_memory() for b in batches]
        ops.init()
        copy_in, copy_out, compute = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        dev_in = [torch.empty_like(batches[0][0]) for _ in range(2)]
        host_outs = [torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        out_ready = [torch.cuda.Event() for _ in range(2)]
        out_free = [torch.cuda.Event() for _ in range(2)]
        for ev in in_free + out_free:
            ev.record(compute)

        def e2e_step(i):
            k = i % 2
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(in_free[k])
                dev_in[k].copy_(host_hidden[i % n_batches], non_blocking=True)
                in_ready[k].record(copy_in)
            compute.wait_event(in_ready[k])
            compute.wait_event(out_free[k])
            result = ops.deepseek_v2_fp8_moe(
                hidden_states=dev_in[k], router_weight=router_w, correction_bias=bias, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2,
                topk=cfg.topk, num_expert_group=cfg.num_expert_group, topk_group=cfg.topk_group, renormalize=cfg.renormalize,
                scoring_func="sigmoid", routed_scaling_factor=cfg.routed_scaling_factor,
            )
            if not isinstance(result, torch.Tensor):
                raise SystemExit(f"the op fell back: {result}")
            in_free[k].record(compute)
            out_ready[k].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(out_ready[k])
                host_outs[k].copy_(result, non_blocking=True)
                result.record_stream(copy_out)
                out_free[k].record(copy_out)

        e2e_sampler = ClockSampler(local_rank)
        for i in range(args.warmup):
            e2e_step(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_sampler.begin()
        e0.record(compute)
        for i in range(args.steps):
            e2e_step(i)
        compute.wait_stream(copy_out)
        compute.wait_stream(copy_in)
        e1.record(compute)
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / args.steps
        line["e2e"] = {
            "value": T / (e2e_ms * 1e-3),
            "unit": UNIT,
            "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": T * cfg.hidden * 2,
            "cpu_affinity": args.cpu_affinity,
            "d2h_bytes_per_step": T * cfg.hidden * 2,
            "api": "aklr_b200.ops.deepseek_v2_fp8_moe (router GEMM included); copies double-buffered on their own streams",
            "clocks": e2e_sampler.stop(),
        }
        del host_hidden, dev_in, host_outs

    # ---- the headline again for two seconds: the clocks settle under the power cap ---------------
    n_long = max(args.steps, int(2000.0 / ms_per_step) + 1)
    long_sampler = ClockSampler(local_rank)
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    long_sampler.begin()
    a.record()
    for i in range(n_long):
        step(i)
    b.record()
    torch.cuda.synchronize()
    long_clocks = long_sampler.stop()
    long_ms = a.elapsed_time(b) / n_long
    ws.check_status()
    line["sustained"] = {
        "steps": n_long, "seconds": long_ms * n_long * 1e-3, "ms_per_step": long_ms, "tokens_per_s": T / (long_ms * 1e-3),
        "clocks": long_clocks, "ms_times_mhz": long_ms * long_clocks["sm_mhz"] if long_clocks.get("sm_mhz") else None,
        "headline_ms_times_mhz": ms_per_step * clocks["sm_mhz"] if clocks.get("sm_mhz") else None,
    }

    # ---- other token counts of this configuration, then the other two FP8 configurations ----------
    tokens_list = [int(v) for v in args.sweep_tokens.split(",")] if args.sweep_tokens else list(SWEEP_TOKENS["deepseek_v3"])
    line["sweep"] = graph_sweep(cfg, tokens_list, (w1, s1, w2, s2), bias, device, peak, peak_fp8, fused_moe_fp8, args.block_m)
    line["sweep_timing"] = "cuda graph replay of 8 calls on rotating batches; weights stream from HBM every call"
    del w1, s1, w2, s2, ws, out, batches
    torch.cuda.empty_cache()
    line["models"] = {}
    for name in ("mixtral", "qwen3"):
        other = wl.CONFIGS[name]
        weights = wl.expert_weights(other, SEED, device)
        line["models"][name] = {
            "workload": f"{name} widths: hidden {other.hidden}, intermediate {other.inter}, {other.n_routed} experts, softmax top-{other.topk}"
                        + (", " + wl.zipf_note() if other.zipf_s > 0 else ""),
            "sweep": graph_sweep(other, SWEEP_TOKENS[name], weights, None, device, peak, peak_fp8, fused_moe_fp8),
        }
        del weights
        torch.cuda.empty_cache()
    line["mxfp4"] = bench_mxfp4_record(cfg, 8192, min(args.steps, 10), 3, device, lib, peak, peak_fp8)
    torch.cuda.empty_cache()

    if not args.no_cpu_baseline:
        cpu = CpuPath(cfg)
        cpu_steps = 12  # ~10 s of CPU work on sixteen cores
        value, elapsed = cpu.time_steps(CPU_SAMPLE_TOKENS, cpu_steps, 1)
        line["cpu_baseline"] = cpu_record(cpu, value, elapsed, cpu_steps, CPU_SAMPLE_TOKENS)
        line["cpu_baseline"]["full_batch_estimate"] = cpu.full_batch_estimate(T)
    return line


# --------------------------------------------------------------------------------------------------
# GPU arm, N > 1: expert parallelism
# --------------------------------------------------------------------------------------------------
def ep_parity(cfg, layer, hidden, logits, bias, mx, device, n_check=4):
    """Rank 0: ``n_check`` of its own tokens through ``layer.forward`` (all ranks take part in the call)
    against the CPU oracle.  Expert weights are seeded per expert, so the experts those tokens hit are
    drawn again here, whichever rank holds them."""
    from oracle import moe_oracle as orc

    out = layer.forward(hidden, logits, bias)
    torch.cuda.synchronize()
    if layer.rank != 0:
        return None
    n_tokens = hidden.shape[0]
    loudest = int(out.float().abs().amax(dim=1).argmax())
    wanted = [0, n_tokens - 1, loudest, n_tokens // 2, n_tokens // 3, 1]
    sample = torch.tensor(sorted(list(dict.fromkeys(t for t in wanted if 0 <= t < n_tokens))[:n_check]))
    ids, w = orc.grouped_sigmoid_topk(logits[sample.to(device)].cpu().float(), bias.cpu().float(), cfg.topk, cfg.num_expert_group, cfg.topk_group,
                                      cfg.renormalize, cfg.routed_scaling_factor)
    ids, w = orc.with_shared_slot(ids, w, cfg.n_routed)
    draw = wl.mx_expert_weights if mx else wl.expert_weights
    cache = {}

    class Lazy:
        def __init__(self, which):
            self.which = which

        def __getitem__(self, e):
            if e not in cache:
                cache[e] = tuple(t[0].cpu() for t in draw(cfg, SEED, device, experts=[e]))
            return cache[e][self.which]

    x = hidden[sample.to(device)].cpu()
    ref = orc.mx_experts(x, ids, w, *(Lazy(i) for i in range(4)), act_bits=8) if mx else orc.fp8_experts(x, ids, w, *(Lazy(i) for i in range(4)))
    gates = orc.output_gates(out[sample.to(device)].cpu(), ref)
    gates["tokens"] = int(sample.numel())
    gates["passed"] = bool(orc.gates_pass(gates))
    gates["against"] = "cpu oracle on rank 0's sampled tokens, experts drawn again from their seeds"
    return gates


def bench_ep(args, cfg, rank, world, device, lib):
    """Every rank holds n_routed/N routed experts + the shared expert and ``args.tokens`` tokens of its own
    (weak scaling).  Rank 0 returns the JSON line."""
    import torch.distributed as dist

    from aklr_b200 import _lib
    from aklr_b200.ep import CudaKernels, ExpertParallelMoE
    from aklr_b200.moe import router_logits

    if cfg.n_routed % world:
        raise SystemExit(f"{cfg.n_routed} routed experts do not split over {world} ranks")
    n_local = cfg.n_routed // world
    mine = list(range(rank * n_local, (rank + 1) * n_local)) + list(range(cfg.n_routed, cfg.n_experts))
    routing = routing_of(cfg)
    peak, peak_fp8, peak_kind = measured_peaks()
    bias = wl.router_inputs(cfg, 1, SEED + 1, device)[2]
    router_w = wl.router_weight(cfg, SEED, device)

    def timed(fn, steps, before_stop=None):
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            fn(i)
        if before_stop is not None:
            before_stop()
        stop.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)  # the slowest rank's device time
        return float(ms) / steps

    def leg(mx: bool, tokens: int, steps: int, with_e2e: bool):
        w1, s1, w2, s2 = (wl.mx_expert_weights if mx else wl.expert_weights)(cfg, SEED, device, experts=mine)
        layer = ExpertParallelMoE(routing, w1, s1, w2, s2, rank, world, kernels=CudaKernels("mxfp4" if mx else "fp8"))
        n_batches = 4
        batches = [wl.router_inputs(cfg, tokens, SEED + 1 + 97 * rank + b, device)[:2] for b in range(n_batches)]
        parity = ep_parity(cfg, layer, batches[0][0], batches[0][1], bias, mx, device)
        verdict = torch.tensor([1 if (parity is None or parity["passed"]) else 0], device=device)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
        if int(verdict) == 0:
            if rank == 0:
                print(f"bench: expert-parallel output failed the parity gates: {parity}", file=sys.stderr)
            raise SystemExit(3)

        def step(i):
            hidden, logits = batches[i % n_batches]
            return layer.forward(hidden, logits, bias)

        sampler = ClockSampler(device.index) if rank == 0 else None
        for i in range(args.warmup):
            step(i)
        torch.cuda.synchronize()
        lib.aklr_profile_begin(0 if mx else 2 * steps)
        launches0 = lib.aklr_kernel_launch_count()
        if sampler:
            sampler.begin()
        ms_per_step = timed(lambda i: step(args.warmup + i), steps)
        clocks = sampler.stop() if sampler else None
        launches = lib.aklr_kernel_launch_count() - launches0
        # stage times of the routed-expert calls (every second recorded call; the other is the shared expert)
        stage_ms = [0.0] * 6 if mx else read_stage_ms(lib, steps, first=1, stride=2)
        lib.aklr_profile_begin(0)
        # rows this rank's experts received and the experts among them that were hit, counted on the last batch
        ids = device_ids(cfg, batches[0][1], bias)[:, : cfg.topk].contiguous()
        gathered = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        all_ids = torch.cat(gathered).flatten()
        local = all_ids[(all_ids >= rank * n_local) & (all_ids < (rank + 1) * n_local)]
        rows_received, experts_hit = int(local.numel()), int(torch.unique(local).numel())
        record = {"ms_per_step": ms_per_step, "clocks": clocks, "launches": int(launches), "stage_ms": dict(zip(STAGES, stage_ms)),
                  "parity": parity, "rows_received_rank0": rows_received, "experts_hit_rank0": experts_hit}

        if with_e2e:
            # End to end from pinned host buffers through the same surface as one GPU: hidden states in,
            # router GEMM on the device, layer, output back to the host.  Two buffers each way and two
            # copy streams; step i's input copy is enqueued before the host blocks on step i's counts.
            host = [h.cpu().pin_memory() for h, _ in batches]
            dev_hidden = [torch.empty_like(batches[0][0]) for _ in range(2)]
            host_out = [torch.empty((tokens, cfg.hidden), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
            copy_in, copy_out, compute = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
            in_ready = [torch.cuda.Event() for _ in range(2)]
            in_free = [torch.cuda.Event() for _ in range(2)]
            out_free = [torch.cuda.Event() for _ in range(2)]

            def enqueue_input(i):
                k = i & 1
                with torch.cuda.stream(copy_in):
                    copy_in.wait_event(in_free[k])  # the step that last read this buffer is past it
                    dev_hidden[k].copy_(host[i % n_batches], non_blocking=True)
                    in_ready[k].record(copy_in)

            def e2e_step(i):
                k = i & 1
                if i == 0:
                    enqueue_input(0)
                compute.wait_event(in_ready[k])
                enqueue_input(i + 1)  # the next step's copy is in the queue before this step's host read
                result = layer.forward(dev_hidden[k], router_logits(dev_hidden[k], router_w), bias)
                in_free[k].record(compute)
                done = torch.cuda.Event()
                done.record(compute)
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(done)
                    copy_out.wait_event(out_free[k])
                    host_out[k].copy_(result, non_blocking=True)
                    result.record_stream(copy_out)
                    out_free[k].record(copy_out)

            def drain():
                compute.wait_stream(copy_out)
                compute.wait_stream(copy_in)

            for ev in in_free + out_free:
                ev.record(compute)
            for i in range(args.warmup):
                e2e_step(i)
            drain()
            torch.cuda.synchronize()
            for ev in in_free + out_free:
                ev.record(compute)
            record["e2e_ms"] = timed(e2e_step, steps, before_stop=drain)

            # the same copies with no compute between them, all ranks at once: what the box's host memory
            # and PCIe links allow for this pattern
            def copy_only(i):
                k = i & 1
                with torch.cuda.stream(copy_in):
                    dev_hidden[k].copy_(host[i % n_batches], non_blocking=True)
                with torch.cuda.stream(copy_out):
                    host_out[k].copy_(dev_hidden[k], non_blocking=True)

            for i in range(3):
                copy_only(i)
            drain()
            record["copy_only_ms"] = timed(copy_only, steps, before_stop=drain)
        return record

    fp8 = leg(False, args.tokens, args.steps, not args.no_e2e)
    torch.cuda.empty_cache()
    mxfp4 = None if args.headline_only else leg(True, 8192, min(args.steps, 10), False)
    if rank != 0:
        return None

    tokens, ms_per_step, stage_ms = args.tokens, fp8["ms_per_step"], [fp8["stage_ms"][s] for s in STAGES]
    h, inter = cfg.hidden, cfg.inter
    rows, hit = fp8["rows_received_rank0"], fp8["experts_hit_rank0"]
    gate_up_bytes = hit * (2 * inter * h + 4 * (2 * inter // 128) * (h // 128)) + rows * (h + 4 * (h // 128) + inter)
    achieved = gate_up_bytes / (stage_ms[3] * 1e-3) / 1e9 if stage_ms[3] > 0 else 0.0
    line = {
        "metric": METRIC,
        "value": world * tokens / (ms_per_step * 1e-3),
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": workload_config(cfg, args),
        "clocks": fp8["clocks"],
        "tflops": world * tokens * cfg.routes_per_token * cfg.flops_per_route / (ms_per_step * 1e-3) / 1e12,
        "parity": fp8["parity"],
        "e2e": None,
        "gpu_launches": fp8["launches"],
        "roofline": {
            "kernel": "gate_up grouped GEMM over the rows rank 0's experts received",
            "bound": "hbm",
            "achieved": achieved,
            "peak": peak,
            "peak_kind": f"of {peak_kind}",
            "unit": "GB/s",
            "frac": achieved / peak,
            "traffic": gate_up_bytes * TRAFFIC_PER_ALGORITHMIC_BYTE["prefill"],
            "traffic_source": "ncu capture of a smaller case of the same kernel on one GPU, scaled by algorithmic bytes",
            "algorithmic_bytes_per_launch": gate_up_bytes,
            "ms_per_launch": stage_ms[3],
            "tflops": rows * 4 * h * inter / (stage_ms[3] * 1e-3) / 1e12 if stage_ms[3] > 0 else None,
            "stage_ms": fp8["stage_ms"],
            "rows_received": rows,
            "experts_hit": hit,
            "note": "rows and experts counted from the routing of one batch of every rank (rank 0's share)",
        },
        "cpu_baseline": None,
    }
    if "e2e_ms" in fp8:
        line["e2e"] = {
            "value": world * tokens / (fp8["e2e_ms"] * 1e-3),
            "unit": UNIT,
            "ms_per_step": fp8["e2e_ms"],
            "h2d_bytes_per_step": tokens * cfg.hidden * 2,
            "cpu_affinity": args.cpu_affinity,
            "d2h_bytes_per_step": tokens * cfg.hidden * 2,
            "api": "router GEMM + aklr_b200.ep.ExpertParallelMoE.forward per rank, from pinned host hidden states; copies on their own streams",
            "copy_only_ms_per_step": fp8["copy_only_ms"],
            "copy_only_note": "the same H2D + D2H per step on every rank at once with no compute: the floor this box's host memory and PCIe set",
        }
    if mxfp4 is not None:
        t5 = 8192
        line["mxfp4"] = {
            "workload": f"deepseek_v3 widths, mxfp4 weights x mxfp8 activations, {t5} tokens per GPU, ep{world}",
            "ms_per_step": mxfp4["ms_per_step"], "tokens_per_s": world * t5 / (mxfp4["ms_per_step"] * 1e-3),
            "tflops": world * t5 * cfg.routes_per_token * cfg.flops_per_route / (mxfp4["ms_per_step"] * 1e-3) / 1e12,
            "parity": mxfp4["parity"], "clocks": mxfp4["clocks"],
        }
    return json.dumps(line)


if __name__ == "__main__":
    main()
