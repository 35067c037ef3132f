"""Benchmark of the FP8 fused-MoE layer (DeepSeek-V3 shape) on B200.

    python bench.py --gpus N --steps K --warmup W [--tokens T] [--impl reference]

One step = one layer call over a batch of T tokens per GPU (routing -> sort -> quant -> gate_up ->
down -> combine).  Prints ONE JSON line.  ``value`` is tokens/s with inputs resident in HBM;
``e2e`` is the same through the reference-facing op (``deepseek_v2_fp8_moe``, router GEMM
included) from pinned HOST buffers with both copies timed; ``roofline`` describes the dominant
kernel (the gate_up grouped GEMM); ``cpu_baseline`` is the CPU oracle timed on a bounded sample.
N > 1: expert parallelism, each rank holds n_routed/N routed experts + the shared expert and its
own T tokens (weak scaling); dispatch and combine are NCCL all-to-alls.
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

import torch

ROOT = pathlib.Path(__file__).resolve().parent
# gate_up grouped GEMM: measured DRAM traffic / algorithmic bytes in the ncu captures summarised in
# profiles/grouped_gemm_prefill_t1024_e64.md (2.157 GB / 2.02 GB) and profiles/grouped_gemm_decode_t64_e64.md (ratio 1.01)
TRAFFIC_PER_ALGORITHMIC_BYTE = {"prefill": 1.068, "decode": 1.01}
sys.path.insert(0, str(ROOT))

from aklr_b200 import workloads as wl  # noqa: E402

METRIC = "fp8_fused_moe_tokens_per_s"
UNIT = "tokens/s"
SEED = 2024
FALLBACK_HBM_GBS = 6650.0


def measured_peak_hbm() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


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


def routing_of(cfg):
    from aklr_b200.moe import Routing

    return Routing(cfg.topk, cfg.scoring, cfg.n_shared, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor)


# --------------------------------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline leg and the --impl reference arm)
# --------------------------------------------------------------------------------------------------
class HostExperts:
    """Expert weights on the host, drawn one expert at a time on first use (outside timing)."""

    def __init__(self, cfg, seed, which):
        self.cfg, self.seed, self.which, self.cache = cfg, seed, which, {}

    def prefetch(self, experts):
        for e in experts:
            if e not in self.cache:
                self.cache[e] = wl.one_expert_weights(self.cfg, self.seed, e, "cpu")

    def __getitem__(self, e):
        self.prefetch([e])
        return self.cache[e][self.which]


def oracle_step(cfg, hidden, logits, bias, host, orc):
    ids, w = orc.grouped_sigmoid_topk(
        logits.float(), bias.float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor
    )
    ids, w = orc.with_shared_slot(ids, w, cfg.n_routed)
    return orc.fp8_experts(hidden, ids, w, host[0], host[1], host[2], host[3])


def oracle_experts_hit(cfg, logits, bias, orc):
    ids, _ = orc.grouped_sigmoid_topk(
        logits.float(), bias.float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor
    )
    return sorted(set(ids.flatten().tolist()) | set(range(cfg.n_routed, cfg.n_experts)))


def time_cpu_oracle(cfg, n_tokens, sample_tokens, steps, warmup):
    """Tokens/s of the CPU oracle over ``steps`` calls on ``sample_tokens`` tokens each."""
    from oracle import moe_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    host = [HostExperts(cfg, SEED, i) for i in range(4)]
    for h in host[1:]:
        h.cache = host[0].cache
    batches = []
    for s in range(steps + warmup):
        hidden, logits, bias = wl.router_inputs(cfg, sample_tokens, SEED + 1000 + s)
        host[0].prefetch(oracle_experts_hit(cfg, logits, bias, orc))
        batches.append((hidden, logits, bias))
    for hidden, logits, bias in batches[:warmup]:
        oracle_step(cfg, hidden, logits, bias, host, orc)
    t0 = time.perf_counter()
    for hidden, logits, bias in batches[warmup:]:
        oracle_step(cfg, hidden, logits, bias, host, orc)
    elapsed = time.perf_counter() - t0
    return sample_tokens * steps / elapsed, elapsed, cores


def run_reference_arm(args, cfg):
    """The reference's CPU implementation of the path (its torch reference, restated in oracle/)
    on this box's host cores, on a bounded sample of the workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 1  # tokens per step: one DeepSeek-V3 token visits 9 experts of 44 MB
    value, elapsed, cores = time_cpu_oracle(cfg, args.tokens, sample, args.steps, args.warmup)
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
        "cpu_baseline": {
            "value": value,
            "unit": UNIT,
            "cores": cores,
            "kind": "port",
            "sample": f"{sample} token(s) of the workload per step, {args.steps} steps, expert weights already in host memory",
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, args):
    return {
        "workload": f"deepseek_v3 fp8 fused-moe layer, {args.tokens} tokens per GPU per step",
        "hidden": cfg.hidden,
        "moe_intermediate": cfg.inter,
        "routed_experts": cfg.n_routed,
        "shared_experts": cfg.n_shared,
        "topk": cfg.topk,
        "routing": "sigmoid + correction bias, 8 groups / top-4 groups / top-8, x2.5",
        "weights": "fp8 e4m3, 128x128 fp32 block scales, N(0,0.02)",
        "activations": "bf16 N(0,1), 1x128 fp8 groups",
        "tokens_per_gpu": args.tokens,
        "parallelism": f"ep{args.gpus}" if args.gpus > 1 else "single gpu",
        "l2": "inputs larger than L2: every step streams all expert weights hit (GBs vs 126 MB); batches rotate",
    }


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def distinct_experts(ids: torch.Tensor) -> int:
    return int(torch.unique(ids).numel())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per GPU per step")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="also time decode/prefill token counts (extra keys)")
    ap.add_argument("--sweep-tokens", default="1,16,64,256,1024,16384", help="token counts of --sweep, comma-separated")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling captures)")
    ap.add_argument("--model", default="deepseek_v3", choices=["deepseek_v3", "mixtral", "qwen3"],
                    help="mixtral / qwen3: the other FP8 configurations, one GPU, timed as CUDA-graph replays over their token counts")
    ap.add_argument("--routed-experts", type=int, default=0, help="shrink the layer to this many routed experts (profiling captures only)")
    ap.add_argument("--block-m", type=int, default=0, help="force the tokens-per-block of the grouped GEMMs")
    ap.add_argument("--format", default="fp8", choices=["fp8", "mxfp4"], help="expert weight format (mxfp4: MXFP8 activations)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    cfg = wl.CONFIGS["deepseek_v3"]
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
        from aklr_b200.ep import bench_ep

        line = bench_ep(args, cfg, rank, world, device, ClockSampler, workload_config, METRIC, UNIT, measured_peak_hbm)
        dist.destroy_process_group()
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        if line is not None:
            print(line, flush=True)
        return

    from aklr_b200 import ops
    from aklr_b200.moe import Workspace, _config, fused_moe_fp8

    routing = routing_of(cfg)
    T = args.tokens
    if args.format == "mxfp4":
        bench_mxfp4(args, cfg, routing, device, lib)
        return
    if args.model != "deepseek_v3":
        bench_other_model(args, wl.CONFIGS[args.model], device, lib)
        return
    w1, s1, w2, s2 = wl.expert_weights(cfg, SEED, device)
    router_w = wl.router_weight(cfg, SEED, device)
    n_batches = 4
    batches = []
    for b in range(n_batches):
        hidden, logits, bias = wl.router_inputs(cfg, T, SEED + 1 + b, device)
        batches.append((hidden, logits))
    bias = wl.router_inputs(cfg, 1, SEED + 1, device)[2]
    out = torch.empty((T, cfg.hidden), dtype=torch.bfloat16, device=device)
    ws = Workspace(_config(T, cfg.hidden, cfg.inter, cfg.n_routed, routing, batches[0][1], bias, args.block_m), device)

    def step(i):
        hidden, logits = batches[i % n_batches]
        fused_moe_fp8(hidden, logits, bias, w1, s1, w2, s2, routing, out=out, workspace=ws, block_m=args.block_m)

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
    total_ms = start.elapsed_time(stop)
    ms_per_step = total_ms / args.steps
    ws.check_status()

    stage_names = ["route", "sort", "quant", "gate_up", "down", "combine"]
    stage_ms = [0.0] * 6
    buf = (ctypes.c_float * 6)()
    for i in range(args.steps):
        _lib.check(lib.aklr_profile_read(i, buf))
        for j in range(6):
            stage_ms[j] += buf[j] / args.steps
    lib.aklr_profile_begin(0)

    # ---- roofline of the dominant kernel (gate_up grouped GEMM): algorithmic bytes / its time ----
    ids = ws.topk_ids()
    experts_hit = distinct_experts(ids)
    routes = T * cfg.routes_per_token
    h, i_dim = cfg.hidden, cfg.inter
    gate_up_bytes = experts_hit * (2 * i_dim * h + 4 * (2 * i_dim // 128) * (h // 128)) + routes * h + routes * (h // 128) * 4 + routes * i_dim
    down_bytes = experts_hit * (h * i_dim + 4 * (h // 128) * (i_dim // 128)) + routes * i_dim + routes * h * 2
    peak, peak_kind = measured_peak_hbm()
    achieved = gate_up_bytes / (stage_ms[3] * 1e-3) / 1e9
    flops, layer_bytes = wl.roofline_work(cfg, T, experts_hit)
    token_major = ws.layout.block_m == 128
    # DRAM bytes of this kernel per launch: ncu (dram__bytes_read + dram__bytes_write) on the small
    # capture of the same kernel divided by that capture's algorithmic bytes, times this launch's
    # algorithmic bytes (traffic grows with the weights streamed; see profiles/)
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
        "stage_ms": dict(zip(stage_names, stage_ms)),
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

    e2e = None
    if not args.no_e2e:
        # ---- end to end through the op API from pinned host buffers --------------------------------
        host_hidden = [b[0].cpu().pin_memory() for b in batches]
        host_out = torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory()
        dev_hidden = torch.empty_like(batches[0][0])
        ops.init()

        # Three streams, two buffers each way: step i's H2D overlaps step i-1's compute and step
        # i-2's D2H, as a serving loop would run it.  Every step still copies its own inputs in and
        # its own result out inside the timed region.
        copy_in, copy_out, compute = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        dev_in = [torch.empty_like(batches[0][0]) for _ in range(2)]
        host_outs = [torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        out_ready = [torch.cuda.Event() for _ in range(2)]
        out_free = [torch.cuda.Event() for _ in range(2)]
        results = [None, None]
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
                hidden_states=dev_in[k],
                router_weight=router_w,
                correction_bias=bias,
                w1=w1,
                w1_scale=s1,
                w2=w2,
                w2_scale=s2,
                topk=cfg.topk,
                num_expert_group=cfg.num_expert_group,
                topk_group=cfg.topk_group,
                renormalize=cfg.renormalize,
                scoring_func="sigmoid",
                routed_scaling_factor=cfg.routed_scaling_factor,
            )
            if not isinstance(result, torch.Tensor):
                raise SystemExit(f"the op fell back: {result}")
            results[k] = result
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
        e2e_clocks = e2e_sampler.stop()
        e2e_ms = e0.elapsed_time(e1) / args.steps
        e2e = {
            "value": T / (e2e_ms * 1e-3),
            "unit": UNIT,
            "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": T * cfg.hidden * 2,
            "d2h_bytes_per_step": T * cfg.hidden * 2,
            "api": "aklr_b200.ops.deepseek_v2_fp8_moe (router GEMM included); copies double-buffered on their own streams",
            "clocks": e2e_clocks,
        }

    sweep = None
    if args.sweep:
        sweep = []
        for t_sweep in (int(v) for v in args.sweep_tokens.split(",")):
            bs = [wl.router_inputs(cfg, t_sweep, SEED + 50 + b, device)[:2] for b in range(8)]
            o = torch.empty((t_sweep, cfg.hidden), dtype=torch.bfloat16, device=device)
            wsx = Workspace(_config(t_sweep, cfg.hidden, cfg.inter, cfg.n_routed, routing, bs[0][1], bias), device)
            for k in range(8):  # every batch once outside a capture
                fused_moe_fp8(bs[k][0], bs[k][1], bias, w1, s1, w2, s2, routing, out=o, workspace=wsx)
            torch.cuda.synchronize()
            # one CUDA graph holding 8 layer calls on the rotating batches, replayed: the reference's
            # protocol (graph replay) -- at T <= 16 the host cannot issue 7 launches as fast as they run
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for k in range(8):
                    fused_moe_fp8(bs[k][0], bs[k][1], bias, w1, s1, w2, s2, routing, out=o, workspace=wsx)
            graph.replay()
            n = 2 if t_sweep >= 1024 else 6
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            hit = 0
            torch.cuda.synchronize()
            a.record()
            for k in range(n):
                graph.replay()
            b_.record()
            torch.cuda.synchronize()
            n *= 8
            for k in range(8):
                hit += distinct_experts(orc_free_ids(cfg, bs[k][1], bias)) / 8
            ms = a.elapsed_time(b_) / n
            _, by = wl.roofline_work(cfg, t_sweep, hit)
            fl = t_sweep * cfg.routes_per_token * cfg.flops_per_route
            sweep.append(
                {
                    "tokens": t_sweep,
                    "us_per_call": ms * 1e3,
                    "tokens_per_s": t_sweep / (ms * 1e-3),
                    "experts_hit": hit,
                    "frac_of_hbm_roofline": by / (peak * 1e9) / (ms * 1e-3),
                    "tflops": fl / (ms * 1e-3) / 1e12,
                    "block_m": wsx.layout.block_m,
                    "timing": "cuda graph replay of 8 calls on rotating batches",
                }
            )

    cpu_baseline = None
    if not args.no_cpu_baseline:
        sample, cpu_steps = 2, 2
        v, elapsed, cores = time_cpu_oracle(cfg, T, sample, cpu_steps, 1)
        cpu_baseline = {
            "value": v,
            "unit": UNIT,
            "cores": cores,
            "kind": "port",
            "sample": f"{cpu_steps} calls of {sample} tokens ({elapsed:.1f} s), expert weights already in host memory",
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
        "e2e": e2e,
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
    }
    if sweep is not None:
        line["sweep"] = sweep
    print(json.dumps(line), flush=True)


def bench_mxfp4(args, cfg, routing, device, lib):
    """The same layer with MXFP4 expert weights and MXFP8 activations (one GPU): extra measurement,
    printed as one JSON line of the same shape with ``config.weights`` saying so."""
    from aklr_b200 import _lib
    from aklr_b200.moe import Workspace, _config, fused_moe_mxfp4

    T = args.tokens
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, SEED, device)
    bias = wl.router_inputs(cfg, 1, SEED + 1, device)[2]
    batches = [wl.router_inputs(cfg, T, SEED + 1 + b, device)[:2] for b in range(4)]
    out = torch.empty((T, cfg.hidden), dtype=torch.bfloat16, device=device)
    ws = Workspace(_config(T, cfg.hidden, cfg.inter, cfg.n_routed, routing, batches[0][1], bias, 128), device)

    def step(i):
        hidden, logits = batches[i % 4]
        fused_moe_mxfp4(hidden, logits, bias, w1, s1, w2, s2, routing, out=out, workspace=ws)

    sampler = ClockSampler(device.index or 0)
    for i in range(args.warmup):
        step(i)
    ws.check_status()
    launches0 = lib.aklr_kernel_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    lib.aklr_profile_begin(args.steps)
    sampler.begin()
    start.record()
    for i in range(args.steps):
        step(args.warmup + i)
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = start.elapsed_time(stop) / args.steps
    stage_ms = [0.0] * 6
    buf = (ctypes.c_float * 6)()
    for i in range(args.steps):
        _lib.check(lib.aklr_profile_read(i, buf))
        for k in range(6):
            stage_ms[k] += buf[k] / args.steps
    lib.aklr_profile_begin(0)
    experts_hit = distinct_experts(ws.topk_ids())
    h, inter = cfg.hidden, cfg.inter
    weight_bytes = experts_hit * (3 * h * inter // 2 + 3 * h * inter // 32)
    flops = T * cfg.routes_per_token * cfg.flops_per_route
    peak, kind = measured_peak_hbm()
    config = workload_config(cfg, args)
    config["weights"] = "mxfp4: e2m1 + e8m0 per 32 along K, N(0,0.02)"
    config["activations"] = "bf16 N(0,1), quantised to MXFP8 (e4m3 + e8m0 per 32)"
    print(json.dumps({
        "metric": METRIC.replace("fp8", "mxfp4"), "value": T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp4 x mxfp8", "data": "synthetic", "config": config, "clocks": clocks, "e2e": None,
        "gpu_launches": int(lib.aklr_kernel_launch_count() - launches0),
        "roofline": {"bound": "hbm" if weight_bytes / (peak * 1e9) > flops / 3.2e15 else "tensor",
                     "achieved": weight_bytes / (ms * 1e-3) / 1e9, "peak": peak, "peak_kind": f"of {kind}", "unit": "GB/s",
                     "frac": weight_bytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "tflops": flops / (ms * 1e-3) / 1e12,
                     "note": "whole layer: weight bytes of the experts hit / layer time",
                     "stage_ms": dict(zip(["route", "sort", "quant", "gate_up", "down", "combine"], stage_ms)),
                     "gate_up_tflops": 2 * flops / 3 / (stage_ms[3] * 1e-3) / 1e12 if stage_ms[3] > 0 else None,
                     "down_tflops": flops / 3 / (stage_ms[4] * 1e-3) / 1e12 if stage_ms[4] > 0 else None},
        "cpu_baseline": None,
    }), flush=True)


# token counts the other FP8 configurations are quoted on
OTHER_MODEL_TOKENS = {"mixtral": (1, 16, 64, 256, 1024, 4096), "qwen3": (1, 32, 256, 2048, 8192)}


def bench_other_model(args, cfg, device, lib):
    """Mixtral-8x7B or Qwen3-30B-A3B widths with softmax top-k routing (seeded logits; Qwen3's carry a
    Zipf(1.1) popularity bias), one GPU: every token count as a CUDA graph of 8 layer calls on rotating
    batches, replayed.  One JSON line; ``value`` is the largest token count's throughput."""
    from aklr_b200.moe import Workspace, _config, fused_moe_fp8

    routing = routing_of(cfg)
    w1, s1, w2, s2 = wl.expert_weights(cfg, SEED, device)
    peak, kind = measured_peak_hbm()
    sampler = ClockSampler(device.index or 0)
    launches0 = lib.aklr_kernel_launch_count()
    sweep = []
    sampler.begin()
    for tokens in OTHER_MODEL_TOKENS[args.model]:
        batches = [wl.router_inputs(cfg, tokens, SEED + 50 + b, device)[:2] for b in range(8)]
        out = torch.empty((tokens, cfg.hidden), dtype=torch.bfloat16, device=device)
        ws = Workspace(_config(tokens, cfg.hidden, cfg.inter, cfg.n_routed, routing, batches[0][1], None, args.block_m), device)
        for hidden, logits in batches:  # every batch once outside a capture
            fused_moe_fp8(hidden, logits, None, w1, s1, w2, s2, routing, out=out, workspace=ws, block_m=args.block_m)
        ws.check_status()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for hidden, logits in batches:
                fused_moe_fp8(hidden, logits, None, w1, s1, w2, s2, routing, out=out, workspace=ws, block_m=args.block_m)
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / (args.steps * 8)
        hit = sum(distinct_experts(orc_free_ids(cfg, logits, None)) for _, logits in batches) / 8
        flops, nbytes = wl.roofline_work(cfg, tokens, hit)
        t_hbm, t_tensor = nbytes / (peak * 1e9), flops / 3.2e15
        sweep.append({
            "tokens": tokens, "us_per_call": ms * 1e3, "tokens_per_s": tokens / (ms * 1e-3), "experts_hit": hit,
            "frac_of_hbm_roofline": t_hbm / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
            "bound": "hbm" if t_hbm > t_tensor else "tensor", "block_m": ws.layout.block_m,
        })
    clocks = sampler.stop()
    last = sweep[-1]
    config = workload_config(cfg, args)
    config["workload"] = f"{cfg.name} fp8 fused-moe layer, token counts {[s['tokens'] for s in sweep]}"
    config["routing"] = f"softmax over the top-{cfg.topk} logits" + (", " + wl.zipf_note() if cfg.zipf_s > 0 else "")
    config["timing"] = "cuda graph replay of 8 calls on rotating batches; weights stream from HBM every call"
    print(json.dumps({
        "metric": METRIC, "value": last["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": last["us_per_call"] * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3", "data": "synthetic", "config": config, "clocks": clocks, "e2e": None,
        "gpu_launches": int(lib.aklr_kernel_launch_count() - launches0),
        "roofline": {"bound": last["bound"], "achieved": last["frac_of_hbm_roofline"] * peak, "peak": peak, "peak_kind": f"of {kind}",
                     "unit": "GB/s", "frac": last["frac_of_hbm_roofline"], "traffic": None,
                     "note": "whole layer at the largest token count: algorithmic bytes / layer time"},
        "cpu_baseline": None, "sweep": sweep,
    }), flush=True)


def orc_free_ids(cfg, logits, bias):
    """Routing ids of a batch computed by the routing kernel itself (for experts-hit counts)."""
    from aklr_b200.moe import route

    return route(logits, bias, routing_of(cfg))[0]


if __name__ == "__main__":
    main()
