#!/usr/bin/env python
"""pi0 action-chunk latency benchmark (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload cfg4|cfg5]

A step is one complete pi0 forward (SigLIP x3 views -> Gemma-2B prefix -> Gemma-300M expert x10 Euler steps)
as ONE launch of the persistent sm_100a kernel on synthetic inputs with random-initialised weights.
`value` is the p50 latency in ms with inputs resident in HBM (CUDA events, max over ranks); `e2e` is the same
call through `NativePi0.sample_actions` with pinned HOST buffers (H2D of images/state/noise and D2H of the
actions inside the timed region).  With --gpus N (launched under torchrun) every rank runs an independent
replica on its own GPU: no data-path collective, only a barrier and a MAX reduction of the timings.
`--impl reference` times the CPU restatement of the reference path (oracle/) on the host cores instead: every step
is one whole forward at full depth and full width (no sampling, no extrapolation).

The native line at N = 1 also carries `gpu_baselines` (the BF16 PyTorch restatement of the model on the same GPU with
the same weights and inputs: eager and CUDA-graph replay; `--gpu-baselines eager,graph,compiled` adds
torch.compile(max-autotune-no-cudagraphs), which takes minutes to tune), `accuracy` (action NRMSE of the engine against
that eager model) and, at every N, `replica_cfg5`: the replica-sweep shape of BASELINE.json configs[4] (16-token
prompt, chunk 63) with per-GPU p50 / p90 and the summed actions/s, while `value` stays on configs[3].
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "pizero-megakernel_b200"))
sys.path.insert(0, str(ROOT))

METRIC = "pi0_10step_action_chunk_latency_p50_ms"
# Operand-format presets for --precision (site patterns of NativePi0's `precision` argument)
PRECISIONS = {
    "nvfp4": "nvfp4",
    "qkv_bf16": {"*.qkv": "bf16"},
    "attention_bf16": {"*.qkv": "bf16", "*.o_proj": "bf16", "*.out": "bf16"},
    "expert_bf16": {"expert.*": "bf16"},
    "attention_expert_bf16": {"*.qkv": "bf16", "*.o_proj": "bf16", "*.out": "bf16", "expert.*": "bf16"},
    "bf16": "bf16",
}
WORKLOADS = {
    # BASELINE.json configs[3]: full forward, 3 views, no prompt, chunk 50, 10 Euler steps
    "cfg4": dict(views=3, prompt=0, chunk=50, steps=10, name="configs[3]: full pi0 forward, batch 1, 3 views 224x224, prompt 0, chunk 50, 10 Euler steps"),
    # BASELINE.json configs[4]: replica sweep shape, 16-token prompt, chunk 63
    "cfg5": dict(views=3, prompt=16, chunk=63, steps=10, name="configs[4]: pi0 forward, 3 views, 16-token prompt, chunk 63, 10 Euler steps"),
}
# Algorithmic work of one forward (GEMM + attention FLOPs) and NVFP4 weight bytes read once.
# dram_bytes: dram__bytes_read.sum + dram__bytes_write.sum of one launch from an ncu capture of this bench (3.52 GB read: the
# 1.29 GB of vision/prefix weights once and the 0.17 GB of expert weights in each of the 10 Euler steps, plus scale atoms and
# activations that had left L2; 1.02 GB written: activations and split-KV partials leaving the L2 behind the weight stream).
# None: not captured.
WORK = {"cfg4": dict(gflop=3997.0, weight_mb=1461.0, dram_bytes=4.54e9), "cfg5": dict(gflop=4136.0, weight_mb=1461.0, dram_bytes=None)}
TRAFFIC_SOURCE = "constant from profiles/pi0_vm_kernel_bench_cfg4_launch_list.md (one ncu capture of this command), not measured in this run"
# Dense NVFP4 tensor peak of a B200 as published (9 PFLOP/s; not measured on this pool) and the best rate this engine's
# own NVFP4 GEMM has sustained stand-alone (gate/up + GeGLU, M 768, N 32768, K 2048; profiles/).
NVFP4_NOMINAL_TFLOPS = 9000.0
# Per phase: GEMM + attention GFLOP of one forward, and the NVFP4 weight MB the phase streams (expert: 175.2 MB x 10 steps).
PHASE_WORK = {"cfg4": dict(vision=(660.5, 232.6), prefix=(2958.7, 1053.4), expert=(379.3, 1752.0)),
              "cfg5": dict(vision=(660.5, 232.6), prefix=(3022.1, 1053.4), expert=(478.6, 1752.0))}


# Libraries (NCCL's version banner, for one) write to file descriptor 1 behind Python's back; the contract is ONE JSON
# line on stdout, so everything else that reaches descriptor 1 is sent to stderr and the line goes out on a saved copy.
_JSON_FD = os.dup(1)
os.dup2(2, 1)


def emit(line):
    os.write(_JSON_FD, (json.dumps(line) + "\n").encode())


def percentile(values, q):
    s = sorted(values)
    if not s:
        return float("nan")
    pos = (len(s) - 1) * q
    lo, hi = int(pos), min(int(pos) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (pos - lo)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for t, l in self.lines if t0 <= t <= t1 + 0.2] or [l.split(", ") for _, l in self.lines[-3:]]
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            try:
                sm.append(float(r[1])), mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, r[5:9]):
                if flag.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return p.get("bf16_tflops", 1590.0), p.get("hbm_gbs", 6650.0), "measured (MEASURED_PEAKS.json, burst cuBLAS bf16 / copy)"
    return 1590.0, 6650.0, "fallback (no MEASURED_PEAKS.json on this box)"


def synthetic_inputs(torch, wl, seed, vocab):
    g = torch.Generator(device="cpu").manual_seed(seed)
    images = torch.rand(wl["views"], 224, 224, 3, generator=g) * 2 - 1          # normalised pixels ~U(-1,1)
    state = torch.randn(1, 32, generator=g)
    noise = torch.randn(1, wl["chunk"], 32, generator=g)
    tokens = torch.randint(0, vocab, (1, wl["prompt"]), generator=g, dtype=torch.int64)
    return images, state, noise, tokens


_CPU_CACHE = {}


def cpu_reference_forward(wl, threads):
    """One whole forward of the CPU restatement of the reference path (oracle/pi0_torch.py, FP32 compute): 27 SigLIP,
    18 Gemma-2B and 18 expert layers at full widths, all Euler steps, on `threads` host threads.  The parameter set is
    built once per process (FP32, 13 GB; every layer has tensors of its own, filled from one random block per shape
    times a per-tensor factor, which is as good as independent draws for a timing).  Returns (ms, description)."""
    import torch
    from oracle.pi0_torch import Pi0Dims, Pi0Torch, init_state_dict
    torch.set_num_threads(threads)
    if "model" not in _CPU_CACHE:
        dims = Pi0Dims(vocab=1024)                  # the embedding table is only indexed (16 rows at most): its size is no work
        tiny = Pi0Dims(vision_layers=1, prefix_layers=1, expert_layers=1, vocab=1024)
        seed_sd = init_state_dict(tiny, seed=0, device="cpu", dtype=torch.float32)
        sd = {}
        import re
        for name, block in seed_sd.items():
            m = re.search(r"layers\.0\.", name)
            if not m:
                sd[name] = block
                continue
            count = dims.vision_layers if "vision_tower" in name else dims.prefix_layers if "language_model" in name else dims.expert_layers
            for i in range(count):
                sd[name.replace("layers.0.", f"layers.{i}.")] = block if i == 0 else block * (1.0 + 0.01 * ((i * 7) % 11 - 5))
        model = Pi0Torch(dims, sd, mode="bf16", compute_dtype=torch.float32)
        _CPU_CACHE["model"] = (dims, model)
    dims, model = _CPU_CACHE["model"]
    images, state, noise, tokens = synthetic_inputs(torch, wl, 1, dims.vocab)
    t0 = time.perf_counter()
    out = model.sample_actions(images, state, noise, tokens, steps=wl["steps"])
    ms = (time.perf_counter() - t0) * 1e3
    if not bool(torch.isfinite(out).all()):
        raise RuntimeError("CPU restatement produced non-finite actions")
    sample = (f"oracle/pi0_torch.py, FP32, {threads} host threads: one whole forward per step ({dims.vision_layers}/{dims.prefix_layers}/"
              f"{dims.expert_layers} layers at full widths, {wl['steps']} Euler steps); nothing sampled or extrapolated")
    return ms, sample


def run_reference(args, wl, rank):
    """--impl reference: the CPU restatement of the reference path on all host threads; rank 0 only."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    samples, desc = [], ""
    for i in range(args.warmup + args.steps):
        ms, desc = cpu_reference_forward(wl, threads)
        if i >= args.warmup:
            samples.append(ms)
    value = percentile(samples, 0.5)
    line = {"metric": METRIC, "value": value, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sum(samples) / len(samples), "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": wl["name"], "note": "OpenPI is not installable offline; the reference path is represented by the CPU restatement"},
            "cpu_baseline": {"value": value, "unit": "ms", "cores": threads, "kind": "port", "sample": desc, "estimated": False},
            "e2e": {"value": value, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def time_gpu_callable(torch, call, steps, warmup=3):
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    events[0].record()
    for i in range(steps):
        call()
        events[i + 1].record()
    torch.cuda.synchronize()
    return percentile([events[i].elapsed_time(events[i + 1]) for i in range(steps)], 0.5)


def gpu_baselines(torch, cfg, sd, wl, dev, which, steps):
    """BF16 PyTorch restatement of the model (oracle/pi0_torch.py, mode "bf16") on this GPU with the engine's weights
    and inputs: labelled baselines, never on the engine's path.  Returns (dict, eager actions)."""
    from oracle.pi0_torch import Pi0Dims, Pi0Torch
    dims = Pi0Dims(**{k: getattr(cfg, k) for k in Pi0Dims.__dataclass_fields__ if k != "views" and hasattr(cfg, k)})
    model = Pi0Torch(dims, sd, mode="bf16")
    run = lambda: model.sample_actions(*dev, steps=wl["steps"])
    nrmse = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())
    eager = run().clone()
    out = {"model": "oracle/pi0_torch.py mode=bf16 (PyTorch restatement of OpenPI's model; OpenPI itself is not installable offline)"}
    n = max(3, min(steps, 10))
    if "eager" in which:
        out["eager"] = {"p50_ms": time_gpu_callable(torch, run, n), "action_nrmse_vs_eager": 0.0}
    if "graph" in which:
        try:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(2):
                    run()
            torch.cuda.current_stream().wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                captured = run()
            graph.replay()
            torch.cuda.synchronize()
            out["cuda_graph"] = {"p50_ms": time_gpu_callable(torch, graph.replay, max(n, 10)), "action_nrmse_vs_eager": nrmse(captured, eager)}
            del graph
        except Exception as error:                       # a baseline that cannot be captured is reported, not fatal
            out["cuda_graph"] = {"unavailable": f"{type(error).__name__}: {str(error)[:200]}"}
    if "compiled" in which:
        try:
            compiled = torch.compile(run, mode="max-autotune-no-cudagraphs")
            got = compiled().clone()
            out["compiled"] = {"p50_ms": time_gpu_callable(torch, compiled, n), "action_nrmse_vs_eager": nrmse(got, eager),
                               "mode": "max-autotune-no-cudagraphs"}
        except Exception as error:
            out["compiled"] = {"unavailable": f"{type(error).__name__}: {str(error)[:200]}"}
    return out, eager


def time_engine(torch, dist, engine, dev, pinned, steps, warmup, world, sampler=None):
    """p50 / p90 of `steps` single launches with resident inputs (CUDA events) and p50 through the host-facing call."""
    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        engine.forward(*dev)
    status = engine.status()
    if status["code"]:
        raise RuntimeError(f"device status {status}")
    barrier()
    if sampler:
        sampler.start()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t_begin = time.perf_counter()
    events[0].record()
    for i in range(steps):
        engine.forward(*dev)
        events[i + 1].record()
    barrier()
    t_end = time.perf_counter()
    per_step = [events[i].elapsed_time(events[i + 1]) for i in range(steps)]
    total_ms = events[0].elapsed_time(events[-1])
    # end to end through the host-facing call (pinned host inputs, H2D + D2H inside the timed region)
    for _ in range(2):
        engine.sample_actions(*pinned)
    barrier()
    e2e = []
    for _ in range(steps):
        t0 = time.perf_counter()
        engine.sample_actions(*pinned)
        e2e.append((time.perf_counter() - t0) * 1e3)
    barrier()
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    status = engine.status()
    if status["code"]:
        raise RuntimeError(f"device status {status}")
    return {"p50": percentile(per_step, 0.5), "p90": percentile(per_step, 0.9), "e2e_p50": percentile(e2e, 0.5),
            "total_ms": total_ms, "clocks": clocks}


def run_engine(args, wl, rank, world):
    import torch
    import torch.distributed as dist
    from native_pi0.model import NativePi0
    from native_pi0.weights import Pi0Config, StateDictModel, random_state_dict

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = Pi0Config()
    replica_wl = None if args.no_replica_shape or args.workload == "cfg5" else WORKLOADS["cfg5"]
    need_table = wl["prompt"] > 0 or replica_wl is not None
    sd = random_state_dict(cfg, seed=1234 + rank, device=device, skip_embedding=not need_table)
    model = StateDictModel(cfg, sd)
    engine = NativePi0(model, num_views=wl["views"], prompt_len=wl["prompt"], chunk_size=wl["chunk"], flow_steps=wl["steps"],
                       precision=PRECISIONS[args.precision])
    host = synthetic_inputs(torch, wl, 100 + rank, cfg.vocab)
    pinned = [t.pin_memory() for t in host]
    dev = [t.to(device) for t in host]
    # nvidia-smi numbers physical GPUs; under CUDA_VISIBLE_DEVICES the CUDA ordinal can be another one: query by UUID
    uuid = getattr(torch.cuda.get_device_properties(device), "uuid", None)
    sampler = ClockSampler(f"GPU-{uuid}" if uuid is not None else local)
    timed = time_engine(torch, dist, engine, dev, pinned, args.steps, args.warmup, world, sampler)
    stats = torch.tensor([timed["p50"], timed["p90"], timed["e2e_p50"], timed["total_ms"]], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    p50, p90, e2e_p50, total_ms = stats.tolist()
    clocks = timed["clocks"]
    # ---- per-phase spans of one instrumented launch (rank 0)
    phases = {}
    if rank == 0:
        engine.enable_timings(True)
        engine.forward(*dev)
        torch.cuda.synchronize()
        prof = engine.stage_profile()
        engine.enable_timings(False)
        for name in ("vision", "prefix", "expert"):
            rows = [r for r in prof if r[0].split(".")[0] == name]
            if rows:
                phases[name + "_ms"] = (max(r[2] for r in rows) - min(r[1] for r in rows)) / 1e6
    actions = engine.forward(*dev).clone()
    plan = engine.plan
    policy = engine.precision_policy
    engine.close()
    # ---- BF16 baselines on the same GPU, same weights, same inputs (rank 0, one GPU)
    baselines, accuracy = None, None
    if rank == 0 and world == 1 and args.gpu_baselines:
        baselines, eager = gpu_baselines(torch, cfg, sd, wl, dev, args.gpu_baselines.split(","), args.steps)
        accuracy = {"action_nrmse_vs_bf16_eager": float((actions - eager).norm() / eager.norm()),
                    "note": "random-init weights: W4A4 noise is amplified layer by layer; --precision bf16 gives 0.0023"}
        torch.cuda.empty_cache()
    # ---- the replica-sweep shape (16-token prompt, chunk 63) on every rank
    replica = None
    if replica_wl is not None:
        engine5 = NativePi0(model, num_views=replica_wl["views"], prompt_len=replica_wl["prompt"], chunk_size=replica_wl["chunk"],
                            flow_steps=replica_wl["steps"], precision=PRECISIONS[args.precision])
        host5 = synthetic_inputs(torch, replica_wl, 200 + rank, cfg.vocab)
        t5 = time_engine(torch, dist, engine5, [t.to(device) for t in host5], [t.pin_memory() for t in host5], args.steps, args.warmup, world)
        engine5.close()
        mine = torch.tensor([t5["p50"], t5["p90"], t5["e2e_p50"]], dtype=torch.float64, device=device)
        every = [torch.zeros_like(mine) for _ in range(world)]
        if world > 1:
            dist.all_gather(every, mine)
        else:
            every = [mine]
        rows = [t.tolist() for t in every]
        replica = {"workload": replica_wl["name"], "per_gpu_p50_ms": [r[0] for r in rows], "per_gpu_p90_ms": [r[1] for r in rows],
                   "per_gpu_e2e_p50_ms": [r[2] for r in rows],
                   "actions_per_s": sum(replica_wl["chunk"] * 1e3 / r[0] for r in rows),
                   "actions_per_s_e2e": sum(replica_wl["chunk"] * 1e3 / r[2] for r in rows)}
    del sd, model
    if rank == 0:
        tf_peak, hbm_peak, peak_src = measured_peaks()
        work = WORK[args.workload]
        achieved = work["gflop"] / p50                      # GFLOP / ms == TFLOP/s
        h2d = sum(t.numel() * t.element_size() for t in pinned)
        d2h = actions.numel() * 4
        line = {"metric": METRIC, "value": p50, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": total_ms / args.steps, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
                "dtype": {"nvfp4": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate; bf16 attention, fp32 heads)",
                          "bf16_reference": "bf16 (fp32 accumulate; fp32 heads)"}.get(policy, f"mixed nvfp4 / bf16 sites ({args.precision})"),
                "data": "synthetic",
                "p90_ms": p90, "replica_actions_per_s": world * wl["chunk"] * 1e3 / p50,
                "config": {"workload": wl["name"], "weights": "random-init N(0,0.02), seeded", "parallelism": f"replicas x{world}, no collective",
                           "l2": "weights (1.46 GB NVFP4) exceed the 126 MB L2; no explicit flush", "program": plan,
                           "precision": args.precision},
                "clocks": clocks, "gpu_launches": args.steps,
                "e2e": {"value": e2e_p50, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s", "frac": achieved / tf_peak,
                             "traffic": work["dram_bytes"], "traffic_unit": "bytes per launch", "traffic_source": TRAFFIC_SOURCE,
                             "peak_source": peak_src, "kernel": "pi0_vm_kernel (one launch per step)",
                             "algorithmic_gflop_per_launch": work["gflop"],
                             "frac_of_nvfp4_nominal": achieved / NVFP4_NOMINAL_TFLOPS, "nvfp4_nominal_tflops": NVFP4_NOMINAL_TFLOPS,
                             "nvfp4_peak_note": "the GEMMs run in NVFP4, whose published dense peak is 9 PFLOP/s (not measured here); `peak` is the measured BF16 cuBLAS figure",
                             "weight_stream_gbs": work["weight_mb"] / p50, "hbm_peak_gbs": hbm_peak},
                "phases": phases,
                "phase_roofline": {name: {"tflops": gf / phases[name + "_ms"], "frac_of_bf16_peak": gf / phases[name + "_ms"] / tf_peak,
                                          "frac_of_nvfp4_nominal": gf / phases[name + "_ms"] / NVFP4_NOMINAL_TFLOPS,
                                          "weight_gbs": mb / phases[name + "_ms"], "frac_of_hbm_peak": mb / phases[name + "_ms"] / hbm_peak}
                                   for name, (gf, mb) in PHASE_WORK[args.workload].items() if phases.get(name + "_ms")}}
        if replica is not None:
            line["replica_cfg5"] = replica
        if baselines is not None:
            line["gpu_baselines"] = baselines
            line["accuracy"] = accuracy
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cpu_reference_forward(wl, threads)                               # warm-up: builds the parameter set, starts the thread pool
            samples = [cpu_reference_forward(wl, threads) for _ in range(2)]
            line["cpu_baseline"] = {"value": min(v for v, _ in samples), "unit": "ms", "cores": threads, "kind": "port",
                                    "sample": samples[0][1] + "; best of 2 after one warm-up", "estimated": False}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=("native", "reference"))
    ap.add_argument("--workload", default="cfg4", choices=tuple(WORKLOADS))
    ap.add_argument("--precision", default="nvfp4", choices=tuple(PRECISIONS), help="operand format of the transformer linears")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-replica-shape", action="store_true", help="skip the configs[4] (prompt 16, chunk 63) block")
    ap.add_argument("--gpu-baselines", default="eager,graph", help="comma list of eager, graph, compiled; empty string: none")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl, rank)
        return
    run_engine(args, wl, rank, world)


if __name__ == "__main__":
    main()
