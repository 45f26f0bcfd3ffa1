#!/usr/bin/env python
"""Benchmark of the hot path: one BERT-base encoder layer (batch 64, seq 384, fp16) per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched with torchrun (one rank per GPU); every rank runs the full workload on its own
GPU (the path shards along M = batch x tokens with no collective, so scaling is "weak") and rank 0
prints ONE JSON line. `value` is sequences per second with inputs resident in HBM, `e2e` the same
metric through Model.run_with_tensors() with pinned host buffers and both copies inside the timed
region. `--impl reference` times the reference's test-oracle expression for the same layer in fp32
on the host cores (the reference's CUDA code generator cannot target sm_100 and its CUTLASS
submodule is not vendored, so its own CPU-side oracle is the reference arm here).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH, SEQ, HIDDEN, HEADS, FFN = 64, 384, 768, 12, 3072
METRIC = "bert_base_layer_seqs_per_sec"
UNIT = "seq/s"
WORKLOAD = "BERT-base encoder layer, fp16, batch 64, seq 384, hidden 768, 12 heads x 64, FFN 3072 (benchmark config 2)"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons while the timed region runs: NVML read-only
    queries from a thread every few milliseconds (the timed region lasts tens of milliseconds), or nvidia-smi in
    a loop when the NVML bindings are missing. Nothing here changes a GPU setting."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None
        self.stop_flag = threading.Event()
        self.sm, self.reasons, self.sm_max = [], set(), None
        self.nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if gpu_index < len(ids) and ids[gpu_index].strip().isdigit():
                    phys = int(ids[gpu_index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception:  # no bindings / no driver access: fall back to nvidia-smi
            self.nvml = None

    def _poll_nvml(self):
        n = self.nvml
        names = {n.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
                 n.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 n.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 n.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(0.002)

    def start(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except (OSError, FileNotFoundError):
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.sm_max,
                    "samples": len(self.sm), "reasons": sorted(self.reasons), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def _cpu_layer_seqs_per_sec(sample_batch: int, min_seconds: float, max_runs: int):
    """Times the fp32 host oracle of the layer on `sample_batch` sequences; returns (seq/s, cores, runs)."""
    import torch

    from aitemplate_b200.testing import workloads
    from oracle import reference_ops

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, params = workloads.bert_layer_inputs(sample_batch, SEQ, HIDDEN, FFN)
    reference_ops.bert_layer(x[:1], params, HEADS)  # warm-up (thread pool, allocator)
    times = []
    t_all = time.perf_counter()
    while len(times) < max_runs and (not times or time.perf_counter() - t_all < min_seconds):
        t0 = time.perf_counter()
        reference_ops.bert_layer(x, params, HEADS)
        times.append(time.perf_counter() - t0)
    return sample_batch / statistics.median(times), cores, len(times)


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    sample = 8
    t0 = time.perf_counter()
    per_step = []
    for _ in range(args.warmup):
        _cpu_layer_seqs_per_sec(sample, 0.0, 1)
    for _ in range(args.steps):
        v, cores, _ = _cpu_layer_seqs_per_sec(sample, 0.0, 1)
        per_step.append(v)
    value = statistics.median(per_step)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * BATCH / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} of {BATCH} sequences per step, fp32 torch oracle, all host threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


PREHEAT_MS = 120.0   # untimed steps (flush + graph replay, the timed pattern) before the first barrier: the clocks
                     # of a freshly leased GPU idle near 340 MHz
LEAD_IN_STEPS = 5    # untimed steps right after the barrier, so the host runs ahead of the GPU in the timed steps


def _bind_to_gpu_numa_node(local_rank: int):
    """Pins this process to the CPUs NVML reports as local to its GPU (read-only query), so that the pinned host
    buffers of the end-to-end pipeline are allocated on that NUMA node: with several ranks per box, copies from a
    remote node share one inter-socket link. Returns the previous affinity (restore it before CPU-side timing)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        phys = local_rank
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            ids = [v for v in visible.split(",") if v.strip()]
            if local_rank < len(ids) and ids[local_rank].strip().isdigit():
                phys = int(ids[local_rank])
        handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        old = os.sched_getaffinity(0)
        cpus &= old
        if cpus and cpus != old:
            os.sched_setaffinity(0, cpus)
            return old
    except Exception:
        pass
    return None


def _gather_rows(dist, row):
    """All ranks contribute one list of floats; every rank gets the [world, len] table."""
    import torch

    t = torch.tensor(row, device="cuda", dtype=torch.float64)
    if dist is None:
        return [t.tolist()]
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


def _load_gemm_traffic():
    """DRAM bytes (read + write) of the four GEMM launches of one step, from the committed ncu summary."""
    path = os.path.join(ROOT, "profiles", "gemm_tc_kernel_bert_layer.md")
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("traffic_bytes_per_step:"):
                    return float(line.split(":", 1)[1].split()[0]), "from_profile"
    except OSError:
        pass
    return None, "no profile summary found"


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch

    from aitemplate_b200 import _lib
    from aitemplate_b200.compiler import compile_model
    from aitemplate_b200.testing import detect_target, workloads

    torch.cuda.set_device(local_rank)
    old_affinity = _bind_to_gpu_numa_node(local_rank) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist

        # in-switch reduction is not needed for a barrier and an all-gather, and ranks here open each other's
        # buffers for the N-split exchange: keep NCCL on plain peer transfers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = _peaks()
    x_cpu, params = workloads.bert_layer_inputs(BATCH, SEQ, HIDDEN, FFN, seed=1334 + rank)
    _, y = workloads.build_bert_layer(BATCH, SEQ, HIDDEN, HEADS, FFN)
    workdir = tempfile.mkdtemp(prefix=f"b200ait_bench_r{rank}_")
    model = compile_model(y, detect_target(), workdir, "bert_layer", num_runtimes=2)
    dev_params = {name: params[key].cuda() for name, key in workloads.BERT_PARAM_NAMES.items()}
    model.set_many_constants_with_tensors(dev_params)
    # device-resident inputs: rotate through several buffers so a step never finds its input in L2
    n_rot = 4
    xs = [x_cpu.cuda() + 0 for _ in range(n_rot)]
    out = torch.empty((BATCH, SEQ, HIDDEN), dtype=torch.float16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB L2
    stream = torch.cuda.current_stream()
    warmup = max(args.warmup, 3)

    def step(i: int, graph: bool = True):
        model.run_with_tensors({"hidden_states": xs[i % n_rot]}, {"output_0": out}, sync=False, graph_mode=graph)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    launches_before = _lib.kernel_launch_count()
    step(0, graph=False)  # one eager step: counts the kernels a step launches (a graph replay re-issues the same nodes)
    torch.cuda.synchronize()
    launches_per_step = _lib.kernel_launch_count() - launches_before
    # preheat: raise the clocks and settle the power state before anything is timed. The clock sampler runs from
    # here to the end of the timed region: the same kernels at the same rate, so its median is the clock under load.
    sampler = ClockSampler(local_rank)
    sampler.start()
    t_pre = time.perf_counter()
    while (time.perf_counter() - t_pre) * 1000.0 < PREHEAT_MS:
        for i in range(20):
            flush.zero_()
            step(i)
        torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput: K steps, each bracketed by events, L2 flushed between steps
    barrier()
    wall0 = time.perf_counter()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for i in range(LEAD_IN_STEPS):
        flush.zero_()
        step(i)
    for i in range(args.steps):
        flush.zero_()
        starts[i].record(stream)
        step(i)
        ends[i].record(stream)
    enqueue_s = time.perf_counter() - wall0
    barrier()
    wall_s = time.perf_counter() - wall0
    clocks = sampler.stop()
    step_ms = sorted(s.elapsed_time(e) for s, e in zip(starts, ends))
    total_ms = sum(step_ms)
    med_ms = statistics.median(step_ms)
    table = _gather_rows(dist, [total_ms, step_ms[0], med_ms, step_ms[int(0.9 * (len(step_ms) - 1))], step_ms[-1],
                                wall_s * 1000.0, enqueue_s * 1000.0, clocks.get("sm_mhz") or 0.0,
                                float(len(clocks.get("reasons", []))), float(len(os.sched_getaffinity(0)))])
    slowest = max(range(world), key=lambda r: table[r][0])
    total_ms = table[slowest][0]
    value = world * BATCH * args.steps / (total_ms / 1000.0)
    per_rank = [{"rank": r, "sum_ms": round(t[0], 3), "step_ms_min": round(t[1], 4), "step_ms_median": round(t[2], 4),
                 "step_ms_p90": round(t[3], 4), "step_ms_max": round(t[4], 4), "wall_ms_between_barriers": round(t[5], 2),
                 "host_enqueue_ms": round(t[6], 2), "sm_mhz_median": t[7], "clock_reasons_seen": int(t[8]), "host_cpus_bound": int(t[9])}
                for r, t in enumerate(table)]

    # ---- end to end through the public API: every step copies its input from pinned host memory to the
    # device, runs Model.run_with_tensors and copies the output back to pinned host memory. The three
    # stages run on three streams over a ring of NB device buffers, so step i+1's upload and step i-1's
    # download overlap step i's kernels; all of it is inside the timed region.
    NB = 3
    x_pins = [x_cpu.pin_memory() for _ in range(2)]
    y_pins = [torch.empty((BATCH, SEQ, HIDDEN), dtype=torch.float16).pin_memory() for _ in range(NB)]
    x_devs = [torch.empty_like(xs[0]) for _ in range(NB)]
    y_devs = [torch.empty_like(out) for _ in range(NB)]
    s_h2d, s_run, s_d2h = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_h2d = [torch.cuda.Event() for _ in range(NB)]
    ev_run = [torch.cuda.Event() for _ in range(NB)]
    ev_d2h = [torch.cuda.Event() for _ in range(NB)]

    def e2e_step(i: int):
        k = i % NB
        with torch.cuda.stream(s_h2d):
            s_h2d.wait_event(ev_run[k])  # the run that last read this input buffer
            x_devs[k].copy_(x_pins[i % 2], non_blocking=True)
            ev_h2d[k].record(s_h2d)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_h2d[k])
            s_run.wait_event(ev_d2h[k])  # the download that last read this output buffer
            model.run_with_tensors({"hidden_states": x_devs[k]}, {"output_0": y_devs[k]},
                                   stream_ptr=s_run.cuda_stream, sync=False, graph_mode=True)
            ev_run[k].record(s_run)
        with torch.cuda.stream(s_d2h):
            s_d2h.wait_event(ev_run[k])
            y_pins[k].copy_(y_devs[k], non_blocking=True)
            ev_d2h[k].record(s_d2h)

    def e2e_join():
        for st in (s_h2d, s_run, s_d2h):
            stream.wait_stream(st)

    for i in range(2 * NB):
        e2e_step(i)
    e2e_join()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for st in (s_h2d, s_run, s_d2h):
        st.wait_event(e0)
    for i in range(args.steps):
        e2e_step(i)
    e2e_join()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    e2e_table = _gather_rows(dist, [e2e_ms])
    e2e_ms = max(t[0] for t in e2e_table)
    y_pin = y_pins[(args.steps - 1) % NB]
    x_pin = x_pins[0]
    h2d_bytes, d2h_bytes = x_pin.numel() * 2, y_pin.numel() * 2
    e2e_value = world * BATCH * args.steps / (e2e_ms / 1000.0)
    checksum = float(y_pin.float().abs().mean())
    for r, t in enumerate(e2e_table):
        per_rank[r]["e2e_ms_per_step"] = round(t[0] / args.steps, 4)
        per_rank[r]["e2e_h2d_gbs"] = round(h2d_bytes * args.steps / (t[0] / 1000.0) / 1e9, 2)
        per_rank[r]["e2e_d2h_gbs"] = round(d2h_bytes * args.steps / (t[0] / 1000.0) / 1e9, 2)

    # ---- N-split variant of the large GEMM (weight rows split over the ranks, one exchange step), once, on a
    # reduced M so that it fits the run: attached to the line so that every multi-GPU run carries it
    nsplit = None
    if world > 1:
        try:
            nsplit = nsplit_forms(dist, rank, world, m=8192, n=8192, k=8192, iters=3)
        except Exception as e:  # never lose the headline line to the side measurement
            nsplit = {"error": f"{type(e).__name__}: {e}"}
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        model.close()
        return

    # ---- rank 0 alone from here on (the other ranks have left; nothing below is inside a timed region)
    if old_affinity is not None:
        os.sched_setaffinity(0, old_affinity)  # the CPU baseline uses every host core
    # roofline of the dominant kernel (the tcgen05 GEMM, 4 launches per step): per-op CUDA-event times from the
    # runtime's profiler (each op timed alone after an L2 flush)
    prof_path = os.path.join(workdir, "profile.json")
    model.profile_with_tensors({"hidden_states": xs[0]}, {"output_0": out}, 20, prof_path)
    with open(prof_path) as f:
        prof = json.load(f)
    gemm_ms, gemm_fl, per_op = 0.0, 0.0, {}
    for name, rec in prof.items():
        per_op[name] = round(rec["ms_per_iter"] * 1000.0, 2)
        if name.startswith("gemm_rcr"):
            ins = rec["input_sizes"]
            mm, kk = int(ins[0][0]), int(ins[0][1])
            nn_ = int(ins[1][0])
            gemm_fl += 2.0 * mm * nn_ * kk
            gemm_ms += rec["ms_per_iter"]
    achieved = gemm_fl / (gemm_ms / 1000.0) / 1e12 if gemm_ms > 0 else None
    # parity of THIS run's batch-64 output: three of its sequences against the CPU oracle
    from oracle import reference_ops

    model.run_with_tensors({"hidden_states": xs[0]}, {"output_0": out}, sync=True, graph_mode=True)
    picks = [0, BATCH // 2 + 5, BATCH - 1]
    want = reference_ops.bert_layer(x_cpu[picks], params, HEADS)
    got = out[picks].float().cpu()
    err = (got - want).abs()
    parity = {"checked": f"sequences {picks} of the batch-{BATCH} graph-mode output vs the fp32 CPU oracle",
              "max_abs_err": float(err.max()), "max_rel_err": float((err / want.abs().clamp_min(1e-2)).max()),
              "tolerance": "atol = rtol = 2e-2 on the whole layer (1e-2 per op)",
              "pass": bool((err <= 2e-2 + 2e-2 * want.abs()).all())}
    cpu_value, cores, runs = _cpu_layer_seqs_per_sec(8, 10.0, 6)
    ops_digest = None
    if world == 1 and not args.no_ops:
        try:
            ops_digest = [compact_op_row(r) for r in ops_rows(peaks, quick=True)]
        except Exception as e:
            ops_digest = [{"error": f"{type(e).__name__}: {e}"}]
    traffic, traffic_src = _load_gemm_traffic()
    ms_per_step = total_ms / args.steps
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "256 MB flush between timed steps; inputs rotate over 4 buffers",
                   "graph_mode": True, "sharding": f"{world} x batch {BATCH}, no collective",
                   "preheat_ms": PREHEAT_MS, "lead_in_steps": LEAD_IN_STEPS},
        "ms_per_step_median_slowest_rank": table[slowest][2], "slowest_rank": slowest,
        "layer_tflops": workloads.bert_layer_flops(BATCH, SEQ, HIDDEN, HEADS, FFN) / (ms_per_step / 1000.0) / 1e12,
        "roofline": {"kernel": "gemm_tc_kernel (4 launches per step)", "bound": "tensor", "achieved": achieved,
                     "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tflops_burst"] if achieved else None,
                     "frac_nominal": achieved / 2250.0 if achieved else None,
                     "peak_source": peaks["source"] + " burst (each kernel timed alone)",
                     "traffic": traffic, "traffic_source": traffic_src,
                     "traffic_unit": "DRAM read + write bytes per step (4 launches); algorithmic bytes 693.6e6",
                     "per_op_us": per_op},
        "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"8 of {BATCH} sequences x {runs} runs, fp32 torch oracle, all host threads"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": d2h_bytes, "ms_per_step": e2e_ms / args.steps,
                "pipeline": "3 streams (upload / run / download), ring of 3 device buffers",
                "output_abs_mean": checksum},
        "parity": parity,
        "gpu_launches": launches_per_step * args.steps,
        "gpu_launches_per_step": launches_per_step,
        "clocks": clocks,
        "per_rank": per_rank,
    }
    if nsplit is not None:
        line["nsplit"] = nsplit
    if ops_digest is not None:
        line["ops"] = ops_digest
    model.close()
    print(json.dumps(line), flush=True)


def _check_sample(sample):
    """Evaluates the CPU oracle on a row's sample. Returns (cpu_ms for the sample, max_abs_err, max_rel_err, pass).
    Inputs are moved to the host first; only the oracle call is timed (median of up to 3 runs, 1 when slow)."""
    import torch

    from oracle import reference_ops as R

    kind = sample["kind"]
    cpu = lambda t: None if t is None else t.detach().float().cpu()  # noqa: E731
    exact = False
    atol = rtol = 1e-2
    if kind == "gemm":
        args = [cpu(sample[k]) for k in ("x", "w", "b", "d0")]
        fn = lambda: R.gemm_rcr(*args, epilogue=sample["epilogue"])  # noqa: E731
    elif kind == "gemm_permute":
        args = [cpu(sample[k]) for k in ("x", "w", "b")]
        fn = lambda: R.gemm_rcr_bias_permute(*args, sample["shape"], "20314")  # noqa: E731
    elif kind == "bmm":
        a, b = cpu(sample["a"]), cpu(sample["b"])
        fn = lambda: R.bmm_rcr(a, b)  # noqa: E731
    elif kind == "attention":
        q, k, v = cpu(sample["q"]), cpu(sample["k"]), cpu(sample["v"])
        fn = lambda: R.mem_eff_attention(q, k, v)  # noqa: E731
    elif kind == "layernorm":
        x, g, bb = cpu(sample["x"]), cpu(sample["gamma"]), cpu(sample["beta"])
        fn = lambda: R.layernorm(x, g, bb, sample["eps"])  # noqa: E731
        atol = rtol = 2e-3
    elif kind == "softmax":
        x = cpu(sample["x"])
        fn = lambda: R.softmax(x, -1)  # noqa: E731
    elif kind == "concatenate":
        parts = [t.cpu() for t in sample["parts"]]
        fn = lambda: R.concatenate(parts, sample["dim"])  # noqa: E731
        exact = True
    elif kind == "split":
        x = sample["x"].cpu()
        fn = lambda: R.split(x, sample["sections"], sample["dim"])  # noqa: E731
        exact = True
    elif kind == "bert_layer":
        fn = lambda: R.bert_layer(sample["x"], sample["params"], sample["heads"])  # noqa: E731
        atol = rtol = 3e-2
    elif kind == "sd_block":
        fn = lambda: R.sd_transformer_block(sample["x"], sample["context"], sample["params"])  # noqa: E731
        atol = rtol = 3e-2
    else:
        raise KeyError(kind)
    times = []
    want = None
    for _ in range(3):
        t0 = time.perf_counter()
        want = fn()
        times.append(time.perf_counter() - t0)
        if sum(times) > 4.0:
            break
    cpu_ms = statistics.median(times) * 1000.0
    got = sample["got"]
    if exact:
        if isinstance(want, (list, tuple)):
            same = all(torch.equal(g.cpu(), w) for g, w in zip(got, want))
        else:
            same = torch.equal(got.cpu(), want)
        return cpu_ms, 0.0 if same else float("nan"), 0.0 if same else float("nan"), bool(same), len(times)
    g = got.detach().float().cpu()
    err = (g - want).abs()
    ok = bool((err <= atol + rtol * want.abs()).all()) and bool(torch.isfinite(g).all())
    return cpu_ms, float(err.max()), float((err / want.abs().clamp_min(atol)).max()), ok, len(times)


def ops_rows(peaks, quick: bool = False, only: str = ""):
    """Per-op rows of the benchmark configurations: GPU time and roofline fractions from the package's sweep, CPU
    time (the oracle expression in fp32 on all host cores, on the row's sample, scaled to the whole op) and the
    error of the kernel's output against that oracle."""
    import torch

    from aitemplate_b200.testing import benchmark_ops

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for row in benchmark_ops.run_suite(peaks, quick=quick, only=only):
        sample = row.pop("_sample", None)
        row["gpu_ms"] = round(row.pop("us") / 1000.0, 5)
        if sample is not None:
            cpu_ms, abs_err, rel_err, ok, runs = _check_sample(sample)
            row.update(cpu_ms=round(cpu_ms * sample["scale"], 2), cpu_cores=cores,
                       cpu_sample=f"{sample['note']} x {runs} run(s), scaled x{sample['scale']:g}",
                       max_abs_err=abs_err, max_rel_err=rel_err)
            row["pass"] = ok
        del sample
        torch.cuda.empty_cache()
        yield row


def compact_op_row(row):
    keep = ("config", "op", "shape", "gpu_ms", "cpu_ms", "cpu_cores", "tflops", "gbs", "frac_measured", "frac_nominal",
            "cublas_linear_us", "cublas_bmm_us", "max_abs_err", "max_rel_err", "pass")
    return {k: row[k] for k in keep if k in row}


def run_ops_suite(args) -> None:
    """Per-op sweep over the benchmark configurations: one JSON line per op (not the driver's contract line)."""
    import torch

    torch.cuda.set_device(0)
    peaks = _peaks()
    for row in ops_rows(peaks, quick=False, only=args.only):
        print(json.dumps(row), flush=True)


def nsplit_forms(dist, rank: int, world: int, m: int, n: int, k: int, iters: int):
    """gemm_rcr_bias_relu [m, k] x [n, k] on `world` GPUs in three partitionings; needs an initialised process group
    when world > 1. Returns the result dict (same on every rank).
      m_sharded      rows split, no collective;
      n_split        weight rows split, X replicated, one NCCL all-gather of the output column shards + re-layout;
      n_split_fused  the GEMM epilogue's TMA stores write every tile into all ranks' row-major Y (peer pointers)."""
    import torch

    from aitemplate_b200 import kernels as K
    from aitemplate_b200 import sharding

    g = torch.Generator(device="cuda").manual_seed(500 + rank)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.01).half()
    b = (torch.randn((n,), generator=g, device="cuda") * 0.01).half()
    start, stop = sharding.shard_range(m, world, rank)
    x_rows = (torch.rand((stop - start, k), generator=g, device="cuda") * 2 - 1).half()
    y_rows = torch.empty((stop - start, n), dtype=torch.float16, device="cuda")
    x_full = (torch.rand((m, k), generator=g, device="cuda") * 2 - 1).half()
    if world > 1:  # the N-split forms need the same X, W and bias on every rank
        for t in (x_full, w, b):
            dist.broadcast(t, 0)
    w_r, b_r = sharding.split_weight_columns(w, b, world, rank)
    y_cols = torch.empty((m, n // world), dtype=torch.float16, device="cuda")
    gathered = torch.empty((world * m, n // world), dtype=torch.float16, device="cuda")

    def timed(fn):
        for _ in range(2):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    ms_m = timed(lambda: K.gemm_rcr(x_rows, w, b, epilogue="relu", out=y_rows))
    ms_gemm = timed(lambda: K.gemm_rcr(x_full, w_r, b_r, epilogue="relu", out=y_cols))
    if world > 1:
        ms_gather = timed(lambda: sharding.gather_columns(y_cols, world, gathered=gathered))
        ms_total = timed(lambda: sharding.gather_columns(
            K.gemm_rcr(x_full, w_r, b_r, epilogue="relu", out=y_cols), world, gathered=gathered))
    else:
        ms_gather, ms_total = 0.0, ms_gemm
    fused = None
    flops = 2.0 * m * n * k
    if world > 1:
        # a rank's timed kernel ends when its own remote stores have completed; no flag or spin between ranks
        ybuf = sharding.PeerBuffer(m, n, torch.float16, rank, world)
        ms_fused = timed(lambda: sharding.gemm_rcr_nsplit_fused(x_full, w_r, b_r, ybuf, "relu"))
        dist.barrier()
        torch.cuda.synchronize()
        want = sharding.gather_columns(K.gemm_rcr(x_full, w_r, b_r, epilogue="relu", out=y_cols), world,
                                       gathered=gathered)
        same = torch.tensor([1 if torch.equal(ybuf.local, want) else 0], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        fused = {"total_ms": ms_fused, "tflops_total": flops / (ms_fused / 1e3) / 1e12,
                 "remote_store_bytes_per_rank": (world - 1) * m * (n // world) * 2,
                 "collective": "none: epilogue TMA stores into peer memory over NVLink",
                 "matches_all_gather_bitwise": bool(same.item())}
        dist.barrier()
        ybuf.close()
    return {
        "workload": f"gemm_rcr_bias_relu M={m} N={n} K={k} fp16", "n_gpus": world,
        "m_sharded": {"ms": ms_m, "tflops_total": flops / (ms_m / 1e3) / 1e12, "collective": None},
        "n_split": {"gemm_ms": ms_gemm, "all_gather_relayout_ms": ms_gather, "total_ms": ms_total,
                    "tflops_total": flops / (ms_total / 1e3) / 1e12,
                    "gathered_bytes_per_rank": (world - 1) * m * (n // world) * 2, "collective": "ncclAllGather"},
        "n_split_fused": fused,
        "matches_all_gather_bitwise": fused["matches_all_gather_bitwise"] if fused else None,
    }


def run_nsplit_suite(args, rank: int, world: int, local_rank: int) -> None:
    """benchmark config 5 at M = 65536, N = K = 8192 on `world` GPUs (see nsplit_forms). Rank 0 prints one JSON line."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    res = nsplit_forms(dist if world > 1 else None, rank, world, 65536, 8192, 8192, max(args.steps // 5, 3))
    if rank == 0:
        print(json.dumps({"suite": "nsplit", **res}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-ops", action="store_true",
                    help="layer suite: leave the per-op digest (GPU time, CPU time, error per op) out of the line")
    ap.add_argument("--only", default="",
                    help="ops suite: run the cases whose label '<config>:<op>:<shape>' contains this, e.g. 5:gemm:16x8192")
    ap.add_argument("--suite", choices=["layer", "ops", "nsplit"], default="layer",
                    help="layer: the contract benchmark (default); ops: per-op sweep; nsplit: config 5 on N GPUs")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.suite == "ops":
        if rank == 0:
            run_ops_suite(args)
        return
    if args.suite == "nsplit":
        run_nsplit_suite(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
