"""Per-op throughput sweep over the benchmark configurations (`python bench.py --suite ops`).

Each row times one op through the C ABI on seeded synthetic inputs: a CUDA graph of `reps` launches
over a rotation of buffer sets larger than L2 (so no launch finds its operands cached), timed with
CUDA events, best of `iters` replays. Reported: microseconds per launch, TFLOP/s or GB/s from the
ALGORITHMIC flops / bytes of the op, and that as a fraction of the measured and of the nominal peak.
The reference's analogue is the per-op profiler loop (python/aitemplate/backend/cuda/gemm_universal/
common.py:439-568: warm-up, timed launches over a rotating memory pool sized to defeat L2).
"""
from __future__ import annotations

import math
import time
from typing import Callable, Dict, List

import torch

from .. import kernels as K

NOMINAL_TFLOPS = 2250.0
NOMINAL_GBS = 8000.0


def _time_graph(fn: Callable[[int], None], reps: int, iters: int = 5) -> float:
    """Milliseconds per call of fn(i), i = 0..reps-1 captured in one CUDA graph."""
    time.sleep(0.2)  # each row is a burst measurement: let the clocks recover from the row before
    fn(0)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn(0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                fn(i)
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps)
    return best


def _rot(nbytes_per_set: int) -> int:
    """How many buffer sets to rotate through so that the working set exceeds the 126 MB L2."""
    return max(2, min(8, math.ceil(300e6 / max(nbytes_per_set, 1))))


def _row(config: str, op: str, shape: str, ms: float, flops: float, nbytes: float, bound: str, peaks: Dict) -> Dict:
    row = {"config": config, "op": op, "shape": shape, "us": round(ms * 1e3, 2), "bound": bound}
    if bound == "tensor":
        tf = flops / (ms * 1e-3) / 1e12
        row.update(tflops=round(tf, 1), frac_measured=round(tf / peaks["tflops_burst"], 3),
                   frac_nominal=round(tf / NOMINAL_TFLOPS, 3))
    else:
        gbs = nbytes / (ms * 1e-3) / 1e9
        row.update(gbs=round(gbs, 1), frac_measured=round(gbs / peaks["hbm_gbs"], 3),
                   frac_nominal=round(gbs / NOMINAL_GBS, 3))
        if flops:
            row["tflops"] = round(flops / (ms * 1e-3) / 1e12, 1)
    return row


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cuda").manual_seed(seed)


def bench_gemm(config: str, m: int, n: int, k: int, epilogue: str, peaks: Dict, residual: bool = False,
               w_scale: float = 0.02, permute=None, seed: int = 1) -> Dict:
    g = _gen(seed)
    nbytes = 2 * (m * k + n * k + n + m * n * (2 if residual else 1))
    sets = _rot(nbytes)
    xs = [(torch.rand((m, k), generator=g, device="cuda") * 2 - 1).half() for _ in range(sets)]
    w = (torch.randn((n, k), generator=g, device="cuda") * w_scale).half()
    b = (torch.randn((n,), generator=g, device="cuda") * w_scale).half()
    ds = [torch.randn((m, n), generator=g, device="cuda").half() for _ in range(sets)] if residual else None
    oshape = (m, n) if permute is None else (permute[1], m // permute[0], permute[2], permute[0], n // (permute[1] * permute[2]))
    outs = [torch.empty(oshape, dtype=torch.float16, device="cuda") for _ in range(sets)]

    def fn(i: int) -> None:
        j = i % sets
        K.gemm_rcr(xs[j], w, b, ds[j] if residual else None, epilogue=epilogue, out=outs[j], permute_shape=permute)

    ms = _time_graph(fn, reps=2 * sets)
    bound = "tensor" if 2.0 * m * n * k / nbytes > 250 else "hbm"
    name = "gemm_rcr_bias" + ("_" + epilogue if epilogue else "") + ("_permute" if permute else "")
    return _row(config, name, f"{m}x{n}x{k}", ms, 2.0 * m * n * k, nbytes, bound, peaks)


def bench_bmm(config: str, batch: int, m: int, n: int, k: int, peaks: Dict) -> Dict:
    g = _gen(2)
    nbytes = 2 * batch * (m * k + n * k + m * n)
    sets = _rot(nbytes)
    a = [(torch.rand((batch, m, k), generator=g, device="cuda") * 2 - 1).half() for _ in range(sets)]
    b = [(torch.rand((batch, n, k), generator=g, device="cuda") * 2 - 1).half() for _ in range(sets)]
    ms = _time_graph(lambda i: K.bmm_rcr(a[i % sets], b[i % sets]), reps=2 * sets)
    return _row(config, "bmm_rcr", f"{batch}x[{m}x{k}].[{n}x{k}]^T", ms, 2.0 * batch * m * n * k, nbytes, "hbm", peaks)


def bench_attention(config: str, b: int, h: int, sq: int, skv: int, d: int, peaks: Dict) -> Dict:
    g = _gen(3)
    nbytes = 2 * b * h * (2 * sq * d + 2 * skv * d)
    sets = _rot(nbytes)
    q = [torch.randn((b, h, sq, d), generator=g, device="cuda").half() for _ in range(sets)]
    k = [torch.randn((b, h, skv, d), generator=g, device="cuda").half() for _ in range(sets)]
    v = [torch.randn((b, h, skv, d), generator=g, device="cuda").half() for _ in range(sets)]
    ms = _time_graph(lambda i: K.mem_eff_attention(q[i % sets], k[i % sets], v[i % sets]), reps=2 * sets)
    return _row(config, "mem_eff_attention", f"B{b} H{h} Sq{sq} Skv{skv} D{d}", ms, 4.0 * b * h * sq * skv * d, nbytes,
                "tensor", peaks)


def bench_layernorm(config: str, m: int, n: int, eps: float, peaks: Dict) -> Dict:
    g = _gen(4)
    nbytes = 2 * (2 * m * n + 2 * n)
    sets = _rot(nbytes)
    xs = [torch.randn((m, n), generator=g, device="cuda").half() for _ in range(sets)]
    gamma = (torch.rand((n,), generator=g, device="cuda") + 0.5).half()
    beta = (torch.randn((n,), generator=g, device="cuda") * 0.1).half()
    ms = _time_graph(lambda i: K.layernorm(xs[i % sets], gamma, beta, eps=eps), reps=2 * sets)
    return _row(config, "layernorm", f"{m}x{n}", ms, 0.0, nbytes, "hbm", peaks)


def bench_softmax(config: str, shape, peaks: Dict) -> Dict:
    g = _gen(5)
    numel = math.prod(shape)
    nbytes = 4 * numel
    sets = 2
    xs = [torch.randn(shape, generator=g, device="cuda").mul_(2).half() for _ in range(sets)]
    ms = _time_graph(lambda i: K.softmax(xs[i % sets], -1), reps=4)
    return _row(config, "softmax", "x".join(map(str, shape)), ms, 0.0, nbytes, "hbm", peaks)


def bench_concat_split(config: str, peaks: Dict) -> List[Dict]:
    g = _gen(6)
    sets = 3
    parts = [[torch.randn((8192, 1024), generator=g, device="cuda").half() for _ in range(4)] for _ in range(sets)]
    cats = [K.concatenate(p, 1) for p in parts]
    nbytes = 2 * 2 * 8192 * 4096
    ms_c = _time_graph(lambda i: K.concatenate(parts[i % sets], 1), reps=2 * sets)
    ms_s = _time_graph(lambda i: K.split(cats[i % sets], [1024] * 4, 1), reps=2 * sets)
    return [_row(config, "concatenate", "4x[8192x1024] dim 1", ms_c, 0.0, nbytes, "hbm", peaks),
            _row(config, "split", "[8192x4096] -> 4 parts", ms_s, 0.0, nbytes, "hbm", peaks)]


def bench_sd_block(config: str, peaks: Dict) -> Dict:
    """The whole Stable-Diffusion UNet transformer block of benchmark configuration 3 through compile_model() and
    Model.benchmark_with_tensors() in graph mode (22 kernels per run)."""
    import tempfile

    from ..compiler import compile_model
    from . import detect_target, workloads

    batch = 2
    x, context, params = workloads.sd_block_inputs(batch)
    y = workloads.build_sd_block(batch)
    module = compile_model(y, detect_target(), tempfile.mkdtemp(prefix="b200ait_sd_"), "sd_block")
    module.set_many_constants_with_tensors({k: v.cuda() for k, v in params.items()})
    out = torch.empty((batch, 4096, 320), dtype=torch.float16, device="cuda")
    ins = {"latent": x.cuda(), "context": context.cuda()}
    module.run_with_tensors(ins, {"output_0": out}, graph_mode=True)
    time.sleep(0.2)
    mean_ms, _, _ = module.benchmark_with_tensors(ins, {"output_0": out}, count=20, repeat=3, graph_mode=True)
    tokens, dim, ctx, cdim = 4096, 320, 77, 768
    gemm = 2.0 * batch * (tokens * dim * dim * 4 + tokens * dim * dim * 2 + 2 * ctx * cdim * dim
                          + 2 * tokens * dim * 4 * dim + tokens * 4 * dim * dim)
    attn = 4.0 * batch * 8 * tokens * (tokens + ctx) * 40
    row = {"config": config, "op": "sd_transformer_block (22 kernels, graph mode)", "shape": "B2 4096x320, ctx 77x768",
           "us": round(mean_ms * 1e3, 2), "bound": "tensor"}
    tf = (gemm + attn) / (mean_ms * 1e-3) / 1e12
    row.update(tflops=round(tf, 1), frac_measured=round(tf / peaks["tflops_burst"], 3),
               frac_nominal=round(tf / NOMINAL_TFLOPS, 3))
    return row


def run_suite(peaks: Dict) -> List[Dict]:
    rows: List[Dict] = []
    rows.append(bench_gemm("1", 256, 3072, 768, "fast_gelu", peaks))
    m2 = 64 * 384
    rows.append(bench_gemm("2", m2, 2304, 768, "", peaks, permute=(384, 3, 12)))
    rows.append(bench_attention("2", 64, 12, 384, 384, 64, peaks))
    rows.append(bench_gemm("2", m2, 768, 768, "add", peaks, residual=True))
    rows.append(bench_layernorm("2", m2, 768, 1e-12, peaks))
    rows.append(bench_gemm("2", m2, 3072, 768, "fast_gelu", peaks))
    rows.append(bench_gemm("2", m2, 768, 3072, "add", peaks, residual=True))
    for n in (768, 1024, 4096):
        rows.append(bench_layernorm("3", 65536, n, 1e-5, peaks))
    rows.append(bench_softmax("3", (512, 1024, 1024), peaks))
    rows.extend(bench_concat_split("3", peaks))
    rows.append(bench_attention("4", 2, 8, 4096, 4096, 40, peaks))
    rows.append(bench_attention("4", 2, 8, 4096, 77, 40, peaks))
    rows.append(bench_gemm("4", 8192, 320, 320, "", peaks))
    rows.append(bench_gemm("4", 8192, 2560, 320, "", peaks))
    rows.append(bench_gemm("4", 8192, 1280, 320, "mul", peaks, residual=True))
    rows.append(bench_gemm("4", 8192, 320, 1280, "add", peaks, residual=True))
    rows.append(bench_layernorm("4", 8192, 320, 1e-5, peaks))
    rows.append(bench_sd_block("4", peaks))
    rows.append(bench_bmm("5", 1024, 512, 512, 64, peaks))
    for m in (1, 16, 128, 1024, 8192, 65536):  # the seconds-long cases last: they leave the GPU power-capped
        rows.append(bench_gemm("5", m, 8192, 8192, "relu", peaks, w_scale=0.01))
    return rows
