"""Per-op throughput sweep over the benchmark configurations (`python bench.py --suite ops`).

Each row times one op through the C ABI on seeded synthetic inputs: a CUDA graph of `reps` launches
over a rotation of buffer sets larger than L2 (so no launch finds its operands cached), timed with
CUDA events, best of `iters` replays. Reported: microseconds per launch, TFLOP/s or GB/s from the
ALGORITHMIC flops / bytes of the op, and that as a fraction of the measured and of the nominal peak.
Each row also carries a `_sample`: a slice of the op's independent units (rows, batches, heads) with
the inputs that produced it and the kernel's output for it, plus the factor by which the whole op is
larger. The caller (bench.py) evaluates its CPU checker on the sample, which gives the row its
cpu_ms and its error columns; this package itself never touches a CPU implementation.
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


def _unit_sample(n: int, take: int) -> torch.Tensor:
    """`take` unit indices out of n: the first, the last, the rest spread evenly (device tensor)."""
    if take >= n:
        return torch.arange(n, device="cuda")
    idx = torch.linspace(0, n - 1, take, device="cuda").round().long()
    return torch.unique(idx)


def bench_gemm(config: str, m: int, n: int, k: int, epilogue: str, peaks: Dict, residual: bool = False,
               w_scale: float = 0.02, permute=None, seed: int = 1, sample_flops: float = 1.2e12) -> Dict:
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
    row = _row(config, name, f"{m}x{n}x{k}", ms, 2.0 * m * n * k, nbytes, bound, peaks)
    # the vendor library on the same buffers, for comparison only: F.linear = cuBLAS GEMM + bias, WITHOUT the
    # activation / residual / permuted store this op fuses
    ms_lib = _time_graph(lambda i: torch.nn.functional.linear(xs[i % sets], w, b), reps=2 * sets, iters=3)
    row["cublas_linear_us"] = round(ms_lib * 1e3, 2)
    fn(0)
    torch.cuda.synchronize()
    if permute is None:
        take = min(m, max(1, int(sample_flops // (2.0 * n * k))))
        rows = _unit_sample(m, take)
        row["_sample"] = {"kind": "gemm", "x": xs[0][rows], "w": w, "b": b, "d0": ds[0][rows] if residual else None,
                          "epilogue": epilogue, "got": outs[0][rows], "scale": m / take,
                          "note": f"{take} of {m} rows"}
    else:  # whole sequences (t1 rows each) so that the permuted output can be sliced along its batch dim
        t1 = permute[0]
        nseq = m // t1
        take = min(nseq, max(1, int(sample_flops // (2.0 * t1 * n * k))))
        seqs = _unit_sample(nseq, take)
        rows = (seqs[:, None] * t1 + torch.arange(t1, device="cuda")[None, :]).reshape(-1)
        row["_sample"] = {"kind": "gemm_permute", "x": xs[0][rows], "w": w, "b": b, "shape": permute,
                          "got": outs[0][:, seqs], "scale": nseq / take, "note": f"{take} of {nseq} sequences"}
    return row


def bench_bmm(config: str, batch: int, m: int, n: int, k: int, peaks: Dict) -> Dict:
    g = _gen(2)
    nbytes = 2 * batch * (m * k + n * k + m * n)
    sets = _rot(nbytes)
    a = [(torch.rand((batch, m, k), generator=g, device="cuda") * 2 - 1).half() for _ in range(sets)]
    b = [(torch.rand((batch, n, k), generator=g, device="cuda") * 2 - 1).half() for _ in range(sets)]
    ms = _time_graph(lambda i: K.bmm_rcr(a[i % sets], b[i % sets]), reps=2 * sets)
    row = _row(config, "bmm_rcr", f"{batch}x[{m}x{k}].[{n}x{k}]^T", ms, 2.0 * batch * m * n * k, nbytes, "hbm", peaks)
    ms_lib = _time_graph(lambda i: torch.bmm(a[i % sets], b[i % sets].transpose(1, 2)), reps=2 * sets, iters=3)
    row["cublas_bmm_us"] = round(ms_lib * 1e3, 2)
    y = K.bmm_rcr(a[0], b[0])
    idx = _unit_sample(batch, min(batch, 128))
    row["_sample"] = {"kind": "bmm", "a": a[0][idx], "b": b[0][idx], "got": y[idx], "scale": batch / idx.numel(),
                      "note": f"{idx.numel()} of {batch} batches"}
    return row


def bench_attention(config: str, b: int, h: int, sq: int, skv: int, d: int, peaks: Dict) -> Dict:
    g = _gen(3)
    nbytes = 2 * b * h * (2 * sq * d + 2 * skv * d)
    sets = _rot(nbytes)
    q = [torch.randn((b, h, sq, d), generator=g, device="cuda").half() for _ in range(sets)]
    k = [torch.randn((b, h, skv, d), generator=g, device="cuda").half() for _ in range(sets)]
    v = [torch.randn((b, h, skv, d), generator=g, device="cuda").half() for _ in range(sets)]
    ms = _time_graph(lambda i: K.mem_eff_attention(q[i % sets], k[i % sets], v[i % sets]), reps=2 * sets)
    row = _row(config, "mem_eff_attention", f"B{b} H{h} Sq{sq} Skv{skv} D{d}", ms, 4.0 * b * h * sq * skv * d, nbytes,
               "tensor", peaks)
    o = K.mem_eff_attention(q[0], k[0], v[0])  # [B, Sq, H, D]
    idx = _unit_sample(b, min(b, max(1, int(6e9 // (4.0 * h * sq * skv * d)))))
    row["_sample"] = {"kind": "attention", "q": q[0][idx], "k": k[0][idx], "v": v[0][idx], "got": o[idx],
                      "scale": b / idx.numel(), "note": f"{idx.numel()} of {b} batches"}
    return row


def bench_layernorm(config: str, m: int, n: int, eps: float, peaks: Dict) -> Dict:
    g = _gen(4)
    nbytes = 2 * (2 * m * n + 2 * n)
    sets = _rot(nbytes)
    xs = [torch.randn((m, n), generator=g, device="cuda").half() for _ in range(sets)]
    gamma = (torch.rand((n,), generator=g, device="cuda") + 0.5).half()
    beta = (torch.randn((n,), generator=g, device="cuda") * 0.1).half()
    ms = _time_graph(lambda i: K.layernorm(xs[i % sets], gamma, beta, eps=eps), reps=2 * sets)
    row = _row(config, "layernorm", f"{m}x{n}", ms, 0.0, nbytes, "hbm", peaks)
    y = K.layernorm(xs[0], gamma, beta, eps=eps)
    rows = _unit_sample(m, min(m, 8192))
    row["_sample"] = {"kind": "layernorm", "x": xs[0][rows], "gamma": gamma, "beta": beta, "eps": eps, "got": y[rows],
                      "scale": m / rows.numel(), "note": f"{rows.numel()} of {m} rows"}
    return row


def bench_softmax(config: str, shape, peaks: Dict) -> Dict:
    g = _gen(5)
    numel = math.prod(shape)
    nbytes = 4 * numel
    sets = 2
    xs = [torch.randn(shape, generator=g, device="cuda").mul_(2).half() for _ in range(sets)]
    ms = _time_graph(lambda i: K.softmax(xs[i % sets], -1), reps=4)
    row = _row(config, "softmax", "x".join(map(str, shape)), ms, 0.0, nbytes, "hbm", peaks)
    y = K.softmax(xs[0], -1)
    take = max(1, shape[0] // 8)
    idx = _unit_sample(shape[0], take)
    row["_sample"] = {"kind": "softmax", "x": xs[0][idx], "got": y[idx], "scale": shape[0] / idx.numel(),
                      "note": f"{idx.numel()} of {shape[0]} outer slices"}
    return row


def bench_concat_split(config: str, peaks: Dict) -> List[Dict]:
    g = _gen(6)
    sets = 3
    parts = [[torch.randn((8192, 1024), generator=g, device="cuda").half() for _ in range(4)] for _ in range(sets)]
    cats = [K.concatenate(p, 1) for p in parts]
    nbytes = 2 * 2 * 8192 * 4096
    ms_c = _time_graph(lambda i: K.concatenate(parts[i % sets], 1), reps=2 * sets)
    ms_s = _time_graph(lambda i: K.split(cats[i % sets], [1024] * 4, 1), reps=2 * sets)
    r_c = _row(config, "concatenate", "4x[8192x1024] dim 1", ms_c, 0.0, nbytes, "hbm", peaks)
    r_s = _row(config, "split", "[8192x4096] -> 4 parts", ms_s, 0.0, nbytes, "hbm", peaks)
    r_c["_sample"] = {"kind": "concatenate", "parts": parts[0], "dim": 1, "got": K.concatenate(parts[0], 1),
                      "scale": 1.0, "note": "whole tensor, bit-exact"}
    r_s["_sample"] = {"kind": "split", "x": cats[0], "sections": [1024] * 4, "dim": 1,
                      "got": K.split(cats[0], [1024] * 4, 1), "scale": 1.0, "note": "whole tensor, bit-exact"}
    return [r_c, r_s]


def bench_sd_block(config: str, peaks: Dict) -> Dict:
    """The whole Stable-Diffusion UNet transformer block of benchmark configuration 3 through compile_model() and
    Model.benchmark_with_tensors() in graph mode; the row's label carries the kernels one run launches."""
    import tempfile

    from .. import _lib
    from ..compiler import compile_model
    from . import detect_target, workloads

    batch = 2
    x, context, params = workloads.sd_block_inputs(batch)
    y = workloads.build_sd_block(batch)
    module = compile_model(y, detect_target(), tempfile.mkdtemp(prefix="b200ait_sd_"), "sd_block")
    module.set_many_constants_with_tensors({k: v.cuda() for k, v in params.items()})
    out = torch.empty((batch, 4096, 320), dtype=torch.float16, device="cuda")
    ins = {"latent": x.cuda(), "context": context.cuda()}
    launches = _lib.kernel_launch_count()
    module.run_with_tensors(ins, {"output_0": out}, graph_mode=False)
    launches = _lib.kernel_launch_count() - launches
    module.run_with_tensors(ins, {"output_0": out}, graph_mode=True)
    time.sleep(0.2)
    mean_ms, _, _ = module.benchmark_with_tensors(ins, {"output_0": out}, count=20, repeat=3, graph_mode=True)
    tokens, dim, ctx, cdim = 4096, 320, 77, 768
    gemm = 2.0 * batch * (tokens * dim * dim * 4 + tokens * dim * dim * 2 + 2 * ctx * cdim * dim
                          + 2 * tokens * dim * 4 * dim + tokens * 4 * dim * dim)
    attn = 4.0 * batch * 8 * tokens * (tokens + ctx) * 40
    row = {"config": config, "op": f"sd_transformer_block ({launches} kernels, graph mode)", "shape": "B2 4096x320, ctx 77x768",
           "us": round(mean_ms * 1e3, 2), "bound": "tensor"}
    tf = (gemm + attn) / (mean_ms * 1e-3) / 1e12
    row.update(tflops=round(tf, 1), frac_measured=round(tf / peaks["tflops_burst"], 3),
               frac_nominal=round(tf / NOMINAL_TFLOPS, 3))
    res = module.run_with_tensors(ins, {"output_0": out}, graph_mode=True)
    row["_sample"] = {"kind": "sd_block", "x": x, "context": context, "params": params, "got": res["output_0"],
                      "scale": 1.0, "note": "whole block"}
    return row


def bench_bert_layer(config: str, batch: int, peaks: Dict) -> Dict:
    """One BERT-base encoder layer at a small batch (the reference's benchmark walks batch sizes from 1 up,
    examples/03_bert/benchmark_ait.py:263-300) through compile_model() and graph mode: the latency side of the
    benchmark configuration whose throughput the layer suite measures at batch 64."""
    import tempfile

    from .. import _lib
    from ..compiler import compile_model
    from . import detect_target, workloads

    seq, hidden, heads, ffn = 384, 768, 12, 3072
    x, params = workloads.bert_layer_inputs(batch, seq, hidden, ffn)
    _, y = workloads.build_bert_layer(batch, seq, hidden, heads, ffn)
    module = compile_model(y, detect_target(), tempfile.mkdtemp(prefix="b200ait_bert_"), f"bert_layer_b{batch}")
    module.set_many_constants_with_tensors({name: params[key].cuda() for name, key in workloads.BERT_PARAM_NAMES.items()})
    out = torch.empty((batch, seq, hidden), dtype=torch.float16, device="cuda")
    ins = {"hidden_states": x.cuda()}
    launches = _lib.kernel_launch_count()
    module.run_with_tensors(ins, {"output_0": out}, graph_mode=False)
    launches = _lib.kernel_launch_count() - launches
    module.run_with_tensors(ins, {"output_0": out}, graph_mode=True)
    time.sleep(0.2)
    mean_ms, _, _ = module.benchmark_with_tensors(ins, {"output_0": out}, count=50, repeat=3, graph_mode=True)
    row = {"config": config, "op": f"bert_layer ({launches} kernels, graph mode)", "shape": f"B{batch} S{seq} H{hidden}",
           "us": round(mean_ms * 1e3, 2), "bound": "tensor"}
    tf = workloads.bert_layer_flops(batch, seq, hidden, heads, ffn) / (mean_ms * 1e-3) / 1e12
    row.update(tflops=round(tf, 1), frac_measured=round(tf / peaks["tflops_burst"], 3),
               frac_nominal=round(tf / NOMINAL_TFLOPS, 3))
    res = module.run_with_tensors(ins, {"output_0": out}, graph_mode=True)
    row["_sample"] = {"kind": "bert_layer", "x": x, "params": params, "heads": heads, "got": res["output_0"],
                      "scale": 1.0, "note": "whole layer"}
    return row


def run_suite(peaks: Dict, quick: bool = False, only: str = ""):
    """Yields one row per op of the benchmark configurations. quick=True shrinks the CPU-side samples (not the GPU
    problems) so that the whole sweep, CPU checks included, stays within about a minute. `only` keeps the cases
    whose label ("<config>:<op>:<shape>", e.g. "5:gemm:16x8192x8192") contains it - for a profiler capture of one
    kernel without the rest of the sweep in front of it."""
    sf = 2.5e11 if quick else 1.2e12
    for label, case in _suite_cases(peaks, sf):
        if only and only not in label:
            continue
        rows = case()
        for r in rows if isinstance(rows, list) else [rows]:
            yield r


def _suite_cases(peaks: Dict, sf: float):
    """(label, thunk) per case, in running order; nothing touches the GPU until a thunk is called."""
    cases = []

    def gemm(config, m, n, k, epilogue, **kw):
        cases.append((f"{config}:gemm:{m}x{n}x{k}", lambda: bench_gemm(config, m, n, k, epilogue, peaks, **kw)))

    def attention(config, b, h, sq, skv, d):
        cases.append((f"{config}:attention:{b}x{h}x{sq}x{skv}x{d}", lambda: bench_attention(config, b, h, sq, skv, d, peaks)))

    def layernorm(config, m, n, eps):
        cases.append((f"{config}:layernorm:{m}x{n}", lambda: bench_layernorm(config, m, n, eps, peaks)))

    gemm("1", 256, 3072, 768, "fast_gelu")
    m2 = 64 * 384
    gemm("2", m2, 2304, 768, "", permute=(384, 3, 12))
    attention("2", 64, 12, 384, 384, 64)
    gemm("2", m2, 768, 768, "add", residual=True)
    layernorm("2", m2, 768, 1e-12)
    gemm("2", m2, 3072, 768, "fast_gelu")
    gemm("2", m2, 768, 3072, "add", residual=True)
    for batch in (1, 4, 16):
        cases.append((f"2:bert_layer:B{batch}", lambda batch=batch: bench_bert_layer("2", batch, peaks)))
    for n in (768, 1024, 4096):
        layernorm("3", 65536, n, 1e-5)
    cases.append(("3:softmax:512x1024x1024", lambda: bench_softmax("3", (512, 1024, 1024), peaks)))
    cases.append(("3:concat_split", lambda: list(bench_concat_split("3", peaks))))
    attention("4", 2, 8, 4096, 4096, 40)
    attention("4", 2, 8, 4096, 77, 40)
    gemm("4", 8192, 320, 320, "")
    gemm("4", 8192, 2560, 320, "")
    gemm("4", 8192, 1280, 320, "mul", residual=True)
    gemm("4", 8192, 320, 1280, "add", residual=True)
    layernorm("4", 8192, 320, 1e-5)
    cases.append(("4:sd_transformer_block", lambda: bench_sd_block("4", peaks)))
    cases.append(("5:bmm:1024x512x512x64", lambda: bench_bmm("5", 1024, 512, 512, 64, peaks)))
    for m in (1, 16, 128, 1024, 8192, 65536):  # the seconds-long cases last: they leave the GPU power-capped
        gemm("5", m, 8192, 8192, "relu", w_scale=0.01, sample_flops=sf)
    return cases
