"""Timing of an eager PyTorch callable with CUDA events (python/aitemplate/testing/benchmark_pt.py:22-58)."""


def benchmark_torch_function(iters: int, function, *args, **kwargs) -> float:
    """Milliseconds per call: 5 warm-up calls, then `iters` calls between two CUDA events."""
    import torch

    for _ in range(5):
        function(*args, **kwargs)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        function(*args, **kwargs)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters
