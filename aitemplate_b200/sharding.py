"""Multi-GPU partitioning of the hot path: one process per GPU, no data-path collective for the
M-sharded form, one all-gather for the N-split form.

The reference is a single-GPU compiler (no NCCL / MPI call site anywhere in it), so this file has
no counterpart there. Every op of the path is independent per row of the activation matrix (GEMM
rows, layernorm / softmax rows, attention per (batch, head), bmm per batch), so rank r simply owns
rows [start, stop) of the inputs, residuals and outputs while weights are replicated. The N-split
variant instead replicates X and gives rank r the weight rows (output columns)
[r N / g, (r + 1) N / g); the column blocks are then exchanged with ONE all-gather (NCCL over NVLink
on GPUs, gloo in the CPU tests) into [g, M, N / g] and re-laid out to [M, N] by the bit-exact permute
kernel.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced partition of `total` units: the first total % world ranks get one extra."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, world: int, rank: int, dim: int = 0) -> torch.Tensor:
    """This rank's slice of `x` along `dim` (a view; call .contiguous() before handing it to a kernel)."""
    start, stop = shard_range(x.shape[dim], world, rank)
    return x.narrow(dim, start, stop - start)


def split_weight_columns(w: torch.Tensor, bias: Optional[torch.Tensor], world: int, rank: int):
    """N-split of a gemm_rcr weight [N, K] (and bias [N]): rank r gets output columns r N/g .. (r+1) N/g.
    N must divide evenly so that the gathered blocks have one shape."""
    n = w.shape[0]
    if n % world:
        raise ValueError(f"N = {n} is not divisible by the world size {world}")
    start, stop = shard_range(n, world, rank)
    return w[start:stop].contiguous(), (None if bias is None else bias[start:stop].contiguous())


def _default_relayout(t: torch.Tensor) -> torch.Tensor:
    from . import kernels

    return kernels.permute(t, (1, 0, 2))


def gather_columns(y_local: torch.Tensor, world: int, group=None,
                   relayout: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
                   gathered: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gathers the [M, N/g] column blocks of every rank and returns the full [M, N] result.

    `relayout` turns the gathered [g, M, N/g] tensor into [M, g, N/g]; it defaults to the library's
    permute kernel (CUDA). The CPU tests pass a torch expression, there is no silent fallback."""
    import torch.distributed as dist

    m, n_local = y_local.shape
    if gathered is None:
        gathered = torch.empty((world * m, n_local), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(gathered.view(world * m, n_local), y_local.contiguous(), group=group)
    fn = relayout or _default_relayout
    return fn(gathered.view(world, m, n_local)).reshape(m, world * n_local)
