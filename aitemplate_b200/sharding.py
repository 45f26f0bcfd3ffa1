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


class PeerBuffer:
    """A [rows, cols] device matrix on every rank of a one-node group, each rank holding pointers to all of
    them (CUDA IPC through the library's b200ait_peer_* entry points; the 64-byte handles travel over the
    process group). `ptrs[r]` is the address of rank r's matrix as seen from this process, `local` this rank's
    matrix as a torch tensor (a view of the same memory, not a copy)."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, rank: int, world: int, group=None) -> None:
        import ctypes

        import torch.distributed as dist

        from . import _lib

        self._lib = _lib.load()
        self.rank, self.world, self.shape, self.dtype = rank, world, (rows, cols), dtype
        nbytes = rows * cols * torch.empty((), dtype=dtype).element_size()
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.check(self._lib.b200ait_peer_alloc(nbytes, ctypes.byref(ptr), handle), "b200ait_peer_alloc")
        self._own = ptr.value
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs, self._opened = [], []
        for r, h in enumerate(handles):
            if r == rank:
                self.ptrs.append(self._own)
                continue
            q = ctypes.c_void_p()
            _lib.check(self._lib.b200ait_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(q)),
                       "b200ait_peer_open")
            self.ptrs.append(q.value)
            self._opened.append(q.value)
        self.local = _tensor_from_ptr(self._own, (rows, cols), dtype)

    def column_ptrs(self, col0: int) -> list:
        """Addresses of column `col0` of row 0 in every rank's matrix, this rank's first."""
        esz = torch.empty((), dtype=self.dtype).element_size()
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self.ptrs[r] + col0 * esz for r in order]

    def close(self) -> None:
        import ctypes

        for q in self._opened:
            self._lib.b200ait_peer_close(ctypes.c_void_p(q))
        self._opened = []
        if self._own is not None:
            self.local = None
            self._lib.b200ait_peer_free(ctypes.c_void_p(self._own))
            self._own = None


def _tensor_from_ptr(ptr: int, shape, dtype: torch.dtype) -> torch.Tensor:
    """A torch view of device memory this process did not allocate through torch."""

    class _Holder:
        pass

    esz = torch.empty((), dtype=dtype).element_size()
    numel = 1
    for d in shape:
        numel *= d
    typestr = {torch.float16: "<f2", torch.bfloat16: "<V2", torch.float32: "<f4"}[dtype]
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (numel,), "typestr": "<f2" if esz == 2 else typestr, "data": (ptr, False),
                                  "version": 3}
    t = torch.as_tensor(h, device="cuda")
    if dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t.view(*shape)


def gemm_rcr_nsplit_fused(x: torch.Tensor, w_shard: torch.Tensor, bias_shard: Optional[torch.Tensor], y: PeerBuffer,
                          epilogue: str = "") -> None:
    """N-split GEMM whose epilogue is the exchange step: this rank computes the column block
    [rank N/g, (rank + 1) N/g) of Y = epilogue(X W^T + b) and its TMA stores place every tile in ALL ranks'
    Y (own memory and peers' over NVLink) while the next tile is computed. The caller synchronises the ranks
    before reading Y (every rank's kernel must have finished)."""
    from . import kernels

    n_local = w_shard.shape[0]
    kernels.gemm_rcr_multi_out(x, w_shard, bias_shard, y.column_ptrs(y.rank * n_local), y.shape[1], epilogue=epilogue)
