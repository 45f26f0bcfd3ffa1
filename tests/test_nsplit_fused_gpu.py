"""Two-GPU parity of the fused N-split exchange: each rank computes one column block of
Y = relu(X W^T + b) and its GEMM epilogue stores every tile into BOTH ranks' Y (own memory + the peer's
through a CUDA IPC mapping). Skipped on a box with a single GPU; the single-GPU form of the same kernel
path (several destinations in local memory) is tests/test_gemm_gpu.py::test_multi_destination_store.
"""
import os
import socket

import pytest
import torch

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, n: int, k: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from aitemplate_b200 import kernels, sharding

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator().manual_seed(77)
        x = (torch.rand((m, k), generator=g) * 2 - 1).half()
        w = (torch.randn((n, k), generator=g) * 0.05).half()
        b = (torch.randn((n,), generator=g) * 0.1).half()
        want = oracle.gemm_rcr(x, w, b, epilogue="relu")
        w_r, b_r = sharding.split_weight_columns(w.cuda(), b.cuda(), world, rank)
        y = sharding.PeerBuffer(m, n, torch.float16, rank, world)
        y.local.fill_(-7.0)
        torch.cuda.synchronize()
        dist.barrier()
        sharding.gemm_rcr_nsplit_fused(x.cuda(), w_r, b_r, y, "relu")
        torch.cuda.synchronize()
        dist.barrier()  # both ranks' kernels, and so their remote stores, are complete
        got = y.local.float().cpu()
        err = (got - want).abs()
        ok = bool((err <= 1e-2 + 1e-2 * want.abs()).all()) and kernels.device_status() == 0
        results[rank] = (ok, float(err.max()))
        dist.barrier()
        y.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("m,n,k", [(1024, 1024, 512), (4096, 2048, 1024)])
def test_fused_nsplit_two_ranks(m, n, k):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, m, n, k, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert all(results[r][0] for r in range(2)), dict(results)
