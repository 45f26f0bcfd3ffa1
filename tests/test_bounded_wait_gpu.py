"""The bounded wait of the pipeline kernels, made to run out once.

Every mbarrier wait in the GEMM and attention kernels goes through one helper that gives up after a
time limit, records a code in the device status word and lets the kernel return. A healthy run
never takes that branch, so the library carries a self-test kernel (csrc/selftest.cu): the same
helper compiled with a 1 ms limit, waiting on a barrier nobody arrives on. It gives up and returns;
nothing faults, traps or hangs. The test checks what the host sees afterwards: the status code, that
reading it clears it, that a synchronous Run turns a pending code into an error, and that the
context and the model stay usable.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _selftest():
    from aitemplate_b200 import _lib

    out = (ctypes.c_int64 * 3)()
    code = _lib.load().b200ait_selftest_bounded_wait(out, torch.cuda.current_stream().cuda_stream)
    assert code == 0, _lib.last_error()
    return list(out)


def test_wait_runs_out_and_reports_status():
    from aitemplate_b200 import kernels

    assert kernels.device_status() == 0
    gave_up, later, ns = _selftest()
    assert gave_up == 0, "the wait on a barrier nobody arrives on must give up"
    assert later == 0, "once the CTA's abort flag is up, later waits return at once"
    assert 0.9e6 <= ns <= 50e6, f"gave up after {ns} ns; the limit is 1 ms"
    assert kernels.device_status() == 5  # kDevWaitOtherTimeout
    assert kernels.device_status() == 0  # reading it cleared it
    # the context is intact: ordinary kernels run and are clean
    x = torch.randn((64, 64), device="cuda").half()
    y = kernels.gemm_rcr(x, x, None)
    assert torch.isfinite(y.float()).all()
    assert kernels.device_status() == 0


def test_synchronous_run_surfaces_a_pending_status_then_recovers(tmp_path):
    from aitemplate_b200.compiler import compile_model, ops
    from aitemplate_b200.frontend import Tensor
    from aitemplate_b200.testing import detect_target

    x = Tensor([32, 64], name="x", is_input=True)
    w = Tensor([48, 64], name="w", is_input=True)
    y = ops.gemm_rcr()(x, w)
    y._attrs["name"] = "y"
    y._attrs["is_output"] = True
    module = compile_model(y, detect_target(), str(tmp_path), "after_timeout")
    xt, wt = torch.randn((32, 64), device="cuda").half(), torch.randn((48, 64), device="cuda").half()
    out = torch.empty((32, 48), dtype=torch.float16, device="cuda")
    module.run_with_tensors({"x": xt, "w": wt}, {"y": out})
    _selftest()  # leaves code 5 in the status word
    with pytest.raises(RuntimeError):
        module.run_with_tensors({"x": xt, "w": wt}, {"y": out}, sync=True)
    res = module.run_with_tensors({"x": xt, "w": wt}, {"y": out}, sync=True)  # the error cleared the word
    want = xt.float() @ wt.float().t()
    assert float((res["y"].float() - want).abs().max()) < 5e-2
    module.close()
