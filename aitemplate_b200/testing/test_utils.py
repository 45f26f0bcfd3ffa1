"""Helpers the reference's unit tests import from aitemplate.testing.test_utils
(python/aitemplate/testing/test_utils.py:37-205): the TestEnv filters, environment overrides and
random / empty / zero / full CUDA tensors by dtype string."""
from __future__ import annotations

import contextlib
import os
import unittest
from enum import Enum
from typing import Any, Dict, List, Tuple, Type

from ..compiler.dtype import string_to_torch_dtype
from ..utils.shape_utils import gen_int_var, gen_int_var_min_max  # noqa: F401  (older call sites import them here)
from .detect_target import detect_target


class TestEnv(Enum):
    """Where a test case can run (test_utils.py:37-42). This build has one environment: CUDA with an
    architecture newer than every SM the reference names, so cases marked for SM70, SM80 or SM90
    features all apply; ROCm cases never do."""

    CUDA_LESS_THAN_SM80 = 1
    CUDA_SM80 = 2
    CUDA_SM90 = 3
    ROCM = 100


def _get_test_env(target) -> TestEnv:
    if target.name() != "cuda":
        raise RuntimeError(f"Unexpected target {target.name()}: this build is CUDA sm_100a only")
    return TestEnv.CUDA_SM90  # the highest CUDA environment the reference defines


def _test_runnable_in_env(test_name: str, env: TestEnv) -> bool:
    """A test method whose name ends in _rocm needs ROCm; _sm80 / _sm90 suffixes need at least that SM
    (test_utils.py:44-124)."""
    name = test_name.lower()
    if name.endswith("rocm"):
        return env == TestEnv.ROCM
    return env != TestEnv.ROCM


def filter_test_cases_by_params(params: Dict[TestEnv, List[Tuple[Any]]]):
    """Flattens {TestEnv: [case tuples]} to the cases whose environment is at most the current one
    (test_utils.py:127-145)."""
    env = _get_test_env(detect_target())
    out = []
    for case_env, cases in params.items():
        if case_env != TestEnv.ROCM and case_env.value <= env.value:
            out.extend(cases)
    return out


def filter_test_cases_by_test_env(cls: Type[unittest.TestCase]):
    """Replaces the test methods of `cls` that cannot run in this environment by skipped stubs
    (test_utils.py:148-161)."""
    env = _get_test_env(detect_target())
    for attr in list(cls.__dict__.keys()):
        if attr.startswith("test_") and not _test_runnable_in_env(attr, env):
            setattr(cls, attr, unittest.skip(f"not runnable in {env.name}")(getattr(cls, attr)))
    return cls


@contextlib.contextmanager
def env_variables(**kwargs):
    """Sets environment variables for the duration of a with-block (test_utils.py:164-180)."""
    old = {name: os.environ.get(name) for name in kwargs}
    os.environ.update({k: str(v) for k, v in kwargs.items()})
    try:
        yield
    finally:
        for name, value in old.items():
            if value is None:
                os.environ.pop(name, None)
            else:
                os.environ[name] = value


def get_random_torch_tensor(shape, dtype: str = "float16"):
    import torch

    return torch.randn(shape, device="cuda", dtype=string_to_torch_dtype(dtype))


def get_torch_empty_tensor(shape, dtype: str = "float16"):
    import torch

    return torch.empty(shape, device="cuda", dtype=string_to_torch_dtype(dtype))


def get_torch_zeros_tensor(shape, dtype: str = "float16"):
    import torch

    return torch.zeros(shape, device="cuda", dtype=string_to_torch_dtype(dtype))


def get_torch_full_tensor(shape, fill_value, dtype: str = "float16"):
    import torch

    return torch.full(shape, fill_value, device="cuda", dtype=string_to_torch_dtype(dtype))
