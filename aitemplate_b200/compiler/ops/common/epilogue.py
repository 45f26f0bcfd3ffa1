"""Element-wise function ids (python/aitemplate/compiler/ops/common/epilogue.py:32-70; same values)."""
from enum import Enum


class EpilogueOp(Enum):
    NA = 1
    BIAS = 2
    BIAS_RELU = 3
    BIAS_RELU_ADD = 4


class FuncEnum(Enum):
    ADD = 1
    SUB = 2
    MUL = 3
    DIV = 4
    TANH = 5
    COS = 6
    SIN = 7
    SIGN = 8
    ABS = 9
    LOGE = 10
    EXP = 11
    SQRT = 12
    MAX = 13
    MIN = 14
    SIGMOID = 15
    LRELU = 16
    HARDTANH = 17
    RELU = 18
    NAN_TO_NUM = 19
    CLAMP_NAN_TO_NUM = 20
    SILU = 21
    POW = 22
    GELU = 23
    FASTGELU = 24
    SOFTPLUS = 25
    ELU = 26
    SOFTSIGN = 27
    FLOOR_DIV = 28
    CELU = 29
    FLOOR = 30
    LOG1P = 31
    RECIPROCAL = 32
