"""gemm_rcr family graph nodes: Y = epilogue(X @ W^T + bias, D0, D1), X [..., K], W [N, K].

API and `_attrs` follow the reference op classes:
  gemm (base)               python/aitemplate/compiler/ops/gemm_universal/gemm_common.py:198-838
  gemm_rcr                  .../gemm_rcr.py:26-153
  gemm_rcr_bias             .../gemm_rcr_bias.py:27-153
  gemm_rcr_bias_<act>       .../gemm_rcr_bias_relu.py:39-43 (and _gelu, _fast_gelu, _sigmoid, _tanh, _swish, _hardswish)
  gemm_rcr_bias_broadcast   .../gemm_rcr_bias_broadcast.py:27-74 and its subclasses (_add, _add_relu, _mul, ...)
  gemm_rcr_bias_permute     .../gemm_rcr_bias_permute.py:30-75
  gemm_rcr_permute          .../gemm_rcr_permute.py
There is no profiler: tile selection happens inside the library at launch.
"""
from __future__ import annotations

from typing import Any, Dict, List, Tuple

from ...base import IntImm, IntVar, Operator, Tensor
from ...tensor_accessor import TensorAccessor
from ..common.view_ops import reshape

# epilogue name -> (u1, b1, b2, u2) codes of include/b200ait.h
_U = {"identity": 0, "relu": 1, "gelu": 2, "fast_gelu": 3, "sigmoid": 4, "tanh": 5, "swish": 6, "hardswish": 7}
_B = {None: 0, "add": 1, "mul": 2}


def epilogue_code(u1="identity", b1=None, b2=None, u2="identity") -> int:
    return _U[u1] | (_B[b1] << 4) | (_B[b2] << 6) | (_U[u2] << 8)


class gemm(Operator):
    """Base GEMM operator."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "gemm"
        self._attrs["has_profiler"] = False
        self._attrs["f_ab_alignment"] = None
        self._attrs["epilogue_alignment"] = 1
        self._attrs["epilogue"] = "LinearCombination"
        self._attrs["workspace"] = 0
        self._attrs["split_k"] = 1
        self._attrs["num_sources"] = 0
        self._attrs["alpha"] = 1.0
        self._attrs["permute_shape"] = ""
        self._epi = ("identity", None, None, "identity")
        self._has_bias = False

    def _infer_shapes(self, a: Tensor, b: Tensor) -> List[IntVar]:
        raise NotImplementedError

    def _sanity_check(self, a: Tensor, b: Tensor) -> None:
        a_shape, b_shape = a._attrs["shape"], b._attrs["shape"]
        if len(a_shape) < 2:
            raise RuntimeError(f"gemm operand A should have >= 2 dimensions! Current shape: {a_shape}.")
        if len(b_shape) != 2:
            raise RuntimeError(f"gemm operand B should have 2 dimensions! Current shape: {b_shape}.")
        if a.dtype() != b.dtype():
            raise RuntimeError(f"gemm operand A and B should have the same data type! {a.dtype()} vs {b.dtype()}")

    def _align_ab(self, a: Tensor, b: Tensor) -> Tuple[Tensor, Tensor]:
        return a, b

    def _finish(self, inputs: List[Tensor], output_shape: List[IntVar]) -> Tensor:
        self._attrs["inputs"] = inputs
        self._attrs["input_accessors"] = [TensorAccessor(t) for t in inputs]
        self._set_depth()
        out = Tensor(output_shape, src_ops={self}, dtype=inputs[0].dtype())
        self._attrs["outputs"] = [out]
        self._attrs["output_accessors"] = [TensorAccessor(out)]
        return out

    def _lower(self) -> Dict[str, Any]:
        ins = self._attrs["inputs"]
        a, b = ins[0], ins[1]
        idx = 2
        bias = d0 = d1 = None
        if self._has_bias:
            bias = ins[idx]
            idx += 1
        if self._attrs["num_sources"] >= 1:
            d0 = ins[idx]
            idx += 1
        if self._attrs["num_sources"] >= 2:
            d1 = ins[idx]
        store_mode, t = 0, (1, 1, 1)
        if self._attrs.get("layout") == "Permute5D_20314":
            store_mode, t = 1, tuple(self._attrs["shape"])
        elif self._attrs.get("layout") == "Permute4D_0213":
            store_mode, t = 2, tuple(self._attrs["shape"]) + (1,)
        acc = self._attrs["output_accessors"][0]
        n = b._attrs["shape"][0].value()
        out_stride = acc.row_stride() if acc.stride_dim is not None else n
        # operand A read in place from a column block of a wider buffer (a fused split): the operand tensor is an
        # alias that starts at the block, so only the row stride is needed; 0 = contiguous rows of K
        a_acc = self._attrs["input_accessors"][0]
        a_stride = a_acc.row_stride() if a_acc.stride_dim is not None else 0
        b_acc = self._attrs["input_accessors"][1]  # the same for operand B ([N, K] only: a block of K columns)
        b_stride = b_acc.row_stride() if b_acc.stride_dim is not None else 0
        return {
            "kernel": "gemm_rcr",
            "operands": [a, b, bias, d0, d1],
            # ints 7, 8: tile width and split-K picked by the compile-time profiler; 0 = the library decides at run
            # time from the actual M. The `split_k` attribute's default of 1 is the reference's placeholder for "not
            # profiled yet" (gemm_common.py:579-594), not a request to never split.
            "ints": [epilogue_code(*self._epi), store_mode, t[0], t[1], t[2], acc.offset, out_stride,
                     int(self._attrs.get("tile_n", 0)) if self._attrs.get("profiled") else 0,
                     int(self._attrs.get("split_k", 0)) if self._attrs.get("profiled") else 0, a_stride, b_stride],
            "floats": [float(self._attrs["alpha"])],
        }


class gemm_rcr(gemm):
    """y = F.linear(a, b): a [..., K] row-major, b [N, K]."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "gemm_rcr"

    def _infer_shapes(self, a: Tensor, b: Tensor) -> List[IntVar]:
        return list(a._attrs["shape"][:-1]) + [b._attrs["shape"][0]]

    def _align_ab(self, a: Tensor, b: Tensor):
        a_shape, b_shape = a._attrs["shape"], b._attrs["shape"]
        if a_shape[-1] != b_shape[-1]:
            raise RuntimeError(f"A/B shape mismatch! A: {a_shape}, B: {b_shape}")
        if not isinstance(a_shape[-1], IntImm):
            raise RuntimeError(f"K must be static! k: {a_shape[-1]}")
        if not isinstance(b_shape[0], IntImm):
            raise RuntimeError(f"N must be static! n: {b_shape[0]}")
        return a, b

    def __call__(self, a: Tensor, b: Tensor) -> Tensor:
        a, b = self._align_ab(a, b)
        self._sanity_check(a, b)
        return self._finish([a, b], self._infer_shapes(a, b))


class gemm_rcr_bias(gemm_rcr):
    """y = F.linear(a, b, bias); bias is a static 1-D tensor of length N."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "gemm_rcr_bias"
        self._has_bias = True

    @staticmethod
    def _check_bias(b: Tensor, bias: Tensor) -> None:
        bias_shape = bias._attrs["shape"]
        if len(bias_shape) != 1:
            raise RuntimeError(f"Bias should be 1D vector! Current bias shape: {bias_shape}")
        if not isinstance(bias_shape[0], IntImm):
            raise RuntimeError(f"Bias should be fixed 1D vector! Current bias shape: {bias_shape}")
        if bias_shape[0] != b._attrs["shape"][0]:
            raise RuntimeError(f"bias length {bias_shape[0].value()} != N {b._attrs['shape'][0]}")

    def __call__(self, a: Tensor, b: Tensor, bias: Tensor) -> Tensor:
        a, b = self._align_ab(a, b)
        self._sanity_check(a, b)
        self._check_bias(b, bias)
        return self._finish([a, b, bias], self._infer_shapes(a, b))


def _activation_variant(suffix: str, unary: str, epilogue_name: str):
    def __init__(self) -> None:
        gemm_rcr_bias.__init__(self)
        self._attrs["op"] = f"gemm_rcr_bias_{suffix}"
        self._attrs["epilogue"] = epilogue_name
        self._epi = (unary, None, None, "identity")

    return type(f"gemm_rcr_bias_{suffix}", (gemm_rcr_bias,), {
        "__init__": __init__,
        "__doc__": f"y = {suffix}(F.linear(a, b, bias)), activation fused in the GEMM epilogue.",
    })


gemm_rcr_bias_relu = _activation_variant("relu", "relu", "LinearCombinationRelu")
gemm_rcr_bias_gelu = _activation_variant("gelu", "gelu", "LinearCombinationGELU")
gemm_rcr_bias_fast_gelu = _activation_variant("fast_gelu", "fast_gelu", "LinearCombinationFastGELU")
gemm_rcr_bias_sigmoid = _activation_variant("sigmoid", "sigmoid", "LinearCombinationSigmoid")
gemm_rcr_bias_tanh = _activation_variant("tanh", "tanh", "LinearCombinationTanh")
gemm_rcr_bias_swish = _activation_variant("swish", "swish", "LinearCombinationSilu")
gemm_rcr_bias_hardswish = _activation_variant("hardswish", "hardswish", "LinearCombinationHardSwish")


class gemm_rcr_fast_gelu(gemm_rcr):
    """y = fast_gelu(F.linear(a, b)) (python/aitemplate/compiler/ops/gemm_universal/gemm_rcr_fast_gelu.py)."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "gemm_rcr_fast_gelu"
        self._attrs["epilogue"] = "LinearCombinationFastGELU"
        self._epi = ("fast_gelu", None, None, "identity")


class gemm_rcr_bias_broadcast(gemm_rcr_bias):
    """Base of the bias + residual epilogues: y = U2(B2(B1(U1(a b^T + bias), d0), d1))."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["epilogue"] = "LinearCombinationResidualBlock"

    def _check_sources(self, out_shape: List[IntVar], sources: List[Tensor]) -> None:
        for i, d in enumerate(sources):
            if d._attrs["shape"] != out_shape:
                raise RuntimeError(
                    f"Tensor d{i} shape should be the same as the output shape! "
                    f"d{i}: {[x.pseudo_code() for x in d._attrs['shape']]}, output: {[x.pseudo_code() for x in out_shape]}")

    def __call__(self, a: Tensor, b: Tensor, bias: Tensor, d0: Tensor, d1: Tensor = None) -> Tensor:
        a, b = self._align_ab(a, b)
        self._sanity_check(a, b)
        self._check_bias(b, bias)
        sources = [d0] if d1 is None else [d0, d1]
        if len(sources) != self._attrs["num_sources"]:
            raise RuntimeError(f"{self._attrs['op']} takes {self._attrs['num_sources']} residual tensor(s)")
        out_shape = self._infer_shapes(a, b)
        self._check_sources(out_shape, sources)
        return self._finish([a, b, bias] + sources, out_shape)


def _broadcast_variant(suffix: str, u1, b1, b2, u2):
    def __init__(self) -> None:
        gemm_rcr_bias_broadcast.__init__(self)
        self._attrs["op"] = f"gemm_rcr_bias_{suffix}"
        self._attrs["num_sources"] = 1 if b2 is None else 2
        self._epi = (u1, b1, b2, u2)

    return type(f"gemm_rcr_bias_{suffix}", (gemm_rcr_bias_broadcast,), {
        "__init__": __init__,
        "__doc__": f"gemm_rcr_bias followed by the '{suffix}' residual epilogue, fused.",
    })


gemm_rcr_bias_add = _broadcast_variant("add", "identity", "add", None, "identity")
gemm_rcr_bias_add_relu = _broadcast_variant("add_relu", "identity", "add", None, "relu")
gemm_rcr_bias_add_add = _broadcast_variant("add_add", "identity", "add", "add", "identity")
gemm_rcr_bias_add_add_relu = _broadcast_variant("add_add_relu", "identity", "add", "add", "relu")
gemm_rcr_bias_mul = _broadcast_variant("mul", "identity", "mul", None, "identity")
gemm_rcr_bias_mul_add = _broadcast_variant("mul_add", "identity", "mul", "add", "identity")
gemm_rcr_bias_mul_tanh = _broadcast_variant("mul_tanh", "identity", "mul", None, "tanh")
gemm_rcr_bias_sigmoid_mul = _broadcast_variant("sigmoid_mul", "sigmoid", "mul", None, "identity")
gemm_rcr_bias_sigmoid_mul_tanh = _broadcast_variant("sigmoid_mul_tanh", "sigmoid", "mul", None, "tanh")


class gemm_rcr_bias_permute(gemm_rcr_bias):
    """GEMM + bias whose [M, N] result is stored as [M/t1, t1, t2, t3, N/(t2 t3)].permute(2, 0, 3, 1, 4);
    returns that 5-D tensor [t2, M/t1, t3, t1, N/t3/t2]."""

    def __init__(self, shape: Tuple[int, ...], layout: str = "20314") -> None:
        super().__init__()
        if layout != "20314":
            raise NotImplementedError(f"{layout} is not implemented!")  # m2n3 / m3n2 are ROCm-only layouts
        self._attrs["op"] = "gemm_rcr_bias_permute"
        self._attrs["shape"] = tuple(shape)
        self._attrs["layout"] = f"Permute5D_{layout}"
        self._attrs["permute_shape"] = "_".join(map(str, shape))

    def _get_op_attributes(self):
        return {"layout": self._attrs["layout"].split("_")[-1], "shape": self._attrs["shape"]}

    def __call__(self, a: Tensor, b: Tensor, bias: Tensor) -> Tensor:
        a, b = self._align_ab(a, b)
        self._sanity_check(a, b)
        self._check_bias(b, bias)
        out_shape = self._infer_shapes(a, b)
        if len(out_shape) != 2 or not all(isinstance(d, IntImm) for d in out_shape):
            raise RuntimeError("gemm_rcr_bias_permute needs a static 2-D problem")
        out = self._finish([a, b, bias], out_shape)
        m, n = out_shape
        t1, t2, t3 = self._attrs["shape"]
        if m.value() % t1 or n.value() % (t2 * t3):
            raise RuntimeError(f"permute shape {self._attrs['shape']} does not divide M={m.value()}, N={n.value()}")
        return reshape()(out, [t2, m.value() // t1, t3, t1, n.value() // t3 // t2])


class gemm_rcr_permute(gemm_rcr):
    """GEMM whose [M, N] result is stored as [M/t1, t1, t2, N/t2].permute(0, 2, 1, 3) (layout "0213")."""

    def __init__(self, shape: Tuple[int, ...], layout: str = "0213") -> None:
        super().__init__()
        if layout != "0213":
            raise NotImplementedError(f"{layout} is not implemented!")
        self._attrs["op"] = "gemm_rcr_permute"
        self._attrs["shape"] = tuple(shape)
        self._attrs["layout"] = f"Permute4D_{layout}"
        self._attrs["permute_shape"] = "_".join(map(str, shape))

    def _get_op_attributes(self):
        return {"layout": self._attrs["layout"].split("_")[-1], "shape": self._attrs["shape"]}

    def __call__(self, a: Tensor, b: Tensor) -> Tensor:
        a, b = self._align_ab(a, b)
        self._sanity_check(a, b)
        out_shape = self._infer_shapes(a, b)
        if len(out_shape) != 2 or not all(isinstance(d, IntImm) for d in out_shape):
            raise RuntimeError("gemm_rcr_permute needs a static 2-D problem")
        out = self._finish([a, b], out_shape)
        m, n = out_shape
        t1, t2 = self._attrs["shape"]
        if m.value() % t1 or n.value() % t2:
            raise RuntimeError(f"permute shape {self._attrs['shape']} does not divide M={m.value()}, N={n.value()}")
        return reshape()(out, [m.value() // t1, t2, t1, n.value() // t2])


# ---- row-major B ("rrr"): Y = X @ W + bias with W stored [K, N]
# (python/aitemplate/compiler/ops/gemm_universal/gemm_rrr.py:26-80, gemm_rrr_bias.py). Same kernel; the runtime
# hands the tensor core W as an MN-major operand.


class gemm_rrr(gemm):
    """y = a @ b: a [..., K] row-major, b [K, N] row-major."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "gemm_rrr"

    def _infer_shapes(self, a: Tensor, b: Tensor) -> List[IntVar]:
        return list(a._attrs["shape"][:-1]) + [b._attrs["shape"][1]]

    def _check_ab(self, a: Tensor, b: Tensor) -> None:
        a_shape, b_shape = a._attrs["shape"], b._attrs["shape"]
        self._sanity_check(a, b)
        if a_shape[-1] != b_shape[0]:
            raise RuntimeError(f"A/B shape mismatch! A: {a_shape}, B: {b_shape}")
        if not isinstance(b_shape[0], IntImm) or not isinstance(b_shape[1], IntImm):
            raise RuntimeError(f"K and N must be static! B: {b_shape}")

    def __call__(self, a: Tensor, b: Tensor) -> Tensor:
        self._check_ab(a, b)
        return self._finish([a, b], self._infer_shapes(a, b))

    def _lower(self) -> Dict[str, Any]:
        low = super()._lower()
        b = self._attrs["inputs"][1]
        acc = self._attrs["output_accessors"][0]
        n = b._attrs["shape"][1].value()
        low["kernel"] = "gemm_rrr"
        low["ints"][6] = acc.row_stride() if acc.stride_dim is not None else n
        return low


class gemm_rrr_bias(gemm_rrr):
    """y = a @ b + bias; bias is a static 1-D tensor of length N."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "gemm_rrr_bias"
        self._has_bias = True

    def __call__(self, a: Tensor, b: Tensor, bias: Tensor) -> Tensor:
        self._check_ab(a, b)
        bias_shape = bias._attrs["shape"]
        if len(bias_shape) != 1:
            raise RuntimeError(f"Bias should be 1D vector! Current bias shape: {bias_shape}")
        if bias_shape[0] != b._attrs["shape"][1]:
            raise RuntimeError(f"bias length {bias_shape[0]} does not match N {b._attrs['shape'][1]}")
        return self._finish([a, b, bias], self._infer_shapes(a, b))
