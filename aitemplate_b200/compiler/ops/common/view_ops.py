"""Zero-copy view ops: reshape, flatten, squeeze, unsqueeze
(python/aitemplate/compiler/ops/common/view_ops.py:111-628). Each returns
`Tensor(is_view_of=x)`; at run time only the shape is evaluated."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from ...base import IntImm, IntVar, IntVarTensor, Operator, Tensor, wrap_dim


def _numel_bounds(shape: List[IntVar]):
    lo = hi = 1
    for d in shape:
        lo *= d.lower_bound()
        hi *= d.upper_bound()
    return lo, hi


class _view(Operator):
    def replace_input_tensor(self, old_tensor, new_tensor) -> None:
        super().replace_input_tensor(old_tensor, new_tensor)
        for out in self._attrs["outputs"] or []:
            if out._attrs["is_view_of"] is old_tensor:
                out._attrs["is_view_of"] = new_tensor

    def _finish(self, x: Tensor, shape: List[IntVar]) -> Tensor:
        self._attrs["inputs"] = [x]
        self._set_depth()
        out = Tensor(shape, src_ops={self}, is_view_of=x, dtype=x.dtype())
        self._attrs["outputs"] = [out]
        return out

    def _lower(self) -> Dict[str, Any]:
        return {"kernel": "view"}


class reshape(_view):
    """reshape()(x, shape): one entry may be -1; entries may be ints, IntImm, IntVar or IntVarTensor."""

    def __init__(self) -> None:
        super().__init__()
        self._attrs["op"] = "reshape"
        self._attrs["unknown_idx"] = -1

    def _infer_shapes(self, x: Tensor, shape: List[Any]) -> List[IntVar]:
        target: List[Optional[IntVar]] = []
        neg = None
        for i, s in enumerate(shape):
            if isinstance(s, IntVarTensor):
                s = s._attrs["int_var"]
            if isinstance(s, IntVar):
                target.append(s)
            elif isinstance(s, int):
                if s == -1:
                    assert neg is None, "Multiple -1 detected in reshape"
                    neg = i
                    target.append(None)
                else:
                    target.append(IntImm(s))
            else:
                raise RuntimeError(f"Unsupported reshape dim: {s}")
        x_shape = x._attrs["shape"]
        x_lo, x_hi = _numel_bounds(x_shape)
        known = [t for t in target if t is not None]
        k_lo, k_hi = _numel_bounds(known)
        x_dyn = [d for d in x_shape if not isinstance(d, IntImm)]
        t_dyn = [d for d in known if not isinstance(d, IntImm)]
        if neg is not None:
            # dynamic dims that appear on both sides cancel; what is left must be static
            rem_x = list(x_dyn)
            leftover = False
            for d in t_dyn:
                if d in rem_x:
                    rem_x.remove(d)
                else:
                    leftover = True
            xs = 1
            for d in x_shape:
                if isinstance(d, IntImm):
                    xs *= d.value()
            ks = 1
            for d in known:
                if isinstance(d, IntImm):
                    ks *= d.value()
            if not rem_x and not leftover:
                if ks == 0:
                    target[neg] = IntImm(0)
                else:
                    assert xs % ks == 0, f"cannot reshape {[d.pseudo_code() for d in x_shape]} into {shape}"
                    target[neg] = IntImm(xs // ks)
            else:
                assert not leftover, "reshape target uses a dynamic dim the input does not have"
                denom_lo = max(ks, 1)
                lo = xs
                hi = xs
                for d in rem_x:
                    lo *= d.lower_bound()
                    hi *= d.upper_bound()
                assert lo % denom_lo == 0 and hi % denom_lo == 0, "reshape -1 does not divide"
                sym = "*".join(str(d._attrs["symbolic_value"]) for d in rem_x) + f"*{xs}/{denom_lo}"
                if len(rem_x) == 1 and xs == denom_lo:
                    target[neg] = rem_x[0]
                else:
                    target[neg] = IntVar([lo // denom_lo, hi // denom_lo], symbolic_value=sym)
                self._attrs["unknown_idx"] = neg
        else:
            assert k_lo <= x_hi and k_hi >= x_lo, f"reshape to {shape} cannot hold the input's elements"
            if not x_dyn and not t_dyn:
                assert x_lo == k_lo, f"reshape: element counts differ ({x_lo} vs {k_lo})"
            new_dyn = [i for i, d in enumerate(target) if not isinstance(d, IntImm) and d not in x_dyn]
            assert len(new_dyn) <= 1, "reshape can infer at most one new dynamic dim"
            if new_dyn:
                self._attrs["unknown_idx"] = new_dyn[0]
        return [t for t in target]

    def __call__(self, x: Tensor, shape: List[Any]) -> Tensor:
        self._attrs["shape"] = list(shape)
        return self._finish(x, self._infer_shapes(x, shape))

    def _inputs_for_pseudo_code(self):
        return [self._attrs["inputs"][0]]


class flatten(_view):
    """flatten(start_dim, end_dim)(x): merges dims start..end (view_ops.py:396-483)."""

    def __init__(self, start_dim: int = 0, end_dim: int = -1) -> None:
        super().__init__()
        self._attrs["op"] = "flatten"
        self._attrs["start"] = start_dim
        self._attrs["end"] = end_dim
        self._attrs["unknown_idx"] = -1

    def _get_op_attributes(self):
        return {"start_dim": self._attrs["start"], "end_dim": self._attrs["end"]}

    def __call__(self, x: Tensor) -> Tensor:
        rank = x._rank()
        start = wrap_dim(self._attrs["start"], rank) if rank else 0
        end = wrap_dim(self._attrs["end"], rank) if rank else 0
        assert start <= end, f"flatten: start_dim {start} > end_dim {end}"
        dims = x._attrs["shape"][start:end + 1]
        lo, hi = _numel_bounds(dims)
        if lo == hi:
            merged: IntVar = IntImm(lo)
        else:
            dyn = [d for d in dims if not isinstance(d, IntImm)]
            static = 1
            for d in dims:
                if isinstance(d, IntImm):
                    static *= d.value()
            merged = dyn[0] if (len(dyn) == 1 and static == 1) else IntVar(
                [lo, hi], symbolic_value="*".join(str(d._attrs["symbolic_value"]) for d in dims))
            self._attrs["unknown_idx"] = start
        shape = list(x._attrs["shape"][:start]) + [merged] + list(x._attrs["shape"][end + 1:])
        return self._finish(x, shape)


class squeeze(_view):
    """squeeze(dim)(x): drops size-1 dims (all of them when dim is None) (view_ops.py:485-584)."""

    def __init__(self, dim: Optional[int]) -> None:
        super().__init__()
        self._attrs["op"] = "squeeze"
        self._attrs["dim"] = dim

    def _get_op_attributes(self):
        return {"dim": self._attrs["dim"]}

    def __call__(self, x: Tensor) -> Tensor:
        dim = self._attrs["dim"]
        shape = x._attrs["shape"]
        if dim is None:
            new = [d for d in shape if d != IntImm(1)]
        else:
            dim = wrap_dim(dim, len(shape))
            new = list(shape)
            if shape[dim] == IntImm(1):
                del new[dim]
        return self._finish(x, new)


class unsqueeze(squeeze):
    """unsqueeze(dim)(x): inserts a size-1 dim (view_ops.py:586-628)."""

    def __init__(self, dim: int) -> None:
        super().__init__(dim)
        self._attrs["op"] = "unsqueeze"

    def __call__(self, x: Tensor) -> Tensor:
        shape = list(x._attrs["shape"])
        dim = self._attrs["dim"]
        if dim < 0:
            dim += len(shape) + 1
        assert 0 <= dim <= len(shape), f"unsqueeze: dim {self._attrs['dim']} out of range"
        shape.insert(dim, IntImm(1))
        return self._finish(x, shape)
