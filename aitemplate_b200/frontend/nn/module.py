"""Module / Parameter: a minimal torch-like container (python/aitemplate/frontend/nn/module.py:71-745,
parameter.py:19-31). Parameters are graph constants; `name_parameter_tensor()` names each one after
its dotted module path with '.' replaced by '_'."""
from __future__ import annotations

from collections import OrderedDict
from typing import Iterator, List, Optional, Tuple

from ...compiler.base import Tensor


class Parameter:
    def __init__(self, shape, dtype: str = "float16", name: Optional[str] = None, value=None) -> None:
        self._tensor = Tensor(shape=list(shape), dtype=dtype, name=name)
        self._value = value

    def tensor(self) -> Tensor:
        return self._tensor

    def value(self):
        return self._value


class Module:
    def __init__(self) -> None:
        object.__setattr__(self, "_parameters", OrderedDict())
        object.__setattr__(self, "_modules", OrderedDict())

    def __setattr__(self, name, value) -> None:
        if isinstance(value, Parameter):
            self._parameters[name] = value
        elif isinstance(value, Module):
            self._modules[name] = value
        object.__setattr__(self, name, value)

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def named_parameters(self, prefix: str = "", recurse: bool = True) -> Iterator[Tuple[str, Parameter]]:
        for name, p in self._parameters.items():
            yield (prefix + ("." if prefix else "") + name, p)
        if recurse:
            for mname, m in self._modules.items():
                yield from m.named_parameters(prefix + ("." if prefix else "") + mname, True)

    def parameters(self, recurse: bool = True) -> Iterator[Parameter]:
        for _, p in self.named_parameters(recurse=recurse):
            yield p

    def named_modules(self, prefix: str = "") -> Iterator[Tuple[str, "Module"]]:
        yield prefix, self
        for mname, m in self._modules.items():
            yield from m.named_modules(prefix + ("." if prefix else "") + mname)

    def children(self) -> Iterator["Module"]:
        return iter(self._modules.values())

    def name_parameter_tensor(self) -> None:
        for name, p in self.named_parameters():
            p.tensor()._attrs["name"] = name.replace(".", "_")


class ModuleList(Module):
    def __init__(self, modules: Optional[List[Module]] = None) -> None:
        super().__init__()
        for m in modules or []:
            self.append(m)

    def append(self, module: Module) -> "ModuleList":
        setattr(self, str(len(self._modules)), module)
        return self

    def __iter__(self):
        return iter(self._modules.values())

    def __len__(self) -> int:
        return len(self._modules)

    def __getitem__(self, idx: int) -> Module:
        return list(self._modules.values())[idx]


class Sequential(ModuleList):
    def forward(self, x):
        for m in self:
            x = m(x)
        return x
