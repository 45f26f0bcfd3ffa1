"""Model: Python binding of the native model container.

Same public methods as the reference binding (python/aitemplate/compiler/model.py:172-1118), over the
same C ABI (include/model_interface.h). `lib_path` names the plan file compile_model() wrote; the
shared library itself is the prebuilt libb200ait.so. Any non-zero status from the library raises
RuntimeError("Error in function: <name>") like the reference (model.py:187-198), with the library's
error text appended.
"""
from __future__ import annotations

import ctypes
import enum
import math
from typing import Dict, Iterable, List, NamedTuple, Optional, Tuple, TypeVar, Union

import numpy as np

from .. import _lib
from .dtype import dtype_enum_to_str, dtype_str_to_enum, string_to_torch_dtype, torch_dtype_to_string

AIT_DEFAULT_NUM_RUNTIMES = 1


class AITemplateMemcpyKind(enum.Enum):
    HostToDevice = 0
    DeviceToHost = 1
    DeviceToDevice = 2


class AITemplateAllocatorKind(enum.Enum):
    DEFAULT = 0
    TRACKING = 1


class AITData(NamedTuple):
    """A tensor passed to the runtime: device (or host) pointer, shape, dtype name."""

    data_ptr: int
    shape: List[int]
    dtype: str


class _AITemplateShape(ctypes.Structure):
    _fields_ = [("shape_data", ctypes.POINTER(ctypes.c_longlong)), ("size", ctypes.c_size_t)]


class _CFormatAITData(ctypes.Structure):
    _fields_ = [("pointer", ctypes.c_void_p), ("shape", _AITemplateShape), ("dtype", ctypes.c_int)]


def _check_tensors(tensors, is_error_fn, list_name: str, condition: str) -> None:
    if isinstance(tensors, dict):
        tensors = tensors.values()
    for i, t in enumerate(tensors):
        if is_error_fn(t):
            raise ValueError(f"{list_name}[{i}] failed check: {condition}")


def _check_tensors_contiguous_and_on_gpu(tensors, name: str) -> None:
    _check_tensors(tensors, lambda t: not t.is_contiguous() or not t.is_cuda, name, "contiguous and on GPU")


def _check_tensors_contiguous_and_on_host(tensors, name: str) -> None:
    _check_tensors(tensors, lambda t: not t.is_contiguous() or t.is_cuda, name, "contiguous and on host")


def torch_to_ait_data(tensor) -> AITData:
    return AITData(tensor.data_ptr(), list(tensor.size()), torch_dtype_to_string(tensor.dtype))


def _convert_tensor_args(params):
    if isinstance(params, dict):
        return {name: torch_to_ait_data(x) for name, x in params.items()}
    return [torch_to_ait_data(x) for x in params]


def _reshape_tensor(tensor, shape: List[int]):
    """Reinterprets the (maximum-size) output buffer as the shape the run produced (model.py:159-169)."""
    assert tensor.ndim == len(shape), (
        f"Expected output tensor's ndim to match the length of Run()'s return value: {tensor.ndim=} != {len(shape)=}")
    numel = math.prod(shape)
    return tensor.flatten()[:numel].reshape(shape)


class Model:
    class _DLLWrapper:
        """Calls into libb200ait.so and turns a non-zero status into RuntimeError."""

        def __init__(self, lib_path: str):
            self.lib_path = lib_path
            self.DLL = _lib.load()
            self.is_open = True

        def close(self) -> None:
            self.is_open = False

        def __getattr__(self, name):
            if not self.is_open:
                raise RuntimeError(f"Cannot use closed AIT library: {self.lib_path}")
            method = getattr(self.DLL, name)
            method.restype = ctypes.c_int

            def _wrapped(*args):
                err = method(*args)
                if err:
                    raise RuntimeError(f"Error in function: {name}: {_lib.last_error()}")

            return _wrapped

    def __init__(self, lib_path: str, num_runtimes: int = AIT_DEFAULT_NUM_RUNTIMES,
                 allocator_kind: Optional[AITemplateAllocatorKind] = None):
        self._allocated_ait_data = set()
        self.handle = ctypes.c_void_p()
        self.allocator_handle = ctypes.c_void_p()
        if num_runtimes <= 0:
            raise ValueError(f"num_runtimes must be positive, but got {num_runtimes}")
        self.DLL = self._DLLWrapper(lib_path)
        self.lib_path = lib_path
        if allocator_kind is not None:
            self.DLL.AITemplateAllocatorCreate(ctypes.byref(self.allocator_handle), ctypes.c_int(allocator_kind.value))
        self.DLL.AITemplateModelContainerCreateFromPlan(
            ctypes.pointer(self.handle), ctypes.c_char_p(lib_path.encode("utf-8")), ctypes.c_size_t(num_runtimes),
            self.allocator_handle)
        self.torch_constant_tensors = {}
        self.debug_sorted_graph = None
        self._output_name_to_index = self._construct_output_name_to_index_map()
        self._input_name_to_index = self._construct_input_name_to_index_map()
        self._output_ndims = [len(self.get_output_maximum_shape(i)) for i in range(len(self._output_name_to_index))]

    def __enter__(self):
        return self

    def __exit__(self, *args):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass

    def close(self) -> None:
        for ptr in list(getattr(self, "_allocated_ait_data", ())):
            self.free_gpu_memory(ptr, sync=True)
        if hasattr(self, "DLL") and self.DLL.is_open:
            if self.handle:
                self.DLL.AITemplateModelContainerDelete(self.handle)
                self.handle = ctypes.c_void_p()
            if self.allocator_handle:
                self.DLL.AITemplateAllocatorDelete(self.allocator_handle)
                self.allocator_handle = ctypes.c_void_p()
            self.DLL.close()

    def __getstate__(self):
        return {"lib_path": self.DLL.lib_path}

    def __setstate__(self, d):
        if "lib_path" not in d:
            raise RuntimeError(f"Didn't find 'lib_path' property in {d}")
        self.__init__(d["lib_path"])

    # ------------------------------------------------------------------ argument marshalling
    @staticmethod
    def _convert_single_param_to_c_format(param: AITData) -> _CFormatAITData:
        pointer, shape, dtype = param
        c_shape_data = (ctypes.c_longlong * len(shape))(*[int(d) for d in shape])
        return _CFormatAITData(ctypes.c_void_p(pointer), _AITemplateShape(c_shape_data, ctypes.c_size_t(len(shape))),
                               dtype_str_to_enum(dtype))

    def _convert_params_to_c_format(self, params: List[AITData]):
        c_params = (_CFormatAITData * len(params))()
        for i, p in enumerate(params):
            c_params[i] = self._convert_single_param_to_c_format(p)
        return c_params

    def _prepare_run(self, inputs, outputs, sync: bool, graph_mode: bool, stream_ptr: Optional[int]):
        c_inputs = self._convert_params_to_c_format(inputs)
        c_outputs = self._convert_params_to_c_format(outputs)
        c_stream = ctypes.c_void_p() if stream_ptr is None else ctypes.c_void_p(stream_ptr)
        num_outputs = len(self._output_ndims)
        c_shapes = [(ctypes.c_longlong * n)() for n in self._output_ndims]
        c_shape_ptrs = (ctypes.POINTER(ctypes.c_longlong) * num_outputs)(
            *[ctypes.cast(s, ctypes.POINTER(ctypes.c_longlong)) for s in c_shapes])
        return c_inputs, c_outputs, c_stream, ctypes.c_bool(sync), ctypes.c_bool(graph_mode), c_shapes, c_shape_ptrs

    def _dict_to_ordered_list(self, params, is_inputs: bool):
        if is_inputs:
            index_map, what = self._input_name_to_index, "inputs"
        else:
            index_map, what = self._output_name_to_index, "outputs"
        if len(params) != len(index_map):
            raise ValueError(f"Did not get correct number of {what} expected {len(index_map)}, got {len(params)}")
        result = [None] * len(index_map)
        for name, tensor in params.items():
            if name not in index_map:
                raise ValueError(f"Got unexpected {what[:-1]}: {name}")
            result[index_map[name]] = tensor
        return result

    def _write_tensors_to_c_shapes(self, outputs: List[AITData], c_shapes) -> Dict[str, AITData]:
        out = {}
        for name, idx in self._output_name_to_index.items():
            out[name] = AITData(outputs[idx].data_ptr, list(c_shapes[idx]), outputs[idx].dtype)
        return out

    # --------------------------------------------------------------------------------- run
    def run(self, inputs, outputs, sync: bool = True, stream_ptr: Optional[int] = None,
            graph_mode: bool = False) -> Dict[str, AITData]:
        """Runs the model on AITData (raw pointers). Output buffers must hold the maximum output
        shape; the returned AITData carry the shapes this run produced."""
        if isinstance(inputs, dict):
            inputs = self._dict_to_ordered_list(inputs, True)
        if isinstance(outputs, dict):
            outputs = self._dict_to_ordered_list(outputs, False)
        c_in, c_out, c_stream, c_sync, c_graph, c_shapes, c_shape_ptrs = self._prepare_run(
            inputs, outputs, sync, graph_mode, stream_ptr)
        self.DLL.AITemplateModelContainerRun(self.handle, c_in, ctypes.c_size_t(len(inputs)), c_out,
                                             ctypes.c_size_t(len(outputs)), c_stream, c_sync, c_graph, c_shape_ptrs)
        return self._write_tensors_to_c_shapes(outputs, c_shapes)

    def _interpret_tensors_as_shapes(self, outputs, outputs_ait: Dict[str, AITData]):
        if isinstance(outputs, dict):
            return {name: _reshape_tensor(t, outputs_ait[name].shape) for name, t in outputs.items()}
        return {name: _reshape_tensor(outputs[idx], outputs_ait[name].shape)
                for name, idx in self._output_name_to_index.items()}

    def run_with_tensors(self, inputs, outputs, stream_ptr: Optional[int] = None, sync: bool = True,
                         graph_mode: bool = False):
        """Runs the model with torch tensors (lists ordered by the index maps, or name -> tensor dicts);
        returns name -> output tensor viewed with the shape the run produced."""
        _check_tensors_contiguous_and_on_gpu(inputs, name="inputs")
        _check_tensors_contiguous_and_on_gpu(outputs, name="outputs")
        if stream_ptr is None:
            import torch

            stream_ptr = torch.cuda.current_stream().cuda_stream
        outputs_ait = self.run(_convert_tensor_args(inputs), _convert_tensor_args(outputs), stream_ptr=stream_ptr,
                               sync=sync, graph_mode=graph_mode)
        return self._interpret_tensors_as_shapes(outputs, outputs_ait)

    def _run_with_outputs_on_host(self, inputs, outputs, stream_ptr: Optional[int] = None, graph_mode: bool = False):
        if isinstance(inputs, dict):
            inputs = self._dict_to_ordered_list(inputs, True)
        if isinstance(outputs, dict):
            outputs = self._dict_to_ordered_list(outputs, False)
        c_in, c_out, c_stream, _, c_graph, c_shapes, c_shape_ptrs = self._prepare_run(
            inputs, outputs, True, graph_mode, stream_ptr)
        self.DLL.AITemplateModelContainerRunWithOutputsOnHost(
            self.handle, c_in, ctypes.c_size_t(len(inputs)), c_out, ctypes.c_size_t(len(outputs)), c_stream, c_graph,
            c_shape_ptrs)
        return self._write_tensors_to_c_shapes(outputs, c_shapes)

    def _run_with_tensors_outputs_on_host(self, inputs, outputs, stream_ptr: Optional[int] = None,
                                          graph_mode: bool = False):
        _check_tensors_contiguous_and_on_gpu(inputs, name="inputs")
        _check_tensors_contiguous_and_on_host(outputs, name="outputs")
        out = self._run_with_outputs_on_host(_convert_tensor_args(inputs), _convert_tensor_args(outputs),
                                             stream_ptr=stream_ptr, graph_mode=graph_mode)
        return self._interpret_tensors_as_shapes(outputs, out)

    def benchmark(self, inputs, outputs, stream_ptr: Optional[int] = None, graph_mode: bool = False, count: int = 10,
                  repeat: int = 1, num_threads: int = 1,
                  use_unique_stream_per_thread: bool = False) -> Tuple[float, float, Dict[str, AITData]]:
        """Returns (mean ms per run, std over repeats, outputs). Timed on the device with CUDA events
        around `count` back-to-back runs, `repeat` times (python/aitemplate/compiler/model.py:634-703)."""
        if isinstance(inputs, dict):
            inputs = self._dict_to_ordered_list(inputs, True)
        if isinstance(outputs, dict):
            outputs = self._dict_to_ordered_list(outputs, False)
        assert repeat > 0, f"repeat must be positive, got {repeat}"
        times = []
        c_shapes = None
        for _ in range(repeat):
            c_in, c_out, c_stream, _, c_graph, c_shapes, c_shape_ptrs = self._prepare_run(
                inputs, outputs, True, graph_mode, stream_ptr)
            ms = ctypes.c_float()
            self.DLL.AITemplateModelContainerBenchmark(
                self.handle, c_in, ctypes.c_size_t(len(inputs)), c_out, ctypes.c_size_t(len(outputs)), c_stream,
                c_graph, ctypes.c_size_t(count), ctypes.c_size_t(num_threads),
                ctypes.c_bool(use_unique_stream_per_thread), ctypes.byref(ms), c_shape_ptrs)
            times.append(ms.value)
        mean = float(np.mean(times))
        std = float(np.std(times))
        return mean, std, self._write_tensors_to_c_shapes(outputs, c_shapes)

    def benchmark_with_tensors(self, inputs, outputs, stream_ptr: Optional[int] = None, graph_mode: bool = False,
                               count: int = 10, repeat: int = 1, num_threads: int = 1,
                               use_unique_stream_per_thread: bool = False):
        _check_tensors_contiguous_and_on_gpu(inputs, name="inputs")
        _check_tensors_contiguous_and_on_gpu(outputs, name="outputs")
        if stream_ptr is None:
            import torch

            stream_ptr = torch.cuda.current_stream().cuda_stream
        mean, std, out = self.benchmark(_convert_tensor_args(inputs), _convert_tensor_args(outputs), stream_ptr,
                                        graph_mode, count, repeat, num_threads, use_unique_stream_per_thread)
        return mean, std, self._interpret_tensors_as_shapes(outputs, out)

    def profile(self, inputs, outputs, num_iters: int, filename: str, stream_ptr: Optional[int] = None) -> None:
        if isinstance(inputs, dict):
            inputs = self._dict_to_ordered_list(inputs, True)
        if isinstance(outputs, dict):
            outputs = self._dict_to_ordered_list(outputs, False)
        c_in, c_out, c_stream, _, _, _, _ = self._prepare_run(inputs, outputs, True, False, stream_ptr)
        self.DLL.AITemplateModelContainerProfile(
            self.handle, c_in, ctypes.c_size_t(len(inputs)), c_out, ctypes.c_size_t(len(outputs)), c_stream,
            ctypes.c_size_t(num_iters), ctypes.c_char_p(filename.encode("utf-8")))

    def profile_with_tensors(self, inputs, outputs, num_iters: int, filename: str,
                             stream_ptr: Optional[int] = None) -> None:
        _check_tensors_contiguous_and_on_gpu(inputs, name="inputs")
        _check_tensors_contiguous_and_on_gpu(outputs, name="outputs")
        self.profile(_convert_tensor_args(inputs), _convert_tensor_args(outputs), num_iters, filename, stream_ptr)

    # ----------------------------------------------------------------------- introspection
    def _get_map_helper(self, n: int, get_name_func) -> Dict[str, int]:
        result = {}
        for i in range(n):
            c_name = ctypes.c_char_p()
            get_name_func(self.handle, ctypes.c_size_t(i), ctypes.byref(c_name))
            result[c_name.value.decode("utf-8")] = i
        return result

    def _construct_input_name_to_index_map(self) -> Dict[str, int]:
        n = ctypes.c_size_t()
        self.DLL.AITemplateModelContainerGetNumInputs(self.handle, ctypes.byref(n))
        return self._get_map_helper(n.value, self.DLL.AITemplateModelContainerGetInputName)

    def get_input_name_to_index_map(self) -> Dict[str, int]:
        return dict(self._input_name_to_index)

    def _construct_output_name_to_index_map(self) -> Dict[str, int]:
        n = ctypes.c_size_t()
        self.DLL.AITemplateModelContainerGetNumOutputs(self.handle, ctypes.byref(n))
        return self._get_map_helper(n.value, self.DLL.AITemplateModelContainerGetOutputName)

    def get_output_name_to_index_map(self) -> Dict[str, int]:
        return dict(self._output_name_to_index)

    def _max_shape(self, idx: Union[int, str], index_map: Dict[str, int], fn) -> List[int]:
        if isinstance(idx, str):
            idx = index_map[idx]
        shape = _AITemplateShape()
        fn(self.handle, ctypes.c_size_t(idx), ctypes.byref(shape))
        return [shape.shape_data[i] for i in range(shape.size)]

    def get_input_maximum_shape(self, input_idx_or_name: Union[int, str]) -> List[int]:
        return self._max_shape(input_idx_or_name, self._input_name_to_index,
                               self.DLL.AITemplateModelContainerGetMaximumInputShape)

    def get_output_maximum_shape(self, output_idx_or_name: Union[int, str]) -> List[int]:
        return self._max_shape(output_idx_or_name, self._output_name_to_index,
                               self.DLL.AITemplateModelContainerGetMaximumOutputShape)

    def get_input_dtype(self, index: int) -> int:
        out = ctypes.c_int()
        self.DLL.AITemplateModelContainerGetInputDtype(self.handle, ctypes.c_size_t(index), ctypes.byref(out))
        return out.value

    def get_output_dtype(self, index: int) -> int:
        out = ctypes.c_int()
        self.DLL.AITemplateModelContainerGetOutputDtype(self.handle, ctypes.c_size_t(index), ctypes.byref(out))
        return out.value

    def get_num_runtimes(self) -> int:
        out = ctypes.c_size_t()
        self.DLL.AITemplateModelContainerGetNumRuntimes(self.handle, ctypes.byref(out))
        return out.value

    # ---------------------------------------------------------------------------- constants
    def set_constant(self, name: str, tensor: AITData) -> None:
        c = self._convert_single_param_to_c_format(tensor)
        self.DLL.AITemplateModelContainerSetConstant(self.handle, ctypes.c_char_p(name.encode("utf-8")), ctypes.byref(c))

    def set_many_constants(self, tensors: Dict[str, AITData]) -> None:
        names = (ctypes.c_char_p * len(tensors))(*[n.encode("utf-8") for n in tensors])
        c = self._convert_params_to_c_format(list(tensors.values()))
        self.DLL.AITemplateModelContainerSetManyConstants(self.handle, names, c, ctypes.c_size_t(len(tensors)))

    def set_double_buffer_constant(self, name: str, tensor: AITData, stream_ptr: Optional[int] = None) -> None:
        c = self._convert_single_param_to_c_format(tensor)
        self.DLL.AITemplateModelContainerSetDoubleBufferConstant(
            self.handle, ctypes.c_void_p(stream_ptr), ctypes.c_char_p(name.encode("utf-8")), ctypes.byref(c))

    def set_many_double_buffer_constants(self, tensors: Dict[str, AITData], stream_ptr: Optional[int] = None) -> None:
        names = (ctypes.c_char_p * len(tensors))(*[n.encode("utf-8") for n in tensors])
        c = self._convert_params_to_c_format(list(tensors.values()))
        self.DLL.AITemplateModelContainerSetManyDoubleBufferConstants(
            self.handle, ctypes.c_void_p(stream_ptr), names, c, ctypes.c_size_t(len(tensors)))

    def set_constant_with_tensor(self, name: str, tensor) -> None:
        """Sets a constant from a contiguous CUDA (or host) torch tensor; the Model keeps a reference."""
        if not tensor.is_contiguous():
            raise ValueError(f"constant {name} failed check: contiguous")
        self.torch_constant_tensors[name] = tensor
        self.set_constant(name, torch_to_ait_data(tensor))

    def set_many_constants_with_tensors(self, tensors: Dict[str, object]) -> None:
        ait = {}
        for name, t in tensors.items():
            if not t.is_contiguous():
                raise ValueError(f"constant {name} failed check: contiguous")
            self.torch_constant_tensors[name] = t
            ait[name] = torch_to_ait_data(t)
        self.set_many_constants(ait)

    def set_double_buffer_constant_with_tensor(self, name: str, tensor, stream_ptr: Optional[int] = None) -> None:
        self.torch_constant_tensors[name] = tensor
        self.set_double_buffer_constant(name, torch_to_ait_data(tensor), stream_ptr)

    def set_many_double_buffer_constants_with_tensors(self, tensors: Dict[str, object],
                                                      stream_ptr: Optional[int] = None) -> None:
        ait = {}
        for name, t in tensors.items():
            self.torch_constant_tensors[name] = t
            ait[name] = torch_to_ait_data(t)
        self.set_many_double_buffer_constants(ait, stream_ptr)

    def get_num_constants(self, unbound_constants_only: bool = True, constant_folding_only: bool = False) -> int:
        out = ctypes.c_size_t()
        self.DLL.AITemplateModelContainerGetNumConstants(
            self.handle, ctypes.c_bool(unbound_constants_only), ctypes.c_bool(constant_folding_only), ctypes.byref(out))
        return out.value

    def get_constant_names(self, unbound_constants_only: bool = True, constant_folding_only: bool = False) -> List[str]:
        n = self.get_num_constants(unbound_constants_only, constant_folding_only)
        names = (ctypes.c_char_p * n)()
        self.DLL.AITemplateModelContainerGetConstantNames(
            self.handle, ctypes.c_bool(unbound_constants_only), ctypes.c_bool(constant_folding_only), names)
        return [x.decode("utf-8") for x in names]

    def get_constant_dtype(self, name: str) -> int:
        out = ctypes.c_int()
        self.DLL.AITemplateModelContainerGetConstantDtype(self.handle, ctypes.c_char_p(name.encode("utf-8")), ctypes.byref(out))
        return out.value

    def get_constant_original_name(self, name: str) -> str:
        out = ctypes.c_char_p()
        self.DLL.AITemplateModelContainerGetConstantOriginalName(
            self.handle, ctypes.c_char_p(name.encode("utf-8")), ctypes.byref(out))
        return out.value.decode("utf-8")

    def fold_constants(self, stream_ptr: Optional[int] = None, sync: bool = True, double_buffer: bool = False) -> None:
        fn = (self.DLL.AITemplateModelContainerFoldConstantsInDoubleBuffer if double_buffer
              else self.DLL.AITemplateModelContainerFoldConstants)
        fn(self.handle, ctypes.c_void_p(stream_ptr), ctypes.c_bool(sync))

    def swap_constants(self) -> None:
        self.DLL.AITemplateModelContainerSwapConstants(self.handle)

    # ------------------------------------------------------------------------ memory helpers
    def allocate_gpu_memory(self, nbytes: int, stream_ptr: Optional[int] = None, sync: bool = True) -> int:
        ptr = ctypes.c_void_p()
        self.DLL.AITemplateDeviceMalloc(ctypes.byref(ptr), ctypes.c_size_t(nbytes), ctypes.c_void_p(stream_ptr),
                                        ctypes.c_bool(sync))
        return ptr.value

    def free_gpu_memory(self, ptr: int, stream_ptr: Optional[int] = None, sync: bool = True) -> None:
        self._allocated_ait_data.discard(ptr)
        self.DLL.AITemplateDeviceFree(ctypes.c_void_p(ptr), ctypes.c_void_p(stream_ptr), ctypes.c_bool(sync))

    def memcpy(self, dst: int, src: int, count: int, kind: AITemplateMemcpyKind, stream_ptr: Optional[int] = None,
               sync: bool = True) -> None:
        self.DLL.AITemplateMemcpy(ctypes.c_void_p(dst), ctypes.c_void_p(src), ctypes.c_size_t(count),
                                  ctypes.c_int(kind.value), ctypes.c_void_p(stream_ptr), ctypes.c_bool(sync))

    def numpy_to_ait_data(self, arr: np.ndarray, stream_ptr: Optional[int] = None, sync: bool = True) -> AITData:
        """Copies a numpy array to the GPU; the memory is freed when the Model is closed."""
        arr = np.ascontiguousarray(arr)
        ptr = self.allocate_gpu_memory(arr.nbytes, stream_ptr=stream_ptr, sync=sync)
        self._allocated_ait_data.add(ptr)
        self.memcpy(ptr, arr.ctypes.data, arr.nbytes, AITemplateMemcpyKind.HostToDevice, stream_ptr, sync)
        return AITData(ptr, list(arr.shape), str(arr.dtype))

    def ait_data_to_numpy(self, ait_data: AITData, stream_ptr: Optional[int] = None, sync: bool = True) -> np.ndarray:
        arr = np.empty(ait_data.shape, dtype=ait_data.dtype)
        self.memcpy(arr.ctypes.data, ait_data.data_ptr, arr.nbytes, AITemplateMemcpyKind.DeviceToHost, stream_ptr, sync)
        return arr
