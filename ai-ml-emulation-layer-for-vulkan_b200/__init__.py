"""Python binding of ``libmlel_b200.so`` (C ABI in ``include/mlel_b200.h``).

The directory name of this package is not a Python identifier; import it through
``__graft_entry__.load_package()`` (registered as module ``mlel_b200``).

The binding is thin on purpose: ``Pipeline`` mirrors the reference's ``GraphPipeline``
(graph/compute_graph_op.hpp:1204-1549) call for call, ``Session`` mirrors the data-graph
pipeline session (graph/graph_layer.cpp:215-298).  All computation happens in the CUDA library;
there is no CPU fallback, and loading fails loudly when the library has not been built.
"""
from __future__ import annotations

import ctypes
import os
from typing import Iterable, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmlel_b200.so")

BOOL, I8, I16, I32, I64, U8, U16, U32, F16, BF16, F32 = range(11)
MAX_RANK = 6
PIPELINE_NO_FUSION = 1
INCOMPLETE = 5
PROPERTY_CREATION_LOG = 0
PROPERTY_PROFILING = 0x7FFFFFFE

NP_TO_DTYPE = {
    np.dtype(np.bool_): BOOL,
    np.dtype(np.int8): I8,
    np.dtype(np.int16): I16,
    np.dtype(np.int32): I32,
    np.dtype(np.int64): I64,
    np.dtype(np.uint8): U8,
    np.dtype(np.uint16): U16,
    np.dtype(np.uint32): U32,
    np.dtype(np.float16): F16,
    np.dtype(np.float32): F32,
}
DTYPE_TO_NP = {v: k for k, v in NP_TO_DTYPE.items()}


class MlelError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"mlel status {status}: {message}")
        self.status = status


class TensorDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("dims", ctypes.c_int64 * MAX_RANK),
        ("strides", ctypes.c_int64 * MAX_RANK),
    ]


class Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("desc", TensorDesc)]


class HostIO(ctypes.Structure):
    _fields_ = [
        ("set", ctypes.c_uint32),
        ("binding", ctypes.c_uint32),
        ("array_index", ctypes.c_uint32),
        ("host_ptr", ctypes.c_void_p),
        ("bytes", ctypes.c_uint64),
    ]


class LiveInterval(ctypes.Structure):
    _fields_ = [("id", ctypes.c_uint64), ("first", ctypes.c_uint32), ("last", ctypes.c_uint32),
                ("size", ctypes.c_uint64), ("order", ctypes.c_uint64)]


class UnseenAllocation(ctypes.Structure):
    _fields_ = [("id", ctypes.c_uint64), ("size", ctypes.c_uint64)]


class PlannedTensor(ctypes.Structure):
    _fields_ = [("tensor", ctypes.c_int32), ("seen", ctypes.c_uint32), ("offset", ctypes.c_uint64),
                ("size", ctypes.c_uint64), ("first", ctypes.c_uint32), ("last", ctypes.c_uint32)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
                "(nvcc, sm_100a). There is no CPU implementation to fall back to.")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.mlel_last_error.restype = ctypes.c_char_p
        _lib.mlel_tosa_op_name.restype = ctypes.c_char_p
        _lib.mlel_pipeline_op_name.restype = ctypes.c_char_p
        _lib.mlel_pipeline_exec_name.restype = ctypes.c_char_p
        _lib.mlel_session_planner_name.restype = ctypes.c_char_p
        _lib.mlel_pipeline_destroy.restype = None
        _lib.mlel_session_destroy.restype = None
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise MlelError(status, (lib().mlel_last_error() or b"").decode())


def make_desc(dtype: int, dims: Sequence[int], strides: Sequence[int] | None = None) -> TensorDesc:
    d = TensorDesc()
    d.dtype = int(dtype)
    d.rank = len(dims)
    for i, v in enumerate(dims[:MAX_RANK]):  # a rank above MAX_RANK is rejected by the library
        d.dims[i] = int(v)
    if strides is not None:
        for i, v in enumerate(strides):
            d.strides[i] = int(v)
    return d


def device_tensor(ptr: int, dtype: int, dims: Sequence[int], strides: Sequence[int] | None = None) -> Tensor:
    t = Tensor()
    t.data = ptr
    t.desc = make_desc(dtype, dims, strides)
    return t


def _i32(values: Iterable[int]):
    values = [int(v) for v in values]
    return (ctypes.c_int32 * len(values))(*values)


def _u32(values: Iterable[int]):
    values = [int(v) for v in values]
    return (ctypes.c_uint32 * len(values))(*values)


def _name(name: str | None):
    return name.encode() if name else None


def tosa_op_names() -> list[str]:
    l = lib()
    return [l.mlel_tosa_op_name(i).decode() for i in range(l.mlel_tosa_op_count())]


def tosa_op_supported(name: str) -> bool:
    return bool(lib().mlel_tosa_op_supported(name.encode()))


def ext_inst_set_registered(name: str) -> bool:
    return bool(lib().mlel_ext_inst_set_registered(name.encode()))


def measure_int8_mma_peak(batches: int, stream: int = 0) -> float:
    """What the int8 tensor pipe sustains, in TOP/s: ``batches`` batches of 64 back-to-back ``tcgen05.mma
    kind::i8`` instructions on every SM (about 5 microseconds per batch)."""
    ms, ops = ctypes.c_float(), ctypes.c_double()
    check(lib().mlel_measure_int8_mma_peak(int(batches), ctypes.c_void_p(stream), ctypes.byref(ms), ctypes.byref(ops)))
    return ops.value / (ms.value * 1e-3) / 1e12


def allocate_intervals(intervals, unseen, alignment):
    """details::allocateIntervals of the reference (graph/interval_memory_planner.cpp:170-216).

    ``intervals``: list of (id, first, last, size, order); ``unseen``: list of (id, size).
    Returns (offsets_by_id, memory_size)."""
    iv = (LiveInterval * max(1, len(intervals)))()
    for k, (i, first, last, size, order) in enumerate(intervals):
        iv[k] = LiveInterval(i, first, last, size, order)
    us = (UnseenAllocation * max(1, len(unseen)))()
    for k, (i, size) in enumerate(unseen):
        us[k] = UnseenAllocation(i, size)
    off = (ctypes.c_uint64 * max(1, len(intervals)))()
    uoff = (ctypes.c_uint64 * max(1, len(unseen)))()
    total = ctypes.c_uint64()
    check(lib().mlel_allocate_intervals(iv, ctypes.c_size_t(len(intervals)), us, ctypes.c_size_t(len(unseen)),
                                        ctypes.c_uint64(alignment), off, uoff, ctypes.byref(total)))
    offsets = {intervals[k][0]: off[k] for k in range(len(intervals))}
    offsets.update({unseen[k][0]: uoff[k] for k in range(len(unseen))})
    return offsets, total.value


class Pipeline:
    """Counterpart of the reference's GraphPipeline; one method per ``make<Op>``."""

    def __init__(self, flags: int = 0):
        self._h = ctypes.c_void_p()
        check(lib().mlel_pipeline_create(ctypes.c_uint32(flags), ctypes.byref(self._h)))

    def __del__(self):
        # at interpreter shutdown the module globals may already be gone; the process is ending anyway
        if getattr(self, "_h", None) and lib is not None:
            lib().mlel_pipeline_destroy(self._h)
            self._h = None

    # ---- properties (vkGetDataGraphPipelineAvailablePropertiesARM / vkGetDataGraphPipelinePropertiesARM) ----
    def available_properties(self) -> list[int]:
        n = ctypes.c_uint32()
        check(lib().mlel_pipeline_available_properties(self._h, ctypes.byref(n), None))
        ids = (ctypes.c_uint32 * max(1, n.value))()
        check(lib().mlel_pipeline_available_properties(self._h, ctypes.byref(n), ids))
        return [ids[i] for i in range(n.value)]

    def text_property(self, prop: int) -> str:
        """Two-call query of a text property; the profiling property waits for the recorded dispatches."""
        size, is_text = ctypes.c_size_t(), ctypes.c_int()
        check(lib().mlel_pipeline_get_property(self._h, ctypes.c_uint32(prop), None, ctypes.byref(size),
                                               ctypes.byref(is_text)))
        buf = ctypes.create_string_buffer(size.value)
        check(lib().mlel_pipeline_get_property(self._h, ctypes.c_uint32(prop), buf, ctypes.byref(size),
                                               ctypes.byref(is_text)))
        assert is_text.value == 1
        return buf.raw[:size.value - 1].decode()

    def profile(self) -> dict:
        """The profiling document (graph/graph_profiler.cpp:563-620) as a dictionary."""
        import json
        return json.loads(self.text_property(PROPERTY_PROFILING))

    def clear_profile(self) -> None:
        check(lib().mlel_pipeline_clear_profile(self._h))

    # ---- tensors ----
    def bind_external(self, set_: int, binding: int, dtype: int, dims, array_index: int = 0, strides=None) -> int:
        out = ctypes.c_int32()
        desc = make_desc(dtype, dims, strides)
        check(lib().mlel_pipeline_bind_external(self._h, set_, binding, array_index, ctypes.byref(desc),
                                                ctypes.byref(out)))
        return out.value

    def get_external(self, set_: int, binding: int, array_index: int = 0) -> int:
        out = ctypes.c_int32()
        check(lib().mlel_pipeline_get_external(self._h, set_, binding, array_index, ctypes.byref(out)))
        return out.value

    def add_constant(self, const_id: int, array: np.ndarray) -> int:
        array = np.ascontiguousarray(array)
        out = ctypes.c_int32()
        desc = make_desc(NP_TO_DTYPE[array.dtype], array.shape)
        check(lib().mlel_pipeline_add_constant(self._h, const_id, ctypes.byref(desc),
                                               ctypes.c_void_p(array.ctypes.data), ctypes.byref(out)))
        return out.value

    def composite_constant(self, array: np.ndarray) -> int:
        array = np.ascontiguousarray(array)
        out = ctypes.c_int32()
        desc = make_desc(NP_TO_DTYPE[array.dtype], array.shape)
        check(lib().mlel_pipeline_make_composite_constant(self._h, ctypes.byref(desc),
                                                          ctypes.c_void_p(array.ctypes.data), ctypes.byref(out)))
        return out.value

    def make_tensor(self, dtype: int, dims, strides=None) -> int:
        out = ctypes.c_int32()
        desc = make_desc(dtype, dims, strides)
        check(lib().mlel_pipeline_make_tensor(self._h, ctypes.byref(desc), ctypes.byref(out)))
        return out.value

    def mark_input(self, t: int) -> None:
        check(lib().mlel_pipeline_mark_input(self._h, t))

    def mark_output(self, t: int) -> None:
        check(lib().mlel_pipeline_mark_output(self._h, t))

    def lower_spvasm(self, text: str) -> None:
        check(lib().mlel_pipeline_lower_spvasm(self._h, text.encode()))

    def tensor_desc(self, t: int):
        d = TensorDesc()
        check(lib().mlel_pipeline_tensor_desc(self._h, t, ctypes.byref(d)))
        return d.dtype, [d.dims[i] for i in range(d.rank)], [d.strides[i] for i in range(d.rank)]

    def op_names(self) -> list[str]:
        l = lib()
        return [l.mlel_pipeline_op_name(self._h, i).decode() for i in range(l.mlel_pipeline_op_count(self._h))]

    def exec_names(self) -> list[str]:
        l = lib()
        n = l.mlel_pipeline_exec_count(self._h)
        if n < 0:
            check(-13)
        return [l.mlel_pipeline_exec_name(self._h, i).decode() for i in range(n)]

    # ---- operators (argument order of graph/compute_graph_op.hpp:1249-1483) ----
    def conv2d(self, input, output, weights, biases, pad, stride, dilation, input_zp, weight_zp, acc_type=1,
               name=None):
        check(lib().mlel_make_conv2d(self._h, input, output, weights, biases, _i32(pad), _i32(stride), _i32(dilation),
                                     ctypes.c_int8(input_zp), ctypes.c_int8(weight_zp), ctypes.c_uint32(acc_type),
                                     _name(name)))

    def depthwise_conv2d(self, input, output, weights, biases, pad, stride, dilation, input_zp, weight_zp,
                         acc_type=1, name=None):
        check(lib().mlel_make_depthwise_conv2d(self._h, input, output, weights, biases, _i32(pad), _i32(stride),
                                               _i32(dilation), ctypes.c_int8(input_zp), ctypes.c_int8(weight_zp),
                                               ctypes.c_uint32(acc_type), _name(name)))

    def matmul(self, input1, input2, output, zp1, zp2, name=None):
        check(lib().mlel_make_matmul(self._h, input1, input2, output, ctypes.c_int32(zp1), ctypes.c_int32(zp2),
                                     _name(name)))

    def rescale(self, input, output, input_zp, output_zp, multiplier, shift, scale32=True, double_round=False,
                per_channel=False, input_unsigned=False, output_unsigned=False, name=None):
        check(lib().mlel_make_rescale(self._h, input, output, ctypes.c_int32(input_zp), ctypes.c_int32(output_zp),
                                      multiplier, shift, int(scale32), int(double_round), int(per_channel),
                                      int(input_unsigned), int(output_unsigned), _name(name)))

    def avg_pool2d(self, input, output, kernel, stride, pad, acc_type, input_zp, output_zp, name=None):
        check(lib().mlel_make_avg_pool2d(self._h, input, output, _i32(kernel), _i32(stride), _i32(pad),
                                         ctypes.c_uint32(acc_type), ctypes.c_int8(input_zp), ctypes.c_int8(output_zp),
                                         _name(name)))

    def max_pool2d(self, input, output, kernel, stride, pad, nan_mode=1, name=None):
        check(lib().mlel_make_max_pool2d(self._h, input, output, _i32(kernel), _i32(stride), _i32(pad),
                                         ctypes.c_uint32(nan_mode), _name(name)))

    def table(self, input, output, table, name=None):
        check(lib().mlel_make_table(self._h, input, output, table, _name(name)))

    def transpose(self, input, output, perms, name=None):
        check(lib().mlel_make_transpose(self._h, input, output, _u32(perms), len(perms), _name(name)))

    def concat(self, inputs, output, axis, name=None):
        arr = (ctypes.c_int32 * len(inputs))(*inputs)
        check(lib().mlel_make_concat(self._h, arr, len(inputs), output, ctypes.c_uint32(axis), _name(name)))

    def clamp(self, input, output, min_value, max_value, nan_mode=1, name=None):
        check(lib().mlel_make_clamp(self._h, input, output, ctypes.c_double(min_value), ctypes.c_double(max_value),
                                    ctypes.c_uint32(nan_mode), _name(name)))

    def binary(self, op_name, input1, input2, output, nan_mode=1, name=None):
        check(lib().mlel_make_binary(self._h, op_name.encode(), input1, input2, output, ctypes.c_uint32(nan_mode),
                                     _name(name)))

    def unary(self, op_name, input, output, name=None):
        check(lib().mlel_make_unary(self._h, op_name.encode(), input, output, _name(name)))

    def mul(self, input1, input2, output, shift, name=None):
        check(lib().mlel_make_mul(self._h, input1, input2, output, ctypes.c_uint32(shift), _name(name)))

    def reduce(self, op_name, input, output, axis, nan_mode=1, name=None):
        check(lib().mlel_make_reduce(self._h, op_name.encode(), input, output, ctypes.c_uint32(axis),
                                     ctypes.c_uint32(nan_mode), _name(name)))

    def cast(self, input, output, name=None):
        check(lib().mlel_make_cast(self._h, input, output, _name(name)))

    def reshape(self, input, output, name=None):
        check(lib().mlel_make_reshape(self._h, input, output, _name(name)))

    def slice(self, input, output, start, name=None):
        check(lib().mlel_make_slice(self._h, input, output, _u32(start), len(start), _name(name)))

    def pad(self, input, output, padding, pad_const, pad_const_int, name=None):
        check(lib().mlel_make_pad(self._h, input, output, padding, ctypes.c_double(pad_const),
                                  ctypes.c_int32(pad_const_int), _name(name)))

    def arithmetic_right_shift(self, input1, input2, output, round_, name=None):
        check(lib().mlel_make_arithmetic_right_shift(self._h, input1, input2, output, int(round_), _name(name)))

    def negate(self, input, output, input_zp, output_zp, name=None):
        check(lib().mlel_make_negate(self._h, input, output, ctypes.c_int32(input_zp), ctypes.c_int32(output_zp),
                                     _name(name)))

    def select(self, input1, input2, input3, output, name=None):
        check(lib().mlel_make_select(self._h, input1, input2, input3, output, _name(name)))


class Session:
    """Counterpart of VkDataGraphPipelineSessionARM: memory requirements, bind, dispatch."""

    def __init__(self, pipeline: Pipeline):
        self._pipeline = pipeline
        self._h = ctypes.c_void_p()
        check(lib().mlel_session_create(pipeline._h, ctypes.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib().mlel_session_destroy(self._h)
            self._h = None

    def memory_requirements(self) -> tuple[int, int]:
        size, align = ctypes.c_uint64(), ctypes.c_uint64()
        check(lib().mlel_session_memory_requirements(self._h, ctypes.byref(size), ctypes.byref(align)))
        return size.value, align.value

    def planner_name(self) -> str:
        return lib().mlel_session_planner_name(self._h).decode()

    def plan(self) -> list[PlannedTensor]:
        """Placement and live range of every session tensor, in session-tensor order."""
        n = ctypes.c_uint32()
        check(lib().mlel_session_plan(self._h, ctypes.byref(n), None))
        out = (PlannedTensor * max(1, n.value))()
        check(lib().mlel_session_plan(self._h, ctypes.byref(n), out))
        return [out[i] for i in range(n.value)]

    def tensor_offset(self, tensor: int) -> int:
        off = ctypes.c_uint64()
        check(lib().mlel_session_tensor_offset(self._h, tensor, ctypes.byref(off)))
        return off.value

    def bind_memory(self, device_ptr: int, offset: int = 0) -> None:
        check(lib().mlel_session_bind_memory(self._h, ctypes.c_void_p(device_ptr), ctypes.c_uint64(offset)))

    def set_external(self, set_: int, binding: int, device_ptr: int, array_index: int = 0) -> None:
        check(lib().mlel_session_set_external(self._h, set_, binding, array_index, ctypes.c_void_p(device_ptr)))

    def dispatch(self, stream: int = 0) -> None:
        check(lib().mlel_session_dispatch(self._h, ctypes.c_void_p(stream)))

    def dispatch_graph(self, stream: int = 0) -> None:
        check(lib().mlel_session_dispatch_graph(self._h, ctypes.c_void_p(stream)))

    def dispatch_profiled(self, stream: int = 0) -> list[float]:
        """Per-kernel device milliseconds of one dispatch (synchronises the stream)."""
        n = self.launch_count()
        ms = (ctypes.c_float * max(1, n))()
        check(lib().mlel_session_dispatch_profiled(self._h, ctypes.c_void_p(stream), ms, n))
        return [ms[i] for i in range(n)]

    def launch_count(self) -> int:
        return lib().mlel_session_launch_count(self._h)

    def run_host(self, inputs, outputs, stream: int = 0) -> None:
        """``inputs`` / ``outputs``: lists of (set, binding, array_index, host_ptr, nbytes)."""
        ins = (HostIO * max(1, len(inputs)))(*[HostIO(*x) for x in inputs])
        outs = (HostIO * max(1, len(outputs)))(*[HostIO(*x) for x in outputs])
        check(lib().mlel_session_run_host(self._h, ins, len(inputs), outs, len(outputs), ctypes.c_void_p(stream)))
