"""ctypes front end of the CPU oracle (``mlel_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and the CPU
baseline legs of ``bench.py``.  The shipped library never loads it.

Each function takes numpy arrays (any strides), runs the C++ restatement of the matching
reference shader (``graph/shaders/graph_op/tosa/<op>.comp``) and returns a new numpy array.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmlel_oracle.so")

BOOL, I8, I16, I32, I64, U8, U16, U32, F16, BF16, F32 = range(11)

_NP2DT = {
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

BINARY_OPS = {
    "ADD": 0, "SUB": 1, "BITWISE_AND": 2, "BITWISE_OR": 3, "BITWISE_XOR": 4, "LOGICAL_AND": 5,
    "LOGICAL_OR": 6, "LOGICAL_XOR": 7, "LOGICAL_LEFT_SHIFT": 8, "LOGICAL_RIGHT_SHIFT": 9,
    "INTDIV": 10, "MAXIMUM": 11, "MINIMUM": 12, "EQUAL": 13, "GREATER": 14, "GREATER_EQUAL": 15, "POW": 16,
}
REDUCE_OPS = {"REDUCE_SUM": 0, "REDUCE_MAX": 1, "REDUCE_MIN": 2, "REDUCE_PRODUCT": 3, "REDUCE_ALL": 4,
              "REDUCE_ANY": 5}
UNARY_OPS = {"ABS": 0, "BITWISE_NOT": 1, "CLZ": 2, "LOGICAL_NOT": 3, "CEIL": 4, "COS": 5, "ERF": 6, "EXP": 7,
             "FLOOR": 8, "LOG": 9, "RECIPROCAL": 10, "RSQRT": 11, "SIGMOID": 12, "SIN": 13, "TANH": 14}
FLOAT_UNARY_OPS = frozenset(UNARY_OPS) - {"BITWISE_NOT", "CLZ", "LOGICAL_NOT"}


class _Tensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("dims", ctypes.c_int64 * 6),
        ("strides", ctypes.c_int64 * 6),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in ``oracle/Makefile`` if it is missing or stale."""
    src = os.path.join(_HERE, "mlel_oracle.cpp")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libmlel_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _t(a: np.ndarray) -> _Tensor:
    t = _Tensor()
    t.data = a.ctypes.data
    t.dtype = _NP2DT[a.dtype]
    t.rank = a.ndim
    for i in range(a.ndim):
        t.dims[i] = a.shape[i]
        t.strides[i] = a.strides[i]
    return t


def _i32(v):
    arr = (ctypes.c_int32 * len(v))(*[int(x) for x in v])
    return arr


def _u32(v):
    arr = (ctypes.c_uint32 * len(v))(*[int(x) for x in v])
    return arr


def _check(rc):
    if rc != 0:
        raise RuntimeError(f"oracle call failed with {rc}")


def conv_out_shape(in_shape, w_shape, pad, stride, dil):
    n, h, w, _ = in_shape
    oc, kh, kw, _ = w_shape
    oh = (h + pad[0] + pad[1] - (kh - 1) * dil[0] - 1) // stride[0] + 1
    ow = (w + pad[2] + pad[3] - (kw - 1) * dil[1] - 1) // stride[1] + 1
    return (n, oh, ow, oc)


def conv2d(x, w, bias, pad, stride, dil, in_zp, w_zp, out_shape=None, generic=False):
    out_dtype = np.int64 if x.dtype == np.int16 else np.int32
    shape = out_shape or conv_out_shape(x.shape, w.shape, pad, stride, dil)
    out = np.zeros(shape, out_dtype)
    fn = lib().orc_conv2d_generic if generic else lib().orc_conv2d
    _check(fn(ctypes.byref(_t(x)), ctypes.byref(_t(w)), ctypes.byref(_t(bias)), ctypes.byref(_t(out)),
              _i32(pad), _i32(stride), _i32(dil), ctypes.c_int32(in_zp), ctypes.c_int32(w_zp)))
    return out


def depthwise_conv2d(x, w, bias, pad, stride, dil, in_zp, w_zp, out_shape=None):
    out_dtype = np.int64 if x.dtype == np.int16 else np.int32
    kh, kw, c, m = w.shape
    n, h, wd, _ = x.shape
    oh = (h + pad[0] + pad[1] - (kh - 1) * dil[0] - 1) // stride[0] + 1
    ow = (wd + pad[2] + pad[3] - (kw - 1) * dil[1] - 1) // stride[1] + 1
    out = np.zeros(out_shape or (n, oh, ow, c * m), out_dtype)
    _check(lib().orc_depthwise_conv2d(ctypes.byref(_t(x)), ctypes.byref(_t(w)), ctypes.byref(_t(bias)),
                                      ctypes.byref(_t(out)), _i32(pad), _i32(stride), _i32(dil),
                                      ctypes.c_int32(in_zp), ctypes.c_int32(w_zp)))
    return out


def matmul(a, b, zp_a, zp_b):
    out_dtype = np.int64 if a.dtype == np.int16 else np.int32
    out = np.zeros((a.shape[0], a.shape[1], b.shape[2]), out_dtype)
    _check(lib().orc_matmul(ctypes.byref(_t(a)), ctypes.byref(_t(b)), ctypes.byref(_t(out)),
                            ctypes.c_int32(zp_a), ctypes.c_int32(zp_b)))
    return out


def rescale(x, mult, shift, in_zp, out_zp, out_dtype, scale32=True, double_round=False, per_channel=False):
    out = np.zeros(x.shape, out_dtype)
    mult = np.ascontiguousarray(mult)
    shift = np.ascontiguousarray(shift, dtype=np.int8)
    _check(lib().orc_rescale(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.byref(_t(mult)),
                             ctypes.byref(_t(shift)), ctypes.c_int32(in_zp), ctypes.c_int32(out_zp),
                             int(scale32), int(double_round), int(per_channel)))
    return out


def _pool_shape(x, kernel, stride, pad):
    n, h, w, c = x.shape
    oh = (h + pad[0] + pad[1] - kernel[0]) // stride[0] + 1
    ow = (w + pad[2] + pad[3] - kernel[1]) // stride[1] + 1
    return (n, oh, ow, c)


def avg_pool2d(x, kernel, stride, pad, in_zp, out_zp, out_shape=None):
    out = np.zeros(out_shape or _pool_shape(x, kernel, stride, pad), x.dtype)
    _check(lib().orc_avg_pool2d(ctypes.byref(_t(x)), ctypes.byref(_t(out)), _i32(kernel), _i32(stride), _i32(pad),
                                ctypes.c_int32(in_zp), ctypes.c_int32(out_zp)))
    return out


def max_pool2d(x, kernel, stride, pad, out_shape=None):
    out = np.zeros(out_shape or _pool_shape(x, kernel, stride, pad), x.dtype)
    _check(lib().orc_max_pool2d(ctypes.byref(_t(x)), ctypes.byref(_t(out)), _i32(kernel), _i32(stride), _i32(pad)))
    return out


def table(x, tbl):
    out = np.zeros(x.shape, np.int8 if x.dtype == np.int8 else np.int32)
    tbl = np.ascontiguousarray(tbl)
    _check(lib().orc_table(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.byref(_t(tbl))))
    return out


def transpose(x, perms):
    out = np.zeros([x.shape[p] for p in perms], x.dtype)
    _check(lib().orc_transpose(ctypes.byref(_t(x)), ctypes.byref(_t(out)), _u32(perms)))
    return out


def concat(inputs, axis):
    shape = list(inputs[0].shape)
    shape[axis] = sum(a.shape[axis] for a in inputs)
    out = np.zeros(shape, inputs[0].dtype)
    offset = 0
    for a in inputs:
        _check(lib().orc_concat(ctypes.byref(_t(a)), ctypes.byref(_t(out)), ctypes.c_uint32(axis),
                                ctypes.c_uint32(offset)))
        offset += a.shape[axis]
    return out


def reshape(x, shape):
    out = np.zeros(shape, x.dtype)
    _check(lib().orc_reshape(ctypes.byref(_t(x)), ctypes.byref(_t(out))))
    return out


def slice_(x, start, size):
    out = np.zeros(size, x.dtype)
    _check(lib().orc_slice(ctypes.byref(_t(x)), ctypes.byref(_t(out)), _u32(start)))
    return out


def pad(x, padding, pad_const):
    """``padding`` is the flat [2*rank] int32 list (before0, after0, before1, ...)."""
    padding = np.ascontiguousarray(padding, dtype=np.int32)
    shape = [x.shape[i] + int(padding[2 * i]) + int(padding[2 * i + 1]) for i in range(x.ndim)]
    out = np.zeros(shape, x.dtype)
    bits = np.zeros(1, np.int64)
    bits.view(x.dtype)[0] = np.array(pad_const).astype(x.dtype)
    _check(lib().orc_pad(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.byref(_t(padding)),
                         ctypes.c_int64(int(bits[0]))))
    return out


def clamp(x, min_v, max_v):
    out = np.zeros(x.shape, x.dtype)
    _check(lib().orc_clamp(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.c_double(min_v), ctypes.c_double(max_v)))
    return out


def _bshape(a, b):
    return tuple(max(x, y) for x, y in zip(a.shape, b.shape))


def binary(op, a, b, out_dtype=None):
    if out_dtype is None:
        out_dtype = np.bool_ if op in ("EQUAL", "GREATER", "GREATER_EQUAL") else a.dtype
    out = np.zeros(_bshape(a, b), out_dtype)
    _check(lib().orc_binary(ctypes.byref(_t(a)), ctypes.byref(_t(b)), ctypes.byref(_t(out)), BINARY_OPS[op]))
    return out


def mul(a, b, shift, out_dtype=None):
    out = np.zeros(_bshape(a, b), out_dtype or (np.float32 if a.dtype == np.float32 else np.int32))
    _check(lib().orc_mul(ctypes.byref(_t(a)), ctypes.byref(_t(b)), ctypes.byref(_t(out)), ctypes.c_uint32(shift)))
    return out


def reduce(op, x, axis):
    shape = list(x.shape)
    shape[axis] = 1
    out = np.zeros(shape, x.dtype)
    _check(lib().orc_reduce(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.c_uint32(axis), REDUCE_OPS[op]))
    return out


def cast(x, out_dtype):
    out = np.zeros(x.shape, out_dtype)
    _check(lib().orc_cast(ctypes.byref(_t(x)), ctypes.byref(_t(out))))
    return out


def arithmetic_right_shift(a, b, round_):
    out = np.zeros(_bshape(a, b), a.dtype)
    _check(lib().orc_arithmetic_right_shift(ctypes.byref(_t(a)), ctypes.byref(_t(b)), ctypes.byref(_t(out)),
                                            int(round_)))
    return out


def negate(x, in_zp, out_zp):
    out = np.zeros(x.shape, x.dtype)
    _check(lib().orc_negate(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.c_int32(in_zp),
                            ctypes.c_int32(out_zp)))
    return out


def select(cond, a, b):
    shape = tuple(max(x, y, z) for x, y, z in zip(cond.shape, a.shape, b.shape))
    out = np.zeros(shape, a.dtype)
    c8 = cond.view(np.uint8) if cond.dtype == np.bool_ else cond
    _check(lib().orc_select(ctypes.byref(_t(c8)), ctypes.byref(_t(a)), ctypes.byref(_t(b)), ctypes.byref(_t(out))))
    return out


def unary(op, x):
    out = np.zeros(x.shape, x.dtype)
    if x.dtype == np.float32:
        assert op in FLOAT_UNARY_OPS
        _check(lib().orc_unary_f32(ctypes.byref(_t(x)), ctypes.byref(_t(out)), UNARY_OPS[op]))
        return out
    _check(lib().orc_unary(ctypes.byref(_t(x)), ctypes.byref(_t(out)), UNARY_OPS[op]))
    return out


def argmax(x, axis):
    out = np.zeros(x.shape[:axis] + x.shape[axis + 1:], np.int32)
    _check(lib().orc_argmax(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.c_uint32(axis)))
    return out


def gather(values, indices):
    out = np.zeros((values.shape[0], indices.shape[1], values.shape[2]), values.dtype)
    _check(lib().orc_gather(ctypes.byref(_t(values)), ctypes.byref(_t(indices)), ctypes.byref(_t(out))))
    return out


def scatter(values_in, indices, input_):
    out = np.zeros(values_in.shape, values_in.dtype)
    _check(lib().orc_scatter(ctypes.byref(_t(values_in)), ctypes.byref(_t(indices)), ctypes.byref(_t(input_)),
                             ctypes.byref(_t(out))))
    return out


def reverse(x, axis):
    out = np.zeros(x.shape, x.dtype)
    _check(lib().orc_reverse(ctypes.byref(_t(x)), ctypes.byref(_t(out)), ctypes.c_uint32(axis)))
    return out


def tile(x, multiples):
    out = np.zeros(tuple(d * m for d, m in zip(x.shape, multiples)), x.dtype)
    _check(lib().orc_tile(ctypes.byref(_t(x)), ctypes.byref(_t(out))))
    return out


def resize(x, out_shape, out_dtype, scale, offset, border, mode):
    """``scale`` = (y_n, y_d, x_n, x_d); ``mode`` 1 = NEAREST, 2 = BILINEAR.  ``border`` only enters the output
    shape, which the caller supplies."""
    out = np.zeros(out_shape, out_dtype)
    _check(lib().orc_resize(ctypes.byref(_t(x)), ctypes.byref(_t(out)), _i32(scale), _i32(offset),
                            ctypes.c_int32(mode)))
    return out


def transpose_conv2d(x, w, bias, out_shape, out_pad, stride, in_zp, w_zp):
    out = np.zeros(out_shape, np.int64 if x.dtype == np.int16 else np.int32)
    _check(lib().orc_transpose_conv2d(ctypes.byref(_t(x)), ctypes.byref(_t(w)), ctypes.byref(_t(bias)),
                                      ctypes.byref(_t(out)), _i32(out_pad), _i32(stride), ctypes.c_int32(in_zp),
                                      ctypes.c_int32(w_zp)))
    return out


def conv3d(x, w, bias, out_shape, pad, stride, dil, in_zp, w_zp):
    out = np.zeros(out_shape, np.int64 if x.dtype == np.int16 else np.int32)
    _check(lib().orc_conv3d(ctypes.byref(_t(x)), ctypes.byref(_t(w)), ctypes.byref(_t(bias)), ctypes.byref(_t(out)),
                            _i32(pad), _i32(stride), _i32(dil), ctypes.c_int32(in_zp), ctypes.c_int32(w_zp)))
    return out


def fft2d(real, imag, inverse):
    out_re, out_im = np.zeros(real.shape, np.float32), np.zeros(real.shape, np.float32)
    _check(lib().orc_fft2d(ctypes.byref(_t(real)), ctypes.byref(_t(imag)), ctypes.byref(_t(out_re)),
                           ctypes.byref(_t(out_im)), int(bool(inverse))))
    return out_re, out_im


def rfft2d(x):
    shape = x.shape[:2] + (x.shape[2] // 2 + 1,)
    out_re, out_im = np.zeros(shape, np.float32), np.zeros(shape, np.float32)
    _check(lib().orc_fft2d(ctypes.byref(_t(x)), None, ctypes.byref(_t(out_re)), ctypes.byref(_t(out_im)), 0))
    return out_re, out_im
