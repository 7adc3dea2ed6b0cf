"""Builds TOSA data graphs and emits them as SPIR-V assembly text (SPV_ARM_graph + TOSA.001000.1).

In the reference's world a graph reaches the layer as a SPIR-V module produced by a model
converter; its tests assemble such modules from text (tests/shader/*.spvasm).  ``GraphBuilder``
writes the same text form — same instructions, same operand order per TOSA operator as decoded
in graph/graph_tosa_1_0_ext_inst.cpp:315-1032 — so a graph built here enters the library exactly
where a real caller's module would: ``Pipeline.lower_spvasm`` after the external bindings and
graph constants have been registered.

The builder records each operator in ``ops`` (name, input values, attributes, output value) so
that a checker can replay the same graph elsewhere.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

_NP_NAME = {
    np.dtype(np.int8): "i8", np.dtype(np.int16): "i16", np.dtype(np.int32): "i32", np.dtype(np.int64): "i64",
    np.dtype(np.bool_): "bool", np.dtype(np.float32): "f32",
}
_WIDTH = {"i8": 8, "i16": 16, "i32": 32, "i64": 64}

# accType / nanMode / rounding-mode codes of the TOSA.001000.1 set as the reference decodes them
ACC_INT32, ACC_FP16, ACC_FP32, ACC_INT64 = 1, 2, 3, 4
NAN_PROPAGATE, NAN_IGNORE = 1, 2
ROUND_SINGLE, ROUND_INEXACT, ROUND_DOUBLE = 1, 2, 3


@dataclass
class Value:
    name: str              # SPIR-V id without '%'
    dtype: np.dtype
    shape: tuple
    kind: str              # "input" | "const" | "inline" | "op"
    data: np.ndarray | None = None
    const_id: int | None = None
    binding: tuple | None = None  # (set, binding) of an input


@dataclass
class OpRecord:
    name: str
    inputs: list
    attrs: dict
    out: Value
    operands: list = field(default_factory=list)  # emitted operand ids in TOSA order
    more_outs: list = field(default_factory=list)  # further results of a multi-result instruction (FFT2D, RFFT2D)


class GraphBuilder:
    def __init__(self, name: str = "main"):
        self.name = name
        self.ops: list[OpRecord] = []
        self.inputs: list[Value] = []
        self.outputs: list[tuple[Value, int, int]] = []   # (value, set, binding)
        self.constants: dict[int, np.ndarray] = {}        # OpGraphConstantARM id -> data
        self._decls: list[str] = []                        # types and constants, in dependency order
        self._declared: set[str] = set()
        self._graph_consts: list[Value] = []
        self._counter = 0
        self._next_binding = 0

    # ------------------------------------------------------------------ declarations
    def _decl(self, ident: str, text: str) -> str:
        if ident not in self._declared:
            self._declared.add(ident)
            self._decls.append(f"%{ident} = {text}")
        return "%" + ident

    def _scalar_type(self, dtype) -> str:
        n = _NP_NAME[np.dtype(dtype)]
        if n == "bool":
            return self._decl("bool", "OpTypeBool")
        if n == "f32":
            return self._decl("f32", "OpTypeFloat 32")
        return self._decl(n, f"OpTypeInt {_WIDTH[n]} 0")

    def _u32(self, v: int) -> str:
        t = self._scalar_type(np.int32)
        return self._decl(f"u32_{v}", f"OpConstant {t} {int(v) & 0xFFFFFFFF}")

    def _scalar_const(self, dtype, v) -> str:
        n = _NP_NAME[np.dtype(dtype)]
        t = self._scalar_type(dtype)
        if n == "bool":
            return self._decl("true" if v else "false", f"OpConstant{'True' if v else 'False'} {t}")
        if n == "f32":
            r = repr(float(v))
            return self._decl("f32_" + r.replace("-", "m").replace(".", "p").replace("+", ""), f"OpConstant {t} {r}")
        bits = int(v) & ((1 << _WIDTH[n]) - 1)  # integer types are declared unsigned; emit the bit pattern
        return self._decl(f"{n}_{bits}", f"OpConstant {t} {bits}")

    def _bool(self, v: bool) -> str:
        return self._scalar_const(np.bool_, bool(v))

    def _shape(self, shape: Sequence[int]) -> str:
        rank = len(shape)
        arr = self._decl(f"arr_{rank}", f"OpTypeArray {self._scalar_type(np.int32)} {self._u32(rank)}")
        elems = " ".join(self._u32(d) for d in shape)
        return self._decl("shape_" + "_".join(str(d) for d in shape), f"OpConstantComposite {arr} {elems}")

    def _tensor_type(self, dtype, shape: Sequence[int]) -> str:
        n = _NP_NAME[np.dtype(dtype)]
        ident = f"t_{n}_" + "_".join(str(d) for d in shape)
        return self._decl(ident, f"OpTypeTensorARM {self._scalar_type(dtype)} {self._u32(len(shape))} "
                                 f"{self._shape(shape)}")

    def _fresh(self, prefix: str) -> str:
        self._counter += 1
        return f"{prefix}{self._counter}"

    # ------------------------------------------------------------------ values
    def input(self, dtype, shape, set_: int = 0, binding: int | None = None) -> Value:
        if binding is None:
            binding = self._next_binding
        self._next_binding = max(self._next_binding, binding + 1)
        v = Value(self._fresh("in"), np.dtype(dtype), tuple(shape), "input", binding=(set_, binding))
        self.inputs.append(v)
        return v

    def constant(self, array: np.ndarray) -> Value:
        """A graph constant (OpGraphConstantARM): data handed over at pipeline creation."""
        array = np.ascontiguousarray(array)
        cid = len(self.constants)
        self.constants[cid] = array
        v = Value(self._fresh("gc"), array.dtype, tuple(array.shape), "const", data=array, const_id=cid)
        self._graph_consts.append(v)
        return v

    def inline(self, array) -> Value:
        """A small constant tensor written into the module (OpConstantComposite / Null / Replicate)."""
        array = np.ascontiguousarray(array)
        t = self._tensor_type(array.dtype, array.shape)
        flat = array.reshape(-1)
        name = self._fresh("k")
        if not flat.any():
            self._decls.append(f"%{name} = OpConstantNull {t}")
        elif flat.size > 1 and (flat == flat[0]).all():
            self._decls.append(f"%{name} = OpConstantCompositeReplicateEXT {t} "
                               f"{self._scalar_const(array.dtype, flat[0])}")
        else:
            elems = " ".join(self._scalar_const(array.dtype, x) for x in flat)
            self._decls.append(f"%{name} = OpConstantComposite {t} {elems}")
        return Value(name, array.dtype, tuple(array.shape), "inline", data=array)

    def output(self, value: Value, set_: int = 0, binding: int | None = None) -> None:
        if binding is None:
            binding = self._next_binding
        self._next_binding = max(self._next_binding, binding + 1)
        self.outputs.append((value, set_, binding))

    def _attr_tensor(self, array, dtype) -> Value:
        array = np.asarray(array, dtype=dtype)
        if array.size > 64:
            return self.constant(array)
        return self.inline(array)

    def _emit(self, name, operands, inputs, attrs, out_dtype, out_shape) -> Value:
        out = Value(self._fresh("v"), np.dtype(out_dtype), tuple(int(d) for d in out_shape), "op")
        self.ops.append(OpRecord(name, list(inputs), dict(attrs), out, list(operands)))
        return out

    # ------------------------------------------------------------------ TOSA operators
    @staticmethod
    def _conv_out(h, w, kh, kw, pad, stride, dil):
        oh = (h + pad[0] + pad[1] - (kh - 1) * dil[0] - 1) // stride[0] + 1
        ow = (w + pad[2] + pad[3] - (kw - 1) * dil[1] - 1) // stride[1] + 1
        return oh, ow

    def conv2d(self, x, w, bias, pad, stride, dilation, in_zp, w_zp, acc_type=ACC_INT32):
        n, h, wd, _ = x.shape
        oc, kh, kw, _ = w.shape
        oh, ow = self._conv_out(h, wd, kh, kw, pad, stride, dilation)
        acc = np.int64 if acc_type == ACC_INT64 else np.int32
        ops = [self.inline(np.asarray(pad, np.int32)).name, self.inline(np.asarray(stride, np.int32)).name,
               self.inline(np.asarray(dilation, np.int32)).name, self._u32(acc_type)[1:], self._bool(False)[1:],
               x.name, w.name, bias.name, self.inline(np.asarray([in_zp], np.int8)).name,
               self.inline(np.asarray([w_zp], np.int8)).name]
        return self._emit("CONV2D", ops, [x, w, bias],
                          dict(pad=list(pad), stride=list(stride), dilation=list(dilation), in_zp=in_zp, w_zp=w_zp),
                          acc, (n, oh, ow, oc))

    def depthwise_conv2d(self, x, w, bias, pad, stride, dilation, in_zp, w_zp, acc_type=ACC_INT32):
        n, h, wd, c = x.shape
        kh, kw, _, m = w.shape
        oh, ow = self._conv_out(h, wd, kh, kw, pad, stride, dilation)
        ops = [self.inline(np.asarray(pad, np.int32)).name, self.inline(np.asarray(stride, np.int32)).name,
               self.inline(np.asarray(dilation, np.int32)).name, self._u32(acc_type)[1:], self._bool(False)[1:],
               x.name, w.name, bias.name, self.inline(np.asarray([in_zp], np.int8)).name,
               self.inline(np.asarray([w_zp], np.int8)).name]
        return self._emit("DEPTHWISE_CONV2D", ops, [x, w, bias],
                          dict(pad=list(pad), stride=list(stride), dilation=list(dilation), in_zp=in_zp, w_zp=w_zp),
                          np.int32, (n, oh, ow, c * m))

    def matmul(self, a, b, zp_a, zp_b):
        ops = [a.name, b.name, self.inline(np.asarray([zp_a], np.int8)).name,
               self.inline(np.asarray([zp_b], np.int8)).name]
        return self._emit("MATMUL", ops, [a, b], dict(zp_a=zp_a, zp_b=zp_b), np.int32,
                          (a.shape[0], a.shape[1], b.shape[2]))

    def rescale(self, x, multiplier, shift, in_zp, out_zp, out_dtype, scale32=True, double_round=False,
                per_channel=False):
        mult = self._attr_tensor(multiplier, np.int32 if scale32 else np.int16)
        sh = self._attr_tensor(shift, np.int8)
        zp_in = self.inline(np.asarray([in_zp], x.dtype))
        zp_out = self.inline(np.asarray([out_zp], out_dtype))
        ops = [self._bool(scale32)[1:], self._u32(ROUND_DOUBLE if double_round else ROUND_SINGLE)[1:],
               self._bool(per_channel)[1:], self._bool(False)[1:], self._bool(False)[1:], x.name, mult.name, sh.name,
               zp_in.name, zp_out.name]
        return self._emit("RESCALE", ops, [x, mult, sh],
                          dict(in_zp=in_zp, out_zp=out_zp, scale32=scale32, double_round=double_round,
                               per_channel=per_channel), out_dtype, x.shape)

    def _pool_shape(self, x, kernel, stride, pad):
        n, h, w, c = x.shape
        return (n, (h + pad[0] + pad[1] - kernel[0]) // stride[0] + 1,
                (w + pad[2] + pad[3] - kernel[1]) // stride[1] + 1, c)

    def avg_pool2d(self, x, kernel, stride, pad, in_zp, out_zp, acc_type=ACC_INT32):
        ops = [self.inline(np.asarray(kernel, np.int32)).name, self.inline(np.asarray(stride, np.int32)).name,
               self.inline(np.asarray(pad, np.int32)).name, self._u32(acc_type)[1:], x.name,
               self.inline(np.asarray([in_zp], np.int8)).name, self.inline(np.asarray([out_zp], np.int8)).name]
        return self._emit("AVG_POOL2D", ops, [x],
                          dict(kernel=list(kernel), stride=list(stride), pad=list(pad), in_zp=in_zp, out_zp=out_zp),
                          x.dtype, self._pool_shape(x, kernel, stride, pad))

    def max_pool2d(self, x, kernel, stride, pad):
        ops = [self.inline(np.asarray(kernel, np.int32)).name, self.inline(np.asarray(stride, np.int32)).name,
               self.inline(np.asarray(pad, np.int32)).name, self._u32(NAN_PROPAGATE)[1:], x.name]
        return self._emit("MAX_POOL2D", ops, [x], dict(kernel=list(kernel), stride=list(stride), pad=list(pad)),
                          x.dtype, self._pool_shape(x, kernel, stride, pad))

    def table(self, x, table):
        t = self._attr_tensor(table, x.dtype)
        return self._emit("TABLE", [x.name, t.name], [x, t], {}, np.int8 if x.dtype == np.int8 else np.int32, x.shape)

    def transpose(self, x, perms):
        p = self.inline(np.asarray(perms, np.int32))
        return self._emit("TRANSPOSE", [p.name, x.name], [x], dict(perms=list(perms)), x.dtype,
                          [x.shape[i] for i in perms])

    def concat(self, inputs, axis):
        shape = list(inputs[0].shape)
        shape[axis] = sum(v.shape[axis] for v in inputs)
        return self._emit("CONCAT", [self._u32(axis)[1:]] + [v.name for v in inputs], list(inputs), dict(axis=axis),
                          inputs[0].dtype, shape)

    def clamp(self, x, min_value, max_value):
        ops = [self._scalar_const(x.dtype, min_value)[1:], self._scalar_const(x.dtype, max_value)[1:],
               self._u32(NAN_PROPAGATE)[1:], x.name]
        return self._emit("CLAMP", ops, [x], dict(min=min_value, max=max_value), x.dtype, x.shape)

    def binary(self, name, a, b, out_dtype=None):
        shape = tuple(max(p, q) for p, q in zip(a.shape, b.shape))
        if out_dtype is None:
            out_dtype = np.bool_ if name in ("EQUAL", "GREATER", "GREATER_EQUAL") else a.dtype
        if name in ("MAXIMUM", "MINIMUM"):
            ops = [self._u32(NAN_PROPAGATE)[1:], a.name, b.name]
        else:
            ops = [a.name, b.name]
        return self._emit(name, ops, [a, b], {}, out_dtype, shape)

    def add(self, a, b):
        return self.binary("ADD", a, b)

    def sub(self, a, b):
        return self.binary("SUB", a, b)

    def unary(self, name, x):
        return self._emit(name, [x.name], [x], {}, x.dtype, x.shape)

    def mul(self, a, b, shift):
        s = self.inline(np.asarray([shift], np.int8))
        shape = tuple(max(p, q) for p, q in zip(a.shape, b.shape))
        return self._emit("MUL", [a.name, b.name, s.name], [a, b], dict(shift=shift), np.int32, shape)

    def reduce(self, name, x, axis):
        shape = list(x.shape)
        shape[axis] = 1
        if name in ("REDUCE_MAX", "REDUCE_MIN"):
            ops = [self._u32(axis)[1:], self._u32(NAN_PROPAGATE)[1:], x.name]
        else:
            ops = [self._u32(axis)[1:], x.name]
        return self._emit(name, ops, [x], dict(axis=axis), x.dtype, shape)

    def cast(self, x, out_dtype):
        return self._emit("CAST", [x.name], [x], {}, out_dtype, x.shape)

    def reshape(self, x, shape):
        s = self.inline(np.asarray(shape, np.int32))
        return self._emit("RESHAPE", [x.name, s.name], [x], dict(shape=list(shape)), x.dtype, shape)

    def slice(self, x, start, size):
        ops = [x.name, self.inline(np.asarray(start, np.int32)).name, self.inline(np.asarray(size, np.int32)).name]
        return self._emit("SLICE", ops, [x], dict(start=list(start), size=list(size)), x.dtype, size)

    def pad(self, x, padding, pad_const):
        p = self.inline(np.asarray(padding, np.int32).reshape(-1))
        c = self.inline(np.asarray([pad_const], x.dtype))
        flat = list(np.asarray(padding).reshape(-1))
        shape = [x.shape[i] + int(flat[2 * i]) + int(flat[2 * i + 1]) for i in range(len(x.shape))]
        return self._emit("PAD", [x.name, p.name, c.name], [x], dict(padding=[int(v) for v in flat],
                                                                    pad_const=pad_const), x.dtype, shape)

    def arithmetic_right_shift(self, a, b, round_):
        shape = tuple(max(p, q) for p, q in zip(a.shape, b.shape))
        return self._emit("ARITHMETIC_RIGHT_SHIFT", [self._bool(round_)[1:], a.name, b.name], [a, b],
                          dict(round=round_), a.dtype, shape)

    def negate(self, x, in_zp, out_zp):
        ops = [x.name, self.inline(np.asarray([in_zp], np.int32)).name,
               self.inline(np.asarray([out_zp], np.int32)).name]
        return self._emit("NEGATE", ops, [x], dict(in_zp=in_zp, out_zp=out_zp), x.dtype, x.shape)

    def select(self, cond, a, b):
        shape = tuple(max(p, q, r) for p, q, r in zip(cond.shape, a.shape, b.shape))
        return self._emit("SELECT", [cond.name, a.name, b.name], [cond, a, b], {}, a.dtype, shape)

    def argmax(self, x, axis, nan_mode=NAN_PROPAGATE):
        shape = x.shape[:axis] + x.shape[axis + 1:]
        return self._emit("ARGMAX", [self._u32(axis)[1:], self._u32(nan_mode)[1:], x.name], [x], dict(axis=axis),
                          np.int32, shape)

    def gather(self, values, indices):
        shape = (values.shape[0], indices.shape[1], values.shape[2])
        return self._emit("GATHER", [values.name, indices.name], [values, indices], {}, values.dtype, shape)

    def scatter(self, values_in, indices, input_):
        return self._emit("SCATTER", [values_in.name, indices.name, input_.name], [values_in, indices, input_], {},
                          values_in.dtype, values_in.shape)

    def reverse(self, x, axis):
        return self._emit("REVERSE", [self._u32(axis)[1:], x.name], [x], dict(axis=axis), x.dtype, x.shape)

    def tile(self, x, multiples):
        m = self.inline(np.asarray(multiples, np.int32))
        shape = tuple(d * int(k) for d, k in zip(x.shape, multiples))
        return self._emit("TILE", [x.name, m.name], [x], dict(multiples=list(multiples)), x.dtype, shape)

    def resize(self, x, scale, offset, border, mode, out_dtype):
        """``scale`` = (y_n, y_d, x_n, x_d); ``mode`` 1 = NEAREST, 2 = BILINEAR.  Output size as in TOSA:
        ``(in - 1) * n - offset + border) // d + 1`` per axis."""
        n, h, w, c = x.shape
        oh = ((h - 1) * scale[0] - offset[0] + border[0]) // scale[1] + 1
        ow = ((w - 1) * scale[2] - offset[1] + border[1]) // scale[3] + 1
        ops = [self._u32(mode)[1:], x.name, self.inline(np.asarray(scale, np.int32)).name,
               self.inline(np.asarray(offset, np.int32)).name, self.inline(np.asarray(border, np.int32)).name]
        return self._emit("RESIZE", ops, [x], dict(scale=list(scale), offset=list(offset), border=list(border),
                                                   mode=mode), out_dtype, (n, oh, ow, c))

    def transpose_conv2d(self, x, w, bias, out_pad, stride, in_zp, w_zp, acc_type=ACC_INT32):
        n, h, wd, _ = x.shape
        oc, kh, kw, _ = w.shape
        oh = (h - 1) * stride[0] + out_pad[0] + out_pad[1] + kh
        ow = (wd - 1) * stride[1] + out_pad[2] + out_pad[3] + kw
        acc = np.int64 if acc_type == ACC_INT64 else np.int32
        ops = [self.inline(np.asarray(out_pad, np.int32)).name, self.inline(np.asarray(stride, np.int32)).name,
               self._u32(acc_type)[1:], self._bool(False)[1:], x.name, w.name, bias.name,
               self.inline(np.asarray([in_zp], np.int8)).name, self.inline(np.asarray([w_zp], np.int8)).name]
        return self._emit("TRANSPOSE_CONV2D", ops, [x, w, bias],
                          dict(out_pad=list(out_pad), stride=list(stride), in_zp=in_zp, w_zp=w_zp), acc,
                          (n, oh, ow, oc))

    def conv3d(self, x, w, bias, pad, stride, dilation, in_zp, w_zp, acc_type=ACC_INT32):
        n, d, h, wd, _ = x.shape
        oc, kd, kh, kw, _ = w.shape
        od = (d + pad[0] + pad[1] - (kd - 1) * dilation[0] - 1) // stride[0] + 1
        oh = (h + pad[2] + pad[3] - (kh - 1) * dilation[1] - 1) // stride[1] + 1
        ow = (wd + pad[4] + pad[5] - (kw - 1) * dilation[2] - 1) // stride[2] + 1
        acc = np.int64 if acc_type == ACC_INT64 else np.int32
        ops = [self.inline(np.asarray(pad, np.int32)).name, self.inline(np.asarray(stride, np.int32)).name,
               self.inline(np.asarray(dilation, np.int32)).name, self._u32(acc_type)[1:], self._bool(False)[1:],
               x.name, w.name, bias.name, self.inline(np.asarray([in_zp], np.int8)).name,
               self.inline(np.asarray([w_zp], np.int8)).name]
        return self._emit("CONV3D", ops, [x, w, bias],
                          dict(pad=list(pad), stride=list(stride), dilation=list(dilation), in_zp=in_zp, w_zp=w_zp),
                          acc, (n, od, oh, ow, oc))

    def _emit2(self, name, operands, inputs, attrs, out_dtype, out_shape):
        """An instruction with two results of one type, returned as a struct and taken apart by
        OpCompositeExtract."""
        first = self._emit(name, operands, inputs, attrs, out_dtype, out_shape)
        second = Value(self._fresh("v"), np.dtype(out_dtype), tuple(int(d) for d in out_shape), "op")
        self.ops[-1].more_outs.append(second)
        return first, second

    def fft2d(self, real, imag, inverse):
        ops = [self._bool(inverse)[1:], self._bool(False)[1:], real.name, imag.name]
        return self._emit2("FFT2D", ops, [real, imag], dict(inverse=bool(inverse)), np.float32, real.shape)

    def rfft2d(self, x):
        shape = x.shape[:2] + (x.shape[2] // 2 + 1,)
        return self._emit2("RFFT2D", [self._bool(False)[1:], x.name], [x], {}, np.float32, shape)

    # ------------------------------------------------------------------ emission
    def spvasm(self) -> str:
        head = [
            "OpCapability VulkanMemoryModel", "OpCapability Shader", "OpCapability Int8", "OpCapability Int16",
            "OpCapability Int64", "OpCapability TensorsARM", "OpCapability GraphARM",
            "OpCapability ReplicatedCompositesEXT", 'OpExtension "SPV_ARM_tensors"', 'OpExtension "SPV_ARM_graph"',
            'OpExtension "SPV_EXT_replicated_composites"', '%tosa = OpExtInstImport "TOSA.001000.1"',
            "OpMemoryModel Logical Vulkan",
        ]
        deco, var_decls, iface = [], [], []
        in_types, out_types = [], []
        for v in self.inputs:
            t = self._tensor_type(v.dtype, v.shape)
            ptr = self._decl("ptr_" + t[1:], f"OpTypePointer UniformConstant {t}")
            var = f"%var_{v.name}"
            deco += [f"OpDecorate {var} DescriptorSet {v.binding[0]}", f"OpDecorate {var} Binding {v.binding[1]}"]
            var_decls.append(f"{var} = OpVariable {ptr} UniformConstant")
            iface.append(var)
            in_types.append(t)
        for k, (v, s, b) in enumerate(self.outputs):
            t = self._tensor_type(v.dtype, v.shape)
            ptr = self._decl("ptr_" + t[1:], f"OpTypePointer UniformConstant {t}")
            var = f"%var_out{k}"
            deco += [f"OpDecorate {var} DescriptorSet {s}", f"OpDecorate {var} Binding {b}"]
            var_decls.append(f"{var} = OpVariable {ptr} UniformConstant")
            iface.append(var)
            out_types.append(t)
        gconsts = [f"%{v.name} = OpGraphConstantARM {self._tensor_type(v.dtype, v.shape)} {v.const_id}"
                   for v in self._graph_consts]
        body = []
        for k, v in enumerate(self.inputs):
            body.append(f"%{v.name} = OpGraphInputARM {self._tensor_type(v.dtype, v.shape)} {self._u32(k)}")
        for op in self.ops:
            t = self._tensor_type(op.out.dtype, op.out.shape)
            args = " ".join("%" + o for o in op.operands)
            if op.more_outs:
                outs = [op.out] + op.more_outs
                types = [self._tensor_type(v.dtype, v.shape) for v in outs]
                st = self._decl("struct_" + "_".join(x[1:] for x in types), "OpTypeStruct " + " ".join(types))
                body.append(f"%{op.out.name}_all = OpExtInst {st} %tosa {op.name} {args}")
                for k, (v, vt) in enumerate(zip(outs, types)):
                    body.append(f"%{v.name} = OpCompositeExtract {vt} %{op.out.name}_all {k}")
                continue
            body.append(f"%{op.out.name} = OpExtInst {t} %tosa {op.name} {args}")
        for k, (v, _, _) in enumerate(self.outputs):
            body.append(f"OpGraphSetOutputARM %{v.name} {self._u32(k)}")
        gtype = f"%graph_t = OpTypeGraphARM {len(self.inputs)} " + " ".join(in_types + out_types)
        lines = (head + deco + self._decls + gconsts + var_decls + [gtype] +
                 [f'OpGraphEntryPointARM %graph "{self.name}" ' + " ".join(iface), "%graph = OpGraphARM %graph_t"] +
                 body + ["OpGraphEndARM"])
        return "\n".join(lines) + "\n"
