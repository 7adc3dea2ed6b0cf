"""Replays a ``GraphBuilder`` graph on the CPU oracle, operator by operator.

Test infrastructure: this is the checker the CUDA path is compared with.  Every operator is
evaluated separately (no fusion), in recording order, with the oracle functions of
``oracle/oracle.py`` — i.e. the reference's one-shader-per-operator execution.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle


def evaluate(graph, inputs, keep_all=False):
    env = {}
    for v, a in zip(graph.inputs, inputs):
        env[v.name] = np.ascontiguousarray(a, dtype=v.dtype)

    def val(v):
        if v.name in env:
            return env[v.name]
        if v.data is not None:
            return v.data
        raise KeyError(v.name)

    for op in graph.ops:
        a, i = op.attrs, [val(v) for v in op.inputs]
        n = op.name
        if n == "CONV2D":
            r = oracle.conv2d(i[0], i[1], i[2], a["pad"], a["stride"], a["dilation"], a["in_zp"], a["w_zp"])
        elif n == "DEPTHWISE_CONV2D":
            r = oracle.depthwise_conv2d(i[0], i[1], i[2], a["pad"], a["stride"], a["dilation"], a["in_zp"], a["w_zp"])
        elif n == "MATMUL":
            r = oracle.matmul(i[0], i[1], a["zp_a"], a["zp_b"])
        elif n == "RESCALE":
            r = oracle.rescale(i[0], i[1], i[2], a["in_zp"], a["out_zp"], op.out.dtype, a["scale32"],
                               a["double_round"], a["per_channel"])
        elif n == "AVG_POOL2D":
            r = oracle.avg_pool2d(i[0], a["kernel"], a["stride"], a["pad"], a["in_zp"], a["out_zp"])
        elif n == "MAX_POOL2D":
            r = oracle.max_pool2d(i[0], a["kernel"], a["stride"], a["pad"])
        elif n == "TABLE":
            r = oracle.table(i[0], i[1])
        elif n == "TRANSPOSE":
            r = oracle.transpose(i[0], a["perms"])
        elif n == "CONCAT":
            r = oracle.concat(i, a["axis"])
        elif n == "CLAMP":
            r = oracle.clamp(i[0], a["min"], a["max"])
        elif n in oracle.BINARY_OPS:
            r = oracle.binary(n, i[0], i[1], op.out.dtype)
        elif n in oracle.UNARY_OPS:
            r = oracle.unary(n, i[0])
        elif n == "MUL":
            r = oracle.mul(i[0], i[1], a["shift"], op.out.dtype)
        elif n in oracle.REDUCE_OPS:
            r = oracle.reduce(n, i[0], a["axis"])
        elif n == "CAST":
            r = oracle.cast(i[0], op.out.dtype)
        elif n == "RESHAPE":
            r = oracle.reshape(i[0], op.out.shape)
        elif n == "SLICE":
            r = oracle.slice_(i[0], a["start"], a["size"])
        elif n == "PAD":
            r = oracle.pad(i[0], a["padding"], a["pad_const"])
        elif n == "ARITHMETIC_RIGHT_SHIFT":
            r = oracle.arithmetic_right_shift(i[0], i[1], a["round"])
        elif n == "NEGATE":
            r = oracle.negate(i[0], a["in_zp"], a["out_zp"])
        elif n == "SELECT":
            r = oracle.select(i[0], i[1], i[2])
        elif n in ("FFT2D", "RFFT2D"):
            r, second = oracle.fft2d(i[0], i[1], a["inverse"]) if n == "FFT2D" else oracle.rfft2d(i[0])
            env[op.more_outs[0].name] = second
        elif n == "ARGMAX":
            r = oracle.argmax(i[0], a["axis"])
        elif n == "GATHER":
            r = oracle.gather(i[0], i[1])
        elif n == "SCATTER":
            r = oracle.scatter(i[0], i[1], i[2])
        elif n == "REVERSE":
            r = oracle.reverse(i[0], a["axis"])
        elif n == "TILE":
            r = oracle.tile(i[0], a["multiples"])
        elif n == "RESIZE":
            r = oracle.resize(i[0], op.out.shape, op.out.dtype, a["scale"], a["offset"], a["border"], a["mode"])
        elif n == "TRANSPOSE_CONV2D":
            r = oracle.transpose_conv2d(i[0], i[1], i[2], op.out.shape, a["out_pad"], a["stride"], a["in_zp"],
                                        a["w_zp"])
        elif n == "CONV3D":
            r = oracle.conv3d(i[0], i[1], i[2], op.out.shape, a["pad"], a["stride"], a["dilation"], a["in_zp"],
                              a["w_zp"])
        else:
            raise NotImplementedError(n)
        assert tuple(r.shape) == tuple(op.out.shape), (n, r.shape, op.out.shape)
        env[op.out.name] = r
    outs = [val(v) for v, _, _ in graph.outputs]
    return (outs, env) if keep_all else outs
