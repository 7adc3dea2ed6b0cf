"""Second, independent restatement of the reference operators in numpy.

TEST INFRASTRUCTURE ONLY.  The C++ oracle (``mlel_oracle.cpp``) walks the shaders statement by
statement; this file states the same mathematics a different way (whole-array int64 numpy,
explicit padding instead of skipped taps) so that a transcription slip in either shows up as
a disagreement.  Operators with no golden vector in the reference's tests (MATMUL,
DEPTHWISE_CONV2D, AVG_POOL2D, TABLE, per-channel / double-round RESCALE ...) are pinned only by
this cross-check: "parity unpinned" by reference data.

Reference shaders: graph/shaders/graph_op/tosa/{conv2d,depthwise_conv2d,matmul,rescale,
avgpool2d,maxpool2d,table,mul}.comp.
"""
from __future__ import annotations

import numpy as np


def _wrap32(a):
    return (np.asarray(a, np.int64) & 0xFFFFFFFF).astype(np.uint32).view(np.int32)


def _windows(xp, kh, kw, stride, dil, oh, ow):
    """Yield (ky, kx, view[n, oh, ow, c]) for each kernel tap over an already padded input."""
    for ky in range(kh):
        for kx in range(kw):
            y0, x0 = ky * dil[0], kx * dil[1]
            yield ky, kx, xp[:, y0:y0 + (oh - 1) * stride[0] + 1:stride[0],
                             x0:x0 + (ow - 1) * stride[1] + 1:stride[1], :]


def _out_hw(h, w, kh, kw, pad, stride, dil):
    oh = (h + pad[0] + pad[1] - (kh - 1) * dil[0] - 1) // stride[0] + 1
    ow = (w + pad[2] + pad[3] - (kw - 1) * dil[1] - 1) // stride[1] + 1
    return oh, ow


def conv2d(x, w, bias, pad, stride, dil, in_zp, w_zp):
    """conv2d.comp: out-of-range taps are skipped == padding with the input zero point."""
    n, h, wd, _ = x.shape
    oc, kh, kw, _ = w.shape
    oh, ow = _out_hw(h, wd, kh, kw, pad, stride, dil)
    xs = x.astype(np.int64) - in_zp
    # pad generously on the bottom/right so that strided windows never run off the array
    xp = np.pad(xs, ((0, 0), (pad[0], pad[1] + kh * dil[0] + stride[0]), (pad[2], pad[3] + kw * dil[1] + stride[1]),
                     (0, 0)))
    ws = w.astype(np.int64) - w_zp
    acc = np.zeros((n, oh, ow, oc), np.int64)
    for ky, kx, win in _windows(xp, kh, kw, stride, dil, oh, ow):
        acc += np.einsum("nhwc,oc->nhwo", win, ws[:, ky, kx, :], optimize=True)
    b = bias.astype(np.int64)
    acc += b[0] if b.shape[0] == 1 else b
    return _wrap32(acc) if x.dtype == np.int8 else acc


def depthwise_conv2d(x, w, bias, pad, stride, dil, in_zp, w_zp):
    n, h, wd, c = x.shape
    kh, kw, _, m = w.shape
    oh, ow = _out_hw(h, wd, kh, kw, pad, stride, dil)
    xs = x.astype(np.int64) - in_zp
    xp = np.pad(xs, ((0, 0), (pad[0], pad[1] + kh * dil[0] + stride[0]), (pad[2], pad[3] + kw * dil[1] + stride[1]),
                     (0, 0)))
    ws = w.astype(np.int64) - w_zp
    acc = np.zeros((n, oh, ow, c, m), np.int64)
    for ky, kx, win in _windows(xp, kh, kw, stride, dil, oh, ow):
        acc += win[..., None] * ws[ky, kx][None, None, None]
    acc = acc.reshape(n, oh, ow, c * m)
    b = bias.astype(np.int64)
    acc += b[0] if b.shape[0] == 1 else b
    return _wrap32(acc) if x.dtype == np.int8 else acc


def matmul(a, b, zp_a, zp_b):
    acc = np.matmul(a.astype(np.int64) - zp_a, b.astype(np.int64) - zp_b)
    return _wrap32(acc) if a.dtype == np.int8 else acc


def rescale(x, mult, shift, in_zp, out_zp, out_dtype, scale32=True, double_round=False, per_channel=False):
    """rescale.comp with arbitrary-precision Python integers (wraps applied explicitly)."""
    info = np.iinfo(out_dtype)
    in_info = np.iinfo(x.dtype)

    def narrow(v, inf):
        span = int(inf.max) - int(inf.min) + 1
        return (int(v) - int(inf.min)) % span + int(inf.min)

    in_zp_n = narrow(in_zp, in_info)
    out_zp_n = narrow(out_zp, info)
    flat = x.reshape(-1, x.shape[-1]) if x.ndim > 0 else x.reshape(1, 1)
    out = np.zeros(flat.shape, out_dtype)
    mult = np.asarray(mult).reshape(-1)
    shift = np.asarray(shift).reshape(-1)
    for c in range(flat.shape[1]):
        m = int(mult[c if per_channel else 0])
        s = int(shift[c if per_channel else 0])
        for r in range(flat.shape[0]):
            v = int(flat[r, c]) - in_zp_n
            rnd = (1 << (s - 1)) if s > 0 else 0
            if scale32 and double_round and s > 31:
                rnd += (1 << 30) if v >= 0 else -(1 << 30)
            res = (v * m + rnd) >> s  # Python >> is arithmetic (floor), like GLSL on signed
            res = narrow(res, np.iinfo(np.int32))
            res = narrow(res + out_zp_n, np.iinfo(np.int32))
            out[r, c] = min(max(res, int(info.min)), int(info.max))
    return out.reshape(x.shape)


def avg_pool2d(x, kernel, stride, pad, in_zp, out_zp):
    n, h, w, c = x.shape
    oh = (h + pad[0] + pad[1] - kernel[0]) // stride[0] + 1
    ow = (w + pad[2] + pad[3] - kernel[1]) // stride[1] + 1
    info = np.iinfo(x.dtype)
    out = np.zeros((n, oh, ow, c), x.dtype)
    xs = x.astype(np.int64) - in_zp
    for oy in range(oh):
        for ox in range(ow):
            y0, x0 = oy * stride[0] - pad[0], ox * stride[1] - pad[2]
            ys = [y for y in range(y0, y0 + kernel[0]) if 0 <= y < h]
            xs_ = [xx for xx in range(x0, x0 + kernel[1]) if 0 <= xx < w]
            count = len(ys) * len(xs_)
            acc = xs[:, ys][:, :, xs_].sum(axis=(1, 2))
            half = count >> 1
            acc = acc + np.where(acc < 0, -half, half)
            q = np.sign(acc) * (np.abs(acc) // count)  # truncation toward zero
            out[:, oy, ox, :] = np.clip(q + out_zp, info.min, info.max).astype(x.dtype)
    return out


def max_pool2d(x, kernel, stride, pad):
    n, h, w, c = x.shape
    oh = (h + pad[0] + pad[1] - kernel[0]) // stride[0] + 1
    ow = (w + pad[2] + pad[3] - kernel[1]) // stride[1] + 1
    lowest = np.iinfo(x.dtype).min
    xp = np.pad(x, ((0, 0), (pad[0], pad[1] + kernel[0] + stride[0]), (pad[2], pad[3] + kernel[1] + stride[1]), (0, 0)),
                constant_values=lowest)
    out = np.full((n, oh, ow, c), lowest, x.dtype)
    for _, _, win in _windows(xp, kernel[0], kernel[1], stride, (1, 1), oh, ow):
        out = np.maximum(out, win)
    return out


def table(x, tbl):
    if x.dtype == np.int8:
        return tbl[x.astype(np.int64) + 128].astype(np.int8)
    v = x.astype(np.int64)
    index = (v + 32768) >> 7
    frac = v & 0x7F
    base = tbl[index].astype(np.int64)
    nxt = tbl[index + 1].astype(np.int64)
    return _wrap32((base << 7) + (nxt - base) * frac)


def mul(a, b, shift):
    r = a.astype(np.int64) * b.astype(np.int64)
    if shift > 0:
        r = (r + (1 << (shift - 1))) >> shift
    return _wrap32(r)
