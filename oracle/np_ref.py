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


# ---- index-driven operators, TRANSPOSE_CONV2D, CONV3D, integer RESIZE: written from the TOSA definitions of
# the operators (scatter-style accumulation for the transposed convolution, explicit zero padding for CONV3D,
# Python integers for RESIZE), i.e. not shaped like the shaders the C++ oracle follows.

def argmax(x, axis):
    return np.argmax(x, axis=axis).astype(np.int32)  # numpy returns the first maximum as well


def gather(values, indices):
    n = np.arange(values.shape[0])[:, None]
    return values[n, indices, :]


def scatter(values_in, indices, input_):
    out = values_in.copy()
    for n in range(indices.shape[0]):
        for w in reversed(range(indices.shape[1])):  # the first occurrence of an index must win
            out[n, indices[n, w]] = input_[n, w]
    return out


def transpose_conv2d(x, w, bias, out_pad, stride, in_zp, w_zp, acc=np.int32):
    n, h, wd, ic = x.shape
    oc, kh, kw, _ = w.shape
    oh = (h - 1) * stride[0] + out_pad[0] + out_pad[1] + kh
    ow = (wd - 1) * stride[1] + out_pad[2] + out_pad[3] + kw
    out = np.zeros((n, oh, ow, oc), dtype=object)
    out[...] = np.broadcast_to(np.asarray(bias, dtype=object), (oc,)) if bias.shape[0] == oc else int(bias[0])
    xs = x.astype(object) - in_zp
    ws = w.astype(object) - w_zp
    for iy in range(h):
        for ix in range(wd):
            for ky in range(kh):
                for kx in range(kw):
                    oy = iy * stride[0] + out_pad[0] + ky
                    ox = ix * stride[1] + out_pad[2] + kx
                    if 0 <= oy < oh and 0 <= ox < ow:
                        out[:, oy, ox, :] += xs[:, iy, ix, :] @ ws[:, ky, kx, :].T
    bits = 64 if acc == np.int64 else 32
    wrap = np.vectorize(lambda v: ((int(v) + (1 << (bits - 1))) % (1 << bits)) - (1 << (bits - 1)), otypes=[object])
    return wrap(out).astype(acc)


def conv3d(x, w, bias, pad, stride, dil, in_zp, w_zp):
    n, d, h, wd, ic = x.shape
    oc, kd, kh, kw, _ = w.shape
    xp = np.full((n, d + pad[0] + pad[1], h + pad[2] + pad[3], wd + pad[4] + pad[5], ic), in_zp, np.int64)
    xp[:, pad[0]:pad[0] + d, pad[2]:pad[2] + h, pad[4]:pad[4] + wd, :] = x
    xp -= in_zp
    ws = w.astype(np.int64) - w_zp
    od = (xp.shape[1] - (kd - 1) * dil[0] - 1) // stride[0] + 1
    oh = (xp.shape[2] - (kh - 1) * dil[1] - 1) // stride[1] + 1
    ow = (xp.shape[3] - (kw - 1) * dil[2] - 1) // stride[2] + 1
    out = np.zeros((n, od, oh, ow, oc), np.int64)
    for a in range(kd):
        for b in range(kh):
            for c in range(kw):
                win = xp[:, a * dil[0]:a * dil[0] + (od - 1) * stride[0] + 1:stride[0],
                         b * dil[1]:b * dil[1] + (oh - 1) * stride[1] + 1:stride[1],
                         c * dil[2]:c * dil[2] + (ow - 1) * stride[2] + 1:stride[2], :]
                out += np.einsum("ndhwi,oi->ndhwo", win, ws[:, a, b, c, :])
    out += bias.astype(np.int64)
    return out.astype(np.int32) if x.dtype == np.int8 else out


def resize(x, scale, offset, border, mode, out_dtype):
    n, h, w, c = x.shape
    yn, yd, xn, xd = scale
    oh = ((h - 1) * yn - offset[0] + border[0]) // yd + 1
    ow = ((w - 1) * xn - offset[1] + border[1]) // xd + 1
    out = np.zeros((n, oh, ow, c), out_dtype)
    for oy in range(oh):
        y = oy * yd + offset[0]
        iy, ry = y // yn, y % yn  # Python's floor division and non-negative remainder
        y0, y1 = max(iy, 0), min(iy + 1, h - 1)
        for ox in range(ow):
            xx = ox * xd + offset[1]
            ix, rx = xx // xn, xx % xn
            x0, x1 = max(ix, 0), min(ix + 1, w - 1)
            if mode == 1:
                out[:, oy, ox, :] = x[:, y1 if 2 * ry >= yn else y0, x1 if 2 * rx >= xn else x0, :]
            else:
                v = (x[:, y0, x0, :].astype(np.int64) * (yn - ry) * (xn - rx) + x[:, y0, x1, :].astype(np.int64) * (yn - ry) * rx +
                     x[:, y1, x0, :].astype(np.int64) * ry * (xn - rx) + x[:, y1, x1, :].astype(np.int64) * ry * rx)
                out[:, oy, ox, :] = v.astype(out_dtype)
    return out
