// Generic (any rank <= 6, any stride, any supported element type) CUDA kernels for the TOSA
// operators of the data-graph path.  One thread produces one output element, exactly the
// work split of the reference's 1-D compute shaders (graph/compute_graph_op.cpp:551-560), so
// every shape and stride the reference accepts is accepted here.  The vectorised and
// tensor-core kernels in the sibling files take over for the packed int8 shapes that dominate
// real graphs; these kernels are the always-correct path behind them.
//
// Reference arithmetic: graph/shaders/graph_op/tosa/<op>.comp (cited per kernel).
#include "device_common.cuh"
#include "kernels.hpp"

namespace mlel {

namespace {

#define GRID_STRIDE(e, total)                                                                                          \
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < (total); e += int64_t(gridDim.x) * blockDim.x)

__host__ __device__ inline int64_t numelOf(const TView &t) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; ++i) {
        n *= t.dims[i];
    }
    return n;
}

// common.comp:64-72
__device__ inline void broadcastIndex(const TView &t, const uint32_t *idx, uint32_t *c) {
#pragma unroll
    for (int i = 0; i < kMaxRank; ++i) {
        c[i] = (i < t.rank && t.dims[i] == 1) ? 0u : idx[i];
    }
}

// ---- CONV2D: conv2d.comp:26-116 ------------------------------------------------------------------
template <typename ACC>
__global__ void conv2dGeneric(TView in, TView w, TView bias, TView out, ConvAttr a) {
    using U = typename std::make_unsigned<ACC>::type;
    const int64_t total = numelOf(out);
    const uint32_t KH = w.dims[1], KW = w.dims[2], IC = in.dims[3], H = in.dims[1], W = in.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], oc = idx[3];
        const uint32_t iy = oy * uint32_t(a.stride[0]) - uint32_t(a.pad[0]);
        const uint32_t ix = ox * uint32_t(a.stride[1]) - uint32_t(a.pad[2]);
        U acc = 0;
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                const uint32_t y = iy + ky * uint32_t(a.dilation[0]);
                const uint32_t x = ix + kx * uint32_t(a.dilation[1]);
                if (y < H && x < W) {
                    const uint32_t ci0[4] = {n, y, x, 0};
                    const uint32_t cw0[4] = {oc, ky, kx, 0};
                    const int64_t io = offsetOf(in, ci0), wo = offsetOf(w, cw0);
                    for (uint32_t ic = 0; ic < IC; ++ic) {
                        const ACC v = ACC(loadIntAt(in, io + int64_t(ic) * in.strides[3])) - ACC(a.inZp);
                        const ACC wt = (wo < 0 || ic >= w.dims[3]) ? ACC(0) - ACC(a.wZp)
                                              : ACC(loadIntAt(w, wo + int64_t(ic) * w.strides[3])) - ACC(a.wZp);
                        acc += U(v) * U(wt);
                    }
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
        acc += U(ACC(loadInt(bias, cb)));
        storeInt(out, idx, int64_t(ACC(acc)));
    }
}

// ---- DEPTHWISE_CONV2D: depthwise_conv2d.comp:31-78 -------------------------------------------------
template <typename ACC>
__global__ void depthwiseGeneric(TView in, TView w, TView bias, TView out, ConvAttr a) {
    using U = typename std::make_unsigned<ACC>::type;
    const int64_t total = numelOf(out);
    const uint32_t KH = w.dims[0], KW = w.dims[1], M = w.dims[3], H = in.dims[1], W = in.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], ocm = idx[3];
        const uint32_t c = ocm / M, m = ocm % M;
        const uint32_t iy = oy * uint32_t(a.stride[0]) - uint32_t(a.pad[0]);
        const uint32_t ix = ox * uint32_t(a.stride[1]) - uint32_t(a.pad[2]);
        U acc = 0;
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                const uint32_t y = iy + ky * uint32_t(a.dilation[0]);
                const uint32_t x = ix + kx * uint32_t(a.dilation[1]);
                if (y < H && x < W) {
                    const uint32_t ci[4] = {n, y, x, c};
                    const uint32_t cw[4] = {ky, kx, c, m};
                    const ACC v = ACC(loadInt(in, ci)) - ACC(a.inZp);
                    const ACC wt = ACC(loadInt(w, cw)) - ACC(a.wZp);
                    acc += U(v) * U(wt);
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : ocm};
        acc += U(ACC(loadInt(bias, cb)));
        storeInt(out, idx, int64_t(ACC(acc)));
    }
}

// ---- MATMUL: matmul.comp:30-73 ---------------------------------------------------------------------
template <typename ACC> __global__ void matmulGeneric(TView a, TView b, TView out, int32_t zpA, int32_t zpB) {
    using U = typename std::make_unsigned<ACC>::type;
    const int64_t total = numelOf(out);
    const uint32_t K = a.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t ca[3] = {idx[0], idx[1], 0};
        const uint32_t cb[3] = {idx[0], 0, idx[2]};
        const int64_t ao = offsetOf(a, ca), bo = offsetOf(b, cb);
        U acc = 0;
        for (uint32_t c = 0; c < K; ++c) {
            const ACC v1 = (ao < 0 ? ACC(0) : ACC(loadIntAt(a, ao + int64_t(c) * a.strides[2]))) - ACC(zpA);
            const ACC v2 = ((bo < 0 || c >= b.dims[1]) ? ACC(0) : ACC(loadIntAt(b, bo + int64_t(c) * b.strides[1]))) -
                           ACC(zpB);
            acc += U(v1) * U(v2);
        }
        storeInt(out, idx, int64_t(ACC(acc)));
    }
}

// ---- RESCALE: rescale.comp:48-72 -------------------------------------------------------------------
__global__ void rescaleGeneric(TView in, TView out, TView mult, TView shift, RescaleAttr a) {
    const int64_t total = numelOf(out);
    const int64_t lo = typeLowest(out.dtype), hi = typeMax(out.dtype);
    const int64_t inZp = wrapTo(in.dtype, a.inZp);
    const int32_t outZp = int32_t(wrapTo(out.dtype, a.outZp));
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t c[1] = {a.perChannel ? idx[out.rank - 1] : 0u};
        const int64_t value = loadInt(in, idx) - inZp;
        const int32_t m = int32_t(loadInt(mult, c));
        const int32_t s = int32_t(int8_t(loadInt(shift, c)));
        int32_t r = applyScale(value, m, s, a.scale32 && a.doubleRound);
        r = int32_t(uint32_t(r) + uint32_t(outZp));
        const int64_t clamped = r < lo ? lo : (r > hi ? hi : int64_t(r));
        storeInt(out, idx, clamped);
    }
}

// ---- AVG_POOL2D: avgpool2d.comp:27-75 (integer path) -----------------------------------------------
__global__ void avgPoolGeneric(TView in, TView out, PoolAttr a) {
    const int64_t total = numelOf(out);
    const int64_t lo = typeLowest(out.dtype), hi = typeMax(out.dtype);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        uint32_t acc = 0, count = 0;
        const uint32_t iy = idx[1] * uint32_t(a.stride[0]) - uint32_t(a.pad[0]);
        const uint32_t ix = idx[2] * uint32_t(a.stride[1]) - uint32_t(a.pad[2]);
        for (uint32_t ky = 0; ky < uint32_t(a.kernel[0]); ++ky) {
            for (uint32_t kx = 0; kx < uint32_t(a.kernel[1]); ++kx) {
                const uint32_t y = iy + ky, x = ix + kx;
                if (y < in.dims[1] && x < in.dims[2]) {
                    const uint32_t ci[4] = {idx[0], y, x, idx[3]};
                    acc += uint32_t(int32_t(loadInt(in, ci))) - uint32_t(a.inZp);
                    count++;
                }
            }
        }
        int32_t v = int32_t(acc);
        if (count == 0) {
            v = 0;
        } else {
            const int32_t round = v < 0 ? -int32_t(count >> 1) : int32_t(count >> 1);
            v = int32_t(uint32_t(v) + uint32_t(round));
            v = v / int32_t(count); // truncates toward zero
        }
        v = int32_t(uint32_t(v) + uint32_t(a.outZp));
        storeInt(out, idx, v < lo ? lo : (v > hi ? hi : int64_t(v)));
    }
}

// ---- MAX_POOL2D: maxpool2d.comp:23-72 (integer path) -----------------------------------------------
__global__ void maxPoolGeneric(TView in, TView out, PoolAttr a) {
    const int64_t total = numelOf(out);
    const int kY = max(a.kernel[0], 0), kX = max(a.kernel[1], 0);
    const int sY = max(a.stride[0], 1), sX = max(a.stride[1], 1);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        int64_t acc = typeLowest(out.dtype);
        const int iy = int(idx[1]) * sY - a.pad[0];
        const int ix = int(idx[2]) * sX - a.pad[2];
        for (int ky = 0; ky < kY; ++ky) {
            for (int kx = 0; kx < kX; ++kx) {
                const int y = iy + ky, x = ix + kx;
                if (y >= 0 && x >= 0 && uint32_t(y) < in.dims[1] && uint32_t(x) < in.dims[2]) {
                    const uint32_t ci[4] = {idx[0], uint32_t(y), uint32_t(x), idx[3]};
                    const int64_t v = loadInt(in, ci);
                    acc = v > acc ? v : acc;
                }
            }
        }
        storeInt(out, idx, acc);
    }
}

// ---- TABLE: table.comp:17-52 -----------------------------------------------------------------------
__global__ void tableGeneric(TView in, TView out, TView table) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        int32_t result;
        if (in.dtype == MLEL_I8) {
            const uint32_t ct[1] = {uint32_t(int32_t(loadInt(in, idx)) + 128)};
            result = int32_t(loadInt(table, ct));
        } else {
            const int32_t v = int32_t(loadInt(in, idx));
            const int32_t index = (v + 32768) >> 7;
            const int32_t fraction = v & 0x7f;
            const uint32_t c0[1] = {uint32_t(index)};
            const uint32_t c1[1] = {uint32_t(index) + 1u};
            const int32_t base = int32_t(loadInt(table, c0));
            const int32_t next = int32_t(loadInt(table, c1));
            const int32_t slope = next - base;
            result = int32_t((uint32_t(base) << 7) + uint32_t(slope) * uint32_t(fraction));
        }
        storeInt(out, idx, result);
    }
}

// ---- data movement: transpose.comp, concat.comp, reshape.comp, slice.comp, pad.comp ----------------
enum MoveKind { MOVE_TRANSPOSE, MOVE_CONCAT, MOVE_RESHAPE, MOVE_SLICE, MOVE_PAD, MOVE_CAST_SAME };

__device__ inline void copyElem(const TView &in, int64_t so, const TView &out, int64_t doff) {
    switch (dtypeSize(out.dtype)) {
    case 1:
        *reinterpret_cast<uint8_t *>(out.ptr + doff) = so < 0 ? 0 : *reinterpret_cast<const uint8_t *>(in.ptr + so);
        break;
    case 2:
        *reinterpret_cast<uint16_t *>(out.ptr + doff) = so < 0 ? 0 : *reinterpret_cast<const uint16_t *>(in.ptr + so);
        break;
    case 4:
        *reinterpret_cast<uint32_t *>(out.ptr + doff) = so < 0 ? 0 : *reinterpret_cast<const uint32_t *>(in.ptr + so);
        break;
    default:
        *reinterpret_cast<uint64_t *>(out.ptr + doff) = so < 0 ? 0 : *reinterpret_cast<const uint64_t *>(in.ptr + so);
        break;
    }
}

__global__ void moveGeneric(TView in, TView out, TView padding, MoveAttr a) {
    // concat iterates the input's elements, everything else the output's (concat.comp:20-22)
    const TView &iter = a.kind == MOVE_CONCAT ? in : out;
    const int64_t total = numelOf(iter);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, src[kMaxRank] = {0, 0, 0, 0, 0, 0},
                 dst[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(iter, uint32_t(e), idx);
        bool isPad = false;
        switch (a.kind) {
        case MOVE_TRANSPOSE:
            for (int i = 0; i < out.rank; ++i) {
                src[a.v[i]] = idx[i];
                dst[i] = idx[i];
            }
            break;
        case MOVE_CONCAT:
            for (int i = 0; i < in.rank; ++i) {
                src[i] = idx[i];
                dst[i] = idx[i];
            }
            dst[a.v[0]] += a.v[1];
            break;
        case MOVE_RESHAPE: {
            uint32_t off = uint32_t(e);
            for (int i = in.rank - 1; i >= 0; --i) {
                src[i] = off % in.dims[i];
                off /= in.dims[i];
            }
            if (off > 0) {
                continue; // common.comp:82-84
            }
            for (int i = 0; i < out.rank; ++i) {
                dst[i] = idx[i];
            }
            break;
        }
        case MOVE_SLICE:
            for (int i = 0; i < out.rank; ++i) {
                src[i] = idx[i] + a.v[i];
                dst[i] = idx[i];
            }
            break;
        case MOVE_PAD:
            for (int i = 0; i < out.rank; ++i) {
                dst[i] = idx[i];
            }
            for (int i = 0; i < out.rank; ++i) {
                const uint32_t cp[1] = {uint32_t(2 * i)};
                const int32_t p = int32_t(loadInt(padding, cp));
                src[i] = idx[i] - uint32_t(p);
                if (src[i] >= in.dims[i]) {
                    isPad = true;
                    break;
                }
            }
            break;
        default:
            for (int i = 0; i < out.rank; ++i) {
                src[i] = idx[i];
                dst[i] = idx[i];
            }
            break;
        }
        const int64_t doff = offsetOf(out, dst);
        if (doff < 0) {
            continue;
        }
        if (isPad) {
            switch (dtypeSize(out.dtype)) {
            case 1:
                *reinterpret_cast<uint8_t *>(out.ptr + doff) = uint8_t(a.padBits);
                break;
            case 2:
                *reinterpret_cast<uint16_t *>(out.ptr + doff) = uint16_t(a.padBits);
                break;
            case 4:
                *reinterpret_cast<uint32_t *>(out.ptr + doff) = uint32_t(a.padBits);
                break;
            default:
                *reinterpret_cast<uint64_t *>(out.ptr + doff) = uint64_t(a.padBits);
                break;
            }
            continue;
        }
        copyElem(in, offsetOf(in, src), out, doff);
    }
}

// ---- CLAMP: clamp.comp:24-53 (integer path) --------------------------------------------------------
__global__ void clampGeneric(TView in, TView out, int64_t lo, int64_t hi) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const int64_t v = loadInt(in, idx);
        const int64_t m = v > lo ? v : lo; // clamp(x, lo, hi) = min(max(x, lo), hi)
        storeInt(out, idx, m < hi ? m : hi);
    }
}

// ---- elementwise binary: elementwise_binary.comp:146-173 -------------------------------------------
__device__ inline float loadF32(const TView &t, const uint32_t *c) {
    const int64_t off = offsetOf(t, c);
    return off < 0 ? 0.0f : *reinterpret_cast<const float *>(t.ptr + off);
}

__global__ void binaryGeneric(TView a, TView b, TView out, int32_t op) {
    const int64_t total = numelOf(out);
    const int32_t dt = a.dtype;
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, ca[kMaxRank], cb[kMaxRank];
        unravel(out, uint32_t(e), idx);
        broadcastIndex(a, idx, ca);
        broadcastIndex(b, idx, cb);
        if (dt == MLEL_F32) {
            const float x = loadF32(a, ca), y = loadF32(b, cb);
            float r = 0.0f;
            int64_t ri = 0;
            bool isBool = false;
            switch (op) {
            case BIN_ADD:
                r = __fadd_rn(x, y);
                break;
            case BIN_SUB:
                r = __fsub_rn(x, y);
                break;
            case BIN_MAXIMUM:
                r = isnan(x) ? x : (isnan(y) ? y : fmaxf(x, y));
                break;
            case BIN_MINIMUM:
                r = isnan(x) ? x : (isnan(y) ? y : fminf(x, y));
                break;
            case BIN_EQUAL:
                ri = x == y, isBool = true;
                break;
            case BIN_GREATER:
                ri = x > y, isBool = true;
                break;
            case BIN_GREATER_EQUAL:
                ri = x >= y, isBool = true;
                break;
            case BIN_POW:
                // elementwise_binary.comp:71-89: a negative base takes an integral exponent only
                if (x >= 0.0f) {
                    r = powf(x, y);
                } else if (fmodf(y, 2.0f) == 0.0f) {
                    r = powf(-x, y);
                } else if (fmodf(y, 1.0f) == 0.0f) {
                    r = -powf(-x, y);
                } else {
                    r = nanf("");
                }
                break;
            default:
                break;
            }
            const int64_t off = offsetOf(out, idx);
            if (off >= 0) {
                if (isBool) {
                    storeIntAt(out, off, ri);
                } else {
                    *reinterpret_cast<float *>(out.ptr + off) = r;
                }
            }
            continue;
        }
        const int64_t x = loadInt(a, ca), y = loadInt(b, cb);
        int64_t r = 0;
        switch (op) {
        case BIN_ADD:
            r = wrapTo(dt, int64_t(uint64_t(x) + uint64_t(y)));
            break;
        case BIN_SUB:
            r = wrapTo(dt, int64_t(uint64_t(x) - uint64_t(y)));
            break;
        case BIN_BITWISE_AND:
            r = x & y;
            break;
        case BIN_BITWISE_OR:
            r = x | y;
            break;
        case BIN_BITWISE_XOR:
            r = x ^ y;
            break;
        case BIN_LOGICAL_AND:
            r = (x != 0) && (y != 0);
            break;
        case BIN_LOGICAL_OR:
            r = (x != 0) || (y != 0);
            break;
        case BIN_LOGICAL_XOR:
            r = (x != 0) != (y != 0);
            break;
        case BIN_LOGICAL_LEFT_SHIFT:
            r = int64_t(uint32_t(uint32_t(x) << (uint32_t(y) & 31u)));
            break;
        case BIN_LOGICAL_RIGHT_SHIFT: {
            const int bits = dtypeSize(dt) * 8;
            const uint32_t z = bits == 8 ? uint32_t(uint8_t(x)) : (bits == 16 ? uint32_t(uint16_t(x)) : uint32_t(x));
            r = int64_t(z >> (uint32_t(y) & 31u));
            break;
        }
        case BIN_INTDIV:
            if (y == 0) {
                r = 0;
            } else if (x == typeLowest(dt) && y == -1) {
                r = x;
            } else {
                r = x / y;
            }
            break;
        case BIN_MAXIMUM:
            r = x > y ? x : y;
            break;
        case BIN_MINIMUM:
            r = x < y ? x : y;
            break;
        case BIN_EQUAL:
            r = x == y;
            break;
        case BIN_GREATER:
            r = x > y;
            break;
        case BIN_GREATER_EQUAL:
            r = x >= y;
            break;
        default:
            break;
        }
        storeInt(out, idx, r);
    }
}

// ---- MUL: mul.comp:24-59 ---------------------------------------------------------------------------
__global__ void mulGeneric(TView a, TView b, TView out, uint32_t shift) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, ca[kMaxRank], cb[kMaxRank];
        unravel(out, uint32_t(e), idx);
        broadcastIndex(a, idx, ca);
        broadcastIndex(b, idx, cb);
        if (a.dtype == MLEL_F32) {
            const int64_t off = offsetOf(out, idx);
            if (off >= 0) {
                *reinterpret_cast<float *>(out.ptr + off) = __fmul_rn(loadF32(a, ca), loadF32(b, cb));
            }
            continue;
        }
        int64_t r = int64_t(uint64_t(loadInt(a, ca)) * uint64_t(loadInt(b, cb)));
        if (shift > 0) {
            r = int64_t(uint64_t(r) + (1ull << ((shift - 1) & 63))) >> (shift & 63);
        }
        storeInt(out, idx, r);
    }
}

// ---- REDUCE_*: reduce.comp:24-70 (integer path) ----------------------------------------------------
__global__ void reduceGeneric(TView in, TView out, uint32_t axis, int32_t op) {
    const int64_t total = numelOf(out);
    const int32_t dt = in.dtype;
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t dim = idx[axis];
        int64_t r = 0;
        if (op == RED_MAX) {
            r = typeLowest(dt);
        } else if (op == RED_MIN) {
            r = typeMax(dt);
        } else if (op == RED_PRODUCT || op == RED_ALL) {
            r = 1;
        }
        for (uint32_t i = 0; i < in.dims[axis]; ++i) {
            idx[axis] = i;
            const int64_t v = loadInt(in, idx);
            switch (op) {
            case RED_SUM:
                r = wrapTo(dt, int64_t(uint64_t(r) + uint64_t(v)));
                break;
            case RED_MAX:
                r = v > r ? v : r;
                break;
            case RED_MIN:
                r = v < r ? v : r;
                break;
            case RED_PRODUCT:
                r = wrapTo(dt, int64_t(uint64_t(r) * uint64_t(v)));
                break;
            case RED_ALL:
                r = (r != 0) && (v != 0);
                break;
            default:
                r = (r != 0) || (v != 0);
                break;
            }
        }
        idx[axis] = dim;
        storeInt(out, idx, r);
    }
}

// ---- CAST: cast.comp:24-103 ------------------------------------------------------------------------
__global__ void castGeneric(TView in, TView out) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const int64_t off = offsetOf(out, idx);
        if (off < 0) {
            continue;
        }
        if (in.dtype == MLEL_F32 && out.dtype == MLEL_F32) {
            *reinterpret_cast<float *>(out.ptr + off) = loadF32(in, idx);
        } else if (in.dtype == MLEL_F32) {
            const float f = loadF32(in, idx);
            if (out.dtype == MLEL_BOOL) {
                storeIntAt(out, off, f != 0.0f);
                continue;
            }
            const int64_t lo = typeLowest(out.dtype), hi = typeMax(out.dtype);
            int64_t r;
            if (f <= float(lo)) {
                r = lo;
            } else if (f >= float(hi)) {
                r = hi;
            } else {
                r = int64_t(rintf(f));
            }
            storeIntAt(out, off, r);
        } else if (out.dtype == MLEL_F32) {
            *reinterpret_cast<float *>(out.ptr + off) = float(loadInt(in, idx));
        } else {
            const int64_t v = loadInt(in, idx);
            storeIntAt(out, off, out.dtype == MLEL_BOOL ? int64_t(v != 0) : v);
        }
    }
}

// ---- ARITHMETIC_RIGHT_SHIFT: arithmetic_right_shift.comp:22-49 -------------------------------------
__global__ void arShiftGeneric(TView a, TView b, TView out, int32_t round) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, ca[kMaxRank], cb[kMaxRank];
        unravel(out, uint32_t(e), idx);
        broadcastIndex(a, idx, ca);
        broadcastIndex(b, idx, cb);
        const int64_t x = loadInt(a, ca), y = loadInt(b, cb);
        int64_t r = x >> (y & 63);
        if (round && y > 0 && ((x >> ((y - 1) & 63)) & 1) != 0) {
            r = wrapTo(a.dtype, r + 1);
        }
        storeInt(out, idx, r);
    }
}

// ---- NEGATE: negate.comp:32-48 (integer path) ------------------------------------------------------
__global__ void negateGeneric(TView in, TView out, int32_t inZp, int32_t outZp) {
    const int64_t total = numelOf(out);
    int64_t lo = typeLowest(out.dtype), hi = typeMax(out.dtype);
    lo = lo < -2147483648ll ? -2147483648ll : lo;
    hi = hi > 2147483647ll ? 2147483647ll : hi;
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const int32_t v = int32_t(loadInt(in, idx));
        const int32_t res = int32_t(uint32_t(inZp) - uint32_t(v) + uint32_t(outZp));
        storeInt(out, idx, res < lo ? lo : (res > hi ? hi : int64_t(res)));
    }
}

// ---- SELECT: select.comp:18-42 ---------------------------------------------------------------------
__global__ void selectGeneric(TView cond, TView a, TView b, TView out) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, c[kMaxRank];
        unravel(out, uint32_t(e), idx);
        broadcastIndex(cond, idx, c);
        const bool pick = (loadInt(cond, c) & 0xff) != 0;
        const TView &src = pick ? a : b;
        broadcastIndex(src, idx, c);
        const int64_t doff = offsetOf(out, idx);
        if (doff >= 0) {
            copyElem(src, offsetOf(src, c), out, doff);
        }
    }
}

// ---- integer unary: elementwise_unary.comp ("abs(value1)", "~value1", "clz(value1)", "!value1") ----
__global__ void unaryGeneric(TView in, TView out, int32_t op) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const int64_t v = loadInt(in, idx);
        int64_t r = 0;
        switch (op) {
        case UN_ABS:
            r = wrapTo(in.dtype, v < 0 ? int64_t(0 - uint64_t(v)) : v);
            break;
        case UN_BITWISE_NOT:
            r = ~v;
            break;
        case UN_CLZ:
            r = __clz(int32_t(v));
            break;
        default:
            r = v == 0;
            break;
        }
        storeInt(out, idx, r);
    }
}

// ---- fp32 unary: elementwise_unary.comp:204-223 with the expressions of graph/compute_graph_op.cpp:2527-2945.
// A NaN input passes through unchanged; LOG of a negative number is NaN (log_guarded, :161-163); TANH is +-1
// beyond |x| = 10 and a four-term series below 0.2 (tanh_clamped, :139-159); SIN uses the odd series through
// x^11 below 1e-3 (sin_hybrid, :166-192).  The transcendental functions themselves are CUDA's single-precision
// ones (at most 2 ulp from the exact result, where the reference inherits its Vulkan device's precision).
__device__ inline float unaryF32(int32_t op, float x) {
    if (isnan(x)) {
        return x;
    }
    switch (op) {
    case UN_ABS:
        return fabsf(x);
    case UN_CEIL:
        return ceilf(x);
    case UN_FLOOR:
        return floorf(x);
    case UN_COS:
        return cosf(x);
    case UN_ERF:
        return erff(x);
    case UN_EXP:
        return expf(x);
    case UN_LOG:
        return x < 0.0f ? nanf("") : logf(x);
    case UN_RECIPROCAL:
        return __fdiv_rn(1.0f, x);
    case UN_RSQRT:
        return rsqrtf(x);
    case UN_SIGMOID:
        return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
    case UN_SIN: {
        if (fabsf(x) < 1.0e-3f) {
            const float x2 = __fmul_rn(x, x);
            float p = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(-1.0f / 39916800.0f, x2), 1.0f / 362880.0f), x2),
                                -1.0f / 5040.0f);
            p = __fadd_rn(__fmul_rn(p, x2), 1.0f / 120.0f);
            p = __fadd_rn(__fmul_rn(p, x2), -1.0f / 6.0f);
            p = __fadd_rn(__fmul_rn(p, x2), 1.0f);
            return __fmul_rn(x, p);
        }
        return sinf(x);
    }
    case UN_TANH: {
        if (x > 10.0f) {
            return 1.0f;
        }
        if (x < -10.0f) {
            return -1.0f;
        }
        if (fabsf(x) < 0.2f) {
            const float x2 = __fmul_rn(x, x);
            const float t = __fsub_rn(2.0f / 15.0f, __fmul_rn(17.0f / 315.0f, x2));
            const float u = __fsub_rn(1.0f / 3.0f, __fmul_rn(x2, t));
            return __fmul_rn(x, __fsub_rn(1.0f, __fmul_rn(x2, u)));
        }
        return tanhf(x);
    }
    default:
        return x;
    }
}

__global__ void unaryF32Generic(TView in, TView out, int32_t op) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const int64_t off = offsetOf(out, idx);
        if (off >= 0) {
            *reinterpret_cast<float *>(out.ptr + off) = unaryF32(op, loadF32(in, idx));
        }
    }
}

// Packed tensors: four elements per thread.
__global__ void unaryF32Packed(const float4 *__restrict__ in, float4 *__restrict__ out, int64_t quads, int32_t op) {
    GRID_STRIDE(e, quads) {
        float4 v = in[e];
        v.x = unaryF32(op, v.x);
        v.y = unaryF32(op, v.y);
        v.z = unaryF32(op, v.z);
        v.w = unaryF32(op, v.w);
        out[e] = v;
    }
}

int finish(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        setLastError(std::string(what) + ": " + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

} // namespace

#define LAUNCH_1D(kernel, total, stream, ...) kernel<<<gridFor(total), kThreads, 0, stream>>>(__VA_ARGS__)

int genericConv2d(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                  cudaStream_t s) {
    const int64_t total = numelOf(out);
    if (out.dtype == MLEL_I32) {
        LAUNCH_1D(conv2dGeneric<int32_t>, total, s, in, w, bias, out, a);
    } else if (out.dtype == MLEL_I64) {
        LAUNCH_1D(conv2dGeneric<int64_t>, total, s, in, w, bias, out, a);
    } else {
        setLastError("CONV2D: unsupported output type");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    return finish("CONV2D");
}

int genericDepthwise(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                     cudaStream_t s) {
    const int64_t total = numelOf(out);
    if (out.dtype == MLEL_I32) {
        LAUNCH_1D(depthwiseGeneric<int32_t>, total, s, in, w, bias, out, a);
    } else if (out.dtype == MLEL_I64) {
        LAUNCH_1D(depthwiseGeneric<int64_t>, total, s, in, w, bias, out, a);
    } else {
        setLastError("DEPTHWISE_CONV2D: unsupported output type");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    return finish("DEPTHWISE_CONV2D");
}

int genericMatmul(const TView &a, const TView &b, const TView &out, int32_t zpA, int32_t zpB, cudaStream_t s) {
    const int64_t total = numelOf(out);
    if (out.dtype == MLEL_I32) {
        LAUNCH_1D(matmulGeneric<int32_t>, total, s, a, b, out, zpA, zpB);
    } else if (out.dtype == MLEL_I64) {
        LAUNCH_1D(matmulGeneric<int64_t>, total, s, a, b, out, zpA, zpB);
    } else {
        setLastError("MATMUL: unsupported output type");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    return finish("MATMUL");
}

int genericRescale(const TView &in, const TView &out, const TView &mult, const TView &shift, const RescaleAttr &a,
                   cudaStream_t s) {
    LAUNCH_1D(rescaleGeneric, numelOf(out), s, in, out, mult, shift, a);
    return finish("RESCALE");
}

int genericAvgPool(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s) {
    LAUNCH_1D(avgPoolGeneric, numelOf(out), s, in, out, a);
    return finish("AVG_POOL2D");
}

int genericMaxPool(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s) {
    LAUNCH_1D(maxPoolGeneric, numelOf(out), s, in, out, a);
    return finish("MAX_POOL2D");
}

int genericTable(const TView &in, const TView &out, const TView &table, cudaStream_t s) {
    LAUNCH_1D(tableGeneric, numelOf(out), s, in, out, table);
    return finish("TABLE");
}

int genericMove(int kind, const TView &in, const TView &out, const TView *padding, const uint32_t *v, int nv,
                int64_t padBits, cudaStream_t s) {
    MoveAttr a{};
    a.kind = kind;
    for (int i = 0; i < nv && i < kMaxRank; ++i) {
        a.v[i] = v[i];
    }
    a.padBits = padBits;
    const int64_t total = kind == MOVE_CONCAT ? numelOf(in) : numelOf(out);
    LAUNCH_1D(moveGeneric, total, s, in, out, padding ? *padding : in, a);
    return finish("data movement");
}

int genericTranspose(const TView &in, const TView &out, const uint32_t *perms, cudaStream_t s) {
    return genericMove(MOVE_TRANSPOSE, in, out, nullptr, perms, out.rank, 0, s);
}
int genericConcat(const TView &in, const TView &out, uint32_t axis, uint32_t offset, cudaStream_t s) {
    const uint32_t v[2] = {axis, offset};
    return genericMove(MOVE_CONCAT, in, out, nullptr, v, 2, 0, s);
}
int genericReshape(const TView &in, const TView &out, cudaStream_t s) {
    return genericMove(MOVE_RESHAPE, in, out, nullptr, nullptr, 0, 0, s);
}
int genericSlice(const TView &in, const TView &out, const uint32_t *start, cudaStream_t s) {
    return genericMove(MOVE_SLICE, in, out, nullptr, start, out.rank, 0, s);
}
int genericPad(const TView &in, const TView &out, const TView &padding, int64_t padBits, cudaStream_t s) {
    return genericMove(MOVE_PAD, in, out, &padding, nullptr, 0, padBits, s);
}

int genericClamp(const TView &in, const TView &out, double minV, double maxV, cudaStream_t s) {
    const int64_t lo = wrapTo(out.dtype, int64_t(minV)), hi = wrapTo(out.dtype, int64_t(maxV));
    LAUNCH_1D(clampGeneric, numelOf(out), s, in, out, lo, hi);
    return finish("CLAMP");
}

int genericBinary(int32_t op, const TView &a, const TView &b, const TView &out, cudaStream_t s) {
    LAUNCH_1D(binaryGeneric, numelOf(out), s, a, b, out, op);
    return finish("elementwise binary");
}

int genericMul(const TView &a, const TView &b, const TView &out, uint32_t shift, cudaStream_t s) {
    LAUNCH_1D(mulGeneric, numelOf(out), s, a, b, out, shift);
    return finish("MUL");
}

int genericReduce(int32_t op, const TView &in, const TView &out, uint32_t axis, cudaStream_t s) {
    LAUNCH_1D(reduceGeneric, numelOf(out), s, in, out, axis, op);
    return finish("REDUCE");
}

int genericCast(const TView &in, const TView &out, cudaStream_t s) {
    LAUNCH_1D(castGeneric, numelOf(out), s, in, out);
    return finish("CAST");
}

int genericArShift(const TView &a, const TView &b, const TView &out, int32_t round, cudaStream_t s) {
    LAUNCH_1D(arShiftGeneric, numelOf(out), s, a, b, out, round);
    return finish("ARITHMETIC_RIGHT_SHIFT");
}

int genericNegate(const TView &in, const TView &out, int32_t inZp, int32_t outZp, cudaStream_t s) {
    LAUNCH_1D(negateGeneric, numelOf(out), s, in, out, inZp, outZp);
    return finish("NEGATE");
}

int genericSelect(const TView &c, const TView &a, const TView &b, const TView &out, cudaStream_t s) {
    LAUNCH_1D(selectGeneric, numelOf(out), s, c, a, b, out);
    return finish("SELECT");
}

int genericUnary(int32_t op, const TView &in, const TView &out, cudaStream_t s) {
    if (in.dtype == MLEL_F32) {
        const auto packed = [](const TView &t) {
            int64_t st = 4;
            for (int i = t.rank - 1; i >= 0; --i) {
                if (t.strides[i] != st) {
                    return false;
                }
                st *= t.dims[i];
            }
            return true;
        };
        const int64_t n = numelOf(out);
        const bool same = in.rank == out.rank && numelOf(in) == n;
        if (same && n % 4 == 0 && packed(in) && packed(out) && ((uintptr_t(in.ptr) | uintptr_t(out.ptr)) & 15u) == 0) {
            unaryF32Packed<<<gridFor(n / 4), kThreads, 0, s>>>(reinterpret_cast<const float4 *>(in.ptr),
                                                               reinterpret_cast<float4 *>(out.ptr), n / 4, op);
        } else {
            LAUNCH_1D(unaryF32Generic, n, s, in, out, op);
        }
        return finish("elementwise unary");
    }
    LAUNCH_1D(unaryGeneric, numelOf(out), s, in, out, op);
    return finish("elementwise unary");
}

} // namespace mlel
