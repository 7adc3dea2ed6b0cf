// CPU oracle for the TOSA data-graph operators of the ML Emulation Layer for Vulkan.
//
// TEST INFRASTRUCTURE ONLY.  This file is a CPU restatement of the arithmetic of the
// reference's GLSL compute shaders; it exists so that the CUDA kernels can be checked
// bit-for-bit.  Nothing in the shipped library links, loads or calls it.
//
// Every function follows one shader of the reference (path inside the reference project):
//   graph/shaders/graph_op/common.comp            index unravel (:74-128), broadcast (:64-72)
//   graph/shaders/graph_op/tosa/<op>.comp         per-operator arithmetic (cited per function)
//   tensor/shaders/tensor.glsl:24-86              tensorReadARM / tensorWriteARM semantics:
//                                                 coordinates are unsigned, any coordinate
//                                                 >= shape reads as 0, out-of-range writes drop
//   tensor/tensor_arm.cpp:82-92                   packed row-major byte strides
// GLSL semantics kept: 32/64-bit integer arithmetic wraps, >> on signed is arithmetic,
// integer division truncates toward zero, narrowing constructors wrap.
//
// Parity pins: the golden vectors of the reference's own tests (tests/vulkan.cpp) for CONV2D,
// int64-accumulate CONV2D, CONV3D, RESCALE+ADD, MAX_POOL2D, CONCAT, SLICE, MAXIMUM are replayed
// against this file by tests/test_oracle_golden.py.  MATMUL, DEPTHWISE_CONV2D, AVG_POOL2D, TABLE,
// TRANSPOSE, CLAMP, MUL, REDUCE_*, per-channel and double-round RESCALE, ARGMAX, GATHER, SCATTER,
// REVERSE, TILE, RESIZE and TRANSPOSE_CONV2D have no golden in the reference: for those this file
// is "parity unpinned" and is cross-checked against an independent numpy restatement
// (oracle/np_ref.py).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <type_traits>

extern "C" {
enum orc_dtype {
    ORC_BOOL = 0,
    ORC_I8 = 1,
    ORC_I16 = 2,
    ORC_I32 = 3,
    ORC_I64 = 4,
    ORC_U8 = 5,
    ORC_U16 = 6,
    ORC_U32 = 7,
    ORC_F16 = 8,
    ORC_BF16 = 9,
    ORC_F32 = 10,
};

struct orc_tensor {
    void *data;
    int32_t dtype;
    int32_t rank;
    int64_t dims[6];
    int64_t strides[6]; // bytes
};
}

namespace {

constexpr int kMaxRank = 6;

int elemSize(int dtype) {
    switch (dtype) {
    case ORC_BOOL:
    case ORC_I8:
    case ORC_U8:
        return 1;
    case ORC_I16:
    case ORC_U16:
    case ORC_F16:
    case ORC_BF16:
        return 2;
    case ORC_I32:
    case ORC_U32:
    case ORC_F32:
        return 4;
    case ORC_I64:
        return 8;
    default:
        return 0;
    }
}

int64_t numel(const orc_tensor &t) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; ++i) {
        n *= t.dims[i];
    }
    return n;
}

// common.comp:74-85 offsetToIndex: last dimension fastest.
void unravel(const orc_tensor &t, uint32_t off, uint32_t *idx) {
    for (int i = t.rank - 1; i >= 0; --i) {
        idx[i] = off % uint32_t(t.dims[i]);
        off /= uint32_t(t.dims[i]);
    }
}

// tensor.glsl:26-50. `lane` is the element of an array read (advances the last coordinate).
template <typename T> T rd(const orc_tensor &t, const uint32_t *c, uint32_t lane = 0) {
    int64_t off = 0;
    for (int i = 0; i < t.rank; ++i) {
        if (int64_t(c[i]) >= t.dims[i]) {
            return T(0);
        }
        off += int64_t(c[i]) * t.strides[i];
    }
    if (int64_t(uint32_t(c[t.rank - 1] + lane)) >= t.dims[t.rank - 1]) {
        return T(0);
    }
    T v;
    std::memcpy(&v, static_cast<const char *>(t.data) + off + int64_t(lane) * int64_t(sizeof(T)), sizeof(T));
    return v;
}

// tensor.glsl:58-81
template <typename T> void wr(const orc_tensor &t, const uint32_t *c, T v) {
    int64_t off = 0;
    for (int i = 0; i < t.rank; ++i) {
        if (int64_t(c[i]) >= t.dims[i]) {
            return;
        }
        off += int64_t(c[i]) * t.strides[i];
    }
    std::memcpy(static_cast<char *>(t.data) + off, &v, sizeof(T));
}

// Reads an integer element of any integer dtype sign/zero-extended into int64.
int64_t rdInt(const orc_tensor &t, const uint32_t *c, uint32_t lane = 0) {
    switch (t.dtype) {
    case ORC_BOOL:
    case ORC_I8:
        return rd<int8_t>(t, c, lane);
    case ORC_U8:
        return rd<uint8_t>(t, c, lane);
    case ORC_I16:
        return rd<int16_t>(t, c, lane);
    case ORC_U16:
        return rd<uint16_t>(t, c, lane);
    case ORC_I32:
        return rd<int32_t>(t, c, lane);
    case ORC_U32:
        return rd<uint32_t>(t, c, lane);
    default:
        return rd<int64_t>(t, c, lane);
    }
}

// Writes with a narrowing (wrapping) constructor of the tensor's own type.
void wrInt(const orc_tensor &t, const uint32_t *c, int64_t v) {
    switch (t.dtype) {
    case ORC_BOOL:
    case ORC_I8:
    case ORC_U8:
        wr<int8_t>(t, c, int8_t(uint8_t(uint64_t(v))));
        break;
    case ORC_I16:
    case ORC_U16:
        wr<int16_t>(t, c, int16_t(uint16_t(uint64_t(v))));
        break;
    case ORC_I32:
    case ORC_U32:
        wr<int32_t>(t, c, int32_t(uint32_t(uint64_t(v))));
        break;
    default:
        wr<int64_t>(t, c, v);
        break;
    }
}

// Wraps a 64-bit value to the width of an integer dtype (result sign- or zero-extended).
int64_t wrapTo(int dtype, int64_t v) {
    switch (dtype) {
    case ORC_BOOL:
        return v != 0 ? 1 : 0;
    case ORC_I8:
        return int8_t(uint8_t(uint64_t(v)));
    case ORC_U8:
        return uint8_t(uint64_t(v));
    case ORC_I16:
        return int16_t(uint16_t(uint64_t(v)));
    case ORC_U16:
        return uint16_t(uint64_t(v));
    case ORC_I32:
        return int32_t(uint32_t(uint64_t(v)));
    case ORC_U32:
        return uint32_t(uint64_t(v));
    default:
        return v;
    }
}

int64_t typeLowest(int dtype) {
    switch (dtype) {
    case ORC_I8:
        return -128;
    case ORC_I16:
        return -32768;
    case ORC_I32:
        return std::numeric_limits<int32_t>::min();
    case ORC_I64:
        return std::numeric_limits<int64_t>::min();
    default:
        return 0;
    }
}

int64_t typeMax(int dtype) {
    switch (dtype) {
    case ORC_BOOL:
        return 1;
    case ORC_I8:
        return 127;
    case ORC_U8:
        return 255;
    case ORC_I16:
        return 32767;
    case ORC_U16:
        return 65535;
    case ORC_I32:
        return std::numeric_limits<int32_t>::max();
    case ORC_U32:
        return 4294967295ll;
    default:
        return std::numeric_limits<int64_t>::max();
    }
}

// Wrapping accumulate helpers: ACC is int32_t or int64_t.
template <typename ACC> struct Wrap {
    using U = std::make_unsigned_t<ACC>;
    static ACC add(ACC a, ACC b) { return ACC(U(a) + U(b)); }
    static ACC sub(ACC a, ACC b) { return ACC(U(a) - U(b)); }
    static ACC mul(ACC a, ACC b) { return ACC(U(a) * U(b)); }
};

// conv2d.comp:26-116.  ACC = accumulator type (int32 for int8 inputs, int64 for int16 inputs).
// Output/bias are of the accumulator's storage type (OUT_T); acc_to_out is a plain constructor.
template <typename ACC>
void conv2dImpl(const orc_tensor &in, const orc_tensor &w, const orc_tensor &bias, const orc_tensor &out,
                const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    const uint32_t N = uint32_t(out.dims[0]), OH = uint32_t(out.dims[1]), OW = uint32_t(out.dims[2]),
                   OC = uint32_t(out.dims[3]);
    const uint32_t KH = uint32_t(w.dims[1]), KW = uint32_t(w.dims[2]);
    const uint32_t H = uint32_t(in.dims[1]), W = uint32_t(in.dims[2]), IC = uint32_t(in.dims[3]);
    const int64_t total = int64_t(N) * OH * OW;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < total; ++p) {
        const uint32_t n = uint32_t(p / (int64_t(OH) * OW));
        const uint32_t oy = uint32_t((p / OW) % OH);
        const uint32_t ox = uint32_t(p % OW);
        const uint32_t iy = oy * uint32_t(stride[0]) - uint32_t(pad[0]);
        const uint32_t ix = ox * uint32_t(stride[1]) - uint32_t(pad[2]);
        for (uint32_t oc = 0; oc < OC; ++oc) {
            ACC acc = 0;
            for (uint32_t ky = 0; ky < KH; ++ky) {
                for (uint32_t kx = 0; kx < KW; ++kx) {
                    const uint32_t y = iy + ky * uint32_t(dil[0]);
                    const uint32_t x = ix + kx * uint32_t(dil[1]);
                    if (y < H && x < W) {
                        for (uint32_t ic = 0; ic < IC; ++ic) {
                            const uint32_t ci[4] = {n, y, x, ic};
                            const uint32_t cw[4] = {oc, ky, kx, ic};
                            const ACC v = Wrap<ACC>::sub(ACC(rdInt(in, ci)), ACC(inZp));
                            const ACC wt = Wrap<ACC>::sub(ACC(rdInt(w, cw)), ACC(wZp));
                            acc = Wrap<ACC>::add(acc, Wrap<ACC>::mul(v, wt));
                        }
                    }
                }
            }
            // conv2d.comp:98-112: one-element bias broadcasts, otherwise read at oc (0 when out of range)
            const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
            acc = Wrap<ACC>::add(acc, ACC(rdInt(bias, cb)));
            const uint32_t co[4] = {n, oy, ox, oc};
            wrInt(out, co, int64_t(acc));
        }
    }
}

// Fast path for packed int8 NHWC x OHWI -> int32: same arithmetic, pointer walking.
bool isPacked(const orc_tensor &t) {
    int64_t s = elemSize(t.dtype);
    for (int i = t.rank - 1; i >= 0; --i) {
        if (t.strides[i] != s) {
            return false;
        }
        s *= t.dims[i];
    }
    return true;
}

void conv2dI8Packed(const orc_tensor &in, const orc_tensor &w, const orc_tensor &bias, const orc_tensor &out,
                    const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    const uint32_t N = uint32_t(out.dims[0]), OH = uint32_t(out.dims[1]), OW = uint32_t(out.dims[2]),
                   OC = uint32_t(out.dims[3]);
    const uint32_t KH = uint32_t(w.dims[1]), KW = uint32_t(w.dims[2]);
    const uint32_t H = uint32_t(in.dims[1]), W = uint32_t(in.dims[2]), IC = uint32_t(in.dims[3]);
    const int8_t *inp = static_cast<const int8_t *>(in.data);
    const int8_t *wp = static_cast<const int8_t *>(w.data);
    const int32_t *bp = static_cast<const int32_t *>(bias.data);
    int32_t *op = static_cast<int32_t *>(out.data);
    const int64_t total = int64_t(N) * OH * OW;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < total; ++p) {
        const uint32_t n = uint32_t(p / (int64_t(OH) * OW));
        const uint32_t oy = uint32_t((p / OW) % OH);
        const uint32_t ox = uint32_t(p % OW);
        const uint32_t iy = oy * uint32_t(stride[0]) - uint32_t(pad[0]);
        const uint32_t ix = ox * uint32_t(stride[1]) - uint32_t(pad[2]);
        for (uint32_t oc = 0; oc < OC; ++oc) {
            uint32_t acc = 0;
            for (uint32_t ky = 0; ky < KH; ++ky) {
                for (uint32_t kx = 0; kx < KW; ++kx) {
                    const uint32_t y = iy + ky * uint32_t(dil[0]);
                    const uint32_t x = ix + kx * uint32_t(dil[1]);
                    if (y < H && x < W) {
                        const int8_t *ip = inp + ((int64_t(n) * H + y) * W + x) * IC;
                        const int8_t *wq = wp + ((int64_t(oc) * KH + ky) * KW + kx) * IC;
                        int32_t s = 0; // |sum| < 2^31 for IC < 2^15: no wrap inside one tap
                        if (IC < 32768) {
                            for (uint32_t ic = 0; ic < IC; ++ic) {
                                s += (int32_t(ip[ic]) - inZp) * (int32_t(wq[ic]) - wZp);
                            }
                            acc += uint32_t(s);
                        } else {
                            for (uint32_t ic = 0; ic < IC; ++ic) {
                                acc += uint32_t((int32_t(ip[ic]) - inZp) * (int32_t(wq[ic]) - wZp));
                            }
                        }
                    }
                }
            }
            acc += uint32_t(bias.dims[0] == 1 ? bp[0] : bp[oc]);
            op[p * OC + oc] = int32_t(acc);
        }
    }
}

// depthwise_conv2d.comp:31-78
template <typename ACC>
void depthwiseImpl(const orc_tensor &in, const orc_tensor &w, const orc_tensor &bias, const orc_tensor &out,
                   const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    const int64_t total = numel(out);
    const uint32_t KH = uint32_t(w.dims[0]), KW = uint32_t(w.dims[1]), M = uint32_t(w.dims[3]);
    const uint32_t H = uint32_t(in.dims[1]), W = uint32_t(in.dims[2]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], ocm = idx[3];
        const uint32_t c = ocm / M, m = ocm % M;
        const uint32_t iy = oy * uint32_t(stride[0]) - uint32_t(pad[0]);
        const uint32_t ix = ox * uint32_t(stride[1]) - uint32_t(pad[2]);
        ACC acc = 0;
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                const uint32_t y = iy + ky * uint32_t(dil[0]);
                const uint32_t x = ix + kx * uint32_t(dil[1]);
                if (y < H && x < W) {
                    const uint32_t ci[4] = {n, y, x, c};
                    const uint32_t cw[4] = {ky, kx, c, m};
                    const ACC v = Wrap<ACC>::sub(ACC(rdInt(in, ci)), ACC(inZp));
                    const ACC wt = Wrap<ACC>::sub(ACC(rdInt(w, cw)), ACC(wZp));
                    acc = Wrap<ACC>::add(acc, Wrap<ACC>::mul(v, wt));
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : ocm};
        acc = Wrap<ACC>::add(ACC(rdInt(bias, cb)), acc);
        wrInt(out, idx, int64_t(acc));
    }
}

// matmul.comp:30-73; COMP_T is the output type for integer inputs.
template <typename ACC>
void matmulImpl(const orc_tensor &a, const orc_tensor &b, const orc_tensor &out, int32_t zpA, int32_t zpB) {
    const int64_t total = numel(out);
    const uint32_t K = uint32_t(a.dims[2]);
    const bool fast = a.dtype == ORC_I8 && b.dtype == ORC_I8 && isPacked(a) && isPacked(b) && K < 32768;
    const int64_t Wd = b.dims[2];
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        ACC acc = 0;
        if (fast) {
            const int8_t *ap = static_cast<const int8_t *>(a.data) + (int64_t(idx[0]) * a.dims[1] + idx[1]) * K;
            const int8_t *bp = static_cast<const int8_t *>(b.data) + int64_t(idx[0]) * K * Wd + idx[2];
            int32_t s = 0;
            for (uint32_t c = 0; c < K; ++c) {
                s += (int32_t(ap[c]) - zpA) * (int32_t(bp[int64_t(c) * Wd]) - zpB);
            }
            acc = ACC(s);
        } else {
            for (uint32_t c = 0; c < K; ++c) {
                const uint32_t ca[3] = {idx[0], idx[1], c};
                const uint32_t cb[3] = {idx[0], c, idx[2]};
                const ACC v1 = Wrap<ACC>::sub(ACC(rdInt(a, ca)), ACC(zpA));
                const ACC v2 = Wrap<ACC>::sub(ACC(rdInt(b, cb)), ACC(zpB));
                acc = Wrap<ACC>::add(acc, Wrap<ACC>::mul(v1, v2));
            }
        }
        wrInt(out, idx, int64_t(acc));
    }
}

// rescale.comp:27-46 applyScale.  shift == 0 gives a rounding term of 0 (the shader's
// 1 << (shift - 1) is undefined there; the reference's GraphConstantARM golden implies 0).
int32_t applyScale(int64_t value, int32_t multiplier, int8_t shift, bool doubleRound) {
    int64_t round = shift > 0 ? int64_t(uint64_t(1) << ((shift - 1) & 63)) : 0;
    if (doubleRound && shift > 31) {
        round += value >= 0 ? (int64_t(1) << 30) : -(int64_t(1) << 30);
    }
    int64_t result = int64_t(uint64_t(value) * uint64_t(int64_t(multiplier)));
    result = int64_t(uint64_t(result) + uint64_t(round));
    result >>= (shift & 63);
    return int32_t(uint32_t(uint64_t(result)));
}

} // namespace

extern "C" {

int orc_elem_size(int dtype) { return elemSize(dtype); }

// graph/shaders/graph_op/tosa/conv2d.comp
int orc_conv2d(const orc_tensor *in, const orc_tensor *w, const orc_tensor *bias, const orc_tensor *out,
               const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    if (out->dtype == ORC_I32) {
        if (in->dtype == ORC_I8 && w->dtype == ORC_I8 && bias->dtype == ORC_I32 && isPacked(*in) && isPacked(*w) &&
            isPacked(*out) && isPacked(*bias)) {
            conv2dI8Packed(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
        } else {
            conv2dImpl<int32_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
        }
    } else if (out->dtype == ORC_I64) {
        conv2dImpl<int64_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else {
        return -1;
    }
    return 0;
}

// Forces the element-by-element restatement (used to validate the packed fast path).
int orc_conv2d_generic(const orc_tensor *in, const orc_tensor *w, const orc_tensor *bias, const orc_tensor *out,
                       const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    if (out->dtype == ORC_I32) {
        conv2dImpl<int32_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else if (out->dtype == ORC_I64) {
        conv2dImpl<int64_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else {
        return -1;
    }
    return 0;
}

// graph/shaders/graph_op/tosa/depthwise_conv2d.comp
int orc_depthwise_conv2d(const orc_tensor *in, const orc_tensor *w, const orc_tensor *bias, const orc_tensor *out,
                         const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    if (out->dtype == ORC_I32) {
        depthwiseImpl<int32_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else if (out->dtype == ORC_I64) {
        depthwiseImpl<int64_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else {
        return -1;
    }
    return 0;
}

// graph/shaders/graph_op/tosa/matmul.comp
int orc_matmul(const orc_tensor *a, const orc_tensor *b, const orc_tensor *out, int32_t zpA, int32_t zpB) {
    if (out->dtype == ORC_I32) {
        matmulImpl<int32_t>(*a, *b, *out, zpA, zpB);
    } else if (out->dtype == ORC_I64) {
        matmulImpl<int64_t>(*a, *b, *out, zpA, zpB);
    } else {
        return -1;
    }
    return 0;
}

// graph/shaders/graph_op/tosa/rescale.comp:48-72
int orc_rescale(const orc_tensor *in, const orc_tensor *out, const orc_tensor *mult, const orc_tensor *shift,
                int32_t inZp, int32_t outZp, int scale32, int doubleRound, int perChannel) {
    const int64_t total = numel(*out);
    const int64_t lo = typeLowest(out->dtype), hi = typeMax(out->dtype);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const uint32_t c[1] = {perChannel ? idx[out->rank - 1] : 0u};
        const int64_t value = rdInt(*in, idx) - wrapTo(in->dtype, inZp);
        const int32_t m = int32_t(rdInt(*mult, c));
        const int8_t s = rd<int8_t>(*shift, c);
        int32_t r = applyScale(value, m, s, scale32 && doubleRound);
        r = int32_t(uint32_t(r) + uint32_t(int32_t(wrapTo(out->dtype, outZp))));
        const int64_t clamped = std::min<int64_t>(std::max<int64_t>(r, lo), hi);
        wrInt(*out, idx, clamped);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/avgpool2d.comp:27-75 (integer path, int32 accumulator)
int orc_avg_pool2d(const orc_tensor *in, const orc_tensor *out, const int32_t *kernel, const int32_t *stride,
                   const int32_t *pad, int32_t inZp, int32_t outZp) {
    const int64_t total = numel(*out);
    const int64_t lo = typeLowest(out->dtype), hi = typeMax(out->dtype);
    const uint32_t H = uint32_t(in->dims[1]), W = uint32_t(in->dims[2]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        uint32_t acc = 0; // int32 accumulator, wrapping
        uint32_t count = 0;
        const uint32_t iy = idx[1] * uint32_t(stride[0]) - uint32_t(pad[0]);
        const uint32_t ix = idx[2] * uint32_t(stride[1]) - uint32_t(pad[2]);
        for (uint32_t ky = 0; ky < uint32_t(kernel[0]); ++ky) {
            for (uint32_t kx = 0; kx < uint32_t(kernel[1]); ++kx) {
                const uint32_t y = iy + ky, x = ix + kx;
                if (y < H && x < W) {
                    const uint32_t ci[4] = {idx[0], y, x, idx[3]};
                    acc += uint32_t(int32_t(rdInt(*in, ci))) - uint32_t(inZp);
                    count++;
                }
            }
        }
        int32_t a = int32_t(acc);
        if (count == 0) {
            a = 0; // division by zero is undefined in the shader; never produced by valid graphs
        } else {
            const int32_t round = a < 0 ? -int32_t(count >> 1) : int32_t(count >> 1);
            a = int32_t(uint32_t(a) + uint32_t(round));
            a = int32_t(int64_t(a) / int64_t(int32_t(count)));
        }
        a = int32_t(uint32_t(a) + uint32_t(outZp));
        const int64_t clamped = std::min<int64_t>(std::max<int64_t>(a, lo), hi);
        wrInt(*out, idx, clamped);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/maxpool2d.comp:23-72 (integer path; initial value = type lowest)
int orc_max_pool2d(const orc_tensor *in, const orc_tensor *out, const int32_t *kernel, const int32_t *stride,
                   const int32_t *pad) {
    const int64_t total = numel(*out);
    const int kY = std::max(kernel[0], 0), kX = std::max(kernel[1], 0);
    const int sY = std::max(stride[0], 1), sX = std::max(stride[1], 1);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        int64_t acc = typeLowest(out->dtype);
        const int iy = int(idx[1]) * sY - pad[0];
        const int ix = int(idx[2]) * sX - pad[2];
        for (int ky = 0; ky < kY; ++ky) {
            for (int kx = 0; kx < kX; ++kx) {
                const int y = iy + ky, x = ix + kx;
                if (y >= 0 && x >= 0 && uint32_t(y) < uint32_t(in->dims[1]) && uint32_t(x) < uint32_t(in->dims[2])) {
                    const uint32_t ci[4] = {idx[0], uint32_t(y), uint32_t(x), idx[3]};
                    acc = std::max(acc, rdInt(*in, ci));
                }
            }
        }
        wrInt(*out, idx, acc);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/table.comp:17-52
int orc_table(const orc_tensor *in, const orc_tensor *out, const orc_tensor *table) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        int32_t result;
        if (in->dtype == ORC_I8) {
            const int8_t v = rd<int8_t>(*in, idx);
            const uint32_t ct[1] = {uint32_t(int32_t(v) + 128)};
            result = rd<int8_t>(*table, ct);
        } else {
            const int16_t v = rd<int16_t>(*in, idx);
            const int32_t index = (int32_t(v) + 32768) >> 7;
            const int32_t fraction = int32_t(v) & 0x7f;
            const uint32_t ct[1] = {uint32_t(index)};
            const int32_t base = rd<int16_t>(*table, ct, 0);
            const int32_t next = rd<int16_t>(*table, ct, 1);
            const int32_t slope = next - base;
            result = int32_t((uint32_t(base) << 7) + uint32_t(slope) * uint32_t(fraction));
        }
        wrInt(*out, idx, result);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/transpose.comp:19-32
int orc_transpose(const orc_tensor *in, const orc_tensor *out, const uint32_t *perms) {
    const int64_t total = numel(*out);
    const int es = elemSize(out->dtype);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], src[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        for (int i = 0; i < out->rank; ++i) {
            src[perms[i]] = idx[i];
        }
        int64_t so = 0, doff = 0;
        bool oob = false;
        for (int i = 0; i < out->rank; ++i) {
            oob |= int64_t(src[i]) >= in->dims[i];
            so += int64_t(src[i]) * in->strides[i];
            doff += int64_t(idx[i]) * out->strides[i];
        }
        char *d = static_cast<char *>(out->data) + doff;
        if (oob) {
            std::memset(d, 0, size_t(es));
        } else {
            std::memcpy(d, static_cast<const char *>(in->data) + so, size_t(es));
        }
    }
    return 0;
}

// Generic "gather by index map" used by the data-movement shaders below.
extern "C++" {
namespace {
template <typename F> void moveElements(const orc_tensor &iter, const orc_tensor &in, const orc_tensor &out, F map) {
    const int64_t total = numel(iter);
    const int es = elemSize(out.dtype);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], src[kMaxRank], dst[kMaxRank];
        unravel(iter, uint32_t(e), idx);
        bool isConst = false;
        int64_t constBits = 0;
        map(idx, src, dst, isConst, constBits);
        int64_t doff = 0;
        bool dropped = false;
        for (int i = 0; i < out.rank; ++i) {
            dropped |= int64_t(dst[i]) >= out.dims[i];
            doff += int64_t(dst[i]) * out.strides[i];
        }
        if (dropped) {
            continue;
        }
        char *d = static_cast<char *>(out.data) + doff;
        if (isConst) {
            std::memcpy(d, &constBits, size_t(es));
            continue;
        }
        int64_t so = 0;
        bool oob = false;
        for (int i = 0; i < in.rank; ++i) {
            oob |= int64_t(src[i]) >= in.dims[i];
            so += int64_t(src[i]) * in.strides[i];
        }
        if (oob) {
            std::memset(d, 0, size_t(es));
        } else {
            std::memcpy(d, static_cast<const char *>(in.data) + so, size_t(es));
        }
    }
}
} // namespace
} // extern "C++"

// graph/shaders/graph_op/tosa/concat.comp:20-34 — one pass per input, iterating the INPUT's elements.
int orc_concat(const orc_tensor *in, const orc_tensor *out, uint32_t axis, uint32_t offset) {
    const int rank = in->rank;
    moveElements(*in, *in, *out, [&](const uint32_t *idx, uint32_t *src, uint32_t *dst, bool &, int64_t &) {
        for (int i = 0; i < rank; ++i) {
            src[i] = idx[i];
            dst[i] = idx[i];
        }
        dst[axis] += offset;
    });
    return 0;
}

// graph/shaders/graph_op/tosa/reshape.comp:17-27 — same linear offset unravelled in both shapes.
int orc_reshape(const orc_tensor *in, const orc_tensor *out) {
    const int64_t total = numel(*out);
    const int es = elemSize(out->dtype);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t di[kMaxRank], si[kMaxRank];
        unravel(*out, uint32_t(e), di);
        // common.comp:82-84: a thread whose offset does not fit the input shape returns early
        uint32_t off = uint32_t(e);
        for (int i = in->rank - 1; i >= 0; --i) {
            si[i] = off % uint32_t(in->dims[i]);
            off /= uint32_t(in->dims[i]);
        }
        if (off > 0) {
            continue;
        }
        int64_t so = 0, doff = 0;
        for (int i = 0; i < in->rank; ++i) {
            so += int64_t(si[i]) * in->strides[i];
        }
        for (int i = 0; i < out->rank; ++i) {
            doff += int64_t(di[i]) * out->strides[i];
        }
        std::memcpy(static_cast<char *>(out->data) + doff, static_cast<const char *>(in->data) + so, size_t(es));
    }
    return 0;
}

// graph/shaders/graph_op/tosa/slice.comp:19-33
int orc_slice(const orc_tensor *in, const orc_tensor *out, const uint32_t *start) {
    const int rank = out->rank;
    moveElements(*out, *in, *out, [&](const uint32_t *idx, uint32_t *src, uint32_t *dst, bool &, int64_t &) {
        for (int i = 0; i < rank; ++i) {
            src[i] = idx[i] + start[i];
            dst[i] = idx[i];
        }
    });
    return 0;
}

// graph/shaders/graph_op/tosa/pad.comp:23-55.  `padding` holds 2*rank int32 values; only the
// leading pad of each dimension (element 2*i) is read.  padConstBits is the already-encoded
// storage value of the pad constant.
int orc_pad(const orc_tensor *in, const orc_tensor *out, const orc_tensor *padding, int64_t padConstBits) {
    const int rank = out->rank;
    moveElements(*out, *in, *out, [&](const uint32_t *idx, uint32_t *src, uint32_t *dst, bool &isConst, int64_t &bits) {
        for (int i = 0; i < rank; ++i) {
            dst[i] = idx[i];
            src[i] = 0;
        }
        for (int i = 0; i < rank; ++i) {
            const uint32_t cp[1] = {uint32_t(2 * i)};
            const int32_t p = rd<int32_t>(*padding, cp);
            src[i] = idx[i] - uint32_t(p);
            if (int64_t(src[i]) >= in->dims[i]) {
                isConst = true;
                bits = padConstBits;
                break;
            }
        }
    });
    return 0;
}

// graph/shaders/graph_op/tosa/clamp.comp:24-53 (integer path): bounds arrive as double and are
// converted with the storage type's constructor.
int orc_clamp(const orc_tensor *in, const orc_tensor *out, double minV, double maxV) {
    const int64_t total = numel(*out);
    const int64_t lo = wrapTo(out->dtype, int64_t(minV)), hi = wrapTo(out->dtype, int64_t(maxV));
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const int64_t v = rdInt(*in, idx);
        // GLSL clamp(x, lo, hi) = min(max(x, lo), hi)
        wrInt(*out, idx, std::min(std::max(v, lo), hi));
    }
    return 0;
}

enum orc_binary_op {
    ORC_ADD = 0,
    ORC_SUB = 1,
    ORC_BITWISE_AND = 2,
    ORC_BITWISE_OR = 3,
    ORC_BITWISE_XOR = 4,
    ORC_LOGICAL_AND = 5,
    ORC_LOGICAL_OR = 6,
    ORC_LOGICAL_XOR = 7,
    ORC_LOGICAL_LEFT_SHIFT = 8,
    ORC_LOGICAL_RIGHT_SHIFT = 9,
    ORC_INTDIV = 10,
    ORC_MAXIMUM = 11,
    ORC_MINIMUM = 12,
    ORC_EQUAL = 13,
    ORC_GREATER = 14,
    ORC_GREATER_EQUAL = 15,
    ORC_POW = 16,
};

namespace {
// common.comp:64-72
void broadcast(const orc_tensor &t, const uint32_t *idx, uint32_t *c) {
    for (int i = t.rank - 1; i >= 0; --i) {
        c[i] = t.dims[i] == 1 ? 0u : idx[i];
    }
}

int bitWidth(int dtype) { return elemSize(dtype) * 8; }
} // namespace

// graph/shaders/graph_op/tosa/elementwise_binary.comp:146-173 with the operation strings of
// graph/compute_graph_op.cpp:2532-2935.  Integer arithmetic is done in the input's own type.
int orc_binary(const orc_tensor *a, const orc_tensor *b, const orc_tensor *out, int op) {
    const int64_t total = numel(*out);
    const int dt = a->dtype;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], ca[kMaxRank], cb[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        broadcast(*a, idx, ca);
        broadcast(*b, idx, cb);
        if (dt == ORC_F32) {
            const float x = rd<float>(*a, ca), y = rd<float>(*b, cb);
            float r = 0.0f;
            int64_t ri = 0;
            bool isBool = false;
            switch (op) {
            case ORC_ADD:
                r = x + y;
                break;
            case ORC_SUB:
                r = x - y;
                break;
            case ORC_MAXIMUM: // NaN propagate mode
                r = std::isnan(x) ? x : (std::isnan(y) ? y : std::max(x, y));
                break;
            case ORC_MINIMUM:
                r = std::isnan(x) ? x : (std::isnan(y) ? y : std::min(x, y));
                break;
            case ORC_EQUAL:
                ri = x == y, isBool = true;
                break;
            case ORC_GREATER:
                ri = x > y, isBool = true;
                break;
            case ORC_GREATER_EQUAL:
                ri = x >= y, isBool = true;
                break;
            case ORC_POW: // elementwise_binary.comp:71-89; the power itself in double, rounded once
                if (x >= 0.0f) {
                    r = float(std::pow(double(x), double(y)));
                } else if (std::fmod(y, 2.0f) == 0.0f) {
                    r = float(std::pow(double(-x), double(y)));
                } else if (std::fmod(y, 1.0f) == 0.0f) {
                    r = float(-std::pow(double(-x), double(y)));
                } else {
                    r = std::numeric_limits<float>::quiet_NaN();
                }
                break;
            default:
                break;
            }
            if (isBool) {
                wrInt(*out, idx, ri);
            } else {
                wr<float>(*out, idx, r);
            }
            continue;
        }
        const int64_t x = rdInt(*a, ca), y = rdInt(*b, cb);
        int64_t r = 0;
        switch (op) {
        case ORC_ADD:
            r = wrapTo(dt, int64_t(uint64_t(x) + uint64_t(y)));
            break;
        case ORC_SUB:
            r = wrapTo(dt, int64_t(uint64_t(x) - uint64_t(y)));
            break;
        case ORC_BITWISE_AND:
            r = x & y;
            break;
        case ORC_BITWISE_OR:
            r = x | y;
            break;
        case ORC_BITWISE_XOR:
            r = x ^ y;
            break;
        case ORC_LOGICAL_AND:
            r = (x != 0) && (y != 0);
            break;
        case ORC_LOGICAL_OR:
            r = (x != 0) || (y != 0);
            break;
        case ORC_LOGICAL_XOR:
            r = (x != 0) != (y != 0);
            break;
        case ORC_LOGICAL_LEFT_SHIFT: // "uint(value1) << uint(value2)": 32-bit shift, then narrowed
            r = int64_t(uint32_t(uint32_t(x) << (uint32_t(y) & 31u)));
            break;
        case ORC_LOGICAL_RIGHT_SHIFT: { // "zeroExtend(value1) >> uint(value2)"
            const uint32_t z = bitWidth(dt) == 8 ? uint8_t(x) : (bitWidth(dt) == 16 ? uint16_t(x) : uint32_t(x));
            r = int64_t(z >> (uint32_t(y) & 31u));
            break;
        }
        case ORC_INTDIV:
            if (y == 0) {
                r = 0; // undefined in the shader
            } else if (x == typeLowest(dt) && y == -1) {
                r = x; // wraps
            } else {
                r = x / y;
            }
            break;
        case ORC_MAXIMUM:
            r = std::max(x, y);
            break;
        case ORC_MINIMUM:
            r = std::min(x, y);
            break;
        case ORC_EQUAL:
            r = x == y;
            break;
        case ORC_GREATER:
            r = x > y;
            break;
        case ORC_GREATER_EQUAL:
            r = x >= y;
            break;
        default:
            break;
        }
        wrInt(*out, idx, r);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/mul.comp:24-59 (integer path)
int orc_mul(const orc_tensor *a, const orc_tensor *b, const orc_tensor *out, uint32_t shift) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], ca[kMaxRank], cb[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        broadcast(*a, idx, ca);
        broadcast(*b, idx, cb);
        if (a->dtype == ORC_F32) {
            wr<float>(*out, idx, rd<float>(*a, ca) * rd<float>(*b, cb));
            continue;
        }
        int64_t r = int64_t(uint64_t(rdInt(*a, ca)) * uint64_t(rdInt(*b, cb)));
        if (shift > 0) {
            r = int64_t(uint64_t(r) + (uint64_t(1) << ((shift - 1) & 63))) >> (shift & 63);
        }
        wrInt(*out, idx, r);
    }
    return 0;
}

enum orc_reduce_op { ORC_RSUM = 0, ORC_RMAX = 1, ORC_RMIN = 2, ORC_RPRODUCT = 3, ORC_RALL = 4, ORC_RANY = 5 };

// graph/shaders/graph_op/tosa/reduce.comp:24-70 (integer path: arithmetic in the storage type,
// MAX/MIN start from the type's lowest/max, graph/compute_graph_op.cpp:2831-2847)
int orc_reduce(const orc_tensor *in, const orc_tensor *out, uint32_t axis, int op) {
    const int64_t total = numel(*out);
    const int dt = in->dtype;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const uint32_t dim = idx[axis];
        int64_t r = 0;
        switch (op) {
        case ORC_RMAX:
            r = typeLowest(dt);
            break;
        case ORC_RMIN:
            r = typeMax(dt);
            break;
        case ORC_RPRODUCT:
        case ORC_RALL:
            r = 1;
            break;
        default:
            r = 0;
            break;
        }
        for (uint32_t i = 0; i < uint32_t(in->dims[axis]); ++i) {
            idx[axis] = i;
            const int64_t v = rdInt(*in, idx);
            switch (op) {
            case ORC_RSUM:
                r = wrapTo(dt, int64_t(uint64_t(r) + uint64_t(v)));
                break;
            case ORC_RMAX:
                r = std::max(r, v);
                break;
            case ORC_RMIN:
                r = std::min(r, v);
                break;
            case ORC_RPRODUCT:
                r = wrapTo(dt, int64_t(uint64_t(r) * uint64_t(v)));
                break;
            case ORC_RALL:
                r = (r != 0) && (v != 0);
                break;
            case ORC_RANY:
                r = (r != 0) || (v != 0);
                break;
            default:
                break;
            }
        }
        idx[axis] = dim;
        wrInt(*out, idx, r);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/cast.comp:24-103: int<->int/bool by constructor; int->f32 plain
// conversion; f32->int saturating round-half-even.
int orc_cast(const orc_tensor *in, const orc_tensor *out) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        if (in->dtype == ORC_F32 && out->dtype == ORC_F32) {
            wr<float>(*out, idx, rd<float>(*in, idx));
        } else if (in->dtype == ORC_F32) {
            const float f = rd<float>(*in, idx);
            if (out->dtype == ORC_BOOL) {
                wrInt(*out, idx, f != 0.0f);
                continue;
            }
            const int64_t lo = typeLowest(out->dtype), hi = typeMax(out->dtype);
            int64_t r;
            if (f <= float(lo)) {
                r = lo;
            } else if (f >= float(hi)) {
                r = hi;
            } else {
                r = int64_t(std::nearbyint(f)); // default rounding mode = round-half-even
            }
            wrInt(*out, idx, r);
        } else if (out->dtype == ORC_F32) {
            wr<float>(*out, idx, float(rdInt(*in, idx)));
        } else {
            const int64_t v = rdInt(*in, idx);
            wrInt(*out, idx, out->dtype == ORC_BOOL ? (v != 0) : v);
        }
    }
    return 0;
}

// graph/shaders/graph_op/tosa/arithmetic_right_shift.comp:22-49 (arithmetic in the storage type)
int orc_arithmetic_right_shift(const orc_tensor *a, const orc_tensor *b, const orc_tensor *out, int round) {
    const int64_t total = numel(*out);
    const int dt = a->dtype;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], ca[kMaxRank], cb[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        broadcast(*a, idx, ca);
        broadcast(*b, idx, cb);
        const int64_t x = rdInt(*a, ca), y = rdInt(*b, cb);
        int64_t r = x >> (y & 63);
        if (round && y > 0 && ((x >> ((y - 1) & 63)) & 1) != 0) {
            r = wrapTo(dt, r + 1);
        }
        wrInt(*out, idx, r);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/negate.comp:32-48 (integer path: int32 arithmetic, clamp to type range)
int orc_negate(const orc_tensor *in, const orc_tensor *out, int32_t inZp, int32_t outZp) {
    const int64_t total = numel(*out);
    const int64_t lo = std::max<int64_t>(typeLowest(out->dtype), std::numeric_limits<int32_t>::min());
    const int64_t hi = std::min<int64_t>(typeMax(out->dtype), std::numeric_limits<int32_t>::max());
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const int32_t v = int32_t(rdInt(*in, idx));
        const int32_t res = int32_t(uint32_t(inZp) - uint32_t(v) + uint32_t(outZp));
        wrInt(*out, idx, std::min<int64_t>(std::max<int64_t>(res, lo), hi));
    }
    return 0;
}

// graph/shaders/graph_op/tosa/select.comp:18-42
int orc_select(const orc_tensor *cond, const orc_tensor *a, const orc_tensor *b, const orc_tensor *out) {
    const int64_t total = numel(*out);
    const int es = elemSize(out->dtype);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], c[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        broadcast(*cond, idx, c);
        const orc_tensor &src = rd<uint8_t>(*cond, c) != 0 ? *a : *b;
        broadcast(src, idx, c);
        int64_t bits = 0;
        switch (es) {
        case 1:
            bits = rd<uint8_t>(src, c);
            break;
        case 2:
            bits = rd<uint16_t>(src, c);
            break;
        case 4:
            bits = rd<uint32_t>(src, c);
            break;
        default:
            bits = rd<int64_t>(src, c);
            break;
        }
        int64_t doff = 0;
        for (int i = 0; i < out->rank; ++i) {
            doff += int64_t(idx[i]) * out->strides[i];
        }
        std::memcpy(static_cast<char *>(out->data) + doff, &bits, size_t(es));
    }
    return 0;
}

enum orc_unary_op { ORC_ABS = 0, ORC_BITWISE_NOT = 1, ORC_CLZ = 2, ORC_LOGICAL_NOT = 3 };

// graph/shaders/graph_op/tosa/elementwise_unary.comp (integer operations only):
// "abs(value1)", "~value1", "clz(value1)" (32-bit leading-zero loop), "!value1".
int orc_unary(const orc_tensor *in, const orc_tensor *out, int op) {
    const int64_t total = numel(*out);
    const int dt = in->dtype;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const int64_t v = rdInt(*in, idx);
        int64_t r = 0;
        switch (op) {
        case ORC_ABS:
            r = wrapTo(dt, v < 0 ? int64_t(0 - uint64_t(v)) : v);
            break;
        case ORC_BITWISE_NOT:
            r = ~v;
            break;
        case ORC_CLZ: {
            const uint32_t u = uint32_t(v);
            int i = 0;
            for (; i < 32; ++i) {
                if ((u & (1u << (31 - i))) != 0) {
                    break;
                }
            }
            r = i;
            break;
        }
        case ORC_LOGICAL_NOT:
            r = v == 0;
            break;
        default:
            break;
        }
        wrInt(*out, idx, r);
    }
    return 0;
}


} // extern "C"

namespace {

// Raw bits of one element (any type); a coordinate out of range reads as zero (tensor.glsl:26-50).
int64_t rdBits(const orc_tensor &t, const uint32_t *c) {
    switch (elemSize(t.dtype)) {
    case 1:
        return rd<uint8_t>(t, c);
    case 2:
        return rd<uint16_t>(t, c);
    case 4:
        return rd<uint32_t>(t, c);
    default:
        return rd<int64_t>(t, c);
    }
}

void wrBits(const orc_tensor &t, const uint32_t *c, int64_t bits) {
    switch (elemSize(t.dtype)) {
    case 1:
        wr<uint8_t>(t, c, uint8_t(bits));
        break;
    case 2:
        wr<uint16_t>(t, c, uint16_t(bits));
        break;
    case 4:
        wr<uint32_t>(t, c, uint32_t(bits));
        break;
    default:
        wr<int64_t>(t, c, bits);
        break;
    }
}

// resize.comp:43-51
int32_t idivFloor(int32_t n, int32_t d) {
    int32_t r = n / d;
    if (r * d > n) {
        --r;
    }
    return r;
}

// resize.comp:53-134 for the integer types: ACC (= the output's own type) holds the products, which wrap.
template <typename ACC>
void resizeImpl(const orc_tensor &in, const orc_tensor &out, const int32_t *scale, const int32_t *offset, int32_t mode) {
    using U = std::make_unsigned_t<ACC>;
    const int64_t total = numel(out);
    const uint32_t H = uint32_t(in.dims[1]), W = uint32_t(in.dims[2]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], c = idx[3];
        const int16_t unitY = int16_t(scale[0]), unitX = int16_t(scale[2]);
        const int32_t y = int32_t(oy * uint32_t(scale[1]) + uint32_t(offset[0]));
        const int16_t iy = int16_t(idivFloor(y, scale[0]));
        const int16_t ry = int16_t(uint32_t(y) - uint32_t(int32_t(iy)) * uint32_t(scale[0]));
        const int32_t x = int32_t(ox * uint32_t(scale[3]) + uint32_t(offset[1]));
        const int16_t ix = int16_t(idivFloor(x, scale[2]));
        const int16_t rx = int16_t(uint32_t(x) - uint32_t(int32_t(ix)) * uint32_t(scale[2]));
        const int16_t dy = ry, dx = rx;
        // GLSL: max(int16_t, int) -> int; min(int, uint) -> uint (the signed operand converts)
        const int16_t iy0 = int16_t(std::max(int32_t(iy), 0));
        const int16_t iy1 = int16_t(std::min(uint32_t(int32_t(iy) + 1), H - 1));
        const int16_t ix0 = int16_t(std::max(int32_t(ix), 0));
        const int16_t ix1 = int16_t(std::min(uint32_t(int32_t(ix) + 1), W - 1));
        const auto at = [&](int16_t yy, int16_t xx) {
            const uint32_t ci[4] = {n, uint32_t(int32_t(yy)), uint32_t(int32_t(xx)), c};
            return U(ACC(rdInt(in, ci)));
        };
        const auto mul3 = [](U a, U b, U cc) { return U(uint64_t(U(uint64_t(a) * uint64_t(b))) * uint64_t(cc)); };
        ACC acc = 0;
        if (mode == 2) {
            const U wy0 = U(ACC(int16_t(unitY - dy))), wy1 = U(ACC(dy));
            const U wx0 = U(ACC(int16_t(unitX - dx))), wx1 = U(ACC(dx));
            U sum = mul3(at(iy0, ix0), wy0, wx0);
            sum = U(sum + mul3(at(iy0, ix1), wy0, wx1));
            sum = U(sum + mul3(at(iy1, ix0), wy1, wx0));
            sum = U(sum + mul3(at(iy1, ix1), wy1, wx1));
            acc = ACC(sum);
        } else if (mode == 1) {
            const int16_t py = (2 * int32_t(dy) >= scale[0]) ? iy1 : iy0;
            const int16_t px = (2 * int32_t(dx) >= scale[2]) ? ix1 : ix0;
            acc = ACC(at(py, px));
        }
        wrInt(out, idx, int64_t(acc));
    }
}

// transpose_conv2d.comp:29-70
template <typename ACC>
void transposeConv2dImpl(const orc_tensor &in, const orc_tensor &w, const orc_tensor &bias, const orc_tensor &out,
                         const int32_t *pad, const int32_t *stride, int32_t inZp, int32_t wZp) {
    const int64_t total = numel(out);
    const uint32_t KH = uint32_t(w.dims[1]), KW = uint32_t(w.dims[2]), IC = uint32_t(in.dims[3]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], oc = idx[3];
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
        ACC acc = ACC(rdInt(bias, cb));
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                int32_t iy = int32_t(oy) - pad[0] - int32_t(ky);
                int32_t ix = int32_t(ox) - pad[2] - int32_t(kx);
                if ((iy % stride[0]) == 0 && (ix % stride[1]) == 0) {
                    iy /= stride[0];
                    ix /= stride[1];
                    if (iy >= 0 && ix >= 0 && int64_t(iy) < in.dims[1] && int64_t(ix) < in.dims[2]) {
                        for (uint32_t ic = 0; ic < IC; ++ic) {
                            const uint32_t ci[4] = {n, uint32_t(iy), uint32_t(ix), ic};
                            const uint32_t cw[4] = {oc, ky, kx, ic};
                            const ACC v = Wrap<ACC>::sub(ACC(rdInt(in, ci)), ACC(inZp));
                            const ACC wt = Wrap<ACC>::sub(ACC(rdInt(w, cw)), ACC(wZp));
                            acc = Wrap<ACC>::add(acc, Wrap<ACC>::mul(v, wt));
                        }
                    }
                }
            }
        }
        wrInt(out, idx, int64_t(acc));
    }
}

// conv3d.comp:33-104, with the shader's own start/stop logic for the taps
template <typename ACC>
void conv3dImpl(const orc_tensor &in, const orc_tensor &w, const orc_tensor &bias, const orc_tensor &out,
                const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    const int64_t total = numel(out);
    const int KD = int(w.dims[1]), KH = int(w.dims[2]), KW = int(w.dims[3]), IC = int(w.dims[4]);
    const int ID = int(in.dims[1]), IH = int(in.dims[2]), IW = int(in.dims[3]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oc = idx[4];
        const int id = int(idx[1]) * stride[0] - pad[0];
        const int iy = int(idx[2]) * stride[1] - pad[2];
        const int ix = int(idx[3]) * stride[2] - pad[4];
        int dStart = id, kdStart = 0;
        if (dStart < 0) {
            kdStart = (-dStart + dil[0] - 1) / dil[0];
            dStart = id + kdStart * dil[0];
        }
        int yStart = iy, kyStart = 0;
        if (yStart < 0) {
            kyStart = (-yStart + dil[1] - 1) / dil[1];
            yStart = iy + kyStart * dil[1];
        }
        int xStart = ix, kxStart = 0;
        if (xStart < 0) {
            kxStart = (-xStart + dil[2] - 1) / dil[2];
            xStart = ix + kxStart * dil[2];
        }
        ACC acc = 0;
        for (int d = dStart, kd = kdStart; kd < KD && d < ID; ++kd, d += dil[0]) {
            for (int y = yStart, ky = kyStart; ky < KH && y < IH; ++ky, y += dil[1]) {
                for (int x = xStart, kx = kxStart; kx < KW && x < IW; ++kx, x += dil[2]) {
                    for (int ic = 0; ic < IC; ++ic) {
                        const uint32_t ci[5] = {n, uint32_t(d), uint32_t(y), uint32_t(x), uint32_t(ic)};
                        const uint32_t cw[5] = {oc, uint32_t(kd), uint32_t(ky), uint32_t(kx), uint32_t(ic)};
                        const ACC v = Wrap<ACC>::sub(ACC(rdInt(in, ci)), ACC(inZp));
                        const ACC wt = Wrap<ACC>::sub(ACC(rdInt(w, cw)), ACC(wZp));
                        acc = Wrap<ACC>::add(acc, Wrap<ACC>::mul(v, wt));
                    }
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
        acc = Wrap<ACC>::add(ACC(rdInt(bias, cb)), acc);
        wrInt(out, idx, int64_t(acc));
    }
}

} // namespace

extern "C" {

// graph/shaders/graph_op/tosa/argmax.comp:26-66, integer inputs
int orc_argmax(const orc_tensor *in, const orc_tensor *out, uint32_t axis) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, src[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(*out, uint32_t(e), idx);
        for (uint32_t i = 0; i < axis; ++i) {
            src[i] = idx[i];
        }
        for (uint32_t i = axis; i < uint32_t(out->rank); ++i) {
            src[i + 1] = idx[i];
        }
        int64_t maxValue = typeLowest(in->dtype);
        int32_t maxIndex = 0;
        for (int32_t i = 0; i < int32_t(in->dims[axis]); ++i) {
            src[axis] = uint32_t(i);
            const int64_t v = rdInt(*in, src);
            if (v > maxValue) {
                maxValue = v;
                maxIndex = i;
            }
        }
        wrInt(*out, idx, maxIndex);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/gather.comp:14-25
int orc_gather(const orc_tensor *values, const orc_tensor *indices, const orc_tensor *out) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const uint32_t ci[2] = {idx[0], idx[1]};
        const uint32_t k = uint32_t(rdInt(*indices, ci));
        const uint32_t cv[3] = {idx[0], k, idx[2]};
        wrBits(*out, idx, rdBits(*values, cv));
    }
    return 0;
}

// graph/shaders/graph_op/tosa/scatter.comp:15-34
int orc_scatter(const orc_tensor *valuesIn, const orc_tensor *indices, const orc_tensor *input,
                const orc_tensor *out) {
    const int64_t total = numel(*out);
    const uint32_t W = uint32_t(indices->dims[1]);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        int64_t bits = rdBits(*valuesIn, idx);
        for (uint32_t w = 0; w < W; ++w) {
            const uint32_t ci[2] = {idx[0], w};
            if (uint32_t(rdInt(*indices, ci)) == idx[1]) {
                const uint32_t cs[3] = {idx[0], w, idx[2]};
                bits = rdBits(*input, cs);
                break;
            }
        }
        wrBits(*out, idx, bits);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/reverse.comp:19-30
int orc_reverse(const orc_tensor *in, const orc_tensor *out, uint32_t axis) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const int64_t bits = rdBits(*in, idx);
        idx[axis] = uint32_t(out->dims[axis]) - 1 - idx[axis];
        wrBits(*out, idx, bits);
    }
    return 0;
}

// graph/shaders/graph_op/tosa/tile.comp:15-30
int orc_tile(const orc_tensor *in, const orc_tensor *out) {
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank], src[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        for (int i = 0; i < out->rank; ++i) {
            src[i] = idx[i] % uint32_t(in->dims[i]);
        }
        wrBits(*out, idx, rdBits(*in, src));
    }
    return 0;
}

// graph/shaders/graph_op/tosa/resize.comp; scale = {y_n, y_d, x_n, x_d}, mode 1 NEAREST / 2 BILINEAR
int orc_resize(const orc_tensor *in, const orc_tensor *out, const int32_t *scale, const int32_t *offset,
               int32_t mode) {
    switch (out->dtype) {
    case ORC_I8:
        resizeImpl<int8_t>(*in, *out, scale, offset, mode);
        return 0;
    case ORC_I16:
        resizeImpl<int16_t>(*in, *out, scale, offset, mode);
        return 0;
    case ORC_I32:
        resizeImpl<int32_t>(*in, *out, scale, offset, mode);
        return 0;
    case ORC_I64:
        resizeImpl<int64_t>(*in, *out, scale, offset, mode);
        return 0;
    default:
        return -1;
    }
}

int orc_transpose_conv2d(const orc_tensor *in, const orc_tensor *w, const orc_tensor *bias, const orc_tensor *out,
                         const int32_t *pad, const int32_t *stride, int32_t inZp, int32_t wZp) {
    if (out->dtype == ORC_I32) {
        transposeConv2dImpl<int32_t>(*in, *w, *bias, *out, pad, stride, inZp, wZp);
    } else if (out->dtype == ORC_I64) {
        transposeConv2dImpl<int64_t>(*in, *w, *bias, *out, pad, stride, inZp, wZp);
    } else {
        return -1;
    }
    return 0;
}

int orc_conv3d(const orc_tensor *in, const orc_tensor *w, const orc_tensor *bias, const orc_tensor *out,
               const int32_t *pad, const int32_t *stride, const int32_t *dil, int32_t inZp, int32_t wZp) {
    if (out->dtype == ORC_I32) {
        conv3dImpl<int32_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else if (out->dtype == ORC_I64) {
        conv3dImpl<int64_t>(*in, *w, *bias, *out, pad, stride, dil, inZp, wZp);
    } else {
        return -1;
    }
    return 0;
}


enum orc_unary_f32_op {
    ORC_F_ABS = 0,
    ORC_F_CEIL = 4,
    ORC_F_COS = 5,
    ORC_F_ERF = 6,
    ORC_F_EXP = 7,
    ORC_F_FLOOR = 8,
    ORC_F_LOG = 9,
    ORC_F_RECIPROCAL = 10,
    ORC_F_RSQRT = 11,
    ORC_F_SIGMOID = 12,
    ORC_F_SIN = 13,
    ORC_F_TANH = 14,
};

// graph/shaders/graph_op/tosa/elementwise_unary.comp:204-223 for fp32 tensors, with the operator expressions of
// graph/compute_graph_op.cpp:2527-2945.  The reference evaluates the transcendental functions with its Vulkan
// device's single-precision builtins, whose last bits differ between devices; this restatement evaluates them
// in double precision and rounds once, i.e. it gives the value every conforming implementation approximates.
// The shader's special cases are kept: NaN passes through, LOG of a negative number is NaN, TANH saturates
// beyond |x| = 10.  Comparisons against this function use a tolerance stated in the tests.
int orc_unary_f32(const orc_tensor *in, const orc_tensor *out, int op) {
    if (in->dtype != ORC_F32 || out->dtype != ORC_F32) {
        return -1;
    }
    const int64_t total = numel(*out);
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*out, uint32_t(e), idx);
        const float xf = rd<float>(*in, idx);
        const double x = double(xf);
        float r = xf;
        if (!std::isnan(xf)) {
            switch (op) {
            case ORC_F_ABS:
                r = std::fabs(xf);
                break;
            case ORC_F_CEIL:
                r = std::ceil(xf);
                break;
            case ORC_F_FLOOR:
                r = std::floor(xf);
                break;
            case ORC_F_COS:
                r = float(std::cos(x));
                break;
            case ORC_F_ERF:
                r = float(std::erf(x));
                break;
            case ORC_F_EXP:
                r = float(std::exp(x));
                break;
            case ORC_F_LOG:
                r = xf < 0.0f ? std::numeric_limits<float>::quiet_NaN() : float(std::log(x));
                break;
            case ORC_F_RECIPROCAL:
                r = 1.0f / xf;
                break;
            case ORC_F_RSQRT:
                r = float(1.0 / std::sqrt(x));
                break;
            case ORC_F_SIGMOID:
                r = float(1.0 / (1.0 + std::exp(-x)));
                break;
            case ORC_F_SIN:
                r = float(std::sin(x));
                break;
            case ORC_F_TANH:
                r = xf > 10.0f ? 1.0f : (xf < -10.0f ? -1.0f : float(std::tanh(x)));
                break;
            default:
                break;
            }
        }
        wr<float>(*out, idx, r);
    }
    return 0;
}


// graph/shaders/graph_op/tosa/fft2d.comp:17-55 (imag != null) and rfft2d.comp:12-71 (imag == null, outputs of
// W / 2 + 1 columns): the defining double sum, evaluated in double precision with the angle's numerator reduced
// modulo H*W and rounded to float once.  The shaders compute the same sums with their device's single-precision
// sine and cosine; comparisons against this function use a tolerance stated in the tests.
int orc_fft2d(const orc_tensor *real, const orc_tensor *imag, const orc_tensor *outReal, const orc_tensor *outImag,
              int inverse) {
    const int64_t total = numel(*outReal);
    const uint32_t H = uint32_t(real->dims[1]), W = uint32_t(real->dims[2]);
    const double kPi = 3.14159265358979323846;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < total; ++e) {
        uint32_t idx[kMaxRank];
        unravel(*outReal, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2];
        const bool skipImag = imag == nullptr && (oy == 0 || oy == H / 2) && (ox == 0 || ox == W / 2);
        long double sumRe = 0.0L, sumIm = 0.0L;
        for (uint32_t iy = 0; iy < H; ++iy) {
            for (uint32_t ix = 0; ix < W; ++ix) {
                const uint32_t ci[3] = {n, iy, ix};
                const double re = rd<float>(*real, ci);
                const double im = imag != nullptr ? double(rd<float>(*imag, ci)) : 0.0;
                const uint64_t num = ((uint64_t(iy) * oy % H) * W + (uint64_t(ix) * ox % W) * H) % (uint64_t(H) * W);
                const double angle = 2.0 * kPi * double(num) / double(uint64_t(H) * W);
                const double cs = std::cos(angle), sn = inverse ? -std::sin(angle) : std::sin(angle);
                sumRe += re * cs + im * sn;
                sumIm += im * cs - re * sn;
            }
        }
        wr<float>(*outReal, idx, float(sumRe));
        wr<float>(*outImag, idx, skipImag ? 0.0f : float(sumIm));
    }
    return 0;
}

} // extern "C"
