// Vectorised kernels for the element-wise, table, reduction and data-movement operators on packed
// tensors.  Each has a generic counterpart in generic_ops.cu that defines the result for every rank, stride
// and type; these take the common case - contiguous tensors, signed integer types, operands of the same
// shape or broadcast along the last axis - and only change how the bytes move: four elements per thread
// with 4-, 8- or 16-byte accesses, no index unravelling, a warp per row for reductions.  The arithmetic is
// the same functions (device_common.cuh), so the results are the same bits.
//
// Every entry point returns false when it does not apply; the caller then runs the generic kernel.
#include <algorithm>
#include <string>

#include "device_common.cuh"
#include "gemm_i8_tcgen05.hpp"
#include "kernels.hpp"

namespace mlel {

namespace {

#define GRID_STRIDE(e, total)                                                                                          \
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < (total); e += int64_t(gridDim.x) * blockDim.x)

int finish(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        setLastError(std::string(what) + ": " + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

// Number of elements of a contiguous (byte strides = packed) tensor, or -1.
int64_t packedNumel(const TView &t) {
    int64_t st = dtypeSize(t.dtype), n = 1;
    for (int i = t.rank - 1; i >= 0; --i) {
        if (t.strides[i] != st) {
            return -1;
        }
        st *= t.dims[i];
        n *= t.dims[i];
    }
    return n;
}

bool sameShape(const TView &a, const TView &b) {
    if (a.rank != b.rank) {
        return false;
    }
    for (int i = 0; i < a.rank; ++i) {
        if (a.dims[i] != b.dims[i]) {
            return false;
        }
    }
    return true;
}

// b has out's shape except for a last axis of 1 (one value per row of out).
bool rowBroadcast(const TView &b, const TView &out) {
    if (b.rank != out.rank || out.rank < 1 || b.dims[b.rank - 1] != 1) {
        return false;
    }
    for (int i = 0; i + 1 < out.rank; ++i) {
        if (b.dims[i] != out.dims[i]) {
            return false;
        }
    }
    return true;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool signedInt(int32_t dtype) { return dtype == MLEL_I8 || dtype == MLEL_I16 || dtype == MLEL_I32; }

// Four consecutive elements of a signed integer type, widened to int32.
template <typename T> __device__ __forceinline__ void load4(const T *p, int32_t (&v)[4]);
template <> __device__ __forceinline__ void load4<int8_t>(const int8_t *p, int32_t (&v)[4]) {
    const uint32_t w = *reinterpret_cast<const uint32_t *>(p);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        v[k] = int32_t(int8_t(w >> (8 * k)));
    }
}
template <> __device__ __forceinline__ void load4<int16_t>(const int16_t *p, int32_t (&v)[4]) {
    const uint2 w = *reinterpret_cast<const uint2 *>(p);
    v[0] = int32_t(int16_t(w.x)), v[1] = int32_t(int16_t(w.x >> 16));
    v[2] = int32_t(int16_t(w.y)), v[3] = int32_t(int16_t(w.y >> 16));
}
template <> __device__ __forceinline__ void load4<int32_t>(const int32_t *p, int32_t (&v)[4]) {
    const int4 w = *reinterpret_cast<const int4 *>(p);
    v[0] = w.x, v[1] = w.y, v[2] = w.z, v[3] = w.w;
}
// Stores the low bits of four values (the caller has clamped or wants the wrap).
template <typename T> __device__ __forceinline__ void store4(T *p, const int32_t (&v)[4]);
template <> __device__ __forceinline__ void store4<int8_t>(int8_t *p, const int32_t (&v)[4]) {
    *reinterpret_cast<uint32_t *>(p) = uint32_t(uint8_t(v[0])) | (uint32_t(uint8_t(v[1])) << 8) |
                                       (uint32_t(uint8_t(v[2])) << 16) | (uint32_t(uint8_t(v[3])) << 24);
}
template <> __device__ __forceinline__ void store4<int16_t>(int16_t *p, const int32_t (&v)[4]) {
    *reinterpret_cast<uint2 *>(p) = make_uint2(uint32_t(uint16_t(v[0])) | (uint32_t(uint16_t(v[1])) << 16),
                                               uint32_t(uint16_t(v[2])) | (uint32_t(uint16_t(v[3])) << 16));
}
template <> __device__ __forceinline__ void store4<int32_t>(int32_t *p, const int32_t (&v)[4]) {
    *reinterpret_cast<int4 *>(p) = make_int4(v[0], v[1], v[2], v[3]);
}

template <typename T> __host__ __device__ constexpr int32_t lowestOf() {
    return sizeof(T) == 1 ? -128 : (sizeof(T) == 2 ? -32768 : int32_t(0x80000000u));
}
template <typename T> __host__ __device__ constexpr int32_t highestOf() {
    return sizeof(T) == 1 ? 127 : (sizeof(T) == 2 ? 32767 : 0x7fffffff);
}

// ---- RESCALE (rescale.comp:27-72) -------------------------------------------------------------------------
// A thread handles Q groups of four consecutive elements so that it writes 16 bytes at once (Q = 4 for int8
// results, 2 for int16, 1 for int32): all of its loads are issued before the first result is computed.  Groups
// past the last whole block of 4 Q elements are handled four elements at a time by the threads after it.
template <typename IN, typename OUT> struct RescaleBlock {
    static constexpr int Q = 4 / int(sizeof(OUT)) > 0 ? 4 / int(sizeof(OUT)) : 1;
};

template <typename IN, typename OUT>
__device__ __forceinline__ void rescaleFour(const int32_t (&v)[4], int32_t (&r)[4], FastRescale f, const int32_t *mult,
                                            const int8_t *shift, int perChannel, int c0, int32_t inZp, int32_t outZp,
                                            int doubleRound) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (perChannel) {
            f = makeFastRescale(__ldg(mult + c0 + k), int32_t(__ldg(shift + c0 + k)), inZp, doubleRound != 0);
        }
        r[k] = fastRescale(f, v[k], outZp, lowestOf<OUT>(), highestOf<OUT>());
    }
}

template <typename IN, typename OUT>
__global__ void rescaleVecKernel(const IN *__restrict__ in, OUT *__restrict__ out, int64_t blocks, int64_t tailGroups,
                                 const int32_t *__restrict__ mult, const int8_t *__restrict__ shift, int perChannel, int C,
                                 int32_t inZp, int32_t outZp, int doubleRound) {
    constexpr int Q = RescaleBlock<IN, OUT>::Q;
    const FastRescale f = makeFastRescale(__ldg(mult), int32_t(__ldg(shift)), inZp, doubleRound != 0);
    GRID_STRIDE(g, blocks + tailGroups) {
        if (g < blocks) {
            const int64_t e0 = g * (4 * Q);
            int32_t v[Q][4], r[Q][4];
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                load4<IN>(in + e0 + 4 * q, v[q]);
            }
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                // C is a multiple of 4 when the parameters are per channel: a group of four never wraps
                const int c0 = perChannel ? int((e0 + 4 * q) % C) : 0;
                rescaleFour<IN, OUT>(v[q], r[q], f, mult, shift, perChannel, c0, inZp, outZp, doubleRound);
            }
            if (Q == 4) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    w[q] = uint32_t(uint8_t(r[q][0])) | (uint32_t(uint8_t(r[q][1])) << 8) | (uint32_t(uint8_t(r[q][2])) << 16) |
                           (uint32_t(uint8_t(r[q][3])) << 24);
                }
                *reinterpret_cast<uint4 *>(out + e0) = make_uint4(w[0], w[1], w[2], w[3]);
            } else if (Q == 2) {
                *reinterpret_cast<uint4 *>(out + e0) =
                    make_uint4(uint32_t(uint16_t(r[0][0])) | (uint32_t(uint16_t(r[0][1])) << 16),
                               uint32_t(uint16_t(r[0][2])) | (uint32_t(uint16_t(r[0][3])) << 16),
                               uint32_t(uint16_t(r[Q - 1][0])) | (uint32_t(uint16_t(r[Q - 1][1])) << 16),
                               uint32_t(uint16_t(r[Q - 1][2])) | (uint32_t(uint16_t(r[Q - 1][3])) << 16));
            } else {
                store4<OUT>(out + e0, r[0]);
            }
        } else {
            const int64_t e0 = blocks * (4 * Q) + (g - blocks) * 4;
            int32_t v[4], r[4];
            load4<IN>(in + e0, v);
            rescaleFour<IN, OUT>(v, r, f, mult, shift, perChannel, perChannel ? int(e0 % C) : 0, inZp, outZp, doubleRound);
            store4<OUT>(out + e0, r);
        }
    }
}

template <typename IN, typename OUT>
void launchRescale(const TView &in, const TView &out, const TView &mult, const TView &shift, const RescaleAttr &a,
                   int64_t n, cudaStream_t s) {
    constexpr int Q = RescaleBlock<IN, OUT>::Q;
    const int C = int(out.dims[out.rank - 1]);
    const int64_t blocks = n / (4 * Q), tailGroups = (n - blocks * 4 * Q) / 4;
    rescaleVecKernel<IN, OUT><<<gridFor(blocks + tailGroups, kThreads, 16), kThreads, 0, s>>>(
        reinterpret_cast<const IN *>(in.ptr), reinterpret_cast<OUT *>(out.ptr), blocks, tailGroups,
        reinterpret_cast<const int32_t *>(mult.ptr), reinterpret_cast<const int8_t *>(shift.ptr), a.perChannel ? 1 : 0, C,
        int32_t(wrapTo(in.dtype, a.inZp)), int32_t(wrapTo(out.dtype, a.outZp)), (a.scale32 && a.doubleRound) ? 1 : 0);
}

// ---- TABLE (table.comp:17-52) -------------------------------------------------------------------------------
__global__ void tableI8Kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t groups,
                              const int8_t *__restrict__ table) {
    __shared__ int8_t lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        lut[i] = table[i];
    }
    __syncthreads();
    GRID_STRIDE(g, groups) {
        const int4 w = *reinterpret_cast<const int4 *>(in + 16 * g);
        const uint32_t words[4] = {uint32_t(w.x), uint32_t(w.y), uint32_t(w.z), uint32_t(w.w)};
        uint32_t res[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t r = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = int(int8_t(words[q] >> (8 * k))) + 128;
                r |= uint32_t(uint8_t(lut[idx])) << (8 * k);
            }
            res[q] = r;
        }
        *reinterpret_cast<int4 *>(out + 16 * g) = make_int4(int(res[0]), int(res[1]), int(res[2]), int(res[3]));
    }
}

__global__ void tableI16Kernel(const int16_t *__restrict__ in, int32_t *__restrict__ out, int64_t groups,
                               const int16_t *__restrict__ table) {
    __shared__ int16_t lut[513];
    for (int i = threadIdx.x; i < 513; i += blockDim.x) {
        lut[i] = table[i];
    }
    __syncthreads();
    GRID_STRIDE(g, groups) {
        int32_t v[4], r[4];
        load4<int16_t>(in + 4 * g, v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int32_t index = (v[k] + 32768) >> 7;
            const int32_t fraction = v[k] & 0x7f;
            const int32_t base = lut[index], next = lut[index + 1];
            r[k] = int32_t((uint32_t(base) << 7) + uint32_t(next - base) * uint32_t(fraction));
        }
        store4<int32_t>(out + 4 * g, r);
    }
}

// ---- ADD / SUB / MUL on int32 (elementwise_binary.comp:146-173, mul.comp:24-59) ---------------------------------
// B_MODE: 0 = same shape, 1 = one value per row of `rowLen` elements, 2 = one value.
enum { kVecAdd = 0, kVecSub = 1, kVecMul = 2 };
template <int OP, int B_MODE>
__global__ void binaryI32Kernel(const int32_t *__restrict__ a, const int32_t *__restrict__ b, int32_t *__restrict__ out,
                                int64_t groups, int rowLen, uint32_t shift) {
    GRID_STRIDE(g, groups) {
        int32_t x[4], y[4], r[4];
        load4<int32_t>(a + 4 * g, x);
        if (B_MODE == 0) {
            load4<int32_t>(b + 4 * g, y);
        } else {
            const int32_t v = __ldg(b + (B_MODE == 1 ? (4 * g) / rowLen : 0));
            y[0] = y[1] = y[2] = y[3] = v;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (OP == kVecAdd) {
                r[k] = int32_t(uint32_t(x[k]) + uint32_t(y[k]));
            } else if (OP == kVecSub) {
                r[k] = int32_t(uint32_t(x[k]) - uint32_t(y[k]));
            } else {
                int64_t p = int64_t(x[k]) * int64_t(y[k]);
                if (shift > 0) {
                    p = int64_t(uint64_t(p) + (1ull << ((shift - 1) & 63))) >> (shift & 63);
                }
                r[k] = int32_t(uint32_t(uint64_t(p)));
            }
        }
        store4<int32_t>(out + 4 * g, r);
    }
}

template <int OP>
void launchBinary(const int32_t *a, const int32_t *b, int32_t *out, int64_t n, int mode, int rowLen, uint32_t shift,
                  cudaStream_t s) {
    const int grid = gridFor(n / 4, kThreads, 16);
    if (mode == 0) {
        binaryI32Kernel<OP, 0><<<grid, kThreads, 0, s>>>(a, b, out, n / 4, rowLen, shift);
    } else if (mode == 1) {
        binaryI32Kernel<OP, 1><<<grid, kThreads, 0, s>>>(a, b, out, n / 4, rowLen, shift);
    } else {
        binaryI32Kernel<OP, 2><<<grid, kThreads, 0, s>>>(a, b, out, n / 4, rowLen, shift);
    }
}

// ---- CLAMP on int8 (clamp.comp:24-53) -----------------------------------------------------------------------
__global__ void clampI8Kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t groups, int lo, int hi) {
    GRID_STRIDE(g, groups) {
        const int4 w = *reinterpret_cast<const int4 *>(in + 16 * g);
        const uint32_t words[4] = {uint32_t(w.x), uint32_t(w.y), uint32_t(w.z), uint32_t(w.w)};
        uint32_t res[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t r = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int v = int(int8_t(words[q] >> (8 * k)));
                r |= uint32_t(uint8_t(min(max(v, lo), hi))) << (8 * k);
            }
            res[q] = r;
        }
        *reinterpret_cast<int4 *>(out + 16 * g) = make_int4(int(res[0]), int(res[1]), int(res[2]), int(res[3]));
    }
}

// ---- fused rows of a quantised softmax ---------------------------------------------------------------------------
// Element access of the two fused kernels below: 16-byte vectors where the tensors allow it, single elements where
// an application tensor sits at an odd address.
template <bool VEC> __device__ __forceinline__ void loadFourI32(const int32_t *p, int32_t (&v)[4]) {
    if (VEC) {
        load4<int32_t>(p, v);
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[k] = p[k];
        }
    }
}
template <bool VEC, typename T> __device__ __forceinline__ void storeFour(T *p, const int32_t (&v)[4]) {
    if (VEC) {
        store4<T>(p, v);
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            p[k] = T(v[k]);
        }
    }
}

// REDUCE_MAX(x) -> SUB(x, max) -> RESCALE (to int16) -> TABLE (int16 -> int32), and REDUCE_SUM of the TABLE's output
// (reduce.comp:24-70, elementwise_binary.comp:146-173, rescale.comp:27-72, table.comp): one warp per row, the row read
// twice (the second time from cache), every step with the arithmetic of the operator's own kernel above.
template <bool VEC>
__global__ void rowExpKernel(const int32_t *__restrict__ x, int32_t *__restrict__ e, int32_t *__restrict__ sums, int64_t rows,
                             int len, const int16_t *__restrict__ table, DevRescale r) {
    __shared__ int16_t lut[513];
    for (int i = threadIdx.x; i < 513; i += blockDim.x) {
        lut[i] = table[i];
    }
    __syncthreads();
    const FastRescale f = makeFastRescale(__ldg(r.mult), int32_t(__ldg(r.shift)), r.inZp, r.doubleRound != 0);
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t row = warp; row < rows; row += warps) {
        const int32_t *src = x + row * len;
        int32_t *dst = e + row * len;
        int32_t top = lowestOf<int32_t>();
        for (int i = lane * 4; i < len; i += 128) {
            int32_t v[4];
            loadFourI32<VEC>(src + i, v);
            top = max(max(top, v[0]), max(v[1], max(v[2], v[3])));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            top = max(top, __shfl_xor_sync(0xffffffffu, top, d));
        }
        int32_t acc = 0;
        for (int i = lane * 4; i < len; i += 128) {
            int32_t v[4], out[4];
            loadFourI32<VEC>(src + i, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int32_t diff = int32_t(uint32_t(v[k]) - uint32_t(top));
                const int32_t q = fastRescale(f, diff, r.outZp, r.lo, r.hi); // an int16 value
                const int32_t index = (q + 32768) >> 7;
                const int32_t fraction = q & 0x7f;
                const int32_t base = lut[index], next = lut[index + 1];
                out[k] = int32_t((uint32_t(base) << 7) + uint32_t(next - base) * uint32_t(fraction));
                acc = int32_t(uint32_t(acc) + uint32_t(out[k]));
            }
            storeFour<VEC, int32_t>(dst + i, out);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            acc = int32_t(uint32_t(acc) + uint32_t(__shfl_xor_sync(0xffffffffu, acc, d)));
        }
        if (lane == 0) {
            sums[row] = acc;
        }
    }
}

// MUL(a, b, shift) -> RESCALE [-> CLAMP] (mul.comp:24-59, rescale.comp:27-72).  B_MODE as in binaryI32Kernel.
template <typename OUT, int B_MODE, bool VEC>
__global__ void mulRescaleKernel(const int32_t *__restrict__ a, const int32_t *__restrict__ b, OUT *__restrict__ out,
                                 int64_t groups, int rowLen, uint32_t shift, DevRescale r) {
    const FastRescale f = makeFastRescale(__ldg(r.mult), int32_t(__ldg(r.shift)), r.inZp, r.doubleRound != 0);
    GRID_STRIDE(g, groups) {
        int32_t x[4], y[4], res[4];
        loadFourI32<VEC>(a + 4 * g, x);
        if (B_MODE == 0) {
            loadFourI32<VEC>(b + 4 * g, y);
        } else {
            const int32_t v = __ldg(b + (B_MODE == 1 ? (4 * g) / rowLen : 0));
            y[0] = y[1] = y[2] = y[3] = v;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int64_t p = int64_t(x[k]) * int64_t(y[k]);
            if (shift > 0) {
                p = int64_t(uint64_t(p) + (1ull << ((shift - 1) & 63))) >> (shift & 63);
            }
            res[k] = fastRescale(f, int32_t(uint32_t(uint64_t(p))), r.outZp, r.lo, r.hi);
        }
        storeFour<VEC, OUT>(out + 4 * g, res);
    }
}

// ---- REDUCE_SUM / MAX / MIN along the last axis (reduce.comp:24-70) ------------------------------------------
// One warp per row: lanes stride through the row four elements at a time, then combine with shuffles.  Integer
// addition wraps, so the order of the partial sums does not change the result.
template <typename T, int OP>
__global__ void rowReduceKernel(const T *__restrict__ in, T *__restrict__ out, int64_t rows, int len) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t row = warp; row < rows; row += warps) {
        const T *src = in + row * len;
        int32_t acc = OP == RED_SUM ? 0 : (OP == RED_MAX ? lowestOf<T>() : highestOf<T>());
        for (int i = lane * 4; i < len; i += 128) {
            int32_t v[4];
            load4<T>(src + i, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (OP == RED_SUM) {
                    acc = int32_t(uint32_t(acc) + uint32_t(v[k]));
                } else if (OP == RED_MAX) {
                    acc = max(acc, v[k]);
                } else {
                    acc = min(acc, v[k]);
                }
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const int32_t o = __shfl_xor_sync(0xffffffffu, acc, d);
            if (OP == RED_SUM) {
                acc = int32_t(uint32_t(acc) + uint32_t(o));
            } else if (OP == RED_MAX) {
                acc = max(acc, o);
            } else {
                acc = min(acc, o);
            }
        }
        if (lane == 0) {
            out[row] = T(acc); // a sum of T keeps T's low bits: the generic kernel wraps to the type after every step
        }
    }
}

template <typename T> void launchRowReduce(int32_t op, const TView &in, const TView &out, int64_t rows, int len, cudaStream_t s) {
    const int grid = gridFor(rows * 32, kThreads, 16);
    const T *pi = reinterpret_cast<const T *>(in.ptr);
    T *po = reinterpret_cast<T *>(out.ptr);
    if (op == RED_SUM) {
        rowReduceKernel<T, RED_SUM><<<grid, kThreads, 0, s>>>(pi, po, rows, len);
    } else if (op == RED_MAX) {
        rowReduceKernel<T, RED_MAX><<<grid, kThreads, 0, s>>>(pi, po, rows, len);
    } else {
        rowReduceKernel<T, RED_MIN><<<grid, kThreads, 0, s>>>(pi, po, rows, len);
    }
}

// ---- TRANSPOSE that keeps the last axis (transpose.comp:19-32) -------------------------------------------------
// Rows of the last axis move as wholes: a thread copies 16 bytes; only the row index is permuted.  The index is
// taken apart with multiply-high divisions by constants made on the host (a 64-bit division per axis and thread was
// most of this kernel's time).
struct RowPermute {
    FastDiv outDims[kMaxRank];  // output dims without the last axis
    int64_t inStride[kMaxRank]; // input byte stride of the axis each output axis comes from
    FastDiv chunksPerRow;
    int rank;                   // number of outer axes
};

__device__ __forceinline__ uint32_t divBy(uint32_t n, const FastDiv &f) { return f.mul == 0u ? n : __umulhi(n, f.mul) >> f.shift; }

__global__ void transposeRowsKernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int64_t chunks, RowPermute p) {
    GRID_STRIDE(e, chunks) { // the launcher refuses 2^31 chunks and more
        uint32_t row = divBy(uint32_t(e), p.chunksPerRow);
        const uint32_t chunk = uint32_t(e) - row * p.chunksPerRow.d;
        int64_t src = 0;
#pragma unroll
        for (int i = kMaxRank - 1; i >= 0; --i) {
            if (i < p.rank) {
                const uint32_t q = divBy(row, p.outDims[i]);
                src += int64_t(row - q * p.outDims[i].d) * p.inStride[i];
                row = q;
            }
        }
        *reinterpret_cast<int4 *>(out + 16 * e) = __ldg(reinterpret_cast<const int4 *>(in + src + 16 * int64_t(chunk)));
    }
}

// ---- TRANSPOSE that swaps the last axis with another one, one-byte elements ------------------------------------
// out[..., c, r] = in[..., r (axis p), ..., c (last axis)]: per combination of the other axes a 2-D transpose of
// an R x Ccols byte matrix whose rows are `inRowStride` bytes apart.  No shared memory: a lane reads 8 rows x 16
// bytes (neighbouring lanes take the two halves of a 32-byte sector), transposes the eight 4 x 4 byte blocks in
// registers with byte permutes, and writes 16 double words, one to each of 16 output rows; the lanes of a warp
// that share a column half hold consecutive row octets, so every such store of the warp is two runs of 128
// contiguous bytes.
struct BatchPermute {
    FastDiv outDims[kMaxRank];  // output dims of the outer axes (all but the last two)
    int64_t inStride[kMaxRank]; // input byte stride of the axis each of them comes from
    FastDiv perBatch;           // warps per matrix
    FastDiv colGroups;          // 32-column groups per matrix
    int rank;
};

__global__ void __launch_bounds__(256) transposeLast2BytesKernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out,
                                                                 int R, int Ccols, int64_t inRowStride, int64_t warps,
                                                                 BatchPermute p) {
    const int lane = threadIdx.x & 31;
    for (int64_t wid = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wid < warps;
         wid += (int64_t(gridDim.x) * blockDim.x) >> 5) {
        uint32_t batch = divBy(uint32_t(wid), p.perBatch);
        const uint32_t inMat = uint32_t(wid) - batch * p.perBatch.d;
        const uint32_t rowGroup = divBy(inMat, p.colGroups);
        const int c0 = int(inMat - rowGroup * p.colGroups.d) * 32 + (lane & 1) * 16;
        const int r = (int(rowGroup) * 16 + (lane >> 1)) * 8;
        uint8_t *dst = out + int64_t(batch) * R * Ccols;
        int64_t src = 0;
#pragma unroll
        for (int i = kMaxRank - 1; i >= 0; --i) {
            if (i < p.rank) {
                const uint32_t q = divBy(batch, p.outDims[i]);
                src += int64_t(batch - q * p.outDims[i].d) * p.inStride[i];
                batch = q;
            }
        }
        if (r >= R || c0 >= Ccols) { // R is a multiple of 8 and Ccols of 16: a block is inside or outside as a whole
            continue;
        }
        uint32_t w[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int4 v = __ldg(reinterpret_cast<const int4 *>(in + src + int64_t(r + i) * inRowStride + c0));
            w[i][0] = uint32_t(v.x), w[i][1] = uint32_t(v.y), w[i][2] = uint32_t(v.z), w[i][3] = uint32_t(v.w);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            // rows r .. r+7, columns c0 + 4g .. +3  ->  output rows c0 + 4g + k, bytes r .. r+7
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t t0 = __byte_perm(w[4 * h][g], w[4 * h + 1][g], 0x5140);
                const uint32_t t1 = __byte_perm(w[4 * h + 2][g], w[4 * h + 3][g], 0x5140);
                const uint32_t t2 = __byte_perm(w[4 * h][g], w[4 * h + 1][g], 0x7362);
                const uint32_t t3 = __byte_perm(w[4 * h + 2][g], w[4 * h + 3][g], 0x7362);
                uint32_t *o = h == 0 ? lo : hi;
                o[0] = __byte_perm(t0, t1, 0x5410), o[1] = __byte_perm(t0, t1, 0x7632);
                o[2] = __byte_perm(t2, t3, 0x5410), o[3] = __byte_perm(t2, t3, 0x7632);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                *reinterpret_cast<uint2 *>(dst + int64_t(c0 + 4 * g + k) * R + r) = make_uint2(lo[k], hi[k]);
            }
        }
    }
}

} // namespace

bool vecRescale(const TView &in, const TView &out, const TView &mult, const TView &shift, const RescaleAttr &a, cudaStream_t s,
                int *rc) {
    const int64_t n = packedNumel(in);
    if (n <= 0 || n != packedNumel(out) || n % 4 != 0 || !sameShape(in, out) || !signedInt(in.dtype) || !signedInt(out.dtype) ||
        !aligned16(in.ptr) || !aligned16(out.ptr) || mult.dtype != MLEL_I32 || shift.dtype != MLEL_I8 ||
        packedNumel(mult) < 1 || packedNumel(shift) < 1 || n >= (int64_t(1) << 40)) {
        return false;
    }
    const int64_t C = out.dims[out.rank - 1];
    if (a.perChannel && (C % 4 != 0 || packedNumel(mult) != C || packedNumel(shift) != C)) {
        return false;
    }
#define MLEL_RESCALE_CASE(IN_ID, IN_T, OUT_ID, OUT_T)                                                                          \
    if (in.dtype == IN_ID && out.dtype == OUT_ID) {                                                                            \
        launchRescale<IN_T, OUT_T>(in, out, mult, shift, a, n, s);                                                             \
        *rc = finish("RESCALE");                                                                                               \
        return true;                                                                                                           \
    }
    MLEL_RESCALE_CASE(MLEL_I32, int32_t, MLEL_I8, int8_t)
    MLEL_RESCALE_CASE(MLEL_I32, int32_t, MLEL_I16, int16_t)
    MLEL_RESCALE_CASE(MLEL_I32, int32_t, MLEL_I32, int32_t)
    MLEL_RESCALE_CASE(MLEL_I8, int8_t, MLEL_I32, int32_t)
    MLEL_RESCALE_CASE(MLEL_I8, int8_t, MLEL_I8, int8_t)
    MLEL_RESCALE_CASE(MLEL_I16, int16_t, MLEL_I32, int32_t)
    MLEL_RESCALE_CASE(MLEL_I16, int16_t, MLEL_I16, int16_t)
    MLEL_RESCALE_CASE(MLEL_I16, int16_t, MLEL_I8, int8_t)
    MLEL_RESCALE_CASE(MLEL_I8, int8_t, MLEL_I16, int16_t)
#undef MLEL_RESCALE_CASE
    return false;
}

bool vecTable(const TView &in, const TView &out, const TView &table, cudaStream_t s, int *rc) {
    const int64_t n = packedNumel(in);
    if (n <= 0 || n != packedNumel(out) || !sameShape(in, out) || !aligned16(in.ptr) || !aligned16(out.ptr) ||
        packedNumel(table) < 0) {
        return false;
    }
    if (in.dtype == MLEL_I8 && out.dtype == MLEL_I8 && table.dtype == MLEL_I8 && packedNumel(table) == 256 && n % 16 == 0) {
        tableI8Kernel<<<gridFor(n / 16, kThreads, 16), kThreads, 0, s>>>(reinterpret_cast<const int8_t *>(in.ptr),
                                                                         reinterpret_cast<int8_t *>(out.ptr), n / 16,
                                                                         reinterpret_cast<const int8_t *>(table.ptr));
        *rc = finish("TABLE");
        return true;
    }
    if (in.dtype == MLEL_I16 && out.dtype == MLEL_I32 && table.dtype == MLEL_I16 && packedNumel(table) == 513 && n % 4 == 0) {
        tableI16Kernel<<<gridFor(n / 4, kThreads, 16), kThreads, 0, s>>>(reinterpret_cast<const int16_t *>(in.ptr),
                                                                        reinterpret_cast<int32_t *>(out.ptr), n / 4,
                                                                        reinterpret_cast<const int16_t *>(table.ptr));
        *rc = finish("TABLE");
        return true;
    }
    return false;
}

// op: BIN_ADD or BIN_SUB of ops.hpp, or -1 for MUL with `shift`.
bool vecBinaryI32(int32_t op, const TView &a, const TView &b, const TView &out, uint32_t shift, cudaStream_t s, int *rc) {
    const int64_t n = packedNumel(out);
    if (n <= 0 || n % 4 != 0 || a.dtype != MLEL_I32 || b.dtype != MLEL_I32 || out.dtype != MLEL_I32 || packedNumel(a) != n ||
        !sameShape(a, out) || packedNumel(b) < 1 || !aligned16(a.ptr) || !aligned16(out.ptr) || shift > 62) {
        return false;
    }
    const int rowLen = int(out.dims[out.rank - 1]);
    int mode;
    if (sameShape(b, out)) {
        mode = 0;
        if (!aligned16(b.ptr)) {
            return false;
        }
    } else if (packedNumel(b) == 1 && b.rank == out.rank) {
        mode = 2;
    } else if (rowBroadcast(b, out) && rowLen % 4 == 0) {
        mode = 1;
    } else {
        return false;
    }
    const auto *pa = reinterpret_cast<const int32_t *>(a.ptr), *pb = reinterpret_cast<const int32_t *>(b.ptr);
    auto *po = reinterpret_cast<int32_t *>(out.ptr);
    if (op == BIN_ADD) {
        launchBinary<kVecAdd>(pa, pb, po, n, mode, rowLen, 0, s);
    } else if (op == BIN_SUB) {
        launchBinary<kVecSub>(pa, pb, po, n, mode, rowLen, 0, s);
    } else if (op == -1) {
        launchBinary<kVecMul>(pa, pb, po, n, mode, rowLen, shift, s);
    } else {
        return false;
    }
    *rc = finish("element-wise int32");
    return true;
}

bool vecClampI8(const TView &in, const TView &out, int64_t lo, int64_t hi, cudaStream_t s, int *rc) {
    const int64_t n = packedNumel(in);
    if (n <= 0 || n % 16 != 0 || n != packedNumel(out) || !sameShape(in, out) || in.dtype != MLEL_I8 || out.dtype != MLEL_I8 ||
        !aligned16(in.ptr) || !aligned16(out.ptr)) {
        return false;
    }
    clampI8Kernel<<<gridFor(n / 16, kThreads, 16), kThreads, 0, s>>>(reinterpret_cast<const int8_t *>(in.ptr),
                                                                     reinterpret_cast<int8_t *>(out.ptr), n / 16, int(lo), int(hi));
    *rc = finish("CLAMP");
    return true;
}

bool vecRowReduce(int32_t op, const TView &in, const TView &out, uint32_t axis, cudaStream_t s, int *rc) {
    const int64_t n = packedNumel(in), rows = packedNumel(out);
    if (n <= 0 || rows <= 0 || in.rank < 1 || int(axis) != in.rank - 1 || out.rank != in.rank || out.dims[axis] != 1 ||
        in.dtype != out.dtype || !signedInt(in.dtype) || (op != RED_SUM && op != RED_MAX && op != RED_MIN) ||
        !aligned16(in.ptr)) {
        return false;
    }
    const int64_t len = in.dims[axis];
    if (len % 4 != 0 || len > (1 << 30) || rows * len != n || (len * dtypeSize(in.dtype)) % 16 != 0) {
        return false;
    }
    if (in.dtype == MLEL_I32) {
        launchRowReduce<int32_t>(op, in, out, rows, int(len), s);
    } else if (in.dtype == MLEL_I16) {
        launchRowReduce<int16_t>(op, in, out, rows, int(len), s);
    } else {
        launchRowReduce<int8_t>(op, in, out, rows, int(len), s);
    }
    *rc = finish("REDUCE");
    return true;
}

bool vecTransposeRows(const TView &in, const TView &out, const uint32_t *perms, cudaStream_t s, int *rc) {
    const int64_t n = packedNumel(in);
    const int rank = out.rank;
    if (n <= 0 || n != packedNumel(out) || rank < 2 || in.rank != rank || in.dtype != out.dtype ||
        int(perms[rank - 1]) != rank - 1 || !aligned16(in.ptr) || !aligned16(out.ptr)) {
        return false;
    }
    const int64_t rowBytes = int64_t(out.dims[rank - 1]) * dtypeSize(out.dtype);
    if (rowBytes % 16 != 0 || rowBytes / 16 > (1 << 24)) {
        return false;
    }
    const int64_t chunks = n * dtypeSize(out.dtype) / 16;
    if (chunks >= (int64_t(1) << 31)) {
        return false;
    }
    RowPermute p{};
    p.rank = rank - 1;
    p.chunksPerRow = makeFastDiv(rowBytes / 16);
    for (int i = 0; i < rank - 1; ++i) {
        if (perms[i] >= uint32_t(rank - 1) || in.dims[perms[i]] != out.dims[i]) {
            return false;
        }
        p.outDims[i] = makeFastDiv(out.dims[i]);
        p.inStride[i] = in.strides[perms[i]];
    }
    transposeRowsKernel<<<gridFor(chunks, kThreads, 16), kThreads, 0, s>>>(reinterpret_cast<const uint8_t *>(in.ptr),
                                                                          reinterpret_cast<uint8_t *>(out.ptr), chunks, p);
    *rc = finish("TRANSPOSE");
    return true;
}

bool vecTransposeLast2Bytes(const TView &in, const TView &out, const uint32_t *perms, cudaStream_t s, int *rc) {
    const int64_t n = packedNumel(in);
    const int rank = out.rank;
    if (n <= 0 || n != packedNumel(out) || rank < 2 || in.rank != rank || in.dtype != out.dtype || dtypeSize(out.dtype) != 1 ||
        int(perms[rank - 2]) != rank - 1 || int(perms[rank - 1]) == rank - 1 || !aligned16(in.ptr) || !aligned16(out.ptr)) {
        return false;
    }
    const uint32_t pAxis = perms[rank - 1];
    const int64_t R = in.dims[pAxis], Ccols = in.dims[rank - 1];
    const int64_t inRowStride = in.strides[pAxis];
    if (R % 8 != 0 || Ccols % 16 != 0 || inRowStride % 16 != 0 || out.dims[rank - 1] != R || out.dims[rank - 2] != Ccols) {
        return false;
    }
    BatchPermute p{};
    p.rank = rank - 2;
    int64_t batches = 1;
    for (int i = 0; i < rank - 2; ++i) {
        if (perms[i] >= uint32_t(rank) || perms[i] == pAxis || int(perms[i]) == rank - 1 || in.dims[perms[i]] != out.dims[i]) {
            return false;
        }
        p.outDims[i] = makeFastDiv(out.dims[i]);
        p.inStride[i] = in.strides[perms[i]];
        if (p.inStride[i] % 16 != 0) {
            return false;
        }
        batches *= out.dims[i];
    }
    const int64_t colGroups = (Ccols + 31) / 32, rowGroups = (R + 127) / 128;
    const int64_t warps = batches * colGroups * rowGroups;
    if (warps >= (int64_t(1) << 31)) {
        return false;
    }
    p.perBatch = makeFastDiv(colGroups * rowGroups);
    p.colGroups = makeFastDiv(colGroups);
    transposeLast2BytesKernel<<<gridFor(warps * 32, 256, 8), 256, 0, s>>>(reinterpret_cast<const uint8_t *>(in.ptr),
                                                                        reinterpret_cast<uint8_t *>(out.ptr), int(R),
                                                                        int(Ccols), inRowStride, warps, p);
    *rc = finish("TRANSPOSE");
    return true;
}

namespace {

// out[row][first[g] + j] = staging[g][row][j] for j < count[g]: joins the column blocks that an all-gather left
// one after another (every block padded to `pitch` bytes per row) into rows of `total` bytes.  One thread moves
// 16 bytes when every block starts and ends on a 16-byte boundary (VEC = 16), else one byte.
struct ColumnBlocks {
    int32_t first[kMaxColumnBlocks];
    int32_t count[kMaxColumnBlocks];
};

template <int VEC>
__global__ void interleaveColumnsKernel(const uint8_t *__restrict__ staging, uint8_t *__restrict__ out, int64_t rows,
                                        int32_t blocks, int32_t pitch, int32_t total, ColumnBlocks cb) {
    const int64_t unitsPerRow = total / VEC;
    GRID_STRIDE(e, rows * unitsPerRow) {
        const int64_t row = e / unitsPerRow;
        const int32_t col = int32_t(e - row * unitsPerRow) * VEC;
        int g = 0;
        while (g + 1 < blocks && col >= cb.first[g + 1]) {
            ++g;
        }
        const uint8_t *src = staging + (int64_t(g) * rows + row) * pitch + (col - cb.first[g]);
        uint8_t *dst = out + row * int64_t(total) + col;
        if (VEC == 16) {
            *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
        } else {
            *dst = *src;
        }
    }
}

} // namespace

int interleaveColumns(const void *staging, void *out, int64_t rows, int32_t blocks, int32_t pitch, const int32_t *first,
                      const int32_t *count, cudaStream_t s) {
    if (blocks < 1 || blocks > kMaxColumnBlocks || rows < 0 || pitch < 0) {
        setLastError("interleave columns: bad block description");
        return MLEL_ERROR_UNKNOWN;
    }
    ColumnBlocks cb{};
    int64_t total = 0;
    bool vec = (reinterpret_cast<uintptr_t>(staging) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
               pitch % 16 == 0;
    for (int g = 0; g < blocks; ++g) {
        if (first[g] != total || count[g] < 0 || count[g] > pitch) {
            setLastError("interleave columns: blocks must follow one another and fit the pitch");
            return MLEL_ERROR_UNKNOWN;
        }
        cb.first[g] = first[g], cb.count[g] = count[g];
        total += count[g];
        vec = vec && first[g] % 16 == 0 && count[g] % 16 == 0;
    }
    if (total == 0 || rows == 0) {
        return MLEL_SUCCESS;
    }
    if (total >= (int64_t(1) << 31)) {
        setLastError("interleave columns: rows too long");
        return MLEL_ERROR_UNKNOWN;
    }
    const int64_t units = rows * (total / (vec ? 16 : 1));
    const int grid = int(std::min<int64_t>((units + 255) / 256, int64_t(kNumSMs) * 16));
    if (vec) {
        interleaveColumnsKernel<16><<<grid, 256, 0, s>>>(static_cast<const uint8_t *>(staging), static_cast<uint8_t *>(out),
                                                         rows, blocks, pitch, int32_t(total), cb);
    } else {
        interleaveColumnsKernel<1><<<grid, 256, 0, s>>>(static_cast<const uint8_t *>(staging), static_cast<uint8_t *>(out),
                                                        rows, blocks, pitch, int32_t(total), cb);
    }
    return finish("interleave columns");
}


int rowExpFused(const TView &x, const TView &table, const TView &e, const TView &sums, const DevRescale &r, cudaStream_t s) {
    const int len = int(x.dims[x.rank - 1]);
    const int64_t n = packedNumel(x);
    if (n <= 0 || len <= 0 || len % 4 != 0 || packedNumel(e) != n || packedNumel(sums) != n / len || packedNumel(table) != 513) {
        setLastError("fused softmax rows: operands do not match");
        return MLEL_ERROR_UNKNOWN;
    }
    const int64_t rows = n / len;
    const int grid = gridFor(rows * 32, kThreads, 16);
    const auto *px = reinterpret_cast<const int32_t *>(x.ptr);
    auto *pe = reinterpret_cast<int32_t *>(e.ptr);
    auto *ps = reinterpret_cast<int32_t *>(sums.ptr);
    const auto *pt = reinterpret_cast<const int16_t *>(table.ptr);
    if (aligned16(x.ptr) && aligned16(e.ptr)) {
        rowExpKernel<true><<<grid, kThreads, 0, s>>>(px, pe, ps, rows, len, pt, r);
    } else {
        rowExpKernel<false><<<grid, kThreads, 0, s>>>(px, pe, ps, rows, len, pt, r);
    }
    return finish("REDUCE_MAX+SUB+RESCALE+TABLE+REDUCE_SUM");
}

namespace {
template <typename OUT>
void launchMulRescale(const TView &a, const TView &b, const TView &out, int64_t n, int mode, int rowLen, uint32_t shift,
                      const DevRescale &r, cudaStream_t s) {
    const int grid = gridFor(n / 4, kThreads, 16);
    const auto *pa = reinterpret_cast<const int32_t *>(a.ptr);
    const auto *pb = reinterpret_cast<const int32_t *>(b.ptr);
    auto *po = reinterpret_cast<OUT *>(out.ptr);
    const bool vec = aligned16(a.ptr) && (mode != 0 || aligned16(b.ptr)) &&
                     (reinterpret_cast<uintptr_t>(out.ptr) & (4 * sizeof(OUT) - 1)) == 0;
#define MLEL_MUL_RESCALE(MODE)                                                                                     \
    if (vec) {                                                                                                     \
        mulRescaleKernel<OUT, MODE, true><<<grid, kThreads, 0, s>>>(pa, pb, po, n / 4, rowLen, shift, r);         \
    } else {                                                                                                       \
        mulRescaleKernel<OUT, MODE, false><<<grid, kThreads, 0, s>>>(pa, pb, po, n / 4, rowLen, shift, r);        \
    }
    if (mode == 0) {
        MLEL_MUL_RESCALE(0)
    } else if (mode == 1) {
        MLEL_MUL_RESCALE(1)
    } else {
        MLEL_MUL_RESCALE(2)
    }
#undef MLEL_MUL_RESCALE
}
} // namespace

int mulRescaleFused(const TView &a, const TView &b, const TView &out, uint32_t shift, const DevRescale &r, cudaStream_t s) {
    const int64_t n = packedNumel(a), nb = packedNumel(b);
    const int rowLen = int(a.dims[a.rank - 1]);
    if (n <= 0 || n % 4 != 0 || rowLen % 4 != 0 || packedNumel(out) != n || nb <= 0) {
        setLastError("fused MUL+RESCALE: operands do not match");
        return MLEL_ERROR_UNKNOWN;
    }
    const int mode = nb == n ? 0 : (nb == 1 ? 2 : 1);
    if (mode == 1 && nb != n / rowLen) {
        setLastError("fused MUL+RESCALE: second operand is neither per row nor a single value");
        return MLEL_ERROR_UNKNOWN;
    }
    if (out.dtype == MLEL_I8) {
        launchMulRescale<int8_t>(a, b, out, n, mode, rowLen, shift, r, s);
    } else if (out.dtype == MLEL_I16) {
        launchMulRescale<int16_t>(a, b, out, n, mode, rowLen, shift, r, s);
    } else {
        setLastError("fused MUL+RESCALE: output type");
        return MLEL_ERROR_UNKNOWN;
    }
    return finish("MUL+RESCALE");
}

} // namespace mlel
