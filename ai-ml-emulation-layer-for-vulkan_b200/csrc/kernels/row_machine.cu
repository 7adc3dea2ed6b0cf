// A run of row-wise integer operators as one kernel (OP_FUSED_ROWS, see RowProgram in ops.hpp).
//
// The chains a quantised softmax or layer norm lowers to -- REDUCE_MAX, SUB, RESCALE, TABLE, REDUCE_SUM, MUL, ... on
// tensors of one shape [..., L] and on one value per row -- are memory-bound as separate kernels: each reads and
// writes tensors of the full size.  Here a warp owns a row: full-shaped values live in shared-memory slots (a lane
// only ever touches its own elements of a slot, so no synchronisation is needed between instructions), per-row
// values in a few words beside them, and the instructions run in order.  Every instruction computes exactly what
// the operator's own kernel computes (reduce.comp, elementwise_binary.comp, mul.comp, rescale.comp, table.comp,
// clamp.comp of the reference, as restated in vector_ops.cu and device_common.cuh), so the results are the same bits.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "device_common.cuh"
#include "kernels.hpp"

namespace mlel {

namespace {

struct DevRowInst {
    int32_t op;
    int32_t dstKind, dst;
    int32_t aKind, a, aImm;
    int32_t bKind, b, bImm;
    int32_t dtype;
    const void *ptr;
    int32_t p[7];
    int32_t pad;
};
struct DevRowProgram {
    int32_t count, len, slots, warps;
    DevRowInst inst[kMaxRowInsts];
};
static_assert(sizeof(DevRowProgram) <= 4000, "the program travels as a kernel parameter");

// Four consecutive elements of a row tensor as int32 (sign-extended), and back (narrowing by the type's own wrap:
// every producer of a narrow type has already clamped or wrapped to it).
__device__ __forceinline__ void loadFour(const void *base, int32_t dtype, int64_t index, int32_t (&v)[4]) {
    if (dtype == MLEL_I8) {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(static_cast<const int8_t *>(base) + index);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[k] = int32_t(int8_t(w >> (8 * k)));
        }
    } else if (dtype == MLEL_I16) {
        const uint2 w = *reinterpret_cast<const uint2 *>(static_cast<const int16_t *>(base) + index);
        v[0] = int32_t(int16_t(w.x)), v[1] = int32_t(int16_t(w.x >> 16));
        v[2] = int32_t(int16_t(w.y)), v[3] = int32_t(int16_t(w.y >> 16));
    } else {
        const int4 w = *reinterpret_cast<const int4 *>(static_cast<const int32_t *>(base) + index);
        v[0] = w.x, v[1] = w.y, v[2] = w.z, v[3] = w.w;
    }
}
__device__ __forceinline__ void storeFour(void *base, int32_t dtype, int64_t index, const int32_t (&v)[4]) {
    if (dtype == MLEL_I8) {
        *reinterpret_cast<uint32_t *>(static_cast<int8_t *>(base) + index) =
            uint32_t(uint8_t(v[0])) | (uint32_t(uint8_t(v[1])) << 8) | (uint32_t(uint8_t(v[2])) << 16) |
            (uint32_t(uint8_t(v[3])) << 24);
    } else if (dtype == MLEL_I16) {
        *reinterpret_cast<uint2 *>(static_cast<int16_t *>(base) + index) =
            make_uint2(uint32_t(uint16_t(v[0])) | (uint32_t(uint16_t(v[1])) << 16),
                       uint32_t(uint16_t(v[2])) | (uint32_t(uint16_t(v[3])) << 16));
    } else {
        *reinterpret_cast<int4 *>(static_cast<int32_t *>(base) + index) = make_int4(v[0], v[1], v[2], v[3]);
    }
}
__device__ __forceinline__ int32_t loadOne(const void *base, int32_t dtype, int64_t index) {
    if (dtype == MLEL_I8) {
        return static_cast<const int8_t *>(base)[index];
    }
    if (dtype == MLEL_I16) {
        return static_cast<const int16_t *>(base)[index];
    }
    return static_cast<const int32_t *>(base)[index];
}
__device__ __forceinline__ void storeOne(void *base, int32_t dtype, int64_t index, int32_t v) {
    if (dtype == MLEL_I8) {
        static_cast<int8_t *>(base)[index] = int8_t(v);
    } else if (dtype == MLEL_I16) {
        static_cast<int16_t *>(base)[index] = int16_t(v);
    } else {
        static_cast<int32_t *>(base)[index] = v;
    }
}

// One element of each operator.
__device__ __forceinline__ int32_t table16(const int16_t *lut, int32_t v) {
    const int32_t index = (v + 32768) >> 7;
    const int32_t fraction = v & 0x7f;
    const int32_t base = __ldg(lut + index), next = __ldg(lut + index + 1);
    return int32_t((uint32_t(base) << 7) + uint32_t(next - base) * uint32_t(fraction));
}
__device__ __forceinline__ int32_t mulShift(int32_t x, int32_t y, uint32_t shift) {
    int64_t p = int64_t(x) * int64_t(y);
    if (shift > 0) {
        p = int64_t(uint64_t(p) + (1ull << ((shift - 1) & 63))) >> (shift & 63);
    }
    return int32_t(uint32_t(uint64_t(p)));
}
// Parameters of an element-wise instruction, copied out of the kernel parameter block once per instruction (not
// once per element).
struct ElementParams {
    FastRescale f;
    int32_t outZp, lo, hi; // RESCALE: output zero point and range; CLAMP: lo, hi
    uint32_t shift;        // MUL
    const void *table;
};
template <int OP> __device__ __forceinline__ int32_t elementOf(int32_t x, int32_t y, const ElementParams &e) {
    if (OP == ROW_RESCALE) {
        return fastRescale(e.f, x, e.outZp, e.lo, e.hi);
    } else if (OP == ROW_TABLE8) {
        return int32_t(__ldg(static_cast<const int8_t *>(e.table) + (x + 128)));
    } else if (OP == ROW_TABLE16) {
        return table16(static_cast<const int16_t *>(e.table), x);
    } else if (OP == ROW_ADD) {
        return int32_t(uint32_t(x) + uint32_t(y));
    } else if (OP == ROW_SUB) {
        return int32_t(uint32_t(x) - uint32_t(y));
    } else if (OP == ROW_MUL) {
        return mulShift(x, y, e.shift);
    } else { // ROW_CLAMP
        return min(max(x, e.lo), e.hi);
    }
}
// One element-wise instruction over a lane's elements of a row.  A_FULL / B_FULL: the operand is a slot (else the
// same value xs / ys for every element).
template <int OP, bool A_FULL, bool B_FULL>
__device__ __forceinline__ void elementLoop(int32_t *dst, const int32_t *a, const int32_t *b, int32_t xs, int32_t ys, int len,
                                            int lane, const ElementParams &e) {
    for (int i = lane * 4; i < len; i += 128) {
        int32_t x[4] = {xs, xs, xs, xs}, y[4] = {ys, ys, ys, ys};
        if (A_FULL) {
            const int4 w = *reinterpret_cast<const int4 *>(a + i);
            x[0] = w.x, x[1] = w.y, x[2] = w.z, x[3] = w.w;
        }
        if (B_FULL) {
            const int4 w = *reinterpret_cast<const int4 *>(b + i);
            y[0] = w.x, y[1] = w.y, y[2] = w.z, y[3] = w.w;
        }
        int32_t r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            r[k] = elementOf<OP>(x[k], y[k], e);
        }
        *reinterpret_cast<int4 *>(dst + i) = make_int4(r[0], r[1], r[2], r[3]);
    }
}
template <int OP>
__device__ __forceinline__ void elementInst(int32_t *dst, const int32_t *a, const int32_t *b, bool aFull, bool bFull, int32_t xs,
                                            int32_t ys, int len, int lane, const ElementParams &e) {
    constexpr bool kBinary = OP == ROW_ADD || OP == ROW_SUB || OP == ROW_MUL;
    if (!kBinary) {
        elementLoop<OP, true, false>(dst, a, b, xs, ys, len, lane, e);
    } else if (aFull && bFull) {
        elementLoop<OP, true, true>(dst, a, b, xs, ys, len, lane, e);
    } else if (aFull) {
        elementLoop<OP, true, false>(dst, a, b, xs, ys, len, lane, e);
    } else {
        elementLoop<OP, false, true>(dst, a, b, xs, ys, len, lane, e);
    }
}
__device__ __forceinline__ int32_t elementAny(int op, int32_t x, int32_t y, const ElementParams &e) {
    switch (op) {
    case ROW_RESCALE:
        return elementOf<ROW_RESCALE>(x, y, e);
    case ROW_TABLE8:
        return elementOf<ROW_TABLE8>(x, y, e);
    case ROW_TABLE16:
        return elementOf<ROW_TABLE16>(x, y, e);
    case ROW_ADD:
        return elementOf<ROW_ADD>(x, y, e);
    case ROW_SUB:
        return elementOf<ROW_SUB>(x, y, e);
    case ROW_MUL:
        return elementOf<ROW_MUL>(x, y, e);
    default:
        return elementOf<ROW_CLAMP>(x, y, e);
    }
}

__global__ void __launch_bounds__(256) rowMachineKernel(const __grid_constant__ DevRowProgram prog, int64_t rows) {
    extern __shared__ int32_t rowSmem[];
    const int lane = threadIdx.x & 31, warpInBlock = threadIdx.x >> 5;
    const int len = prog.len;
    int32_t *slots = rowSmem + size_t(warpInBlock) * (size_t(prog.slots) * len + kMaxRowValues);
    int32_t *values = slots + size_t(prog.slots) * len;
    const int64_t warp = int64_t(blockIdx.x) * prog.warps + warpInBlock;
    const int64_t warps = int64_t(gridDim.x) * prog.warps;
    for (int64_t row = warp; row < rows; row += warps) {
        for (int n = 0; n < prog.count; ++n) {
            const DevRowInst &in = prog.inst[n];
            const int op = in.op;
            if (op == ROW_LOAD) {
                if (in.dstKind == ROW_FULL) {
                    for (int i = lane * 4; i < len; i += 128) {
                        int32_t v[4];
                        loadFour(in.ptr, in.dtype, row * len + i, v);
                        *reinterpret_cast<int4 *>(slots + in.dst * len + i) = make_int4(v[0], v[1], v[2], v[3]);
                    }
                } else {
                    __syncwarp();
                    if (lane == 0) {
                        values[in.dst] = loadOne(in.ptr, in.dtype, row);
                    }
                    __syncwarp();
                }
                continue;
            }
            if (op == ROW_STORE) {
                if (in.aKind == ROW_FULL) {
                    for (int i = lane * 4; i < len; i += 128) {
                        const int4 w = *reinterpret_cast<const int4 *>(slots + in.a * len + i);
                        const int32_t v[4] = {w.x, w.y, w.z, w.w};
                        storeFour(const_cast<void *>(in.ptr), in.dtype, row * len + i, v);
                    }
                } else if (lane == 0) {
                    storeOne(const_cast<void *>(in.ptr), in.dtype, row, values[in.a]);
                }
                continue;
            }
            if (op == ROW_REDUCE_SUM || op == ROW_REDUCE_MAX || op == ROW_REDUCE_MIN) {
                int32_t acc = op == ROW_REDUCE_SUM ? 0 : (op == ROW_REDUCE_MAX ? int32_t(0x80000000u) : 0x7fffffff);
                for (int i = lane * 4; i < len; i += 128) {
                    const int4 w = *reinterpret_cast<const int4 *>(slots + in.a * len + i);
                    const int32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        acc = op == ROW_REDUCE_SUM ? int32_t(uint32_t(acc) + uint32_t(v[k]))
                                                   : (op == ROW_REDUCE_MAX ? max(acc, v[k]) : min(acc, v[k]));
                    }
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) {
                    const int32_t o = __shfl_xor_sync(0xffffffffu, acc, d);
                    acc = op == ROW_REDUCE_SUM ? int32_t(uint32_t(acc) + uint32_t(o))
                                               : (op == ROW_REDUCE_MAX ? max(acc, o) : min(acc, o));
                }
                if (lane == 0) {
                    values[in.dst] = acc;
                }
                __syncwarp();
                continue;
            }
            // element-wise operators: one or two operands, each a slot, a per-row value or an immediate
            ElementParams e{};
            if (op == ROW_RESCALE) {
                e.f = makeFastRescale(in.p[0], in.p[1], in.p[2], in.p[6] != 0);
                e.outZp = in.p[3], e.lo = in.p[4], e.hi = in.p[5];
            } else if (op == ROW_CLAMP) {
                e.lo = in.p[0], e.hi = in.p[1];
            }
            e.shift = uint32_t(in.p[0]);
            e.table = in.ptr;
            const int32_t xs = in.aKind == ROW_VALUE ? values[in.a] : in.aImm;
            const int32_t ys = in.bKind == ROW_VALUE ? values[in.b] : in.bImm;
            if (in.dstKind == ROW_FULL) {
                int32_t *dst = slots + in.dst * len;
                const int32_t *a = slots + in.a * len, *b = slots + in.b * len;
                const bool aFull = in.aKind == ROW_FULL, bFull = in.bKind == ROW_FULL;
                switch (op) {
                case ROW_RESCALE:
                    elementInst<ROW_RESCALE>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                case ROW_TABLE8:
                    elementInst<ROW_TABLE8>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                case ROW_TABLE16:
                    elementInst<ROW_TABLE16>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                case ROW_ADD:
                    elementInst<ROW_ADD>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                case ROW_SUB:
                    elementInst<ROW_SUB>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                case ROW_MUL:
                    elementInst<ROW_MUL>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                default:
                    elementInst<ROW_CLAMP>(dst, a, b, aFull, bFull, xs, ys, len, lane, e);
                    break;
                }
            } else {
                const int32_t r = elementAny(op, xs, ys, e); // the same value in every lane
                __syncwarp();
                if (lane == 0) {
                    values[in.dst] = r;
                }
                __syncwarp();
            }
        }
    }
}

} // namespace

// How many warps of a block can keep `slots` rows of `len` int32 values in shared memory; 0 = the run does not fit.
int rowMachineWarps(int slots, int len) {
    const size_t perWarp = (size_t(slots) * size_t(len) + kMaxRowValues) * sizeof(int32_t);
    const size_t budget = 200 * 1024;
    const size_t warps = perWarp == 0 ? 0 : budget / perWarp;
    return int(warps > 8 ? 8 : warps);
}

int rowMachine(const RowProgram &program, const TView *T, cudaStream_t s) {
    DevRowProgram prog{};
    if (program.insts.size() > size_t(kMaxRowInsts) || program.len <= 0 || program.len % 4 != 0) {
        setLastError("fused rows: program out of range");
        return MLEL_ERROR_UNKNOWN;
    }
    prog.count = int32_t(program.insts.size());
    prog.len = program.len;
    prog.slots = program.slots;
    prog.warps = rowMachineWarps(program.slots, program.len);
    if (prog.warps < 1) {
        setLastError("fused rows: a row does not fit into shared memory");
        return MLEL_ERROR_UNKNOWN;
    }
    for (int n = 0; n < prog.count; ++n) {
        const RowInst &in = program.insts[size_t(n)];
        DevRowInst &d = prog.inst[n];
        d.op = in.op;
        d.dstKind = in.dst.kind, d.dst = in.dst.index;
        d.aKind = in.a.kind, d.a = in.a.index, d.aImm = in.a.imm;
        d.bKind = in.b.kind, d.b = in.b.index, d.bImm = in.b.imm;
        d.dtype = in.dtype;
        d.ptr = in.tensor >= 0 ? T[in.tensor].ptr : nullptr;
        for (int k = 0; k < 7; ++k) {
            d.p[k] = in.p[k];
        }
        if ((in.op == ROW_LOAD || in.op == ROW_STORE) && (reinterpret_cast<uintptr_t>(d.ptr) & 15u) != 0) {
            setLastError("fused rows: a tensor is not 16-byte aligned");
            return MLEL_ERROR_UNKNOWN;
        }
    }
    const size_t smemBytes = size_t(prog.warps) * (size_t(prog.slots) * prog.len + kMaxRowValues) * sizeof(int32_t);
    {
        // more than 48 KB of dynamic shared memory is an opt-in per device
        static std::mutex lock;
        static bool optedIn[64] = {};
        int device = 0;
        cudaGetDevice(&device);
        std::lock_guard<std::mutex> guard(lock);
        if (device < 0 || device >= 64 || !optedIn[device]) {
            if (cudaFuncSetAttribute(rowMachineKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024) != cudaSuccess) {
                setLastError("fused rows: shared memory opt-in failed");
                return MLEL_ERROR_DEVICE;
            }
            if (device >= 0 && device < 64) {
                optedIn[device] = true;
            }
        }
    }
    const int64_t blocksWanted = (program.rows + prog.warps - 1) / prog.warps;
    const int64_t cap = int64_t(kNumSMs) * 8;
    const int grid = int(blocksWanted < cap ? (blocksWanted < 1 ? 1 : blocksWanted) : cap);
    rowMachineKernel<<<grid, prog.warps * 32, smemBytes, s>>>(prog, program.rows);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        setLastError(std::string("fused rows: ") + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

} // namespace mlel
