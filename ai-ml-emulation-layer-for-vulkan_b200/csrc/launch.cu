// Operator dispatch: picks the kernel for one OpDesc.  The order of preference is
//   1. tensor-core / vectorised kernels for packed int8 shapes (fast_*.cu, gemm_*.cu),
//   2. the one-thread-per-element kernels (generic_ops.cu, fused_generic.cu).
// There is no CPU path: every branch ends in a CUDA launch or an error.
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "kernels/device_common.cuh"
#include "kernels/gemm_i8_tcgen05.hpp"
#include "kernels/kernels.hpp"
#include "ops.hpp"

namespace mlel {

namespace {

thread_local std::string g_lastError;

ConvAttr convAttr(const OpDesc &op) {
    ConvAttr a{};
    for (int k = 0; k < 4; ++k) {
        a.pad[k] = op.i[k];
    }
    a.stride[0] = op.i[4], a.stride[1] = op.i[5], a.dilation[0] = op.i[6], a.dilation[1] = op.i[7];
    a.inZp = op.i[8], a.wZp = op.i[9];
    return a;
}

// Runs q on the paired tensor-core kernel when it applies and the selection allows it; *rc is the launch status when
// the result is true.  Matrix products take it by default; convolutions only on request ("pair_kernel" 2): on the
// ResNet-50 layer shapes the single-CTA kernels measured as fast or faster (their tiles fill the SMs better and the
// epilogue, not the main loop, bounds those layers).
bool tryPairKernel(const GemmI8Problem &q, bool convolution, cudaStream_t s, int *rc) {
    const int mode = tensorCoreTuning().pairKernel.load(std::memory_order_relaxed);
    if (mode < (convolution ? 2 : 1) || !gemmI8PairApplies(q)) {
        return false;
    }
    bool taken = false;
    *rc = gemmI8PairLaunch(q, s, &taken);
    return taken || *rc != MLEL_SUCCESS;
}

PoolAttr poolAttr(const OpDesc &op) {
    PoolAttr a{};
    a.kernel[0] = op.i[0], a.kernel[1] = op.i[1], a.stride[0] = op.i[2], a.stride[1] = op.i[3];
    for (int k = 0; k < 4; ++k) {
        a.pad[k] = op.i[4 + k];
    }
    a.inZp = op.i[8], a.outZp = op.i[9];
    return a;
}

DevRescale devRescale(const FusedRescale &f, const TView *T) {
    DevRescale r{};
    r.mult = reinterpret_cast<const int32_t *>(T[f.multTensor].ptr);
    r.shift = reinterpret_cast<const int8_t *>(T[f.shiftTensor].ptr);
    r.inZp = int32_t(wrapTo(f.inDtype, f.attr.inZp));
    r.outZp = int32_t(wrapTo(f.outDtype, f.attr.outZp));
    r.lo = f.lo, r.hi = f.hi;
    r.perChannel = f.attr.perChannel;
    r.doubleRound = f.attr.scale32 && f.attr.doubleRound;
    return r;
}

DevEpilogue devEpilogue(const FusedEpilogue &e, const TView *T) {
    DevEpilogue d{};
    d.hasMain = e.hasMain;
    if (e.hasMain) {
        d.main = devRescale(e.main, T);
    }
    d.hasResidual = e.hasResidual;
    if (e.hasResidual) {
        d.a = devRescale(e.a, T);
        d.b = devRescale(e.b, T);
        d.out = devRescale(e.out, T);
        d.shortcut = e.shortcutTensor >= 0 ? reinterpret_cast<const int8_t *>(T[e.shortcutTensor].ptr) : nullptr;
    }
    return d;
}

int64_t numelOf(const TView &t) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; ++i) {
        n *= t.dims[i];
    }
    return n;
}

// Storage bits of a PAD constant (pad.comp:46-50): int32 tensors take padConstInt, other integer
// types the double constant converted by the storage type's constructor, fp32 the float value.
int64_t padBits(const OpDesc &op, int32_t dtype) {
    if (dtype == MLEL_I32) {
        return int64_t(uint32_t(op.i[0]));
    }
    if (dtype == MLEL_F32) {
        const float f = float(op.d[0]);
        uint32_t u;
        memcpy(&u, &f, 4);
        return u;
    }
    return wrapTo(dtype, int64_t(op.d[0]));
}

// CONV2D / fused CONV2D on the tensor cores (the node was prepared by GraphPipeline::prepareTensorCore).
int launchConvTensorCore(const OpDesc &op, const TView *T, cudaStream_t s, LaunchChain *chain, const LaunchChain *consumed) {
    const TView &in = T[op.in[0]], &w = T[op.in[1]], &out = T[op.out[0]];
    GemmI8Problem q{};
    GemmI8Params &p = q.params;
    const int64_t OH = out.dims[1], OW = out.dims[2];
    p.M = int32_t(int64_t(out.dims[0]) * OH * OW);
    p.N = int32_t(out.dims[3]);
    p.K = int32_t(w.dims[1] * w.dims[2] * w.dims[3]);
    p.ldOut = p.N;
    p.in = reinterpret_cast<const int8_t *>(in.ptr);
    p.H = int32_t(in.dims[1]), p.W = int32_t(in.dims[2]), p.IC = int32_t(in.dims[3]);
    p.OH = int32_t(OH), p.OW = int32_t(OW), p.KH = int32_t(w.dims[1]), p.KW = int32_t(w.dims[2]);
    p.padTop = op.i[0], p.padLeft = op.i[2], p.strideY = op.i[4], p.strideX = op.i[5], p.dilY = op.i[6], p.dilX = op.i[7];
    p.corr = reinterpret_cast<const int32_t *>(T[op.aux[0]].ptr);
    p.rowClass = reinterpret_cast<const uint8_t *>(T[op.aux[1]].ptr);
    p.colClass = reinterpret_cast<const uint8_t *>(T[op.aux[2]].ptr);
    p.numColClasses = op.auxi[0];
    p.numClasses = op.auxi[1];
    p.baseClass = op.auxi[3];
    p.corrSmall = op.auxi[4];
    if (p.numClasses <= 1) {
        p.rowClass = p.colClass = nullptr; // no window crosses the border: one correction row serves every pixel
        p.baseClass = 0;
    }
    if (op.kind == OP_FUSED_CONV2D) {
        p.out8 = reinterpret_cast<int8_t *>(out.ptr);
        p.epi = devEpilogue(op.epi, T);
        if (op.epi.hasResidual && op.tc == 1 && op.aux[3] >= 0) {
            p.residualTable = reinterpret_cast<const uint8_t *>(T[op.aux[3]].ptr);
        }
    } else {
        p.out32 = reinterpret_cast<int32_t *>(out.ptr);
    }
    q.batches = 1;
    if (op.tc == 2) {
        // Channel count not a multiple of 16: gather, by a table of offsets, from a copy of the input with
        // zero-padded channels and borders.
        const TView &copy = T[op.scratch];
        const int rc = padImageI8(p.in, reinterpret_cast<int8_t *>(copy.ptr), int(in.dims[0]), p.H, p.W, p.IC,
                                  int(copy.dims[1]), int(copy.dims[2]), int(copy.dims[3]), p.padTop, p.padLeft, s);
        if (rc != MLEL_SUCCESS) {
            return rc;
        }
        p.in = reinterpret_cast<const int8_t *>(copy.ptr);
        p.H = int32_t(copy.dims[1]), p.W = int32_t(copy.dims[2]), p.IC = int32_t(copy.dims[3]);
        p.padTop = p.padLeft = 0;
        p.K = int32_t(T[op.aux[3]].dims[1]);
        if (p.KH == 1 && p.KW == 1 && p.strideY == 1 && p.strideX == 1 && p.H == p.OH && p.W == p.OW && p.IC % 16 == 0 &&
            p.K == p.IC) {
            // A 1x1 convolution over the copy (channels padded to a multiple of 16, weights padded alike) is a plain
            // [pixels][channels] matrix product: TMA tiles instead of the table gather, and the channel-major kernel
            // where it applies (e.g. the 24 -> 144 expansions of a MobileNetV2-shaped graph: 48 -> 20 us).
            q.aMatrix = copy.ptr;
            q.aRowBytes = uint64_t(p.IC);
            q.aBatchBytes = uint64_t(p.IC) * uint64_t(p.M);
            q.bMatrix = T[op.aux[3]].ptr;
            q.bRowBytes = uint64_t(p.K);
            q.bBatchBytes = 0;
            q.bMnMajor = false;
            return gemmI8OcMajorApplies(q) ? gemmI8OcMajorLaunch(q, s) : gemmI8Launch(q, s);
        }
        p.chunkBytes = op.auxi[2];
        p.gatherTable = reinterpret_cast<const int32_t *>(T[op.aux[4]].ptr);
        q.bMatrix = T[op.aux[3]].ptr;
        q.bRowBytes = uint64_t(p.K);
        q.bBatchBytes = 0;
        q.bMnMajor = false;
        return gemmI8Launch(q, s);
    }
    // A 1x1, stride-1, unpadded convolution reads the input as a plain [pixels][IC] matrix.
    const bool plain = p.KH == 1 && p.KW == 1 && p.strideY == 1 && p.strideX == 1 && op.i[0] == 0 && op.i[1] == 0 &&
                       op.i[2] == 0 && op.i[3] == 0 && (reinterpret_cast<uintptr_t>(in.ptr) & 15u) == 0;
    if (plain) {
        q.aMatrix = in.ptr;
        q.aRowBytes = uint64_t(p.IC);
        q.aBatchBytes = uint64_t(p.IC) * uint64_t(p.M);
    }
    q.bMatrix = w.ptr;
    q.bRowBytes = uint64_t(p.K);
    q.bBatchBytes = 0;
    q.bMnMajor = false;
    int rc = MLEL_SUCCESS;
    if (tryPairKernel(q, true, s, &rc)) {
        return rc;
    }
    return gemmI8OcMajorApplies(q) ? gemmI8OcMajorLaunch(q, s, chain, consumed) : gemmI8Launch(q, s);
}

// MATMUL / fused MATMUL: second input constant and pre-transposed (tc == 1), or transposed here (tc == 3).
int launchMatmulTensorCore(const OpDesc &op, const TView *T, cudaStream_t s) {
    const TView &a = T[op.in[0]], &out = T[op.out[0]];
    GemmI8Problem q{};
    GemmI8Params &p = q.params;
    p.M = int32_t(a.dims[1]);
    p.K = int32_t(a.dims[2]);
    p.batchedB = 1;
    p.numClasses = 1;
    p.numColClasses = 1;
    p.batchedCorr = 1;
    // |correction| = |zero point of A| * |column sum of B| <= 128 * K * |zp|: small enough for the short RESCALE form
    // whenever that bound is (see GemmI8Params::corrSmall)
    {
        const int64_t corrBound = int64_t(op.i[0] < 0 ? -op.i[0] : op.i[0]) * p.K * 128;
        const bool tiny = corrBound + int64_t(p.K) * (int64_t(1) << 14) + 256 < (int64_t(1) << 29);
        p.corrSmall = tiny ? 2 : (corrBound <= (int64_t(1) << 30) - 256 ? 1 : 0);
    }
    if (op.kind == OP_FUSED_MATMUL) {
        p.out8 = reinterpret_cast<int8_t *>(out.ptr);
        p.epi = devEpilogue(op.epi, T);
    } else {
        p.out32 = reinterpret_cast<int32_t *>(out.ptr);
    }
    q.batches = int32_t(a.dims[0]);
    q.aMatrix = a.ptr;
    q.aRowBytes = uint64_t(p.K);
    q.aBatchBytes = uint64_t(p.K) * uint64_t(p.M);
    const void *bt = nullptr;
    if (op.tc == 3) {
        const TView &b = T[op.in[1]];
        p.N = int32_t(b.dims[2]);
        p.ldOut = p.N;
        int8_t *scratch = reinterpret_cast<int8_t *>(T[op.scratch].ptr);
        int32_t *corr = reinterpret_cast<int32_t *>(scratch + op.auxi[2]);
        p.corr = corr;
        // The paired kernel reads the run-time operand where it lies ([C][W], the output column contiguous: an
        // MN-major tensor-core operand) and only needs the column sums; the single-CTA kernel takes a transposed
        // copy, made together with the sums.
        q.bMatrix = b.ptr;
        q.bRowBytes = uint64_t(p.N);
        q.bBatchBytes = uint64_t(p.K) * uint64_t(p.N);
        q.bMnMajor = true;
        if (tensorCoreTuning().pairKernel.load(std::memory_order_relaxed) != 0 && gemmI8PairApplies(q)) {
            int rc = columnSumsForMatmul(reinterpret_cast<const int8_t *>(b.ptr), corr, int(b.dims[0]), p.K, p.N, op.i[0], s);
            if (rc != MLEL_SUCCESS) {
                return rc;
            }
            bool taken = false;
            rc = gemmI8PairLaunch(q, s, &taken);
            if (taken || rc != MLEL_SUCCESS) {
                return rc;
            }
        }
        const int rc = transposeForMatmul(reinterpret_cast<const int8_t *>(b.ptr), scratch, corr, int(b.dims[0]), p.K, p.N,
                                          op.i[0], s);
        if (rc != MLEL_SUCCESS) {
            return rc;
        }
        bt = scratch;
    } else {
        p.N = int32_t(T[op.aux[3]].dims[1]);
        p.ldOut = p.N;
        bt = T[op.aux[3]].ptr;
        p.corr = reinterpret_cast<const int32_t *>(T[op.aux[0]].ptr);
    }
    q.bMatrix = bt;
    q.bRowBytes = uint64_t(p.K);
    q.bBatchBytes = uint64_t(p.K) * uint64_t(p.N);
    q.bMnMajor = false;
    int rc = MLEL_SUCCESS;
    if (tryPairKernel(q, false, s, &rc)) {
        return rc;
    }
    return gemmI8Launch(q, s);
}

} // namespace

void setLastError(const std::string &msg) { g_lastError = msg; }
const std::string &lastError() { return g_lastError; }

int launchOp(const OpDesc &op, const TView *T, cudaStream_t s, LaunchChain *chain) {
    const auto in = [&](size_t k) -> const TView & { return T[op.in[k]]; };
    const TView &out = T[op.out[0]];
    int rc = MLEL_SUCCESS; // status of a vectorised kernel that took the operator
    // What the launch before this operator publishes may only be used by this operator: take it away from the chain,
    // so that any kernel but the channel-major convolution (which records its own) leaves nothing behind.
    LaunchChain consumed{};
    if (chain != nullptr) {
        consumed = *chain;
        chain->forget();
    }
    if (op.tc) {
        // Addresses are only known here: pointers that are not 16-byte aligned go to the generic kernels.
        const bool aligned = ((reinterpret_cast<uintptr_t>(in(0).ptr) | reinterpret_cast<uintptr_t>(out.ptr)) & 15u) == 0;
        if (aligned && (op.kind == OP_CONV2D || op.kind == OP_FUSED_CONV2D)) {
            return launchConvTensorCore(op, T, s, chain, &consumed);
        }
        if (aligned && (op.kind == OP_MATMUL || op.kind == OP_FUSED_MATMUL) &&
            (op.tc != 3 || (reinterpret_cast<uintptr_t>(in(1).ptr) & 15u) == 0)) {
            return launchMatmulTensorCore(op, T, s);
        }
    }
    switch (op.kind) {
    case OP_CONV2D:
        return genericConv2d(in(0), in(1), in(2), out, convAttr(op), s);
    case OP_DEPTHWISE_CONV2D:
        if (depthwise3x3Eligible(in(0), in(1), in(2), out, convAttr(op), false)) {
            return depthwise3x3(in(0), in(1), in(2), out, convAttr(op), nullptr, s);
        }
        return genericDepthwise(in(0), in(1), in(2), out, convAttr(op), s);
    case OP_MATMUL:
        return genericMatmul(in(0), in(1), out, op.i[0], op.i[1], s);
    case OP_RESCALE: {
        RescaleAttr a{op.i[0], op.i[1], op.i[2], op.i[3], op.i[4]};
        if (vecRescale(in(0), out, in(1), in(2), a, s, &rc)) {
            return rc;
        }
        return genericRescale(in(0), out, in(1), in(2), a, s);
    }
    case OP_AVG_POOL2D:
        if (avgPoolI8Eligible(in(0), out, poolAttr(op))) {
            return avgPoolI8(in(0), out, poolAttr(op), s);
        }
        return genericAvgPool(in(0), out, poolAttr(op), s);
    case OP_MAX_POOL2D:
        if (maxPoolI8Eligible(in(0), out)) {
            return maxPoolI8(in(0), out, poolAttr(op), s);
        }
        return genericMaxPool(in(0), out, poolAttr(op), s);
    case OP_TABLE:
        if (vecTable(in(0), out, in(1), s, &rc)) {
            return rc;
        }
        return genericTable(in(0), out, in(1), s);
    case OP_TRANSPOSE: {
        uint32_t perms[kMaxRank];
        for (int k = 0; k < kMaxRank; ++k) {
            perms[k] = uint32_t(op.i[k]);
        }
        if (vecTransposeRows(in(0), out, perms, s, &rc) || vecTransposeLast2Bytes(in(0), out, perms, s, &rc)) {
            return rc;
        }
        return genericTranspose(in(0), out, perms, s);
    }
    case OP_CONCAT:
        return genericConcat(in(0), out, uint32_t(op.i[0]), uint32_t(op.i[1]), s);
    case OP_CLAMP:
        if (vecClampI8(in(0), out, wrapTo(out.dtype, int64_t(op.d[0])), wrapTo(out.dtype, int64_t(op.d[1])), s, &rc)) {
            return rc;
        }
        return genericClamp(in(0), out, op.d[0], op.d[1], s);
    case OP_BINARY:
        if ((op.sub == BIN_ADD || op.sub == BIN_SUB) && vecBinaryI32(op.sub, in(0), in(1), out, 0, s, &rc)) {
            return rc;
        }
        return genericBinary(op.sub, in(0), in(1), out, s);
    case OP_UNARY:
        return genericUnary(op.sub, in(0), out, s);
    case OP_MUL:
        if (vecBinaryI32(-1, in(0), in(1), out, uint32_t(op.i[0]), s, &rc)) {
            return rc;
        }
        return genericMul(in(0), in(1), out, uint32_t(op.i[0]), s);
    case OP_REDUCE:
        if (vecRowReduce(op.sub, in(0), out, uint32_t(op.i[0]), s, &rc)) {
            return rc;
        }
        return genericReduce(op.sub, in(0), out, uint32_t(op.i[0]), s);
    case OP_CAST:
        return genericCast(in(0), out, s);
    case OP_RESHAPE: {
        // same linear index on both sides: packed tensors of equal size are one device-to-device copy
        const auto packedBytes = [](const TView &t) -> int64_t {
            int64_t st = dtypeSize(t.dtype);
            for (int i = t.rank - 1; i >= 0; --i) {
                if (t.strides[i] != st) {
                    return -1;
                }
                st *= t.dims[i];
            }
            return st;
        };
        const int64_t nin = packedBytes(in(0)), nout = packedBytes(out);
        if (nin > 0 && nin == nout && in(0).dtype == out.dtype) {
            if (in(0).ptr == out.ptr) {
                return MLEL_SUCCESS; // the session gave both tensors one storage: nothing to move
            }
            if (cudaMemcpyAsync(out.ptr, in(0).ptr, size_t(nin), cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
                setLastError("RESHAPE: device-to-device copy failed");
                return MLEL_ERROR_DEVICE;
            }
            return MLEL_SUCCESS;
        }
        return genericReshape(in(0), out, s);
    }
    case OP_SLICE: {
        uint32_t start[kMaxRank];
        for (int k = 0; k < kMaxRank; ++k) {
            start[k] = uint32_t(op.i[k]);
        }
        return genericSlice(in(0), out, start, s);
    }
    case OP_PAD:
        return genericPad(in(0), out, in(1), padBits(op, out.dtype), s);
    case OP_ARITHMETIC_RIGHT_SHIFT:
        return genericArShift(in(0), in(1), out, op.i[0], s);
    case OP_NEGATE:
        return genericNegate(in(0), out, op.i[0], op.i[1], s);
    case OP_SELECT:
        return genericSelect(in(0), in(1), in(2), out, s);
    case OP_FFT2D:
        return fft2d(&in(0), &in(1), out, T[op.out[1]], op.i[0] != 0, s);
    case OP_RFFT2D:
        return fft2d(&in(0), nullptr, out, T[op.out[1]], false, s);
    case OP_ARGMAX:
        return indexArgmax(in(0), out, uint32_t(op.i[0]), s);
    case OP_GATHER:
        return indexGather(in(0), in(1), out, s);
    case OP_SCATTER:
        return indexScatter(in(0), in(1), in(2), out, s);
    case OP_REVERSE:
        return indexReverse(in(0), out, uint32_t(op.i[0]), s);
    case OP_TILE:
        return indexTile(in(0), out, s);
    case OP_RESIZE: {
        ResizeAttr a{};
        for (int k = 0; k < 4; ++k) {
            a.scale[k] = op.i[k];
        }
        a.offset[0] = op.i[4], a.offset[1] = op.i[5], a.border[0] = op.i[6], a.border[1] = op.i[7], a.mode = op.i[8];
        return resizeInteger(in(0), out, a, s);
    }
    case OP_TRANSPOSE_CONV2D:
        return transposeConv2d(in(0), in(1), in(2), out, convAttr(op), s);
    case OP_CONV3D: {
        Conv3dAttr a{};
        for (int k = 0; k < 6; ++k) {
            a.pad[k] = op.i[k];
        }
        for (int k = 0; k < 3; ++k) {
            a.stride[k] = op.i[6 + k];
            a.dilation[k] = op.i[9 + k];
        }
        a.inZp = op.i[12], a.wZp = op.i[13];
        return conv3d(in(0), in(1), in(2), out, a, s);
    }
    case OP_FUSED_CONV2D:
        return fusedConv2dGeneric(in(0), in(1), in(2), out, convAttr(op), devEpilogue(op.epi, T), s);
    case OP_FUSED_DEPTHWISE: {
        const DevEpilogue epi = devEpilogue(op.epi, T);
        if (!epi.hasResidual && depthwise3x3Eligible(in(0), in(1), in(2), out, convAttr(op), true)) {
            return depthwise3x3(in(0), in(1), in(2), out, convAttr(op), &epi, s);
        }
        return fusedDepthwiseGeneric(in(0), in(1), in(2), out, convAttr(op), epi, s);
    }
    case OP_FUSED_MATMUL:
        return fusedMatmulGeneric(in(0), in(1), out, op.i[0], op.i[1], devEpilogue(op.epi, T), s);
    case OP_FUSED_ROWS:
        if (!op.rows) {
            setLastError("fused rows: no program");
            return MLEL_ERROR_UNKNOWN;
        }
        return rowMachine(*op.rows, T, s);
    case OP_FUSED_ROW_EXP:
        return rowExpFused(in(0), in(1), T[op.out[0]], T[op.out[1]], devRescale(op.epi.main, T), s);
    case OP_FUSED_MUL_RESCALE:
        return mulRescaleFused(in(0), in(1), out, uint32_t(op.i[0]), devRescale(op.epi.main, T), s);
    case OP_FUSED_ADD:
        return fusedAdd(reinterpret_cast<const int8_t *>(in(0).ptr), reinterpret_cast<const int8_t *>(in(1).ptr),
                        reinterpret_cast<int8_t *>(out.ptr), numelOf(out), devEpilogue(op.epi, T), s);
    default:
        setLastError("unknown operator kind");
        return MLEL_ERROR_UNKNOWN;
    }
}

} // namespace mlel
