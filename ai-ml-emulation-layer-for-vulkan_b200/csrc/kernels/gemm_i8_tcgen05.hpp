// Interface of the tcgen05 int8 contraction kernel (gemm_i8_tcgen05.cu).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "kernels.hpp"

namespace mlel {

// Division of a number below 2^31 by a constant as a multiply-high and a shift (Granlund and Montgomery): with
// l = ceil(log2 d), mul = ceil(2^(31 + l) / d) fits 32 bits and n / d = (n * mul) >> (31 + l) for every n < 2^31.
// The kernels divide tile and pixel indices several times per tile and warp; a hardware-less 32-bit division is
// some twenty instructions.  mul == 0 stands for d == 1.
struct FastDiv {
    uint32_t mul = 0, shift = 0, d = 1;
};
inline FastDiv makeFastDiv(int64_t divisor) {
    FastDiv f;
    const uint64_t d = divisor > 1 ? uint64_t(divisor) : 1;
    f.d = uint32_t(d);
    if (d > 1) {
        uint32_t l = 0;
        while ((uint64_t(1) << l) < d) {
            ++l;
        }
        f.mul = uint32_t(((uint64_t(1) << (31 + l)) + d - 1) / d);
        f.shift = l - 1;
    }
    return f;
}

// Device-side parameters (passed by value to the kernel).
struct GemmI8Params {
    int32_t M, N, K;     // per batch: rows, columns (output channels), contraction length in bytes
    int32_t ldOut;       // elements between consecutive output rows
    int32_t batches;     // number of independent [M,K]x[K,N] problems (filled in by gemmI8Launch)
    int32_t batchedB;    // K-major B only: B has one matrix per batch (else one shared matrix)
    // implicit-GEMM geometry (used only when A is gathered): NHWC input, window, output grid
    const int8_t *in;
    int32_t H, W, IC, OH, OW, KH, KW;
    int32_t strideY, strideX, padTop, padLeft, dilY, dilX;
    // Table gather (a convolution over a zero-padded copy of its input, where every tap is in range): piece q
    // of a pixel's K row is chunkBytes (4, 8 or 16) bytes at gatherTable[q] from the window origin
    // in + ((n * H + oy * strideY) * W + ox * strideX) * IC.  Null => gather 16-byte pieces with bounds checks.
    const int32_t *gatherTable;
    int32_t chunkBytes;
    // filled in by the launchers: divisors OH * OW and OW (pixel index -> image, row, column), and the two inner
    // extents of the tile index (fastest first)
    FastDiv divPlane, divOW, divTiles0, divTiles1;
    // im2col TMA mode (set by the launchers): K blocks per tap = ceil(IC / 128), each zero-filled past IC; 0 = off
    int32_t kbPerTap;
    // correction term added to the raw accumulator: corr[(batch,) class, n]
    const int32_t *corr;
    const uint8_t *rowClass; // [OH] border class of an output row, or null (single class)
    const uint8_t *colClass; // [OW]
    int32_t numColClasses, numClasses, batchedCorr;
    int32_t baseClass;       // the most common class: its correction row is staged in shared memory
    int32_t corrSmall;       // 1: every |corr| <= 2^30 - 256: accumulator + correction - zero point stays inside int32;
                             // 2: it even stays below 2^29 in size
    // outputs: exactly one of out32 / out8 is set
    int32_t *out32;
    int8_t *out8;
    DevEpilogue epi;
    // Fused residual tail as one table: residualTable[(m + 128) * kResidualRowBytes + s] is the output byte for
    // main-stage value m (int8) and raw shortcut byte s, i.e. RESCALE_out(RESCALE_a(m) + RESCALE_b(int8(s)))
    // with its clamp.  256 rows of kResidualRowBytes bytes (the last four of a row unused), 16-byte aligned, or
    // null when the node has none.
    static constexpr int kResidualRowBytes = 260;
    const uint8_t *residualTable;
    // Tile-level hand-over between two consecutive channel-major launches of one stream (see LaunchChain; null
    // pointers: off).  progressOut[j] counts the channel tiles of this launch's pixel tile j whose bytes have reached
    // memory.  A launch with progressIn reads its pixel operand as soon as the counters of the producer's pixel tiles
    // that cover it have reached progressInTarget, instead of waiting for the whole producing grid; it still waits
    // for that grid before its first store.
    uint32_t *progressOut;
    const uint32_t *progressIn;
    int32_t progressInTilePixels; // pixels per tile of the producing launch
    uint32_t progressInTarget;    // its channel tiles per pixel tile
    int32_t channelFastest;       // tile order: 1 = a pixel tile's channel tiles are consecutive tile indices
};

// What one dispatch keeps between consecutive launches so that a channel-major convolution can start on the finished
// pixel tiles of the convolution before it.  `words` is zeroed when the dispatch starts; every publishing launch takes
// its counters from it.  `prev*` describe what the launch just enqueued publishes; launchOp() takes them away before
// every operator, so only the immediately preceding launch is ever consumed (see the ordering argument in
// gemm_i8_ocmajor.cu).
struct LaunchChain {
    uint32_t *words = nullptr;
    size_t capacity = 0, used = 0;
    bool publishNext = false; // the operator enqueued next reads this operator's output as its pixel operand
    const void *prevTensor = nullptr;
    uint32_t *prevCounters = nullptr;
    int32_t prevTilePixels = 0;
    uint32_t prevTarget = 0;
    int64_t prevPixels = 0;
    void forget() {
        prevTensor = nullptr;
        prevCounters = nullptr;
    }
};

struct GemmI8Problem {
    GemmI8Params params;
    int32_t batches;
    // A as a matrix [batches][M][K] (K contiguous) for TMA; null => gather from params.in
    const void *aMatrix;
    uint64_t aRowBytes, aBatchBytes;
    // B: K-major [batchesB][N][K] or (bMnMajor) N-major [batches][K][N]
    const void *bMatrix;
    uint64_t bRowBytes, bBatchBytes;
    bool bMnMajor;
};

// Enqueues the kernel.  Preconditions (checked by the caller): K % 16 == 0, K <= 65536, operands
// 16-byte aligned with row pitches that are multiples of 16 bytes.
int gemmI8Launch(const GemmI8Problem &problem, cudaStream_t stream);

// Channel-major variant (gemm_i8_ocmajor.cu) for fused int8 convolutions with more than 64 output channels:
// same problem description, weights as the tensor-core A operand.  `Applies` tells whether it can take q.
bool gemmI8OcMajorApplies(const GemmI8Problem &problem);
// `chain` (may be null): where the launch records what it publishes; `consumed` (may be null): what the launch before it
// in the stream published.
int gemmI8OcMajorLaunch(const GemmI8Problem &problem, cudaStream_t stream, LaunchChain *chain = nullptr,
                        const LaunchChain *consumed = nullptr);
int ocMajorErrorWord();

// Paired variant (gemm_i8_pair.cu): two CTAs of a cluster share one 256-channel tile through
// tcgen05.mma.cta_group::2.  `Applies` tells whether it can take q; Launch sets *taken to false (and returns
// success) when the driver refuses the tensor maps, so that the caller can use another kernel.
bool gemmI8PairApplies(const GemmI8Problem &problem);
int gemmI8PairLaunch(const GemmI8Problem &problem, cudaStream_t stream, bool *taken);
int pairErrorWord();

// Kernel-selection knobs of the tensor-core launchers (mlel_set_tuning): 0 = the library's own choice.
struct TensorCoreTuning {
    std::atomic<int> pairKernel{1};        // paired kernel for: 0 nothing, 1 matrix products, 2 convolutions too
    std::atomic<int> pairTilePixels{0};    // 128, 192 or 256: pixels per tile of the paired kernel
    std::atomic<int> ocTilePixels{0};      // 128, 192 or 256: pixels per tile of the channel-major kernel
    std::atomic<int> ocTileRule{3};        // >= 1: narrow tiles for layers that would leave a quarter of the SMs idle;
                                           // r >= 2: 256-pixel tiles for layers with at least r rounds of tiles per SM
    std::atomic<int> dependentLaunch{1};   // 0: launch the tensor-core kernels without programmatic dependent launch
    std::atomic<int> tileProgress{7};      // tile-level hand-over: bit 0 read by tiles, 1 publish, 2 channel tiles first
};
TensorCoreTuning &tensorCoreTuning();

// Launches of the three tensor-core kernels since the library was loaded: 0 pixel-major (gemm_i8_tcgen05.cu),
// 1 channel-major (gemm_i8_ocmajor.cu), 2 paired (gemm_i8_pair.cu).  Tests use them to see which kernel took a case.
extern std::atomic<long long> g_tensorCoreLaunches[3];

// Value of the device-side error word written by a bounded wait that ran out (0 = none).
int tcgen05ErrorFlag();
// Runs a one-thread kernel whose bounded wait (limit about 1 ms) cannot be satisfied; *codeOut receives the code the
// wait recorded (99), 0 if the wait did not give up.  The recorded code is cleared again.
int waitTimeoutSelfTest(cudaStream_t stream, int *codeOut);

} // namespace mlel
