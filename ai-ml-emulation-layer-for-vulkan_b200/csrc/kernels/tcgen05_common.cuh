// Shared device and host helpers of the tcgen05 int8 kernels (PTX wrappers for mbarrier, TMA, tcgen05 and
// the tensor-map encoder).  Included by gemm_i8_tcgen05.cu and gemm_i8_ocmajor.cu.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <atomic>
#include <mutex>
#include <set>
#include <string>
#include <utility>

#include "device_common.cuh"
#include "gemm_i8_tcgen05.hpp"

namespace mlel {

namespace tc {

// Error word of the including translation unit: a bounded wait that ran out stores its code here.
static __device__ int g_tcgen05Error = 0;

// Reads this translation unit's error word (0 = none).
static inline int readErrorWord() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_tcgen05Error, sizeof(int));
    return v;
}
static inline void clearErrorWord() {
    const int zero = 0;
    cudaMemcpyToSymbol(g_tcgen05Error, &zero, sizeof(int));
}

constexpr int BM = 128;    // rows per tile (UMMA M)
constexpr int BK = 128;    // bytes (= int8 elements) of K per pipeline stage
constexpr int UMMA_K = 32; // K per tcgen05.mma for 8-bit operands
constexpr int kEpilogueWarps = 16;
constexpr int kTmaWarp = kEpilogueWarps;
constexpr int kMmaWarp = kEpilogueWarps + 1;
constexpr int kGatherWarp0 = kEpilogueWarps + 2;
constexpr int kThreadsTma = (kEpilogueWarps + 2) * 32;
constexpr int kThreadsGather = (kEpilogueWarps + 6) * 32;
constexpr long long kWaitLimitCycles = 4000000000ll;

__device__ __forceinline__ uint32_t smemAddr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbarInit(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void mbarArriveExpectTx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smemAddr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// The same with a suspend-time hint: the thread may stay suspended in hardware for up to `hintNs`
// nanoseconds waiting for the phase to complete, instead of coming back to poll.
__device__ __forceinline__ bool mbarTryWaitHint(uint64_t *bar, uint32_t parity, uint32_t hintNs) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smemAddr(bar)), "r"(parity), "r"(hintNs)
                 : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and records `code`) when the barrier did not complete in time.  A waiter that
// does not get through at once suspends in hardware between checks, so that a waiting role does not take issue
// slots from the warps that share its scheduler (the epilogue warps do the arithmetic); the clock is read every
// 64th check.
__device__ __forceinline__ bool mbarWaitLimit(uint64_t *bar, uint32_t parity, int code, long long limitCycles) {
    if (mbarTryWait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    unsigned polls = 0;
    while (!mbarTryWaitHint(bar, parity, 1000u)) {
        if ((++polls & 63u) == 0) {
            if (clock64() - start > limitCycles) {
                atomicCAS(&g_tcgen05Error, 0, code);
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool mbarWait(uint64_t *bar, uint32_t parity, int code) {
    return mbarWaitLimit(bar, parity, code, kWaitLimitCycles);
}

__device__ __forceinline__ void tmaLoad3d(const CUtensorMap *map, void *dst, uint64_t *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smemAddr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smemAddr(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// TMA load in im2col mode from an NHWC tensor {C, W, H, N}: pixelsPerColumn consecutive window positions
// (x fastest, then y, then image; stepping by the convolution stride inside the map's bounding box) starting
// at the window whose first tap is at input pixel (w, h) of image n; of each window the tap at offset
// (offW, offH) from the first one is read, channelsPerPixel channels from channel c on.  Positions outside
// the tensor read zeros.
__device__ __forceinline__ void tmaLoadIm2col4d(const CUtensorMap *map, void *dst, uint64_t *bar, int c, int w, int h, int n,
                                                uint16_t offW, uint16_t offH) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smemAddr(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smemAddr(bar)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(offW), "h"(offH)
                 : "memory");
}

// The producer's side of ummaBlockPeek: the loads of one stage -- expected byte count, weight tile, pixel tile --
// with a non-blocking test of the NEXT stage's `empty` barrier issued ahead of them, so that its answer arrives
// while the loads go out instead of stalling the thread between two stages.  Returns 1 when that barrier's phase
// `peekParity` is complete; 0 means "not yet known".
__device__ __forceinline__ uint32_t tmaStagePeekTiled(uint64_t *fullBar, uint32_t bytes, const CUtensorMap *mapW, void *dstW,
                                                      int w0, int w1, int w2, const CUtensorMap *mapX, void *dstX, int x0,
                                                      int x1, int x2, uint64_t *peekBar, uint32_t peekParity) {
    uint32_t ready;
    asm volatile("{\n\t.reg .pred q;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
                 "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %4;\n\t"
                 "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%5], [%6, {%7, %8, %9}], [%3];\n\t"
                 "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%10], [%11, {%12, %13, %14}], [%3];\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ready)
                 : "r"(smemAddr(peekBar)), "r"(peekParity), "r"(smemAddr(fullBar)), "r"(bytes), "r"(smemAddr(dstW)),
                   "l"(reinterpret_cast<uint64_t>(mapW)), "r"(w0), "r"(w1), "r"(w2), "r"(smemAddr(dstX)),
                   "l"(reinterpret_cast<uint64_t>(mapX)), "r"(x0), "r"(x1), "r"(x2)
                 : "memory");
    return ready;
}
// The same with the pixel tile fetched in im2col mode (see tmaLoadIm2col4d).
__device__ __forceinline__ uint32_t tmaStagePeekIm2col(uint64_t *fullBar, uint32_t bytes, const CUtensorMap *mapW, void *dstW,
                                                       int w0, int w1, int w2, const CUtensorMap *mapX, void *dstX, int c,
                                                       int w, int h, int n, uint16_t offW, uint16_t offH, uint64_t *peekBar,
                                                       uint32_t peekParity) {
    uint32_t ready;
    asm volatile("{\n\t.reg .pred q;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
                 "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %4;\n\t"
                 "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%5], [%6, {%7, %8, %9}], [%3];\n\t"
                 "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
                 "[%10], [%11, {%12, %13, %14, %15}], [%3], {%16, %17};\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ready)
                 : "r"(smemAddr(peekBar)), "r"(peekParity), "r"(smemAddr(fullBar)), "r"(bytes), "r"(smemAddr(dstW)),
                   "l"(reinterpret_cast<uint64_t>(mapW)), "r"(w0), "r"(w1), "r"(w2), "r"(smemAddr(dstX)),
                   "l"(reinterpret_cast<uint64_t>(mapX)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(offW), "h"(offH)
                 : "memory");
    return ready;
}

// Shared-memory matrix descriptor for a SWIZZLE_128B tile whose 8-row groups are 1024 bytes apart.
// bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
// [46,48) descriptor version (1 on sm_100), [61,64) layout type (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t smemDesc(uint32_t addr, uint32_t lboBytes, uint32_t sboBytes) {
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFF);
    d |= uint64_t((lboBytes >> 4) & 0x3FFF) << 16;
    d |= uint64_t((sboBytes >> 4) & 0x3FFF) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}

// Instruction descriptor for kind::i8: D = s32 (c_format 2), A and B signed 8-bit (format 1),
// bit 15/16 = A/B major (0 = K-major, 1 = MN-major), [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t instrDesc(int n, bool bMnMajor) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(bMnMajor) << 16) | (uint32_t(n >> 3) << 17) |
           (uint32_t(BM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
}
__device__ __forceinline__ void ummaCommit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar))
                 : "memory");
}
// One 128-byte K block: up to four MMAs of 32 bytes of K each (`count` of them: the tail of a K block that only
// holds zero fill is skipped; descriptors advance by stepA / stepB units of 16 bytes, 2 for a K-major SWIZZLE_128B
// tile), the commit that hands the stage back, and -- issued AHEAD of them -- a non-blocking test of the barrier the
// next K block will wait for.  Why in one statement: an mbarrier test issued after MMAs and a commit takes about 185
// cycles to answer even when the phase has long completed (it queues behind them), and the thread that needs the
// answer stalls for it; measured on a loop of this shape, 626 cycles per K block whatever N is, against 384 for the
// four MMAs of N = 192 alone.  Asked before the MMAs are issued, the answer arrives while they and the commit go out
// (463 cycles per K block; 513 = the pipe's own time at N = 256).  Returns 1 when the next barrier's phase
// `peekParity` is complete; 0 means "not yet known": wait for it in the ordinary way.
__device__ __forceinline__ uint32_t ummaBlockPeek(uint32_t tmemD, uint64_t descA, uint64_t stepA, uint64_t descB,
                                                  uint64_t stepB, uint32_t idesc, uint32_t accumulateFirst, int count,
                                                  uint64_t *commitBar, uint64_t *peekBar, uint32_t peekParity) {
    uint32_t ready;
    asm volatile("{\n\t.reg .pred q, a0, a1, g1, g2, g3;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
                 "setp.ne.b32 a0, %9, 0;\n\t"
                 "setp.ne.b32 a1, %10, 0;\n\t"
                 "setp.gt.s32 g1, %17, 1;\n\t"
                 "setp.gt.s32 g2, %17, 2;\n\t"
                 "setp.gt.s32 g3, %17, 3;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%3], %4, %5, %8, {%11, %11, %11, %11}, a0;\n\t"
                 "@g1 tcgen05.mma.cta_group::1.kind::i8 [%3], %6, %7, %8, {%11, %11, %11, %11}, a1;\n\t"
                 "@g2 tcgen05.mma.cta_group::1.kind::i8 [%3], %12, %13, %8, {%11, %11, %11, %11}, a1;\n\t"
                 "@g3 tcgen05.mma.cta_group::1.kind::i8 [%3], %14, %15, %8, {%11, %11, %11, %11}, a1;\n\t"
                 "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%16];\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ready)
                 : "r"(smemAddr(peekBar)), "r"(peekParity), "r"(tmemD), "l"(descA), "l"(descB), "l"(descA + stepA),
                   "l"(descB + stepB), "r"(idesc), "r"(accumulateFirst), "r"(1u), "r"(0u), "l"(descA + 2 * stepA),
                   "l"(descB + 2 * stepB), "l"(descA + 3 * stepA), "l"(descB + 3 * stepB), "r"(smemAddr(commitBar)), "r"(count)
                 : "memory");
    return ready;
}
// How many of a K block's four MMAs have anything but zero fill to multiply: `valid` = bytes of K in the block.
__device__ __forceinline__ int ummaCountFor(int valid) { return valid >= BK ? BK / UMMA_K : (valid + UMMA_K - 1) / UMMA_K; }
__device__ __forceinline__ void tmemLoad16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}

// Waits for this warp's outstanding tcgen05.ld.  The loaded registers pass through the statement so that the
// compiler cannot schedule a use of them above the wait.
__device__ __forceinline__ void tmemWait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

// Programmatic dependent launch.  A kernel launched with launchDependent() may start while the kernel before
// it in the stream is still running (on SMs that kernel has already left): everything up to this call - barrier
// and TMEM set-up, tables built from graph constants - overlaps the predecessor's tail.  The wait returns when
// the predecessor has completed and its writes are visible; nothing before it may touch memory that another
// kernel of the stream writes or reads for writing later.  The trigger lets the successor start as early as
// it finds room.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void gridDependencySync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Barrier among the epilogue warps only (named barrier 1).
// n / f.d for n < 2^31 (see FastDiv)
__device__ __forceinline__ uint32_t fastDiv(uint32_t n, const FastDiv &f) {
    return f.mul == 0u ? n : __umulhi(n, f.mul) >> f.shift;
}

__device__ __forceinline__ void epilogueSync() {
    asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
}

// ---- implicit-GEMM gather of one tile row per K block (im2col on the fly) -------------------------------
// The K axis of a convolution is (ky, kx, channel).  When the channel count is 16, 32, 64 or a multiple of
// 128, a 128-byte K block splits into equal segments of 16 * SEG contiguous bytes of one tap, and which tap
// (and which channel offset) a segment covers is the same for every row of the tile.  A row then only
// needs, once per tile, the address of its window's first tap and a bit mask of its in-range taps; per
// segment it adds a tabulated tap offset and issues SEG 16-byte copies (zero-filled when the tap is out
// of range).  This keeps the producer warps at a handful of instructions per K block.
constexpr int kMaxTaps = 64;       // bits of the in-range mask
constexpr int kTapTabEntries = 80; // taps plus the run-off of the last K block

struct GatherRow {
    const int8_t *origin; // address of tap (0, 0), channel 0 of the window; may lie outside the tensor
    uint64_t mask;        // bit ky * KW + kx: that tap is inside the tensor
};

template <class Params>
__device__ __forceinline__ bool fastGatherApplies(const Params &p) {
    return p.gatherTable == nullptr && p.KH * p.KW <= kMaxTaps &&
           (p.IC == 16 || p.IC == 32 || p.IC == 64 || p.IC % 128 == 0);
}

// Byte offset of tap t from tap 0 (0 past the window); filled once per CTA by the producer warps.
template <class Params>
__device__ __forceinline__ void fillTapTable(const Params &p, int32_t *tapTab, int firstThread, int numThreads) {
    for (int t = int(threadIdx.x) - firstThread; t < kTapTabEntries; t += numThreads) {
        const int ky = t / p.KW, kx = t - ky * p.KW;
        tapTab[t] = ky < p.KH ? (ky * p.dilY * p.W + kx * p.dilX) * p.IC : 0;
    }
}

template <class Params>
__device__ __forceinline__ GatherRow gatherRowSetup(const Params &p, int64_t m) {
    GatherRow r;
    r.origin = p.in;
    r.mask = 0;
    if (m < p.M) {
        const int n = int(fastDiv(uint32_t(m), p.divPlane));
        const int rem = int(uint32_t(m) - uint32_t(n) * p.divPlane.d);
        const int oy = int(fastDiv(uint32_t(rem), p.divOW)), ox = rem - oy * p.OW;
        const int iy0 = oy * p.strideY - p.padTop, ix0 = ox * p.strideX - p.padLeft;
        uint32_t colMask = 0;
        for (int kx = 0; kx < p.KW; ++kx) {
            const int x = ix0 + kx * p.dilX;
            colMask |= (x >= 0 && x < p.W) ? (1u << kx) : 0u;
        }
        for (int ky = 0; ky < p.KH; ++ky) {
            const int y = iy0 + ky * p.dilY;
            if (y >= 0 && y < p.H) {
                r.mask |= uint64_t(colMask) << (ky * p.KW);
            }
        }
        const int64_t off = ((int64_t(n) * p.H + iy0) * p.W + ix0) * p.IC;
        r.origin = reinterpret_cast<const int8_t *>(reinterpret_cast<intptr_t>(p.in) + off);
    }
    return r;
}

// One 128-byte K block for ROWS tile rows (ROW_STEP rows apart, a multiple of 8) of one thread.  (t, c0) is the running position
// on the K axis: tap index and channel offset of the next segment.
template <int SEG, int ROWS, int ROW_STEP>
__device__ __forceinline__ void gatherSegments(const GatherRow (&rows)[ROWS], const int32_t *tapTab, int taps, int IC,
                                               int &t, int &c0, uint32_t dstRow, uint32_t swz, const int8_t *dummy) {
#pragma unroll
    for (int sg = 0; sg < 8 / SEG; ++sg) {
        const bool tapInWindow = t < taps;
        const int32_t off = tapTab[t] + c0;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const bool valid = tapInWindow && ((rows[r].mask >> (t & 63)) & 1ull) != 0;
            const int8_t *src = valid ? rows[r].origin + off : dummy;
            const uint32_t bytes = valid ? 16u : 0u; // 0 source bytes: the 16 bytes are zero-filled
#pragma unroll
            for (int j = 0; j < SEG; ++j) {
                const uint32_t dst = dstRow + uint32_t(r * ROW_STEP * 128) + ((uint32_t(sg * SEG + j) ^ swz) << 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src + 16 * j), "r"(bytes)
                             : "memory");
            }
        }
        c0 += SEG * 16;
        if (c0 >= IC) {
            c0 = 0;
            ++t;
        }
    }
}

template <int ROWS, int ROW_STEP = 128>
__device__ __forceinline__ void gatherBlock(const GatherRow (&rows)[ROWS], const int32_t *tapTab, int taps, int IC, int &t,
                                            int &c0, uint32_t dstRow, uint32_t swz, const int8_t *dummy) {
    if (IC >= 128) {
        gatherSegments<8, ROWS, ROW_STEP>(rows, tapTab, taps, IC, t, c0, dstRow, swz, dummy);
    } else if (IC == 64) {
        gatherSegments<4, ROWS, ROW_STEP>(rows, tapTab, taps, IC, t, c0, dstRow, swz, dummy);
    } else if (IC == 32) {
        gatherSegments<2, ROWS, ROW_STEP>(rows, tapTab, taps, IC, t, c0, dstRow, swz, dummy);
    } else {
        gatherSegments<1, ROWS, ROW_STEP>(rows, tapTab, taps, IC, t, c0, dstRow, swz, dummy);
    }
}


// ---- host side ----
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encodeTiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    });
    return fn;
}

// 3-D uint8 tensor map {d0 (contiguous), d1, d2} with a {b0, b1, 1} box and 128-byte swizzle.
inline bool makeMap(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1,
             uint64_t stride2, uint32_t b0, uint32_t b1, bool swizzle128 = true) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        setLastError("cuTensorMapEncodeTiled is not available from the driver");
        return false;
    }
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {stride1, stride2}; // bytes, for dims 1 and 2
    const cuuint32_t box[3] = {b0, b1, 1};
    const cuuint32_t elemStrides[3] = {1, 1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box,
                           elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        setLastError("cuTensorMapEncodeTiled failed with code " + std::to_string(int(rc)));
        return false;
    }
    return true;
}

// Weights [OC][taps][IC] (OHWI) as a 3-D map {IC, taps, OC} with a {128, 1, rows} box: one load brings 128
// channels of one tap for `rows` output channels, zero-filled past IC.  Pairs with the im2col map below, whose
// loads are padded the same way, so that any channel count that is a multiple of 16 works.
inline bool makeWeightTapMap(CUtensorMap *map, const void *base, int IC, int taps, int OC, uint32_t rows) {
    EncodeTiledFn fn = encodeTiled();
    if (fn == nullptr) {
        return false;
    }
    const cuuint64_t dims[3] = {cuuint64_t(IC), cuuint64_t(taps), cuuint64_t(OC)};
    const cuuint64_t strides[2] = {cuuint64_t(IC), cuuint64_t(IC) * taps};
    const cuuint32_t box[3] = {128, 1, rows};
    const cuuint32_t elemStrides[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, elemStrides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

using EncodeIm2colFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

inline EncodeIm2colFn encodeIm2col() {
    static EncodeIm2colFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeIm2colFn>(sym);
        }
    });
    return fn;
}

// Im2col tensor map over an int8 NHWC tensor for a convolution window: 128 channels per pixel (one 128-byte
// swizzled row per window position), `pixels` window positions per load.  The bounding box of the windows'
// first taps runs from -pad to the last position a window still fits with its far-side padding.
// Returns false without setting an error text when the driver refuses the geometry.
inline bool makeIm2colMap(CUtensorMap *map, const void *base, int N, int H, int W, int C, int KH, int KW, int padTop,
                          int padLeft, int OH, int OW, int strideY, int strideX, int dilY, int dilX, uint32_t pixels) {
    EncodeIm2colFn fn = encodeIm2col();
    if (fn == nullptr) {
        return false;
    }
    const cuuint64_t dims[4] = {cuuint64_t(C), cuuint64_t(W), cuuint64_t(H), cuuint64_t(N)};
    const cuuint64_t strides[3] = {cuuint64_t(C), cuuint64_t(C) * W, cuuint64_t(C) * W * H};
    // the last window of a row starts at (OW - 1) * stride - pad; relative to the tensor's last pixel W - 1
    const int lower[2] = {-padLeft, -padTop};
    const int upper[2] = {(OW - 1) * strideX - padLeft - (W - 1), (OH - 1) * strideY - padTop - (H - 1)};
    for (int i = 0; i < 2; ++i) {
        if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) {
            return false;
        }
    }
    if ((KW - 1) * dilX > 255 || (KH - 1) * dilY > 255 || strideX > 8 || strideY > 8) {
        return false;
    }
    const cuuint32_t elemStrides[4] = {1, cuuint32_t(strideX), cuuint32_t(strideY), 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, lower, upper, 128,
                           pixels, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// Launches `kernel` so that it may overlap the end of its predecessor in the stream (see gridDependencySync).
template <class... Params, class... Args>
inline cudaError_t launchDependent(void (*kernel)(Params...), int grid, int threads, size_t smemBytes, cudaStream_t stream,
                                   Args &&...args) {
    const bool disabled = tensorCoreTuning().dependentLaunch.load(std::memory_order_relaxed) == 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(threads));
    cfg.dynamicSmemBytes = smemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = disabled ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Number of SMs of the device that is current (cached per device).
inline int smCount() {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> counts[kMaxDevices];
    int dev = 0;
    cudaGetDevice(&dev);
    const bool cached = dev >= 0 && dev < kMaxDevices;
    int count = cached ? counts[dev].load(std::memory_order_relaxed) : 0;
    if (count == 0) {
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) {
            count = kNumSMs;
        }
        if (cached) {
            counts[dev].store(count, std::memory_order_relaxed);
        }
    }
    return count;
}

// Opts `kernel` in to `bytes` of dynamic shared memory on the device that is current.  The attribute belongs to
// the (kernel, device) pair, so it is set once for each; safe to call from several host threads.
inline bool allowDynamicSmem(const void *kernel, size_t bytes) {
    static std::mutex mutex;
    static std::set<std::pair<const void *, int>> done;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mutex);
    if (done.count({kernel, dev}) != 0) {
        return true;
    }
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess) {
        setLastError("cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
        return false;
    }
    done.insert({kernel, dev});
    return true;
}

} // namespace tc
} // namespace mlel
