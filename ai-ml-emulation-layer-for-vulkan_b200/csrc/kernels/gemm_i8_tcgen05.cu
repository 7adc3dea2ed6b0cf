// int8 x int8 -> int32 contraction on the 5th-generation tensor cores (tcgen05.mma kind::i8, TMEM
// accumulator) with the TOSA epilogue fused in.  One persistent kernel serves CONV2D (implicit GEMM),
// 1x1 CONV2D and MATMUL:
//
//   D[m, n] = sum_k A[m, k] * B[n, k]         m: output pixel (or matmul row), n: output channel
//
//   A operand  - TMA tile loads when A is a plain row-major matrix (1x1 stride-1 convolution, MATMUL);
//              - TMA im2col loads for a convolution window over a multiple of 16 channels: one instruction
//                fetches one tap, 128 channels (zero-filled past the last one), of the tile's 128 windows;
//              - otherwise gathered by four producer warps with cp.async: 16-byte pieces with bounds
//                checks (any kernel size, stride, dilation and padding; out-of-range taps zero-filled), or
//                4/8/16-byte pieces at tabulated offsets from a zero-padded copy of the input (channel
//                counts that are not multiples of 16, e.g. an RGB stem)
//   B operand  - TMA tile loads of the K-major weight matrix [N][K] (OHWI weights are exactly that; in im2col
//                mode through a {IC, taps, OC} map that pads each tap like the A loads), or of an N-major
//                [K][N] matrix with an MN-major descriptor
//   schedule   - one CTA per SM walks the output tiles (n fastest, so concurrently running CTAs share
//                their A rows in L2); 128-byte K blocks in SWIZZLE_128B shared-memory tiles form an
//                mbarrier ring that runs on across tiles; two TMEM accumulators alternate so that the
//                epilogue of tile i overlaps the main loop of tile i+1
//   warps      - 0-15 epilogue (four per TMEM lane quarter, each a quarter of the columns), 16 TMA
//                producer, 17 MMA issuer and TMEM owner, 18-21 A gather (gathered variants only)
//   epilogue   - tcgen05.ld of the int32 accumulator, zero-point/bias correction, then either a raw
//                int32 store or RESCALE (+CLAMP, + residual RESCALE/ADD/RESCALE) to int8, with the
//                per-column constants read from shared memory
//
// Fused int8 convolutions with more than 64 output channels run on the channel-major companion kernel
// (gemm_i8_ocmajor.cu) instead, whose epilogue keeps the per-channel constants in registers.
//
// Exactness.  The tensor core sums raw products A*B in int32 (no overflow is possible for K <= 65536).
// The reference computes sum over in-range taps of (x - zx) * w  (conv2d.comp:59-96).  With zero-filled
// out-of-range taps this equals  sum(x * w) - zx * sum over in-range taps of w, and the second term only
// depends on the output channel and on which taps are in range, i.e. on a small "border class" of the
// output pixel.  The host tabulates corr[class][n] = bias[n] - zx * sum_valid_taps(w[n]) once per
// pipeline; the epilogue adds it (mod 2^32, like the reference's int32 arithmetic).
//
// Every wait on an mbarrier is bounded: after about two seconds a waiter records an error code in
// g_tcgen05Error and leaves its loop, all roles fall through to the common exit, and TMEM is freed.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "gemm_i8_tcgen05.hpp"
#include "tcgen05_common.cuh"

namespace mlel {

namespace {

using namespace tc;

struct __align__(8) PipeBarriers {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t accFull[2];
    uint64_t accEmpty[2];
    uint32_t tmemBase;
    uint32_t pad;
};

// Constants of the main RESCALE stage for one output column (see FastRescale): two shared-memory reads per
// element, by shared address.  A table is built in one of two forms.  General: {mult, corr0, rnLo, rnHi} with the
// rounding constant for v < zpIn (input zero point folded in).  High-word form, when every shift of the table is
// at least 32 and the corrections are small (see scaleHigh): {mult, corr0 - zpIn, rnM} with the rounding constant
// without the zero-point fold.  32-bit form, when in addition every shift is at most 60 and the host has bounded
// |x| below 2^29 (see scaleHigh32): {mult, 4 * (corr0 - zpIn), rounding units, shift - 30} -- one read per element.
struct __align__(16) ColConst {
    int32_t mult;
    int32_t corr;        // general: correction of the most common border class; high-word form: that minus zpIn
    uint32_t rnLo, rnHi; // rounding constant (see above)
    int32_t s2;          // max(shift - 32, 0)
    uint32_t bump;       // what the constant for v >= zpIn adds: 2^31 with double rounding and shift > 31, else 0
    int32_t s1;          // min(shift, 32)
    int32_t corr0;       // correction of the most common border class (what a border pixel swaps for its own)
};

// High word of (accumulator + correction - zpIn) * mult + rounding: with x = v - zpIn the double-rounding test
// v >= zpIn is the sign of x, and bumpMask (2^31 or 0) & ~x adds the 2^31 for x >= 0.  The caller shifts the high
// word by shift - 32.  Exact while x does not overflow, which the host's bound on the corrections guarantees.
__device__ __forceinline__ int32_t scaleHigh(int32_t x, int32_t mult, uint64_t rn, uint32_t bumpMask) {
    const uint64_t prod = uint64_t(int64_t(x) * int64_t(mult));
    const uint32_t extra = ~uint32_t(x) & bumpMask;
    const uint64_t sum = prod + rn + uint64_t(extra);
    return int32_t(uint32_t(sum >> 32));
}

__device__ __forceinline__ void ldsV2(uint32_t addr, uint32_t &a, uint32_t &b) {
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}
__device__ __forceinline__ int32_t ldsS32(uint32_t addr) {
    int32_t v;
    asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void ldsV4(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}

constexpr int kAGather = 0, kATiled = 1, kAIm2col = 2;
constexpr int kMaxGatherPieces = 1024; // entries of the shared-memory copy of GemmI8Params::gatherTable

struct TileCoord {
    int m0, n0, batch;
};

// Packs the low bytes of four int32 values, e0 in the lowest byte (values are already clamped to int8).
__device__ __forceinline__ uint32_t pack4(int32_t e0, int32_t e1, int32_t e2, int32_t e3) {
    const uint32_t lo = __byte_perm(uint32_t(e0), uint32_t(e1), 0x0040);
    const uint32_t hi = __byte_perm(uint32_t(e2), uint32_t(e3), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

// The epilogue of the persistent kernel (warps 0-15).  Each warp owns 32 TMEM lanes (tile rows) and a quarter
// of the tile's columns, which it walks in 16-column steps: one tcgen05.ld, 16 RESCALEs, one 16-byte store.
// 16 columns of one row in the 32-bit form of the constants table (see ColConst), packed four results to a word.
template <bool SIGNED>
__device__ __forceinline__ void rescale16Words32(const uint32_t (&acc)[16], uint32_t tabAddr, int32_t outZp, int32_t lo,
                                                 int32_t hi, uint32_t (&packed)[4]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        int32_t y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = 4 * q + e;
            uint32_t mult, corrX4, c32, shift32;
            ldsV4(tabAddr + uint32_t(j) * 32u, mult, corrX4, c32, shift32);
            const int32_t x4 = int32_t(acc[j] * 4u + corrX4);
            const int32_t h = scaleHigh32<SIGNED>(x4, int32_t(mult), int32_t(c32));
            y[e] = min(__viaddmax_s32(h >> shift32, outZp, lo), hi);
        }
        packed[q] = pack4(y[0], y[1], y[2], y[3]);
    }
}

template <int BN, int NSTAGE, bool RESIDUAL>
__device__ __forceinline__ void epilogueInt8(const GemmI8Params &p, PipeBarriers *bars, ColConst *colTab,
                                             uint32_t tmemBase, int warp, int lane, int64_t numTiles, int mTiles,
                                             int nTiles) {
    const int quarter = warp & 3; // TMEM lanes [32 * quarter, 32 * quarter + 32)
    const int half = warp >> 2;   // which half of the tile's columns
    constexpr int kColsPerWarp = BN / (kEpilogueWarps / 4);
    constexpr int kSteps = kColsPerWarp / 16;
    const int row = quarter * 32 + lane;
    FastRescale fa{}, fb{}, fo{};
    if (RESIDUAL) {
        fa = makeFastRescale(__ldg(p.epi.a.mult), int32_t(__ldg(p.epi.a.shift)), p.epi.a.inZp, p.epi.a.doubleRound != 0);
        fb = makeFastRescale(__ldg(p.epi.b.mult), int32_t(__ldg(p.epi.b.shift)), p.epi.b.inZp, p.epi.b.doubleRound != 0);
        fo = makeFastRescale(__ldg(p.epi.out.mult), int32_t(__ldg(p.epi.out.shift)), p.epi.out.inZp,
                             p.epi.out.doubleRound != 0);
    }
    const int32_t zpMain = p.epi.main.inZp, outZpMain = p.epi.main.outZp;
    const uint32_t tabAddr = smemAddr(colTab);
    // what holds for every column of the table -- bit 0: a shift of at least 32; bit 1: a shift of 32..60; bit 2: no
    // negative multiplier
    volatile uint32_t *fastFlag = &bars->pad;
    bool fast = false, high = false, words32 = false, signFree = false; // forms of the table: see ColConst
    const uint32_t bumpMask = p.epi.main.doubleRound != 0 ? 0x80000000u : 0u;
    const int32_t loMain = p.epi.main.lo, hiMain = p.epi.main.hi;
    uint32_t tileCount = 0;
    int tabN0 = -1, tabBatch = -1; // what the shared constants table was built for
    for (int64_t t = blockIdx.x; t < numTiles; t += gridDim.x, ++tileCount) {
        // the launcher refuses 2^31 tiles and more: divisions by multiply-high (see FastDiv)
        const uint32_t overN = fastDiv(uint32_t(t), p.divTiles0), overM = fastDiv(overN, p.divTiles1);
        const int n0 = int(uint32_t(t) - overN * uint32_t(nTiles)) * BN;
        const int m0 = int(overN - overM * uint32_t(mTiles)) * BM;
        const int batch = int(overM);
        const uint32_t buf = tileCount & 1u;
        const int32_t *corrBatch = p.corr + (p.batchedCorr ? int64_t(batch) * p.numClasses * p.N : 0);
        // Per-column constants shared by the 128 rows of the tile: the main RESCALE stage and the correction
        // of the most common border class.
        if (n0 != tabN0 || (p.batchedCorr && batch != tabBatch)) {
            epilogueSync(); // everyone is done with the previous table
            if (threadIdx.x == 0) {
                *fastFlag = 7;
            }
            epilogueSync();
            FastRescale f{};
            int32_t corr0 = 0;
            if (threadIdx.x < BN) {
                const int col = n0 + int(threadIdx.x);
                const int ci = (p.epi.main.perChannel && col < p.N) ? col : 0;
                f = makeFastRescale(__ldg(p.epi.main.mult + ci), int32_t(__ldg(p.epi.main.shift + ci)), zpMain,
                                    p.epi.main.doubleRound != 0);
                const int shift = f.s1 + f.s2;
                // (a shift below 32 in this tile: the low word of the product matters)
                const uint32_t fails = (f.s1 != 32 ? 1u : 0u) | ((shift < 32 || shift > 60) ? 2u : 0u) | (f.mult < 0 ? 4u : 0u);
                if (fails != 0) {
                    atomicAnd(const_cast<uint32_t *>(fastFlag), ~fails);
                }
                corr0 = col < p.N ? __ldg(corrBatch + int64_t(p.baseClass) * p.N + col) : 0;
            }
            epilogueSync();
            const uint32_t holds = *fastFlag;
            fast = (holds & 1u) != 0;
            high = fast && p.corrSmall != 0 && !RESIDUAL;
            words32 = high && p.corrSmall >= 2 && (holds & 2u) != 0;
            // the sign of x only matters to double rounding, and not where every x < 0 ends at the lower clamp bound
            signFree = p.epi.main.doubleRound == 0 || (loMain >= outZpMain && (holds & 4u) != 0);
            if (threadIdx.x < BN) {
                ColConst c;
                c.mult = f.mult, c.s1 = f.s1, c.s2 = f.s2, c.corr0 = corr0;
                c.bump = f.rpLo - f.rnLo; // (rp - rn) mod 2^32: 0 or 2^31
                if (words32) {
                    const int shift = f.s1 + f.s2;
                    c.corr = int32_t((uint32_t(corr0) - uint32_t(f.zpIn)) * 4u);
                    c.rnLo = (1u << ((shift - 31) & 31)) + (p.epi.main.doubleRound != 0 ? 1u : 0u);
                    c.rnHi = uint32_t(shift - 30);
                } else if (high) {
                    const bool twoRounds = p.epi.main.doubleRound != 0;
                    const uint64_t rn = (uint64_t(1) << (f.s1 + f.s2 - 1)) - (twoRounds ? (uint64_t(1) << 30) : 0);
                    c.corr = int32_t(uint32_t(corr0) - uint32_t(f.zpIn));
                    c.rnLo = uint32_t(rn), c.rnHi = uint32_t(rn >> 32);
                } else {
                    c.corr = corr0, c.rnLo = f.rnLo, c.rnHi = f.rnHi;
                }
                colTab[threadIdx.x] = c;
            }
            epilogueSync();
            tabN0 = n0;
            tabBatch = batch;
        }
        const int64_t m = int64_t(m0) + row;
        const bool rowValid = m < p.M;
        int cls = p.baseClass;
        if (p.rowClass != nullptr && rowValid) {
            const uint32_t rem = uint32_t(m) - fastDiv(uint32_t(m), p.divPlane) * p.divPlane.d; // pixel inside its image
            const uint32_t oy = fastDiv(rem, p.divOW);
            cls = int(__ldg(p.rowClass + oy)) * p.numColClasses + int(__ldg(p.colClass + (rem - oy * uint32_t(p.OW))));
        }
        const int64_t outRow = (int64_t(batch) * p.M + m) * p.ldOut;

        if (!mbarWait(&bars->accFull[buf], (tileCount >> 1) & 1u, 4)) {
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmemBase + buf * uint32_t(BN) + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
        for (int st = 0; st < kSteps; ++st) {
            const int cl = half * kColsPerWarp + st * 16; // column inside the tile
            uint32_t acc[16];
            tmemLoad16(taddr + uint32_t(cl), acc);
            tmemWait16(acc);
            if (st == kSteps - 1) {
                // this warp's part of the accumulator is in registers: hand the buffer back to the MMA warp
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                if (lane == 0) {
                    mbarArrive(&bars->accEmpty[buf]);
                }
            }
            const int col0 = n0 + cl;
            if (!rowValid || col0 >= p.N) {
                continue;
            }
            const int ncols = min(16, p.N - col0);
            int8_t *dst = p.out8 + outRow + col0;
            const bool vec = ncols == 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
            if (cls != p.baseClass) {
                // a pixel whose window crosses the border: swap the table's correction for its own class's
                const int32_t *own = corrBatch + int64_t(cls) * p.N + col0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j < ncols) {
                        acc[j] += uint32_t(__ldg(own + j)) - uint32_t(colTab[cl + j].corr0);
                    }
                }
            }
            uint32_t sc[4] = {0, 0, 0, 0}; // 16 shortcut bytes of this row
            if (RESIDUAL) {
                const int8_t *scp = p.epi.shortcut + outRow + col0;
                if (vec) {
                    const int4 s0 = __ldg(reinterpret_cast<const int4 *>(scp));
                    sc[0] = uint32_t(s0.x), sc[1] = uint32_t(s0.y), sc[2] = uint32_t(s0.z), sc[3] = uint32_t(s0.w);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (j < ncols) {
                            sc[j >> 2] |= uint32_t(uint8_t(scp[j])) << (8 * (j & 3));
                        }
                    }
                }
            }
            uint32_t packed[4];
            if (!RESIDUAL && words32) {
                // (two copies of the loop behind one branch: as a select per element the compiler computed the sign
                // term for every element and dropped it afterwards)
                if (signFree) {
                    rescale16Words32<false>(acc, tabAddr + uint32_t(cl) * 32u, outZpMain, loMain, hiMain, packed);
                } else {
                    rescale16Words32<true>(acc, tabAddr + uint32_t(cl) * 32u, outZpMain, loMain, hiMain, packed);
                }
            } else if (!RESIDUAL && high) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    int32_t y[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 4 * q + e;
                        uint32_t mult, corrX, rnLo, rnHi;
                        ldsV4(tabAddr + uint32_t(cl + j) * 32u, mult, corrX, rnLo, rnHi);
                        const int32_t s2 = ldsS32(tabAddr + uint32_t(cl + j) * 32u + 16u);
                        const int32_t h = scaleHigh(int32_t(acc[j] + corrX), int32_t(mult), (uint64_t(rnHi) << 32) | rnLo,
                                                    bumpMask);
                        y[e] = min(__viaddmax_s32(h >> s2, outZpMain, loMain), hiMain);
                    }
                    packed[q] = pack4(y[0], y[1], y[2], y[3]);
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    int32_t y[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 4 * q + e;
                        uint32_t mult, corr0, rnLo, rnHi, s2, bump;
                        ldsV4(tabAddr + uint32_t(cl + j) * 32u, mult, corr0, rnLo, rnHi);
                        ldsV2(tabAddr + uint32_t(cl + j) * 32u + 16u, s2, bump);
                        const int32_t v = int32_t(acc[j] + corr0);
                        // the double-rounding choice is the third input of the 64-bit addition after the multiply
                        const uint64_t sum = uint64_t(int64_t(v) * int64_t(int32_t(mult))) + ((uint64_t(rnHi) << 32) | rnLo) +
                                             uint64_t(v >= zpMain ? bump : 0u);
                        int32_t q32;
                        if (fast) {
                            q32 = int32_t(uint32_t(sum >> 32)); // shifts of 32 and more only see the high word
                        } else {
                            const uint32_t s1 = uint32_t(ldsS32(tabAddr + uint32_t(cl + j) * 32u + 24u));
                            q32 = int32_t(__funnelshift_rc(uint32_t(sum), uint32_t(sum >> 32), s1));
                        }
                        int32_t r = min(__viaddmax_s32(q32 >> s2, outZpMain, loMain), hiMain);
                        if (RESIDUAL) {
                            const int32_t ta = fastRescale(fa, r, p.epi.a.outZp, p.epi.a.lo, p.epi.a.hi);
                            const int32_t sv = int32_t(int8_t(sc[q] >> (8 * e)));
                            const int32_t tb = fastRescale(fb, sv, p.epi.b.outZp, p.epi.b.lo, p.epi.b.hi);
                            r = fastRescale(fo, int32_t(uint32_t(ta) + uint32_t(tb)), p.epi.out.outZp, p.epi.out.lo,
                                            p.epi.out.hi);
                        }
                        y[e] = r;
                    }
                    packed[q] = pack4(y[0], y[1], y[2], y[3]);
                }
            }
            if (vec) {
                *reinterpret_cast<int4 *>(dst) = make_int4(int(packed[0]), int(packed[1]), int(packed[2]), int(packed[3]));
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j < ncols) {
                        dst[j] = int8_t(packed[j >> 2] >> (8 * (j & 3)));
                    }
                }
            }
        }
    }
}

// int32 output: accumulator + correction, no RESCALE.
// `staging` (or null): 32 rows x 16 int32 per epilogue warp, rows kStageInts words apart.  A thread holds 16 columns of
// ONE row, so a warp's 16-byte stores would go to 32 different rows (32 lines per instruction); through the staging
// block four lanes write one row's 64 bytes and an instruction touches 8 lines.  (The attention-score product of the
// BERT-shaped encoder, 226 MB of int32 per layer: 140 -> about 85 us.)
constexpr int kStageInts = 20;                      // 16 values + 4 words of padding: no shared-memory bank conflicts
constexpr int kStageBytesPerWarp = 32 * kStageInts * 4;
template <int BN, int NSTAGE>
__device__ __forceinline__ void epilogueInt32(const GemmI8Params &p, PipeBarriers *bars, uint32_t tmemBase, int warp,
                                              int lane, int64_t numTiles, int mTiles, int nTiles, int32_t *staging) {
    const int quarter = warp & 3;
    const int half = warp >> 2;
    constexpr int kColsPerWarp = BN / (kEpilogueWarps / 4);
    constexpr int kSteps = kColsPerWarp / 16;
    const int row = quarter * 32 + lane;
    uint32_t tileCount = 0;
    for (int64_t t = blockIdx.x; t < numTiles; t += gridDim.x, ++tileCount) {
        // the launcher refuses 2^31 tiles and more: divisions by multiply-high (see FastDiv)
        const uint32_t overN = fastDiv(uint32_t(t), p.divTiles0), overM = fastDiv(overN, p.divTiles1);
        const int n0 = int(uint32_t(t) - overN * uint32_t(nTiles)) * BN;
        const int m0 = int(overN - overM * uint32_t(mTiles)) * BM;
        const int batch = int(overM);
        const uint32_t buf = tileCount & 1u;
        const int64_t m = int64_t(m0) + row;
        const bool rowValid = m < p.M;
        const int32_t *corr = p.corr;
        if (corr != nullptr) {
            int cls = 0;
            if (p.rowClass != nullptr && rowValid) {
                // m < 2^31 and the output plane is smaller: 32-bit divisions (a 64-bit one is a long subroutine)
                const uint32_t rem = uint32_t(m) % (uint32_t(p.OH) * uint32_t(p.OW));
                cls = int(__ldg(p.rowClass + rem / uint32_t(p.OW))) * p.numColClasses + int(__ldg(p.colClass + rem % uint32_t(p.OW)));
            }
            corr += (p.batchedCorr ? int64_t(batch) * p.numClasses * p.N : 0) + int64_t(cls) * p.N;
        }
        const int64_t outRow = (int64_t(batch) * p.M + m) * p.ldOut;
        if (!mbarWait(&bars->accFull[buf], (tileCount >> 1) & 1u, 4)) {
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmemBase + buf * uint32_t(BN) + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
        for (int st = 0; st < kSteps; ++st) {
            const int cl = half * kColsPerWarp + st * 16;
            uint32_t acc[16];
            tmemLoad16(taddr + uint32_t(cl), acc);
            tmemWait16(acc);
            if (st == kSteps - 1) {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                if (lane == 0) {
                    mbarArrive(&bars->accEmpty[buf]);
                }
            }
            const int col0 = n0 + cl;
            if (staging != nullptr && col0 + 16 <= p.N) {
                // whole 16-column block inside the matrix (rows past the end are dropped below): the warp's 32 x 16
                // block goes through shared memory so that four lanes write one row's 64 bytes
                if (corr != nullptr && rowValid) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        acc[j] += uint32_t(__ldg(corr + col0 + j));
                    }
                }
                int32_t *mine = staging + warp * (32 * kStageInts);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    *reinterpret_cast<int4 *>(mine + lane * kStageInts + 4 * q) =
                        make_int4(int(acc[4 * q]), int(acc[4 * q + 1]), int(acc[4 * q + 2]), int(acc[4 * q + 3]));
                }
                __syncwarp();
                const int64_t firstRow = int64_t(m0) + quarter * 32;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = 8 * j + (lane >> 2), piece = lane & 3;
                    if (firstRow + r < p.M) {
                        const int4 v = *reinterpret_cast<const int4 *>(mine + r * kStageInts + 4 * piece);
                        *reinterpret_cast<int4 *>(p.out32 + (int64_t(batch) * p.M + firstRow + r) * p.ldOut + col0 + 4 * piece) = v;
                    }
                }
                __syncwarp();
                continue;
            }
            if (!rowValid || col0 >= p.N) {
                continue;
            }
            const int ncols = min(16, p.N - col0);
            int32_t *dst = p.out32 + outRow + col0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (corr != nullptr && j < ncols) {
                    acc[j] += uint32_t(__ldg(corr + col0 + j));
                }
            }
            if (ncols == 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    reinterpret_cast<int4 *>(dst)[q] =
                        make_int4(int(acc[4 * q]), int(acc[4 * q + 1]), int(acc[4 * q + 2]), int(acc[4 * q + 3]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j < ncols) {
                        dst[j] = int32_t(acc[j]);
                    }
                }
            }
        }
    }
}

template <int BN, int NSTAGE>
__device__ __forceinline__ void epilogueWarps(const GemmI8Params &p, PipeBarriers *bars, ColConst *colTab,
                                              uint32_t tmemBase, int warp, int lane, int64_t numTiles, int mTiles,
                                              int nTiles, int32_t *staging) {
    if (p.out32 != nullptr) {
        // the staged stores need 16-byte aligned rows
        const bool staged = staging != nullptr && p.ldOut % 4 == 0 && (reinterpret_cast<uintptr_t>(p.out32) & 15u) == 0;
        epilogueInt32<BN, NSTAGE>(p, bars, tmemBase, warp, lane, numTiles, mTiles, nTiles, staged ? staging : nullptr);
    } else if (p.epi.hasResidual) {
        epilogueInt8<BN, NSTAGE, true>(p, bars, colTab, tmemBase, warp, lane, numTiles, mTiles, nTiles);
    } else {
        epilogueInt8<BN, NSTAGE, false>(p, bars, colTab, tmemBase, warp, lane, numTiles, mTiles, nTiles);
    }
}

// Table gather of one 128-byte K block of one tile row: BK / G pieces of G bytes, piece j from origin + tab[j],
// written to its place in the SWIZZLE_128B row at dstRow (swz = row & 7).
// Only the first `bytes` bytes of the row are gathered (in groups of four pieces): the MMAs of a K block's zero-filled
// tail are not issued (ummaCountFor), so nothing reads the rest of the row.
template <int G>
__device__ __forceinline__ void gatherPieces(const int8_t *origin, const int32_t *tab, uint32_t dstRow, uint32_t swz,
                                             int bytes) {
#pragma unroll
    for (int j4 = 0; j4 < BK / G; j4 += 4) {
        if (j4 * G >= bytes) {
            break;
        }
        const int4 off = *reinterpret_cast<const int4 *>(tab + j4);
        const int offs[4] = {off.x, off.y, off.z, off.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int o = (j4 + e) * G; // byte position inside the K block
            const uint32_t dst = dstRow + ((uint32_t(o >> 4) ^ swz) << 4) + uint32_t(o & 15);
            const int8_t *src = origin + offs[e];
            if (G == 4) {
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
            } else if (G == 8) {
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
            } else {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            }
        }
    }
}

// A_MODE: how the A (pixel) operand arrives: kAGather = gathered from the NHWC input described by p, kATiled =
// tmapA is a plain matrix, kAIm2col = tmapA is an im2col map of the NHWC input and tmapB a {IC, taps, OC} map.
// B_MN : B is an N-contiguous [K][N] matrix (MN-major operand), otherwise a K-contiguous [N][K] matrix.
// STAGE32: shared memory for the staged int32 stores of epilogueInt32 is set aside (see there).
template <int BN, int NSTAGE, int A_MODE, bool B_MN, bool STAGE32 = false>
__global__ void __launch_bounds__(A_MODE != kAGather ? kThreadsTma : kThreadsGather, 1)
gemmI8Tcgen05(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, const GemmI8Params p) {
    constexpr bool A_TMA = A_MODE != kAGather;
    extern __shared__ uint8_t rawSmem[];
    // SWIZZLE_128B tiles must start on 1024-byte boundaries.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    constexpr int kTileA = BM * BK;
    constexpr int kTileB = BN * BK;
    uint8_t *tilesA = smem;
    uint8_t *tilesB = smem + NSTAGE * kTileA;
    ColConst *colTab = reinterpret_cast<ColConst *>(smem + NSTAGE * (kTileA + kTileB));
    PipeBarriers *bars = reinterpret_cast<PipeBarriers *>(smem + NSTAGE * (kTileA + kTileB) + BN * sizeof(ColConst));
    // gather variants only: the table of piece offsets (at most kMaxGatherPieces entries), 16-byte aligned
    int32_t *gatherTab = reinterpret_cast<int32_t *>(
        (reinterpret_cast<uintptr_t>(bars) + sizeof(PipeBarriers) + 15) & ~uintptr_t(15));
    int32_t *tapTab = gatherTab + kMaxGatherPieces; // tap offsets of the segment gather
    // STAGE32 (TMA variants only: no gather tables): the epilogue warps' staging blocks follow the barriers
    int32_t *staging = STAGE32 ? gatherTab : nullptr;
    const bool fastGather = !A_TMA && fastGatherApplies(p);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int numKb = A_MODE == kAIm2col ? p.KH * p.KW * p.kbPerTap : (p.K + BK - 1) / BK;
    const int mTiles = (p.M + BM - 1) / BM;
    const int nTiles = (p.N + BN - 1) / BN;
    const int64_t numTiles = int64_t(mTiles) * nTiles * p.batches;
    const auto tileOf = [&](int64_t tile) {
        // the launcher refuses 2^31 tiles and more: divisions by multiply-high (see FastDiv)
        const uint32_t overN = fastDiv(uint32_t(tile), p.divTiles0), overM = fastDiv(overN, p.divTiles1);
        TileCoord c;
        c.n0 = int(uint32_t(tile) - overN * uint32_t(nTiles)) * BN;
        c.m0 = int(overN - overM * uint32_t(mTiles)) * BM;
        c.batch = int(overM);
        return c;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbarInit(&bars->full[s], A_TMA ? 1u : 1u + 128u);
            mbarInit(&bars->empty[s], 1u);
        }
        for (int b = 0; b < 2; ++b) {
            mbarInit(&bars->accFull[b], 1u);
            mbarInit(&bars->accEmpty[b], uint32_t(kEpilogueWarps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (fastGather && warp >= kGatherWarp0) {
        fillTapTable(p, tapTab, kGatherWarp0 * 32, 128);
    }
    if (!A_TMA && p.gatherTable != nullptr && warp >= kGatherWarp0) {
        const int pieces = ((p.K + BK - 1) / BK) * (BK / p.chunkBytes);
        for (int i = int(threadIdx.x) - kGatherWarp0 * 32; i < pieces && i < kMaxGatherPieces; i += 128) {
            gatherTab[i] = __ldg(p.gatherTable + i);
        }
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&bars->tmemBase)),
                     "r"(uint32_t(2 * BN))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmemBase = bars->tmemBase;
    gridDependencySync(); // from here on activations are read and written

    if (warp == kTmaWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t ready = 0; // 1: the stage of the coming K block is known to be empty (see tmaStagePeekTiled)
            int s = 0;          // the ring runs on across tiles
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                const TileCoord tc = tileOf(t);
                // im2col mode: first tap of the tile's first window, and the running position on the K axis
                int w0 = 0, h0 = 0, n0 = 0, kx = 0, ky = 0, cb = 0;
                if (A_MODE == kAIm2col) {
                    n0 = int(fastDiv(uint32_t(tc.m0), p.divPlane));
                    const int rem = tc.m0 - n0 * p.OH * p.OW;
                    const int oy = int(fastDiv(uint32_t(rem), p.divOW));
                    h0 = oy * p.strideY - p.padTop;
                    w0 = (rem - oy * p.OW) * p.strideX - p.padLeft;
                }
                for (int kb = 0; kb < numKb; ++kb) {
                    if (ready == 0) {
                        ok = mbarWait(&bars->empty[s], phase ^ 1u, 1);
                        if (!ok) {
                            break;
                        }
                    }
                    const int sNext = s + 1 == NSTAGE ? 0 : s + 1;
                    const uint32_t phaseNext = sNext == 0 ? phase ^ 1u : phase;
                    uint8_t *dstA = tilesA + s * kTileA, *dstB = tilesB + s * kTileB;
                    if (A_MODE == kAIm2col) {
                        ready = tmaStagePeekIm2col(&bars->full[s], uint32_t(kTileA + kTileB), &tmapB, dstB, cb, ky * p.KW + kx,
                                                   tc.n0, &tmapA, dstA, cb, w0, h0, n0, uint16_t(kx * p.dilX),
                                                   uint16_t(ky * p.dilY), &bars->empty[sNext], phaseNext ^ 1u);
                        cb += BK;
                        if (cb >= p.IC) {
                            cb = 0;
                            if (++kx == p.KW) {
                                kx = 0;
                                ++ky;
                            }
                        }
                    } else if (A_MODE == kATiled) {
                        if (B_MN) {
                            ready = tmaStagePeekTiled(&bars->full[s], uint32_t(kTileA + kTileB), &tmapB, dstB, tc.n0, kb * BK,
                                                      tc.batch, &tmapA, dstA, kb * BK, tc.m0, tc.batch, &bars->empty[sNext],
                                                      phaseNext ^ 1u);
                        } else {
                            ready = tmaStagePeekTiled(&bars->full[s], uint32_t(kTileA + kTileB), &tmapB, dstB, kb * BK, tc.n0,
                                                      p.batchedB ? tc.batch : 0, &tmapA, dstA, kb * BK, tc.m0, tc.batch,
                                                      &bars->empty[sNext], phaseNext ^ 1u);
                        }
                    } else {
                        // gathered pixel operand: only the weight tile comes by TMA
                        mbarArriveExpectTx(&bars->full[s], uint32_t(kTileB));
                        if (B_MN) {
                            tmaLoad3d(&tmapB, dstB, &bars->full[s], tc.n0, kb * BK, tc.batch);
                        } else {
                            tmaLoad3d(&tmapB, dstB, &bars->full[s], kb * BK, tc.n0, p.batchedB ? tc.batch : 0);
                        }
                    }
                    s = sNext;
                    phase = phaseNext;
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = instrDesc(BN, B_MN);
            static_assert(BK / UMMA_K == 4, "ummaBlockPeek issues the four MMAs of a K block");
            // K-major: step 32 bytes inside the 128-byte swizzle row; MN-major: step 32 K-rows of 128 bytes
            const uint64_t descA0 = smemDesc(smemAddr(tilesA), 16, 1024);
            const uint64_t descB0 = B_MN ? smemDesc(smemAddr(tilesB), BK * 128, 1024) : smemDesc(smemAddr(tilesB), 16, 1024);
            constexpr uint64_t kStepB = B_MN ? uint64_t(UMMA_K * 128) >> 4 : 2;
            uint32_t tileCount = 0;
            uint32_t ready = 0; // 1: the stage of the coming K block is known to be full (see ummaBlockPeek)
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileCount) {
                const uint32_t buf = tileCount & 1u;
                // wait until the epilogue has drained this accumulator (passes at once for the first two tiles)
                ok = mbarWait(&bars->accEmpty[buf], ((tileCount >> 1) & 1u) ^ 1u, 5);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmemD = tmemBase + buf * uint32_t(BN);
                int kLeft = A_MODE == kAIm2col ? p.IC : p.K; // bytes of K in the coming block's tap or K axis
                for (int kb = 0; kb < numKb; ++kb) {
                    if (ready == 0) {
                        ok = mbarWait(&bars->full[s], phase, 2);
                        if (!ok) {
                            break;
                        }
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // the ring runs on across tiles: the next K block's stage follows this one whatever tile it is in
                    const int sNext = s + 1 == NSTAGE ? 0 : s + 1;
                    const uint32_t phaseNext = sNext == 0 ? phase ^ 1u : phase;
                    ready = ummaBlockPeek(tmemD, descA0 + uint64_t(uint32_t(s) * uint32_t(kTileA >> 4)), 2,
                                          descB0 + uint64_t(uint32_t(s) * uint32_t(kTileB >> 4)), kStepB, idesc,
                                          kb != 0 ? 1u : 0u, ummaCountFor(kLeft), &bars->empty[s], &bars->full[sNext], phaseNext);
                    kLeft -= BK;
                    if (kLeft <= 0) {
                        kLeft = A_MODE == kAIm2col ? p.IC : 0;
                    }
                    s = sNext;
                    phase = phaseNext;
                }
                if (ok) {
                    ummaCommit(&bars->accFull[buf]);
                }
            }
        }
    } else if (warp >= kGatherWarp0) {
        // ---------------- A gather (implicit GEMM): one tile row per thread ----------------
        if (!A_TMA) {
            const int row = (warp - kGatherWarp0) * 32 + lane;
            const uint32_t swz = uint32_t(row & 7);
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                const TileCoord tc = tileOf(t);
                const int64_t m = int64_t(tc.m0) + row;
                if (fastGather) {
                    const GatherRow rows[1] = {gatherRowSetup(p, m)};
                    int tap = 0, c0 = 0;
                    for (int kb = 0; kb < numKb; ++kb, ++it) {
                        const int s = int(it % NSTAGE);
                        const uint32_t phase = (it / NSTAGE) & 1u;
                        ok = mbarWait(&bars->empty[s], phase ^ 1u, 3);
                        if (!ok) {
                            break;
                        }
                        const uint32_t dstRow = smemAddr(tilesA + s * kTileA) + uint32_t(row) * 128u;
                        gatherBlock<1>(rows, tapTab, p.KH * p.KW, p.IC, tap, c0, dstRow, swz, p.in);
                        asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(smemAddr(&bars->full[s]))
                                     : "memory");
                        mbarArrive(&bars->full[s]);
                    }
                    continue;
                }
                const bool rowValid = m < p.M;
                int n = 0, oy = 0, ox = 0;
                if (rowValid) {
                    n = int(fastDiv(uint32_t(m), p.divPlane));
                    const uint32_t rem = uint32_t(m) - uint32_t(n) * p.divPlane.d;
                    oy = int(fastDiv(rem, p.divOW));
                    ox = int(rem) - oy * p.OW;
                }
                const int iy0 = oy * p.strideY - p.padTop;
                const int ix0 = ox * p.strideX - p.padLeft;
                const int8_t *base = p.in + int64_t(n) * p.H * p.W * p.IC;
                int c = 0, kx = 0, ky = 0; // position of the next 16-byte chunk inside K = (ky, kx, c)
                for (int kb = 0; kb < numKb; ++kb, ++it) {
                    const int s = int(it % NSTAGE);
                    const uint32_t phase = (it / NSTAGE) & 1u;
                    ok = mbarWait(&bars->empty[s], phase ^ 1u, 3);
                    if (!ok) {
                        break;
                    }
                    const uint32_t dstRow = smemAddr(tilesA + s * kTileA) + uint32_t(row) * 128u;
                    if (p.gatherTable != nullptr) {
                        // every tap is in range (zero-padded copy): pieces at tabulated offsets from the origin
                        const int8_t *origin =
                            rowValid ? base + (int64_t(oy * p.strideY) * p.W + ox * p.strideX) * p.IC : p.in;
                        // bytes of K this block holds, rounded up to the MMAs that will read them
                        const int blockBytes = ummaCountFor(p.K - kb * BK) * UMMA_K;
                        if (p.chunkBytes == 4) {
                            gatherPieces<4>(origin, gatherTab + kb * (BK / 4), dstRow, swz, blockBytes);
                        } else if (p.chunkBytes == 8) {
                            gatherPieces<8>(origin, gatherTab + kb * (BK / 8), dstRow, swz, blockBytes);
                        } else {
                            gatherPieces<16>(origin, gatherTab + kb * (BK / 16), dstRow, swz, blockBytes);
                        }
                        asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(smemAddr(&bars->full[s]))
                                     : "memory");
                        mbarArrive(&bars->full[s]);
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int y = iy0 + ky * p.dilY;
                        const int x = ix0 + kx * p.dilX;
                        const bool valid = rowValid && ky < p.KH && y >= 0 && y < p.H && x >= 0 && x < p.W;
                        const int8_t *src = valid ? base + (int64_t(y) * p.W + x) * p.IC + c : p.in;
                        const uint32_t dst = dstRow + ((uint32_t(j) ^ swz) << 4);
                        const uint32_t bytes = valid ? 16u : 0u; // 0 source bytes => the 16 bytes are zero-filled
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                                     : "memory");
                        c += 16;
                        if (c >= p.IC) {
                            c = 0;
                            if (++kx == p.KW) {
                                kx = 0;
                                ++ky;
                            }
                        }
                    }
                    // The stage's barrier completes when these copies have landed and every producer arrived.
                    asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(smemAddr(&bars->full[s]))
                                 : "memory");
                    mbarArrive(&bars->full[s]);
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 0-15 ----------------
        epilogueWarps<BN, NSTAGE>(p, bars, colTab, tmemBase, warp, lane, numTiles, mTiles, nTiles, staging);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(uint32_t(2 * BN))
                     : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------------------

template <int BN, int NSTAGE, int A_MODE, bool B_MN, bool STAGE32 = false>
int launchVariant(const CUtensorMap &mapA, const CUtensorMap &mapB, const GemmI8Params &params, cudaStream_t s) {
    static_assert(!STAGE32 || A_MODE != kAGather, "the staging blocks take the place of the gather tables");
    GemmI8Params p = params;
    p.divPlane = makeFastDiv(int64_t(p.OH) * p.OW), p.divOW = makeFastDiv(p.OW);
    p.divTiles0 = makeFastDiv((p.N + BN - 1) / BN), p.divTiles1 = makeFastDiv((p.M + BM - 1) / BM);
    constexpr size_t smemBytes =
        size_t(NSTAGE) * (BM * BK + BN * BK) + BN * sizeof(ColConst) + sizeof(PipeBarriers) + 1024 +
        (A_MODE != kAGather ? 0 : (kMaxGatherPieces + kTapTabEntries) * sizeof(int32_t) + 16) +
        (STAGE32 ? size_t(kEpilogueWarps) * kStageBytesPerWarp + 16 : 0);
    static_assert(smemBytes <= 232448, "shared memory per CTA");
    auto kernel = gemmI8Tcgen05<BN, NSTAGE, A_MODE, B_MN, STAGE32>;
    if (!allowDynamicSmem(reinterpret_cast<const void *>(kernel), smemBytes)) {
        return MLEL_ERROR_DEVICE;
    }
    const int64_t tiles = int64_t((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batches;
    if (tiles >= (int64_t(1) << 31)) {
        setLastError("tcgen05 int8 GEMM: too many tiles");
        return MLEL_ERROR_UNKNOWN;
    }
    const int grid = int(tiles < smCount() ? tiles : smCount()); // persistent: one CTA per SM
    const cudaError_t err = launchDependent(kernel, grid, A_MODE != kAGather ? kThreadsTma : kThreadsGather, smemBytes, s, mapA, mapB, p);
    if (err != cudaSuccess) {
        setLastError(std::string("tcgen05 int8 GEMM launch: ") + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

} // namespace

std::atomic<long long> g_tensorCoreLaunches[3];

TensorCoreTuning &tensorCoreTuning() {
    static TensorCoreTuning t;
    return t;
}

int gemmI8Launch(const GemmI8Problem &q, cudaStream_t s) {
    g_tensorCoreLaunches[0].fetch_add(1, std::memory_order_relaxed);
    GemmI8Params p = q.params;
    p.batches = q.batches;
    CUtensorMap mapA{}, mapB{};
    // 64-column tiles for narrow outputs, and where 128-column tiles would occupy less than half of the SMs (a
    // classifier's product of a few rows with a wide weight matrix: twice the CTAs each stream half the weights)
    const int64_t wideTiles = int64_t((p.M + BM - 1) / BM) * ((p.N + 127) / 128) * q.batches;
    const int bn = (!q.bMnMajor && (p.N <= 64 || 2 * wideTiles <= smCount())) ? 64 : 128;
    int aMode = kAGather;
    if (q.aMatrix != nullptr) {
        // A: [batches][M][K], K contiguous
        if (!makeMap(&mapA, q.aMatrix, uint64_t(p.K), uint64_t(p.M), uint64_t(q.batches), uint64_t(q.aRowBytes),
                     uint64_t(q.aBatchBytes), BK, BM)) {
            return MLEL_ERROR_DEVICE;
        }
        aMode = kATiled;
    } else if (p.gatherTable == nullptr && !q.bMnMajor && !p.batchedB && q.batches == 1 && p.IC % 16 == 0 && p.KH > 0 &&
               ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(q.bMatrix)) & 15u) == 0 &&
               makeIm2colMap(&mapA, p.in, p.M / (p.OH * p.OW), p.H, p.W, p.IC, p.KH, p.KW, p.padTop, p.padLeft, p.OH, p.OW,
                             p.strideY, p.strideX, p.dilY, p.dilX, BM) &&
               makeWeightTapMap(&mapB, q.bMatrix, p.IC, p.KH * p.KW, p.N, uint32_t(bn))) {
        // a window over a multiple of 16 channels: hardware im2col loads, zero-filled past the last channel
        aMode = kAIm2col;
        p.kbPerTap = (p.IC + 127) / 128;
    }
    if (aMode == kAIm2col) {
        // tmapB is the {IC, taps, OC} weight map made above
    } else if (q.bMnMajor) {
        // B: [batches][K][N], N contiguous
        if (!makeMap(&mapB, q.bMatrix, uint64_t(p.N), uint64_t(p.K), uint64_t(q.batches), uint64_t(q.bRowBytes),
                     uint64_t(q.bBatchBytes), 128, BK)) {
            return MLEL_ERROR_DEVICE;
        }
    } else {
        // B: [batchesB][N][K], K contiguous
        if (!makeMap(&mapB, q.bMatrix, uint64_t(p.K), uint64_t(p.N), uint64_t(p.batchedB ? q.batches : 1),
                     uint64_t(q.bRowBytes), uint64_t(q.bBatchBytes ? q.bBatchBytes : q.bRowBytes * uint64_t(p.N)),
                     BK, uint32_t(bn))) {
            return MLEL_ERROR_DEVICE;
        }
    }
    if (q.bMnMajor) {
        return aMode == kATiled ? launchVariant<128, 6, kATiled, true>(mapA, mapB, p, s)
                                : launchVariant<128, 6, kAGather, true>(mapA, mapB, p, s);
    }
    if (bn == 64) {
        return aMode == kATiled    ? launchVariant<64, 8, kATiled, false>(mapA, mapB, p, s)
               : aMode == kAIm2col ? launchVariant<64, 8, kAIm2col, false>(mapA, mapB, p, s)
                                   : launchVariant<64, 8, kAGather, false>(mapA, mapB, p, s);
    }
    if (aMode == kATiled && p.out32 != nullptr) {
        // a matrix product with an int32 result (attention scores): one stage fewer, staged stores
        return launchVariant<128, 5, kATiled, false, true>(mapA, mapB, p, s);
    }
    return aMode == kATiled    ? launchVariant<128, 6, kATiled, false>(mapA, mapB, p, s)
           : aMode == kAIm2col ? launchVariant<128, 6, kAIm2col, false>(mapA, mapB, p, s)
                               : launchVariant<128, 6, kAGather, false>(mapA, mapB, p, s);
}

namespace {
// Self-test of the give-up path of the bounded waits: one thread waits on an mbarrier that nobody arrives at, with
// a limit of about a millisecond instead of the kernels' two seconds, records the code and returns.
__global__ void waitTimeoutSelfTestKernel(int code, long long limitCycles, int *gaveUp) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        tc::mbarInit(&bar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *gaveUp = tc::mbarWaitLimit(&bar, 0u, code, limitCycles) ? 0 : 1;
    }
}
} // namespace

int waitTimeoutSelfTest(cudaStream_t s, int *codeOut) {
    constexpr int kCode = 99;
    int *flag = nullptr;
    if (cudaMalloc(&flag, sizeof(int)) != cudaSuccess) {
        setLastError("wait self-test: cudaMalloc failed");
        return MLEL_ERROR_DEVICE;
    }
    cudaMemsetAsync(flag, 0xff, sizeof(int), s);
    waitTimeoutSelfTestKernel<<<1, 32, 0, s>>>(kCode, 2000000ll, flag); // about 1 ms of SM clock
    int gaveUp = -1;
    const bool ok = cudaMemcpyAsync(&gaveUp, flag, sizeof(int), cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                    cudaStreamSynchronize(s) == cudaSuccess;
    cudaFree(flag);
    if (!ok) {
        setLastError("wait self-test: kernel or copy failed");
        return MLEL_ERROR_DEVICE;
    }
    const int recorded = tc::readErrorWord();
    if (recorded == kCode) {
        tc::clearErrorWord(); // only the self-test's own code is cleared: a real time-out stays recorded
    }
    *codeOut = gaveUp == 1 ? recorded : 0;
    return MLEL_SUCCESS;
}

int tcgen05ErrorFlag() {
    const int v = tc::readErrorWord();
    if (v != 0) {
        return v;
    }
    const int w = ocMajorErrorWord();
    return w != 0 ? w : pairErrorWord();
}

} // namespace mlel
