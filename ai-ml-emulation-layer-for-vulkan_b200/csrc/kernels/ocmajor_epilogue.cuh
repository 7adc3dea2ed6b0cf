// Epilogue of the channel-major tcgen05 int8 kernels (gemm_i8_ocmajor.cu: one CTA per tile; gemm_i8_pair.cu: a
// pair of CTAs per tile): accumulator lanes are output channels, so a thread keeps its channel's RESCALE
// constants and zero-point correction in registers; results go through a [pixels][128 channels] byte tile in
// shared memory to a TMA store.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_i8_tcgen05.hpp"
#include "tcgen05_common.cuh"

namespace mlel {
namespace {

using namespace tc;

constexpr int kOcTile = 128; // output channels per tile (UMMA M)

// Warp roles of this kernel, EW = number of epilogue warps (8 or 12): 0..EW-1 epilogue (EW / 4 per TMEM lane
// quarter, each with its own share of the tile's pixels), EW TMA producer, EW + 1 MMA issuer and TMEM owner,
// EW + 2 and EW + 3 pixel gather (implicit-GEMM variants only).  The register file bounds the count: the
// epilogue needs about 128 registers per thread, which a CTA of up to 512 threads (EW = 12 with both gather
// warps) still gets; with 16 epilogue warps it spilled.
constexpr int kOcGatherThreads = 64;
// The residual table: 256 rows (main-stage value) of 256 bytes (shortcut byte), rows 260 bytes apart.  With rows
// of 256 bytes the shared-memory bank of an entry would depend on the shortcut byte alone, and the lanes of a
// warp -- whose shortcut values are often equal (activations clamped by a ReLU) while their main-stage values
// differ -- would all hit one bank; the extra word per row spreads them over the banks.
constexpr int kResidualRowBytes = GemmI8Params::kResidualRowBytes;
constexpr int kResidualTableBytes = 256 * kResidualRowBytes;
static_assert(kResidualTableBytes % 16 == 0, "bulk copies move multiples of 16 bytes");
constexpr int ocThreads(int ew, bool gather) { return (ew + 2) * 32 + (gather ? kOcGatherThreads : 0); }

// Barrier among the epilogue warps only (named barrier 1).
template <int EW> __device__ __forceinline__ void ocEpilogueSync() {
    asm volatile("bar.sync 1, %0;" ::"r"(EW * 32) : "memory");
}

constexpr int kXGather = 0, kXTiled = 1, kXIm2col = 2;

struct __align__(8) OcBarriers {
    uint64_t full[6];
    uint64_t empty[6];
    uint64_t accFull[2];
    uint64_t accEmpty[2];
    uint64_t cFull[2];  // the shortcut bytes of a tile have landed in its C/D tile
    uint64_t cdEmpty[2]; // the store of a C/D tile has finished reading it: the tile may be loaded again
    uint64_t cdFull[2];  // kernels with a store warp: the epilogue warps have filled the C/D tile
    uint64_t tabFull;    // the residual table has landed in shared memory
    uint32_t tmemBase;
    uint32_t pad;
};

struct OcTile {
    int c0, m0, batch;
};

// Tile index -> (pixel tile, channel tile, batch).  Pixel tile fastest by default: a CTA's consecutive tiles then
// mostly share their channels, so the per-channel constants are reloaded rarely.  Channel tile fastest when the
// launch publishes its progress per pixel tile (GemmI8Params::progressOut): the channel tiles of a pixel tile then
// run side by side and low pixel tiles are complete long before the launch ends.  The launcher sets divTiles0 /
// divTiles1 to the extents in the chosen order and refuses 2^31 tiles and more (divisions by multiply-high).
struct TileIndex {
    uint32_t pix, chan, batch;
};
__device__ __forceinline__ TileIndex decodeTile(const GemmI8Params &p, int64_t tile, int pTiles, int cTiles) {
    const uint32_t over0 = fastDiv(uint32_t(tile), p.divTiles0), over1 = fastDiv(over0, p.divTiles1);
    TileIndex i;
    if (p.channelFastest != 0) {
        i.chan = uint32_t(tile) - over0 * uint32_t(cTiles);
        i.pix = over0 - over1 * uint32_t(pTiles);
    } else {
        i.pix = uint32_t(tile) - over0 * uint32_t(pTiles);
        i.chan = over0 - over1 * uint32_t(cTiles);
    }
    i.batch = over1;
    return i;
}

// One more channel tile of pixel tile `pix` has reached memory.  Called by the thread that issued the tile's TMA store,
// after cp.async.bulk.wait_group 0 (the writes are complete and visible to this thread); the release makes them visible
// to whoever acquires the counter.
__device__ __forceinline__ void publishTile(uint32_t *counters, uint32_t pix) {
    asm volatile("fence.proxy.async.global;" ::: "memory");
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(counters + pix), "r"(1u) : "memory");
}

// Waits until every counter of [first, last] has reached `target` (bounded like mbarWait: gives up with `code` in the
// error word), then orders the TMA loads that follow after what was acquired.
__device__ __forceinline__ bool waitTiles(const uint32_t *counters, uint32_t first, uint32_t last, uint32_t target, int code) {
    for (uint32_t j = first; j <= last; ++j) {
        const long long start = clock64();
        unsigned polls = 0;
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counters + j) : "memory");
            if (v >= target) {
                break;
            }
            __nanosleep(100);
            if ((++polls & 63u) == 0 && clock64() - start > kWaitLimitCycles) {
                atomicCAS(&g_tcgen05Error, 0, code);
                return false;
            }
        }
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");
    return true;
}

// Plain (untiled) bulk copy global -> shared, completing on an mbarrier; both addresses and the size are
// multiples of 16 bytes.
__device__ __forceinline__ void bulkLoad(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smemAddr(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smemAddr(bar))
                 : "memory");
}

__device__ __forceinline__ void tmaStore3d(const CUtensorMap *map, const void *src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(smemAddr(src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// Shared-memory accesses by 32-bit shared address (a pointer into dynamic shared memory that has been passed
// through a few functions is otherwise accessed with generic 64-bit loads and stores).
__device__ __forceinline__ uint32_t ldsU8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void stsU8(uint32_t addr, int32_t v) {
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// The rest of such a RESCALE: remaining shift, output zero point (wrapping add), clamp.
__device__ __forceinline__ int32_t finishHigh(int32_t high, int32_t s2, int32_t outZp, int32_t lo, int32_t hi) {
    return min(__viaddmax_s32(high >> s2, outZp, lo), hi);
}

// Constants of one epilogue thread (one output channel) and of the per-tensor output stage.
struct EpiConsts {
    FastRescale fm;
    uint64_t rnM;    // scaleHigh: rounding constant without the zero-point fold, for x < 0
    uint32_t bumpM;  // scaleHigh: 2^31 with double rounding, else 0
    int32_t corr0;   // correction of the most common border class
    int32_t corrX;   // corr0 - input zero point: accumulator + corrX is x of scaleHigh
    int32_t outZpMain, loMain, hiMain;
    bool fast; // the shift is at least 32 and the corrections are small: see scaleHigh
    // 0: the 64-bit forms above; 1: scaleHigh32 with the sign of x; 2: scaleHigh32 without it
    int words32;
    int32_t corrX4, c32, shift32; // scaleHigh32: 4 * corrX, rounding units, shift - 30
};

// 16 pixels of one channel: accumulator slice -> bytes in the C/D tile (column `cd`, rows 128 bytes apart).
// All shortcut bytes are read before the first result is written: the compiler must assume that a byte store
// may alias any later load, and 16 load-compute-store chains in a row would run one after the other.
template <bool RESIDUAL, bool FAST, int WORDS32 = 0>
__device__ __forceinline__ void rescaleSliceImpl(const uint32_t (&acc)[16], const EpiConsts &k, uint32_t tab128,
                                                 uint32_t cd) {
    constexpr int CH = 8; // pixels per group: enough independent chains, few enough live registers
#pragma unroll
    for (int g = 0; g < 16; g += CH) {
        uint32_t sc[CH];
        if (RESIDUAL) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                sc[j] = ldsU8(cd + 128 * (g + j));
            }
        }
        int32_t r[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            if (WORDS32 != 0) {
                const int32_t x4 = int32_t(acc[g + j] * 4u + uint32_t(k.corrX4));
                const int32_t q = scaleHigh32<WORDS32 == 1>(x4, k.fm.mult, k.c32) >> k.shift32;
                if (RESIDUAL) {
                    r[j] = __viaddmin_s32_relu(q, k.outZpMain - k.loMain, k.hiMain - k.loMain);
                } else {
                    r[j] = min(__viaddmax_s32(q, k.outZpMain, k.loMain), k.hiMain);
                }
            } else if (FAST) {
                const int32_t x = int32_t(acc[g + j] + uint32_t(k.corrX));
                const int32_t high = scaleHigh(x, k.fm.mult, k.rnM, k.bumpM);
                if (RESIDUAL) {
                    // the value is only used as a row number of the residual table: clamp(q + zp, lo, hi) - lo is one
                    // add-min-relu, and the table's base address takes the - lo
                    r[j] = __viaddmin_s32_relu(high >> k.fm.s2, k.outZpMain - k.loMain, k.hiMain - k.loMain);
                } else {
                    r[j] = finishHigh(high, k.fm.s2, k.outZpMain, k.loMain, k.hiMain);
                }
            } else {
                const int32_t v = int32_t(acc[g + j] + uint32_t(k.corr0));
                r[j] = fastRescale(k.fm, v, k.outZpMain, k.loMain, k.hiMain) - (RESIDUAL ? k.loMain : 0);
            }
        }
        if (RESIDUAL) {
            // the whole tail -- both input RESCALEs, the ADD, the output RESCALE and its clamp -- is one byte
            // of the table, addressed by the main stage's value and the shortcut byte
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                r[j] = int32_t(ldsU8(tab128 + sc[j] + uint32_t(r[j] * kResidualRowBytes)));
            }
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            stsU8(cd + 128 * (g + j), r[j]);
        }
    }
}

// cd: shared address of this thread's column of the C/D tile at the slice's first pixel; tab128: shared address
// of the residual table's row for the lowest main-stage value.
template <bool RESIDUAL>
__device__ __forceinline__ void rescaleSlice(const uint32_t (&acc)[16], const EpiConsts &k, uint32_t tab128, uint32_t cd) {
    if (k.words32 == 2) {
        rescaleSliceImpl<RESIDUAL, true, 2>(acc, k, tab128, cd);
    } else if (k.words32 == 1) {
        rescaleSliceImpl<RESIDUAL, true, 1>(acc, k, tab128, cd);
    } else if (k.fast) {
        rescaleSliceImpl<RESIDUAL, true>(acc, k, tab128, cd);
    } else {
        rescaleSliceImpl<RESIDUAL, false>(acc, k, tab128, cd);
    }
}


// Which tiles the epilogue warps of one CTA walk, and where they hand a drained accumulator back.  A CTA that
// works alone walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... and arrives on its own barriers; the two CTAs
// of a pair walk the pair's tiles, the second one 128 channels further on, and both arrive on the barriers of
// the CTA that issues the MMAs (shared::cluster addresses).
struct EpiWalk {
    int64_t first, stride;
    int cOffset;
    uint32_t accEmpty[2];
};

// Arrival on an mbarrier of any CTA of the cluster, by its shared::cluster address.
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}

// The epilogue warps.  Warp w owns TMEM lanes 32 * (w & 3) .. +31 (output channels) and half of the tile's
// pixels, which it walks in slices of 16 pixels; the tcgen05.ld of the next slice is in flight while the
// current one is rescaled.  C_TILE: output channels per tile (128, or 256 for a pair of CTAs).
template <int BNP, int EW, bool RESIDUAL, int C_TILE, bool STORE_WARP = false>
__device__ __forceinline__ void epilogueOcMajor(const CUtensorMap *tmapD, const GemmI8Params &p, OcBarriers *bars,
                                                const uint8_t *resTab, uint8_t *cdTiles,
                                                uint32_t tmemBase, int warp, int lane, int64_t numTiles, int pTiles,
                                                int cTiles, const EpiWalk &walk) {
    constexpr bool PAIR = C_TILE != kOcTile;
    const auto accDrained = [&](uint32_t buf) {
        if (PAIR) {
            mbarArriveCluster(walk.accEmpty[buf]);
        } else {
            mbarArrive(&bars->accEmpty[buf]);
        }
    };
    const int quarter = warp & 3;
    const int part = warp >> 2;
    constexpr int kColsPerWarp = BNP / (EW / 4);
    constexpr int kSteps = kColsPerWarp / 16;
    static_assert(EW % 4 == 0 && kColsPerWarp * (EW / 4) == BNP && kColsPerWarp % 16 == 0, "pixel shares of the warps");
    static_assert(kSteps % 2 == 0, "slices are processed in pairs");
    static_assert(kColsPerWarp % 32 == 0, "a lane holds the classes of whole pixels of its warp's share");
    EpiConsts k{};
    k.outZpMain = p.epi.main.outZp, k.loMain = p.epi.main.lo, k.hiMain = p.epi.main.hi;
    // row of the lowest main-stage value: the element loop counts rows from there
    const uint32_t tab128 = smemAddr(resTab) + uint32_t((128 + p.epi.main.lo) * kResidualRowBytes);
    bool tableReady = !RESIDUAL;
    int curC0 = -1, curBatch = -1;
    const bool hasClasses = p.rowClass != nullptr;
    const int baseClass = p.baseClass;
    // issues the tile stores and tracks their completion (kernels with a store warp: that warp does, see storeWarpOcMajor)
    const bool storer = !STORE_WARP && warp == 0 && lane == 0;
    constexpr uint32_t kNoTile = 0xffffffffu;
    uint32_t storedPix = kNoTile; // pixel tile of the store in flight (published once it has reached memory)
    uint32_t tileCount = 0;
    for (int64_t t = walk.first; t < numTiles; t += walk.stride, ++tileCount) {
        const TileIndex ti = decodeTile(p, t, pTiles, cTiles);
        const int m0 = int(ti.pix) * BNP;
        const int c0 = int(ti.chan) * C_TILE + walk.cOffset;
        const int batch = int(ti.batch);
        const uint32_t buf = tileCount & 1u;
        const uint32_t par = (tileCount >> 1) & 1u;
        const int oc = c0 + quarter * 32 + lane;
        const bool ocValid = oc < p.N;
        const bool warpLive = c0 + quarter * 32 < p.N; // else all 32 channels of this warp are past the end
        const int32_t *corrBatch = p.corr + (p.batchedCorr ? int64_t(batch) * p.numClasses * p.N : 0);
        if (RESIDUAL && storer) {
            // The previous tile's store has read its C/D tile (and so have all before it): the shortcut bytes of the
            // next tile may be loaded into it.  (This waits for a store that was issued a moment ago; without a
            // shortcut to fetch the wait is put off to the end of the tile, see there.)
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            if (tileCount > 0) {
                mbarArrive(&bars->cdEmpty[buf ^ 1u]);
            }
        }
        if (c0 != curC0 || (p.batchedCorr && batch != curBatch)) {
            const int ci = (p.epi.main.perChannel && ocValid) ? oc : 0;
            k.fm = makeFastRescale(__ldg(p.epi.main.mult + ci), int32_t(__ldg(p.epi.main.shift + ci)), p.epi.main.inZp,
                                   p.epi.main.doubleRound != 0);
            k.corr0 = ocValid ? __ldg(corrBatch + int64_t(baseClass) * p.N + oc) : 0;
            k.corrX = int32_t(uint32_t(k.corr0) - uint32_t(k.fm.zpIn));
            // shift >= 32 here whenever the constants below are used
            const bool twoRounds = p.epi.main.doubleRound != 0;
            const int shiftM = k.fm.s1 + k.fm.s2;
            k.rnM = (uint64_t(1) << ((shiftM > 0 ? shiftM : 1) - 1)) - (twoRounds ? (uint64_t(1) << 30) : 0);
            k.bumpM = twoRounds ? 0x80000000u : 0u;
            k.fast = __all_sync(0xffffffffu, k.fm.s1 == 32) && p.corrSmall != 0;
            // 32-bit words only: every lane's shift is 32..60 and the host has bounded |x| below 2^29.  The sign of x is
            // left out without double rounding, and where every x < 0 ends at the lower clamp bound whichever way it was
            // rounded (no negative multiplier, bound not below the output zero point).
            k.words32 = 0;
            if (p.corrSmall >= 2 && __all_sync(0xffffffffu, shiftM >= 32 && shiftM <= 60)) {
                const bool signFree = !twoRounds || (k.loMain >= k.outZpMain && __all_sync(0xffffffffu, k.fm.mult >= 0));
                k.words32 = signFree ? 2 : 1;
                k.corrX4 = int32_t(uint32_t(k.corrX) * 4u);
                k.c32 = (shiftM >= 32 ? int32_t(1) << ((shiftM - 31) & 31) : 0) + (twoRounds ? 1 : 0);
                k.shift32 = shiftM - 30;
            }
            curC0 = c0;
            curBatch = batch;
        }
        // Border class of every pixel of this warp's share of the tile, in registers: lane l holds the classes of the
        // share's pixels l, l + 32, ...  (A table in shared memory for all warps needed a barrier among the epilogue
        // warps in every tile.)
        constexpr int kClassRegs = kColsPerWarp / 32;
        int clsReg[kClassRegs];
        if (hasClasses) {
#pragma unroll
            for (int q = 0; q < kClassRegs; ++q) {
                const int64_t m = int64_t(m0) + part * kColsPerWarp + q * 32 + lane;
                int c = baseClass;
                if (m < p.M) {
                    const uint32_t rem = uint32_t(m) - fastDiv(uint32_t(m), p.divPlane) * p.divPlane.d; // pixel inside its image
                    const uint32_t oy = fastDiv(rem, p.divOW);
                    c = int(__ldg(p.rowClass + oy)) * p.numColClasses + int(__ldg(p.colClass + (rem - oy * uint32_t(p.OW))));
                }
                clsReg[q] = c;
            }
        }
        if (!tableReady) {
            if (!mbarWait(&bars->tabFull, 0u, 7)) {
                break;
            }
            tableReady = true;
        }
        if (RESIDUAL && !mbarWait(&bars->cFull[buf], par, 6)) {
            break;
        }
        if (STORE_WARP && !RESIDUAL && !mbarWait(&bars->cdEmpty[buf], par ^ 1u, 18)) {
            break; // (the store that last read this C/D tile; passes at once for the first two tiles)
        }
        if (!mbarWait(&bars->accFull[buf], par, 4)) {
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmemBase + buf * uint32_t(BNP) + (uint32_t(quarter * 32) << 16) + uint32_t(part * kColsPerWarp);
        // this thread's column of the C/D tile, at the first pixel of its half
        const uint32_t cd = smemAddr(cdTiles + buf * (BNP * 128) + (part * kColsPerWarp) * 128 + quarter * 32 + lane);
        const auto borderFix = [&](uint32_t (&acc)[16], int col) {
            // pixels of this slice (col .. col + 15 of the warp's share) whose window crosses the border take their own
            // class's correction; their classes sit in lanes col % 32 .. of register col / 32
            int mine = clsReg[0];
#pragma unroll
            for (int q = 1; q < kClassRegs; ++q) {
                mine = (col >> 5) == q ? clsReg[q] : mine;
            }
            const uint32_t borderMask = (__ballot_sync(0xffffffffu, mine != baseClass) >> (col & 31)) & 0xffffu;
            if (borderMask != 0) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if ((borderMask >> j) & 1u) {
                        const int c = __shfl_sync(0xffffffffu, mine, (col & 31) + j);
                        if (ocValid) {
                            acc[j] += uint32_t(__ldg(corrBatch + int64_t(c) * p.N + oc)) - uint32_t(k.corr0);
                        }
                    }
                }
            }
        };
        uint32_t accA[16], accB[16];
        // With sixteen epilogue warps a thread has about a hundred registers: too few for a second accumulator slice
        // in flight.
        constexpr bool kOneSliceAtATime = EW > 12;
        if (kOneSliceAtATime) {
#pragma unroll 1
            for (int st = 0; st < kSteps; ++st) {
                tmemLoad16(taddr + uint32_t(16 * st), accA);
                tmemWait16(accA);
                if (st == kSteps - 1) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    if (lane == 0) {
                        accDrained(buf);
                    }
                }
                if (hasClasses) {
                    borderFix(accA, 16 * st);
                }
                if (warpLive) {
                    rescaleSlice<RESIDUAL>(accA, k, tab128, cd + uint32_t((16 * st) * 128));
                }
            }
        } else {
        tmemLoad16(taddr, accA);
#pragma unroll 1
        for (int st = 0; st < kSteps; st += 2) {
            tmemWait16(accA);
            tmemLoad16(taddr + uint32_t(16 * (st + 1)), accB);
            if (hasClasses) {
                borderFix(accA, 16 * st);
            }
            if (warpLive) {
                rescaleSlice<RESIDUAL>(accA, k, tab128, cd + uint32_t((16 * st) * 128));
            }
            tmemWait16(accB);
            if (st + 2 < kSteps) {
                tmemLoad16(taddr + uint32_t(16 * (st + 2)), accA);
            } else {
                // this warp's part of the accumulator is in registers: hand the buffer back to the MMA warp
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                if (lane == 0) {
                    accDrained(buf);
                }
            }
            if (hasClasses) {
                borderFix(accB, 16 * (st + 1));
            }
            if (warpLive) {
                rescaleSlice<RESIDUAL>(accB, k, tab128, cd + uint32_t((16 * (st + 1)) * 128));
            }
        }
        }
        // make the tile visible to the TMA unit, then one thread stores it (pixels and channels past the
        // tensor's end are clipped by the tensor map)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (STORE_WARP) {
            // hand the tile to the store warp; no barrier among the epilogue warps
            __syncwarp();
            if (lane == 0) {
                mbarArrive(&bars->cdFull[buf]);
            }
            continue;
        }
        if (storer) {
            if (p.progressOut != nullptr) {
                // the previous tile's store -- issued a whole tile ago -- has reached memory: publish that tile
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                if (storedPix != kNoTile) {
                    publishTile(p.progressOut, storedPix);
                }
            } else if (!RESIDUAL) {
                // The other C/D tile is written from the next tile on, by warps that have passed the barrier below: the
                // store that last read it -- issued a whole tile ago, so normally long finished -- must be through.
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }
        }
        ocEpilogueSync<EW>();
        if (storer) {
            if (p.progressIn != nullptr && tileCount == 0) {
                // This launch started on the finished tiles of the launch before it.  Its output may lie where that
                // launch's input lay (the session plans memory by life times), so nothing is written before that
                // launch has ended.
                gridDependencySync();
            }
            tmaStore3d(tmapD, cdTiles + buf * (BNP * 128), c0, m0, batch);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            storedPix = ti.pix;
        }
    }
    if (storer) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (p.progressOut != nullptr && storedPix != kNoTile) {
            publishTile(p.progressOut, storedPix);
        }
    }
}

// The store warp of a kernel that has one (lane 0 works): takes every C/D tile the epilogue warps have filled, stores
// it, frees the tile for the tile after next as soon as the store has read it and, when the launch publishes its
// progress, counts the tile in once the store has reached memory.  Keeping this out of the epilogue warps matters for
// the last step: waiting for the completion of a store and the release that follows cost about half a microsecond per
// tile when the thread that did it was one of theirs (1.10 -> 1.20 ms per 64-image ResNet-50 dispatch).
template <int BNP, int EW, int C_TILE>
__device__ __forceinline__ void storeWarpOcMajor(const CUtensorMap *tmapD, const GemmI8Params &p, OcBarriers *bars,
                                                 uint8_t *cdTiles, int64_t numTiles, int pTiles, int cTiles,
                                                 const EpiWalk &walk) {
    uint32_t tileCount = 0;
    for (int64_t t = walk.first; t < numTiles; t += walk.stride, ++tileCount) {
        const TileIndex ti = decodeTile(p, t, pTiles, cTiles);
        const uint32_t buf = tileCount & 1u;
        if (!mbarWait(&bars->cdFull[buf], (tileCount >> 1) & 1u, 19)) {
            break;
        }
        if (p.progressIn != nullptr && tileCount == 0) {
            // This launch started on the finished tiles of the launch before it.  Its output may lie where that
            // launch's input lay (the session plans memory by life times), so nothing is written before that
            // launch has ended.
            gridDependencySync();
        }
        tmaStore3d(tmapD, cdTiles + buf * (BNP * 128), int(ti.chan) * C_TILE + walk.cOffset, int(ti.pix) * BNP, int(ti.batch));
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbarArrive(&bars->cdEmpty[buf]);
        if (p.progressOut != nullptr) {
            // Published as soon as the store has reached memory.  (Publishing one store behind, so that this thread
            // never waits for the store it has just issued, was slower: 1.069 against 1.052 ms per ResNet-50 dispatch;
            // the launch that follows is waiting for exactly these counters.)
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            publishTile(p.progressOut, ti.pix);
        }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

} // namespace
} // namespace mlel
