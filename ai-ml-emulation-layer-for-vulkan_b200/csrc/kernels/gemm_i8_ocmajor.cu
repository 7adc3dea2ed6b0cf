// int8 convolution on the tcgen05 tensor cores with the output channel on the TMEM lane ("channel-major"
// accumulator).  Companion of gemm_i8_tcgen05.cu for fused int8 outputs with many output channels:
//
//   D[oc, pix] = sum_k W[oc, k] * X[pix, k]
//
//   A operand  - weight tile, 128 output channels x 128 K bytes, TMA from the OHWI weight matrix [OC][K]
//   B operand  - BNP (128 or 256) output pixels x 128 K bytes: TMA tiles of a row-major pixel matrix (1x1
//                stride-1 convolution); TMA in im2col mode for other windows (one instruction fetches one tap,
//                128 channels, of all the tile's windows, zero-filled outside the image and past the last
//                channel, so any channel count that is a multiple of 16 works; the weight tile is zero-filled
//                the same way); gathered with 16-byte cp.async (segment gather) if the driver refuses the map
//   accumulator- TMEM lane = output channel, TMEM column = pixel; two accumulators of BNP columns alternate
//   C/D tile   - a [BNP pixels][128 channels] byte tile in shared memory, two of them alternating with the
//                accumulators: TMA brings the shortcut bytes of the residual tail into it, the epilogue
//                replaces them in place by the results, TMA stores the tile.  Tensor bounds clip both
//                directions, so the epilogue has no address arithmetic and no validity tests per element.
//
// Why a second orientation.  The TOSA RESCALE constants (multiplier, shift, folded rounding term) and the
// zero-point correction are per output channel.  With the channel on the lane every epilogue thread keeps
// the constants of its own channel in registers for the whole tile, where the pixel-major kernel reads
// them from shared memory for every element.  A 256-pixel tile also moves 48 KB from L2 per 4.2 M
// multiply-accumulates instead of 32 KB per 2.1 M.
//
// The residual tail (RESCALE of the main value and of the shortcut, ADD, RESCALE) takes its two
// int8 -> int32 RESCALEs from 256-entry tables computed once per launch with the very function the
// element-wise kernels use, so the results are the same bits.
//
// Zero-point correction, border classes and the bounded waits are those of gemm_i8_tcgen05.cu.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "gemm_i8_tcgen05.hpp"
#include "tcgen05_common.cuh"

#include "ocmajor_epilogue.cuh"

namespace mlel {
namespace {

using namespace tc;


// Threads per CTA: the TMA variants have a store warp where the gather variants have their two gather warps' first.
constexpr int ocThreadsFor(int ew, int xMode) { return xMode == kXGather ? ocThreads(ew, true) : (ew + 3) * 32; }

// X_MODE: how the pixel operand arrives: kXGather = gathered from the NHWC input described by p, kXTiled = tmapX
// is a plain matrix, kXIm2col = tmapX is an im2col map of the NHWC input.
// RESIDUAL: the fused residual tail is present (tmapC describes the shortcut tensor).
template <int BNP, int NSTAGE, int EW, int X_MODE, bool RESIDUAL>
__global__ void __launch_bounds__(ocThreadsFor(EW, X_MODE), 1)
gemmI8OcMajor(const __grid_constant__ CUtensorMap tmapX, const __grid_constant__ CUtensorMap tmapW,
              const __grid_constant__ CUtensorMap tmapC, const __grid_constant__ CUtensorMap tmapD, const GemmI8Params p) {
    extern __shared__ uint8_t rawSmem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    constexpr int kTileW = kOcTile * BK;
    constexpr int kTileX = BNP * BK;
    constexpr int kTileCd = BNP * 128;
    uint8_t *tilesW = smem;
    uint8_t *tilesX = smem + NSTAGE * kTileW;
    uint8_t *cdTiles = smem + NSTAGE * (kTileW + kTileX);
    uint8_t *resTab = cdTiles + 2 * kTileCd; // the residual tail as a table (RESIDUAL only)
    int32_t *tapTab = reinterpret_cast<int32_t *>(resTab + (RESIDUAL ? kResidualTableBytes : 0));
    OcBarriers *bars = reinterpret_cast<OcBarriers *>(tapTab + kTapTabEntries);

    constexpr bool X_TMA = X_MODE != kXGather;
    static_assert(NSTAGE <= 6, "OcBarriers holds six stages");
    constexpr int kOcTmaWarp = EW, kOcMmaWarp = EW + 1, kOcGatherWarp0 = EW + 2; // TMA variants: EW + 2 = store warp
    constexpr uint32_t kTmemCols = 2 * BNP <= 256 ? 256u : 512u; // two accumulators; allocations are powers of two
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int numKb = X_MODE == kXIm2col ? p.KH * p.KW * p.kbPerTap : (p.K + BK - 1) / BK;
    const int pTiles = (p.M + BNP - 1) / BNP;
    const int cTiles = (p.N + kOcTile - 1) / kOcTile;
    const int64_t numTiles = int64_t(pTiles) * cTiles * p.batches;
    const auto tileOf = [&](int64_t tile) {
        const TileIndex ti = decodeTile(p, tile, pTiles, cTiles);
        OcTile c;
        c.m0 = int(ti.pix) * BNP;
        c.c0 = int(ti.chan) * kOcTile;
        c.batch = int(ti.batch);
        return c;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbarInit(&bars->full[s], X_TMA ? 1u : 1u + uint32_t(kOcGatherThreads));
            mbarInit(&bars->empty[s], 1u);
        }
        for (int b = 0; b < 2; ++b) {
            mbarInit(&bars->accFull[b], 1u);
            mbarInit(&bars->accEmpty[b], uint32_t(EW));
            mbarInit(&bars->cFull[b], 1u);
            mbarInit(&bars->cdEmpty[b], 1u);
            mbarInit(&bars->cdFull[b], uint32_t(EW));
        }
        mbarInit(&bars->tabFull, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kOcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&bars->tmemBase)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!X_TMA && warp >= kOcGatherWarp0) {
        fillTapTable(p, tapTab, kOcGatherWarp0 * 32, kOcGatherThreads);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmemBase = bars->tmemBase;
    if (RESIDUAL && warp == kOcTmaWarp && lane == 0) {
        // the table is a constant of the pipeline, not an activation: it may be fetched before the previous
        // kernel of the stream has finished
        mbarArriveExpectTx(&bars->tabFull, uint32_t(kResidualTableBytes));
        bulkLoad(resTab, p.residualTable, uint32_t(kResidualTableBytes), &bars->tabFull);
    }
    // From here on activations are read and written.  With a progress table of the launch before (TMA variants
    // only) the producer lane waits per tile for the pixel tiles it reads and the storing thread waits for the whole
    // grid before its first store; nobody else touches activations.
    const bool byTiles = X_TMA && p.progressIn != nullptr;
    if (!byTiles) {
        gridDependencySync();
    } else {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    if (warp == kOcTmaWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t tileCount = 0;
            uint32_t ready = 0; // 1: the stage of the coming K block is known to be empty (see tmaStagePeekTiled)
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileCount) {
                const OcTile tc = tileOf(t);
                // im2col mode: first tap of the tile's first window, and the running position on the K axis
                int w0 = 0, h0 = 0, n0 = 0, kx = 0, ky = 0, cb = 0;
                if (X_MODE == kXIm2col) {
                    n0 = int(fastDiv(uint32_t(tc.m0), p.divPlane));
                    const int rem = tc.m0 - n0 * p.OH * p.OW;
                    const int oy = int(fastDiv(uint32_t(rem), p.divOW));
                    h0 = oy * p.strideY - p.padTop;
                    w0 = (rem - oy * p.OW) * p.strideX - p.padLeft;
                }
                if (byTiles) {
                    // input pixels this tile reads, as a range of the producing launch's pixel index (whole input rows
                    // from the first window's first row to the last window's last row)
                    const int mLast = min(tc.m0 + BNP, p.M) - 1;
                    int64_t lo = tc.m0, hi = mLast;
                    if (X_MODE == kXIm2col) {
                        const int n1 = int(fastDiv(uint32_t(mLast), p.divPlane));
                        const int oy0 = int(fastDiv(uint32_t(tc.m0 - n0 * p.OH * p.OW), p.divOW));
                        const int oy1 = int(fastDiv(uint32_t(mLast - n1 * p.OH * p.OW), p.divOW));
                        const int yLo = max(oy0 * p.strideY - p.padTop, 0);
                        const int yHi = min(oy1 * p.strideY - p.padTop + (p.KH - 1) * p.dilY, p.H - 1);
                        lo = (int64_t(n0) * p.H + yLo) * p.W;
                        hi = (int64_t(n1) * p.H + yHi) * p.W + p.W - 1;
                    }
                    if (lo <= hi) {
                        ok = waitTiles(p.progressIn, uint32_t(lo / p.progressInTilePixels), uint32_t(hi / p.progressInTilePixels),
                                       p.progressInTarget, 17);
                        if (!ok) {
                            break;
                        }
                    }
                }
                for (int kb = 0; kb < numKb; ++kb) {
                    if (ready == 0) {
                        ok = mbarWait(&bars->empty[s], phase ^ 1u, 11);
                        if (!ok) {
                            break;
                        }
                    }
                    // the ring runs on across tiles: the next K block's stage follows this one whatever tile it is in
                    const int sNext = s + 1 == NSTAGE ? 0 : s + 1;
                    const uint32_t phaseNext = sNext == 0 ? phase ^ 1u : phase;
                    if (X_MODE == kXTiled) {
                        ready = tmaStagePeekTiled(&bars->full[s], uint32_t(kTileW + kTileX), &tmapW, tilesW + s * kTileW, kb * BK,
                                                  tc.c0, 0, &tmapX, tilesX + s * kTileX, kb * BK, tc.m0, tc.batch,
                                                  &bars->empty[sNext], phaseNext ^ 1u);
                    } else if (X_MODE == kXIm2col) {
                        ready = tmaStagePeekIm2col(&bars->full[s], uint32_t(kTileW + kTileX), &tmapW, tilesW + s * kTileW, cb,
                                                   ky * p.KW + kx, tc.c0, &tmapX, tilesX + s * kTileX, cb, w0, h0, n0,
                                                   uint16_t(kx * p.dilX), uint16_t(ky * p.dilY), &bars->empty[sNext],
                                                   phaseNext ^ 1u);
                        cb += BK;
                        if (cb >= p.IC) {
                            cb = 0;
                            if (++kx == p.KW) {
                                kx = 0;
                                ++ky;
                            }
                        }
                    } else {
                        mbarArriveExpectTx(&bars->full[s], uint32_t(kTileW));
                        tmaLoad3d(&tmapW, tilesW + s * kTileW, &bars->full[s], kb * BK, tc.c0, 0);
                    }
                    s = sNext;
                    phase = phaseNext;
                }
                if (RESIDUAL && ok) {
                    // the tile's shortcut bytes, once the store that last used this C/D tile has read it
                    const uint32_t buf = tileCount & 1u;
                    ok = mbarWait(&bars->cdEmpty[buf], ((tileCount >> 1) & 1u) ^ 1u, 16);
                    if (ok) {
                        mbarArriveExpectTx(&bars->cFull[buf], uint32_t(kTileCd));
                        tmaLoad3d(&tmapC, cdTiles + buf * kTileCd, &bars->cFull[buf], tc.c0, tc.m0, 0);
                    }
                }
            }
        }
    } else if (warp == kOcMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = instrDesc(BNP, false);
            static_assert(BK / UMMA_K == 4, "ummaBlockPeek issues the four MMAs of a K block");
            const uint64_t descW0 = smemDesc(smemAddr(tilesW), 16, 1024), descX0 = smemDesc(smemAddr(tilesX), 16, 1024);
            uint32_t it = 0, tileCount = 0;
            uint32_t ready = 0; // 1: the stage of the coming K block is known to be full (see ummaBlockPeek)
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileCount) {
                const uint32_t buf = tileCount & 1u;
                ok = mbarWait(&bars->accEmpty[buf], ((tileCount >> 1) & 1u) ^ 1u, 15);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmemD = tmemBase + buf * uint32_t(BNP);
                int kLeft = X_MODE == kXIm2col ? p.IC : p.K;
                for (int kb = 0; kb < numKb; ++kb, ++it) {
                    if (ready == 0) {
                        ok = mbarWait(&bars->full[s], phase, 12);
                        if (!ok) {
                            break;
                        }
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // the ring runs on across tiles: the next K block's stage follows this one whatever tile it is in
                    const int sNext = s + 1 == NSTAGE ? 0 : s + 1;
                    const uint32_t phaseNext = sNext == 0 ? phase ^ 1u : phase;
                    ready = ummaBlockPeek(tmemD, descW0 + uint64_t(uint32_t(s) * uint32_t(kTileW >> 4)), 2,
                                          descX0 + uint64_t(uint32_t(s) * uint32_t(kTileX >> 4)), 2, idesc, kb != 0 ? 1u : 0u,
                                          ummaCountFor(kLeft), &bars->empty[s], &bars->full[sNext], phaseNext);
                    // bytes of K in the next block: the rest of the tap's channels (im2col) or of the whole K axis
                    kLeft -= BK;
                    if (kLeft <= 0) {
                        kLeft = X_MODE == kXIm2col ? p.IC : 0;
                    }
                    s = sNext;
                    phase = phaseNext;
                }
                if (ok) {
                    ummaCommit(&bars->accFull[buf]);
                }
            }
        }
    } else if (warp >= kOcGatherWarp0) {
        if (X_TMA) {
            // ---------------- store warp ----------------
            if (lane == 0) {
                EpiWalk walk{};
                walk.first = blockIdx.x, walk.stride = gridDim.x;
                storeWarpOcMajor<BNP, EW, kOcTile>(&tmapD, p, bars, cdTiles, numTiles, pTiles, cTiles, walk);
            }
        }
        // ---------------- pixel gather (implicit GEMM): BNP / 64 tile rows per thread ----------------
        if (!X_TMA) {
            constexpr int kRows = BNP / kOcGatherThreads;
            const int row0 = (warp - kOcGatherWarp0) * 32 + lane;
            const uint32_t swz = uint32_t(row0 & 7); // rows 64 apart share the swizzle phase
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                const OcTile tc = tileOf(t);
                GatherRow rows[kRows];
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    rows[r] = gatherRowSetup(p, int64_t(tc.m0) + row0 + r * kOcGatherThreads);
                }
                int tap = 0, c0 = 0;
                for (int kb = 0; kb < numKb; ++kb, ++it) {
                    const int s = int(it % NSTAGE);
                    const uint32_t phase = (it / NSTAGE) & 1u;
                    ok = mbarWait(&bars->empty[s], phase ^ 1u, 13);
                    if (!ok) {
                        break;
                    }
                    const uint32_t dstRow = smemAddr(tilesX + s * kTileX) + uint32_t(row0) * 128u;
                    gatherBlock<kRows, kOcGatherThreads>(rows, tapTab, p.KH * p.KW, p.IC, tap, c0, dstRow, swz, p.in);
                    // The stage's barrier completes when these copies have landed and every producer arrived.
                    asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(smemAddr(&bars->full[s]))
                                 : "memory");
                    mbarArrive(&bars->full[s]);
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        EpiWalk walk{};
        walk.first = blockIdx.x, walk.stride = gridDim.x;
        epilogueOcMajor<BNP, EW, RESIDUAL, kOcTile, X_TMA>(&tmapD, p, bars, resTab, cdTiles, tmemBase, warp, lane,
                                                           numTiles, pTiles, cTiles, walk);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kOcMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(kTmemCols)
                     : "memory");
    }
}

struct OcMaps {
    CUtensorMap x, w, c, d;
};

template <int BNP, int NSTAGE, int EW, int X_MODE, bool RESIDUAL>
int launchOcMajor(const OcMaps &maps, const GemmI8Params &params, cudaStream_t s) {
    GemmI8Params p = params;
    p.divPlane = makeFastDiv(int64_t(p.OH) * p.OW), p.divOW = makeFastDiv(p.OW);
    const int pixelTiles = (p.M + BNP - 1) / BNP, channelTiles = (p.N + kOcTile - 1) / kOcTile;
    p.divTiles0 = makeFastDiv(p.channelFastest != 0 ? channelTiles : pixelTiles);
    p.divTiles1 = makeFastDiv(p.channelFastest != 0 ? pixelTiles : channelTiles);
    constexpr size_t smemBytes = size_t(NSTAGE) * (kOcTile * BK + BNP * BK) + 2 * size_t(BNP) * 128 +
                                 (RESIDUAL ? size_t(kResidualTableBytes) : 0) +
                                 kTapTabEntries * sizeof(int32_t) + sizeof(OcBarriers) + 1024;
    static_assert(smemBytes <= 232448, "shared memory per CTA");
    auto kernel = gemmI8OcMajor<BNP, NSTAGE, EW, X_MODE, RESIDUAL>;
    if (!allowDynamicSmem(reinterpret_cast<const void *>(kernel), smemBytes)) {
        return MLEL_ERROR_DEVICE;
    }
    const int64_t tiles = int64_t((p.M + BNP - 1) / BNP) * ((p.N + kOcTile - 1) / kOcTile) * p.batches;
    if (tiles >= (int64_t(1) << 31)) {
        setLastError("channel-major int8 GEMM: too many tiles");
        return MLEL_ERROR_UNKNOWN;
    }
    const int grid = int(tiles < smCount() ? tiles : smCount());
    const cudaError_t err = launchDependent(kernel, grid, ocThreadsFor(EW, X_MODE), smemBytes, s, maps.x, maps.w,
                                            maps.c, maps.d, p);
    if (err != cudaSuccess) {
        setLastError(std::string("tcgen05 channel-major convolution launch: ") + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

// The residual table takes 64 KB of shared memory: the variants with a residual tail run with fewer stages
// (they are 1x1 convolutions of one to four K blocks, and the pipeline runs across tile boundaries).
template <int BNP, int NSTAGE, int EW, int X_MODE>
int launchOcMajorMode(const OcMaps &maps, const GemmI8Params &p, cudaStream_t s) {
    constexpr int kStagesResidual = BNP == 128 ? 4 : 2;
    return p.epi.hasResidual ? launchOcMajor<BNP, kStagesResidual, EW, X_MODE, true>(maps, p, s)
                             : launchOcMajor<BNP, NSTAGE, EW, X_MODE, false>(maps, p, s);
}

template <int BNP, int NSTAGE, int EW>
int launchOcMajorShape(const OcMaps &maps, const GemmI8Params &p, int xMode, cudaStream_t s) {
    if (xMode == kXTiled) {
        return launchOcMajorMode<BNP, NSTAGE, EW, kXTiled>(maps, p, s);
    }
    if (xMode == kXIm2col) {
        return launchOcMajorMode<BNP, NSTAGE, EW, kXIm2col>(maps, p, s);
    }
    return launchOcMajorMode<BNP, NSTAGE, EW, kXGather>(maps, p, s);
}

} // namespace

bool gemmI8OcMajorApplies(const GemmI8Problem &q) {
    const GemmI8Params &p = q.params;
    if (p.out8 == nullptr || !p.epi.hasMain || q.bMnMajor || p.batchedB || q.batches != 1 || p.N <= 64) {
        return false;
    }
    // the output (and the shortcut) move as TMA tiles of 16-byte aligned rows
    if (p.N % 16 != 0 || p.ldOut % 16 != 0 || (reinterpret_cast<uintptr_t>(p.out8) & 15u) != 0) {
        return false;
    }
    // a gathered pixel operand goes through the segment gather
    if (q.aMatrix == nullptr && !(p.gatherTable == nullptr && p.KH * p.KW <= kMaxTaps &&
                                  (p.IC == 16 || p.IC == 32 || p.IC == 64 || p.IC % 128 == 0))) {
        return false;
    }
    // the residual table is indexed by the int8 value of the main stage and the shortcut byte
    return !p.epi.hasResidual ||
           (p.residualTable != nullptr && (reinterpret_cast<uintptr_t>(p.residualTable) & 15u) == 0 &&
            p.epi.main.lo >= -128 && p.epi.main.hi <= 127 && (reinterpret_cast<uintptr_t>(p.epi.shortcut) & 15u) == 0);
}

// Tile-level hand-over between consecutive launches (GemmI8Params::progressOut / progressIn, LaunchChain).
//
// Why it is safe.  Launch C follows launch B in the stream, both with programmatic dependent launch, and C's pixel
// operand is B's output.  (1) C's CTAs only become resident once every CTA of B has started (that is when B has
// triggered its dependents), and one CTA fills an SM, so a CTA of C never keeps a CTA of B from running: B's
// counters always advance.  (2) A counter is incremented after the tile's store has completed, with release
// semantics; C acquires it before the TMA loads of the pixels under it.  (3) Before its first store B itself has
// waited for the whole grid before it (at its start, or before that store if it reads by tiles too); so a counter
// of B also tells C that every launch before B has finished, which covers C's other activation input, the shortcut
// tensor of a residual tail.  (4) The session may place C's output where B's input lay: C does not store before
// griddepcontrol.wait has returned, i.e. before B has ended.  (5) The counters are zeroed by a memset at the start of
// the dispatch, which is ordered after the previous dispatch like any other operation of the stream.
int gemmI8OcMajorLaunch(const GemmI8Problem &q, cudaStream_t s, LaunchChain *chain, const LaunchChain *consumed) {
    g_tensorCoreLaunches[1].fetch_add(1, std::memory_order_relaxed);
    GemmI8Params p = q.params;
    p.batches = q.batches;
    p.progressOut = nullptr, p.progressIn = nullptr, p.channelFastest = 0;
    LaunchChain before{}; // what the launch before this one publishes
    if (consumed != nullptr) {
        before = *consumed;
    }
    // Pixels per tile.  Wider tiles move less operand data per multiply-accumulate and spread a tile's fixed work over
    // more outputs, narrower ones fill the last round of CTAs better.  192 pixels (twelve epilogue warps) is the
    // base: measured on the ResNet-50 shapes it beat 128 and 256 pixels for every layer and a rule that weighed
    // waves against width.  Two exceptions follow: layers that underfill the GPU, and layers with many rounds of
    // tiles.  Problems of at most 128 pixels take the narrow tile.
    int width = p.M <= 128 ? 128 : 192;
    {
        // a layer that leaves a quarter of the SMs without a tile takes the narrow tile if that fills more of them
        const int64_t cT = (p.N + kOcTile - 1) / kOcTile;
        const int64_t tiles192 = int64_t((p.M + 191) / 192) * cT, tiles128 = int64_t((p.M + 127) / 128) * cT;
        const int rule = tensorCoreTuning().ocTileRule.load(std::memory_order_relaxed);
        if (rule != 0 && tiles192 * 4 <= int64_t(smCount()) * 3 && tiles128 <= int64_t(smCount())) {
            width = 128;
        }
        // a layer with at least `rule` (default three) rounds of 192-pixel tiles per SM takes the wide tile with its
        // sixteen epilogue warps: what a warp does per tile beside the elements is spread over a third more of them,
        // and the partly filled last round weighs little (0.977 against 1.009 ms per ResNet-50 dispatch; with two the
        // same, with four or more rounds less gain; 256 pixels for every layer: 1.014 ms)
        if (rule >= 2 && tiles192 >= int64_t(smCount()) * rule) {
            width = 256;
        }
    }
    const int forced = tensorCoreTuning().ocTilePixels.load(std::memory_order_relaxed);
    if (forced == 128 || forced == 192 || forced == 256) {
        width = forced;
    }
    OcMaps maps{};
    const uint32_t boxPixels = uint32_t(width);
    int xMode = kXGather;
    if (q.aMatrix != nullptr) {
        // one box = the whole pixel tile of one K block
        if (!makeMap(&maps.x, q.aMatrix, uint64_t(p.K), uint64_t(p.M), uint64_t(q.batches), uint64_t(q.aRowBytes),
                     uint64_t(q.aBatchBytes), BK, uint32_t(width))) {
            return MLEL_ERROR_DEVICE;
        }
        xMode = kXTiled;
    } else if (p.gatherTable == nullptr && p.IC % 16 == 0 && (reinterpret_cast<uintptr_t>(p.in) & 15u) == 0 &&
               (reinterpret_cast<uintptr_t>(q.bMatrix) & 15u) == 0 &&
               makeIm2colMap(&maps.x, p.in, p.M / (p.OH * p.OW), p.H, p.W, p.IC, p.KH, p.KW, p.padTop, p.padLeft, p.OH, p.OW,
                             p.strideY, p.strideX, p.dilY, p.dilX, boxPixels) &&
               makeWeightTapMap(&maps.w, q.bMatrix, p.IC, p.KH * p.KW, p.N, kOcTile)) {
        xMode = kXIm2col;
        p.kbPerTap = (p.IC + 127) / 128;
    }
    if (xMode != kXIm2col && !makeMap(&maps.w, q.bMatrix, uint64_t(p.K), uint64_t(p.N), 1, uint64_t(q.bRowBytes),
                                      uint64_t(q.bRowBytes) * uint64_t(p.N), BK, kOcTile)) {
        return MLEL_ERROR_DEVICE;
    }
    // output and shortcut: [pixels][channels] bytes, unswizzled tiles of 128 channels x (128 or 256) pixels
    const uint64_t plane = uint64_t(p.ldOut) * uint64_t(p.M);
    if (!makeMap(&maps.d, p.out8, uint64_t(p.N), uint64_t(p.M), 1, uint64_t(p.ldOut), plane, kOcTile, boxPixels, false)) {
        return MLEL_ERROR_DEVICE;
    }
    if (p.epi.hasResidual &&
        !makeMap(&maps.c, p.epi.shortcut, uint64_t(p.N), uint64_t(p.M), 1, uint64_t(p.ldOut), plane, kOcTile, boxPixels, false)) {
        return MLEL_ERROR_DEVICE;
    }
    const int progressMode = tensorCoreTuning().tileProgress.load(std::memory_order_relaxed);
    const bool handOver = chain != nullptr && xMode != kXGather && progressMode != 0 &&
                          tensorCoreTuning().dependentLaunch.load(std::memory_order_relaxed) != 0;
    if (handOver && before.prevCounters != nullptr && (progressMode & 1)) {
        // read by tiles when the launch before this one wrote exactly this launch's pixel operand
        const void *input = q.aMatrix != nullptr ? q.aMatrix : static_cast<const void *>(p.in);
        const int64_t inputPixels = q.aMatrix != nullptr ? int64_t(p.M) : int64_t(p.M / (p.OH * p.OW)) * p.H * p.W;
        if (before.prevTensor == input && before.prevPixels == inputPixels) {
            p.progressIn = before.prevCounters;
            p.progressInTilePixels = before.prevTilePixels;
            p.progressInTarget = before.prevTarget;
        }
    }
    if (handOver && chain->publishNext && (progressMode & 2)) {
        const size_t pixelTiles = size_t((p.M + width - 1) / width);
        if (chain->used + pixelTiles <= chain->capacity) {
            p.progressOut = chain->words + chain->used;
            p.channelFastest = (progressMode & 4) ? 1 : 0;
            chain->used += pixelTiles;
            chain->prevTensor = p.out8;
            chain->prevCounters = p.progressOut;
            chain->prevTilePixels = width;
            chain->prevTarget = uint32_t((p.N + kOcTile - 1) / kOcTile);
            chain->prevPixels = p.M;
        }
    }
    if (width == 256) {
        return launchOcMajorShape<256, 3, 16>(maps, p, xMode, s);
    }
    return width == 192 ? launchOcMajorShape<192, 4, 12>(maps, p, xMode, s)
                        : launchOcMajorShape<128, 5, 16>(maps, p, xMode, s);
}

int ocMajorErrorWord() { return tc::readErrorWord(); }

} // namespace mlel
