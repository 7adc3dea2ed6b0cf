// int8 convolution / matrix product on the tcgen05 tensor cores by pairs of CTAs (a cluster of two, one CTA per
// SM of a TPC), channel-major like gemm_i8_ocmajor.cu:
//
//   D[oc, pix] = sum_k W[oc, k] * X[pix, k]      one tile = 256 output channels x BNP pixels (128, 192 or 256)
//
// One `tcgen05.mma.cta_group::2` of shape M = 256, N = BNP reads the A operand (weights) half from each CTA's
// shared memory -- CTA r of the pair holds channels 128 r .. 128 r + 127 -- and the B operand (pixels) half
// from each as well: CTA r loads pixels r BNP / 2 .. of the tile.  Each CTA gets the accumulator of its own 128
// channels for all BNP pixels in its own tensor memory and runs the epilogue of gemm_i8_ocmajor.cu on it.
//
// Why pairs.  The main loop of the single-CTA kernels is bound by the bytes that move from L2 to shared memory:
// a 128 x 192 tile brings 40 KB per 3.1 M multiply-accumulates.  Here a CTA brings 16 KB of weights and
// BNP / 2 rows of pixels (16 KB for BNP = 256) per 4.2 M multiply-accumulates, and in im2col mode half as many
// window rows per multiply-accumulate.
//
// Protocol of a pair (rank 0 = leader, the only CTA that issues MMAs):
//   full[s]     lives in the leader.  The loads of both CTAs complete on it: every load is the `.cta_group::2` form
//               of the bulk tensor copy, which may complete on a barrier of the peer CTA; the leader's producer
//               announces the bytes of both CTAs with its one arrival.  No load is shared between the CTAs:
//               each fetches its own tiles into its own shared memory.
//   empty[s]    one in each CTA, for that CTA's producer.  The leader commits the stage's MMAs to both, with one
//               `tcgen05.commit` per barrier (the second one names the peer's barrier by its shared::cluster
//               address).
//   accFull[b]  one in each CTA (its epilogue waits on it), committed the same way.
//   accEmpty[b] lives in the leader; the epilogue warps of both CTAs arrive on it.
// All waits are bounded like those of the single-CTA kernels; every thread of both CTAs reaches the cluster
// barrier in front of the TMEM release whatever happened before.
//
// Operands: weights as a K-major matrix [N][K] (optionally one per batch), as the {IC, taps, OC} tap map of an
// OHWI tensor (im2col mode), or as an N-contiguous matrix [batch][K][N] (the run-time second input of a MATMUL,
// an "MN-major" A operand); pixels as a K-major matrix [batch][M][K] or through an im2col map of an NHWC
// tensor.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "gemm_i8_tcgen05.hpp"
#include "tcgen05_common.cuh"

#include "ocmajor_epilogue.cuh"

namespace mlel {
namespace {

using namespace tc;

constexpr int kPairChannels = 2 * kOcTile; // output channels per tile


__device__ __forceinline__ uint32_t clusterCtaRank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapToCta(uint32_t ctaAddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(ctaAddr), "r"(rank));
    return r;
}

__device__ __forceinline__ void clusterSync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Tiled bulk tensor load of one CTA of a pair: lands in this CTA's shared memory, completes on `barAddr`, a
// shared::cluster address that may name a barrier of the peer CTA.
__device__ __forceinline__ void tmaLoad3dPair(const CUtensorMap *map, void *dst, uint32_t barAddr, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smemAddr(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(barAddr), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// The same in im2col mode (see tmaLoadIm2col4d).
__device__ __forceinline__ void tmaLoadIm2col4dPair(const CUtensorMap *map, void *dst, uint32_t barAddr, int c, int w, int h,
                                                    int n, uint16_t offW, uint16_t offH) {
    asm volatile("cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smemAddr(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(barAddr), "r"(c), "r"(w), "r"(h), "r"(n), "h"(offW), "h"(offH)
                 : "memory");
}

// kind::i8 instruction descriptor of the pair's MMA (see instrDesc): M = 256, A optionally MN-major.
__host__ __device__ constexpr uint32_t instrDescPair(int n, bool aMnMajor) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(aMnMajor) << 15) | (uint32_t(n >> 3) << 17) |
           (uint32_t(256 >> 4) << 24);
}

__device__ __forceinline__ void ummaPair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
}

// Makes the barrier at `barAddr` (shared::cluster address, this CTA's or the peer's) complete one arrival when
// all MMAs issued so far by this thread have finished.
__device__ __forceinline__ void ummaCommitPair(uint32_t barAddr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barAddr) : "memory");
}

// One K block of the pair: the four MMAs, the two commits that hand the stage back to both CTAs and, issued ahead
// of them, a non-blocking test of the barrier the next K block waits for (see ummaBlockPeek).
__device__ __forceinline__ uint32_t ummaBlockPeekPair(uint32_t tmemD, uint64_t descA, uint64_t stepA, uint64_t descB,
                                                      uint64_t stepB, uint32_t idesc, uint32_t accumulateFirst, int count,
                                                      uint32_t commitOwn, uint32_t commitPeer, uint64_t *peekBar,
                                                      uint32_t peekParity) {
    uint32_t ready;
    asm volatile("{\n\t.reg .pred q, a0, a1, g1, g2, g3;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
                 "setp.ne.b32 a0, %9, 0;\n\t"
                 "setp.ne.b32 a1, %10, 0;\n\t"
                 "setp.gt.s32 g1, %18, 1;\n\t"
                 "setp.gt.s32 g2, %18, 2;\n\t"
                 "setp.gt.s32 g3, %18, 3;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%3], %4, %5, %8, {%11, %11, %11, %11, %11, %11, %11, %11}, a0;\n\t"
                 "@g1 tcgen05.mma.cta_group::2.kind::i8 [%3], %6, %7, %8, {%11, %11, %11, %11, %11, %11, %11, %11}, a1;\n\t"
                 "@g2 tcgen05.mma.cta_group::2.kind::i8 [%3], %12, %13, %8, {%11, %11, %11, %11, %11, %11, %11, %11}, a1;\n\t"
                 "@g3 tcgen05.mma.cta_group::2.kind::i8 [%3], %14, %15, %8, {%11, %11, %11, %11, %11, %11, %11, %11}, a1;\n\t"
                 "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%16];\n\t"
                 "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%17];\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ready)
                 : "r"(smemAddr(peekBar)), "r"(peekParity), "r"(tmemD), "l"(descA), "l"(descB), "l"(descA + stepA),
                   "l"(descB + stepB), "r"(idesc), "r"(accumulateFirst), "r"(1u), "r"(0u), "l"(descA + 2 * stepA),
                   "l"(descB + 2 * stepB), "l"(descA + 3 * stepA), "l"(descB + 3 * stepB), "r"(commitOwn), "r"(commitPeer),
                   "r"(count)
                 : "memory");
    return ready;
}

// The producer's counterpart (see tmaStagePeekTiled): the stage's two loads of this CTA, completing on the leader's
// barrier `fullAddr`; `expectBytes` != 0 (the leader only) announces the bytes of both CTAs on `fullOwn` first.
__device__ __forceinline__ uint32_t tmaStagePeekTiledPair(uint64_t *fullOwn, uint32_t expectBytes, uint32_t fullAddr,
                                                          const CUtensorMap *mapW, void *dstW, int w0, int w1, int w2,
                                                          const CUtensorMap *mapX, void *dstX, int x0, int x1, int x2,
                                                          uint64_t *peekBar, uint32_t peekParity) {
    uint32_t ready;
    asm volatile("{\n\t.reg .pred q, e;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
                 "setp.ne.b32 e, %4, 0;\n\t"
                 "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %4;\n\t"
                 "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%5], [%6, {%7, %8, %9}], [%15];\n\t"
                 "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%10], [%11, {%12, %13, %14}], [%15];\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ready)
                 : "r"(smemAddr(peekBar)), "r"(peekParity), "r"(smemAddr(fullOwn)), "r"(expectBytes), "r"(smemAddr(dstW)),
                   "l"(reinterpret_cast<uint64_t>(mapW)), "r"(w0), "r"(w1), "r"(w2), "r"(smemAddr(dstX)),
                   "l"(reinterpret_cast<uint64_t>(mapX)), "r"(x0), "r"(x1), "r"(x2), "r"(fullAddr)
                 : "memory");
    return ready;
}
__device__ __forceinline__ uint32_t tmaStagePeekIm2colPair(uint64_t *fullOwn, uint32_t expectBytes, uint32_t fullAddr,
                                                           const CUtensorMap *mapW, void *dstW, int w0, int w1, int w2,
                                                           const CUtensorMap *mapX, void *dstX, int c, int w, int h, int n,
                                                           uint16_t offW, uint16_t offH, uint64_t *peekBar,
                                                           uint32_t peekParity) {
    uint32_t ready;
    asm volatile("{\n\t.reg .pred q, e;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
                 "setp.ne.b32 e, %4, 0;\n\t"
                 "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%3], %4;\n\t"
                 "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%5], [%6, {%7, %8, %9}], [%18];\n\t"
                 "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%10], [%11, {%12, %13, %14, %15}], [%18], {%16, %17};\n\t"
                 "selp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ready)
                 : "r"(smemAddr(peekBar)), "r"(peekParity), "r"(smemAddr(fullOwn)), "r"(expectBytes), "r"(smemAddr(dstW)),
                   "l"(reinterpret_cast<uint64_t>(mapW)), "r"(w0), "r"(w1), "r"(w2), "r"(smemAddr(dstX)),
                   "l"(reinterpret_cast<uint64_t>(mapX)), "r"(c), "r"(w), "r"(h), "r"(n), "h"(offW), "h"(offH), "r"(fullAddr)
                 : "memory");
    return ready;
}

// X_MODE: kXTiled = tmapX is a K-major matrix {K, M, batches}; kXIm2col = tmapX is an im2col map of the NHWC input
//         and tmapW the {IC, taps, OC} weight map.
// W_MN  : tmapW is {N, K, batches}, N contiguous (kXTiled only).
template <int BNP, int NSTAGE, int EW, int X_MODE, bool W_MN, bool RESIDUAL>
__global__ void __launch_bounds__((EW + 4) * 32, 1)
gemmI8Pair(const __grid_constant__ CUtensorMap tmapX, const __grid_constant__ CUtensorMap tmapW,
           const __grid_constant__ CUtensorMap tmapC, const __grid_constant__ CUtensorMap tmapD, const GemmI8Params p) {
    extern __shared__ uint8_t rawSmem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    constexpr int kHalf = BNP / 2; // pixels this CTA loads per K block
    constexpr int kTileW = kOcTile * BK;
    constexpr int kTileX = kHalf * BK;
    constexpr int kTileCd = BNP * 128;
    static_assert(kTileX % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
    uint8_t *tilesW = smem;
    uint8_t *tilesX = smem + NSTAGE * kTileW;
    uint8_t *cdTiles = smem + NSTAGE * (kTileW + kTileX);
    uint8_t *resTab = cdTiles + 2 * kTileCd;
    OcBarriers *bars = reinterpret_cast<OcBarriers *>(resTab + (RESIDUAL ? kResidualTableBytes : 0));

    static_assert(NSTAGE <= 6, "OcBarriers holds six stages");
    static_assert(BK / UMMA_K == 4, "the MMA loop issues four instructions per K block");
    // Warp roles: 0 MMA issuer (leader CTA) and TMEM owner, 1 TMA producer, 2 tile stores, 3 idle, 4 .. EW + 3 epilogue (a warp
    // reads the TMEM lane quarter given by its index modulo 4, so the epilogue starts on a multiple of four).  The two
    // single-lane roles come first: where the warp schedulers prefer older warps, their few instructions, which pace
    // the whole pair, are not held up by the epilogue warps that share their schedulers.
    constexpr int kMmaWarpP = 0, kTmaWarpP = 1, kStoreWarpP = 2, kFirstEpiWarp = 4;
    constexpr uint32_t kTmemCols = 2 * BNP <= 256 ? 256u : 512u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = clusterCtaRank();
    const int64_t pairIdx = blockIdx.x >> 1, numPairs = gridDim.x >> 1;
    const int numKb = X_MODE == kXIm2col ? p.KH * p.KW * p.kbPerTap : (p.K + BK - 1) / BK;
    const int pTiles = (p.M + BNP - 1) / BNP;
    const int cTiles = (p.N + kPairChannels - 1) / kPairChannels;
    const int64_t numTiles = int64_t(pTiles) * cTiles * p.batches;
    const auto tileOf = [&](int64_t tile) {
        const uint32_t overP = fastDiv(uint32_t(tile), p.divTiles0), overC = fastDiv(overP, p.divTiles1);
        OcTile c;
        c.m0 = int(uint32_t(tile) - overP * uint32_t(pTiles)) * BNP;
        c.c0 = int(overP - overC * uint32_t(cTiles)) * kPairChannels + int(rank) * kOcTile;
        c.batch = int(overC);
        return c;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbarInit(&bars->full[s], 1u); // the leader's producer (the barrier is used in the leader only)
            mbarInit(&bars->empty[s], 1u);
        }
        for (int b = 0; b < 2; ++b) {
            mbarInit(&bars->accFull[b], 1u);
            mbarInit(&bars->accEmpty[b], uint32_t(2 * EW)); // epilogue warps of both CTAs (used in the leader only)
            mbarInit(&bars->cFull[b], 1u);
            mbarInit(&bars->cdEmpty[b], 1u);
            mbarInit(&bars->cdFull[b], uint32_t(EW));
        }
        mbarInit(&bars->tabFull, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarpP) {
        // the same warp of both CTAs: the pair's tensor memory is allocated (and later released) together
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&bars->tmemBase)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    clusterSync(); // barriers of both CTAs are initialised before either signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmemBase = bars->tmemBase;
    if (rank != 0 && threadIdx.x == 0) {
        // the leader's MMAs write both accumulators at one address: both allocations must have the same base
        uint32_t leaderBase;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(leaderBase) : "r"(mapToCta(smemAddr(&bars->tmemBase), 0u)));
        if (leaderBase != tmemBase) {
            atomicCAS(&g_tcgen05Error, 0, 29);
        }
    }
    if (RESIDUAL && warp == kTmaWarpP && lane == 0) {
        mbarArriveExpectTx(&bars->tabFull, uint32_t(kResidualTableBytes));
        bulkLoad(resTab, p.residualTable, uint32_t(kResidualTableBytes), &bars->tabFull);
    }
    gridDependencySync(); // from here on activations are read and written

    if (warp == kTmaWarpP) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            const uint32_t fullLeader = mapToCta(smemAddr(&bars->full[0]), 0u);
            uint32_t tileCount = 0;
            uint32_t ready = 0; // 1: the stage of the coming K block is known to be empty (see tmaStagePeekTiled)
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = pairIdx; t < numTiles && ok; t += numPairs, ++tileCount) {
                const OcTile tc = tileOf(t);
                // first pixel of this CTA's half of the tile; a half that lies past the last pixel loads pixel 0
                // on (its results are clipped by the store)
                int mh = tc.m0 + int(rank) * kHalf;
                if (mh >= p.M) {
                    mh = 0;
                }
                int w0 = 0, h0 = 0, n0 = 0, kx = 0, ky = 0, cb = 0;
                if (X_MODE == kXIm2col) {
                    n0 = int(fastDiv(uint32_t(mh), p.divPlane));
                    const int rem = mh - n0 * p.OH * p.OW;
                    const int oy = int(fastDiv(uint32_t(rem), p.divOW));
                    h0 = oy * p.strideY - p.padTop;
                    w0 = (rem - oy * p.OW) * p.strideX - p.padLeft;
                }
                for (int kb = 0; kb < numKb; ++kb) {
                    if (ready == 0) {
                        ok = mbarWait(&bars->empty[s], phase ^ 1u, 21);
                        if (!ok) {
                            break;
                        }
                    }
                    const int sNext = s + 1 == NSTAGE ? 0 : s + 1;
                    const uint32_t phaseNext = sNext == 0 ? phase ^ 1u : phase;
                    const uint32_t fullAddr = fullLeader + uint32_t(s) * uint32_t(sizeof(uint64_t));
                    // The leader announces the bytes of both CTAs.  The peer's copies need no arrival of their own: they
                    // are issued after the peer's empty[s] completed, i.e. after the MMAs that read the stage's previous
                    // contents, which themselves waited for the previous phase of this barrier; so they can only count
                    // towards the phase this announcement belongs to (before it, the count of pending bytes is
                    // transiently negative).  A release-arrival on the leader's barrier per stage was measured at about
                    // 1000 cycles in the peer's producer, which then paced the whole pair.
                    const uint32_t expectBytes = rank == 0 ? uint32_t(2 * (kTileW + kTileX)) : 0u;
                    if (X_MODE == kXIm2col) {
                        ready = tmaStagePeekIm2colPair(&bars->full[s], expectBytes, fullAddr, &tmapW, tilesW + s * kTileW, cb,
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
                    } else if (W_MN) {
                        ready = tmaStagePeekTiledPair(&bars->full[s], expectBytes, fullAddr, &tmapW, tilesW + s * kTileW, tc.c0,
                                                      kb * BK, tc.batch, &tmapX, tilesX + s * kTileX, kb * BK, mh, tc.batch,
                                                      &bars->empty[sNext], phaseNext ^ 1u);
                    } else {
                        ready = tmaStagePeekTiledPair(&bars->full[s], expectBytes, fullAddr, &tmapW, tilesW + s * kTileW,
                                                      kb * BK, tc.c0, p.batchedB ? tc.batch : 0, &tmapX, tilesX + s * kTileX,
                                                      kb * BK, mh, tc.batch, &bars->empty[sNext], phaseNext ^ 1u);
                    }
                    s = sNext;
                    phase = phaseNext;
                }
                if (RESIDUAL && ok) {
                    // the shortcut bytes of this CTA's 128 channels, once the store that last used the C/D tile has read it
                    const uint32_t buf = tileCount & 1u;
                    ok = mbarWait(&bars->cdEmpty[buf], ((tileCount >> 1) & 1u) ^ 1u, 26);
                    if (ok) {
                        mbarArriveExpectTx(&bars->cFull[buf], uint32_t(kTileCd));
                        tmaLoad3d(&tmapC, cdTiles + buf * kTileCd, &bars->cFull[buf], tc.c0, tc.m0, tc.batch);
                    }
                }
            }
        }
    } else if (warp == kMmaWarpP) {
        // ---------------- MMA issuer (leader only) ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instrDescPair(BNP, W_MN);
            // Everything the loop needs per K block is kept in registers and stepped, not recomputed: the stage's two
            // operand descriptors (the address field counts 16-byte units and never leaves its 14 bits), its barrier
            // addresses in both CTAs, its phase.  This one thread's instruction stream paces the pair: with the
            // barrier tested after the MMAs and commits about 630 cycles per K block were measured, with or without
            // the copies, against 512 that the MMAs take; hence the test ahead of them (ummaBlockPeekPair).
            const uint64_t descW0 =
                W_MN ? smemDesc(smemAddr(tilesW), BK * 128, 1024) : smemDesc(smemAddr(tilesW), 16, 1024);
            const uint64_t descX0 = smemDesc(smemAddr(tilesX), 16, 1024);
            constexpr uint64_t kStepW = uint64_t(W_MN ? UMMA_K * 128 : UMMA_K) >> 4, kStepX = uint64_t(UMMA_K) >> 4;
            const uint32_t emptyOwn0 = smemAddr(&bars->empty[0]), emptyPeer0 = mapToCta(emptyOwn0, 1u);
            const uint32_t accFullOwn = smemAddr(&bars->accFull[0]), accFullPeer = mapToCta(accFullOwn, 1u);
            uint64_t dw = descW0, dx = descX0;
            uint32_t s = 0, phase = 0, tileCount = 0;
            uint32_t ready = 0; // 1: the stage of the coming K block is known to be full (see ummaBlockPeek)
            bool ok = true;
            for (int64_t t = pairIdx; t < numTiles && ok; t += numPairs, ++tileCount) {
                const uint32_t buf = tileCount & 1u;
                ok = mbarWait(&bars->accEmpty[buf], ((tileCount >> 1) & 1u) ^ 1u, 25);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmemD = tmemBase + buf * uint32_t(BNP);
                int kLeft = X_MODE == kXIm2col ? p.IC : p.K; // bytes of K in the coming block's tap or K axis
                for (int kb = 0; kb < numKb; ++kb) {
                    if (ready == 0) {
                        ok = mbarWait(&bars->full[s], phase, 22);
                        if (!ok) {
                            break;
                        }
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sNext = s + 1 == uint32_t(NSTAGE) ? 0u : s + 1;
                    const uint32_t phaseNext = sNext == 0 ? phase ^ 1u : phase;
                    // the stage is free in both CTAs once these MMAs have read it
                    ready = ummaBlockPeekPair(tmemD, dw, kStepW, dx, kStepX, idesc, kb != 0 ? 1u : 0u, ummaCountFor(kLeft),
                                              emptyOwn0 + s * 8u, emptyPeer0 + s * 8u, &bars->full[sNext], phaseNext);
                    kLeft -= BK;
                    if (kLeft <= 0) {
                        kLeft = X_MODE == kXIm2col ? p.IC : 0;
                    }
                    if (sNext == 0) {
                        dw = descW0, dx = descX0;
                    } else {
                        dw += uint64_t(kTileW >> 4), dx += uint64_t(kTileX >> 4);
                    }
                    s = sNext;
                    phase = phaseNext;
                }
                if (ok) {
                    ummaCommitPair(accFullOwn + buf * 8u);
                    ummaCommitPair(accFullPeer + buf * 8u);
                }
            }
        }
    } else if (warp == kStoreWarpP) {
        // ---------------- store warp (both CTAs) ----------------
        if (lane == 0) {
            EpiWalk walk{};
            walk.first = pairIdx, walk.stride = numPairs;
            walk.cOffset = int(rank) * kOcTile;
            storeWarpOcMajor<BNP, EW, kPairChannels>(&tmapD, p, bars, cdTiles, numTiles, pTiles, cTiles, walk);
        }
    } else if (warp >= kFirstEpiWarp) {
        // ---------------- epilogue (both CTAs, each on its own 128 channels) ----------------
        EpiWalk walk{};
        walk.first = pairIdx, walk.stride = numPairs;
        walk.cOffset = int(rank) * kOcTile;
        walk.accEmpty[0] = mapToCta(smemAddr(&bars->accEmpty[0]), 0u);
        walk.accEmpty[1] = mapToCta(smemAddr(&bars->accEmpty[1]), 0u);
        epilogueOcMajor<BNP, EW, RESIDUAL, kPairChannels, true>(&tmapD, p, bars, resTab, cdTiles, tmemBase,
                                                                warp - kFirstEpiWarp, lane, numTiles, pTiles, cTiles, walk);
    }

    // Neither CTA may leave (or release tensor memory) while the other's MMAs, commits or arrivals can still
    // reach it.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    clusterSync();
    if (warp == kMmaWarpP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(kTmemCols) : "memory");
    }
}

struct PairMaps {
    CUtensorMap x, w, c, d;
};

template <int BNP, int NSTAGE, int EW, int X_MODE, bool W_MN, bool RESIDUAL>
int launchPair(const PairMaps &maps, const GemmI8Params &params, cudaStream_t s) {
    GemmI8Params p = params;
    p.divPlane = makeFastDiv(int64_t(p.OH) * p.OW), p.divOW = makeFastDiv(p.OW);
    p.divTiles0 = makeFastDiv((p.M + BNP - 1) / BNP), p.divTiles1 = makeFastDiv((p.N + kPairChannels - 1) / kPairChannels);
    constexpr size_t smemBytes = size_t(NSTAGE) * (kOcTile * BK + (BNP / 2) * BK) + 2 * size_t(BNP) * 128 +
                                 (RESIDUAL ? size_t(kResidualTableBytes) : 0) + sizeof(OcBarriers) + 1024;
    static_assert(smemBytes <= 232448, "shared memory per CTA");
    auto kernel = gemmI8Pair<BNP, NSTAGE, EW, X_MODE, W_MN, RESIDUAL>;
    if (!allowDynamicSmem(reinterpret_cast<const void *>(kernel), smemBytes)) {
        return MLEL_ERROR_DEVICE;
    }
    const int64_t tiles = int64_t((p.M + BNP - 1) / BNP) * ((p.N + kPairChannels - 1) / kPairChannels) * p.batches;
    if (tiles >= (int64_t(1) << 31)) {
        setLastError("paired int8 GEMM: too many tiles");
        return MLEL_ERROR_UNKNOWN;
    }
    const int maxPairs = smCount() / 2;
    const int pairs = int(tiles < maxPairs ? tiles : maxPairs);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(2 * pairs));
    cfg.blockDim = dim3(unsigned((EW + 4) * 32));
    cfg.dynamicSmemBytes = smemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attrs[2]{};
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 2, attrs[0].val.clusterDim.y = 1, attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, maps.x, maps.w, maps.c, maps.d, p);
    if (err != cudaSuccess) {
        setLastError(std::string("tcgen05 paired convolution launch: ") + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

template <int BNP, int NSTAGE, int NSTAGE_RES, int EW>
int launchPairShape(const PairMaps &maps, const GemmI8Params &p, int xMode, bool wMn, cudaStream_t s) {
    if (p.epi.hasResidual) {
        return xMode == kXIm2col ? launchPair<BNP, NSTAGE_RES, EW, kXIm2col, false, true>(maps, p, s)
                                 : launchPair<BNP, NSTAGE_RES, EW, kXTiled, false, true>(maps, p, s);
    }
    if (xMode == kXIm2col) {
        return launchPair<BNP, NSTAGE, EW, kXIm2col, false, false>(maps, p, s);
    }
    return wMn ? launchPair<BNP, NSTAGE, EW, kXTiled, true, false>(maps, p, s)
               : launchPair<BNP, NSTAGE, EW, kXTiled, false, false>(maps, p, s);
}

} // namespace

bool gemmI8PairApplies(const GemmI8Problem &q) {
    const GemmI8Params &p = q.params;
    if (p.out8 == nullptr || !p.epi.hasMain || p.N <= kOcTile || p.gatherTable != nullptr) {
        return false;
    }
    if (p.N % 16 != 0 || p.ldOut % 16 != 0 || p.K % 16 != 0 || (reinterpret_cast<uintptr_t>(p.out8) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(q.bMatrix) & 15u) != 0) {
        return false;
    }
    if (q.aMatrix != nullptr) {
        if ((reinterpret_cast<uintptr_t>(q.aMatrix) & 15u) != 0 || q.aRowBytes % 16 != 0) {
            return false;
        }
    } else if (q.bMnMajor || p.batchedB || q.batches != 1 || p.IC % 16 != 0 || p.KH <= 0 ||
               (reinterpret_cast<uintptr_t>(p.in) & 15u) != 0) {
        return false; // the pixel operand of a window comes through an im2col map or not at all
    }
    if (p.epi.hasResidual &&
        (q.bMnMajor || q.batches != 1 || p.residualTable == nullptr || (reinterpret_cast<uintptr_t>(p.residualTable) & 15u) != 0 ||
         p.epi.main.lo < -128 || p.epi.main.hi > 127 || (reinterpret_cast<uintptr_t>(p.epi.shortcut) & 15u) != 0)) {
        return false;
    }
    return true;
}

// Pixels per tile for a problem of `pixels` x `channels` x `batches`: the width whose tiles fill the pairs' waves
// best, wider tiles (less operand traffic per multiply-accumulate) winning ties.
static int pairTileWidth(int64_t pixels, int64_t channels, int64_t batches, int numKb, int pairs) {
    const int forced = tensorCoreTuning().pairTilePixels.load(std::memory_order_relaxed);
    if (forced == 128 || forced == 192 || forced == 256) {
        return forced;
    }
    const int64_t cTiles = (channels + kPairChannels - 1) / kPairChannels;
    int best = 256;
    double bestCost = 0;
    for (const int width : {256, 192, 128}) {
        const int64_t tiles = ((pixels + width - 1) / width) * cTiles * batches;
        const int64_t waves = (tiles + pairs - 1) / pairs;
        // time of a tile: its K blocks (bytes a CTA brings per block) plus an epilogue share per pixel
        const double perTile = numKb * (16.0 + width / 16.0) + 0.25 * width;
        const double cost = double(waves) * perTile;
        if (width == 256 || cost < bestCost * 0.97) {
            best = width;
            bestCost = cost;
        }
    }
    return best;
}

int gemmI8PairLaunch(const GemmI8Problem &q, cudaStream_t s, bool *taken) {
    *taken = false;
    GemmI8Params p = q.params;
    p.batches = q.batches;
    const int pairs = smCount() / 2;
    const bool im2col = q.aMatrix == nullptr;
    const int numKb = im2col ? p.KH * p.KW * ((p.IC + 127) / 128) : (p.K + BK - 1) / BK;
    const int width = pairTileWidth(p.M, p.N, q.batches, numKb, pairs);
    const uint32_t half = uint32_t(width / 2);
    PairMaps maps{};
    int xMode = kXTiled;
    if (!im2col) {
        if (!makeMap(&maps.x, q.aMatrix, uint64_t(p.K), uint64_t(p.M), uint64_t(q.batches), uint64_t(q.aRowBytes),
                     uint64_t(q.aBatchBytes), BK, half)) {
            return MLEL_ERROR_DEVICE;
        }
        if (q.bMnMajor) {
            // weights [batches][K][N], N contiguous
            if (!makeMap(&maps.w, q.bMatrix, uint64_t(p.N), uint64_t(p.K), uint64_t(q.batches), uint64_t(q.bRowBytes),
                         uint64_t(q.bBatchBytes), kOcTile, BK)) {
                return MLEL_ERROR_DEVICE;
            }
        } else if (!makeMap(&maps.w, q.bMatrix, uint64_t(p.K), uint64_t(p.N), uint64_t(p.batchedB ? q.batches : 1),
                            uint64_t(q.bRowBytes), uint64_t(q.bBatchBytes ? q.bBatchBytes : q.bRowBytes * uint64_t(p.N)), BK,
                            kOcTile)) {
            return MLEL_ERROR_DEVICE;
        }
    } else {
        if (!makeIm2colMap(&maps.x, p.in, p.M / (p.OH * p.OW), p.H, p.W, p.IC, p.KH, p.KW, p.padTop, p.padLeft, p.OH, p.OW,
                           p.strideY, p.strideX, p.dilY, p.dilX, half) ||
            !makeWeightTapMap(&maps.w, q.bMatrix, p.IC, p.KH * p.KW, p.N, kOcTile)) {
            return MLEL_SUCCESS; // the driver refused the geometry: not taken, the caller uses another kernel
        }
        xMode = kXIm2col;
        p.kbPerTap = (p.IC + 127) / 128;
    }
    const uint64_t plane = uint64_t(p.ldOut) * uint64_t(p.M);
    if (!makeMap(&maps.d, p.out8, uint64_t(p.N), uint64_t(p.M), uint64_t(q.batches), uint64_t(p.ldOut), plane, kOcTile,
                 uint32_t(width), false)) {
        return MLEL_ERROR_DEVICE;
    }
    if (p.epi.hasResidual && !makeMap(&maps.c, p.epi.shortcut, uint64_t(p.N), uint64_t(p.M), 1, uint64_t(p.ldOut), plane,
                                      kOcTile, uint32_t(width), false)) {
        return MLEL_ERROR_DEVICE;
    }
    *taken = true;
    g_tensorCoreLaunches[2].fetch_add(1, std::memory_order_relaxed);
    if (width == 256) {
        return launchPairShape<256, 4, 3, 16>(maps, p, xMode, q.bMnMajor, s);
    }
    return width == 192 ? launchPairShape<192, 5, 4, 12>(maps, p, xMode, q.bMnMajor, s)
                        : launchPairShape<128, 6, 4, 8>(maps, p, xMode, q.bMnMajor, s);
}

int pairErrorWord() { return tc::readErrorWord(); }


} // namespace mlel
