// int8 convolution on the tcgen05 tensor cores with the output channel on the TMEM lane ("channel-major"
// accumulator).  Companion of gemm_i8_tcgen05.cu for fused int8 outputs with many output channels:
//
//   D[oc, pix] = sum_k W[oc, k] * X[pix, k]
//
//   A operand  - weight tile, 128 output channels x 128 K bytes, TMA from the OHWI weight matrix [OC][K]
//   B operand  - BNP (128 or 256) output pixels x 128 K bytes: TMA from a row-major pixel matrix (1x1
//                stride-1 convolution, materialised im2col), else gathered with 16-byte cp.async
//   accumulator- TMEM lane = output channel, TMEM column = pixel; two accumulators of BNP columns alternate
//
// Why a second orientation.  The TOSA RESCALE constants (multiplier, shift, folded rounding term) and the
// zero-point correction are per output channel.  With the channel on the lane every epilogue thread keeps
// the constants of its own channel in registers for the whole tile, where the pixel-major kernel reads
// them from shared memory for every element; the instruction count per output element roughly halves.
// A 256-pixel tile also moves 48 KB from L2 per 4.2 M multiply-accumulates instead of 32 KB per 2.1 M.
// Stores are one byte per thread; a warp writes 32 consecutive channels of one pixel (one 32-byte sector).
//
// The residual tail (RESCALE of the main value and of the shortcut, ADD, RESCALE) takes its two
// int8 -> int32 RESCALEs from 256-entry tables computed once per launch with the very function the
// element-wise kernels use, so the results are the same bits.
//
// Zero-point correction, border classes and the bounded waits are those of gemm_i8_tcgen05.cu.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_i8_tcgen05.hpp"
#include "tcgen05_common.cuh"

namespace mlel {
namespace {

using namespace tc;

constexpr int kOcTile = 128; // output channels per tile (UMMA M)

struct __align__(8) OcBarriers {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t accFull[2];
    uint64_t accEmpty[2];
    uint32_t tmemBase;
    uint32_t pad;
};

struct OcTile {
    int c0, m0, batch;
};

template <int BNP, bool RESIDUAL>
__device__ __forceinline__ void epilogueOcMajor(const GemmI8Params &p, OcBarriers *bars, uint8_t *clsTab,
                                                const int32_t *lutA, const int32_t *lutB, uint32_t tmemBase, int warp,
                                                int lane, int64_t numTiles, int pTiles, int cTiles) {
    const int quarter = warp & 3; // TMEM lanes [32 * quarter, +32): output channels of the tile
    const int part = warp >> 2;   // which quarter of the tile's pixels
    constexpr int kColsPerWarp = BNP / (kEpilogueWarps / 4);
    constexpr int kSteps = kColsPerWarp / 16;
    FastRescale fo{};
    if (RESIDUAL) {
        fo = makeFastRescale(__ldg(p.epi.out.mult), int32_t(__ldg(p.epi.out.shift)), p.epi.out.inZp,
                             p.epi.out.doubleRound != 0);
    }
    const int32_t outZpMain = p.epi.main.outZp, loMain = p.epi.main.lo, hiMain = p.epi.main.hi;
    FastRescale fm{}; // main RESCALE stage of this thread's output channel
    int32_t corr0 = 0;
    int curC0 = -1, curBatch = -1;
    const bool hasClasses = p.rowClass != nullptr;
    const int baseClass = p.baseClass;
    uint32_t tileCount = 0;
    for (int64_t t = blockIdx.x; t < numTiles; t += gridDim.x, ++tileCount) {
        int64_t tt = t;
        const int c0 = int(tt % cTiles) * kOcTile;
        tt /= cTiles;
        const int m0 = int(tt % pTiles) * BNP;
        const int batch = int(tt / pTiles);
        const uint32_t buf = tileCount & 1u;
        const int oc = c0 + quarter * 32 + lane;
        const bool ocValid = oc < p.N;
        const int32_t *corrBatch = p.corr + (p.batchedCorr ? int64_t(batch) * p.numClasses * p.N : 0);
        if (c0 != curC0 || (p.batchedCorr && batch != curBatch)) {
            const int ci = (p.epi.main.perChannel && ocValid) ? oc : 0;
            fm = makeFastRescale(__ldg(p.epi.main.mult + ci), int32_t(__ldg(p.epi.main.shift + ci)), p.epi.main.inZp,
                                 p.epi.main.doubleRound != 0);
            corr0 = ocValid ? __ldg(corrBatch + int64_t(p.baseClass) * p.N + oc) : 0;
            curC0 = c0;
            curBatch = batch;
        }
        uint8_t *cls = clsTab + buf * BNP;
        if (p.rowClass != nullptr) {
            // border class of every pixel of the tile; the table alternates with the accumulator, so a warp that
            // is a tile ahead never overwrites what a slower warp still reads
            if (threadIdx.x < BNP) {
                const int64_t m = int64_t(m0) + threadIdx.x;
                int c = p.baseClass;
                if (m < p.M) {
                    const int rem = int(m % (int64_t(p.OH) * p.OW));
                    c = int(__ldg(p.rowClass + rem / p.OW)) * p.numColClasses + int(__ldg(p.colClass + rem % p.OW));
                }
                cls[threadIdx.x] = uint8_t(c);
            }
            epilogueSync();
        }
        if (!mbarWait(&bars->accFull[buf], (tileCount >> 1) & 1u, 4)) {
            break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmemBase + buf * uint32_t(BNP) + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
        for (int st = 0; st < kSteps; ++st) {
            const int col = part * kColsPerWarp + st * 16; // first pixel of this step inside the tile
            uint32_t acc[16];
            tmemLoad16(taddr + uint32_t(col), acc);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (st == kSteps - 1) {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                if (lane == 0) {
                    mbarArrive(&bars->accEmpty[buf]);
                }
            }
            const int64_t mBase = int64_t(m0) + col;
            if (mBase >= p.M) {
                continue; // the same for the whole warp
            }
            const int npix = int(min(int64_t(16), int64_t(p.M) - mBase));
            // pixels of this step whose window crosses the border (their class differs from the common one)
            uint32_t borderMask = 0;
            if (hasClasses) {
                borderMask = __ballot_sync(0xffffffffu, lane < 16 && int(cls[col + (lane & 15)]) != baseClass);
            }
            if (ocValid) {
                // pixel part of the address: the same for the whole warp; channel part: 32 bits per thread
                const int64_t off0 = (int64_t(batch) * p.M + mBase) * p.ldOut;
                int8_t *dstRow = p.out8 + off0;
                const uint32_t ld = uint32_t(p.ldOut);
                if (borderMask != 0) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if ((borderMask >> j) & 1u) {
                            const int c = int(cls[col + j]);
                            acc[j] += uint32_t(__ldg(corrBatch + int64_t(c) * p.N + oc)) - uint32_t(corr0);
                        }
                    }
                }
                int32_t sc[16];
                if (RESIDUAL) {
                    const int8_t *scRow = p.epi.shortcut + off0;
                    if (npix == 16) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            sc[j] = int32_t(__ldg(scRow + (uint32_t(j) * ld + uint32_t(oc))));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            sc[j] = j < npix ? int32_t(__ldg(scRow + (uint32_t(j) * ld + uint32_t(oc)))) : 0;
                        }
                    }
                }
                int32_t r[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    r[j] = fastRescale(fm, int32_t(acc[j] + uint32_t(corr0)), outZpMain, loMain, hiMain);
                }
                if (RESIDUAL) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int32_t ta = lutA[r[j] + 128];
                        const int32_t tb = lutB[sc[j] + 128];
                        r[j] = fastRescale(fo, int32_t(uint32_t(ta) + uint32_t(tb)), p.epi.out.outZp, p.epi.out.lo,
                                           p.epi.out.hi);
                    }
                }
                if (npix == 16) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        dstRow[uint32_t(j) * ld + uint32_t(oc)] = int8_t(r[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (j < npix) {
                            dstRow[uint32_t(j) * ld + uint32_t(oc)] = int8_t(r[j]);
                        }
                    }
                }
            }
            __syncwarp(); // channels past the end skipped the block: converge before the next aligned TMEM load
        }
    }
}

// X_TMA: the pixel operand comes through tmapX; otherwise it is gathered from the NHWC input described by p.
template <int BNP, int NSTAGE, bool X_TMA>
__global__ void __launch_bounds__(X_TMA ? kThreadsTma : kThreadsGather, 1)
gemmI8OcMajor(const __grid_constant__ CUtensorMap tmapX, const __grid_constant__ CUtensorMap tmapW, const GemmI8Params p) {
    extern __shared__ uint8_t rawSmem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    constexpr int kTileW = kOcTile * BK;
    constexpr int kTileX = BNP * BK;
    uint8_t *tilesW = smem;
    uint8_t *tilesX = smem + NSTAGE * kTileW;
    int32_t *lutA = reinterpret_cast<int32_t *>(smem + NSTAGE * (kTileW + kTileX));
    int32_t *lutB = lutA + 256;
    uint8_t *clsTab = reinterpret_cast<uint8_t *>(lutB + 256);
    int32_t *tapTab = reinterpret_cast<int32_t *>(clsTab + 2 * BNP);
    OcBarriers *bars = reinterpret_cast<OcBarriers *>(tapTab + kTapTabEntries);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int numKb = (p.K + BK - 1) / BK;
    const int pTiles = (p.M + BNP - 1) / BNP;
    const int cTiles = (p.N + kOcTile - 1) / kOcTile;
    const int64_t numTiles = int64_t(pTiles) * cTiles * p.batches;
    const auto tileOf = [&](int64_t t) {
        OcTile c;
        c.c0 = int(t % cTiles) * kOcTile;
        t /= cTiles;
        c.m0 = int(t % pTiles) * BNP;
        c.batch = int(t / pTiles);
        return c;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbarInit(&bars->full[s], X_TMA ? 1u : 1u + 128u);
            mbarInit(&bars->empty[s], 1u);
        }
        for (int b = 0; b < 2; ++b) {
            mbarInit(&bars->accFull[b], 1u);
            mbarInit(&bars->accEmpty[b], uint32_t(kEpilogueWarps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&bars->tmemBase)),
                     "r"(uint32_t(2 * BNP))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    const bool fastGather = !X_TMA && fastGatherApplies(p);
    if (fastGather && warp >= kGatherWarp0) {
        fillTapTable(p, tapTab, kGatherWarp0 * 32, 128);
    }
    if (p.epi.hasResidual && threadIdx.x < 256) {
        // the two int8 -> int32 RESCALEs of the residual tail, tabulated over their whole domain
        const int32_t v = int32_t(threadIdx.x) - 128;
        const FastRescale fa =
            makeFastRescale(__ldg(p.epi.a.mult), int32_t(__ldg(p.epi.a.shift)), p.epi.a.inZp, p.epi.a.doubleRound != 0);
        const FastRescale fb =
            makeFastRescale(__ldg(p.epi.b.mult), int32_t(__ldg(p.epi.b.shift)), p.epi.b.inZp, p.epi.b.doubleRound != 0);
        lutA[threadIdx.x] = fastRescale(fa, v, p.epi.a.outZp, p.epi.a.lo, p.epi.a.hi);
        lutB[threadIdx.x] = fastRescale(fb, v, p.epi.b.outZp, p.epi.b.lo, p.epi.b.hi);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmemBase = bars->tmemBase;

    if (warp == kTmaWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                const OcTile tc = tileOf(t);
                for (int kb = 0; kb < numKb; ++kb, ++it) {
                    const int s = int(it % NSTAGE);
                    const uint32_t phase = (it / NSTAGE) & 1u;
                    ok = mbarWait(&bars->empty[s], phase ^ 1u, 11);
                    if (!ok) {
                        break;
                    }
                    mbarArriveExpectTx(&bars->full[s], uint32_t(kTileW + (X_TMA ? kTileX : 0)));
                    tmaLoad3d(&tmapW, tilesW + s * kTileW, &bars->full[s], kb * BK, tc.c0, 0);
                    if (X_TMA) {
                        // boxes hold at most 256 rows of 128 bytes: one copy per 128 pixels
#pragma unroll
                        for (int h = 0; h < BNP / 128; ++h) {
                            tmaLoad3d(&tmapX, tilesX + s * kTileX + h * 128 * BK, &bars->full[s], kb * BK, tc.m0 + h * 128,
                                      tc.batch);
                        }
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = instrDesc(BNP, false);
            uint32_t it = 0, tileCount = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x, ++tileCount) {
                const uint32_t buf = tileCount & 1u;
                ok = mbarWait(&bars->accEmpty[buf], ((tileCount >> 1) & 1u) ^ 1u, 15);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmemD = tmemBase + buf * uint32_t(BNP);
                for (int kb = 0; kb < numKb; ++kb, ++it) {
                    const int s = int(it % NSTAGE);
                    const uint32_t phase = (it / NSTAGE) & 1u;
                    ok = mbarWait(&bars->full[s], phase, 12);
                    if (!ok) {
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t wAddr = smemAddr(tilesW + s * kTileW);
                    const uint32_t xAddr = smemAddr(tilesX + s * kTileX);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        umma(tmemD, smemDesc(wAddr + k * UMMA_K, 16, 1024), smemDesc(xAddr + k * UMMA_K, 16, 1024), idesc,
                             (kb | k) != 0 ? 1u : 0u);
                    }
                    ummaCommit(&bars->empty[s]);
                }
                if (ok) {
                    ummaCommit(&bars->accFull[buf]);
                }
            }
        }
    } else if (warp >= kGatherWarp0) {
        // ---------------- pixel gather (implicit GEMM): BNP / 128 tile rows per thread ----------------
        if (!X_TMA) {
            constexpr int kRows = BNP / 128;
            const int row0 = (warp - kGatherWarp0) * 32 + lane;
            const uint32_t swz = uint32_t(row0 & 7); // rows 128 apart share the swizzle phase
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
                const OcTile tc = tileOf(t);
                if (fastGather) {
                    GatherRow rows[kRows];
#pragma unroll
                    for (int r = 0; r < kRows; ++r) {
                        rows[r] = gatherRowSetup(p, int64_t(tc.m0) + row0 + r * 128);
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
                        gatherBlock<kRows>(rows, tapTab, p.KH * p.KW, p.IC, tap, c0, dstRow, swz, p.in);
                        asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(smemAddr(&bars->full[s]))
                                     : "memory");
                        mbarArrive(&bars->full[s]);
                    }
                    continue;
                }
                int iy0[kRows], ix0[kRows];
                const int8_t *base[kRows];
                bool rowValid[kRows];
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    const int64_t m = int64_t(tc.m0) + row0 + r * 128;
                    rowValid[r] = m < p.M;
                    int n = 0, oy = 0, ox = 0;
                    if (rowValid[r]) {
                        n = int(m / (int64_t(p.OH) * p.OW));
                        const int rem = int(m - int64_t(n) * p.OH * p.OW);
                        oy = rem / p.OW;
                        ox = rem - oy * p.OW;
                    }
                    iy0[r] = oy * p.strideY - p.padTop;
                    ix0[r] = ox * p.strideX - p.padLeft;
                    base[r] = p.in + int64_t(n) * p.H * p.W * p.IC;
                }
                int c = 0, kx = 0, ky = 0;
                for (int kb = 0; kb < numKb; ++kb, ++it) {
                    const int s = int(it % NSTAGE);
                    const uint32_t phase = (it / NSTAGE) & 1u;
                    ok = mbarWait(&bars->empty[s], phase ^ 1u, 13);
                    if (!ok) {
                        break;
                    }
                    const uint32_t dstRow = smemAddr(tilesX + s * kTileX) + uint32_t(row0) * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int dy = ky * p.dilY, dx = kx * p.dilX;
#pragma unroll
                        for (int r = 0; r < kRows; ++r) {
                            const int y = iy0[r] + dy;
                            const int x = ix0[r] + dx;
                            const bool valid = rowValid[r] && ky < p.KH && y >= 0 && y < p.H && x >= 0 && x < p.W;
                            const int8_t *src = valid ? base[r] + (int64_t(y) * p.W + x) * p.IC + c : p.in;
                            const uint32_t dst = dstRow + uint32_t(r) * (128u * 128u) + ((uint32_t(j) ^ swz) << 4);
                            const uint32_t bytes = valid ? 16u : 0u;
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                                         : "memory");
                        }
                        c += 16;
                        if (c >= p.IC) {
                            c = 0;
                            if (++kx == p.KW) {
                                kx = 0;
                                ++ky;
                            }
                        }
                    }
                    asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(smemAddr(&bars->full[s]))
                                 : "memory");
                    mbarArrive(&bars->full[s]);
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        if (p.epi.hasResidual) {
            epilogueOcMajor<BNP, true>(p, bars, clsTab, lutA, lutB, tmemBase, warp, lane, numTiles, pTiles, cTiles);
        } else {
            epilogueOcMajor<BNP, false>(p, bars, clsTab, lutA, lutB, tmemBase, warp, lane, numTiles, pTiles, cTiles);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(uint32_t(2 * BNP))
                     : "memory");
    }
}

template <int BNP, int NSTAGE, bool X_TMA>
int launchOcMajor(const CUtensorMap &mapX, const CUtensorMap &mapW, const GemmI8Params &p, cudaStream_t s) {
    constexpr size_t smemBytes =
        size_t(NSTAGE) * (kOcTile * BK + BNP * BK) + 2 * 256 * sizeof(int32_t) + 2 * BNP +
        kTapTabEntries * sizeof(int32_t) + sizeof(OcBarriers) + 1024;
    auto kernel = gemmI8OcMajor<BNP, NSTAGE, X_TMA>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smemBytes)) != cudaSuccess) {
            setLastError("cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
            return MLEL_ERROR_DEVICE;
        }
        configured = true;
    }
    const int64_t tiles = int64_t((p.M + BNP - 1) / BNP) * ((p.N + kOcTile - 1) / kOcTile) * p.batches;
    const int grid = int(tiles < smCount() ? tiles : smCount());
    kernel<<<grid, X_TMA ? kThreadsTma : kThreadsGather, smemBytes, s>>>(mapX, mapW, p);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        setLastError(std::string("tcgen05 channel-major convolution launch: ") + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

} // namespace

bool gemmI8OcMajorApplies(const GemmI8Problem &q) {
    const GemmI8Params &p = q.params;
    if (p.out8 == nullptr || !p.epi.hasMain || q.bMnMajor || p.batchedB || p.N <= 64 || p.ldOut >= (1 << 27)) {
        return false;
    }
    // the residual tables are indexed by the int8 value of the main stage
    return !p.epi.hasResidual || (p.epi.main.lo >= -128 && p.epi.main.hi <= 127);
}

int gemmI8OcMajorLaunch(const GemmI8Problem &q, cudaStream_t s) {
    GemmI8Params p = q.params;
    p.batches = q.batches;
    // 256-pixel tiles halve the operand traffic per multiply-accumulate; 128-pixel tiles fill the last wave
    // better on small layers.  Pick by the number of waves times the work of one tile.
    const int64_t cTiles = (p.N + kOcTile - 1) / kOcTile;
    const int64_t t256 = int64_t((p.M + 255) / 256) * cTiles * q.batches;
    const int64_t t128 = int64_t((p.M + 127) / 128) * cTiles * q.batches;
    const int64_t sms = smCount();
    const bool wide = ((t256 + sms - 1) / sms) * 2 <= (t128 + sms - 1) / sms;
    CUtensorMap mapX{}, mapW{};
    const bool xTma = q.aMatrix != nullptr;
    if (xTma && !makeMap(&mapX, q.aMatrix, uint64_t(p.K), uint64_t(p.M), uint64_t(q.batches), uint64_t(q.aRowBytes),
                         uint64_t(q.aBatchBytes), BK, 128)) {
        return MLEL_ERROR_DEVICE;
    }
    if (!makeMap(&mapW, q.bMatrix, uint64_t(p.K), uint64_t(p.N), 1, uint64_t(q.bRowBytes),
                 uint64_t(q.bRowBytes) * uint64_t(p.N), BK, kOcTile)) {
        return MLEL_ERROR_DEVICE;
    }
    if (wide) {
        return xTma ? launchOcMajor<256, 4, true>(mapX, mapW, p, s) : launchOcMajor<256, 4, false>(mapX, mapW, p, s);
    }
    return xTma ? launchOcMajor<128, 6, true>(mapX, mapW, p, s) : launchOcMajor<128, 6, false>(mapX, mapW, p, s);
}

int ocMajorErrorWord() { return tc::readErrorWord(); }

} // namespace mlel
