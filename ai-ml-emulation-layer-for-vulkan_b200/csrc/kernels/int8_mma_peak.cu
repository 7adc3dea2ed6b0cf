// Measures what the int8 tensor pipe of the current GPU sustains: every SM issues tcgen05.mma kind::i8
// (M = 128, N = 256, K = 32) back to back on operands that stay in shared memory, with nothing else to do.
// The figure is the denominator of the tensor-bound roofline fractions that bench.py reports: the machine's
// own measured-peaks file holds a copy bandwidth and a bf16 matmul rate but no int8 rate.
//
// One CTA per SM, one issuing thread per CTA.  The two TMEM accumulators (2 x 256 columns) alternate between
// batches of 64 instructions; a batch is committed to an mbarrier, and the thread waits for the batch before
// the last one, so the pipe always has one full batch queued behind the one that is running.  Every wait is
// bounded (see mbarWait) and the kernel frees its TMEM on every path.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "gemm_i8_tcgen05.hpp"
#include "tcgen05_common.cuh"

namespace mlel {

namespace {
using namespace tc;

constexpr int kPeakN = 256;          // columns of one accumulator
constexpr int kPeakBatch = 64;       // instructions between two commits
constexpr int kPeakTileA = BM * BK;  // 128 rows x 128 bytes
constexpr int kPeakTileB = kPeakN * BK;

struct __align__(8) PeakBarriers {
    uint64_t done[2];
    uint32_t tmemBase;
    uint32_t pad;
};

__global__ void __launch_bounds__(128, 1) int8MmaPeakKernel(int batches) {
    extern __shared__ uint8_t rawSmem[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~uintptr_t(1023));
    uint8_t *tileA = smem;
    uint8_t *tileB = smem + kPeakTileA;
    PeakBarriers *bars = reinterpret_cast<PeakBarriers *>(tileB + kPeakTileB);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // operand bytes: any values do (the rate does not depend on them); not all zero, so that the multipliers toggle
    for (int i = threadIdx.x; i < (kPeakTileA + kPeakTileB) / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t *>(smem)[i] = 0x9E3779B9u * uint32_t(i + 1 + blockIdx.x);
    }
    if (threadIdx.x == 0) {
        mbarInit(&bars->done[0], 1u);
        mbarInit(&bars->done[1], 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&bars->tmemBase)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the generic-proxy writes above must be visible to the tensor core's reads of shared memory
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmemBase = bars->tmemBase;

    if (warp == 0 && lane == 0) {
        constexpr uint32_t idesc = instrDesc(kPeakN, false);
        const uint32_t aAddr = smemAddr(tileA), bAddr = smemAddr(tileB);
        bool ok = true;
        for (int b = 0; b < batches && ok; ++b) {
            const uint32_t buf = uint32_t(b) & 1u;
            if (b >= 2) {
                // the batch that last used this accumulator (and this barrier) has left the pipe
                ok = mbarWait(&bars->done[buf], (uint32_t(b - 2) >> 1) & 1u, 21);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            const uint32_t tmemD = tmemBase + buf * uint32_t(kPeakN);
#pragma unroll 4
            for (int i = 0; i < kPeakBatch; ++i) {
                const int k = i & 3;
                umma(tmemD, smemDesc(aAddr + k * UMMA_K, 16, 1024), smemDesc(bAddr + k * UMMA_K, 16, 1024), idesc,
                     i != 0 ? 1u : 0u);
            }
            ummaCommit(&bars->done[buf]);
        }
        // drain: the last two batches
        for (int b = (batches > 2 ? batches - 2 : 0); b < batches && ok; ++b) {
            ok = mbarWait(&bars->done[uint32_t(b) & 1u], (uint32_t(b) >> 1) & 1u, 22);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(512u) : "memory");
    }
}

} // namespace

// Runs the loop for `batches` batches of 64 instructions per SM on `stream` and reports the device time and the
// number of int8 operations (2 per multiply-accumulate) it stands for.
int int8MmaPeak(int batches, cudaStream_t stream, float *msOut, double *opsOut) {
    if (batches < 1 || batches > (1 << 24)) {
        setLastError("int8 MMA peak loop: batches out of range");
        return MLEL_ERROR_UNKNOWN;
    }
    constexpr size_t smemBytes = size_t(kPeakTileA + kPeakTileB) + sizeof(PeakBarriers) + 1024;
    if (!allowDynamicSmem(reinterpret_cast<const void *>(int8MmaPeakKernel), smemBytes)) {
        return MLEL_ERROR_DEVICE;
    }
    const int grid = smCount();
    cudaEvent_t start = nullptr, stop = nullptr;
    if (cudaEventCreate(&start) != cudaSuccess || cudaEventCreate(&stop) != cudaSuccess) {
        setLastError("cudaEventCreate failed");
        return MLEL_ERROR_DEVICE;
    }
    cudaEventRecord(start, stream);
    int8MmaPeakKernel<<<grid, 128, smemBytes, stream>>>(batches);
    cudaEventRecord(stop, stream);
    const cudaError_t err = cudaEventSynchronize(stop);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, start, stop);
    cudaEventDestroy(start);
    cudaEventDestroy(stop);
    if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) {
        setLastError(std::string("int8 MMA peak loop: ") + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    if (tc::readErrorWord() != 0) {
        setLastError("int8 MMA peak loop: a bounded wait ran out");
        return MLEL_ERROR_DEVICE;
    }
    *msOut = ms;
    *opsOut = double(grid) * double(batches) * double(kPeakBatch) * 2.0 * double(BM) * double(kPeakN) * double(UMMA_K);
    return MLEL_SUCCESS;
}

} // namespace mlel
