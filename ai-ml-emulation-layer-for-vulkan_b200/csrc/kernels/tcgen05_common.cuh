// Shared device and host helpers of the tcgen05 int8 kernels (PTX wrappers for mbarrier, TMA, tcgen05 and
// the tensor-map encoder).  Included by gemm_i8_tcgen05.cu and gemm_i8_ocmajor.cu.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "device_common.cuh"

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
// Bounded wait: returns false (and records `code`) when the barrier did not complete in time.  Between
// polls the waiter sleeps `sleepNs` so that a waiting role does not take issue slots from the warps that
// share its scheduler (the epilogue warps do the arithmetic).
__device__ __forceinline__ bool mbarWait(uint64_t *bar, uint32_t parity, int code, unsigned sleepNs = 32) {
    if (mbarTryWait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    while (!mbarTryWait(bar, parity)) {
        __nanosleep(sleepNs);
        if (clock64() - start > kWaitLimitCycles) {
            atomicCAS(&g_tcgen05Error, 0, code);
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void tmaLoad3d(const CUtensorMap *map, void *dst, uint64_t *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smemAddr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smemAddr(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
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
__device__ __forceinline__ void tmemLoad16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}

// Barrier among the epilogue warps only (named barrier 1).
__device__ __forceinline__ void epilogueSync() {
    asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
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
             uint64_t stride2, uint32_t b0, uint32_t b1) {
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
                           elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        setLastError("cuTensorMapEncodeTiled failed with code " + std::to_string(int(rc)));
        return false;
    }
    return true;
}

inline int smCount() {
    static int count = 0;
    if (count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) {
            count = kNumSMs;
        }
    }
    return count;
}


} // namespace tc
} // namespace mlel
