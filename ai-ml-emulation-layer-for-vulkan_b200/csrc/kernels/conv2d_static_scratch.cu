// mlel_cuda_conv2d_static_scratch: int8 CONV2D -> int32 for callers that are not allowed to allocate.
//
// Who needs this.  The other tensor-core convolution paths of this library take their working memory
// from somewhere that was allocated for them: a session's transient memory (sized by the memory planner
// and handed over by the application) or the pipeline's constant slab (cudaMalloc at first use).  Some
// hosts of this code cannot do either at the point where they need a convolution: a Vulkan layer's
// dispatch hook runs while the application is recording or replaying work and must not touch the CUDA
// allocator (allocation synchronises the device and can fail after the application has already been told
// the pipeline is valid); code running under a fixed device-memory budget owned by another runtime has
// no allocator it may call at all.  For them this entry point brings its own working memory: a fixed
// array in the library image, present on every GPU that loads the library from load until exit.
//
// What it computes.  Exactly mlel_cuda_conv2d (the reference's conv2d.comp:26-116 for int8 input, int8
// OHWI weights with zero point 0, int32 bias and int32 output), for any channel count, on the tensor
// cores.  Three kernels run back to back on the caller's stream, all working memory inside g_scratch:
//   1. pad the weight rows to a multiple of 16 bytes and form corr[oc] = bias[oc] - zp_in * sum(w[oc]),
//   2. write the im2col matrix [pixels][kPad]; taps outside the image are filled with the input zero
//      point (not zero), so that one correction per channel is exact for every pixel,
//   3. the tcgen05 matrix product of gemm_i8_tcgen05.cu with the int32 epilogue.
//
// Limits and sharing.  kScratchBytes (32 MiB) bounds  pixels * kPad + OC * kPad + 4 * OC; larger
// problems are rejected with MLEL_ERROR_UNKNOWN and a message, never truncated.  All calls on a device
// share the one array and it keeps the last call's contents.  Every call rewrites each byte it later
// reads (nothing has to start at zero), so calls that run one after another are independent; calls whose
// GPU work overlaps (different streams, or host threads racing on one stream's order) race on the array
// and must be serialised by the caller.  The first call on a device looks up the array's device address;
// make that first call outside any stream capture.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <exception>
#include <string>

#include "device_common.cuh"
#include "gemm_i8_tcgen05.hpp"

namespace mlel {

namespace {

constexpr size_t kScratchBytes = size_t(32) << 20;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; kernels receive the looked-up pointer.
static __device__ __align__(256) uint8_t g_scratch[kScratchBytes];

std::mutex g_setupMutex;
uint8_t *g_scratchAddress[kMaxDevices] = {};

// Device address of g_scratch on the current device (looked up once per device).
int scratchBase(uint8_t **base) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        setLastError("conv2d_static_scratch: no usable current CUDA device");
        return MLEL_ERROR_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_setupMutex);
    if (g_scratchAddress[device] == nullptr) {
        void *ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            setLastError(std::string("conv2d_static_scratch: cudaGetSymbolAddress failed: ") + cudaGetErrorString(err));
            return MLEL_ERROR_DEVICE;
        }
        g_scratchAddress[device] = static_cast<uint8_t *>(ptr);
    }
    *base = g_scratchAddress[device];
    return MLEL_SUCCESS;
}

// One block per output channel: copy the weight row into its zero-padded slot and reduce its sum.
__global__ void padWeightsAndCorrect(const int8_t *__restrict__ w, const int32_t *__restrict__ bias, int biasCount,
                                     int8_t *__restrict__ wPad, int32_t *__restrict__ corr, int K, int kPad, int zpIn) {
    const int oc = blockIdx.x;
    int sum = 0;
    for (int k = threadIdx.x; k < kPad; k += blockDim.x) {
        const int8_t v = k < K ? w[int64_t(oc) * K + k] : int8_t(0);
        wPad[int64_t(oc) * kPad + k] = v;
        sum += v;
    }
    __shared__ int partial[32];
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_down_sync(0xffffffffu, sum, off);
    }
    if ((threadIdx.x & 31) == 0) {
        partial[threadIdx.x >> 5] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int i = 0; i < int(blockDim.x >> 5); ++i) {
            total += partial[i];
        }
        const uint32_t b = uint32_t(bias[biasCount == 1 ? 0 : oc]);
        corr[oc] = int32_t(b - uint32_t(zpIn) * uint32_t(total)); // modulo 2^32, like the reference's accumulator
    }
}

// im2col with the input zero point in place of out-of-image taps.  One warp per pixel at a time; lane l
// writes the 32-bit words l, l+32, ... of the row (coalesced), bytes past K are zero.
__global__ void im2colZeroPointFill(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t M, int H, int W,
                                    int IC, int OH, int OW, int KW, int strideY, int strideX, int padTop, int padLeft,
                                    int dilY, int dilX, int K, int kPad, int zpIn) {
    const int lane = threadIdx.x & 31;
    const int64_t warpId = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t numWarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const int words = kPad >> 2;
    const uint32_t fill = uint32_t(uint8_t(int8_t(zpIn)));
    for (int w0 = 0; w0 < words; w0 += 32) {
        const int w = w0 + lane;
        int dy[4], dx[4], ci[4];
        bool inK[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int k = 4 * w + b;
            inK[b] = w < words && k < K;
            const int tap = inK[b] ? k / IC : 0;
            ci[b] = inK[b] ? k - tap * IC : 0;
            const int ky = tap / KW;
            dy[b] = ky * dilY;
            dx[b] = (tap - ky * KW) * dilX;
        }
        for (int64_t m = warpId; m < M; m += numWarps) {
            const int n = int(m / (int64_t(OH) * OW));
            const int rem = int(m - int64_t(n) * OH * OW);
            const int oy = rem / OW, ox = rem - oy * OW;
            const int iy0 = oy * strideY - padTop, ix0 = ox * strideX - padLeft;
            const int8_t *base = in + int64_t(n) * H * W * IC;
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (inK[b]) {
                    const int y = iy0 + dy[b], x = ix0 + dx[b];
                    const bool inside = y >= 0 && y < H && x >= 0 && x < W;
                    const uint32_t v = inside ? uint32_t(uint8_t(base[(int64_t(y) * W + x) * IC + ci[b]])) : fill;
                    word |= v << (8 * b);
                }
            }
            if (w < words) {
                reinterpret_cast<uint32_t *>(out + m * kPad)[w] = word;
            }
        }
    }
}

bool packedDesc(const mlel_tensor_desc &d) {
    if (d.strides[0] == 0) {
        return true;
    }
    int64_t s = dtypeSize(d.dtype);
    for (int i = d.rank - 1; i >= 0; --i) {
        if (d.strides[i] != s) {
            return false;
        }
        s *= d.dims[i];
    }
    return true;
}

int fail(const std::string &msg) {
    setLastError("conv2d_static_scratch: " + msg);
    return MLEL_ERROR_UNKNOWN;
}

} // namespace

} // namespace mlel

namespace mlel {
namespace {
int conv2dStaticScratch(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                        const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2],
                        int32_t input_zp, int32_t weight_zp, void *cuda_stream);
} // namespace
} // namespace mlel

using namespace mlel;

extern "C" int mlel_cuda_conv2d_static_scratch(const mlel_tensor *input, const mlel_tensor *weights,
                                               const mlel_tensor *biases, const mlel_tensor *output,
                                               const int32_t pad[4], const int32_t stride[2],
                                               const int32_t dilation[2], int32_t input_zp, int32_t weight_zp,
                                               void *cuda_stream) {
    // no exception may cross the C boundary (the messages below build strings)
    try {
        return conv2dStaticScratch(input, weights, biases, output, pad, stride, dilation, input_zp, weight_zp, cuda_stream);
    } catch (const std::exception &e) {
        try {
            setLastError(std::string("conv2d_static_scratch: ") + e.what());
        } catch (...) {
        }
        return MLEL_ERROR_UNKNOWN;
    } catch (...) {
        return MLEL_ERROR_UNKNOWN;
    }
}

namespace mlel {
namespace {

int conv2dStaticScratch(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                        const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2],
                        int32_t input_zp, int32_t weight_zp, void *cuda_stream) {
    if (input == nullptr || weights == nullptr || biases == nullptr || output == nullptr || pad == nullptr ||
        stride == nullptr || dilation == nullptr) {
        return fail("null argument");
    }
    const mlel_tensor_desc &di = input->desc, &dw = weights->desc, &db = biases->desc, &dout = output->desc;
    if (di.dtype != MLEL_I8 || dw.dtype != MLEL_I8 || db.dtype != MLEL_I32 || dout.dtype != MLEL_I32 || di.rank != 4 ||
        dw.rank != 4 || db.rank != 1 || dout.rank != 4) {
        return fail("needs int8 NHWC input, int8 OHWI weights, int32 bias and int32 NHWC output");
    }
    if (!packedDesc(di) || !packedDesc(dw) || !packedDesc(db) || !packedDesc(dout)) {
        return fail("tensors must be packed");
    }
    if (weight_zp != 0) {
        return fail("a weight zero point other than 0 is not supported");
    }
    if (input_zp < -128 || input_zp > 127) {
        // the working copy of the input is int8 and its padding is filled with the zero point
        return fail("the input zero point must be in the int8 range");
    }
    const int64_t N = di.dims[0], H = di.dims[1], W = di.dims[2], IC = di.dims[3];
    const int64_t OC = dw.dims[0], KH = dw.dims[1], KW = dw.dims[2];
    const int64_t OH = dout.dims[1], OW = dout.dims[2];
    if (dw.dims[3] != IC || dout.dims[0] != N || dout.dims[3] != OC || (db.dims[0] != OC && db.dims[0] != 1)) {
        return fail("operand shapes do not agree");
    }
    if (stride[0] <= 0 || stride[1] <= 0 || dilation[0] <= 0 || dilation[1] <= 0 || OC % 16 != 0) {
        return fail("strides and dilations must be positive and the output channel count a multiple of 16");
    }
    const auto outDim = [](int64_t in, int64_t before, int64_t after, int64_t k, int64_t dil, int64_t st) {
        return (in + before + after - (k - 1) * dil - 1) / st + 1;
    };
    if (pad[0] < 0 || pad[1] < 0 || pad[2] < 0 || pad[3] < 0 || KH <= 0 || KW <= 0 ||
        OH != outDim(H, pad[0], pad[1], KH, dilation[0], stride[0]) ||
        OW != outDim(W, pad[2], pad[3], KW, dilation[1], stride[1])) {
        return fail("the output size does not follow from input size, padding, window, dilation and stride");
    }
    const int64_t K = KH * KW * IC, kPad = (K + 15) / 16 * 16, M = N * OH * OW;
    if (K > 65536 || M <= 0 || M >= (int64_t(1) << 31)) {
        return fail("contraction length above 65536 or pixel count out of range");
    }
    // scratch layout: [im2col M x kPad][weights OC x kPad][corr OC x int32], each part 256-byte aligned
    const auto align256 = [](uint64_t v) { return (v + 255) / 256 * 256; };
    const uint64_t offW = align256(uint64_t(M) * uint64_t(kPad));
    const uint64_t offCorr = offW + align256(uint64_t(OC) * uint64_t(kPad));
    const uint64_t need = offCorr + align256(uint64_t(OC) * 4);
    if (need > kScratchBytes) {
        return fail("problem needs " + std::to_string(need) + " bytes of working memory, the built-in array holds " +
                    std::to_string(kScratchBytes));
    }
    uint8_t *base = nullptr;
    const int rc = scratchBase(&base);
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    int8_t *aPad = reinterpret_cast<int8_t *>(base);
    int8_t *wPad = reinterpret_cast<int8_t *>(base + offW);
    int32_t *corr = reinterpret_cast<int32_t *>(base + offCorr);

    padWeightsAndCorrect<<<unsigned(OC), 128, 0, s>>>(static_cast<const int8_t *>(weights->data),
                                                     static_cast<const int32_t *>(biases->data), int(db.dims[0]), wPad,
                                                     corr, int(K), int(kPad), int(int8_t(input_zp)));
    const int64_t warps = M < int64_t(kNumSMs) * 64 ? M : int64_t(kNumSMs) * 64;
    const int blocks = int((warps * 32 + kThreads - 1) / kThreads);
    im2colZeroPointFill<<<blocks < 1 ? 1 : blocks, kThreads, 0, s>>>(
        static_cast<const int8_t *>(input->data), aPad, M, int(H), int(W), int(IC), int(OH), int(OW), int(KW), stride[0],
        stride[1], pad[0], pad[2], dilation[0], dilation[1], int(K), int(kPad), int(int8_t(input_zp)));
    if (cudaGetLastError() != cudaSuccess) {
        setLastError("conv2d_static_scratch: kernel launch failed");
        return MLEL_ERROR_DEVICE;
    }

    GemmI8Problem q{};
    GemmI8Params &p = q.params;
    p.M = int32_t(M), p.N = int32_t(OC), p.K = int32_t(kPad), p.ldOut = int32_t(OC);
    p.corr = corr;
    p.numClasses = 1, p.numColClasses = 1;
    p.out32 = static_cast<int32_t *>(output->data);
    q.batches = 1;
    q.aMatrix = aPad, q.aRowBytes = uint64_t(kPad), q.aBatchBytes = uint64_t(kPad) * uint64_t(M);
    q.bMatrix = wPad, q.bRowBytes = uint64_t(kPad), q.bBatchBytes = 0;
    q.bMnMajor = false;
    return gemmI8Launch(q, s);
}

} // namespace
} // namespace mlel
