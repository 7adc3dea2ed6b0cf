// Vectorised kernels for the packed int8 NHWC shapes that dominate real graphs.  Each has a generic
// counterpart in generic_ops.cu that defines the result; these only change how the bytes move.
#include "device_common.cuh"
#include "kernels.hpp"

namespace mlel {

namespace {

// ---- im2col for convolutions whose channel count is not a multiple of 16 (e.g. an RGB stem) ---------
// Writes A'[m][k], m = output pixel, k = (ky, kx, ic) flattened and zero-padded to kPad (a multiple of
// 16), out-of-range taps as zeros (the tensor-core kernel's border-class correction assumes exactly
// that).  One warp owns one pixel at a time: lane l produces the 32-bit words l, l+32, ... of the row,
// so a row is written with coalesced 128-byte stores while the byte gathers hit L1.
__global__ void im2colSmallIcKernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t M, int H, int W,
                                    int IC, int OH, int OW, int KH, int KW, int strideY, int strideX, int padTop,
                                    int padLeft, int dilY, int dilX, int K, int kPad) {
    const int lane = threadIdx.x & 31;
    const int64_t warpId = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t numWarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const int words = kPad >> 2;
    for (int w0 = 0; w0 < words; w0 += 32) {
        const int w = w0 + lane;
        // tap decomposition of this lane's four bytes: fixed for every pixel
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
                const int y = iy0 + dy[b], x = ix0 + dx[b];
                if (inK[b] && y >= 0 && y < H && x >= 0 && x < W) {
                    word |= uint32_t(uint8_t(__ldg(base + (int64_t(y) * W + x) * IC + ci[b]))) << (8 * b);
                }
            }
            if (w < words) {
                reinterpret_cast<uint32_t *>(out + m * kPad)[w] = word;
            }
        }
    }
}

// ---- MAX_POOL2D, int8 NHWC, C % 16 == 0 (maxpool2d.comp:23-72) --------------------------------------
// One thread per (pixel, 16-channel group): 16-byte loads, per-byte signed max, one 16-byte store.
__global__ void maxPoolI8Kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t total, int H, int W,
                                int C, int OH, int OW, PoolAttr a) {
    const int groups = C >> 4;
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += int64_t(gridDim.x) * blockDim.x) {
        const int g = int(e % groups);
        int64_t pix = e / groups;
        const int ox = int(pix % OW);
        pix /= OW;
        const int oy = int(pix % OH);
        const int n = int(pix / OH);
        const int iy0 = oy * max(a.stride[0], 1) - a.pad[0], ix0 = ox * max(a.stride[1], 1) - a.pad[2];
        uint32_t acc[4] = {0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u}; // int8 lowest
        for (int ky = 0; ky < a.kernel[0]; ++ky) {
            const int y = iy0 + ky;
            if (y < 0 || y >= H) {
                continue;
            }
            for (int kx = 0; kx < a.kernel[1]; ++kx) {
                const int x = ix0 + kx;
                if (x < 0 || x >= W) {
                    continue;
                }
                const int4 v = __ldg(reinterpret_cast<const int4 *>(in + ((int64_t(n) * H + y) * W + x) * C) + g);
                acc[0] = __vmaxs4(acc[0], uint32_t(v.x));
                acc[1] = __vmaxs4(acc[1], uint32_t(v.y));
                acc[2] = __vmaxs4(acc[2], uint32_t(v.z));
                acc[3] = __vmaxs4(acc[3], uint32_t(v.w));
            }
        }
        reinterpret_cast<int4 *>(out + ((int64_t(n) * OH + oy) * OW + ox) * C)[g] =
            make_int4(int(acc[0]), int(acc[1]), int(acc[2]), int(acc[3]));
    }
}

int finish(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        setLastError(std::string(what) + ": " + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

} // namespace

int im2colSmallIc(const int8_t *in, int8_t *out, int64_t M, int H, int W, int IC, int OH, int OW, int KH, int KW,
                  const ConvAttr &a, int K, int kPad, cudaStream_t s) {
    const int64_t warps = M < int64_t(kNumSMs) * 64 ? M : int64_t(kNumSMs) * 64;
    const int blocks = int((warps * 32 + kThreads - 1) / kThreads);
    im2colSmallIcKernel<<<blocks < 1 ? 1 : blocks, kThreads, 0, s>>>(in, out, M, H, W, IC, OH, OW, KH, KW, a.stride[0],
                                                                      a.stride[1], a.pad[0], a.pad[2], a.dilation[0],
                                                                      a.dilation[1], K, kPad);
    return finish("im2col");
}

bool maxPoolI8Eligible(const TView &in, const TView &out) {
    const auto packed = [](const TView &t) {
        int64_t s = 1;
        for (int i = t.rank - 1; i >= 0; --i) {
            if (t.strides[i] != s) {
                return false;
            }
            s *= t.dims[i];
        }
        return true;
    };
    return in.dtype == MLEL_I8 && out.dtype == MLEL_I8 && in.rank == 4 && out.rank == 4 && in.dims[3] % 16 == 0 &&
           in.dims[3] == out.dims[3] && in.dims[0] == out.dims[0] && packed(in) && packed(out) &&
           ((reinterpret_cast<uintptr_t>(in.ptr) | reinterpret_cast<uintptr_t>(out.ptr)) & 15u) == 0;
}

int maxPoolI8(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s) {
    const int64_t total = int64_t(out.dims[0]) * out.dims[1] * out.dims[2] * (out.dims[3] >> 4);
    maxPoolI8Kernel<<<gridFor(total, kThreads, 16), kThreads, 0, s>>>(
        reinterpret_cast<const int8_t *>(in.ptr), reinterpret_cast<int8_t *>(out.ptr), total, int(in.dims[1]),
        int(in.dims[2]), int(in.dims[3]), int(out.dims[1]), int(out.dims[2]), a);
    return finish("MAX_POOL2D");
}

} // namespace mlel
