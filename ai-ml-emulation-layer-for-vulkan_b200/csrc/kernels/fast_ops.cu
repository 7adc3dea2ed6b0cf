// Vectorised kernels for the packed int8 NHWC shapes that dominate real graphs.  Each has a generic
// counterpart in generic_ops.cu that defines the result; these only change how the bytes move.
#include "device_common.cuh"
#include "kernels.hpp"

namespace mlel {

namespace {

// ---- padded copy for convolutions whose channel count is not a multiple of 16 (an RGB stem) ---------
// Copies an NHWC int8 tensor [N][H][W][C] into [N][Hp][Wp][Cp] (Cp >= C a multiple of 4) at row offset
// padTop and column offset padLeft; the new channels and the border are zero.  One thread per 32-bit word
// of the copy: byte reads hit L1, writes are coalesced.
__global__ void padImageKernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t words, int H, int W, int C,
                               int Hp, int Wp, int Cp, int padTop, int padLeft) {
    const int wordsPerPixel = Cp >> 2;
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < words; e += int64_t(gridDim.x) * blockDim.x) {
        int64_t pix = e / wordsPerPixel;
        const int c0 = int(e - pix * wordsPerPixel) * 4;
        const int x = int(pix % Wp) - padLeft;
        pix /= Wp;
        const int y = int(pix % Hp) - padTop;
        const int64_t n = pix / Hp;
        uint32_t word = 0;
        if (y >= 0 && y < H && x >= 0 && x < W) {
            const int8_t *src = in + ((n * H + y) * W + x) * C;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (c0 + b < C) {
                    word |= uint32_t(uint8_t(__ldg(src + c0 + b))) << (8 * b);
                }
            }
        }
        reinterpret_cast<uint32_t *>(out)[e] = word;
    }
}

// The same copy for Cp == 4 and an even Wp (the RGB stem): one block per row of the copy, two pixels (one 8-byte
// store) per thread, no divisions in the element loop.
__global__ void __launch_bounds__(128) padImageRows4Kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int H,
                                                          int W, int C, int Hp, int Wp, int padTop, int padLeft) {
    const int row = blockIdx.x; // n * Hp + yp
    const int n = row / Hp;
    const int y = row - n * Hp - padTop;
    const bool rowLive = y >= 0 && y < H;
    const int8_t *src = in + (int64_t(n) * H + (rowLive ? y : 0)) * W * C;
    uint2 *dst = reinterpret_cast<uint2 *>(out + int64_t(row) * Wp * 4);
    for (int q = threadIdx.x; 2 * q < Wp; q += blockDim.x) {
        uint32_t w[2] = {0u, 0u};
        if (rowLive) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int x = 2 * q + j - padLeft;
                if (x >= 0 && x < W) {
                    const int8_t *px = src + x * C;
                    for (int b = 0; b < C; ++b) {
                        w[j] |= uint32_t(uint8_t(__ldg(px + b))) << (8 * b);
                    }
                }
            }
        }
        dst[q] = make_uint2(w[0], w[1]);
    }
}

// ---- transpose of MATMUL's second input [N][C][W] -> [N][W][C] with column sums ---------------------------
// A block owns 64 columns (w) of one batch and walks the rows (c) in tiles of 64: 16-byte loads of the
// tile, byte transposition through shared memory, 16-byte stores; each thread keeps the running sum of the
// bytes it moved, and four neighbouring lanes combine them into the column sum at the end.
__global__ void __launch_bounds__(256) transposeColsumKernel(const int8_t *__restrict__ b, int8_t *__restrict__ bt,
                                                             int32_t *__restrict__ corr, int C, int W, int32_t za) {
    __shared__ int8_t tile[64][64 + 16]; // [c][w], rows padded to spread the banks of the column reads
    const int n = blockIdx.y;
    const int w0 = blockIdx.x * 64;
    const int t = threadIdx.x;
    const int8_t *src = b + int64_t(n) * C * W;
    int8_t *dst = bt + int64_t(n) * W * C;
    // load role: row (c) t / 4, 16-byte segment (w) t % 4; store role: column (w) t / 4, segment (c) t % 4
    const int lr = t >> 2, ls = (t & 3) * 16;
    int32_t sum = 0;
    for (int c0 = 0; c0 < C; c0 += 64) {
        int4 v = make_int4(0, 0, 0, 0);
        if (c0 + lr < C && w0 + ls < W) {
            v = __ldg(reinterpret_cast<const int4 *>(src + int64_t(c0 + lr) * W + w0 + ls));
        }
        *reinterpret_cast<int4 *>(&tile[lr][ls]) = v;
        __syncthreads();
        uint32_t words[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int8_t x = tile[ls + i][lr];
            sum += x;
            words[i >> 2] |= uint32_t(uint8_t(x)) << (8 * (i & 3));
        }
        if (w0 + lr < W && c0 + ls < C) {
            *reinterpret_cast<int4 *>(dst + int64_t(w0 + lr) * C + c0 + ls) =
                make_int4(int(words[0]), int(words[1]), int(words[2]), int(words[3]));
        }
        __syncthreads();
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((t & 3) == 0 && w0 + lr < W) {
        corr[int64_t(n) * W + w0 + lr] = int32_t(uint32_t(0) - uint32_t(za) * uint32_t(sum));
    }
}

// ---- column sums of MATMUL's second input [N][C][W]: corr[n][w] = -za * sum_c b[n][c][w] --------------------
// For the tensor-core path that reads the operand where it lies (no transposed copy).  A block owns 64 columns
// of one batch: 4 lanes hold 16 columns each (one 16-byte load per row), 64 slices share the rows, eight rows in
// flight per thread, and add their partial sums in shared memory.  Each byte goes through one dp4a against a
// one-hot selector, which sign-extends and accumulates it.
__global__ void __launch_bounds__(256) columnSumKernel(const int8_t *__restrict__ b, int32_t *__restrict__ corr, int C, int W,
                                                       int32_t za) {
    __shared__ int32_t part[64][64 + 1];
    const int n = blockIdx.y;
    const int w0 = blockIdx.x * 64;
    const int seg = threadIdx.x & 3, slice = threadIdx.x >> 2;
    const int w = w0 + seg * 16;
    const int8_t *src = b + int64_t(n) * C * W + w;
    int32_t acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc[i] = 0;
    }
    if (w < W) { // W is a multiple of 16: a 16-byte segment is inside or outside as a whole
        for (int c0 = slice; c0 < C; c0 += 8 * 64) {
            int4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int c = c0 + 64 * u;
                v[u] = c < C ? __ldg(reinterpret_cast<const int4 *>(src + int64_t(c) * W)) : make_int4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int words[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    acc[i] = __dp4a(words[i >> 2], 1 << (8 * (i & 3)), acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        part[slice][seg * 16 + i] = acc[i];
    }
    __syncthreads();
    if (threadIdx.x < 64 && w0 + threadIdx.x < W) {
        int32_t sum = 0;
#pragma unroll 8
        for (int sl = 0; sl < 64; ++sl) {
            sum += part[sl][threadIdx.x];
        }
        corr[int64_t(n) * W + w0 + threadIdx.x] = int32_t(uint32_t(0) - uint32_t(za) * uint32_t(sum));
    }
}

// ---- AVG_POOL2D, int8 NHWC, C % 4 == 0 (avgpool2d.comp:27-75) ---------------------------------------------
// A 256-thread block owns one output pixel and up to 128 channels: 32 lanes hold four channels each (one
// coalesced 128-byte read per tap), eight slices share the window's taps and add their partial sums in
// shared memory.  Built for the global pooling at the end of a classifier, where the generic kernel's one
// thread per output walks 49 dependent loads.
__global__ void __launch_bounds__(256) avgPoolI8Kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int H, int W,
                                                       int C, int OH, int OW, PoolAttr a) {
    __shared__ int32_t part[8][32][4];
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int chunks = (C + 127) / 128;
    int64_t b = blockIdx.x;
    const int c0 = int(b % chunks) * 128 + lane * 4;
    b /= chunks;
    const int ox = int(b % OW);
    b /= OW;
    const int oy = int(b % OH);
    const int n = int(b / OH);
    const int iy = oy * a.stride[0] - a.pad[0], ix = ox * a.stride[1] - a.pad[2];
    const int taps = a.kernel[0] * a.kernel[1];
    int32_t acc[4] = {0, 0, 0, 0};
    // in-range taps of the whole window: (rows inside) x (columns inside)
    const int ny = min(iy + a.kernel[0], H) - max(iy, 0), nx = min(ix + a.kernel[1], W) - max(ix, 0);
    const int count = (ny > 0 && nx > 0) ? ny * nx : 0;
    // eight taps of this slice at a time: all their loads are issued before the first sum
    const int8_t *image = in + int64_t(n) * H * W * C + c0;
    for (int t0 = slice; t0 < taps; t0 += 64) {
        uint32_t word[8];
        bool live[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int t = t0 + 8 * i;
            const int ky = t / a.kernel[1], kx = t - ky * a.kernel[1];
            const int y = iy + ky, x = ix + kx;
            live[i] = t < taps && y >= 0 && y < H && x >= 0 && x < W && c0 < C;
            word[i] = live[i] ? __ldg(reinterpret_cast<const uint32_t *>(image + (int64_t(y) * W + x) * C)) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (live[i]) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    acc[k] += int32_t(int8_t(word[i] >> (8 * k))) - a.inZp;
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        part[slice][lane][k] = acc[k];
    }
    __syncthreads();
    if (slice == 0 && c0 < C) {
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int32_t v = 0;
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
                v = int32_t(uint32_t(v) + uint32_t(part[sl][lane][k]));
            }
            if (count == 0) {
                v = 0;
            } else {
                const int32_t round = v < 0 ? -(count >> 1) : (count >> 1);
                v = int32_t(uint32_t(v) + uint32_t(round)) / count; // truncates toward zero
            }
            v = int32_t(uint32_t(v) + uint32_t(a.outZp));
            v = v < -128 ? -128 : (v > 127 ? 127 : v);
            word |= uint32_t(uint8_t(v)) << (8 * k);
        }
        *reinterpret_cast<uint32_t *>(out + ((int64_t(n) * OH + oy) * OW + ox) * C + c0) = word;
    }
}

// ---- MAX_POOL2D, int8 NHWC, C % 16 == 0 (maxpool2d.comp:23-72) --------------------------------------
// One thread per (pixel, 16-channel group): 16-byte loads, per-byte signed max, one 16-byte store.
//
// There is no four-lane byte maximum in hardware, but there is a three-input one on two 16-bit lanes.  A word of
// four int8 is therefore split into its even and its odd bytes, each moved to the HIGH byte of a 16-bit lane with
// a zero below it: the signed order of the lanes is the signed order of the bytes.  One byte permute per half and
// one three-input maximum per half and pair of taps replace the emulated byte maximum.
__device__ __forceinline__ uint32_t evenBytesHigh(uint32_t v) { return __byte_perm(v, 0u, 0x2404); }
__device__ __forceinline__ uint32_t oddBytesHigh(uint32_t v) { return __byte_perm(v, 0u, 0x3414); }
__device__ __forceinline__ uint32_t max3Lanes(uint32_t a, uint32_t b, uint32_t c) { return __vimax3_s16x2(a, b, c); }

struct PoolAcc {
    uint32_t even[4], odd[4];
    __device__ __forceinline__ PoolAcc() {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            even[i] = odd[i] = 0x80008000u; // int8 lowest in both lanes
        }
    }
    __device__ __forceinline__ void take(const int4 &p, const int4 &q) {
        const uint32_t a[4] = {uint32_t(p.x), uint32_t(p.y), uint32_t(p.z), uint32_t(p.w)};
        const uint32_t b[4] = {uint32_t(q.x), uint32_t(q.y), uint32_t(q.z), uint32_t(q.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            even[i] = max3Lanes(even[i], evenBytesHigh(a[i]), evenBytesHigh(b[i]));
            odd[i] = max3Lanes(odd[i], oddBytesHigh(a[i]), oddBytesHigh(b[i]));
        }
    }
    __device__ __forceinline__ void take(const PoolAcc &o) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            even[i] = max3Lanes(even[i], o.even[i], o.even[i]);
            odd[i] = max3Lanes(odd[i], o.odd[i], o.odd[i]);
        }
    }
    __device__ __forceinline__ int4 packed() const {
        // byte 0 and 2 from the high bytes of `even`, byte 1 and 3 from the high bytes of `odd`
        return make_int4(int(__byte_perm(even[0], odd[0], 0x7351)), int(__byte_perm(even[1], odd[1], 0x7351)),
                         int(__byte_perm(even[2], odd[2], 0x7351)), int(__byte_perm(even[3], odd[3], 0x7351)));
    }
};

// KH, KW > 0: the window is known at compile time, all its loads are issued before the first maximum.
// KH == 0: any window, two taps at a time.
template <int KH, int KW>
__global__ void maxPoolI8Kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t total, int H, int W,
                                int C, int OH, int OW, PoolAttr a) {
    const int groups = C >> 4;
    const int4 lowest = make_int4(int(0x80808080u), int(0x80808080u), int(0x80808080u), int(0x80808080u));
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += int64_t(gridDim.x) * blockDim.x) {
        const int g = int(e % groups);
        int64_t pix = e / groups;
        const int ox = int(pix % OW);
        pix /= OW;
        const int oy = int(pix % OH);
        const int n = int(pix / OH);
        const int iy0 = oy * max(a.stride[0], 1) - a.pad[0], ix0 = ox * max(a.stride[1], 1) - a.pad[2];
        const int4 *image = reinterpret_cast<const int4 *>(in + int64_t(n) * H * W * C) + g;
        const auto tap = [&](int y, int x) {
            return (unsigned(y) < unsigned(H) && unsigned(x) < unsigned(W)) ? __ldg(image + (int64_t(y) * W + x) * groups)
                                                                            : lowest;
        };
        PoolAcc acc;
        if constexpr (KH > 0) {
            constexpr int kTaps = KH * KW;
            int4 v[kTaps + 1];
#pragma unroll
            for (int t = 0; t < kTaps; ++t) {
                v[t] = tap(iy0 + t / KW, ix0 + t % KW);
            }
            v[kTaps] = lowest;
#pragma unroll
            for (int t = 0; t < kTaps; t += 2) {
                acc.take(v[t], v[t + 1]);
            }
        } else {
            const int taps = a.kernel[0] * a.kernel[1];
            for (int t = 0; t < taps; t += 2) {
                const int4 p = tap(iy0 + t / a.kernel[1], ix0 + t % a.kernel[1]);
                const int4 q = t + 1 < taps ? tap(iy0 + (t + 1) / a.kernel[1], ix0 + (t + 1) % a.kernel[1]) : lowest;
                acc.take(p, q);
            }
        }
        reinterpret_cast<int4 *>(out + ((int64_t(n) * OH + oy) * OW + ox) * C)[g] = acc.packed();
    }
}

// The 3x3 window with stride 2 (the stem pool of the residual networks): one thread makes two horizontally
// adjacent outputs, whose windows share a column, from 15 loads instead of 18.  OW must be even.
__global__ void maxPool3x3s2PairKernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t total, int H,
                                       int W, int C, int OH, int OW, int padTop, int padLeft) {
    const int groups = C >> 4, pairs = OW >> 1;
    const int4 lowest = make_int4(int(0x80808080u), int(0x80808080u), int(0x80808080u), int(0x80808080u));
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += int64_t(gridDim.x) * blockDim.x) {
        const int g = int(e % groups);
        int64_t pix = e / groups;
        const int ox = int(pix % pairs) * 2;
        pix /= pairs;
        const int oy = int(pix % OH);
        const int n = int(pix / OH);
        const int iy0 = oy * 2 - padTop, ix0 = ox * 2 - padLeft;
        const int4 *image = reinterpret_cast<const int4 *>(in + int64_t(n) * H * W * C) + g;
        int4 v[3][5];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
#pragma unroll
            for (int kx = 0; kx < 5; ++kx) {
                const int y = iy0 + ky, x = ix0 + kx;
                v[ky][kx] = (unsigned(y) < unsigned(H) && unsigned(x) < unsigned(W))
                                ? __ldg(image + (int64_t(y) * W + x) * groups)
                                : lowest;
            }
        }
        PoolAcc left, right, shared;
        shared.take(v[0][2], v[1][2]);
        shared.take(v[2][2], lowest);
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            left.take(v[ky][0], v[ky][1]);
            right.take(v[ky][3], v[ky][4]);
        }
        left.take(shared);
        right.take(shared);
        int4 *o = reinterpret_cast<int4 *>(out + ((int64_t(n) * OH + oy) * OW + ox) * C) + g;
        o[0] = left.packed();
        o[groups] = right.packed();
    }
}

// The same window and stride, a block of 2 x 2 outputs per thread (OH and OW even): the four windows cover 5 x 5
// input pixels, 25 loads instead of 36.  Every pixel word is split into its even and odd byte lanes once; a row
// gives the horizontal maxima of the left and of the right window, which the upper and the lower output share.
struct LaneWords {
    uint32_t even[4], odd[4];
};
__device__ __forceinline__ LaneWords toLanes(const int4 &v) {
    const uint32_t w[4] = {uint32_t(v.x), uint32_t(v.y), uint32_t(v.z), uint32_t(v.w)};
    LaneWords l;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        l.even[i] = evenBytesHigh(w[i]);
        l.odd[i] = oddBytesHigh(w[i]);
    }
    return l;
}
__device__ __forceinline__ LaneWords max3(const LaneWords &a, const LaneWords &b, const LaneWords &c) {
    LaneWords r;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r.even[i] = max3Lanes(a.even[i], b.even[i], c.even[i]);
        r.odd[i] = max3Lanes(a.odd[i], b.odd[i], c.odd[i]);
    }
    return r;
}
__device__ __forceinline__ int4 packLanes(const LaneWords &l) {
    return make_int4(int(__byte_perm(l.even[0], l.odd[0], 0x7351)), int(__byte_perm(l.even[1], l.odd[1], 0x7351)),
                     int(__byte_perm(l.even[2], l.odd[2], 0x7351)), int(__byte_perm(l.even[3], l.odd[3], 0x7351)));
}

__global__ void maxPool3x3s2QuadKernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int64_t total, int H,
                                       int W, int C, int OH, int OW, int padTop, int padLeft) {
    const int groups = C >> 4, pairsX = OW >> 1, pairsY = OH >> 1;
    const int4 lowest = make_int4(int(0x80808080u), int(0x80808080u), int(0x80808080u), int(0x80808080u));
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += int64_t(gridDim.x) * blockDim.x) {
        const int g = int(e % groups);
        int64_t pix = e / groups;
        const int ox = int(pix % pairsX) * 2;
        pix /= pairsX;
        const int oy = int(pix % pairsY) * 2;
        const int n = int(pix / pairsY);
        const int iy0 = oy * 2 - padTop, ix0 = ox * 2 - padLeft;
        const int4 *image = reinterpret_cast<const int4 *>(in + int64_t(n) * H * W * C) + g;
        LaneWords rowL[5], rowR[5];
#pragma unroll
        for (int ky = 0; ky < 5; ++ky) {
            int4 v[5];
#pragma unroll
            for (int kx = 0; kx < 5; ++kx) {
                const int y = iy0 + ky, x = ix0 + kx;
                v[kx] = (unsigned(y) < unsigned(H) && unsigned(x) < unsigned(W)) ? __ldg(image + (int64_t(y) * W + x) * groups)
                                                                                 : lowest;
            }
            const LaneWords mid = toLanes(v[2]);
            rowL[ky] = max3(toLanes(v[0]), toLanes(v[1]), mid);
            rowR[ky] = max3(mid, toLanes(v[3]), toLanes(v[4]));
        }
        int4 *o = reinterpret_cast<int4 *>(out + ((int64_t(n) * OH + oy) * OW + ox) * C) + g;
        o[0] = packLanes(max3(rowL[0], rowL[1], rowL[2]));
        o[groups] = packLanes(max3(rowR[0], rowR[1], rowR[2]));
        o[int64_t(OW) * groups] = packLanes(max3(rowL[2], rowL[3], rowL[4]));
        o[int64_t(OW) * groups + groups] = packLanes(max3(rowR[2], rowR[3], rowR[4]));
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

int padImageI8(const int8_t *in, int8_t *out, int N, int H, int W, int C, int Hp, int Wp, int Cp, int padTop, int padLeft,
               cudaStream_t s) {
    if (Cp == 4 && C <= 4 && Wp % 2 == 0 && int64_t(N) * Hp < (int64_t(1) << 31) &&
        (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
        padImageRows4Kernel<<<unsigned(N * Hp), 128, 0, s>>>(in, out, H, W, C, Hp, Wp, padTop, padLeft);
        return finish("padded copy");
    }
    const int64_t words = int64_t(N) * Hp * Wp * (Cp >> 2);
    padImageKernel<<<gridFor(words, kThreads, 8), kThreads, 0, s>>>(in, out, words, H, W, C, Hp, Wp, Cp, padTop, padLeft);
    return finish("padded copy");
}

int transposeForMatmul(const int8_t *b, int8_t *bt, int32_t *corr, int batches, int C, int W, int32_t za, cudaStream_t s) {
    const dim3 grid(unsigned((W + 63) / 64), unsigned(batches));
    transposeColsumKernel<<<grid, 256, 0, s>>>(b, bt, corr, C, W, za);
    return finish("MATMUL operand transpose");
}

int columnSumsForMatmul(const int8_t *b, int32_t *corr, int batches, int C, int W, int32_t za, cudaStream_t s) {
    const dim3 grid(unsigned((W + 63) / 64), unsigned(batches));
    columnSumKernel<<<grid, 256, 0, s>>>(b, corr, C, W, za);
    return finish("MATMUL operand column sums");
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

bool avgPoolI8Eligible(const TView &in, const TView &out, const PoolAttr &a) {
    // one block per output pixel and 128 channels: worthwhile when the window is large
    return maxPoolI8Eligible(in, out) && a.kernel[0] > 0 && a.kernel[1] > 0 && a.kernel[0] * a.kernel[1] >= 16 &&
           a.stride[0] > 0 && a.stride[1] > 0 &&
           int64_t(out.dims[0]) * out.dims[1] * out.dims[2] * ((out.dims[3] + 127) / 128) < (int64_t(1) << 30);
}

int avgPoolI8(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s) {
    const int C = int(in.dims[3]);
    const int64_t blocks = int64_t(out.dims[0]) * out.dims[1] * out.dims[2] * ((C + 127) / 128);
    avgPoolI8Kernel<<<unsigned(blocks), 256, 0, s>>>(reinterpret_cast<const int8_t *>(in.ptr),
                                                    reinterpret_cast<int8_t *>(out.ptr), int(in.dims[1]), int(in.dims[2]), C,
                                                    int(out.dims[1]), int(out.dims[2]), a);
    return finish("AVG_POOL2D");
}

int maxPoolI8(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s) {
    const int64_t total = int64_t(out.dims[0]) * out.dims[1] * out.dims[2] * (out.dims[3] >> 4);
    const auto launch = [&](auto kernel) {
        kernel<<<gridFor(total, kThreads, 16), kThreads, 0, s>>>(
            reinterpret_cast<const int8_t *>(in.ptr), reinterpret_cast<int8_t *>(out.ptr), total, int(in.dims[1]),
            int(in.dims[2]), int(in.dims[3]), int(out.dims[1]), int(out.dims[2]), a);
    };
    if (a.kernel[0] == 3 && a.kernel[1] == 3 && a.stride[0] == 2 && a.stride[1] == 2 && out.dims[2] % 2 == 0 &&
        out.dims[1] % 2 == 0) {
        const int64_t quads = total / 4;
        maxPool3x3s2QuadKernel<<<gridFor(quads, 128, 16), 128, 0, s>>>(
            reinterpret_cast<const int8_t *>(in.ptr), reinterpret_cast<int8_t *>(out.ptr), quads, int(in.dims[1]),
            int(in.dims[2]), int(in.dims[3]), int(out.dims[1]), int(out.dims[2]), a.pad[0], a.pad[2]);
    } else if (a.kernel[0] == 3 && a.kernel[1] == 3 && a.stride[0] == 2 && a.stride[1] == 2 && out.dims[2] % 2 == 0) {
        const int64_t pairs = total / 2;
        maxPool3x3s2PairKernel<<<gridFor(pairs, kThreads, 16), kThreads, 0, s>>>(
            reinterpret_cast<const int8_t *>(in.ptr), reinterpret_cast<int8_t *>(out.ptr), pairs, int(in.dims[1]),
            int(in.dims[2]), int(in.dims[3]), int(out.dims[1]), int(out.dims[2]), a.pad[0], a.pad[2]);
    } else if (a.kernel[0] == 3 && a.kernel[1] == 3) {
        launch(maxPoolI8Kernel<3, 3>);
    } else if (a.kernel[0] == 2 && a.kernel[1] == 2) {
        launch(maxPoolI8Kernel<2, 2>);
    } else {
        launch(maxPoolI8Kernel<0, 0>);
    }
    return finish("MAX_POOL2D");
}

} // namespace mlel
