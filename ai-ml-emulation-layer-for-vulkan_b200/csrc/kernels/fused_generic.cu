// Fused contraction + RESCALE (+ CLAMP, + residual tail) kernels in their simplest form: one
// thread per output element.  They define the fused operators' results for every shape and are
// what the tensor-core kernels are checked against and fall back to for shapes those do not take
// (odd channel counts, non-zero weight zero point, explicit strides).
//
// Arithmetic: conv2d.comp:59-112 / depthwise_conv2d.comp:47-75 / matmul.comp:42-69 followed per
// element by rescale.comp:27-72 and clamp.comp:24-53.
#include <utility>

#include "device_common.cuh"
#include "gemm_i8_tcgen05.hpp"
#include "kernels.hpp"

namespace mlel {

namespace {

#define GRID_STRIDE(e, total)                                                                                          \
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < (total); e += int64_t(gridDim.x) * blockDim.x)

__device__ inline int32_t stage(const DevRescale &r, int64_t v, uint32_t c) {
    const uint32_t ci = r.perChannel ? c : 0u;
    return rescaleValue(v, r.inZp, r.mult[ci], int32_t(r.shift[ci]), r.doubleRound != 0, r.outZp, r.lo, r.hi);
}

// acc is the int32 contraction result (bias included); c the channel (last output coordinate);
// flat the packed element offset of the output.
__device__ inline int32_t epilogue(const DevEpilogue &e, int32_t acc, uint32_t c, int64_t flat) {
    int32_t y = stage(e.main, int64_t(acc), c);
    if (e.hasResidual) {
        const int32_t ta = stage(e.a, int64_t(y), c);
        const int32_t tb = stage(e.b, int64_t(e.shortcut[flat]), c);
        const int32_t sum = int32_t(uint32_t(ta) + uint32_t(tb));
        y = stage(e.out, int64_t(sum), c);
    }
    return y;
}

__host__ __device__ inline int64_t numelOf(const TView &t) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; ++i) {
        n *= t.dims[i];
    }
    return n;
}

__global__ void fusedConvKernel(TView in, TView w, TView bias, TView out, ConvAttr a, DevEpilogue epi) {
    const int64_t total = numelOf(out);
    const uint32_t KH = w.dims[1], KW = w.dims[2], IC = in.dims[3], H = in.dims[1], W = in.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], oc = idx[3];
        const uint32_t iy = oy * uint32_t(a.stride[0]) - uint32_t(a.pad[0]);
        const uint32_t ix = ox * uint32_t(a.stride[1]) - uint32_t(a.pad[2]);
        uint32_t acc = 0;
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                const uint32_t y = iy + ky * uint32_t(a.dilation[0]);
                const uint32_t x = ix + kx * uint32_t(a.dilation[1]);
                if (y < H && x < W) {
                    const uint32_t ci0[4] = {n, y, x, 0};
                    const uint32_t cw0[4] = {oc, ky, kx, 0};
                    const int64_t io = offsetOf(in, ci0), wo = offsetOf(w, cw0);
                    for (uint32_t ic = 0; ic < IC; ++ic) {
                        const int32_t v = int32_t(loadIntAt(in, io + int64_t(ic) * in.strides[3])) - a.inZp;
                        const int32_t wt = ((wo < 0 || ic >= w.dims[3])
                                                ? 0
                                                : int32_t(loadIntAt(w, wo + int64_t(ic) * w.strides[3]))) -
                                           a.wZp;
                        acc += uint32_t(v) * uint32_t(wt);
                    }
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
        acc += uint32_t(int32_t(loadInt(bias, cb)));
        storeInt(out, idx, epilogue(epi, int32_t(acc), oc, e));
    }
}

__global__ void fusedDepthwiseKernel(TView in, TView w, TView bias, TView out, ConvAttr a, DevEpilogue epi) {
    const int64_t total = numelOf(out);
    const uint32_t KH = w.dims[0], KW = w.dims[1], M = w.dims[3], H = in.dims[1], W = in.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], ocm = idx[3];
        const uint32_t c = ocm / M, m = ocm % M;
        const uint32_t iy = oy * uint32_t(a.stride[0]) - uint32_t(a.pad[0]);
        const uint32_t ix = ox * uint32_t(a.stride[1]) - uint32_t(a.pad[2]);
        uint32_t acc = 0;
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                const uint32_t y = iy + ky * uint32_t(a.dilation[0]);
                const uint32_t x = ix + kx * uint32_t(a.dilation[1]);
                if (y < H && x < W) {
                    const uint32_t ci[4] = {n, y, x, c};
                    const uint32_t cw[4] = {ky, kx, c, m};
                    const int32_t v = int32_t(loadInt(in, ci)) - a.inZp;
                    const int32_t wt = int32_t(loadInt(w, cw)) - a.wZp;
                    acc += uint32_t(v) * uint32_t(wt);
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : ocm};
        acc += uint32_t(int32_t(loadInt(bias, cb)));
        storeInt(out, idx, epilogue(epi, int32_t(acc), ocm, e));
    }
}

// ---- DEPTHWISE_CONV2D 3x3, packed int8 NHWC, channel multiplier 1 (depthwise_conv2d.comp:31-78) ----------
// Memory-bound shape of a MobileNet block.  A thread owns four channels (one 32-bit word) of PX consecutive
// output pixels of one row: the 36 weights of its channels live in registers for all of them, every input
// word is loaded once per row of the window and serves up to three neighbouring outputs, and each output
// pixel is one 32-bit store.  Out-of-range taps read the input zero point instead of being skipped, which
// gives the same sum: (zp - zp) * w = 0.  SX = x stride (1 or 2); the y stride is free; dilation is 1.
// OUT8: fused RESCALE(+CLAMP) to int8, else the raw int32 result.
template <int PX, int SX, bool OUT8>
__global__ void depthwise3x3Kernel(const int8_t *__restrict__ in, const int8_t *__restrict__ w,
                                   const int32_t *__restrict__ bias, int biasCount, void *__restrict__ out, int N, int H,
                                   int W, int C, int OH, int OW, ConvAttr a, DevEpilogue epi) {
    constexpr int COLS = (PX - 1) * SX + 3;
    const int cw = C >> 2;
    const int groupsX = (OW + PX - 1) / PX;
    const int64_t total = int64_t(N) * OH * groupsX * cw;
    const uint32_t zword = uint32_t(uint8_t(a.inZp)) * 0x01010101u;
    GRID_STRIDE(e, total) {
        int64_t t = e;
        const int c0 = int(t % cw) * 4;
        t /= cw;
        const int ox0 = int(t % groupsX) * PX;
        t /= groupsX;
        const int oy = int(t % OH);
        const int n = int(t / OH);
        int32_t acc[PX][4];
#pragma unroll
        for (int px = 0; px < PX; ++px) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[px][k] = 0;
            }
        }
        int32_t wsum[4] = {0, 0, 0, 0};
        const int x0 = ox0 * SX - a.pad[2];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const int y = oy * a.stride[0] - a.pad[0] + ky;
            const bool rowOk = y >= 0 && y < H;
            const int8_t *row = in + ((int64_t(n) * H + (rowOk ? y : 0)) * W) * C + c0;
            uint32_t cols[COLS];
#pragma unroll
            for (int i = 0; i < COLS; ++i) {
                const int x = x0 + i;
                cols[i] = (rowOk && x >= 0 && x < W) ? __ldg(reinterpret_cast<const uint32_t *>(row + int64_t(x) * C)) : zword;
            }
#pragma unroll
            for (int kx = 0; kx < 3; ++kx) {
                const uint32_t wword = __ldg(reinterpret_cast<const uint32_t *>(w + (ky * 3 + kx) * C + c0));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int32_t wt = int32_t(int8_t(wword >> (8 * k))) - a.wZp;
                    wsum[k] += wt;
#pragma unroll
                    for (int px = 0; px < PX; ++px) {
                        const int32_t x = int32_t(int8_t(cols[px * SX + kx] >> (8 * k)));
                        acc[px][k] = int32_t(uint32_t(acc[px][k]) + uint32_t(x) * uint32_t(wt));
                    }
                }
            }
        }
        int32_t add[4];
        FastRescale fr[4]; // the fused RESCALE of this thread's four channels (OUT8 only)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int32_t b = __ldg(bias + (biasCount == 1 ? 0 : c0 + k));
            add[k] = int32_t(uint32_t(b) - uint32_t(a.inZp) * uint32_t(wsum[k]));
            if (OUT8) {
                const int ci = epi.main.perChannel ? c0 + k : 0;
                fr[k] = makeFastRescale(__ldg(epi.main.mult + ci), int32_t(__ldg(epi.main.shift + ci)), epi.main.inZp,
                                        epi.main.doubleRound != 0);
            }
        }
#pragma unroll
        for (int px = 0; px < PX; ++px) {
            const int ox = ox0 + px;
            if (ox >= OW) {
                break;
            }
            const int64_t flat = ((int64_t(n) * OH + oy) * OW + ox) * C + c0;
            if (OUT8) {
                uint32_t word = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int32_t v = int32_t(uint32_t(acc[px][k]) + uint32_t(add[k]));
                    word |= uint32_t(uint8_t(fastRescale(fr[k], v, epi.main.outZp, epi.main.lo, epi.main.hi))) << (8 * k);
                }
                *reinterpret_cast<uint32_t *>(static_cast<int8_t *>(out) + flat) = word;
            } else {
                int4 v;
                v.x = int32_t(uint32_t(acc[px][0]) + uint32_t(add[0]));
                v.y = int32_t(uint32_t(acc[px][1]) + uint32_t(add[1]));
                v.z = int32_t(uint32_t(acc[px][2]) + uint32_t(add[2]));
                v.w = int32_t(uint32_t(acc[px][3]) + uint32_t(add[3]));
                *reinterpret_cast<int4 *>(static_cast<int32_t *>(out) + flat) = v;
            }
        }
    }
}

// ---- The same operator with the taps of a window row packed for dp4a (weight zero point 0) ------------------------
// A thread owns four channels (one 32-bit word per pixel) of a block of 4 output pixels x R output rows.  Input rows
// stream through once: a row's pixel words are transposed four at a time (4 pixels x 4 channels -> 4 channels x
// 4 pixels, eight byte-permutes), so that three neighbouring taps of one channel lie in one word; one dp4a against
// the channel's three weights of that window row (kept in two words, at byte offset 0 and at byte offset 1, for the
// windows that start at the word's first and second pixel) gives three multiply-accumulates.  An input row feeds
// the up to three output rows whose windows contain it, so the loads and transposes are shared vertically as
// well.  Out-of-range taps read the input zero point, and bias - zp * (sum of weights) corrects for the raw sums,
// as in depthwise3x3Kernel.  About 4.5 instructions per output for the convolution against 27 there.
__device__ __forceinline__ void transpose4x4Bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&o)[4]) {
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140); // [a0 b0 a1 b1], [c0 d0 c1 d1]
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362); // [a2 b2 a3 b3], [c2 d2 c3 d3]
    o[0] = __byte_perm(t0, t1, 0x5410), o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410), o[3] = __byte_perm(t2, t3, 0x7632);
}

template <int R, int SX, bool OUT8>
__global__ void __launch_bounds__(128) depthwise3x3RowsKernel(const int8_t *__restrict__ in, const int8_t *__restrict__ w,
                                                              const int32_t *__restrict__ bias, int biasCount,
                                                              void *__restrict__ out, int N, int H, int W, int C, int OH,
                                                              int OW, ConvAttr a, DevEpilogue epi) {
    constexpr int PX = 4;
    constexpr int COLS = (PX - 1) * SX + 3; // input pixels under the four windows of a row: 6 or 9
    constexpr int NT = SX == 1 ? 2 : 4;     // transposed groups of four pixels per input row
    // Launched so that it may be scheduled while the kernel before it in the stream drains, and lets the kernel after
    // it do the same (programmatic dependent launch): nothing is read or written before the wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int cw = C >> 2;
    const int groupsX = (OW + PX - 1) / PX, groupsY = (OH + R - 1) / R;
    const int64_t total = int64_t(N) * groupsY * groupsX * cw;
    const uint32_t zword = uint32_t(uint8_t(a.inZp)) * 0x01010101u;
    GRID_STRIDE(e, total) {
        int64_t t = e;
        const int c0 = int(t % cw) * 4;
        t /= cw;
        const int ox0 = int(t % groupsX) * PX;
        t /= groupsX;
        const int oy0 = int(t % groupsY) * R;
        const int n = int(t / groupsY);
        // the three weights of a window row of one channel at byte offsets 0 and 1, and their sum
        uint32_t wa[3][4], wb[3][4];
        int32_t wsum[4] = {0, 0, 0, 0};
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const uint32_t w0 = __ldg(reinterpret_cast<const uint32_t *>(w + (ky * 3 + 0) * C + c0));
            const uint32_t w1 = __ldg(reinterpret_cast<const uint32_t *>(w + (ky * 3 + 1) * C + c0));
            const uint32_t w2 = __ldg(reinterpret_cast<const uint32_t *>(w + (ky * 3 + 2) * C + c0));
            uint32_t tw[4];
            transpose4x4Bytes(w0, w1, w2, 0u, tw); // tw[k] = [w(kx=0) w(kx=1) w(kx=2) 0] of channel k
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                wa[ky][k] = tw[k];
                wb[ky][k] = tw[k] << 8;
                wsum[k] = __dp4a(int32_t(tw[k]), 0x01010101, wsum[k]);
            }
        }
        int32_t acc[R][PX][4];
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int px = 0; px < PX; ++px) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    acc[r][px][k] = 0;
                }
            }
        }
        const int x0 = ox0 * SX - a.pad[2];
        const int yFirst = oy0 * SX - a.pad[0];
        constexpr int ROWS = (R - 1) * SX + 3; // input rows under the R windows of a column (y stride = x stride)
#pragma unroll
        for (int iy = 0; iy < ROWS; ++iy) {
            const int y = yFirst + iy;
            const bool rowOk = y >= 0 && y < H;
            const int8_t *row = in + ((int64_t(n) * H + (rowOk ? y : 0)) * W) * C + c0;
            uint32_t cols[COLS];
#pragma unroll
            for (int i = 0; i < COLS; ++i) {
                const int x = x0 + i;
                cols[i] = (rowOk && x >= 0 && x < W) ? __ldg(reinterpret_cast<const uint32_t *>(row + int64_t(x) * C)) : zword;
            }
            // tr[g][k]: four consecutive pixels of channel k.  Stride 1: pixels 0-3 and 2-5; window px starts at byte
            // px & 1 of group px >> 1.  Stride 2: pixels 0-3, 2-5, 4-7, 5-8; windows start at bytes 0, 0, 0, 1.
            uint32_t tr[NT][4];
            transpose4x4Bytes(cols[0], cols[1], cols[2], cols[3], tr[0]);
            transpose4x4Bytes(cols[2], cols[3], cols[4], cols[5], tr[1]);
            if (SX == 2) {
                transpose4x4Bytes(cols[4], cols[5], cols[6], cols[7], tr[2]);
                transpose4x4Bytes(cols[5], cols[6], cols[7], cols[8], tr[3]);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int ky = iy - r * SX; // this input row as a row of output row r's window (a compile-time value)
                if (ky >= 0 && ky < 3) {
#pragma unroll
                    for (int px = 0; px < PX; ++px) {
                        const int g = SX == 1 ? px >> 1 : px;
                        const bool second = SX == 1 ? (px & 1) != 0 : px == 3;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t wsel = second ? wb[ky][k] : wa[ky][k];
                            acc[r][px][k] = __dp4a(int32_t(tr[g][k]), int32_t(wsel), acc[r][px][k]);
                        }
                    }
                }
            }
        }
        int32_t add[4];
        FastRescale fr[4]; // the fused RESCALE of this thread's four channels (OUT8 only)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int32_t b = __ldg(bias + (biasCount == 1 ? 0 : c0 + k));
            add[k] = int32_t(uint32_t(b) - uint32_t(a.inZp) * uint32_t(wsum[k]));
            if (OUT8) {
                const int ci = epi.main.perChannel ? c0 + k : 0;
                fr[k] = makeFastRescale(__ldg(epi.main.mult + ci), int32_t(__ldg(epi.main.shift + ci)), epi.main.inZp,
                                        epi.main.doubleRound != 0);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int oy = oy0 + r;
            if (oy >= OH) {
                break;
            }
#pragma unroll
            for (int px = 0; px < PX; ++px) {
                const int ox = ox0 + px;
                if (ox >= OW) {
                    break;
                }
                const int64_t flat = ((int64_t(n) * OH + oy) * OW + ox) * C + c0;
                if (OUT8) {
                    uint32_t word = 0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int32_t v = int32_t(uint32_t(acc[r][px][k]) + uint32_t(add[k]));
                        word |= uint32_t(uint8_t(fastRescale(fr[k], v, epi.main.outZp, epi.main.lo, epi.main.hi))) << (8 * k);
                    }
                    *reinterpret_cast<uint32_t *>(static_cast<int8_t *>(out) + flat) = word;
                } else {
                    int4 v;
                    v.x = int32_t(uint32_t(acc[r][px][0]) + uint32_t(add[0]));
                    v.y = int32_t(uint32_t(acc[r][px][1]) + uint32_t(add[1]));
                    v.z = int32_t(uint32_t(acc[r][px][2]) + uint32_t(add[2]));
                    v.w = int32_t(uint32_t(acc[r][px][3]) + uint32_t(add[3]));
                    *reinterpret_cast<int4 *>(static_cast<int32_t *>(out) + flat) = v;
                }
            }
        }
    }
}

__global__ void fusedMatmulKernel(TView a, TView b, TView out, int32_t zpA, int32_t zpB, DevEpilogue epi) {
    const int64_t total = numelOf(out);
    const uint32_t K = a.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank];
        unravel(out, uint32_t(e), idx);
        const uint32_t ca[3] = {idx[0], idx[1], 0};
        const uint32_t cb[3] = {idx[0], 0, idx[2]};
        const int64_t ao = offsetOf(a, ca), bo = offsetOf(b, cb);
        uint32_t acc = 0;
        for (uint32_t c = 0; c < K; ++c) {
            const int32_t v1 = (ao < 0 ? 0 : int32_t(loadIntAt(a, ao + int64_t(c) * a.strides[2]))) - zpA;
            const int32_t v2 =
                ((bo < 0 || c >= b.dims[1]) ? 0 : int32_t(loadIntAt(b, bo + int64_t(c) * b.strides[1]))) - zpB;
            acc += uint32_t(v1) * uint32_t(v2);
        }
        storeInt(out, idx, epilogue(epi, int32_t(acc), idx[2], e));
    }
}

// 16 int8 elements per thread, 16-byte loads and stores; n is padded work in 16-element groups.
__global__ void fusedAddKernel(const int8_t *__restrict__ x, const int8_t *__restrict__ y, int8_t *__restrict__ out,
                               int64_t n, int64_t groups, DevEpilogue epi) {
    const FastRescale fa = makeFastRescale(epi.a.mult[0], epi.a.shift[0], epi.a.inZp, epi.a.doubleRound != 0);
    const FastRescale fb = makeFastRescale(epi.b.mult[0], epi.b.shift[0], epi.b.inZp, epi.b.doubleRound != 0);
    const FastRescale fo = makeFastRescale(epi.out.mult[0], epi.out.shift[0], epi.out.inZp, epi.out.doubleRound != 0);
    const auto one = [&](int8_t vx, int8_t vy) -> int8_t {
        const int32_t ta = fastRescale(fa, vx, epi.a.outZp, epi.a.lo, epi.a.hi);
        const int32_t tb = fastRescale(fb, vy, epi.b.outZp, epi.b.lo, epi.b.hi);
        const int32_t sum = int32_t(uint32_t(ta) + uint32_t(tb));
        return int8_t(fastRescale(fo, sum, epi.out.outZp, epi.out.lo, epi.out.hi));
    };
    GRID_STRIDE(g, groups) {
        const int4 vx = reinterpret_cast<const int4 *>(x)[g];
        const int4 vy = reinterpret_cast<const int4 *>(y)[g];
        int4 vo;
        const int8_t *px = reinterpret_cast<const int8_t *>(&vx);
        const int8_t *py = reinterpret_cast<const int8_t *>(&vy);
        int8_t *po = reinterpret_cast<int8_t *>(&vo);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            po[k] = one(px[k], py[k]);
        }
        reinterpret_cast<int4 *>(out)[g] = vo;
    }
    // elements past the last full group (all of them when the pointers are not 16-byte aligned)
    const int64_t rest = n - groups * 16;
    GRID_STRIDE(t, rest) {
        const int64_t k = groups * 16 + t;
        out[k] = one(x[k], y[k]);
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

int fusedConv2dGeneric(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                       const DevEpilogue &epi, cudaStream_t s) {
    fusedConvKernel<<<gridFor(numelOf(out)), kThreads, 0, s>>>(in, w, bias, out, a, epi);
    return finish("CONV2D+RESCALE");
}

int fusedDepthwiseGeneric(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                          const DevEpilogue &epi, cudaStream_t s) {
    fusedDepthwiseKernel<<<gridFor(numelOf(out)), kThreads, 0, s>>>(in, w, bias, out, a, epi);
    return finish("DEPTHWISE_CONV2D+RESCALE");
}

bool depthwise3x3Eligible(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                          bool fused) {
    const auto packed = [](const TView &t) {
        int64_t s = dtypeSize(t.dtype); // strides are in bytes
        for (int i = t.rank - 1; i >= 0; --i) {
            if (t.strides[i] != s) {
                return false;
            }
            s *= t.dims[i];
        }
        return true;
    };
    if (in.dtype != MLEL_I8 || w.dtype != MLEL_I8 || bias.dtype != MLEL_I32 || out.dtype != (fused ? MLEL_I8 : MLEL_I32) ||
        in.rank != 4 || w.rank != 4 || out.rank != 4 || !packed(in) || !packed(w) || !packed(bias) || !packed(out)) {
        return false;
    }
    const int64_t C = in.dims[3];
    if (w.dims[0] != 3 || w.dims[1] != 3 || w.dims[2] != C || w.dims[3] != 1 || out.dims[3] != C || C % 4 != 0 ||
        out.dims[0] != in.dims[0] || (bias.dims[0] != C && bias.dims[0] != 1) || a.dilation[0] != 1 || a.dilation[1] != 1 ||
        a.stride[0] < 1 || (a.stride[1] != 1 && a.stride[1] != 2) || numelOf(in) >= (int64_t(1) << 31) ||
        numelOf(out) >= (int64_t(1) << 31)) {
        return false;
    }
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(in.ptr) | reinterpret_cast<uintptr_t>(w.ptr) |
                           reinterpret_cast<uintptr_t>(bias.ptr);
    return (ptrs & 3u) == 0 && (reinterpret_cast<uintptr_t>(out.ptr) & (fused ? 3u : 15u)) == 0;
}

// Launch with programmatic stream serialization (the kernel must execute griddepcontrol.wait before it touches
// memory): its blocks may be scheduled while the previous kernel of the stream drains.
template <class... Params, class... Args>
static void launchOverlapping(void (*kernel)(Params...), int grid, int threads, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(unsigned(threads));
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = tensorCoreTuning().dependentLaunch.load(std::memory_order_relaxed) != 0 ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

int depthwise3x3(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                 const DevEpilogue *epi, cudaStream_t s) {
    constexpr int PX = 4;
    const int N = int(in.dims[0]), H = int(in.dims[1]), W = int(in.dims[2]), C = int(in.dims[3]);
    const int OH = int(out.dims[1]), OW = int(out.dims[2]);
    const auto *pi = reinterpret_cast<const int8_t *>(in.ptr);
    const auto *pw = reinterpret_cast<const int8_t *>(w.ptr);
    const auto *pb = reinterpret_cast<const int32_t *>(bias.ptr);
    const int nb = int(bias.dims[0]);
    const DevEpilogue none{};
    const DevEpilogue &e = epi != nullptr ? *epi : none;
    if (a.wZp == 0 && a.stride[0] == a.stride[1]) {
        // tap-packed kernel; fewer output rows per thread where four would leave SMs without work
        const int64_t blocks4 = int64_t(N) * ((OH + 3) / 4) * ((OW + PX - 1) / PX) * (C / 4);
        const bool four = blocks4 >= int64_t(kNumSMs) * 128 * 4;
        const int R = four ? 4 : 2;
        const int64_t total = int64_t(N) * ((OH + R - 1) / R) * ((OW + PX - 1) / PX) * (C / 4);
        const int grid = gridFor(total, 128, 16);
#define MLEL_LAUNCH_ROWS(RR, SS, O8) \
    launchOverlapping(depthwise3x3RowsKernel<RR, SS, O8>, grid, 128, s, pi, pw, pb, nb, out.ptr, N, H, W, C, OH, OW, a, e)
        if (epi != nullptr) {
            if (a.stride[1] == 1) {
                if (four) { MLEL_LAUNCH_ROWS(4, 1, true); } else { MLEL_LAUNCH_ROWS(2, 1, true); }
            } else {
                if (four) { MLEL_LAUNCH_ROWS(4, 2, true); } else { MLEL_LAUNCH_ROWS(2, 2, true); }
            }
        } else if (a.stride[1] == 1) {
            if (four) { MLEL_LAUNCH_ROWS(4, 1, false); } else { MLEL_LAUNCH_ROWS(2, 1, false); }
        } else {
            if (four) { MLEL_LAUNCH_ROWS(4, 2, false); } else { MLEL_LAUNCH_ROWS(2, 2, false); }
        }
#undef MLEL_LAUNCH_ROWS
        return finish("DEPTHWISE_CONV2D 3x3");
    }
    const int64_t total = int64_t(N) * OH * ((OW + PX - 1) / PX) * (C / 4);
    const int grid = gridFor(total, 128, 16);
    if (epi != nullptr) {
        if (a.stride[1] == 1) {
            depthwise3x3Kernel<PX, 1, true><<<grid, 128, 0, s>>>(pi, pw, pb, nb, out.ptr, N, H, W, C, OH, OW, a, *epi);
        } else {
            depthwise3x3Kernel<PX, 2, true><<<grid, 128, 0, s>>>(pi, pw, pb, nb, out.ptr, N, H, W, C, OH, OW, a, *epi);
        }
    } else if (a.stride[1] == 1) {
        depthwise3x3Kernel<PX, 1, false><<<grid, 128, 0, s>>>(pi, pw, pb, nb, out.ptr, N, H, W, C, OH, OW, a, none);
    } else {
        depthwise3x3Kernel<PX, 2, false><<<grid, 128, 0, s>>>(pi, pw, pb, nb, out.ptr, N, H, W, C, OH, OW, a, none);
    }
    return finish("DEPTHWISE_CONV2D 3x3");
}

int fusedMatmulGeneric(const TView &a, const TView &b, const TView &out, int32_t zpA, int32_t zpB,
                       const DevEpilogue &epi, cudaStream_t s) {
    fusedMatmulKernel<<<gridFor(numelOf(out)), kThreads, 0, s>>>(a, b, out, zpA, zpB, epi);
    return finish("MATMUL+RESCALE");
}

int fusedAdd(const int8_t *x, const int8_t *y, int8_t *out, int64_t n, const DevEpilogue &epi, cudaStream_t s) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                           reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const int64_t groups = aligned ? n / 16 : 0;
    fusedAddKernel<<<gridFor(aligned ? groups + 16 : n), kThreads, 0, s>>>(x, y, out, n, groups, epi);
    return finish("RESCALE+ADD+RESCALE");
}

} // namespace mlel
