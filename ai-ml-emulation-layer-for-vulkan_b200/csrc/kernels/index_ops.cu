// Index-driven and less common TOSA operators: ARGMAX, GATHER, SCATTER, REVERSE, TILE, RESIZE (integer
// modes), TRANSPOSE_CONV2D, CONV3D, FFT2D and RFFT2D.  As in generic_ops.cu one thread produces one output element, the
// work split of the reference's 1-D compute shaders, with any rank, stride and integer element type the
// reference accepts; element moves copy raw bits, so they carry float types too.
//
// Reference arithmetic: graph/shaders/graph_op/tosa/<op>.comp (cited per kernel).
#include <string>

#include "device_common.cuh"
#include "kernels.hpp"

namespace mlel {

namespace {

#define GRID_STRIDE(e, total)                                                                                          \
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < (total); e += int64_t(gridDim.x) * blockDim.x)

__host__ __device__ inline int64_t numelOf(const TView &t) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; ++i) {
        n *= t.dims[i];
    }
    return n;
}

int finish(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        setLastError(std::string(what) + ": " + cudaGetErrorString(err));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

// Raw-bit element copy; a source offset < 0 (coordinate out of range) reads as zero.
__device__ inline void moveElem(const TView &in, int64_t so, const TView &out, int64_t doff) {
    if (doff >= 0) {
        storeIntAt(out, doff, so < 0 ? 0 : loadIntAt(in, so));
    }
}

// ---- ARGMAX: argmax.comp:26-66 (integer path: first strictly greater value wins, start = lowest) ----------
__global__ void argmaxKernel(TView in, TView out, uint32_t axis) {
    const int64_t total = numelOf(out);
    const int64_t lowest = typeLowest(in.dtype);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, src[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        for (uint32_t i = 0; i < axis; ++i) {
            src[i] = idx[i];
        }
        for (uint32_t i = axis; i < uint32_t(out.rank); ++i) {
            src[i + 1] = idx[i];
        }
        int64_t best = lowest;
        int32_t bestIndex = 0;
        for (uint32_t k = 0; k < in.dims[axis]; ++k) {
            src[axis] = k;
            const int64_t v = loadInt(in, src);
            if (v > best) {
                best = v;
                bestIndex = int32_t(k);
            }
        }
        storeInt(out, idx, bestIndex);
    }
}

// ---- GATHER: gather.comp:14-25 -----------------------------------------------------------------------------
__global__ void gatherKernel(TView values, TView indices, TView out) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        const uint32_t ci[2] = {idx[0], idx[1]};
        const uint32_t k = uint32_t(loadInt(indices, ci));
        const uint32_t cv[3] = {idx[0], k, idx[2]};
        moveElem(values, offsetOf(values, cv), out, offsetOf(out, idx));
    }
}

// ---- SCATTER: scatter.comp:15-34 (the first index that names this row wins; otherwise values_in) ---------
__global__ void scatterKernel(TView valuesIn, TView indices, TView input, TView out) {
    const int64_t total = numelOf(out);
    const uint32_t W = indices.dims[1];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        const TView *src = &valuesIn;
        uint32_t cs[3] = {idx[0], idx[1], idx[2]};
        for (uint32_t w = 0; w < W; ++w) {
            const uint32_t ci[2] = {idx[0], w};
            if (uint32_t(loadInt(indices, ci)) == idx[1]) {
                src = &input;
                cs[1] = w;
                break;
            }
        }
        moveElem(*src, offsetOf(*src, cs), out, offsetOf(out, idx));
    }
}

// ---- REVERSE: reverse.comp:19-30, TILE: tile.comp:15-30 ---------------------------------------------------
__global__ void reverseKernel(TView in, TView out, uint32_t axis) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        const int64_t so = offsetOf(in, idx);
        idx[axis] = out.dims[axis] - 1 - idx[axis];
        moveElem(in, so, out, offsetOf(out, idx));
    }
}

__global__ void tileKernel(TView in, TView out) {
    const int64_t total = numelOf(out);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0}, src[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        for (int i = 0; i < out.rank; ++i) {
            src[i] = idx[i] % in.dims[i];
        }
        moveElem(in, offsetOf(in, src), out, offsetOf(out, idx));
    }
}

// ---- RESIZE: resize.comp:43-134, integer types ------------------------------------------------------------
// ACC is the output's own type (int8/int16 for NEAREST, int32/int64 for BILINEAR); the positions and weights
// are 16-bit as in the shader, the products wrap in ACC.
__device__ inline int32_t idivFloor(int32_t n, int32_t d) {
    int32_t r = n / d;
    if (r * d > n) {
        --r;
    }
    return r;
}

template <typename ACC> __global__ void resizeKernel(TView in, TView out, ResizeAttr a) {
    using U = typename std::make_unsigned<ACC>::type;
    const int64_t total = numelOf(out);
    const uint32_t H = in.dims[1], W = in.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], c = idx[3];
        const int16_t unitY = int16_t(a.scale[0]), unitX = int16_t(a.scale[2]);
        const int32_t y = int32_t(oy * uint32_t(a.scale[1]) + uint32_t(a.offset[0]));
        const int16_t iy = int16_t(idivFloor(y, a.scale[0]));
        const int16_t dy = int16_t(uint32_t(y) - uint32_t(int32_t(iy)) * uint32_t(a.scale[0]));
        const int32_t x = int32_t(ox * uint32_t(a.scale[3]) + uint32_t(a.offset[1]));
        const int16_t ix = int16_t(idivFloor(x, a.scale[2]));
        const int16_t dx = int16_t(uint32_t(x) - uint32_t(int32_t(ix)) * uint32_t(a.scale[2]));
        // max(int16, int) is signed; min(int, uint) converts to unsigned (resize.comp:97-100)
        const int16_t iy0 = int16_t(iy > 0 ? iy : 0);
        const uint32_t y1u = uint32_t(int32_t(iy) + 1), x1u = uint32_t(int32_t(ix) + 1);
        const int16_t iy1 = int16_t(y1u < H - 1 ? y1u : H - 1);
        const int16_t ix0 = int16_t(ix > 0 ? ix : 0);
        const int16_t ix1 = int16_t(x1u < W - 1 ? x1u : W - 1);
        const auto at = [&](int16_t yy, int16_t xx) {
            const uint32_t ci[4] = {n, uint32_t(int32_t(yy)), uint32_t(int32_t(xx)), c};
            return ACC(loadInt(in, ci));
        };
        ACC acc = 0;
        if (a.mode == 2) { // BILINEAR
            const U wy0 = U(ACC(int16_t(unitY - dy))), wy1 = U(ACC(dy));
            const U wx0 = U(ACC(int16_t(unitX - dx))), wx1 = U(ACC(dx));
            U s = U(at(iy0, ix0)) * wy0 * wx0;
            s += U(at(iy0, ix1)) * wy0 * wx1;
            s += U(at(iy1, ix0)) * wy1 * wx0;
            s += U(at(iy1, ix1)) * wy1 * wx1;
            acc = ACC(s);
        } else if (a.mode == 1) { // NEAREST
            const int16_t py = (2 * int32_t(dy) >= a.scale[0]) ? iy1 : iy0;
            const int16_t px = (2 * int32_t(dx) >= a.scale[2]) ? ix1 : ix0;
            acc = at(py, px);
        }
        storeInt(out, idx, int64_t(acc));
    }
}

// ---- TRANSPOSE_CONV2D: transpose_conv2d.comp:29-70 ---------------------------------------------------------
// GLSL's % and / on signed integers truncate toward zero like C's, so a negative position that is a multiple
// of the stride passes the first test and is rejected by the range test afterwards, as in the shader.
template <typename ACC> __global__ void transposeConv2dKernel(TView in, TView w, TView bias, TView out, ConvAttr a) {
    using U = typename std::make_unsigned<ACC>::type;
    const int64_t total = numelOf(out);
    const uint32_t KH = w.dims[1], KW = w.dims[2], IC = in.dims[3], H = in.dims[1], W = in.dims[2];
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2], oc = idx[3];
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
        U acc = U(ACC(loadInt(bias, cb)));
        for (uint32_t ky = 0; ky < KH; ++ky) {
            for (uint32_t kx = 0; kx < KW; ++kx) {
                int32_t iy = int32_t(oy) - a.pad[0] - int32_t(ky);
                int32_t ix = int32_t(ox) - a.pad[2] - int32_t(kx);
                if (iy % a.stride[0] != 0 || ix % a.stride[1] != 0) {
                    continue;
                }
                iy /= a.stride[0];
                ix /= a.stride[1];
                if (iy < 0 || ix < 0 || uint32_t(iy) >= H || uint32_t(ix) >= W) {
                    continue;
                }
                for (uint32_t ic = 0; ic < IC; ++ic) {
                    const uint32_t ci[4] = {n, uint32_t(iy), uint32_t(ix), ic};
                    const uint32_t cw[4] = {oc, ky, kx, ic};
                    const ACC v = ACC(loadInt(in, ci)) - ACC(a.inZp);
                    const ACC wt = ACC(loadInt(w, cw)) - ACC(a.wZp);
                    acc += U(v) * U(wt);
                }
            }
        }
        storeInt(out, idx, int64_t(ACC(acc)));
    }
}

// ---- CONV3D: conv3d.comp:33-104 ------------------------------------------------------------------------------
// The shader skips the taps left of the input (it starts at the first tap whose position is >= 0) and stops at
// the first tap right of it; with the signed positions used here that is the same set of taps.
template <typename ACC> __global__ void conv3dKernel(TView in, TView w, TView bias, TView out, Conv3dAttr a) {
    using U = typename std::make_unsigned<ACC>::type;
    const int64_t total = numelOf(out);
    const int32_t KD = int32_t(w.dims[1]), KH = int32_t(w.dims[2]), KW = int32_t(w.dims[3]), IC = int32_t(w.dims[4]);
    const int32_t ID = int32_t(in.dims[1]), IH = int32_t(in.dims[2]), IW = int32_t(in.dims[3]);
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(out, uint32_t(e), idx);
        const uint32_t n = idx[0], oc = idx[4];
        const int32_t id = int32_t(idx[1]) * a.stride[0] - a.pad[0];
        const int32_t iy = int32_t(idx[2]) * a.stride[1] - a.pad[2];
        const int32_t ix = int32_t(idx[3]) * a.stride[2] - a.pad[4];
        const auto firstTap = [](int32_t pos, int32_t dil) { return pos < 0 ? (-pos + dil - 1) / dil : 0; };
        const int32_t kd0 = firstTap(id, a.dilation[0]), ky0 = firstTap(iy, a.dilation[1]),
                      kx0 = firstTap(ix, a.dilation[2]);
        U acc = 0;
        for (int32_t kd = kd0, d = id + kd0 * a.dilation[0]; kd < KD && d < ID; ++kd, d += a.dilation[0]) {
            for (int32_t ky = ky0, y = iy + ky0 * a.dilation[1]; ky < KH && y < IH; ++ky, y += a.dilation[1]) {
                for (int32_t kx = kx0, x = ix + kx0 * a.dilation[2]; kx < KW && x < IW; ++kx, x += a.dilation[2]) {
                    for (int32_t ic = 0; ic < IC; ++ic) {
                        const uint32_t ci[5] = {n, uint32_t(d), uint32_t(y), uint32_t(x), uint32_t(ic)};
                        const uint32_t cw[5] = {oc, uint32_t(kd), uint32_t(ky), uint32_t(kx), uint32_t(ic)};
                        const ACC v = ACC(loadInt(in, ci)) - ACC(a.inZp);
                        const ACC wt = ACC(loadInt(w, cw)) - ACC(a.wZp);
                        acc += U(v) * U(wt);
                    }
                }
            }
        }
        const uint32_t cb[1] = {bias.dims[0] == 1 ? 0u : oc};
        acc += U(ACC(loadInt(bias, cb)));
        storeInt(out, idx, int64_t(ACC(acc)));
    }
}

// ---- FFT2D: fft2d.comp:17-55, RFFT2D: rfft2d.comp:12-71 ------------------------------------------------------
// Both shaders evaluate the defining double sum directly, one output element per invocation; so does this
// kernel.  The angle of a term is 2*pi*(iy*oy/H + ix*ox/W); its numerator is reduced modulo H*W in integers (as
// rfft2d.comp:44-49 does) so that sine and cosine are taken of an angle in [0, 2*pi) at full precision, and the
// sums are kept in double (fft2d.comp accumulates in DOUBLE; rfft2d.comp compensates its float sum).  RFFT2D
// writes an exact zero for the imaginary part of the four self-conjugate bins (rfft2d.comp:33-38).
// imag.ptr == nullptr: real input, outputs hold W / 2 + 1 columns.
__global__ void fft2dKernel(TView real, TView imag, TView outReal, TView outImag, int32_t inverse) {
    const int64_t total = numelOf(outReal);
    const uint32_t H = real.dims[1], W = real.dims[2];
    const bool realOnly = imag.ptr == nullptr;
    GRID_STRIDE(e, total) {
        uint32_t idx[kMaxRank] = {0, 0, 0, 0, 0, 0};
        unravel(outReal, uint32_t(e), idx);
        const uint32_t n = idx[0], oy = idx[1], ox = idx[2];
        const bool skipImag = realOnly && (oy == 0 || oy == H / 2) && (ox == 0 || ox == W / 2);
        double sumRe = 0.0, sumIm = 0.0;
        for (uint32_t iy = 0; iy < H; ++iy) {
            const uint64_t rowTerm = uint64_t((uint64_t(iy) * oy) % H) * W;
            for (uint32_t ix = 0; ix < W; ++ix) {
                const uint32_t ci[3] = {n, iy, ix};
                const int64_t ro = offsetOf(real, ci);
                const double re = ro < 0 ? 0.0 : double(*reinterpret_cast<const float *>(real.ptr + ro));
                double im = 0.0;
                if (!realOnly) {
                    const int64_t io = offsetOf(imag, ci);
                    im = io < 0 ? 0.0 : double(*reinterpret_cast<const float *>(imag.ptr + io));
                }
                const uint64_t num = (rowTerm + uint64_t((uint64_t(ix) * ox) % W) * H) % (uint64_t(H) * W);
                double sn, cs;
                sincospi(2.0 * double(num) / double(uint64_t(H) * W), &sn, &cs);
                if (inverse) {
                    sn = -sn;
                }
                sumRe += re * cs + im * sn;
                sumIm += im * cs - re * sn;
            }
        }
        const int64_t orOff = offsetOf(outReal, idx), oiOff = offsetOf(outImag, idx);
        if (orOff >= 0) {
            *reinterpret_cast<float *>(outReal.ptr + orOff) = float(sumRe);
        }
        if (oiOff >= 0) {
            *reinterpret_cast<float *>(outImag.ptr + oiOff) = skipImag ? 0.0f : float(sumIm);
        }
    }
}

} // namespace

#define LAUNCH_1D(kernel, total, stream, ...) kernel<<<gridFor(total), kThreads, 0, stream>>>(__VA_ARGS__)

int indexArgmax(const TView &in, const TView &out, uint32_t axis, cudaStream_t s) {
    LAUNCH_1D(argmaxKernel, numelOf(out), s, in, out, axis);
    return finish("ARGMAX");
}

int indexGather(const TView &values, const TView &indices, const TView &out, cudaStream_t s) {
    LAUNCH_1D(gatherKernel, numelOf(out), s, values, indices, out);
    return finish("GATHER");
}

int indexScatter(const TView &valuesIn, const TView &indices, const TView &input, const TView &out, cudaStream_t s) {
    LAUNCH_1D(scatterKernel, numelOf(out), s, valuesIn, indices, input, out);
    return finish("SCATTER");
}

int indexReverse(const TView &in, const TView &out, uint32_t axis, cudaStream_t s) {
    LAUNCH_1D(reverseKernel, numelOf(out), s, in, out, axis);
    return finish("REVERSE");
}

int indexTile(const TView &in, const TView &out, cudaStream_t s) {
    LAUNCH_1D(tileKernel, numelOf(out), s, in, out);
    return finish("TILE");
}

int resizeInteger(const TView &in, const TView &out, const ResizeAttr &a, cudaStream_t s) {
    const int64_t total = numelOf(out);
    switch (out.dtype) {
    case MLEL_I8:
        LAUNCH_1D(resizeKernel<int8_t>, total, s, in, out, a);
        break;
    case MLEL_I16:
        LAUNCH_1D(resizeKernel<int16_t>, total, s, in, out, a);
        break;
    case MLEL_I32:
        LAUNCH_1D(resizeKernel<int32_t>, total, s, in, out, a);
        break;
    case MLEL_I64:
        LAUNCH_1D(resizeKernel<int64_t>, total, s, in, out, a);
        break;
    default:
        setLastError("RESIZE: unsupported output type");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    return finish("RESIZE");
}

int transposeConv2d(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                    cudaStream_t s) {
    const int64_t total = numelOf(out);
    if (out.dtype == MLEL_I32) {
        LAUNCH_1D(transposeConv2dKernel<int32_t>, total, s, in, w, bias, out, a);
    } else if (out.dtype == MLEL_I64) {
        LAUNCH_1D(transposeConv2dKernel<int64_t>, total, s, in, w, bias, out, a);
    } else {
        setLastError("TRANSPOSE_CONV2D: unsupported output type");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    return finish("TRANSPOSE_CONV2D");
}

int fft2d(const TView *real, const TView *imag, const TView &outReal, const TView &outImag, bool inverse,
          cudaStream_t s) {
    if (uint64_t(real->dims[1]) * real->dims[2] >= (uint64_t(1) << 31)) {
        setLastError("FFT2D: more than 2^31 points per image");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    TView none{};
    // one output element per thread, each a sum over the whole image: small blocks spread the work over all SMs
    const int64_t total = numelOf(outReal);
    const int threads = 64;
    const int64_t blocks = (total + threads - 1) / threads;
    fft2dKernel<<<unsigned(blocks < 1 ? 1 : (blocks > 148 * 64 ? 148 * 64 : blocks)), threads, 0, s>>>(
        *real, imag != nullptr ? *imag : none, outReal, outImag, inverse ? 1 : 0);
    return finish(imag != nullptr ? "FFT2D" : "RFFT2D");
}

int conv3d(const TView &in, const TView &w, const TView &bias, const TView &out, const Conv3dAttr &a, cudaStream_t s) {
    const int64_t total = numelOf(out);
    if (out.dtype == MLEL_I32) {
        LAUNCH_1D(conv3dKernel<int32_t>, total, s, in, w, bias, out, a);
    } else if (out.dtype == MLEL_I64) {
        LAUNCH_1D(conv3dKernel<int64_t>, total, s, in, w, bias, out, a);
    } else {
        setLastError("CONV3D: unsupported output type");
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    }
    return finish("CONV3D");
}

} // namespace mlel
