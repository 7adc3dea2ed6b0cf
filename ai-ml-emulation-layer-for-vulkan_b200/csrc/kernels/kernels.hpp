// Launchers of the CUDA kernels, grouped by file.  All return 0 or a negative mlel_status.
#pragma once

#include <cuda_runtime.h>

#include "../ops.hpp"

namespace mlel {

struct MoveAttr {
    int32_t kind;
    uint32_t v[kMaxRank]; // perms / (axis, offset) / start
    int64_t padBits;
};

// Device form of a fused RESCALE (+CLAMP) stage: rescale.comp:27-72 applied in registers.
struct DevRescale {
    const int32_t *mult; // [C] or [1]
    const int8_t *shift; // [C] or [1]
    int32_t inZp;        // narrowed to the stage's input type
    int32_t outZp;       // narrowed to the stage's output type
    int32_t lo, hi;      // output range (type range intersected with a following CLAMP)
    int32_t perChannel;
    int32_t doubleRound; // scale32 && double_round
};

struct DevEpilogue {
    int32_t hasMain;
    DevRescale main;
    int32_t hasResidual;
    const int8_t *shortcut; // packed, same shape as the output
    DevRescale a, b, out;   // a: main path, b: shortcut, out: after the ADD
};

// fused_generic.cu: one-thread-per-output fused kernels (always-correct path of the fused kinds)
int fusedConv2dGeneric(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                       const DevEpilogue &epi, cudaStream_t s);
int fusedDepthwiseGeneric(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                          const DevEpilogue &epi, cudaStream_t s);
// 3x3 depthwise convolution of packed int8 NHWC tensors with channel multiplier 1; epi == nullptr: int32 output
bool depthwise3x3Eligible(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                          bool fused);
int depthwise3x3(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                 const DevEpilogue *epi, cudaStream_t s);
int fusedMatmulGeneric(const TView &a, const TView &b, const TView &out, int32_t zpA, int32_t zpB,
                       const DevEpilogue &epi, cudaStream_t s);
// out[i] = clamp(rescale_out(rescale_a(x[i]) + rescale_b(y[i]))), all tensors packed int8 of n elements
int fusedAdd(const int8_t *x, const int8_t *y, int8_t *out, int64_t n, const DevEpilogue &epi, cudaStream_t s);

// fast_ops.cu: vectorised kernels for packed int8 NHWC tensors
int padImageI8(const int8_t *in, int8_t *out, int N, int H, int W, int C, int Hp, int Wp, int Cp, int padTop, int padLeft,
               cudaStream_t s);
// bt[n][w][c] = b[n][c][w]; corr[n][w] = -za * sum_c b[n][c][w] (mod 2^32).  C and W multiples of 16.
int transposeForMatmul(const int8_t *b, int8_t *bt, int32_t *corr, int batches, int C, int W, int32_t za, cudaStream_t s);
// corr[n][w] = -za * sum_c b[n][c][w] (mod 2^32) alone, for the kernel that reads b where it lies.  W a multiple of 16.
int columnSumsForMatmul(const int8_t *b, int32_t *corr, int batches, int C, int W, int32_t za, cudaStream_t s);
bool maxPoolI8Eligible(const TView &in, const TView &out);
// packed int8 NHWC tensors (same conditions as maxPoolI8Eligible) with a window of at least 16 taps
bool avgPoolI8Eligible(const TView &in, const TView &out, const PoolAttr &a);
int avgPoolI8(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s);
int maxPoolI8(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s);

// vector_ops.cu: vectorised kernels for packed tensors.  Each returns false when it does not apply (the caller
// then runs the generic kernel); otherwise *rc is the launch status.
bool vecRescale(const TView &in, const TView &out, const TView &mult, const TView &shift, const RescaleAttr &a, cudaStream_t s,
                int *rc);
bool vecTable(const TView &in, const TView &out, const TView &table, cudaStream_t s, int *rc);
// op: BIN_ADD or BIN_SUB, or -1 for MUL with `shift`
// A fused run of row-wise operators (OP_FUSED_ROWS): row_machine.cu.  rowMachineWarps tells how many rows a block can
// hold at once for `slots` full-shaped values of `len` elements (0: the run cannot be fused).
int rowMachineWarps(int slots, int len);
int rowMachine(const RowProgram &program, const TView *tensors, cudaStream_t s);
// Fused nodes of the fusion pass (OP_FUSED_ROW_EXP, OP_FUSED_MUL_RESCALE): see vector_ops.cu.
int rowExpFused(const TView &x, const TView &table, const TView &e, const TView &sums, const DevRescale &r, cudaStream_t s);
int mulRescaleFused(const TView &a, const TView &b, const TView &out, uint32_t shift, const DevRescale &r, cudaStream_t s);
bool vecBinaryI32(int32_t op, const TView &a, const TView &b, const TView &out, uint32_t shift, cudaStream_t s, int *rc);
bool vecClampI8(const TView &in, const TView &out, int64_t lo, int64_t hi, cudaStream_t s, int *rc);
bool vecRowReduce(int32_t op, const TView &in, const TView &out, uint32_t axis, cudaStream_t s, int *rc);
bool vecTransposeRows(const TView &in, const TView &out, const uint32_t *perms, cudaStream_t s, int *rc);
// one-byte elements, the input's last axis becomes the output's second-to-last and another axis its last
bool vecTransposeLast2Bytes(const TView &in, const TView &out, const uint32_t *perms, cudaStream_t s, int *rc);

// Joins column blocks of byte rows: out[row][first[g] + j] = staging[(g * rows + row) * pitch + j], j < count[g].
// The blocks follow one another (first[0] = 0, first[g + 1] = first[g] + count[g]); at most kMaxColumnBlocks.
constexpr int kMaxColumnBlocks = 64;
int interleaveColumns(const void *staging, void *out, int64_t rows, int32_t blocks, int32_t pitch, const int32_t *first,
                      const int32_t *count, cudaStream_t s);

// generic_ops.cu
int genericConv2d(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                  cudaStream_t s);
int genericDepthwise(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                     cudaStream_t s);
int genericMatmul(const TView &a, const TView &b, const TView &out, int32_t zpA, int32_t zpB, cudaStream_t s);
int genericRescale(const TView &in, const TView &out, const TView &mult, const TView &shift, const RescaleAttr &a,
                   cudaStream_t s);
int genericAvgPool(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s);
int genericMaxPool(const TView &in, const TView &out, const PoolAttr &a, cudaStream_t s);
int genericTable(const TView &in, const TView &out, const TView &table, cudaStream_t s);
int genericTranspose(const TView &in, const TView &out, const uint32_t *perms, cudaStream_t s);
int genericConcat(const TView &in, const TView &out, uint32_t axis, uint32_t offset, cudaStream_t s);
int genericReshape(const TView &in, const TView &out, cudaStream_t s);
int genericSlice(const TView &in, const TView &out, const uint32_t *start, cudaStream_t s);
int genericPad(const TView &in, const TView &out, const TView &padding, int64_t padBits, cudaStream_t s);
int genericClamp(const TView &in, const TView &out, double minV, double maxV, cudaStream_t s);
int genericBinary(int32_t op, const TView &a, const TView &b, const TView &out, cudaStream_t s);
int genericMul(const TView &a, const TView &b, const TView &out, uint32_t shift, cudaStream_t s);
int genericReduce(int32_t op, const TView &in, const TView &out, uint32_t axis, cudaStream_t s);
int genericCast(const TView &in, const TView &out, cudaStream_t s);
int genericArShift(const TView &a, const TView &b, const TView &out, int32_t round, cudaStream_t s);
int genericNegate(const TView &in, const TView &out, int32_t inZp, int32_t outZp, cudaStream_t s);
int genericSelect(const TView &c, const TView &a, const TView &b, const TView &out, cudaStream_t s);
int genericUnary(int32_t op, const TView &in, const TView &out, cudaStream_t s);

// index_ops.cu: ARGMAX, GATHER, SCATTER, REVERSE, TILE, integer RESIZE, TRANSPOSE_CONV2D, CONV3D
int indexArgmax(const TView &in, const TView &out, uint32_t axis, cudaStream_t s);
int indexGather(const TView &values, const TView &indices, const TView &out, cudaStream_t s);
int indexScatter(const TView &valuesIn, const TView &indices, const TView &input, const TView &out, cudaStream_t s);
int indexReverse(const TView &in, const TView &out, uint32_t axis, cudaStream_t s);
int indexTile(const TView &in, const TView &out, cudaStream_t s);
int resizeInteger(const TView &in, const TView &out, const ResizeAttr &a, cudaStream_t s);
int transposeConv2d(const TView &in, const TView &w, const TView &bias, const TView &out, const ConvAttr &a,
                    cudaStream_t s);
// FFT2D (imag != nullptr) and RFFT2D (imag == nullptr, outputs hold W / 2 + 1 columns): direct sums in double
int fft2d(const TView *real, const TView *imag, const TView &outReal, const TView &outImag, bool inverse,
          cudaStream_t s);
int conv3d(const TView &in, const TView &w, const TView &bias, const TView &out, const Conv3dAttr &a, cudaStream_t s);

// int8_mma_peak.cu: back-to-back tcgen05.mma kind::i8 on shared-memory operands, every SM: device time and the
// int8 operations it stands for
int int8MmaPeak(int batches, cudaStream_t stream, float *msOut, double *opsOut);

} // namespace mlel
