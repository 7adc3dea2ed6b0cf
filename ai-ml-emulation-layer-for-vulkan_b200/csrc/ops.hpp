// Operator descriptors shared by the graph layer (host) and the kernel launchers.
//
// One OpDesc is what one GraphPipeline::make<Op> call of the reference records
// (graph/compute_graph_op.hpp:1249-1483): the operator kind, its attributes (the reference's
// push constants / specialisation constants) and its tensor operands.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../../include/mlel_b200.h"

struct CUstream_st;
using cudaStream_t = CUstream_st *;

namespace mlel {

constexpr int kMaxRank = MLEL_MAX_RANK;

// Device-visible view of a tensor: address, element type, shape and byte strides.
struct TView {
    char *ptr;
    int32_t dtype;
    int32_t rank;
    uint32_t dims[kMaxRank];
    int64_t strides[kMaxRank];
};

enum OpKind : int32_t {
    OP_CONV2D = 0,
    OP_DEPTHWISE_CONV2D,
    OP_MATMUL,
    OP_RESCALE,
    OP_AVG_POOL2D,
    OP_MAX_POOL2D,
    OP_TABLE,
    OP_TRANSPOSE,
    OP_CONCAT,
    OP_CLAMP,
    OP_BINARY,
    OP_UNARY,
    OP_MUL,
    OP_REDUCE,
    OP_CAST,
    OP_RESHAPE,
    OP_SLICE,
    OP_PAD,
    OP_ARITHMETIC_RIGHT_SHIFT,
    OP_NEGATE,
    OP_SELECT,
    OP_ARGMAX,
    OP_GATHER,
    OP_SCATTER,
    OP_REVERSE,
    OP_TILE,
    OP_RESIZE,
    OP_TRANSPOSE_CONV2D,
    OP_CONV3D,
    OP_FFT2D,  // in = {real, imag}, out = {real, imag}
    OP_RFFT2D, // in = {real},       out = {real, imag}
    // Produced only by the fusion pass:
    OP_FUSED_CONV2D,     // CONV2D -> RESCALE [-> CLAMP] [-> residual RESCALE/ADD/RESCALE [-> CLAMP]]
    OP_FUSED_DEPTHWISE,  // DEPTHWISE_CONV2D -> RESCALE [-> CLAMP]
    OP_FUSED_MATMUL,     // MATMUL -> RESCALE [-> CLAMP]
    OP_FUSED_ADD,        // RESCALE(a), RESCALE(b) -> ADD -> RESCALE [-> CLAMP]
    // Row-wise exponentials of a quantised softmax: REDUCE_MAX(x) -> SUB(x, max) -> RESCALE -> TABLE, and the
    // REDUCE_SUM of the TABLE's output.  in = {x, table}, out = {table output, row sums}; epi.main is the RESCALE.
    OP_FUSED_ROW_EXP,
    // MUL(a, b, shift) -> RESCALE [-> CLAMP] on int32 operands (b: same shape, one value per row, or one value).
    // in = {a, b}, i[0] = shift, epi.main is the RESCALE.
    OP_FUSED_MUL_RESCALE,
    // A contiguous run of row-wise integer operators (RESCALE, TABLE, ADD, SUB, MUL, last-axis REDUCE, CLAMP) as one
    // kernel: see RowProgram.  in = every tensor read from memory (tables included), out = every tensor written.
    OP_FUSED_ROWS,
    OP_KIND_COUNT
};

enum BinaryOp : int32_t {
    BIN_ADD = 0,
    BIN_SUB,
    BIN_BITWISE_AND,
    BIN_BITWISE_OR,
    BIN_BITWISE_XOR,
    BIN_LOGICAL_AND,
    BIN_LOGICAL_OR,
    BIN_LOGICAL_XOR,
    BIN_LOGICAL_LEFT_SHIFT,
    BIN_LOGICAL_RIGHT_SHIFT,
    BIN_INTDIV,
    BIN_MAXIMUM,
    BIN_MINIMUM,
    BIN_EQUAL,
    BIN_GREATER,
    BIN_GREATER_EQUAL,
    BIN_POW, // fp32 only
    BIN_COUNT
};

enum UnaryOp : int32_t {
    UN_ABS = 0,
    UN_BITWISE_NOT,
    UN_CLZ,
    UN_LOGICAL_NOT,
    // fp32 only from here on
    UN_CEIL,
    UN_COS,
    UN_ERF,
    UN_EXP,
    UN_FLOOR,
    UN_LOG,
    UN_RECIPROCAL,
    UN_RSQRT,
    UN_SIGMOID,
    UN_SIN,
    UN_TANH,
    UN_COUNT
};
enum ReduceOp : int32_t { RED_SUM = 0, RED_MAX, RED_MIN, RED_PRODUCT, RED_ALL, RED_ANY, RED_COUNT };

// CONV2D / DEPTHWISE_CONV2D attributes (the push constants of conv2d.comp:26-33).
struct ConvAttr {
    int32_t pad[4];      // top, bottom, left, right
    int32_t stride[2];   // y, x
    int32_t dilation[2]; // y, x
    int32_t inZp;
    int32_t wZp;
};

// CONV3D attributes (the push constants of conv3d.comp:17-23).
struct Conv3dAttr {
    int32_t pad[6];      // front, back, top, bottom, left, right
    int32_t stride[3];   // d, y, x
    int32_t dilation[3]; // d, y, x
    int32_t inZp;
    int32_t wZp;
};

// RESIZE attributes (resize.comp:16-39).
struct ResizeAttr {
    int32_t scale[4];  // y numerator, y denominator, x numerator, x denominator
    int32_t offset[2]; // y, x
    int32_t border[2]; // y, x
    int32_t mode;      // 1 = NEAREST, 2 = BILINEAR
};

// RESCALE attributes (rescale.comp:11-19).
struct RescaleAttr {
    int32_t inZp;
    int32_t outZp;
    int32_t scale32;
    int32_t doubleRound;
    int32_t perChannel;
};

// AVG_POOL2D / MAX_POOL2D attributes (avgpool2d.comp:14-20).
struct PoolAttr {
    int32_t kernel[2];
    int32_t stride[2];
    int32_t pad[4];
    int32_t inZp;
    int32_t outZp;
};

// One RESCALE (optionally followed by a CLAMP) folded into another kernel.  Host form: the
// multiplier/shift are tensor ids; the session turns them into device pointers.
struct FusedRescale {
    int32_t multTensor{-1};
    int32_t shiftTensor{-1};
    int32_t inDtype{MLEL_I32};
    int32_t outDtype{MLEL_I8};
    RescaleAttr attr{};
    int32_t lo{-128}, hi{127}; // output range after the optional CLAMP
};

// What the fusion pass attaches to a contraction:
//   y   = clamp(rescale_main(acc))                                   -- CONV/MATMUL -> RESCALE [-> CLAMP]
//   out = clamp(rescale_out(rescale_a(y) + rescale_b(shortcut)))     -- optional residual tail
struct FusedEpilogue {
    bool hasMain{false};
    FusedRescale main;
    bool hasResidual{false};
    bool mainIsFirst{true}; // ADD(main, shortcut) or ADD(shortcut, main)
    int32_t shortcutTensor{-1};
    FusedRescale a, b, out;
};

// A run of row-wise integer operators fused into one kernel (OP_FUSED_ROWS): every tensor of the run has the run's
// full shape [..., L], the same shape with a last dimension of 1 (one value per row) or one element.  A warp owns
// a row, keeps the full-shaped values in shared-memory slots and the per-row values in a few words beside them, and
// executes the instructions in order, each with the arithmetic of the operator's own kernel.
enum RowOpcode : int32_t {
    ROW_LOAD = 0,   // dst <- tensor (full: a row of `dtype` elements; per-row value: element `row`)
    ROW_STORE,      // tensor <- a
    ROW_RESCALE,    // p = {mult, shift, inZp, outZp, lo, hi, doubleRound}
    ROW_TABLE8,     // int8 -> int8 by 256 entries
    ROW_TABLE16,    // int16 -> int32 by 513 entries with interpolation
    ROW_ADD,
    ROW_SUB,
    ROW_MUL,        // p[0] = shift
    ROW_REDUCE_SUM, // full -> per-row value
    ROW_REDUCE_MAX,
    ROW_REDUCE_MIN,
    ROW_CLAMP,      // p = {lo, hi}
};
enum RowOperandKind : int32_t { ROW_NONE = 0, ROW_FULL, ROW_VALUE, ROW_IMMEDIATE };
struct RowOperand {
    int32_t kind{ROW_NONE};
    int32_t index{0}; // slot (ROW_FULL) or per-row word (ROW_VALUE)
    int32_t imm{0};   // ROW_IMMEDIATE
};
struct RowInst {
    int32_t op{ROW_LOAD};
    RowOperand dst, a, b;
    int32_t tensor{-1}; // LOAD / STORE: the tensor; TABLE: the table
    int32_t dtype{MLEL_I32};
    int32_t p[7]{};
};
struct RowProgram {
    std::vector<RowInst> insts;
    int32_t slots{0}, values{0};
    int64_t rows{0};
    int32_t len{0};
};
constexpr int kMaxRowInsts = 40, kMaxRowValues = 16;

struct OpDesc {
    OpKind kind{OP_CAST};
    int32_t sub{0};          // BinaryOp / UnaryOp / ReduceOp
    int32_t i[24]{};         // integer attributes (layout per kind: see graph_pipeline.cpp)
    double d[2]{};           // CLAMP bounds / PAD constant
    std::string name;        // debug name ("CONV2D", ...), as logged by the reference
    std::vector<int32_t> in; // tensor ids: data inputs, then attribute tensors
    std::vector<int32_t> out;
    FusedEpilogue epi;              // fused kinds only
    std::vector<int32_t> fusedOps;  // indices of the logical ops an exec node stands for
    std::shared_ptr<RowProgram> rows; // OP_FUSED_ROWS only
    // Tensor-core path (set by GraphPipeline::prepareTensorCore when the node qualifies):
    //   CONV2D kinds: aux[0] correction table int32 [classes][OC], aux[1] row classes u8 [OH],
    //                 aux[2] column classes u8 [OW]; auxi[0] = number of column classes, auxi[1] = classes,
    //                 auxi[3] = the most common class, auxi[4] = 1 when every correction is below 2^30 - 256 in size,
    //                 2 when correction + raw sum stay below 2^29
    //                 with a fused residual tail and tc == 1: aux[3] = the tail as a table of 256 x 256 bytes
    //   MATMUL kinds with a constant second input: aux[0] correction int32 [batches][W],
    //                 aux[3] the second input transposed to [batches][W][C]
    //   CONV2D kinds with tc == 2 (channel count not a multiple of 16): scratch = session tensor
    //                 [N][Hp][Wp][ICp], a copy of the input with zero-padded channels and borders;
    //                 aux[3] weights re-laid to the gather's K order [OC][kPad]; aux[4] int32 byte offset
    //                 of every gathered piece from a pixel's window origin; auxi[2] = bytes per piece
    int32_t tc{0};
    int32_t scratch{-1};
    int32_t aux[5]{-1, -1, -1, -1, -1};
    int32_t auxi[5]{0, 0, 0, 0, 0};
};

// Launches one operator.  `tensors` is indexed by tensor id (op.in / op.out / op.epi hold ids).
// Returns 0 or a negative mlel_status and sets the thread's last-error message.
struct LaunchChain; // kernels/gemm_i8_tcgen05.hpp: tile-level hand-over between consecutive tensor-core launches
int launchOp(const OpDesc &op, const TView *tensors, cudaStream_t stream, LaunchChain *chain = nullptr);

void setLastError(const std::string &msg);
int elemSize(int32_t dtype);

} // namespace mlel
