// GraphPipeline: operator recording, validation, fusion and constant upload.
//
// Attribute layout of OpDesc::i per kind (the reference keeps these in per-op push-constant
// structs, graph/compute_graph_op.hpp):
//   CONV2D, DEPTHWISE_CONV2D  i[0..3] pad(top,bottom,left,right) i[4..5] stride i[6..7] dilation
//                             i[8] inputZeroPoint i[9] weightZeroPoint i[10] accType
//                             in = {input, weights, biases}
//   MATMUL                    i[0] zeroPoint1 i[1] zeroPoint2            in = {input1, input2}
//   RESCALE                   i[0] inputZeroPoint i[1] outputZeroPoint i[2] scale32 i[3] doubleRound
//                             i[4] perChannel i[5] inputUnsigned i[6] outputUnsigned
//                             in = {input, multiplier, shift}
//   AVG_POOL2D                i[0..1] kernel i[2..3] stride i[4..7] pad i[8] inZp i[9] outZp i[10] accType
//   MAX_POOL2D                i[0..1] kernel i[2..3] stride i[4..7] pad i[8] nanMode
//   TABLE                     in = {input, table}
//   TRANSPOSE                 i[0..rank-1] perms
//   CONCAT                    i[0] axis i[1] offset      (one op per input, compute_graph_op.cpp:2607-2615)
//   CLAMP                     d[0] min d[1] max i[0] nanMode
//   BINARY / UNARY / REDUCE   sub = operator; BINARY i[0] nanMode; REDUCE i[0] axis i[1] nanMode
//   MUL                       i[0] shift
//   SLICE                     i[0..rank-1] start
//   PAD                       d[0] padConst i[0] padConstInt    in = {input, padding}
//   ARITHMETIC_RIGHT_SHIFT    i[0] round
//   NEGATE                    i[0] inputZeroPoint i[1] outputZeroPoint
//   SELECT                    in = {condition, input2, input3}
//   ARGMAX                    i[0] axis i[1] nanMode
//   FFT2D                     i[0] inverse     in = {real, imag}  out = {real, imag}
//   RFFT2D                    in = {input}     out = {real, imag}
//   GATHER                    in = {values, indices}
//   SCATTER                   in = {values_in, indices, input}
//   REVERSE                   i[0] axis
//   RESIZE                    i[0..3] scale (y_n, y_d, x_n, x_d) i[4..5] offset i[6..7] border i[8] mode
//   TRANSPOSE_CONV2D          i[0..3] out_pad i[4..5] stride i[8] inputZeroPoint i[9] weightZeroPoint i[10] accType
//                             in = {input, weights, biases}
//   CONV3D                    i[0..5] pad i[6..8] stride i[9..11] dilation i[12] inputZeroPoint
//                             i[13] weightZeroPoint i[14] accType      in = {input, weights, biases}
#include "graph_pipeline.hpp"
#include "kernels/device_common.cuh"
#include "kernels/gemm_i8_tcgen05.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <map>
#include <functional>
#include <cstring>
#include <queue>
#include <set>

namespace mlel {

int elemSize(int32_t dtype) {
    switch (dtype) {
    case MLEL_BOOL:
    case MLEL_I8:
    case MLEL_U8:
        return 1;
    case MLEL_I16:
    case MLEL_U16:
    case MLEL_F16:
    case MLEL_BF16:
        return 2;
    case MLEL_I32:
    case MLEL_U32:
    case MLEL_F32:
        return 4;
    case MLEL_I64:
        return 8;
    default:
        return 0;
    }
}

int64_t TensorDescriptor::numel() const {
    int64_t n = 1;
    for (auto d : dims) {
        n *= d;
    }
    return n;
}

uint64_t TensorDescriptor::sizeBytes() const {
    if (dims.empty()) {
        return uint64_t(elemSize(dtype));
    }
    return uint64_t(dims[0]) * uint64_t(strides[0]);
}

bool TensorDescriptor::packed() const {
    int64_t s = elemSize(dtype);
    for (int i = rank() - 1; i >= 0; --i) {
        if (strides[size_t(i)] != s) {
            return false;
        }
        s *= dims[size_t(i)];
    }
    return true;
}

namespace {

std::vector<int64_t> packedStrides(int32_t dtype, const std::vector<int64_t> &dims) {
    // tensor/tensor_arm.cpp:82-92
    std::vector<int64_t> strides(dims.size());
    if (dims.empty()) {
        return strides;
    }
    strides.back() = elemSize(dtype);
    for (size_t i = dims.size() - 1; i > 0; --i) {
        strides[i - 1] = strides[i] * dims[i];
    }
    return strides;
}

std::unique_ptr<TensorDescriptor> fromDesc(const mlel_tensor_desc &desc) {
    if (desc.rank <= 0 || desc.rank > kMaxRank) {
        throw std::runtime_error("Tensor dimension count not supported: " + std::to_string(desc.rank));
    }
    if (elemSize(desc.dtype) == 0) {
        throw UnsupportedError("Unsupported tensor buffer format: " + std::to_string(desc.dtype));
    }
    auto t = std::make_unique<TensorDescriptor>();
    t->dtype = desc.dtype;
    t->dims.assign(desc.dims, desc.dims + desc.rank);
    for (auto d : t->dims) {
        if (d <= 0) {
            throw std::runtime_error("Tensor dimensions must be greater than zero");
        }
    }
    if (desc.strides[0] == 0) {
        t->strides = packedStrides(desc.dtype, t->dims);
    } else {
        t->strides.assign(desc.strides, desc.strides + desc.rank);
        if (t->strides[0] < 0) {
            throw std::runtime_error("Strides must be greater than zero."); // graph/tensor.cpp:194-196
        }
    }
    // Element counts are 32-bit in the reference's dispatch (graph/compute_graph_op.cpp:554).
    if (t->numel() >= (int64_t(1) << 32)) {
        throw UnsupportedError("Tensors with 2^32 or more elements are not supported");
    }
    return t;
}

bool isIntegerType(int32_t dt) { return dt >= MLEL_BOOL && dt <= MLEL_U32; }

} // namespace

int32_t GraphPipeline::addTensor(std::unique_ptr<TensorDescriptor> t) {
    t->id = int32_t(tensors_.size());
    tensors_.push_back(std::move(t));
    return tensors_.back()->id;
}

void GraphPipeline::requireMutable() const {
    if (finalized_) {
        throw std::runtime_error("pipeline is immutable once a session exists");
    }
}

int32_t GraphPipeline::makeConstTensor(uint32_t id, const mlel_tensor_desc &desc, const void *data) {
    requireMutable();
    auto t = fromDesc(desc);
    t->cls = TensorClass::Constant;
    if (data == nullptr) {
        throw std::runtime_error("constant tensor without data");
    }
    const auto *bytes = static_cast<const uint8_t *>(data);
    t->hostData.assign(bytes, bytes + t->sizeBytes()); // constants are copied at create time
    const int32_t tid = addTensor(std::move(t));
    constTensorMap_[id] = tid;
    return tid;
}

int32_t GraphPipeline::getConstTensor(uint32_t id) const { return constTensorMap_.at(id); }

int32_t GraphPipeline::makeConstCompositeTensor(int32_t dtype, const std::vector<int64_t> &dims, const void *data) {
    requireMutable();
    mlel_tensor_desc desc{};
    desc.dtype = dtype;
    desc.rank = int32_t(dims.size());
    for (size_t i = 0; i < dims.size(); ++i) {
        desc.dims[i] = dims[i];
    }
    auto t = fromDesc(desc);
    t->cls = TensorClass::Constant;
    const auto *bytes = static_cast<const uint8_t *>(data);
    t->hostData.assign(bytes, bytes + t->sizeBytes());
    return addTensor(std::move(t));
}

int32_t GraphPipeline::makeDescriptorSetBinding(uint32_t set, uint32_t binding, uint32_t arrayIndex,
                                                const mlel_tensor_desc &desc) {
    requireMutable();
    auto t = fromDesc(desc);
    t->cls = TensorClass::External;
    t->set = set;
    t->binding = binding;
    t->arrayIndex = arrayIndex;
    const int32_t tid = addTensor(std::move(t));
    externalMap_[std::make_tuple(set, binding, arrayIndex)] = tid;
    return tid;
}

int32_t GraphPipeline::getTensor(uint32_t set, uint32_t binding, uint32_t arrayIndex) const {
    return externalMap_.at(std::make_tuple(set, binding, arrayIndex));
}

int32_t GraphPipeline::makeTensor(int32_t dtype, const std::vector<int64_t> &dims,
                                  const std::vector<int64_t> &strides) {
    requireMutable();
    mlel_tensor_desc desc{};
    desc.dtype = dtype;
    desc.rank = int32_t(dims.size());
    for (size_t i = 0; i < dims.size(); ++i) {
        desc.dims[i] = dims[i];
        desc.strides[i] = strides.empty() ? 0 : strides[i];
    }
    auto t = fromDesc(desc);
    t->cls = TensorClass::Session;
    t->sessionOrder = int32_t(sessionTensors_.size());
    const int32_t tid = addTensor(std::move(t));
    sessionTensors_.push_back(tid);
    return tid;
}

void GraphPipeline::makeInput(int32_t t) {
    requireMutable();
    tensor(t).isGraphInput = true;
    inputs_.push_back(t);
}

void GraphPipeline::makeOutput(int32_t t) {
    requireMutable();
    tensor(t).isGraphOutput = true;
    outputs_.push_back(t);
}

OpDesc &GraphPipeline::pushOp(OpKind kind, const std::string &name, std::vector<int32_t> in,
                              std::vector<int32_t> out) {
    requireMutable();
    for (auto t : in) {
        (void)tensor(t);
    }
    for (auto t : out) {
        if (tensor(t).cls == TensorClass::Constant) {
            throw std::runtime_error(name + ": a constant tensor cannot be an operator output");
        }
    }
    OpDesc op;
    op.kind = kind;
    op.name = name;
    op.in = std::move(in);
    op.out = std::move(out);
    ops_.push_back(std::move(op));
    return ops_.back();
}

namespace {
void need(bool cond, const std::string &what) {
    if (!cond) {
        throw UnsupportedError(what);
    }
}
} // namespace

void GraphPipeline::makeConv2D(int32_t input, int32_t output, int32_t weights, int32_t biases,
                               const std::vector<int32_t> &pad, const std::vector<int32_t> &stride,
                               const std::vector<int32_t> &dilation, int8_t inputZeroPoint, int8_t weightZeroPoint,
                               uint32_t accType, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &w = tensor(weights), &b = tensor(biases);
    need(in.rank() == 4 && out.rank() == 4 && w.rank() == 4 && b.rank() == 1, debugName + ": rank mismatch");
    need(pad.size() == 4 && stride.size() == 2 && dilation.size() == 2, debugName + ": attribute size mismatch");
    // accType codes: 1 int32, 2 fp16, 3 fp32, 4 int64 (graph/compute_graph_op.cpp:39-67)
    need(accType == 1 || accType == 4, debugName + ": only integer accumulators are built (accType 1 or 4)");
    need((in.dtype == MLEL_I8 && out.dtype == MLEL_I32) || (in.dtype == MLEL_I16 && out.dtype == MLEL_I64),
         debugName + ": supported types are int8->int32 and int16->int64");
    need(w.dtype == MLEL_I8 && b.dtype == out.dtype, debugName + ": weights must be int8, bias of the output type");
    auto &op = pushOp(OP_CONV2D, debugName, {input, weights, biases}, {output});
    for (int k = 0; k < 4; ++k) {
        op.i[k] = pad[size_t(k)];
    }
    op.i[4] = stride[0], op.i[5] = stride[1], op.i[6] = dilation[0], op.i[7] = dilation[1];
    op.i[8] = inputZeroPoint, op.i[9] = weightZeroPoint, op.i[10] = int32_t(accType);
}

void GraphPipeline::makeDepthwiseConv2D(int32_t input, int32_t output, int32_t weights, int32_t biases,
                                        const std::vector<int32_t> &pad, const std::vector<int32_t> &stride,
                                        const std::vector<int32_t> &dilation, int8_t inputZeroPoint,
                                        int8_t weightZeroPoint, uint32_t accType, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &w = tensor(weights), &b = tensor(biases);
    need(in.rank() == 4 && out.rank() == 4 && w.rank() == 4 && b.rank() == 1, debugName + ": rank mismatch");
    need(pad.size() == 4 && stride.size() == 2 && dilation.size() == 2, debugName + ": attribute size mismatch");
    need(accType == 1 || accType == 4, debugName + ": only integer accumulators are built (accType 1 or 4)");
    need((in.dtype == MLEL_I8 && out.dtype == MLEL_I32) || (in.dtype == MLEL_I16 && out.dtype == MLEL_I64),
         debugName + ": supported types are int8->int32 and int16->int64");
    need(w.dtype == MLEL_I8 && b.dtype == out.dtype, debugName + ": weights must be int8, bias of the output type");
    auto &op = pushOp(OP_DEPTHWISE_CONV2D, debugName, {input, weights, biases}, {output});
    for (int k = 0; k < 4; ++k) {
        op.i[k] = pad[size_t(k)];
    }
    op.i[4] = stride[0], op.i[5] = stride[1], op.i[6] = dilation[0], op.i[7] = dilation[1];
    op.i[8] = inputZeroPoint, op.i[9] = weightZeroPoint, op.i[10] = int32_t(accType);
}

void GraphPipeline::makeMatmul(int32_t input1, int32_t input2, int32_t output, int32_t zp1, int32_t zp2,
                               const std::string &debugName) {
    const auto &a = tensor(input1), &b = tensor(input2), &out = tensor(output);
    need(a.rank() == 3 && b.rank() == 3 && out.rank() == 3, debugName + ": rank mismatch");
    need(a.dtype == b.dtype, debugName + ": input types differ");
    need((a.dtype == MLEL_I8 && out.dtype == MLEL_I32) || (a.dtype == MLEL_I16 && out.dtype == MLEL_I64),
         debugName + ": supported types are int8->int32 and int16->int64");
    auto &op = pushOp(OP_MATMUL, debugName, {input1, input2}, {output});
    op.i[0] = zp1, op.i[1] = zp2;
}

void GraphPipeline::makeRescale(int32_t input, int32_t output, int32_t inputZeroPoint, int32_t outputZeroPoint,
                                int32_t multiplier, int32_t shift, bool scale32, bool doubleRound, bool perChannel,
                                bool inputUnsigned, bool outputUnsigned, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &m = tensor(multiplier), &s = tensor(shift);
    // The reference's unsigned variants mix signed and unsigned operands in clamp(); their result
    // depends on GLSL overload resolution and no reference test pins it.
    need(!inputUnsigned && !outputUnsigned, debugName + ": unsigned RESCALE variants are not built");
    need(in.dtype == MLEL_I8 || in.dtype == MLEL_I16 || in.dtype == MLEL_I32, debugName + ": input type");
    need(out.dtype == MLEL_I8 || out.dtype == MLEL_I16 || out.dtype == MLEL_I32, debugName + ": output type");
    need((m.dtype == MLEL_I32 || m.dtype == MLEL_I16) && s.dtype == MLEL_I8, debugName + ": multiplier/shift type");
    need(m.rank() == 1 && s.rank() == 1, debugName + ": multiplier/shift must be rank 1");
    auto &op = pushOp(OP_RESCALE, debugName, {input, multiplier, shift}, {output});
    op.i[0] = inputZeroPoint, op.i[1] = outputZeroPoint, op.i[2] = scale32, op.i[3] = doubleRound;
    op.i[4] = perChannel, op.i[5] = inputUnsigned, op.i[6] = outputUnsigned;
}

void GraphPipeline::makeAvgPool2D(int32_t input, int32_t output, const std::vector<int32_t> &kernel,
                                  const std::vector<int32_t> &stride, const std::vector<int32_t> &pad,
                                  uint32_t accType, int8_t inputZeroPoint, int8_t outputZeroPoint,
                                  const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == 4 && out.rank() == 4, debugName + ": rank mismatch");
    need(kernel.size() == 2 && stride.size() == 2 && pad.size() == 4, debugName + ": attribute size mismatch");
    need(accType == 1 && (in.dtype == MLEL_I8 || in.dtype == MLEL_I16) && in.dtype == out.dtype,
         debugName + ": only int8/int16 with an int32 accumulator is built");
    auto &op = pushOp(OP_AVG_POOL2D, debugName, {input}, {output});
    op.i[0] = kernel[0], op.i[1] = kernel[1], op.i[2] = stride[0], op.i[3] = stride[1];
    for (int k = 0; k < 4; ++k) {
        op.i[4 + k] = pad[size_t(k)];
    }
    op.i[8] = inputZeroPoint, op.i[9] = outputZeroPoint, op.i[10] = int32_t(accType);
}

void GraphPipeline::makeMaxPool2D(int32_t input, int32_t output, const std::vector<int32_t> &kernel,
                                  const std::vector<int32_t> &stride, const std::vector<int32_t> &pad,
                                  uint32_t nanMode, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == 4 && out.rank() == 4, debugName + ": rank mismatch");
    need(kernel.size() == 2 && stride.size() == 2 && pad.size() == 4, debugName + ": attribute size mismatch");
    need((in.dtype == MLEL_I8 || in.dtype == MLEL_I16 || in.dtype == MLEL_I32) && in.dtype == out.dtype,
         debugName + ": only integer types are built");
    auto &op = pushOp(OP_MAX_POOL2D, debugName, {input}, {output});
    op.i[0] = kernel[0], op.i[1] = kernel[1], op.i[2] = stride[0], op.i[3] = stride[1];
    for (int k = 0; k < 4; ++k) {
        op.i[4 + k] = pad[size_t(k)];
    }
    op.i[8] = int32_t(nanMode);
}

void GraphPipeline::makeTable(int32_t input, int32_t output, int32_t table, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &t = tensor(table);
    need((in.dtype == MLEL_I8 && out.dtype == MLEL_I8) || (in.dtype == MLEL_I16 && out.dtype == MLEL_I32),
         debugName + ": supported types are int8->int8 and int16->int32");
    need(t.dtype == in.dtype && t.rank() == 1, debugName + ": table must be rank 1 of the input type");
    pushOp(OP_TABLE, debugName, {input, table}, {output});
}

void GraphPipeline::makeTranspose(int32_t input, int32_t output, const std::vector<uint32_t> &perms,
                                  const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == out.rank() && int(perms.size()) == in.rank(), debugName + ": rank mismatch");
    need(elemSize(in.dtype) == elemSize(out.dtype), debugName + ": element size mismatch");
    for (auto p : perms) {
        need(int(p) < in.rank(), debugName + ": permutation out of range");
    }
    auto &op = pushOp(OP_TRANSPOSE, debugName, {input}, {output});
    for (size_t k = 0; k < perms.size(); ++k) {
        op.i[k] = int32_t(perms[k]);
    }
}

void GraphPipeline::makeConcat(const std::vector<int32_t> &inputs, int32_t output, uint32_t axis,
                               const std::string &debugName) {
    uint32_t offset = 0;
    for (auto input : inputs) {
        const auto &in = tensor(input);
        need(in.rank() == tensor(output).rank() && int(axis) < in.rank(), debugName + ": rank/axis mismatch");
        need(elemSize(in.dtype) == elemSize(tensor(output).dtype), debugName + ": element size mismatch");
        auto &op = pushOp(OP_CONCAT, debugName, {input}, {output});
        op.i[0] = int32_t(axis), op.i[1] = int32_t(offset);
        offset += uint32_t(in.dims[axis]);
    }
}

void GraphPipeline::makeClamp(int32_t input, int32_t output, double min, double max, uint32_t nanMode,
                              const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need((in.dtype == MLEL_I8 || in.dtype == MLEL_I16 || in.dtype == MLEL_I32) && in.dtype == out.dtype,
         debugName + ": only integer types are built");
    auto &op = pushOp(OP_CLAMP, debugName, {input}, {output});
    op.d[0] = min, op.d[1] = max, op.i[0] = int32_t(nanMode);
}

void GraphPipeline::makeBinary(BinaryOp opk, int32_t input1, int32_t input2, int32_t output, uint32_t nanMode,
                               const std::string &debugName) {
    const auto &a = tensor(input1), &b = tensor(input2), &out = tensor(output);
    need(a.dtype == b.dtype, debugName + ": input types differ");
    need(a.rank() == b.rank() && a.rank() == out.rank(), debugName + ": rank mismatch");
    const bool f32ok = a.dtype == MLEL_F32 && (opk == BIN_ADD || opk == BIN_SUB || opk == BIN_MAXIMUM ||
                                               opk == BIN_MINIMUM || opk >= BIN_EQUAL);
    need((isIntegerType(a.dtype) && a.dtype < MLEL_U8 && opk != BIN_POW) || f32ok, debugName + ": input type not built");
    if (a.dtype == MLEL_F32 && (opk == BIN_MAXIMUM || opk == BIN_MINIMUM)) {
        need(nanMode != 2, debugName + ": NaN-ignore mode is not built");
    }
    auto &op = pushOp(OP_BINARY, debugName, {input1, input2}, {output});
    op.sub = opk;
    op.i[0] = int32_t(nanMode);
}

void GraphPipeline::makeUnary(UnaryOp opk, int32_t input, int32_t output, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    if (opk >= UN_CEIL) {
        need(in.dtype == MLEL_F32 && out.dtype == MLEL_F32, debugName + ": only fp32 is built");
    } else if (in.dtype == MLEL_F32) {
        need(opk == UN_ABS && out.dtype == MLEL_F32, debugName + ": not a floating-point operator");
    } else {
        need(isIntegerType(in.dtype) && in.dtype < MLEL_U8, debugName + ": input type not built");
    }
    need(in.rank() == out.rank(), debugName + ": rank mismatch");
    auto &op = pushOp(OP_UNARY, debugName, {input}, {output});
    op.sub = opk;
}

void GraphPipeline::makeMul(int32_t input1, int32_t input2, int32_t output, uint32_t shift,
                            const std::string &debugName) {
    const auto &a = tensor(input1), &b = tensor(input2), &out = tensor(output);
    need(a.dtype == b.dtype && a.rank() == b.rank() && a.rank() == out.rank(), debugName + ": operand mismatch");
    need((a.dtype == MLEL_F32 && out.dtype == MLEL_F32) ||
             ((a.dtype == MLEL_I8 || a.dtype == MLEL_I16 || a.dtype == MLEL_I32) && out.dtype == MLEL_I32),
         debugName + ": supported types are int8/int16/int32->int32 and fp32");
    auto &op = pushOp(OP_MUL, debugName, {input1, input2}, {output});
    op.i[0] = int32_t(shift);
}

void GraphPipeline::makeReduce(ReduceOp opk, int32_t input, int32_t output, uint32_t axis, uint32_t nanMode,
                               const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == out.rank() && int(axis) < in.rank(), debugName + ": rank/axis mismatch");
    need(isIntegerType(in.dtype) && in.dtype < MLEL_U8 && in.dtype == out.dtype,
         debugName + ": only integer types are built");
    auto &op = pushOp(OP_REDUCE, debugName, {input}, {output});
    op.sub = opk;
    op.i[0] = int32_t(axis);
    op.i[1] = 1; // integers force NaN mode PROPAGATE (graph/compute_graph_op.cpp:1674-1682)
    (void)nanMode;
}

void GraphPipeline::makeCast(int32_t input, int32_t output, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    const auto ok = [](int32_t dt) { return (isIntegerType(dt) && dt < MLEL_U8) || dt == MLEL_F32; };
    need(ok(in.dtype) && ok(out.dtype), debugName + ": type not built");
    need(in.rank() == out.rank(), debugName + ": rank mismatch");
    pushOp(OP_CAST, debugName, {input}, {output});
}

void GraphPipeline::makeReshape(int32_t input, int32_t output, const std::string &debugName) {
    need(elemSize(tensor(input).dtype) == elemSize(tensor(output).dtype), debugName + ": element size mismatch");
    pushOp(OP_RESHAPE, debugName, {input}, {output});
}

void GraphPipeline::makeSlice(int32_t input, int32_t output, const std::vector<uint32_t> &start,
                              const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == out.rank() && int(start.size()) == in.rank(), debugName + ": rank mismatch");
    need(elemSize(in.dtype) == elemSize(out.dtype), debugName + ": element size mismatch");
    auto &op = pushOp(OP_SLICE, debugName, {input}, {output});
    for (size_t k = 0; k < start.size(); ++k) {
        op.i[k] = int32_t(start[k]);
    }
}

void GraphPipeline::makePad(int32_t input, int32_t output, int32_t padding, double padConst, int32_t padConstInt,
                            const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &p = tensor(padding);
    need(in.rank() == out.rank() && in.dtype == out.dtype, debugName + ": operand mismatch");
    need(p.dtype == MLEL_I32 && p.rank() == 1, debugName + ": padding must be a rank-1 int32 tensor");
    need((isIntegerType(in.dtype) && in.dtype < MLEL_U8) || in.dtype == MLEL_F32, debugName + ": type not built");
    auto &op = pushOp(OP_PAD, debugName, {input, padding}, {output});
    op.d[0] = padConst;
    op.i[0] = padConstInt;
}

void GraphPipeline::makeArithmeticRightShift(int32_t input1, int32_t input2, int32_t output, bool round,
                                             const std::string &debugName) {
    const auto &a = tensor(input1), &b = tensor(input2);
    need(a.dtype == b.dtype && (a.dtype == MLEL_I8 || a.dtype == MLEL_I16 || a.dtype == MLEL_I32),
         debugName + ": only int8/int16/int32 are built");
    auto &op = pushOp(OP_ARITHMETIC_RIGHT_SHIFT, debugName, {input1, input2}, {output});
    op.i[0] = round;
}

void GraphPipeline::makeNegate(int32_t input, int32_t output, int32_t inputZeroPoint, int32_t outputZeroPoint,
                               const std::string &debugName) {
    const auto &in = tensor(input);
    need(in.dtype == MLEL_I8 || in.dtype == MLEL_I16 || in.dtype == MLEL_I32, debugName + ": only integers built");
    auto &op = pushOp(OP_NEGATE, debugName, {input}, {output});
    op.i[0] = inputZeroPoint, op.i[1] = outputZeroPoint;
}

void GraphPipeline::makeSelect(int32_t input1, int32_t input2, int32_t input3, int32_t output,
                               const std::string &debugName) {
    need(elemSize(tensor(input1).dtype) == 1, debugName + ": condition must be an 8-bit tensor");
    need(tensor(input2).dtype == tensor(input3).dtype, debugName + ": value types differ");
    pushOp(OP_SELECT, debugName, {input1, input2, input3}, {output});
}

void GraphPipeline::makeFft2D(int32_t inputReal, int32_t inputImag, int32_t outputReal, int32_t outputImag,
                              bool inverse, const std::string &debugName) {
    const auto &re = tensor(inputReal), &im = tensor(inputImag), &ore = tensor(outputReal), &oim = tensor(outputImag);
    need(re.dtype == MLEL_F32 && im.dtype == MLEL_F32 && ore.dtype == MLEL_F32 && oim.dtype == MLEL_F32,
         debugName + ": only fp32 is built");
    need(re.rank() == 3 && im.dims == re.dims && ore.dims == re.dims && oim.dims == re.dims,
         debugName + ": all four tensors must have the same [N, H, W] shape");
    auto &op = pushOp(OP_FFT2D, debugName, {inputReal, inputImag}, {outputReal, outputImag});
    op.i[0] = inverse;
}

void GraphPipeline::makeRfft2D(int32_t input, int32_t outputReal, int32_t outputImag, const std::string &debugName) {
    const auto &in = tensor(input), &ore = tensor(outputReal), &oim = tensor(outputImag);
    need(in.dtype == MLEL_F32 && ore.dtype == MLEL_F32 && oim.dtype == MLEL_F32, debugName + ": only fp32 is built");
    need(in.rank() == 3 && ore.rank() == 3 && oim.dims == ore.dims && ore.dims[0] == in.dims[0] &&
             ore.dims[1] == in.dims[1] && ore.dims[2] == in.dims[2] / 2 + 1,
         debugName + ": outputs must have the shape [N, H, W / 2 + 1]");
    pushOp(OP_RFFT2D, debugName, {input}, {outputReal, outputImag});
}

void GraphPipeline::makeArgmax(int32_t input, int32_t output, uint32_t axis, uint32_t nanMode,
                               const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.dtype == MLEL_I8 || in.dtype == MLEL_I16 || in.dtype == MLEL_I32, debugName + ": only integers built");
    need(out.dtype == MLEL_I32, debugName + ": the output holds int32 indices");
    need(int(axis) < in.rank() && out.rank() == in.rank() - 1, debugName + ": axis or rank mismatch");
    auto &op = pushOp(OP_ARGMAX, debugName, {input}, {output});
    op.i[0] = int32_t(axis), op.i[1] = int32_t(nanMode);
}

void GraphPipeline::makeGather(int32_t values, int32_t indices, int32_t output, const std::string &debugName) {
    const auto &v = tensor(values), &ix = tensor(indices), &out = tensor(output);
    need(v.rank() == 3 && ix.rank() == 2 && out.rank() == 3, debugName + ": rank mismatch");
    need(ix.dtype == MLEL_I32, debugName + ": indices must be int32");
    need(elemSize(v.dtype) == elemSize(out.dtype), debugName + ": element size mismatch");
    pushOp(OP_GATHER, debugName, {values, indices}, {output});
}

void GraphPipeline::makeScatter(int32_t input, int32_t values, int32_t indices, int32_t output,
                                const std::string &debugName) {
    const auto &in = tensor(input), &v = tensor(values), &ix = tensor(indices), &out = tensor(output);
    need(in.rank() == 3 && v.rank() == 3 && ix.rank() == 2 && out.rank() == 3, debugName + ": rank mismatch");
    need(ix.dtype == MLEL_I32, debugName + ": indices must be int32");
    need(elemSize(v.dtype) == elemSize(out.dtype) && elemSize(in.dtype) == elemSize(out.dtype),
         debugName + ": element size mismatch");
    pushOp(OP_SCATTER, debugName, {values, indices, input}, {output});
}

void GraphPipeline::makeReverse(int32_t input, int32_t output, uint32_t axis, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == out.rank() && int(axis) < in.rank(), debugName + ": axis or rank mismatch");
    need(elemSize(in.dtype) == elemSize(out.dtype), debugName + ": element size mismatch");
    auto &op = pushOp(OP_REVERSE, debugName, {input}, {output});
    op.i[0] = int32_t(axis);
}

void GraphPipeline::makeTile(int32_t input, int32_t output, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == out.rank(), debugName + ": rank mismatch");
    need(elemSize(in.dtype) == elemSize(out.dtype), debugName + ": element size mismatch");
    for (int k = 0; k < in.rank(); ++k) {
        need(in.dims[size_t(k)] > 0, debugName + ": empty input dimension");
    }
    pushOp(OP_TILE, debugName, {input}, {output});
}

void GraphPipeline::makeResize(int32_t input, int32_t output, const std::vector<int32_t> &scale,
                               const std::vector<int32_t> &offset, const std::vector<int32_t> &border, uint32_t mode,
                               const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output);
    need(in.rank() == 4 && out.rank() == 4, debugName + ": rank mismatch");
    need(scale.size() == 4 && offset.size() == 2 && border.size() == 2, debugName + ": attribute size mismatch");
    need(mode == 1 || mode == 2, debugName + ": mode must be NEAREST (1) or BILINEAR (2)");
    need(scale[0] > 0 && scale[2] > 0, debugName + ": scale numerators must be positive");
    // integer variants of the operator: int8 -> int8 / int32, int16 -> int16 / int64 (48-bit)
    const bool ok = (in.dtype == MLEL_I8 && (out.dtype == MLEL_I8 || out.dtype == MLEL_I32)) ||
                    (in.dtype == MLEL_I16 && (out.dtype == MLEL_I16 || out.dtype == MLEL_I64));
    need(ok, debugName + ": only the integer variants are built");
    auto &op = pushOp(OP_RESIZE, debugName, {input}, {output});
    for (int k = 0; k < 4; ++k) {
        op.i[k] = scale[size_t(k)];
    }
    op.i[4] = offset[0], op.i[5] = offset[1], op.i[6] = border[0], op.i[7] = border[1], op.i[8] = int32_t(mode);
}

void GraphPipeline::makeTransposeConv2D(int32_t input, int32_t output, int32_t weights, int32_t biases,
                                        const std::vector<int32_t> &outPad, const std::vector<int32_t> &stride,
                                        int8_t inputZeroPoint, int8_t weightZeroPoint, uint32_t accType,
                                        const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &w = tensor(weights), &b = tensor(biases);
    need(in.rank() == 4 && out.rank() == 4 && w.rank() == 4 && b.rank() == 1, debugName + ": rank mismatch");
    need(outPad.size() == 4 && stride.size() == 2, debugName + ": attribute size mismatch");
    need(stride[0] > 0 && stride[1] > 0, debugName + ": strides must be positive");
    need(accType == 1 || accType == 4, debugName + ": only integer accumulators are built (accType 1 or 4)");
    need((in.dtype == MLEL_I8 && out.dtype == MLEL_I32) || (in.dtype == MLEL_I16 && out.dtype == MLEL_I64),
         debugName + ": supported types are int8->int32 and int16->int64");
    need(w.dtype == MLEL_I8 && b.dtype == out.dtype, debugName + ": weights must be int8, bias of the output type");
    auto &op = pushOp(OP_TRANSPOSE_CONV2D, debugName, {input, weights, biases}, {output});
    for (int k = 0; k < 4; ++k) {
        op.i[k] = outPad[size_t(k)];
    }
    op.i[4] = stride[0], op.i[5] = stride[1], op.i[6] = 1, op.i[7] = 1;
    op.i[8] = inputZeroPoint, op.i[9] = weightZeroPoint, op.i[10] = int32_t(accType);
}

void GraphPipeline::makeConv3D(int32_t input, int32_t output, int32_t weights, int32_t biases,
                               const std::vector<int32_t> &pad, const std::vector<int32_t> &stride,
                               const std::vector<int32_t> &dilation, int8_t inputZeroPoint, int8_t weightZeroPoint,
                               uint32_t accType, const std::string &debugName) {
    const auto &in = tensor(input), &out = tensor(output), &w = tensor(weights), &b = tensor(biases);
    need(in.rank() == 5 && out.rank() == 5 && w.rank() == 5 && b.rank() == 1, debugName + ": rank mismatch");
    need(pad.size() == 6 && stride.size() == 3 && dilation.size() == 3, debugName + ": attribute size mismatch");
    need(dilation[0] > 0 && dilation[1] > 0 && dilation[2] > 0, debugName + ": dilations must be positive");
    need(accType == 1 || accType == 4, debugName + ": only integer accumulators are built (accType 1 or 4)");
    need((in.dtype == MLEL_I8 && out.dtype == MLEL_I32) || (in.dtype == MLEL_I16 && out.dtype == MLEL_I64),
         debugName + ": supported types are int8->int32 and int16->int64");
    need(w.dtype == MLEL_I8 && b.dtype == out.dtype, debugName + ": weights must be int8, bias of the output type");
    auto &op = pushOp(OP_CONV3D, debugName, {input, weights, biases}, {output});
    for (int k = 0; k < 6; ++k) {
        op.i[k] = pad[size_t(k)];
    }
    for (int k = 0; k < 3; ++k) {
        op.i[6 + k] = stride[size_t(k)];
        op.i[9 + k] = dilation[size_t(k)];
    }
    op.i[12] = inputZeroPoint, op.i[13] = weightZeroPoint, op.i[14] = int32_t(accType);
}

/*******************************************************************************
 * Fusion
 *******************************************************************************/

namespace {

FusedRescale toFusedRescale(const GraphPipeline &p, const OpDesc &r) {
    FusedRescale f;
    f.multTensor = r.in[1];
    f.shiftTensor = r.in[2];
    f.inDtype = p.tensor(r.in[0]).dtype;
    f.outDtype = p.tensor(r.out[0]).dtype;
    f.attr.inZp = r.i[0];
    f.attr.outZp = r.i[1];
    f.attr.scale32 = r.i[2];
    f.attr.doubleRound = r.i[3];
    f.attr.perChannel = r.i[4];
    f.lo = f.outDtype == MLEL_I8 ? -128 : (f.outDtype == MLEL_I16 ? -32768 : INT32_MIN);
    f.hi = f.outDtype == MLEL_I8 ? 127 : (f.outDtype == MLEL_I16 ? 32767 : INT32_MAX);
    return f;
}

} // namespace

// Contiguous runs of row-wise integer operators -> OP_FUSED_ROWS nodes (see RowProgram in ops.hpp and
// kernels/row_machine.cu).  A run is a maximal stretch of consecutive, not yet grouped operators of the kinds RESCALE
// (per tensor, constant parameters), TABLE (constant table), ADD, SUB, MUL on int32, REDUCE_SUM/MAX/MIN along the last
// axis of an int32 tensor and CLAMP, whose tensors all have the run's full shape F = [..., L] (L a multiple of 4), F
// with a last dimension of 1, or one constant element.  Because the run is contiguous in creation order, everything it
// reads from outside exists before its first operator and nothing outside it runs between its operators, so the node
// can stand at the position of the last one.  Tensors used only inside the run are never written to memory.
void GraphPipeline::fuseRowRuns(std::vector<int> &group, const std::vector<UseInfo> &uses,
                                const std::function<void(OpDesc, const std::vector<int> &)> &emit) {
    const int n = int(ops_.size());
    enum { kNone = 0, kFull, kValue, kOne };
    const auto shapeKind = [&](int32_t t, const std::vector<int64_t> &F) {
        const TensorDescriptor &td = tensor(t);
        if (!td.packed()) {
            return int(kNone);
        }
        if (td.dims == F) {
            return int(kFull);
        }
        if (td.dims.size() == F.size() && td.dims.back() == 1 &&
            std::equal(F.begin(), F.end() - 1, td.dims.begin())) {
            return int(kValue);
        }
        return td.numel() == 1 ? int(kOne) : int(kNone);
    };
    const auto intType = [](int32_t d) { return d == MLEL_I8 || d == MLEL_I16 || d == MLEL_I32; };
    const auto isConst = [&](int32_t t) { return tensor(t).cls == TensorClass::Constant; };
    // Whether `op` can be an instruction of a run of shape F (operand shapes are checked by the caller's build).
    const auto accepted = [&](const OpDesc &op, const std::vector<int64_t> &F) {
        const auto kindOf = [&](int32_t t) { return shapeKind(t, F); };
        switch (op.kind) {
        case OP_RESCALE: {
            const int32_t di = tensor(op.in[0]).dtype, dout = tensor(op.out[0]).dtype;
            return intType(di) && intType(dout) && op.i[2] && !op.i[4] && !op.i[5] && !op.i[6] && isConst(op.in[1]) &&
                   isConst(op.in[2]) && tensor(op.in[1]).dtype == MLEL_I32 && tensor(op.in[1]).hostData.size() >= 4 &&
                   !tensor(op.in[2]).hostData.empty() && kindOf(op.in[0]) != kNone && kindOf(op.in[0]) != kOne &&
                   kindOf(op.out[0]) == kindOf(op.in[0]);
        }
        case OP_TABLE: {
            const TensorDescriptor &tb = tensor(op.in[1]);
            const int32_t di = tensor(op.in[0]).dtype, dout = tensor(op.out[0]).dtype;
            const bool t8 = di == MLEL_I8 && dout == MLEL_I8 && tb.dtype == MLEL_I8 && tb.numel() == 256;
            const bool t16 = di == MLEL_I16 && dout == MLEL_I32 && tb.dtype == MLEL_I16 && tb.numel() == 513;
            return isConst(op.in[1]) && (t8 || t16) && kindOf(op.in[0]) != kNone && kindOf(op.in[0]) != kOne &&
                   kindOf(op.out[0]) == kindOf(op.in[0]);
        }
        case OP_BINARY:
        case OP_MUL: {
            if (op.kind == OP_BINARY && op.sub != BIN_ADD && op.sub != BIN_SUB) {
                return false;
            }
            if (op.kind == OP_MUL && (op.i[0] < 0 || op.i[0] > 62)) {
                return false;
            }
            const int ka = kindOf(op.in[0]), kb = kindOf(op.in[1]), ko = kindOf(op.out[0]);
            if (tensor(op.in[0]).dtype != MLEL_I32 || tensor(op.in[1]).dtype != MLEL_I32 ||
                tensor(op.out[0]).dtype != MLEL_I32 || ka == kNone || kb == kNone) {
                return false;
            }
            if ((ka == kOne && !isConst(op.in[0])) || (kb == kOne && !isConst(op.in[1]))) {
                return false; // a single run-time value is neither per row nor an immediate
            }
            const int widest = (ka == kFull || kb == kFull) ? kFull : kValue;
            return ko == widest && (ka != kOne || kb != kOne);
        }
        case OP_REDUCE:
            return (op.sub == RED_SUM || op.sub == RED_MAX || op.sub == RED_MIN) && tensor(op.in[0]).dtype == MLEL_I32 &&
                   tensor(op.out[0]).dtype == MLEL_I32 && op.i[0] == int(F.size()) - 1 && kindOf(op.in[0]) == kFull &&
                   kindOf(op.out[0]) == kValue;
        case OP_CLAMP:
            return intType(tensor(op.in[0]).dtype) && tensor(op.in[0]).dtype == tensor(op.out[0]).dtype &&
                   kindOf(op.in[0]) != kNone && kindOf(op.in[0]) != kOne && kindOf(op.out[0]) == kindOf(op.in[0]);
        default:
            return false;
        }
    };
    // Translates ops_[first .. last] into a program, unless it needs more instructions, values or shared memory than the
    // kernel has (kTooLarge) or does not pay (kNotWorthIt: saves no pass over a full-shaped tensor, or costs more in
    // the row kernel than as separate kernels).
    enum { kBuilt = 0, kTooLarge, kNotWorthIt };
    const auto build = [&](int first, int last, const std::vector<int64_t> &F, OpDesc *node) -> int {
        auto prog = std::make_shared<RowProgram>();
        prog->len = int32_t(F.back());
        prog->rows = 1;
        for (size_t k = 0; k + 1 < F.size(); ++k) {
            prog->rows *= F[k];
        }
        std::map<int32_t, RowOperand> where; // tensor -> slot, per-row word or immediate
        std::map<int32_t, int> lastUse;      // tensor -> last operator of the run that reads it
        for (int k = first; k <= last; ++k) {
            for (int32_t t : ops_[size_t(k)].in) {
                lastUse[t] = k;
            }
        }
        std::vector<int> freeSlots, freeValues;
        int slots = 0, values = 0, elided = 0;
        std::vector<int32_t> reads, writes;
        const auto take = [&](int kind) {
            RowOperand o;
            o.kind = kind == kFull ? ROW_FULL : ROW_VALUE;
            std::vector<int> &pool = kind == kFull ? freeSlots : freeValues;
            if (!pool.empty()) {
                o.index = pool.back();
                pool.pop_back();
            } else {
                o.index = kind == kFull ? slots++ : values++;
            }
            return o;
        };
        const auto release = [&](const RowOperand &o) {
            if (o.kind == ROW_FULL) {
                freeSlots.push_back(o.index);
            } else if (o.kind == ROW_VALUE) {
                freeValues.push_back(o.index);
            }
        };
        const auto operand = [&](int32_t t) -> RowOperand {
            const auto it = where.find(t);
            if (it != where.end()) {
                return it->second;
            }
            const TensorDescriptor &td = tensor(t);
            const int kind = shapeKind(t, F);
            RowOperand o;
            if (kind == kOne && isConst(t)) {
                o.kind = ROW_IMMEDIATE;
                int64_t v = 0;
                const uint8_t *d = td.hostData.data();
                if (td.dtype == MLEL_I8) {
                    v = int8_t(d[0]);
                } else if (td.dtype == MLEL_I16) {
                    int16_t x;
                    std::memcpy(&x, d, 2);
                    v = x;
                } else {
                    int32_t x;
                    std::memcpy(&x, d, 4);
                    v = x;
                }
                o.imm = int32_t(v);
            } else {
                o = take(kind == kFull ? kFull : kValue);
                RowInst ld;
                ld.op = ROW_LOAD;
                ld.dst = o;
                ld.tensor = t;
                ld.dtype = td.dtype;
                prog->insts.push_back(ld);
                reads.push_back(t);
            }
            where[t] = o;
            return o;
        };
        for (int k = first; k <= last; ++k) {
            const OpDesc &op = ops_[size_t(k)];
            RowInst in;
            const int dataInputs = (op.kind == OP_BINARY || op.kind == OP_MUL) ? 2 : 1;
            in.a = operand(op.in[0]);
            if (dataInputs == 2) {
                in.b = operand(op.in[1]);
            }
            switch (op.kind) {
            case OP_RESCALE: {
                const TensorDescriptor &m = tensor(op.in[1]), &sh = tensor(op.in[2]);
                const int32_t di = tensor(op.in[0]).dtype, dout = tensor(op.out[0]).dtype;
                int32_t mult;
                std::memcpy(&mult, m.hostData.data(), 4);
                in.op = ROW_RESCALE;
                in.p[0] = mult;
                in.p[1] = int32_t(int8_t(sh.hostData[0]));
                in.p[2] = int32_t(wrapTo(di, op.i[0]));
                in.p[3] = int32_t(wrapTo(dout, op.i[1]));
                in.p[4] = int32_t(typeLowest(dout));
                in.p[5] = int32_t(typeMax(dout));
                in.p[6] = (op.i[2] && op.i[3]) ? 1 : 0;
                break;
            }
            case OP_TABLE:
                in.op = tensor(op.in[0]).dtype == MLEL_I8 ? ROW_TABLE8 : ROW_TABLE16;
                in.tensor = op.in[1];
                reads.push_back(op.in[1]);
                break;
            case OP_BINARY:
                in.op = op.sub == BIN_ADD ? ROW_ADD : ROW_SUB;
                break;
            case OP_MUL:
                in.op = ROW_MUL;
                in.p[0] = op.i[0];
                break;
            case OP_REDUCE:
                in.op = op.sub == RED_SUM ? ROW_REDUCE_SUM : (op.sub == RED_MAX ? ROW_REDUCE_MAX : ROW_REDUCE_MIN);
                break;
            default: { // OP_CLAMP
                const int32_t dt = tensor(op.in[0]).dtype;
                const double lo = std::max(op.d[0], double(typeLowest(dt))), hi = std::min(op.d[1], double(typeMax(dt)));
                in.op = ROW_CLAMP;
                in.p[0] = int32_t(lo);
                in.p[1] = int32_t(hi);
                break;
            }
            }
            // operands that nobody reads after this operator give their place back before the result takes one (an
            // element-wise result may overwrite its own operand: a lane only touches its own elements)
            for (int32_t t : {op.in[0], dataInputs == 2 ? op.in[1] : int32_t(-1)}) {
                if (t >= 0 && lastUse[t] == k && where.count(t)) {
                    release(where[t]);
                    where.erase(t);
                }
            }
            const int32_t out = op.out[0];
            const int outKind = shapeKind(out, F);
            in.dst = take(outKind == kFull ? kFull : kValue);
            where[out] = in.dst;
            prog->insts.push_back(in);
            // written to memory if anything outside the run reads it (or the application does)
            const TensorDescriptor &od = tensor(out);
            bool needed = od.cls != TensorClass::Session || od.isGraphOutput || uses[size_t(out)].producers != 1;
            for (int c : uses[size_t(out)].consumers) {
                needed = needed || c < first || c > last;
            }
            if (needed) {
                RowInst st;
                st.op = ROW_STORE;
                st.a = in.dst;
                st.tensor = out;
                st.dtype = od.dtype;
                prog->insts.push_back(st);
                writes.push_back(out);
            } else if (outKind == kFull) {
                ++elided;
            }
            if (!lastUse.count(out) || lastUse[out] <= k) {
                release(in.dst); // no reader inside the run
                where.erase(out);
            }
        }
        prog->slots = slots;
        prog->values = values;
        if (prog->insts.size() > size_t(kMaxRowInsts) || values > kMaxRowValues || rowMachineWarps(slots, prog->len) < 2) {
            return kTooLarge;
        }
        if (elided == 0 || writes.empty()) {
            return kNotWorthIt;
        }
        // Is the run worth it?  In the row kernel every instruction costs issue slots (it is bound by instructions, at
        // about half an instruction per cycle and scheduler); as kernels of their own the same operators are bound by
        // the bytes they move, or by the same arithmetic.  Picoseconds per element of the full shape, measured on a
        // B200 with softmax rows of 384 and layer-norm rows of 768 elements (the row kernel's figures include its
        // per-instruction overhead):
        const auto machineCost = [](int op) {
            switch (op) {
            case ROW_RESCALE:
            case ROW_TABLE16:
                return 1.2;
            case ROW_MUL:
                return 0.8;
            case ROW_TABLE8:
                return 0.5;
            case ROW_LOAD:
            case ROW_STORE:
            case ROW_REDUCE_SUM:
            case ROW_REDUCE_MAX:
            case ROW_REDUCE_MIN:
                return 0.2;
            default:
                return 0.27; // ADD, SUB, CLAMP
            }
        };
        double fusedCost = 0.0;
        for (const RowInst &in : prog->insts) {
            const bool full = in.dst.kind == ROW_FULL || in.a.kind == ROW_FULL;
            fusedCost += full ? machineCost(in.op) : 0.0;
        }
        // The alternative: one kernel per operator at 0.18 ps per byte of full-shaped operand or result (5.5 TB/s), not
        // below 0.6 of its arithmetic in the row kernel; the two smaller fused nodes of this pass (the exponential rows
        // of a softmax, MUL + RESCALE) count as one kernel each.
        const auto fullBytes = [&](int32_t t) { return shapeKind(t, F) == kFull ? double(dtypeSize(tensor(t).dtype)) : 0.0; };
        const auto kindAt = [&](int k, OpKind kind, int sub) {
            return k <= last && ops_[size_t(k)].kind == kind && (sub < 0 || ops_[size_t(k)].sub == sub);
        };
        const auto rowOpOf = [&](const OpDesc &op) {
            switch (op.kind) {
            case OP_RESCALE:
                return int(ROW_RESCALE);
            case OP_TABLE:
                return tensor(op.in[0]).dtype == MLEL_I8 ? int(ROW_TABLE8) : int(ROW_TABLE16);
            case OP_MUL:
                return int(ROW_MUL);
            case OP_REDUCE:
                return int(ROW_REDUCE_SUM);
            default:
                return int(ROW_ADD);
            }
        };
        double separateCost = 0.0;
        for (int k = first; k <= last; ++k) {
            int span = 1;
            if (kindAt(k, OP_REDUCE, RED_MAX) && kindAt(k + 1, OP_BINARY, BIN_SUB) && kindAt(k + 2, OP_RESCALE, -1) &&
                kindAt(k + 3, OP_TABLE, -1) && kindAt(k + 4, OP_REDUCE, RED_SUM)) {
                span = 5;
            } else if (kindAt(k, OP_MUL, -1) && kindAt(k + 1, OP_RESCALE, -1)) {
                span = 2;
            }
            // bytes: what the span reads from outside itself and its last full-shaped result (a softmax's exponentials
            // are written as well: the TABLE's result)
            double bytes = 0.0, arithmetic = 0.0;
            for (int m = k; m < k + span; ++m) {
                const OpDesc &op = ops_[size_t(m)];
                const int dataInputs = (op.kind == OP_BINARY || op.kind == OP_MUL) ? 2 : 1;
                for (int q = 0; q < dataInputs; ++q) {
                    bool inside = false;
                    for (int w = k; w < m; ++w) {
                        inside = inside || ops_[size_t(w)].out[0] == op.in[size_t(q)];
                    }
                    bytes += inside ? 0.0 : fullBytes(op.in[size_t(q)]);
                }
                const bool lastOfSpan = m == k + span - 1, tableOfSoftmax = span == 5 && m == k + 3;
                bytes += (lastOfSpan || tableOfSoftmax) ? fullBytes(op.out[0]) : 0.0;
                const bool full = shapeKind(op.out[0], F) == kFull || shapeKind(op.in[0], F) == kFull;
                arithmetic += full ? machineCost(rowOpOf(op)) : 0.0;
            }
            separateCost += std::max(0.18 * bytes, 0.6 * arithmetic);
            k += span - 1;
        }
        if (fusedCost >= separateCost) {
            return kNotWorthIt;
        }
        std::sort(reads.begin(), reads.end());
        reads.erase(std::unique(reads.begin(), reads.end()), reads.end());
        node->kind = OP_FUSED_ROWS;
        node->in = reads;
        node->out = writes;
        node->rows = prog;
        node->name = "ROWS";
        for (int k = first; k <= last; ++k) {
            node->name += (k == first ? "(" : "+") + ops_[size_t(k)].name;
        }
        node->name += ")";
        return kBuilt;
    };
    for (int i = 0; i < n; ++i) {
        if (group[size_t(i)] >= 0) {
            continue;
        }
        const OpDesc &head = ops_[size_t(i)];
        if (head.kind != OP_RESCALE && head.kind != OP_TABLE && head.kind != OP_BINARY && head.kind != OP_MUL &&
            head.kind != OP_REDUCE && head.kind != OP_CLAMP) {
            continue;
        }
        // the run's full shape: what its first operator reads (a reduction) or writes
        const std::vector<int64_t> F = head.kind == OP_REDUCE ? tensor(head.in[0]).dims : tensor(head.out[0]).dims;
        if (F.empty() || F.back() < 4 || F.back() % 4 != 0 || F.back() > (int64_t(1) << 20)) {
            continue;
        }
        int j = i;
        while (j < n && group[size_t(j)] < 0 && accepted(ops_[size_t(j)], F)) {
            ++j;
        }
        // The whole stretch, or -- only if the kernel cannot hold it -- its longest prefix that fits.  A stretch that is
        // not worth fusing is left alone as a whole: cutting it elsewhere would also cut the smaller patterns in it.
        for (int last = j - 1; last > i; --last) {
            OpDesc node = ops_[size_t(last)];
            const int verdict = build(i, last, F, &node);
            if (verdict == kBuilt) {
                std::vector<int> members;
                for (int k = i; k <= last; ++k) {
                    members.push_back(k);
                }
                emit(std::move(node), members);
                i = last;
                break;
            }
            if (verdict == kNotWorthIt) {
                i = j - 1;
                break;
            }
        }
    }
}

// Fusion keeps the arithmetic of every absorbed operator unchanged (the same integer steps run
// back to back in registers), so results stay bit-identical to the one-kernel-per-op list; it only
// removes the round trips of intermediates through memory.  A tensor may be elided when it lives
// in session memory, is not a graph output, is written by exactly one operator and read by
// exactly one.  The fused node runs at the position of its last absorbed operator.
void GraphPipeline::fuse() {
    exec_.clear();
    const int n = int(ops_.size());
    if (flags_ & MLEL_PIPELINE_NO_FUSION) {
        for (int i = 0; i < n; ++i) {
            exec_.push_back(ops_[size_t(i)]);
            exec_.back().fusedOps = {i};
        }
        return;
    }
    std::vector<UseInfo> uses(tensors_.size());
    std::vector<int> producer(tensors_.size(), -1);
    for (int i = 0; i < n; ++i) {
        for (auto t : ops_[size_t(i)].in) {
            uses[size_t(t)].consumers.push_back(i);
        }
        for (auto t : ops_[size_t(i)].out) {
            uses[size_t(t)].producers++;
            producer[size_t(t)] = i;
        }
    }
    // The single consumer of an elidable tensor, or -1.
    const auto soleConsumer = [&](int32_t t) -> int {
        const auto &td = tensor(t);
        if (td.cls != TensorClass::Session || td.isGraphOutput || td.isGraphInput || !td.packed()) {
            return -1;
        }
        const auto &u = uses[size_t(t)];
        if (u.producers != 1 || u.consumers.size() != 1) {
            return -1;
        }
        return u.consumers[0];
    };
    const auto isConst = [&](int32_t t) { return tensor(t).cls == TensorClass::Constant; };

    std::vector<int> group(size_t(n), -1); // op -> index into fused
    struct Group {
        OpDesc node;
        int last;
    };
    std::vector<Group> fused;

    const auto absorb = [&](Group &g, int gi, int opIndex) {
        group[size_t(opIndex)] = gi;
        g.node.fusedOps.push_back(opIndex);
        g.last = std::max(g.last, opIndex);
    };

    // Tries to extend `cur` (an int8 tensor) through an optional CLAMP; returns the new tail tensor.
    const auto tryClamp = [&](Group &g, int gi, int32_t cur, FusedRescale &stage) -> int32_t {
        const int c = soleConsumer(cur);
        if (c < 0 || group[size_t(c)] >= 0 || ops_[size_t(c)].kind != OP_CLAMP) {
            return cur;
        }
        const OpDesc &cl = ops_[size_t(c)];
        const auto &td = tensor(cl.out[0]);
        if (td.dtype != stage.outDtype) {
            return cur;
        }
        const int64_t lo = int64_t(cl.d[0]), hi = int64_t(cl.d[1]);
        if (lo > hi || lo < stage.lo || hi > stage.hi) {
            return cur;
        }
        stage.lo = int32_t(lo);
        stage.hi = int32_t(hi);
        absorb(g, gi, c);
        return cl.out[0];
    };

    // Phase 0: contractions with their RESCALE and the quantised residual add.  Between the phases: contiguous runs of
    // row-wise operators (fuseRowRuns).  Phase 1: the two smaller row patterns, for what the runs left over.
    for (int phase = 0; phase < 2; ++phase) {
    if (phase == 1) {
        fuseRowRuns(group, uses, [&](OpDesc node, const std::vector<int> &members) {
            Group g;
            g.node = std::move(node);
            g.node.fusedOps.clear();
            g.last = members.back();
            const int gi = int(fused.size());
            for (int k : members) {
                absorb(g, gi, k);
            }
            fused.push_back(std::move(g));
        });
    }
    for (int i = 0; i < n; ++i) {
        if (group[size_t(i)] >= 0) {
            continue;
        }
        const OpDesc &op = ops_[size_t(i)];
        const bool contraction = op.kind == OP_CONV2D || op.kind == OP_MATMUL || op.kind == OP_DEPTHWISE_CONV2D;
        if (contraction && tensor(op.out[0]).dtype == MLEL_I32 && tensor(op.in[0]).dtype == MLEL_I8) {
            const int r = soleConsumer(op.out[0]);
            if (r < 0 || group[size_t(r)] >= 0 || ops_[size_t(r)].kind != OP_RESCALE) {
                continue;
            }
            const OpDesc &rs = ops_[size_t(r)];
            if (rs.in[0] != op.out[0] || tensor(rs.out[0]).dtype != MLEL_I8 || !rs.i[2] || rs.i[5] || rs.i[6] ||
                !isConst(rs.in[1]) || !isConst(rs.in[2]) || tensor(rs.in[1]).dtype != MLEL_I32) {
                continue;
            }
            if (rs.i[4] && tensor(rs.in[1]).dims[0] != tensor(rs.out[0]).dims.back()) {
                continue; // a per-channel table shorter than the channel count reads zeros: leave unfused
            }
            Group g;
            g.node = op;
            g.node.kind = op.kind == OP_CONV2D ? OP_FUSED_CONV2D
                                               : (op.kind == OP_MATMUL ? OP_FUSED_MATMUL : OP_FUSED_DEPTHWISE);
            g.node.name = op.name + "+RESCALE";
            g.node.fusedOps.clear();
            g.last = i;
            const int gi = int(fused.size());
            absorb(g, gi, i);
            absorb(g, gi, r);
            g.node.epi.hasMain = true;
            g.node.epi.main = toFusedRescale(*this, rs);
            int32_t tail = tryClamp(g, gi, rs.out[0], g.node.epi.main);
            if (tail != rs.out[0]) {
                g.node.name += "+CLAMP";
            }
            g.node.out = {tail};
            fused.push_back(std::move(g));
            continue;
        }
        // A per-tensor RESCALE with constant parameters and signed operands, as the fused kernels evaluate it.
        const auto plainRescale = [&](const OpDesc &r, int32_t inDtype, int32_t outDtype) {
            return r.kind == OP_RESCALE && tensor(r.in[0]).dtype == inDtype && tensor(r.out[0]).dtype == outDtype && r.i[2] &&
                   !r.i[4] && !r.i[5] && !r.i[6] && isConst(r.in[1]) && isConst(r.in[2]) && tensor(r.in[1]).dtype == MLEL_I32 &&
                   tensor(r.out[0]).packed();
        };
        // REDUCE_MAX(x) -> SUB(x, max) -> RESCALE(int16) -> TABLE, and REDUCE_SUM of the TABLE's output: the row-wise
        // exponentials of a quantised softmax.  One kernel reads a row of x once and writes the TABLE's output and the
        // row sum, instead of five passes over tensors of x's size.
        if (phase == 1 && op.kind == OP_REDUCE && op.sub == RED_MAX && tensor(op.in[0]).dtype == MLEL_I32 &&
            tensor(op.in[0]).packed()) {
            const TensorDescriptor &x = tensor(op.in[0]);
            const int rank = x.rank();
            const int sb = soleConsumer(op.out[0]);
            if (rank < 1 || op.i[0] != rank - 1 || x.dims.back() % 4 != 0 || sb < 0 || group[size_t(sb)] >= 0) {
                continue;
            }
            const OpDesc &sub = ops_[size_t(sb)];
            if (sub.kind != OP_BINARY || sub.sub != BIN_SUB || sub.in[0] != op.in[0] || sub.in[1] != op.out[0] ||
                tensor(sub.out[0]).dims != x.dims) {
                continue;
            }
            const int rsI = soleConsumer(sub.out[0]);
            if (rsI < 0 || group[size_t(rsI)] >= 0 || !plainRescale(ops_[size_t(rsI)], MLEL_I32, MLEL_I16)) {
                continue;
            }
            const OpDesc &rs = ops_[size_t(rsI)];
            const int tbI = soleConsumer(rs.out[0]);
            if (tbI < 0 || group[size_t(tbI)] >= 0 || ops_[size_t(tbI)].kind != OP_TABLE) {
                continue;
            }
            const OpDesc &tb = ops_[size_t(tbI)];
            const TensorDescriptor &e = tensor(tb.out[0]);
            if (tb.in[0] != rs.out[0] || !isConst(tb.in[1]) || tensor(tb.in[1]).dtype != MLEL_I16 ||
                tensor(tb.in[1]).numel() != 513 || e.dtype != MLEL_I32 || !e.packed() || e.cls != TensorClass::Session ||
                uses[size_t(tb.out[0])].producers != 1) {
                continue;
            }
            // the TABLE's output stays in memory (the softmax multiplies it later); its row sum joins the kernel if it
            // is taken right away, i.e. before any other reader of the TABLE's output
            int sumI = -1;
            int firstOther = n;
            for (int c : uses[size_t(tb.out[0])].consumers) {
                const OpDesc &co = ops_[size_t(c)];
                if (sumI < 0 && co.kind == OP_REDUCE && co.sub == RED_SUM && co.i[0] == rank - 1 && group[size_t(c)] < 0) {
                    sumI = c;
                } else {
                    firstOther = std::min(firstOther, c);
                }
            }
            if (sumI < 0 || sumI > firstOther || !tensor(ops_[size_t(sumI)].out[0]).packed()) {
                continue;
            }
            Group g;
            g.node = op;
            g.node.kind = OP_FUSED_ROW_EXP;
            g.node.name = "REDUCE_MAX+SUB+RESCALE+TABLE+REDUCE_SUM";
            g.node.in = {op.in[0], tb.in[1]};
            g.node.out = {tb.out[0], ops_[size_t(sumI)].out[0]};
            g.node.fusedOps.clear();
            g.last = i;
            const int gi = int(fused.size());
            for (int k : {i, sb, rsI, tbI, sumI}) {
                absorb(g, gi, k);
            }
            g.node.epi.hasMain = true;
            g.node.epi.main = toFusedRescale(*this, rs);
            fused.push_back(std::move(g));
            continue;
        }
        // MUL(a, b, shift) -> RESCALE [-> CLAMP] on int32: the last step of a quantised softmax or layer norm
        if (phase == 1 && op.kind == OP_MUL && tensor(op.out[0]).dtype == MLEL_I32 && tensor(op.in[0]).dtype == MLEL_I32 &&
            tensor(op.in[1]).dtype == MLEL_I32 && tensor(op.in[0]).packed() && tensor(op.in[1]).packed() &&
            tensor(op.in[0]).dims == tensor(op.out[0]).dims && tensor(op.out[0]).dims.back() % 4 == 0) {
            const auto &da = tensor(op.in[0]).dims, &db = tensor(op.in[1]).dims;
            bool perRow = db.size() == da.size() && db.back() == 1;
            for (size_t k = 0; perRow && k + 1 < da.size(); ++k) {
                perRow = da[k] == db[k];
            }
            const bool oneValue = tensor(op.in[1]).numel() == 1;
            const int rsI = soleConsumer(op.out[0]);
            if (!(db == da || perRow || oneValue) || rsI < 0 || group[size_t(rsI)] >= 0 ||
                !(plainRescale(ops_[size_t(rsI)], MLEL_I32, MLEL_I8) || plainRescale(ops_[size_t(rsI)], MLEL_I32, MLEL_I16))) {
                continue;
            }
            const OpDesc &rs = ops_[size_t(rsI)];
            Group g;
            g.node = op;
            g.node.kind = OP_FUSED_MUL_RESCALE;
            g.node.name = "MUL+RESCALE";
            g.node.fusedOps.clear();
            g.last = i;
            const int gi = int(fused.size());
            absorb(g, gi, i);
            absorb(g, gi, rsI);
            g.node.epi.hasMain = true;
            g.node.epi.main = toFusedRescale(*this, rs);
            int32_t tail = tryClamp(g, gi, rs.out[0], g.node.epi.main);
            if (tail != rs.out[0]) {
                g.node.name += "+CLAMP";
            }
            g.node.out = {tail};
            fused.push_back(std::move(g));
            continue;
        }
        // RESCALE(a) + RESCALE(b) -> ADD -> RESCALE [-> CLAMP]  (quantised residual add)
        if (op.kind == OP_BINARY && op.sub == BIN_ADD && tensor(op.out[0]).dtype == MLEL_I32) {
            const int pa = producer[size_t(op.in[0])], pb = producer[size_t(op.in[1])];
            if (pa < 0 || pb < 0 || pa == pb || group[size_t(pa)] >= 0 || group[size_t(pb)] >= 0) {
                continue;
            }
            const OpDesc &ra = ops_[size_t(pa)], &rb = ops_[size_t(pb)];
            const auto okIn = [&](const OpDesc &r, int32_t t) {
                return r.kind == OP_RESCALE && soleConsumer(t) == i && tensor(r.in[0]).dtype == MLEL_I8 &&
                       tensor(r.in[0]).packed() && r.i[2] && !r.i[5] && !r.i[6] && !r.i[4] && isConst(r.in[1]) &&
                       isConst(r.in[2]) && tensor(r.in[1]).dtype == MLEL_I32;
            };
            if (!okIn(ra, op.in[0]) || !okIn(rb, op.in[1])) {
                continue;
            }
            const auto &da = tensor(ra.in[0]).dims, &db = tensor(rb.in[0]).dims, &dout = tensor(op.out[0]).dims;
            if (da != dout || db != dout) {
                continue; // broadcasting adds stay on the generic kernels
            }
            const int ro = soleConsumer(op.out[0]);
            if (ro < 0 || group[size_t(ro)] >= 0 || ops_[size_t(ro)].kind != OP_RESCALE) {
                continue;
            }
            const OpDesc &rs = ops_[size_t(ro)];
            if (tensor(rs.out[0]).dtype != MLEL_I8 || !rs.i[2] || rs.i[5] || rs.i[6] || rs.i[4] ||
                !isConst(rs.in[1]) || !isConst(rs.in[2]) || tensor(rs.in[1]).dtype != MLEL_I32 ||
                !tensor(rs.out[0]).packed()) {
                continue;
            }
            Group g;
            g.node = op;
            g.node.kind = OP_FUSED_ADD;
            g.node.name = "RESCALE+RESCALE+ADD+RESCALE";
            g.node.in = {ra.in[0], rb.in[0]};
            g.node.fusedOps.clear();
            g.last = i;
            const int gi = int(fused.size());
            absorb(g, gi, pa);
            absorb(g, gi, pb);
            absorb(g, gi, i);
            absorb(g, gi, ro);
            g.node.epi.hasResidual = true;
            g.node.epi.a = toFusedRescale(*this, ra);
            g.node.epi.b = toFusedRescale(*this, rb);
            g.node.epi.out = toFusedRescale(*this, rs);
            int32_t tail = tryClamp(g, gi, rs.out[0], g.node.epi.out);
            if (tail != rs.out[0]) {
                g.node.name += "+CLAMP";
            }
            g.node.out = {tail};
            fused.push_back(std::move(g));
        }
    }
    } // phases
    // Residual tail into the producing convolution: when one operand of a fused add is the (otherwise
    // unused) output of a fused CONV2D, the add and its three RESCALEs run in that convolution's epilogue
    // on the value still in registers; the other operand (the shortcut) is read there.  The merged node
    // runs where the add would have run, so the shortcut is complete by then.
    std::vector<bool> dead(fused.size(), false);
    for (size_t ga = 0; ga < fused.size(); ++ga) {
        Group &add = fused[ga];
        if (add.node.kind != OP_FUSED_ADD) {
            continue;
        }
        for (int side = 0; side < 2; ++side) {
            const int32_t mainT = add.node.in[size_t(side)], shortT = add.node.in[size_t(1 - side)];
            const int prod = producer[size_t(mainT)];
            if (prod < 0 || group[size_t(prod)] < 0) {
                continue;
            }
            const size_t gc = size_t(group[size_t(prod)]);
            Group &conv = fused[gc];
            if (dead[gc] || conv.node.kind != OP_FUSED_CONV2D || conv.node.epi.hasResidual ||
                conv.node.out[0] != mainT || mainT == shortT) {
                continue;
            }
            // the convolution's own output must feed nothing but this add's RESCALE
            const int consumer = soleConsumer(mainT);
            if (consumer < 0 || group[size_t(consumer)] != int(ga) || !tensor(shortT).packed() ||
                tensor(shortT).dims != tensor(mainT).dims) {
                continue;
            }
            conv.node.epi.hasResidual = true;
            conv.node.epi.a = side == 0 ? add.node.epi.a : add.node.epi.b;
            conv.node.epi.b = side == 0 ? add.node.epi.b : add.node.epi.a;
            conv.node.epi.out = add.node.epi.out;
            conv.node.epi.shortcutTensor = shortT;
            conv.node.out = add.node.out;
            conv.node.name += add.node.name.find("+CLAMP") != std::string::npos ? "+ADD+RESCALE+CLAMP" : "+ADD+RESCALE";
            for (int opIndex : add.node.fusedOps) {
                group[size_t(opIndex)] = int(gc);
                conv.node.fusedOps.push_back(opIndex);
            }
            conv.last = std::max(conv.last, add.last);
            dead[ga] = true;
            break;
        }
    }
    // The two input RESCALEs of a fused add come before the ADD in op order, possibly far before;
    // moving them to the ADD's position is legal because their inputs are written exactly once.
    // A fused node is emitted at the position of its last absorbed operator.
    for (int i = 0; i < n; ++i) {
        const int gi = group[size_t(i)];
        if (gi < 0) {
            exec_.push_back(ops_[size_t(i)]);
            exec_.back().fusedOps = {i};
        } else if (fused[size_t(gi)].last == i) {
            std::sort(fused[size_t(gi)].node.fusedOps.begin(), fused[size_t(gi)].node.fusedOps.end());
            exec_.push_back(fused[size_t(gi)].node);
        }
    }
}

int32_t GraphPipeline::addDerivedConstant(int32_t dtype, const std::vector<int64_t> &dims, const void *data) {
    auto t = std::make_unique<TensorDescriptor>();
    t->dtype = dtype;
    t->dims = dims;
    t->strides = packedStrides(dtype, dims);
    t->cls = TensorClass::Constant;
    const auto *bytes = static_cast<const uint8_t *>(data);
    t->hostData.assign(bytes, bytes + t->sizeBytes());
    return addTensor(std::move(t));
}

// Session-memory scratch of one launched node (planned like any other intermediate tensor).
int32_t GraphPipeline::addScratchTensor(int32_t dtype, const std::vector<int64_t> &dims) {
    auto t = std::make_unique<TensorDescriptor>();
    t->dtype = dtype;
    t->dims = dims;
    t->strides = packedStrides(dtype, dims);
    t->cls = TensorClass::Session;
    t->sessionOrder = int32_t(sessionTensors_.size());
    const int32_t tid = addTensor(std::move(t));
    sessionTensors_.push_back(tid);
    return tid;
}

// Decides, per launched node, whether the tcgen05 kernel can take it, and tabulates what that kernel
// needs beyond the graph's own tensors.  Everything here is derived once from constant data.
//
// CONV2D (plain or fused): int8 NHWC input, packed; constant int8 OHWI weights with zero point 0;
// constant int32 bias; IC and OC multiples of 16; K = KH*KW*IC <= 65536 so that the raw int32 sum of
// products cannot overflow.  The correction table holds, per border class of an output pixel,
//     corr[class][oc] = bias[oc] - inputZeroPoint * sum over the taps that are in range of w[oc, tap, :]
// which turns the tensor core's sum(x * w) over zero-filled taps into the reference's
// sum over in-range taps of (x - zp) * w + bias   (conv2d.comp:59-112), modulo 2^32.
//
// MATMUL (plain or fused) with a constant second input [Nb, C, W] and zero point 0 on it: the input
// is transposed once to K-major [Nb][W][C]; corr[b][w] = -zeroPoint1 * sum_c B[b, c, w].
// The residual tail of a fused convolution maps (main-stage int8 value m, shortcut int8 value s) to one output
// byte: RESCALE_out(RESCALE_a(m) + RESCALE_b(s)) with the clamps of each stage.  All three RESCALEs are
// per-tensor with constant parameters, so the whole map is 256 x 256 bytes, computed here once with the
// reference's own arithmetic (rescale.comp:27-72 via rescaleValue) and looked up by the kernel's epilogue.
void GraphPipeline::buildResidualTable(OpDesc &op) {
    struct Stage {
        int32_t mult, shift, inZp, outZp, lo, hi;
        bool doubleRound;
    };
    const auto stageOf = [&](const FusedRescale &f, Stage &st) {
        if (f.multTensor < 0 || f.shiftTensor < 0 || f.attr.perChannel) {
            return false;
        }
        const TensorDescriptor &m = tensor(f.multTensor), &sh = tensor(f.shiftTensor);
        if (m.cls != TensorClass::Constant || sh.cls != TensorClass::Constant || m.dtype != MLEL_I32 ||
            elemSize(sh.dtype) != 1 || m.hostData.size() < 4 || sh.hostData.empty() || !f.attr.scale32) {
            return false;
        }
        std::memcpy(&st.mult, m.hostData.data(), 4);
        const int32_t shift = int32_t(int8_t(sh.hostData[0]));
        st.shift = shift < 0 ? 0 : (shift > 62 ? 62 : shift);
        st.inZp = int32_t(wrapTo(f.inDtype, f.attr.inZp));
        st.outZp = int32_t(wrapTo(f.outDtype, f.attr.outZp));
        st.lo = f.lo, st.hi = f.hi;
        st.doubleRound = f.attr.doubleRound != 0;
        return true;
    };
    Stage a{}, b{}, o{};
    if (!stageOf(op.epi.a, a) || !stageOf(op.epi.b, b) || !stageOf(op.epi.out, o)) {
        return;
    }
    const auto run = [](const Stage &st, int64_t v) {
        return rescaleValue(v, st.inZp, st.mult, st.shift, st.doubleRound, st.outZp, st.lo, st.hi);
    };
    int32_t fromMain[256], fromShortcut[256];
    for (int v = -128; v < 128; ++v) {
        fromMain[v + 128] = run(a, v);
        fromShortcut[uint8_t(int8_t(v))] = run(b, v);
    }
    constexpr int kRow = GemmI8Params::kResidualRowBytes; // rows are padded: see gemm_i8_ocmajor.cu
    std::vector<uint8_t> table(size_t(256 * kRow), 0);
    for (int m = 0; m < 256; ++m) {
        for (int sc = 0; sc < 256; ++sc) {
            const int32_t sum = int32_t(uint32_t(fromMain[m]) + uint32_t(fromShortcut[sc]));
            table[size_t(m * kRow + sc)] = uint8_t(run(o, sum));
        }
    }
    op.aux[3] = addDerivedConstant(MLEL_U8, {int64_t(table.size())}, table.data());
}

void GraphPipeline::prepareTensorCore() {
    for (auto &op : exec_) {
        const bool conv = op.kind == OP_CONV2D || op.kind == OP_FUSED_CONV2D;
        const bool mm = op.kind == OP_MATMUL || op.kind == OP_FUSED_MATMUL;
        if (!conv && !mm) {
            continue;
        }
        const TensorDescriptor &in = tensor(op.in[0]);
        const TensorDescriptor &out = tensor(op.out[0]);
        const bool fusedOut = op.kind == OP_FUSED_CONV2D || op.kind == OP_FUSED_MATMUL;
        if (in.dtype != MLEL_I8 || !in.packed() || !out.packed() || out.dtype != (fusedOut ? MLEL_I8 : MLEL_I32)) {
            continue;
        }
        if (conv) {
            const TensorDescriptor &w = tensor(op.in[1]);
            const TensorDescriptor &b = tensor(op.in[2]);
            if (w.cls != TensorClass::Constant || b.cls != TensorClass::Constant || !w.packed() || !b.packed() ||
                w.dtype != MLEL_I8 || b.dtype != MLEL_I32 || op.i[9] != 0) {
                continue;
            }
            const int64_t OC = w.dims[0], KH = w.dims[1], KW = w.dims[2], IC = w.dims[3];
            const int64_t H = in.dims[1], W = in.dims[2], OH = out.dims[1], OW = out.dims[2];
            const int padTop = op.i[0], padLeft = op.i[2], sy = op.i[4], sx = op.i[5], dy = op.i[6], dx = op.i[7];
            if (sy <= 0 || sx <= 0 || dy <= 0 || dx <= 0) {
                continue;
            }
            // Channel counts that are not multiples of 16 (an RGB stem) cannot be gathered in 16-byte pieces
            // from the tensor itself.  Such a convolution (tc == 2) first copies its input into session memory
            // with the channels zero-padded to 4, 8 or a multiple of 16 and the padding border materialised as
            // zeros, and then gathers from the copy, where every tap is in range, by a table of byte offsets.
            // Where the window's rows are contiguous and suitably aligned in the copy (unit x dilation, x stride
            // times padded channels a multiple of 8 bytes) one piece is 8 or 16 bytes of a window row, and each
            // window row is padded to whole pieces in the K order (with zero weights); otherwise one piece is
            // one tap (or 16 bytes of one).
            const bool padChannels = IC % 16 != 0;
            const int64_t ICp = !padChannels ? IC : (IC <= 4 ? 4 : (IC <= 8 ? 8 : (IC + 15) / 16 * 16));
            const bool rowRuns = padChannels && dx == 1 && ICp < 16 && (sx * ICp) % 8 == 0;
            const int64_t piece = !padChannels ? 16 : (rowRuns ? ((sx * ICp) % 16 == 0 ? 16 : 8) : std::min<int64_t>(ICp, 16));
            const int64_t runBytes = rowRuns ? (KW * ICp + piece - 1) / piece * piece : KW * ICp; // K bytes per window row
            const int64_t kPad = (KH * runBytes + 15) / 16 * 16;
            if (in.dims[3] != IC || out.dims[3] != OC || kPad > 65536 ||
                (b.dims[0] != OC && b.dims[0] != 1) || out.numel() >= (int64_t(1) << 31) ||
                in.numel() >= (int64_t(1) << 31)) {
                continue;
            }

            // Border classes: the set of in-range taps along each axis.
            const auto classify = [](int64_t outDim, int64_t inDim, int64_t k, int stride, int pad, int dil,
                                     std::vector<uint8_t> &cls, std::vector<std::vector<bool>> &masks) {
                cls.resize(size_t(outDim));
                std::map<std::vector<bool>, int> ids;
                for (int64_t o = 0; o < outDim; ++o) {
                    std::vector<bool> mask(size_t(k), false);
                    for (int64_t t = 0; t < k; ++t) {
                        const int64_t i = o * stride - pad + t * dil;
                        mask[size_t(t)] = i >= 0 && i < inDim;
                    }
                    auto it = ids.find(mask);
                    if (it == ids.end()) {
                        it = ids.emplace(mask, int(masks.size())).first;
                        masks.push_back(mask);
                    }
                    if (it->second > 255) {
                        return false;
                    }
                    cls[size_t(o)] = uint8_t(it->second);
                }
                return true;
            };
            std::vector<uint8_t> rowCls, colCls;
            std::vector<std::vector<bool>> rowMasks, colMasks;
            if (!classify(OH, H, KH, sy, padTop, dy, rowCls, rowMasks) ||
                !classify(OW, W, KW, sx, padLeft, dx, colCls, colMasks)) {
                continue;
            }
            if (rowMasks.size() * colMasks.size() * size_t(OC) > (size_t(1) << 22)) {
                continue;
            }
            const auto *wd = reinterpret_cast<const int8_t *>(w.hostData.data());
            const auto *bd = reinterpret_cast<const int32_t *>(b.hostData.data());
            std::vector<int64_t> wsum(size_t(KH * KW * OC), 0); // [ky][kx][oc]
            for (int64_t oc = 0; oc < OC; ++oc) {
                for (int64_t t = 0; t < KH * KW; ++t) {
                    int64_t acc = 0;
                    const int8_t *row = wd + (oc * KH * KW + t) * IC;
                    for (int64_t ic = 0; ic < IC; ++ic) {
                        acc += row[ic];
                    }
                    wsum[size_t(t * OC + oc)] = acc;
                }
            }
            const int64_t zx = op.i[8];
            std::vector<int32_t> corr(rowMasks.size() * colMasks.size() * size_t(OC));
            for (size_t rc = 0; rc < rowMasks.size(); ++rc) {
                for (size_t cc = 0; cc < colMasks.size(); ++cc) {
                    for (int64_t oc = 0; oc < OC; ++oc) {
                        int64_t sum = 0;
                        for (int64_t ky = 0; ky < KH; ++ky) {
                            for (int64_t kx = 0; kx < KW; ++kx) {
                                if (rowMasks[rc][size_t(ky)] && colMasks[cc][size_t(kx)]) {
                                    sum += wsum[size_t((ky * KW + kx) * OC + oc)];
                                }
                            }
                        }
                        const int64_t v = int64_t(bd[b.dims[0] == 1 ? 0 : oc]) - zx * sum;
                        corr[(rc * colMasks.size() + cc) * size_t(OC) + size_t(oc)] = int32_t(uint32_t(uint64_t(v)));
                    }
                }
            }
            {
                // With corrections this small, accumulator + correction - zero point cannot leave int32 (the raw sum
                // of at most 65536 products is at most 2^30 in size): the epilogue may then fold the three terms into
                // one 32-bit addition without changing the reference's 64-bit arithmetic.
                // Level 2: the three terms together stay below 2^29 in size (a product is at most 2^14), which the
                // epilogue's RESCALE from 32-bit words asks for.
                bool small = true, tiny = true;
                const int64_t rawBound = KH * KW * IC * (int64_t(1) << 14) + 256;
                for (const int32_t c : corr) {
                    small = small && c >= -((1 << 30) - 256) && c <= (1 << 30) - 256;
                    tiny = tiny && (c < 0 ? -int64_t(c) : int64_t(c)) + rawBound < (int64_t(1) << 29);
                }
                op.auxi[4] = tiny ? 2 : (small ? 1 : 0);
            }
            op.aux[0] = addDerivedConstant(MLEL_I32, {int64_t(corr.size())}, corr.data());
            op.aux[1] = addDerivedConstant(MLEL_U8, {OH}, rowCls.data());
            op.aux[2] = addDerivedConstant(MLEL_U8, {OW}, colCls.data());
            op.auxi[0] = int32_t(colMasks.size());
            op.auxi[1] = int32_t(rowMasks.size() * colMasks.size());
            {
                // the most common class (normally "every tap in range"): its correction row is what the
                // kernel stages in shared memory
                std::vector<int64_t> rowCount(rowMasks.size(), 0), colCount(colMasks.size(), 0);
                for (auto c : rowCls) {
                    rowCount[c]++;
                }
                for (auto c : colCls) {
                    colCount[c]++;
                }
                const size_t rBest = size_t(std::max_element(rowCount.begin(), rowCount.end()) - rowCount.begin());
                const size_t cBest = size_t(std::max_element(colCount.begin(), colCount.end()) - colCount.begin());
                op.auxi[3] = int32_t(rBest * colMasks.size() + cBest);
            }
            op.tc = 1;
            if (!padChannels && op.kind == OP_FUSED_CONV2D && op.epi.hasResidual) {
                buildResidualTable(op);
            }
            if (padChannels) {
                // geometry of the padded copy: rows and columns that any window can touch
                const int64_t Hp = std::max<int64_t>(H + padTop, (OH - 1) * sy + (KH - 1) * dy + 1);
                const int64_t xReach = rowRuns ? runBytes / ICp : (KW - 1) * dx + 1;
                const int64_t Wp = std::max<int64_t>(W + padLeft, (OW - 1) * sx + xReach);
                const int64_t numChunks = (kPad + 127) / 128 * 128 / piece;
                if (in.dims[0] * Hp * Wp * ICp >= (int64_t(1) << 31) || numChunks > 1024) {
                    op.tc = 0;
                    continue;
                }
                std::vector<int8_t> wPad(size_t(OC * kPad), 0);
                for (int64_t oc = 0; oc < OC; ++oc) {
                    for (int64_t ky = 0; ky < KH; ++ky) {
                        for (int64_t kx = 0; kx < KW; ++kx) {
                            std::memcpy(&wPad[size_t(oc * kPad + ky * runBytes + kx * ICp)],
                                        wd + ((oc * KH + ky) * KW + kx) * IC, size_t(IC));
                        }
                    }
                }
                std::vector<int32_t> table(size_t(numChunks), 0); // pieces past the window read offset 0 (weights 0)
                for (int64_t q = 0; q < numChunks; ++q) {
                    const int64_t k = q * piece;
                    if (k >= KH * runBytes) {
                        continue;
                    }
                    const int64_t ky = k / runBytes, r = k % runBytes;
                    const int64_t xBytes = rowRuns ? r : (r / ICp) * dx * ICp + r % ICp;
                    table[size_t(q)] = int32_t(ky * dy * Wp * ICp + xBytes);
                }
                op.aux[3] = addDerivedConstant(MLEL_I8, {OC, kPad}, wPad.data());
                op.aux[4] = addDerivedConstant(MLEL_I32, {numChunks}, table.data());
                op.scratch = addScratchTensor(MLEL_I8, {in.dims[0], Hp, Wp, ICp});
                op.auxi[2] = int32_t(piece);
                op.tc = 2;
            }
        } else {
            const TensorDescriptor &b = tensor(op.in[1]);
            if (!b.packed() || b.dtype != MLEL_I8 || op.i[1] != 0 || b.dims.size() != 3) {
                continue;
            }
            const int64_t Nb = b.dims[0], C = b.dims[1], W = b.dims[2];
            if (in.dims[0] != Nb || in.dims[2] != C || C % 16 != 0 || C > 65536 ||
                out.numel() >= (int64_t(1) << 31) || in.numel() >= (int64_t(1) << 31)) {
                continue;
            }
            if (b.cls != TensorClass::Constant) {
                // Second input produced at run time (tc == 3): a kernel in front of the product transposes it to
                // the K-contiguous form the tensor core reads and sums its columns for the zero-point
                // correction; both land in one scratch tensor: [Nb][W][C] bytes, then [Nb][W] int32.
                if (W % 16 != 0 || b.numel() >= (int64_t(1) << 31)) {
                    continue;
                }
                const int64_t btBytes = (Nb * W * C + 255) / 256 * 256;
                op.scratch = addScratchTensor(MLEL_I8, {btBytes + Nb * W * 4});
                op.auxi[2] = int32_t(btBytes);
                op.tc = 3;
                continue;
            }
            const auto *bdata = reinterpret_cast<const int8_t *>(b.hostData.data());
            std::vector<int8_t> bt(size_t(Nb * W * C));
            std::vector<int32_t> corr(size_t(Nb * W));
            const int64_t za = op.i[0];
            for (int64_t n = 0; n < Nb; ++n) {
                for (int64_t w = 0; w < W; ++w) {
                    int64_t sum = 0;
                    for (int64_t c = 0; c < C; ++c) {
                        const int8_t v = bdata[(n * C + c) * W + w];
                        bt[size_t((n * W + w) * C + c)] = v;
                        sum += v;
                    }
                    corr[size_t(n * W + w)] = int32_t(uint32_t(uint64_t(-za * sum)));
                }
            }
            op.aux[0] = addDerivedConstant(MLEL_I32, {Nb * W}, corr.data());
            op.aux[3] = addDerivedConstant(MLEL_I8, {Nb, W, C}, bt.data());
            op.tc = 1;
        }
    }
}

const std::vector<OpDesc> &GraphPipeline::getExecList() {
    finalize();
    return exec_;
}

void GraphPipeline::finalize() {
    if (finalized_) {
        return;
    }
    fuse();
    if (!(flags_ & MLEL_PIPELINE_NO_TENSOR_CORE)) {
        prepareTensorCore();
    }
    // Lay constants out in one slab, each on a 256-byte boundary.
    uint64_t offset = 0;
    for (auto &t : tensors_) {
        if (t->cls == TensorClass::Constant) {
            t->constOffset = offset;
            offset += (t->sizeBytes() + 255) / 256 * 256;
        }
    }
    constSlabBytes_ = offset;
    finalized_ = true;
}

char *GraphPipeline::constantBase() {
    finalize();
    if (constSlab_ != nullptr || constSlabBytes_ == 0) {
        return constSlab_;
    }
    if (cudaGetDevice(&constDevice_) != cudaSuccess) {
        throw std::runtime_error("no CUDA device is available");
    }
    void *p = nullptr;
    if (cudaMalloc(&p, constSlabBytes_) != cudaSuccess) {
        throw std::runtime_error("out of device memory for graph constants");
    }
    constSlab_ = static_cast<char *>(p);
    std::vector<uint8_t> staging(constSlabBytes_, 0);
    for (auto &t : tensors_) {
        if (t->cls == TensorClass::Constant) {
            std::memcpy(staging.data() + t->constOffset, t->hostData.data(), t->hostData.size());
        }
    }
    if (cudaMemcpy(constSlab_, staging.data(), constSlabBytes_, cudaMemcpyHostToDevice) != cudaSuccess) {
        throw std::runtime_error("upload of graph constants failed");
    }
    return constSlab_;
}

GraphPipeline::GraphPipeline(uint32_t flags) : flags_(flags) {
    if (GraphProfiler::isEnabled()) {
        profiler_ = std::make_unique<GraphProfiler>();
    }
}

GraphPipeline::~GraphPipeline() {
    profiler_.reset(); // its events go before the constants
    if (constSlab_ != nullptr) {
        cudaFree(constSlab_);
    }
}

/*******************************************************************************
 * Interval planner
 *******************************************************************************/

namespace {

struct ActiveAllocation {
    uint32_t last;
    uint64_t offset;
    uint64_t size;
    uint64_t order;
};
// The allocation that ends first (then the oldest) is on top.
struct EndsLater {
    bool operator()(const ActiveAllocation &l, const ActiveAllocation &r) const {
        return l.last != r.last ? l.last > r.last : l.order > r.order;
    }
};
struct FreeBlock {
    uint64_t offset;
    uint64_t size;
    uint64_t order;
};
struct SmallestFirst {
    bool operator()(const FreeBlock &l, const FreeBlock &r) const {
        return l.size != r.size ? l.size < r.size : l.order < r.order;
    }
};
uint64_t roundUp(uint64_t v, uint64_t a) { return a == 0 ? v : (v + a - 1) / a * a; }

} // namespace

// Same policy as the reference's details::allocateIntervals (graph/interval_memory_planner.cpp:
// 170-216): sort by (first use, larger first, creation order); release allocations whose last use
// precedes the interval's first use into a free list; take the smallest free block that fits and
// split off the remainder (blocks are never merged); otherwise grow the arena.  Tensors no
// operator touches get their own storage at the end.
AllocationPlan allocateIntervals(std::vector<LiveInterval> intervals, const std::vector<UnseenAllocation> &unseen,
                                 uint64_t alignment) {
    std::stable_sort(intervals.begin(), intervals.end(), [](const LiveInterval &l, const LiveInterval &r) {
        if (l.first != r.first) {
            return l.first < r.first;
        }
        if (l.size != r.size) {
            return l.size > r.size;
        }
        return l.order < r.order;
    });
    AllocationPlan plan;
    std::priority_queue<ActiveAllocation, std::vector<ActiveAllocation>, EndsLater> active;
    std::multiset<FreeBlock, SmallestFirst> freeBlocks;
    uint64_t freeOrder = 0;
    for (const auto &iv : intervals) {
        while (!active.empty() && active.top().last < iv.first) {
            freeBlocks.insert({active.top().offset, active.top().size, freeOrder++});
            active.pop();
        }
        uint64_t offset = UINT64_MAX;
        auto it = freeBlocks.lower_bound(FreeBlock{0, iv.size, 0});
        if (it != freeBlocks.end()) {
            offset = it->offset;
            if (it->size > iv.size) {
                freeBlocks.insert({it->offset + iv.size, it->size - iv.size, it->order});
            }
            freeBlocks.erase(it);
        } else {
            offset = roundUp(plan.memorySize, alignment);
            plan.memorySize = offset + iv.size;
        }
        plan.offsets[iv.id] = offset;
        active.push({iv.last, offset, iv.size, iv.order});
    }
    for (const auto &u : unseen) {
        const uint64_t offset = roundUp(plan.memorySize, alignment);
        plan.offsets[u.id] = offset;
        plan.memorySize = offset + u.size;
    }
    plan.memorySize = roundUp(plan.memorySize, alignment);
    return plan;
}

} // namespace mlel
