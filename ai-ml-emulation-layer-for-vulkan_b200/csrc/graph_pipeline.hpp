// Host-side graph layer: the counterpart of the reference's GraphPipeline
// (graph/compute_graph_op.hpp:1204-1549) without Vulkan objects.  It records the operator
// list in creation (= SPIR-V) order, owns constant tensors, tracks application ("external")
// tensors by (set, binding, array index) and session tensors in creation order — the order the
// interval planner depends on (graph/interval_memory_planner.cpp:73-115).
#pragma once

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "graph_profiler.hpp"
#include "ops.hpp"

namespace mlel {

enum class TensorClass : int32_t { External = 0, Constant = 1, Session = 2 };

// Counterpart of graph/tensor.hpp:61-113 TensorDescriptor.
struct TensorDescriptor {
    int32_t id{-1};
    int32_t dtype{MLEL_I8};
    std::vector<int64_t> dims;
    std::vector<int64_t> strides; // bytes
    TensorClass cls{TensorClass::Session};
    uint32_t set{0}, binding{0}, arrayIndex{0}; // External only
    std::vector<uint8_t> hostData;              // Constant only
    uint64_t constOffset{0};                    // Constant only: offset in the pipeline's device slab
    int32_t sessionOrder{-1};                   // Session only: index in creation order
    bool isGraphInput{false};
    bool isGraphOutput{false};

    int rank() const { return int(dims.size()); }
    int64_t numel() const;
    // graph/tensor.cpp:193-199 getSize(): dims[0] * strides[0]
    uint64_t sizeBytes() const;
    bool packed() const;
};

class UnsupportedError : public std::runtime_error {
  public:
    using std::runtime_error::runtime_error;
};

// Who reads and writes a tensor, by operator index (the fusion pass).
struct UseInfo {
    std::vector<int> consumers; // op indices reading the tensor
    int producers{0};
};

class GraphPipeline {
  public:
    explicit GraphPipeline(uint32_t flags);
    GraphPipeline(const GraphPipeline &) = delete;
    GraphPipeline &operator=(const GraphPipeline &) = delete;

    // Present when VMEL_GRAPH_PROFILING was truthy at creation (graph/graph_layer.cpp:318-322); every
    // dispatch of a session of this pipeline is then timed operator by operator.
    GraphProfiler *profiler() { return profiler_.get(); }

    // --- tensors (names follow the reference) ---
    int32_t makeConstTensor(uint32_t id, const mlel_tensor_desc &desc, const void *data);
    int32_t getConstTensor(uint32_t id) const;
    int32_t makeConstCompositeTensor(int32_t dtype, const std::vector<int64_t> &dims, const void *data);
    int32_t makeDescriptorSetBinding(uint32_t set, uint32_t binding, uint32_t arrayIndex,
                                     const mlel_tensor_desc &desc);
    int32_t getTensor(uint32_t set, uint32_t binding, uint32_t arrayIndex = 0) const;
    int32_t makeTensor(int32_t dtype, const std::vector<int64_t> &dims, const std::vector<int64_t> &strides = {});
    void makeInput(int32_t tensor);
    void makeOutput(int32_t tensor);

    // --- TOSA operators: argument lists of graph/compute_graph_op.hpp:1249-1483 ---
    void makeConv2D(int32_t input, int32_t output, int32_t weights, int32_t biases, const std::vector<int32_t> &pad,
                    const std::vector<int32_t> &stride, const std::vector<int32_t> &dilation, int8_t inputZeroPoint,
                    int8_t weightZeroPoint, uint32_t accType, const std::string &debugName);
    void makeDepthwiseConv2D(int32_t input, int32_t output, int32_t weights, int32_t biases,
                             const std::vector<int32_t> &pad, const std::vector<int32_t> &stride,
                             const std::vector<int32_t> &dilation, int8_t inputZeroPoint, int8_t weightZeroPoint,
                             uint32_t accType, const std::string &debugName);
    void makeMatmul(int32_t input1, int32_t input2, int32_t output, int32_t inputZeroPoint1, int32_t inputZeroPoint2,
                    const std::string &debugName);
    void makeRescale(int32_t input, int32_t output, int32_t inputZeroPoint, int32_t outputZeroPoint,
                     int32_t multiplier, int32_t shift, bool scale32, bool doubleRound, bool perChannel,
                     bool inputUnsigned, bool outputUnsigned, const std::string &debugName);
    void makeAvgPool2D(int32_t input, int32_t output, const std::vector<int32_t> &kernel,
                       const std::vector<int32_t> &stride, const std::vector<int32_t> &pad, uint32_t accType,
                       int8_t inputZeroPoint, int8_t outputZeroPoint, const std::string &debugName);
    void makeMaxPool2D(int32_t input, int32_t output, const std::vector<int32_t> &kernel,
                       const std::vector<int32_t> &stride, const std::vector<int32_t> &pad, uint32_t nanMode,
                       const std::string &debugName);
    void makeTable(int32_t input, int32_t output, int32_t table, const std::string &debugName);
    void makeTranspose(int32_t input, int32_t output, const std::vector<uint32_t> &perms,
                       const std::string &debugName);
    void makeConcat(const std::vector<int32_t> &inputs, int32_t output, uint32_t axis, const std::string &debugName);
    void makeClamp(int32_t input, int32_t output, double min, double max, uint32_t nanMode,
                   const std::string &debugName);
    void makeBinary(BinaryOp op, int32_t input1, int32_t input2, int32_t output, uint32_t nanMode,
                    const std::string &debugName);
    void makeUnary(UnaryOp op, int32_t input, int32_t output, const std::string &debugName);
    void makeMul(int32_t input1, int32_t input2, int32_t output, uint32_t shift, const std::string &debugName);
    void makeReduce(ReduceOp op, int32_t input, int32_t output, uint32_t axis, uint32_t nanMode,
                    const std::string &debugName);
    void makeCast(int32_t input, int32_t output, const std::string &debugName);
    void makeReshape(int32_t input, int32_t output, const std::string &debugName);
    void makeSlice(int32_t input, int32_t output, const std::vector<uint32_t> &start, const std::string &debugName);
    void makePad(int32_t input, int32_t output, int32_t padding, double padConst, int32_t padConstInt,
                 const std::string &debugName);
    void makeArithmeticRightShift(int32_t input1, int32_t input2, int32_t output, bool round,
                                  const std::string &debugName);
    void makeNegate(int32_t input, int32_t output, int32_t inputZeroPoint, int32_t outputZeroPoint,
                    const std::string &debugName);
    void makeSelect(int32_t input1, int32_t input2, int32_t input3, int32_t output, const std::string &debugName);
    void makeFft2D(int32_t inputReal, int32_t inputImag, int32_t outputReal, int32_t outputImag, bool inverse,
                   const std::string &debugName);
    void makeRfft2D(int32_t input, int32_t outputReal, int32_t outputImag, const std::string &debugName);
    void makeArgmax(int32_t input, int32_t output, uint32_t axis, uint32_t nanMode, const std::string &debugName);
    void makeGather(int32_t values, int32_t indices, int32_t output, const std::string &debugName);
    void makeScatter(int32_t input, int32_t values, int32_t indices, int32_t output, const std::string &debugName);
    void makeReverse(int32_t input, int32_t output, uint32_t axis, const std::string &debugName);
    void makeTile(int32_t input, int32_t output, const std::string &debugName);
    void makeResize(int32_t input, int32_t output, const std::vector<int32_t> &scale,
                    const std::vector<int32_t> &offset, const std::vector<int32_t> &border, uint32_t mode,
                    const std::string &debugName);
    void makeTransposeConv2D(int32_t input, int32_t output, int32_t weights, int32_t biases,
                             const std::vector<int32_t> &outPad, const std::vector<int32_t> &stride,
                             int8_t inputZeroPoint, int8_t weightZeroPoint, uint32_t accType,
                             const std::string &debugName);
    void makeConv3D(int32_t input, int32_t output, int32_t weights, int32_t biases, const std::vector<int32_t> &pad,
                    const std::vector<int32_t> &stride, const std::vector<int32_t> &dilation, int8_t inputZeroPoint,
                    int8_t weightZeroPoint, uint32_t accType, const std::string &debugName);

    // --- access ---
    const std::vector<OpDesc> &getPipelines() const { return ops_; }   // logical op list
    const std::vector<OpDesc> &getExecList();                           // after fusion (finalises)
    const std::vector<int32_t> &getTensors() const { return sessionTensors_; }
    const TensorDescriptor &tensor(int32_t id) const { return *tensors_.at(size_t(id)); }
    TensorDescriptor &tensor(int32_t id) { return *tensors_.at(size_t(id)); }
    int32_t tensorCount() const { return int32_t(tensors_.size()); }
    const std::vector<int32_t> &graphInputs() const { return inputs_; }
    const std::vector<int32_t> &graphOutputs() const { return outputs_; }
    uint32_t flags() const { return flags_; }
    bool finalized() const { return finalized_; }

    // Constants on the device: one slab, uploaded on first use (with the device current then).
    void finalize();
    char *constantBase();
    ~GraphPipeline();

  private:
    int32_t addTensor(std::unique_ptr<TensorDescriptor> t);
    OpDesc &pushOp(OpKind kind, const std::string &name, std::vector<int32_t> in, std::vector<int32_t> out);
    void requireMutable() const;
    void fuse();
    void fuseRowRuns(std::vector<int> &group, const std::vector<UseInfo> &uses,
                     const std::function<void(OpDesc, const std::vector<int> &)> &emit);
    void prepareTensorCore();
    void buildResidualTable(OpDesc &op);
    int32_t addDerivedConstant(int32_t dtype, const std::vector<int64_t> &dims, const void *data);
    int32_t addScratchTensor(int32_t dtype, const std::vector<int64_t> &dims);

    uint32_t flags_;
    std::unique_ptr<GraphProfiler> profiler_;
    bool finalized_{false};
    std::vector<std::unique_ptr<TensorDescriptor>> tensors_;
    std::vector<int32_t> sessionTensors_;
    std::map<uint32_t, int32_t> constTensorMap_;
    std::map<std::tuple<uint32_t, uint32_t, uint32_t>, int32_t> externalMap_;
    std::vector<int32_t> inputs_, outputs_;
    std::vector<OpDesc> ops_;
    std::vector<OpDesc> exec_;
    char *constSlab_{nullptr};
    uint64_t constSlabBytes_{0};
    int constDevice_{-1};
};

// details::allocateIntervals, graph/interval_memory_planner.cpp:170-216
struct LiveInterval {
    uint64_t id;
    uint32_t first;
    uint32_t last;
    uint64_t size;
    uint64_t order;
};
struct UnseenAllocation {
    uint64_t id;
    uint64_t size;
};
struct AllocationPlan {
    uint64_t memorySize{0};
    std::map<uint64_t, uint64_t> offsets;
};
AllocationPlan allocateIntervals(std::vector<LiveInterval> intervals, const std::vector<UnseenAllocation> &unseen,
                                 uint64_t alignment);

// Lowers SPIR-V assembly text through the TOSA.001000.1 registry into `pipeline`.
void lowerSpvasm(GraphPipeline &pipeline, const std::string &text);

// TOSA registry queries
bool extInstSetRegistered(const std::string &importName);
const std::vector<std::string> &tosaOpNames();
bool tosaOpSupported(const std::string &name);

// Session memory alignment: the reference takes the maximum tensor alignment reported by the
// Vulkan device; on the CUDA side every session tensor is placed on a 256-byte boundary so
// that 16-byte vector access and TMA descriptors are always legal.
constexpr uint64_t kSessionAlignment = 256;

} // namespace mlel
