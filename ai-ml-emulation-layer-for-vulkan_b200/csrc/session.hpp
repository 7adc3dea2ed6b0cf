// Session: the counterpart of DataGraphPipelineSessionARM (graph/graph_layer.cpp:215-298) and
// of IntervalMemoryPlanner (graph/interval_memory_planner.cpp:222-272).  It plans transient
// memory for the intermediate tensors of a pipeline, takes one device allocation from the
// caller, binds application tensors, and enqueues the operator list on a CUDA stream.
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <tuple>
#include <vector>

#include "graph_pipeline.hpp"

namespace mlel {

// The three session memory planners of the reference (graph/graph_layer.cpp:282-297).
enum class PlannerKind { Interval, Linear, BestFit };
PlannerKind plannerFromEnvironment(); // reads VMEL_MEMORY_PLANNER
const char *plannerName(PlannerKind kind);

// Placement of one session tensor: where it lies in the session memory and over which launches
// (index 0 = graph inputs, 1..n = launched operators, n + 1 = graph outputs) it is alive.
struct PlannedTensor {
    int32_t tensor;
    uint64_t offset;
    uint64_t size;
    uint32_t first;
    uint32_t last;
    bool seen; // false: no launched operator touches it (only kept when fusion is off)
};

class Session {
  public:
    explicit Session(GraphPipeline *pipeline);
    ~Session();

    uint64_t memorySize() const { return memorySize_; }
    uint64_t alignment() const { return kSessionAlignment; }
    bool tensorOffset(int32_t tensor, uint64_t *offset) const;
    PlannerKind planner() const { return planner_; }
    const std::vector<PlannedTensor> &plannedTensors() const { return planned_; }

    void bindMemory(void *memory, uint64_t offset);
    void setExternal(uint32_t set, uint32_t binding, uint32_t arrayIndex, void *devicePtr);

    int dispatch(cudaStream_t stream);
    int dispatchGraph(cudaStream_t stream);
    int dispatchProfiled(cudaStream_t stream, float *msOut, uint32_t capacity);
    int launchCount() const { return int(pipeline_->getExecList().size()); }
    int runHost(const mlel_host_io *inputs, uint32_t nIn, const mlel_host_io *outputs, uint32_t nOut,
                cudaStream_t stream);

  private:
    void plan();
    void planInterval();
    void planLinear();
    void planBestFit();
    int resolve(); // fills views_ with device addresses; fails if something is unbound

    GraphPipeline *pipeline_;
    uint64_t memorySize_{0};
    PlannerKind planner_{PlannerKind::Interval};
    std::vector<PlannedTensor> planned_;
    std::map<int32_t, uint64_t> offsets_; // session tensor id -> offset
    char *memory_{nullptr};
    std::map<std::tuple<uint32_t, uint32_t, uint32_t>, char *> external_;
    std::vector<TView> views_;
    bool resolved_{false};
    // Captured dispatches, one per set of bound addresses (session memory, then every external tensor in key
    // order): a host that alternates between a few input buffers replays a graph for each of them.
    struct CapturedGraph {
        cudaGraph_t graph{nullptr};
        cudaGraphExec_t exec{nullptr};
        uint64_t lastUse{0}; // value of useCounter_ at the last launch: the entry with the smallest one is evicted
    };
    // Counters of the tile-level hand-over between consecutive tensor-core launches (LaunchChain): a small device
    // allocation of the session, made at its first dispatch and zeroed at the start of every dispatch.
    uint32_t *progressWords_{nullptr};
    size_t progressCapacity_{0}; // words: one per 128 output pixels of every convolution that can publish
    uint64_t useCounter_{0};
    std::map<std::vector<const void *>, CapturedGraph> graphs_;
    std::vector<const void *> bindingKey() const;
    void dropGraphs();
};

const std::string &lastError();

} // namespace mlel
