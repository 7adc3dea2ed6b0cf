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

class Session {
  public:
    explicit Session(GraphPipeline *pipeline);
    ~Session();

    uint64_t memorySize() const { return memorySize_; }
    uint64_t alignment() const { return kSessionAlignment; }
    bool tensorOffset(int32_t tensor, uint64_t *offset) const;

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
    int resolve(); // fills views_ with device addresses; fails if something is unbound

    GraphPipeline *pipeline_;
    uint64_t memorySize_{0};
    std::map<int32_t, uint64_t> offsets_; // session tensor id -> offset
    char *memory_{nullptr};
    std::map<std::tuple<uint32_t, uint32_t, uint32_t>, char *> external_;
    std::vector<TView> views_;
    bool resolved_{false};
    cudaGraphExec_t graphExec_{nullptr};
    cudaGraph_t graph_{nullptr};
};

const std::string &lastError();

} // namespace mlel
