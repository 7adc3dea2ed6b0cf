// Per-operator device-time profiling of data-graph dispatches, the counterpart of the reference's
// GraphProfiler (graph/graph_profiler.cpp).  The reference writes a timestamp query before and after
// every operator's compute dispatch (graph_profiler.cpp:157-191), harvests the queries lazily once the
// submission has completed (:292-338) and returns one JSON document per pipeline (:563-620).  Here the
// timestamps are CUDA events recorded on the dispatching stream around every launched kernel; they are
// read when the document is asked for, after waiting for the recorded work.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

namespace mlel {

class GraphProfiler {
  public:
    // Nanoseconds per tick of the "cycle_count" fields.  CUDA events report elapsed time, so the ticks are
    // nanoseconds since the first profiled dispatch of this pipeline.
    static constexpr double kTimestampPeriodNs = 1.0;

    struct Sample {
        uint64_t submission;
        uint64_t graphDispatch;
        uint32_t pipelineIndex;
        std::string pipelineKind;
        std::string operatorName;
        uint64_t before;
        uint64_t after;
        uint64_t delta;
        double milliseconds;
    };

    // VMEL_GRAPH_PROFILING set to anything but "", 0, false, off, no (any case): graph_profiler.cpp:29-38, 107.
    static bool isEnabled();
    static bool isTruthy(const char *value);

    GraphProfiler() = default;
    ~GraphProfiler();
    GraphProfiler(const GraphProfiler &) = delete;
    GraphProfiler &operator=(const GraphProfiler &) = delete;

    // One profiled dispatch: beginDispatch() records the first timestamp and returns a token;
    // afterOperator() records the timestamp that closes operator `pipelineIndex` (and opens the next).
    size_t beginDispatch(cudaStream_t stream, size_t operatorCount);
    void afterOperator(size_t token, uint32_t pipelineIndex, const std::string &operatorName, cudaStream_t stream);

    // Waits for every recorded dispatch, turns its events into samples, and returns all samples so far.
    const std::vector<Sample> &collect();
    std::string makeJson();
    void clear();

    // The document for a given list of samples; separate from the device so that it can be tested alone.
    static std::string makeJson(const std::vector<Sample> &samples, double timestampPeriodNs);

  private:
    struct Pending {
        uint64_t submission;
        uint64_t graphDispatch;
        std::vector<cudaEvent_t> events; // operatorCount + 1
        std::vector<std::string> names;
        size_t recorded{0};
    };
    void release(Pending &p);

    std::mutex mutex_;
    std::vector<Pending> pending_;
    std::vector<Sample> samples_;
    cudaEvent_t epoch_{nullptr};
};

} // namespace mlel
