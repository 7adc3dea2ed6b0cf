#include "session.hpp"

#include <algorithm>
#include <set>

namespace mlel {

namespace {
uint64_t roundUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
} // namespace

Session::Session(GraphPipeline *pipeline) : pipeline_(pipeline) {
    pipeline_->finalize();
    plan();
}

Session::~Session() {
    if (graphExec_ != nullptr) {
        cudaGraphExecDestroy(graphExec_);
    }
    if (graph_ != nullptr) {
        cudaGraphDestroy(graph_);
    }
}

// Live range of a session tensor = [first, last] execution index over {inputs node = 0,
// operators 1..n, outputs node = n + 1} that touch it (graph/interval_memory_planner.cpp:53-115).
// The operator list used is the one that is actually launched: with fusion on, an elided
// intermediate is touched by nothing and the fused node keeps its inputs alive until it runs.
void Session::plan() {
    const auto &exec = pipeline_->getExecList();
    const auto &sessionTensors = pipeline_->getTensors();
    std::map<int32_t, std::pair<uint32_t, uint32_t>> ranges;
    const auto touch = [&](int32_t t, uint32_t index) {
        if (t < 0 || pipeline_->tensor(t).cls != TensorClass::Session) {
            return;
        }
        auto it = ranges.find(t);
        if (it == ranges.end()) {
            ranges[t] = {index, index};
        } else {
            it->second.first = std::min(it->second.first, index);
            it->second.second = std::max(it->second.second, index);
        }
    };
    uint32_t index = 0;
    for (auto t : pipeline_->graphInputs()) {
        touch(t, index);
    }
    ++index;
    for (const auto &op : exec) {
        for (auto t : op.in) {
            touch(t, index);
        }
        for (auto t : op.out) {
            touch(t, index);
        }
        touch(op.epi.shortcutTensor, index);
        touch(op.scratch, index);
        ++index;
    }
    for (auto t : pipeline_->graphOutputs()) {
        touch(t, index);
    }

    std::vector<LiveInterval> intervals;
    std::vector<UnseenAllocation> unseen;
    for (size_t order = 0; order < sessionTensors.size(); ++order) {
        const int32_t t = sessionTensors[order];
        const uint64_t size = roundUp(pipeline_->tensor(t).sizeBytes(), kSessionAlignment);
        const auto it = ranges.find(t);
        if (it != ranges.end()) {
            intervals.push_back({uint64_t(order), it->second.first, it->second.second, size, uint64_t(order)});
        } else if (pipeline_->flags() & MLEL_PIPELINE_NO_FUSION) {
            unseen.push_back({uint64_t(order), size});
        }
        // With fusion on, a tensor nothing touches was elided and needs no storage.
    }
    const AllocationPlan plan = allocateIntervals(std::move(intervals), unseen, kSessionAlignment);
    memorySize_ = plan.memorySize;
    for (const auto &[order, offset] : plan.offsets) {
        offsets_[sessionTensors[size_t(order)]] = offset;
    }
}

bool Session::tensorOffset(int32_t tensor, uint64_t *offset) const {
    const auto it = offsets_.find(tensor);
    if (it == offsets_.end()) {
        return false;
    }
    *offset = it->second;
    return true;
}

void Session::bindMemory(void *memory, uint64_t offset) {
    memory_ = static_cast<char *>(memory) + offset;
    resolved_ = false;
}

void Session::setExternal(uint32_t set, uint32_t binding, uint32_t arrayIndex, void *devicePtr) {
    (void)pipeline_->getTensor(set, binding, arrayIndex); // throws std::out_of_range when unknown
    char *&slot = external_[std::make_tuple(set, binding, arrayIndex)];
    if (slot != static_cast<char *>(devicePtr)) {
        slot = static_cast<char *>(devicePtr);
        resolved_ = false;
    }
}

int Session::resolve() {
    if (resolved_) {
        return MLEL_SUCCESS;
    }
    if (graphExec_ != nullptr) { // bindings changed: the captured graph holds stale addresses
        cudaGraphExecDestroy(graphExec_);
        cudaGraphDestroy(graph_);
        graphExec_ = nullptr;
        graph_ = nullptr;
    }
    const int32_t n = pipeline_->tensorCount();
    views_.assign(size_t(n), TView{});
    char *constBase = pipeline_->constantBase();
    // Only tensors some launched operator touches must be bound.
    std::set<int32_t> used;
    for (const auto &op : pipeline_->getExecList()) {
        used.insert(op.in.begin(), op.in.end());
        used.insert(op.out.begin(), op.out.end());
        for (const FusedRescale *f : {&op.epi.main, &op.epi.a, &op.epi.b, &op.epi.out}) {
            used.insert(f->multTensor);
            used.insert(f->shiftTensor);
        }
        used.insert(op.epi.shortcutTensor);
        used.insert(std::begin(op.aux), std::end(op.aux));
        used.insert(op.scratch);
    }
    used.erase(-1);
    for (int32_t t = 0; t < n; ++t) {
        const TensorDescriptor &td = pipeline_->tensor(t);
        TView &v = views_[size_t(t)];
        v.dtype = td.dtype;
        v.rank = td.rank();
        for (int i = 0; i < td.rank(); ++i) {
            v.dims[i] = uint32_t(td.dims[size_t(i)]);
            v.strides[i] = td.strides[size_t(i)];
        }
        switch (td.cls) {
        case TensorClass::Constant:
            v.ptr = constBase + td.constOffset;
            break;
        case TensorClass::Session: {
            const auto it = offsets_.find(t);
            if (it != offsets_.end()) {
                if (memory_ == nullptr && used.count(t)) {
                    setLastError("session memory is not bound");
                    return MLEL_ERROR_UNKNOWN;
                }
                v.ptr = memory_ + it->second;
            }
            break;
        }
        case TensorClass::External: {
            const auto it = external_.find(std::make_tuple(td.set, td.binding, td.arrayIndex));
            if (it == external_.end() || it->second == nullptr) {
                if (used.count(t)) {
                    setLastError("external tensor (set " + std::to_string(td.set) + ", binding " +
                                 std::to_string(td.binding) + ", element " + std::to_string(td.arrayIndex) +
                                 ") is not bound");
                    return MLEL_ERROR_UNKNOWN;
                }
            } else {
                v.ptr = it->second;
            }
            break;
        }
        }
    }
    resolved_ = true;
    return MLEL_SUCCESS;
}

int Session::dispatch(cudaStream_t stream) {
    const int rc = resolve();
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    // Operators run in creation order on one stream: the stream order is the full
    // write-to-read barrier the reference records between consecutive dispatches
    // (graph/compute_graph_op.cpp:251-299).
    for (const auto &op : pipeline_->getExecList()) {
        const int r = launchOp(op, views_.data(), stream);
        if (r != MLEL_SUCCESS) {
            return r;
        }
    }
    return MLEL_SUCCESS;
}

int Session::dispatchProfiled(cudaStream_t stream, float *msOut, uint32_t capacity) {
    const int rc = resolve();
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    const auto &exec = pipeline_->getExecList();
    if (capacity < exec.size()) {
        setLastError("dispatch_profiled: output array too short");
        return MLEL_INCOMPLETE;
    }
    std::vector<cudaEvent_t> events(exec.size() + 1);
    for (auto &e : events) {
        cudaEventCreate(&e);
    }
    int result = MLEL_SUCCESS;
    cudaEventRecord(events[0], stream);
    for (size_t k = 0; k < exec.size() && result == MLEL_SUCCESS; ++k) {
        result = launchOp(exec[k], views_.data(), stream);
        cudaEventRecord(events[k + 1], stream);
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess && result == MLEL_SUCCESS) {
        setLastError("dispatch_profiled: stream synchronisation failed");
        result = MLEL_ERROR_DEVICE;
    }
    for (size_t k = 0; k < exec.size() && result == MLEL_SUCCESS; ++k) {
        cudaEventElapsedTime(&msOut[k], events[k], events[k + 1]);
    }
    for (auto &e : events) {
        cudaEventDestroy(e);
    }
    return result;
}

int Session::dispatchGraph(cudaStream_t stream) {
    int rc = resolve();
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    if (graphExec_ == nullptr) {
        cudaStream_t capture = nullptr;
        if (cudaStreamCreateWithFlags(&capture, cudaStreamNonBlocking) != cudaSuccess) {
            setLastError("cudaStreamCreate failed");
            return MLEL_ERROR_DEVICE;
        }
        cudaError_t err = cudaStreamBeginCapture(capture, cudaStreamCaptureModeThreadLocal);
        if (err == cudaSuccess) {
            rc = dispatch(capture);
            err = cudaStreamEndCapture(capture, &graph_);
        }
        if (err == cudaSuccess && rc == MLEL_SUCCESS) {
            err = cudaGraphInstantiate(&graphExec_, graph_, 0);
        }
        cudaStreamDestroy(capture);
        if (rc != MLEL_SUCCESS) {
            return rc;
        }
        if (err != cudaSuccess) {
            setLastError(std::string("CUDA graph capture failed: ") + cudaGetErrorString(err));
            return MLEL_ERROR_DEVICE;
        }
    }
    if (cudaGraphLaunch(graphExec_, stream) != cudaSuccess) {
        setLastError("cudaGraphLaunch failed");
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

int Session::runHost(const mlel_host_io *inputs, uint32_t nIn, const mlel_host_io *outputs, uint32_t nOut,
                     cudaStream_t stream) {
    int rc = resolve();
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    const auto devPtr = [&](const mlel_host_io &io, uint64_t *bytes) -> char * {
        const int32_t t = pipeline_->getTensor(io.set, io.binding, io.array_index);
        *bytes = pipeline_->tensor(t).sizeBytes();
        return views_[size_t(t)].ptr;
    };
    for (uint32_t k = 0; k < nIn; ++k) {
        uint64_t bytes = 0;
        char *d = devPtr(inputs[k], &bytes);
        if (d == nullptr || inputs[k].bytes != bytes) {
            setLastError("run_host: input size does not match the bound tensor");
            return MLEL_ERROR_UNKNOWN;
        }
        if (cudaMemcpyAsync(d, inputs[k].host_ptr, bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) {
            setLastError("run_host: host-to-device copy failed");
            return MLEL_ERROR_DEVICE;
        }
    }
    rc = dispatchGraph(stream);
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    for (uint32_t k = 0; k < nOut; ++k) {
        uint64_t bytes = 0;
        char *d = devPtr(outputs[k], &bytes);
        if (d == nullptr || outputs[k].bytes != bytes) {
            setLastError("run_host: output size does not match the bound tensor");
            return MLEL_ERROR_UNKNOWN;
        }
        if (cudaMemcpyAsync(outputs[k].host_ptr, d, bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess) {
            setLastError("run_host: device-to-host copy failed");
            return MLEL_ERROR_DEVICE;
        }
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess) {
        setLastError(std::string("run_host: ") + cudaGetErrorString(cudaGetLastError()));
        return MLEL_ERROR_DEVICE;
    }
    return MLEL_SUCCESS;
}

} // namespace mlel
