#include "session.hpp"

#include "kernels/gemm_i8_tcgen05.hpp"

#include <algorithm>
#include <cstdlib>
#include <set>
#include <string>

namespace mlel {

namespace {
uint64_t roundUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
} // namespace

Session::Session(GraphPipeline *pipeline) : pipeline_(pipeline) {
    pipeline_->finalize();
    plan();
    // Counters of the tile-level hand-over, if two tensor-core convolutions follow each other anywhere in the list.
    // Made here and not at the first dispatch, which may run inside a stream capture.  Without them (no
    // device, no memory) the dispatch simply does without the hand-over.
    const auto &exec = pipeline_->getExecList();
    // one counter per 128 output pixels (the narrowest tile) of every convolution whose output the next one reads
    size_t words = 0;
    for (size_t k = 0; k + 1 < exec.size(); ++k) {
        if (exec[k].tc != 0 && exec[k + 1].tc != 0 && !exec[k].out.empty() && !exec[k + 1].in.empty() &&
            exec[k + 1].in[0] == exec[k].out[0]) {
            const TensorDescriptor &out = pipeline_->tensor(exec[k].out[0]);
            int64_t pixels = 1;
            for (int i = 0; i + 1 < out.rank(); ++i) {
                pixels *= out.dims[size_t(i)];
            }
            words += size_t((pixels + 127) / 128);
        }
    }
    if (words != 0 && (cudaMalloc(&progressWords_, words * sizeof(uint32_t)) != cudaSuccess ||
                       cudaMemset(progressWords_, 0, words * sizeof(uint32_t)) != cudaSuccess)) {
        if (progressWords_ != nullptr) {
            cudaFree(progressWords_);
        }
        progressWords_ = nullptr;
        cudaGetLastError();
    }
    progressCapacity_ = progressWords_ != nullptr ? words : 0;
}

Session::~Session() {
    dropGraphs();
    if (progressWords_ != nullptr) {
        cudaFree(progressWords_);
    }
}

void Session::dropGraphs() {
    for (auto &entry : graphs_) {
        if (entry.second.exec != nullptr) {
            cudaGraphExecDestroy(entry.second.exec);
        }
        if (entry.second.graph != nullptr) {
            cudaGraphDestroy(entry.second.graph);
        }
    }
    graphs_.clear();
}

std::vector<const void *> Session::bindingKey() const {
    std::vector<const void *> key{memory_};
    for (const auto &entry : external_) {
        key.push_back(entry.second);
    }
    return key;
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

    // With fusion on, a RESHAPE between two packed session tensors of one size moves no bytes: its result shares
    // its input's storage (the launch skips the copy when both addresses are equal), and the shared storage
    // lives as long as either tensor.  Chains of such RESHAPEs resolve to the first tensor.
    std::map<int32_t, int32_t> aliasOf;
    if (!(pipeline_->flags() & MLEL_PIPELINE_NO_FUSION)) {
        for (const auto &op : exec) {
            if (op.kind != OP_RESHAPE || op.in.empty() || op.out.empty()) {
                continue;
            }
            const int32_t src = op.in[0], dst = op.out[0];
            if (src < 0 || dst < 0 || src == dst) {
                continue;
            }
            const TensorDescriptor &a = pipeline_->tensor(src), &b = pipeline_->tensor(dst);
            if (a.cls != TensorClass::Session || b.cls != TensorClass::Session || !a.packed() || !b.packed() ||
                a.dtype != b.dtype || a.sizeBytes() != b.sizeBytes()) {
                continue;
            }
            const auto rootIt = aliasOf.find(src);
            const int32_t root = rootIt != aliasOf.end() ? rootIt->second : src;
            if (!ranges.count(root) || !ranges.count(dst)) {
                continue;
            }
            aliasOf[dst] = root;
            auto &r = ranges[root];
            const auto d = ranges[dst];
            r.first = std::min(r.first, d.first);
            r.second = std::max(r.second, d.second);
            ranges.erase(dst);
        }
    }

    // One record per session tensor that needs storage, in session-tensor order.
    planned_.clear();
    for (size_t order = 0; order < sessionTensors.size(); ++order) {
        const int32_t t = sessionTensors[order];
        const uint64_t size = roundUp(pipeline_->tensor(t).sizeBytes(), kSessionAlignment);
        const auto it = ranges.find(t);
        if (it != ranges.end()) {
            planned_.push_back({t, 0, size, it->second.first, it->second.second, true});
        } else if (pipeline_->flags() & MLEL_PIPELINE_NO_FUSION) {
            planned_.push_back({t, 0, size, 0, 0, false});
        }
        // With fusion on, a tensor nothing touches was elided and needs no storage.
    }
    planner_ = plannerFromEnvironment();
    switch (planner_) {
    case PlannerKind::Linear:
        planLinear();
        break;
    case PlannerKind::BestFit:
        planBestFit();
        break;
    case PlannerKind::Interval:
        planInterval();
        break;
    }
    offsets_.clear();
    for (const auto &p : planned_) {
        offsets_[p.tensor] = p.offset;
    }
    for (const auto &alias : aliasOf) {
        const auto it = offsets_.find(alias.second);
        if (it != offsets_.end()) {
            offsets_[alias.first] = it->second;
        }
    }
}

// The session's planner is chosen by VMEL_MEMORY_PLANNER exactly as the reference chooses it
// (graph/graph_layer.cpp:282-297): "Linear", "BestFit", anything else (or unset) = interval.
PlannerKind plannerFromEnvironment() {
    const char *name = std::getenv("VMEL_MEMORY_PLANNER");
    if (name != nullptr && std::string(name) == "Linear") {
        return PlannerKind::Linear;
    }
    if (name != nullptr && std::string(name) == "BestFit") {
        return PlannerKind::BestFit;
    }
    return PlannerKind::Interval;
}

const char *plannerName(PlannerKind kind) {
    switch (kind) {
    case PlannerKind::Linear:
        return "Linear";
    case PlannerKind::BestFit:
        return "BestFit";
    case PlannerKind::Interval:
        break;
    }
    return "Interval";
}

void Session::planInterval() {
    std::vector<LiveInterval> intervals;
    std::vector<UnseenAllocation> unseen;
    for (size_t k = 0; k < planned_.size(); ++k) {
        const auto &p = planned_[k];
        if (p.seen) {
            intervals.push_back({uint64_t(k), p.first, p.last, p.size, uint64_t(k)});
        } else {
            unseen.push_back({uint64_t(k), p.size});
        }
    }
    const AllocationPlan plan = allocateIntervals(std::move(intervals), unseen, kSessionAlignment);
    memorySize_ = plan.memorySize;
    for (const auto &[k, offset] : plan.offsets) {
        planned_[size_t(k)].offset = offset;
    }
}

// Every tensor gets storage of its own, one after the other (LinearMemoryPlanner,
// graph/memory_planner.cpp:52-98).  Sizes are already multiples of the alignment.
void Session::planLinear() {
    uint64_t offset = 0;
    for (auto &p : planned_) {
        p.offset = offset;
        offset += p.size;
    }
    memorySize_ = offset;
}

// Best fit (BestFitMemoryPlanner, graph/memory_planner.cpp:239-263, 284-310, 352-381): tensors are
// taken largest first; each looks, among the already placed tensors that are at least as large and
// that it may share memory with, for the smallest one whose slot holds only tensors it may share
// with, and moves in at that slot's address; if there is none it opens a new slot at the end.
// Two tensors may share memory when their live ranges over the launched operator list do not
// intersect -- the relation the reference derives by passing tensor references along the graph's
// edges (memory_planner.cpp:154-237) stated on the linear execution order that a stream gives.
// A tensor no operator touches never shares.
void Session::planBestFit() {
    std::vector<size_t> order(planned_.size());
    for (size_t k = 0; k < order.size(); ++k) {
        order[k] = k;
    }
    std::stable_sort(order.begin(), order.end(),
                     [&](size_t a, size_t b) { return planned_[a].size > planned_[b].size; });
    const auto mayShare = [&](size_t a, size_t b) {
        const auto &x = planned_[a];
        const auto &y = planned_[b];
        return x.seen && y.seen && (x.last < y.first || y.last < x.first);
    };
    std::vector<int> slotOf(planned_.size(), -1);
    std::vector<std::vector<size_t>> slots; // occupants of each slot; all share the slot's address
    std::vector<size_t> placed;             // tensors placed so far, smallest first (stable)
    uint64_t end = 0;
    for (const size_t k : order) {
        int chosen = -1;
        for (const size_t alt : placed) {
            if (planned_[alt].size < planned_[k].size || !mayShare(k, alt)) {
                continue;
            }
            const auto &occupants = slots[size_t(slotOf[alt])];
            if (std::all_of(occupants.begin(), occupants.end(), [&](size_t o) { return mayShare(k, o); })) {
                chosen = slotOf[alt];
                planned_[k].offset = planned_[alt].offset;
                break;
            }
        }
        if (chosen < 0) {
            chosen = int(slots.size());
            slots.emplace_back();
            planned_[k].offset = end;
            end += planned_[k].size;
        }
        slotOf[k] = chosen;
        slots[size_t(chosen)].push_back(k);
        // keep `placed` sorted by size ascending; among equal sizes earlier placements come first
        const auto pos = std::upper_bound(placed.begin(), placed.end(), k, [&](size_t a, size_t b) {
            return planned_[a].size < planned_[b].size;
        });
        placed.insert(pos, k);
    }
    memorySize_ = end;
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
    const auto &exec = pipeline_->getExecList();
    GraphProfiler *profiler = pipeline_->profiler();
    if (profiler != nullptr) {
        // The reference wraps every operator's dispatch in a pair of timestamp writes when profiling is on
        // (graph/graph_profiler.cpp:157-191); one event after each kernel closes it and opens the next.
        const size_t token = profiler->beginDispatch(stream, exec.size());
        for (size_t k = 0; k < exec.size(); ++k) {
            const int r = launchOp(exec[k], views_.data(), stream);
            if (r != MLEL_SUCCESS) {
                return r;
            }
            profiler->afterOperator(token, uint32_t(k), exec[k].name, stream);
        }
        return MLEL_SUCCESS;
    }
    // Consecutive convolutions hand their output over tile by tile where the kernels can (LaunchChain).  The
    // counters are the session's own (allocated with the session), zeroed in stream order before the first kernel.
    LaunchChain chain{};
    if (progressWords_ != nullptr) {
        if (cudaMemsetAsync(progressWords_, 0, progressCapacity_ * sizeof(uint32_t), stream) != cudaSuccess) {
            setLastError("cudaMemsetAsync of the progress counters failed");
            return MLEL_ERROR_DEVICE;
        }
        chain.words = progressWords_;
        chain.capacity = progressCapacity_;
    }
    for (size_t k = 0; k < exec.size(); ++k) {
        const OpDesc &op = exec[k];
        // does the next operator read this one's output as the pixel operand of a tensor-core convolution?
        chain.publishNext = k + 1 < exec.size() && exec[k + 1].tc != 0 &&
                            (exec[k + 1].kind == OP_CONV2D || exec[k + 1].kind == OP_FUSED_CONV2D) && !op.out.empty() &&
                            !exec[k + 1].in.empty() && exec[k + 1].in[0] == op.out[0];
        const int r = launchOp(op, views_.data(), stream, chain.words != nullptr ? &chain : nullptr);
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
    if (pipeline_->profiler() != nullptr) {
        return dispatch(stream); // timestamps go between the kernels, which a replayed graph has no place for
    }
    int rc = resolve();
    if (rc != MLEL_SUCCESS) {
        return rc;
    }
    // A captured graph holds the addresses that were bound when it was taken: one graph per set of bindings.
    constexpr size_t kMaxCapturedGraphs = 64;
    const std::vector<const void *> key = bindingKey();
    auto found = graphs_.find(key);
    if (found == graphs_.end()) {
        if (graphs_.size() >= kMaxCapturedGraphs) {
            // Make room for one: the entry that was launched longest ago goes.  Its last launch may still be running
            // on the caller's stream, so wait for that stream before the executable graph is destroyed.
            auto oldest = graphs_.begin();
            for (auto it = graphs_.begin(); it != graphs_.end(); ++it) {
                if (it->second.lastUse < oldest->second.lastUse) {
                    oldest = it;
                }
            }
            cudaStreamSynchronize(stream);
            if (oldest->second.exec != nullptr) {
                cudaGraphExecDestroy(oldest->second.exec);
            }
            if (oldest->second.graph != nullptr) {
                cudaGraphDestroy(oldest->second.graph);
            }
            graphs_.erase(oldest);
        }
        CapturedGraph captured;
        cudaStream_t capture = nullptr;
        if (cudaStreamCreateWithFlags(&capture, cudaStreamNonBlocking) != cudaSuccess) {
            setLastError("cudaStreamCreate failed");
            return MLEL_ERROR_DEVICE;
        }
        cudaError_t err = cudaStreamBeginCapture(capture, cudaStreamCaptureModeThreadLocal);
        if (err == cudaSuccess) {
            rc = dispatch(capture);
            err = cudaStreamEndCapture(capture, &captured.graph);
        }
        if (err == cudaSuccess && rc == MLEL_SUCCESS) {
            err = cudaGraphInstantiate(&captured.exec, captured.graph, 0);
        }
        cudaStreamDestroy(capture);
        if (rc != MLEL_SUCCESS || err != cudaSuccess) {
            if (captured.exec != nullptr) {
                cudaGraphExecDestroy(captured.exec);
            }
            if (captured.graph != nullptr) {
                cudaGraphDestroy(captured.graph);
            }
            if (rc != MLEL_SUCCESS) {
                return rc;
            }
            setLastError(std::string("CUDA graph capture failed: ") + cudaGetErrorString(err));
            return MLEL_ERROR_DEVICE;
        }
        found = graphs_.emplace(key, captured).first;
    }
    found->second.lastUse = ++useCounter_;
    if (cudaGraphLaunch(found->second.exec, stream) != cudaSuccess) {
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
