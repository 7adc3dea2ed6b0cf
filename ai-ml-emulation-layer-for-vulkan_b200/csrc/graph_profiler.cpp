#include "graph_profiler.hpp"

#include <algorithm>
#include <atomic>
#include <cctype>
#include <charconv>
#include <cmath>
#include <cstdlib>
#include <limits>
#include <map>
#include <stdexcept>
#include <utility>

namespace mlel {

namespace {

std::atomic<uint64_t> g_nextSubmission{0};
std::atomic<uint64_t> g_nextGraphDispatch{0};

// ---- a small writer for the one document shape this file produces (two-space indentation, ": " after keys,
// shortest round-trip floating point with a ".0" on whole numbers), which is what the reference's
// nlohmann::ordered_json::dump(2) prints (graph_profiler.cpp:619).

void appendEscaped(std::string &out, const std::string &s) {
    out.push_back('"');
    for (const unsigned char c : s) {
        switch (c) {
        case '"':
            out += "\\\"";
            break;
        case '\\':
            out += "\\\\";
            break;
        case '\n':
            out += "\\n";
            break;
        case '\r':
            out += "\\r";
            break;
        case '\t':
            out += "\\t";
            break;
        default:
            if (c < 0x20) {
                static const char *hex = "0123456789abcdef";
                out += "\\u00";
                out.push_back(hex[c >> 4]);
                out.push_back(hex[c & 15]);
            } else {
                out.push_back(char(c));
            }
        }
    }
    out.push_back('"');
}

void appendDouble(std::string &out, double v) {
    if (!std::isfinite(v)) {
        out += "null";
        return;
    }
    char buf[40];
    const auto r = std::to_chars(buf, buf + sizeof(buf), v);
    std::string text(buf, r.ptr);
    if (text.find_first_of(".eE") == std::string::npos) {
        text += ".0";
    }
    out += text;
}

struct ObjectWriter {
    std::string &out;
    std::string indent;
    bool first{true};
    ObjectWriter(std::string &o, std::string ind) : out(o), indent(std::move(ind)) { out += "{"; }
    void key(const char *k) {
        out += first ? "\n" : ",\n";
        first = false;
        out += indent + "  ";
        appendEscaped(out, k);
        out += ": ";
    }
    void field(const char *k, uint64_t v) {
        key(k);
        out += std::to_string(v);
    }
    void field(const char *k, double v) {
        key(k);
        appendDouble(out, v);
    }
    void field(const char *k, const std::string &v) {
        key(k);
        appendEscaped(out, v);
    }
    void close() { out += first ? "}" : "\n" + indent + "}"; }
};

struct Aggregate {
    uint64_t count{0};
    double total{0.0};
    double min{std::numeric_limits<double>::max()};
    double max{0.0};
};

} // namespace

bool GraphProfiler::isTruthy(const char *value) {
    if (value == nullptr || value[0] == '\0') {
        return false;
    }
    std::string s(value);
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return char(std::tolower(c)); });
    return s != "0" && s != "false" && s != "off" && s != "no";
}

bool GraphProfiler::isEnabled() { return isTruthy(std::getenv("VMEL_GRAPH_PROFILING")); }

GraphProfiler::~GraphProfiler() {
    for (auto &p : pending_) {
        release(p);
    }
    if (epoch_ != nullptr) {
        cudaEventDestroy(epoch_);
    }
}

void GraphProfiler::release(Pending &p) {
    for (auto e : p.events) {
        if (e != nullptr) {
            cudaEventDestroy(e);
        }
    }
    p.events.clear();
}

size_t GraphProfiler::beginDispatch(cudaStream_t stream, size_t operatorCount) {
    std::lock_guard<std::mutex> lock(mutex_);
    Pending p;
    p.submission = g_nextSubmission++;
    p.graphDispatch = g_nextGraphDispatch++;
    p.events.assign(operatorCount + 1, nullptr);
    p.names.resize(operatorCount);
    for (auto &e : p.events) {
        if (cudaEventCreate(&e) != cudaSuccess) {
            release(p);
            throw std::runtime_error("graph profiling: cannot create a CUDA event");
        }
    }
    if (epoch_ == nullptr) {
        if (cudaEventCreate(&epoch_) != cudaSuccess) {
            release(p);
            throw std::runtime_error("graph profiling: cannot create a CUDA event");
        }
        cudaEventRecord(epoch_, stream);
    }
    cudaEventRecord(p.events[0], stream);
    pending_.push_back(std::move(p));
    return pending_.size() - 1;
}

void GraphProfiler::afterOperator(size_t token, uint32_t pipelineIndex, const std::string &operatorName,
                                  cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(mutex_);
    Pending &p = pending_.at(token);
    cudaEventRecord(p.events.at(size_t(pipelineIndex) + 1), stream);
    p.names.at(pipelineIndex) = operatorName.empty() ? "UNKNOWN" : operatorName; // graph_profiler.cpp:40-45
    p.recorded = std::max(p.recorded, size_t(pipelineIndex) + 1);
}

const std::vector<GraphProfiler::Sample> &GraphProfiler::collect() {
    std::lock_guard<std::mutex> lock(mutex_);
    for (auto &p : pending_) {
        if (p.recorded > 0 && cudaEventSynchronize(p.events[p.recorded]) == cudaSuccess) {
            float sinceEpoch = 0.0f;
            cudaEventElapsedTime(&sinceEpoch, epoch_, p.events[0]);
            // Ticks are nanoseconds.  Each operator's own duration is read directly (not as a difference of two
            // large numbers) and the running sum gives the absolute ticks, so that delta == after - before.
            uint64_t before = uint64_t(std::llround(std::max(0.0, double(sinceEpoch)) * 1.0e6));
            for (size_t k = 0; k < p.recorded; ++k) {
                float ms = 0.0f;
                cudaEventElapsedTime(&ms, p.events[k], p.events[k + 1]);
                const uint64_t delta = uint64_t(std::llround(std::max(0.0, double(ms)) * 1.0e6));
                const uint64_t after = before + delta;
                samples_.push_back({p.submission, p.graphDispatch, uint32_t(k), "tosa", p.names[k], before, after,
                                    delta, double(delta) * kTimestampPeriodNs / 1000000.0});
                before = after;
            }
        }
        release(p);
    }
    pending_.clear();
    return samples_;
}

void GraphProfiler::clear() {
    std::lock_guard<std::mutex> lock(mutex_);
    for (auto &p : pending_) {
        release(p);
    }
    pending_.clear();
    samples_.clear();
}

std::string GraphProfiler::makeJson() {
    const auto &samples = collect();
    return makeJson(samples, kTimestampPeriodNs);
}

// Document layout of the reference (graph_profiler.cpp:563-620): "timestamp_period_ns", "samples" in the order
// they were taken, "by_operator" keyed and ordered by (pipeline_kind, operator_name).
std::string GraphProfiler::makeJson(const std::vector<Sample> &samples, double timestampPeriodNs) {
    std::map<std::pair<std::string, std::string>, Aggregate> aggregates;
    for (const auto &s : samples) {
        auto &a = aggregates[{s.pipelineKind, s.operatorName}];
        a.count++;
        a.total += s.milliseconds;
        a.min = std::min(a.min, s.milliseconds);
        a.max = std::max(a.max, s.milliseconds);
    }
    std::string out;
    out += "{\n  \"timestamp_period_ns\": ";
    appendDouble(out, timestampPeriodNs);
    out += ",\n  \"samples\": [";
    bool first = true;
    for (const auto &s : samples) {
        out += first ? "\n    " : ",\n    ";
        first = false;
        ObjectWriter w(out, "    ");
        w.field("submission", s.submission);
        w.field("graph_dispatch", s.graphDispatch);
        w.field("pipeline_index", uint64_t(s.pipelineIndex));
        w.field("pipeline_kind", s.pipelineKind);
        w.field("operator_name", s.operatorName);
        w.field("cycle_count_before", s.before);
        w.field("cycle_count_after", s.after);
        w.field("cycle_count_delta", s.delta);
        w.field("time_ms", s.milliseconds);
        w.close();
    }
    out += first ? "]" : "\n  ]";
    out += ",\n  \"by_operator\": [";
    first = true;
    for (const auto &[key, a] : aggregates) {
        out += first ? "\n    " : ",\n    ";
        first = false;
        const bool has = a.count > 0;
        ObjectWriter w(out, "    ");
        w.field("pipeline_kind", key.first);
        w.field("operator_name", key.second);
        w.field("dispatch_count", a.count);
        w.field("total_time_ms", a.total);
        w.field("average_time_ms", has ? a.total / double(a.count) : 0.0);
        w.field("min_time_ms", has ? a.min : 0.0);
        w.field("max_time_ms", has ? a.max : 0.0);
        w.close();
    }
    out += first ? "]" : "\n  ]";
    out += "\n}";
    return out;
}

} // namespace mlel
