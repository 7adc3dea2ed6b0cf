// extern "C" boundary (declared in include/mlel_b200.h).  Exceptions of the C++ graph layer are
// turned into status codes here; the reference lets std::runtime_error escape its Vulkan entry
// points (graph/graph_layer.cpp:815-964), which a C ABI must not do.
#include <algorithm>
#include <cstring>
#include <memory>
#include <string>
#include <unordered_map>

#include "graph_pipeline.hpp"
#include "kernels/device_common.cuh"
#include "kernels/gemm_i8_tcgen05.hpp"
#include "kernels/kernels.hpp"
#include "session.hpp"

using namespace mlel;

struct mlel_pipeline {
    explicit mlel_pipeline(uint32_t flags) : impl(std::make_shared<GraphPipeline>(flags)) {}
    std::shared_ptr<GraphPipeline> impl;
};

struct mlel_session {
    explicit mlel_session(const std::shared_ptr<GraphPipeline> &p) : pipeline(p), impl(p.get()) {}
    std::shared_ptr<GraphPipeline> pipeline; // a session keeps its pipeline alive (graph_layer.cpp:1326-1327)
    Session impl;
};

namespace {

template <typename F> int guarded(F &&f) {
    try {
        return f();
    } catch (const UnsupportedError &e) {
        setLastError(e.what());
        return MLEL_ERROR_FEATURE_NOT_PRESENT;
    } catch (const std::bad_alloc &) {
        setLastError("out of host memory");
        return MLEL_ERROR_UNKNOWN;
    } catch (const std::exception &e) {
        setLastError(e.what());
        return MLEL_ERROR_UNKNOWN;
    }
}

std::string nameOr(const char *debugName, const char *fallback) {
    return debugName != nullptr && debugName[0] != 0 ? debugName : fallback;
}

template <typename T> std::vector<T> vec(const T *p, size_t n) { return std::vector<T>(p, p + n); }

TView viewOf(const mlel_tensor &t) {
    TView v{};
    v.ptr = static_cast<char *>(t.data);
    v.dtype = t.desc.dtype;
    v.rank = t.desc.rank;
    int64_t stride = dtypeSize(t.desc.dtype);
    for (int i = t.desc.rank - 1; i >= 0; --i) {
        v.dims[i] = uint32_t(t.desc.dims[i]);
        v.strides[i] = t.desc.strides[0] == 0 ? stride : t.desc.strides[i];
        stride *= t.desc.dims[i];
    }
    return v;
}

const std::unordered_map<std::string, BinaryOp> kBinary = {
    {"ADD", BIN_ADD},
    {"POW", BIN_POW},
    {"SUB", BIN_SUB},
    {"BITWISE_AND", BIN_BITWISE_AND},
    {"BITWISE_OR", BIN_BITWISE_OR},
    {"BITWISE_XOR", BIN_BITWISE_XOR},
    {"LOGICAL_AND", BIN_LOGICAL_AND},
    {"LOGICAL_OR", BIN_LOGICAL_OR},
    {"LOGICAL_XOR", BIN_LOGICAL_XOR},
    {"LOGICAL_LEFT_SHIFT", BIN_LOGICAL_LEFT_SHIFT},
    {"LOGICAL_RIGHT_SHIFT", BIN_LOGICAL_RIGHT_SHIFT},
    {"INTDIV", BIN_INTDIV},
    {"MAXIMUM", BIN_MAXIMUM},
    {"MINIMUM", BIN_MINIMUM},
    {"EQUAL", BIN_EQUAL},
    {"GREATER", BIN_GREATER},
    {"GREATER_EQUAL", BIN_GREATER_EQUAL},
};
const std::unordered_map<std::string, UnaryOp> kUnary = {
    {"ABS", UN_ABS},     {"BITWISE_NOT", UN_BITWISE_NOT}, {"CLZ", UN_CLZ},         {"LOGICAL_NOT", UN_LOGICAL_NOT},
    {"CEIL", UN_CEIL},   {"COS", UN_COS},                 {"ERF", UN_ERF},         {"EXP", UN_EXP},
    {"FLOOR", UN_FLOOR}, {"LOG", UN_LOG},                 {"RECIPROCAL", UN_RECIPROCAL},
    {"RSQRT", UN_RSQRT}, {"SIGMOID", UN_SIGMOID},         {"SIN", UN_SIN},         {"TANH", UN_TANH}};
const std::unordered_map<std::string, ReduceOp> kReduce = {
    {"REDUCE_SUM", RED_SUM},         {"REDUCE_MAX", RED_MAX}, {"REDUCE_MIN", RED_MIN},
    {"REDUCE_PRODUCT", RED_PRODUCT}, {"REDUCE_ALL", RED_ALL}, {"REDUCE_ANY", RED_ANY}};

} // namespace

extern "C" {

const char *mlel_last_error(void) { return lastError().c_str(); }
int mlel_elem_size(int32_t dtype) { return elemSize(dtype); }
int mlel_device_error(void) {
    cudaDeviceSynchronize();
    return tcgen05ErrorFlag();
}

int mlel_set_tuning(const char *key, int value) {
    return guarded([&] {
        TensorCoreTuning &t = tensorCoreTuning();
        const std::string k = key != nullptr ? key : "";
        const bool width = value == 0 || value == 128 || value == 192 || value == 256;
        if (k == "pair_kernel" && value >= 0 && value <= 2) {
            t.pairKernel = value;
        } else if (k == "tile_progress" && value >= 0 && value <= 7) {
            t.tileProgress = value;
        } else if (k == "oc_tile_rule" && value >= 0 && value <= 8) {
            t.ocTileRule = value;
        } else if (k == "dependent_launch") {
            t.dependentLaunch = value != 0;
        } else if (k == "pair_tile_pixels" && width) {
            t.pairTilePixels = value;
        } else if (k == "oc_tile_pixels" && width) {
            t.ocTilePixels = value;
        } else {
            setLastError("mlel_set_tuning: unknown key or value: " + k);
            return int(MLEL_ERROR_UNKNOWN);
        }
        return int(MLEL_SUCCESS);
    });
}

long long mlel_tensor_core_launches(int kernel) {
    return kernel >= 0 && kernel < 3 ? g_tensorCoreLaunches[kernel].load(std::memory_order_relaxed) : -1;
}

int mlel_selftest_wait_timeout(void *cuda_stream, int *recorded_code) {
    return guarded([&] { return waitTimeoutSelfTest(static_cast<cudaStream_t>(cuda_stream), recorded_code); });
}

int mlel_pipeline_create(uint32_t flags, mlel_pipeline **out) {
    return guarded([&] {
        *out = new mlel_pipeline(flags);
        return MLEL_SUCCESS;
    });
}

void mlel_pipeline_destroy(mlel_pipeline *p) { delete p; }

int mlel_pipeline_bind_external(mlel_pipeline *p, uint32_t set, uint32_t binding, uint32_t array_index,
                                const mlel_tensor_desc *desc, mlel_tensor_id *out) {
    return guarded([&] {
        const int32_t t = p->impl->makeDescriptorSetBinding(set, binding, array_index, *desc);
        if (out != nullptr) {
            *out = t;
        }
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_get_external(mlel_pipeline *p, uint32_t set, uint32_t binding, uint32_t array_index,
                               mlel_tensor_id *out) {
    return guarded([&] {
        *out = p->impl->getTensor(set, binding, array_index);
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_add_constant(mlel_pipeline *p, uint32_t id, const mlel_tensor_desc *desc, const void *host_data,
                               mlel_tensor_id *out) {
    return guarded([&] {
        const int32_t t = p->impl->makeConstTensor(id, *desc, host_data);
        if (out != nullptr) {
            *out = t;
        }
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_get_constant(mlel_pipeline *p, uint32_t id, mlel_tensor_id *out) {
    return guarded([&] {
        *out = p->impl->getConstTensor(id);
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_make_composite_constant(mlel_pipeline *p, const mlel_tensor_desc *desc, const void *host_data,
                                          mlel_tensor_id *out) {
    return guarded([&] {
        *out = p->impl->makeConstCompositeTensor(desc->dtype, vec(desc->dims, size_t(desc->rank)), host_data);
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_make_tensor(mlel_pipeline *p, const mlel_tensor_desc *desc, mlel_tensor_id *out) {
    return guarded([&] {
        std::vector<int64_t> strides;
        if (desc->strides[0] != 0) {
            strides = vec(desc->strides, size_t(desc->rank));
        }
        *out = p->impl->makeTensor(desc->dtype, vec(desc->dims, size_t(desc->rank)), strides);
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_mark_input(mlel_pipeline *p, mlel_tensor_id t) {
    return guarded([&] {
        p->impl->makeInput(t);
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_mark_output(mlel_pipeline *p, mlel_tensor_id t) {
    return guarded([&] {
        p->impl->makeOutput(t);
        return MLEL_SUCCESS;
    });
}

int mlel_pipeline_lower_spvasm(mlel_pipeline *p, const char *text) {
    return guarded([&] {
        lowerSpvasm(*p->impl, text);
        return MLEL_SUCCESS;
    });
}

int mlel_ext_inst_set_registered(const char *import_name) { return extInstSetRegistered(import_name) ? 1 : 0; }
int mlel_tosa_op_count(void) { return int(tosaOpNames().size()); }
const char *mlel_tosa_op_name(int index) {
    const auto &names = tosaOpNames();
    return index >= 0 && size_t(index) < names.size() ? names[size_t(index)].c_str() : nullptr;
}
int mlel_tosa_op_supported(const char *op_name) { return tosaOpSupported(op_name) ? 1 : 0; }
int mlel_tosa_lookup(const char *import_name, const char *op_name) {
    if (import_name == nullptr || op_name == nullptr || !extInstSetRegistered(import_name)) {
        return -1;
    }
    const auto &names = tosaOpNames();
    for (size_t i = 0; i < names.size(); ++i) {
        if (names[i] == op_name) {
            return tosaOpSupported(op_name) ? int(i) : -1;
        }
    }
    return -1;
}

int mlel_pipeline_op_count(const mlel_pipeline *p) { return int(p->impl->getPipelines().size()); }
const char *mlel_pipeline_op_name(const mlel_pipeline *p, int index) {
    const auto &ops = p->impl->getPipelines();
    return index >= 0 && size_t(index) < ops.size() ? ops[size_t(index)].name.c_str() : nullptr;
}
int mlel_pipeline_exec_count(mlel_pipeline *p) {
    int n = -1;
    guarded([&] {
        n = int(p->impl->getExecList().size());
        return MLEL_SUCCESS;
    });
    return n;
}
const char *mlel_pipeline_exec_name(mlel_pipeline *p, int index) {
    const char *name = nullptr;
    guarded([&] {
        const auto &ops = p->impl->getExecList();
        if (index >= 0 && size_t(index) < ops.size()) {
            name = ops[size_t(index)].name.c_str();
        }
        return MLEL_SUCCESS;
    });
    return name;
}
int mlel_pipeline_tensor_desc(const mlel_pipeline *p, mlel_tensor_id tensor, mlel_tensor_desc *out) {
    return guarded([&] {
        const auto &t = p->impl->tensor(tensor);
        std::memset(out, 0, sizeof(*out));
        out->dtype = t.dtype;
        out->rank = t.rank();
        for (int i = 0; i < t.rank(); ++i) {
            out->dims[i] = t.dims[size_t(i)];
            out->strides[i] = t.strides[size_t(i)];
        }
        return MLEL_SUCCESS;
    });
}

/* ---- operators ---- */

int mlel_make_conv2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                     mlel_tensor_id biases, const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2],
                     int8_t input_zp, int8_t weight_zp, uint32_t acc_type, const char *debug_name) {
    return guarded([&] {
        p->impl->makeConv2D(input, output, weights, biases, vec(pad, 4), vec(stride, 2), vec(dilation, 2), input_zp,
                            weight_zp, acc_type, nameOr(debug_name, "CONV2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_depthwise_conv2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                               mlel_tensor_id biases, const int32_t pad[4], const int32_t stride[2],
                               const int32_t dilation[2], int8_t input_zp, int8_t weight_zp, uint32_t acc_type,
                               const char *debug_name) {
    return guarded([&] {
        p->impl->makeDepthwiseConv2D(input, output, weights, biases, vec(pad, 4), vec(stride, 2), vec(dilation, 2),
                                     input_zp, weight_zp, acc_type, nameOr(debug_name, "DEPTHWISE_CONV2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_matmul(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2, mlel_tensor_id output,
                     int32_t input1_zp, int32_t input2_zp, const char *debug_name) {
    return guarded([&] {
        p->impl->makeMatmul(input1, input2, output, input1_zp, input2_zp, nameOr(debug_name, "MATMUL"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_rescale(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, int32_t input_zp,
                      int32_t output_zp, mlel_tensor_id multiplier, mlel_tensor_id shift, int scale32,
                      int double_round, int per_channel, int input_unsigned, int output_unsigned,
                      const char *debug_name) {
    return guarded([&] {
        p->impl->makeRescale(input, output, input_zp, output_zp, multiplier, shift, scale32 != 0, double_round != 0,
                             per_channel != 0, input_unsigned != 0, output_unsigned != 0,
                             nameOr(debug_name, "RESCALE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_avg_pool2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const int32_t kernel[2],
                         const int32_t stride[2], const int32_t pad[4], uint32_t acc_type, int8_t input_zp,
                         int8_t output_zp, const char *debug_name) {
    return guarded([&] {
        p->impl->makeAvgPool2D(input, output, vec(kernel, 2), vec(stride, 2), vec(pad, 4), acc_type, input_zp,
                               output_zp, nameOr(debug_name, "AVG_POOL2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_max_pool2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const int32_t kernel[2],
                         const int32_t stride[2], const int32_t pad[4], uint32_t nan_mode, const char *debug_name) {
    return guarded([&] {
        p->impl->makeMaxPool2D(input, output, vec(kernel, 2), vec(stride, 2), vec(pad, 4), nan_mode,
                               nameOr(debug_name, "MAX_POOL2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_table(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id table,
                    const char *debug_name) {
    return guarded([&] {
        p->impl->makeTable(input, output, table, nameOr(debug_name, "TABLE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_transpose(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const uint32_t *perms,
                        uint32_t perm_count, const char *debug_name) {
    return guarded([&] {
        p->impl->makeTranspose(input, output, vec(perms, perm_count), nameOr(debug_name, "TRANSPOSE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_concat(mlel_pipeline *p, const mlel_tensor_id *inputs, uint32_t input_count, mlel_tensor_id output,
                     uint32_t axis, const char *debug_name) {
    return guarded([&] {
        p->impl->makeConcat(vec(inputs, input_count), output, axis, nameOr(debug_name, "CONCAT"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_clamp(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, double min_value,
                    double max_value, uint32_t nan_mode, const char *debug_name) {
    return guarded([&] {
        p->impl->makeClamp(input, output, min_value, max_value, nan_mode, nameOr(debug_name, "CLAMP"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_binary(mlel_pipeline *p, const char *op_name, mlel_tensor_id input1, mlel_tensor_id input2,
                     mlel_tensor_id output, uint32_t nan_mode, const char *debug_name) {
    return guarded([&] {
        const auto it = kBinary.find(op_name);
        if (it == kBinary.end()) {
            throw UnsupportedError(std::string("unknown elementwise binary operator ") + op_name);
        }
        p->impl->makeBinary(it->second, input1, input2, output, nan_mode, nameOr(debug_name, op_name));
        return MLEL_SUCCESS;
    });
}

int mlel_make_unary(mlel_pipeline *p, const char *op_name, mlel_tensor_id input, mlel_tensor_id output,
                    const char *debug_name) {
    return guarded([&] {
        const auto it = kUnary.find(op_name);
        if (it == kUnary.end()) {
            throw UnsupportedError(std::string("unknown elementwise unary operator ") + op_name);
        }
        p->impl->makeUnary(it->second, input, output, nameOr(debug_name, op_name));
        return MLEL_SUCCESS;
    });
}

int mlel_make_mul(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2, mlel_tensor_id output,
                  uint32_t shift, const char *debug_name) {
    return guarded([&] {
        p->impl->makeMul(input1, input2, output, shift, nameOr(debug_name, "MUL"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_reduce(mlel_pipeline *p, const char *op_name, mlel_tensor_id input, mlel_tensor_id output,
                     uint32_t axis, uint32_t nan_mode, const char *debug_name) {
    return guarded([&] {
        const auto it = kReduce.find(op_name);
        if (it == kReduce.end()) {
            throw UnsupportedError(std::string("unknown reduce operator ") + op_name);
        }
        p->impl->makeReduce(it->second, input, output, axis, nan_mode, nameOr(debug_name, op_name));
        return MLEL_SUCCESS;
    });
}

int mlel_make_cast(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const char *debug_name) {
    return guarded([&] {
        p->impl->makeCast(input, output, nameOr(debug_name, "CAST"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_reshape(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const char *debug_name) {
    return guarded([&] {
        p->impl->makeReshape(input, output, nameOr(debug_name, "RESHAPE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_slice(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const uint32_t *start,
                    uint32_t start_count, const char *debug_name) {
    return guarded([&] {
        p->impl->makeSlice(input, output, vec(start, start_count), nameOr(debug_name, "SLICE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_pad(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id padding,
                  double pad_const, int32_t pad_const_int, const char *debug_name) {
    return guarded([&] {
        p->impl->makePad(input, output, padding, pad_const, pad_const_int, nameOr(debug_name, "PAD"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_arithmetic_right_shift(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2,
                                     mlel_tensor_id output, int round, const char *debug_name) {
    return guarded([&] {
        p->impl->makeArithmeticRightShift(input1, input2, output, round != 0,
                                          nameOr(debug_name, "ARITHMETIC_RIGHT_SHIFT"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_negate(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, int32_t input_zp,
                     int32_t output_zp, const char *debug_name) {
    return guarded([&] {
        p->impl->makeNegate(input, output, input_zp, output_zp, nameOr(debug_name, "NEGATE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_select(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2, mlel_tensor_id input3,
                     mlel_tensor_id output, const char *debug_name) {
    return guarded([&] {
        p->impl->makeSelect(input1, input2, input3, output, nameOr(debug_name, "SELECT"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_fft2d(mlel_pipeline *p, mlel_tensor_id input_real, mlel_tensor_id input_imag, mlel_tensor_id output_real,
                    mlel_tensor_id output_imag, int inverse, const char *debug_name) {
    return guarded([&] {
        p->impl->makeFft2D(input_real, input_imag, output_real, output_imag, inverse != 0, nameOr(debug_name, "FFT2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_rfft2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output_real, mlel_tensor_id output_imag,
                     const char *debug_name) {
    return guarded([&] {
        p->impl->makeRfft2D(input, output_real, output_imag, nameOr(debug_name, "RFFT2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_argmax(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, uint32_t axis, uint32_t nan_mode,
                     const char *debug_name) {
    return guarded([&] {
        p->impl->makeArgmax(input, output, axis, nan_mode, nameOr(debug_name, "ARGMAX"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_gather(mlel_pipeline *p, mlel_tensor_id values, mlel_tensor_id indices, mlel_tensor_id output,
                     const char *debug_name) {
    return guarded([&] {
        p->impl->makeGather(values, indices, output, nameOr(debug_name, "GATHER"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_scatter(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id values, mlel_tensor_id indices,
                      mlel_tensor_id output, const char *debug_name) {
    return guarded([&] {
        p->impl->makeScatter(input, values, indices, output, nameOr(debug_name, "SCATTER"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_reverse(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, uint32_t axis,
                      const char *debug_name) {
    return guarded([&] {
        p->impl->makeReverse(input, output, axis, nameOr(debug_name, "REVERSE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_tile(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const char *debug_name) {
    return guarded([&] {
        p->impl->makeTile(input, output, nameOr(debug_name, "TILE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_resize(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const int32_t scale[4],
                     const int32_t offset[2], const int32_t border[2], uint32_t mode, const char *debug_name) {
    return guarded([&] {
        p->impl->makeResize(input, output, vec(scale, 4), vec(offset, 2), vec(border, 2), mode,
                            nameOr(debug_name, "RESIZE"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_transpose_conv2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                               mlel_tensor_id biases, const int32_t out_pad[4], const int32_t stride[2],
                               int8_t input_zp, int8_t weight_zp, uint32_t acc_type, const char *debug_name) {
    return guarded([&] {
        p->impl->makeTransposeConv2D(input, output, weights, biases, vec(out_pad, 4), vec(stride, 2), input_zp,
                                     weight_zp, acc_type, nameOr(debug_name, "TRANSPOSE_CONV2D"));
        return MLEL_SUCCESS;
    });
}

int mlel_make_conv3d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                     mlel_tensor_id biases, const int32_t pad[6], const int32_t stride[3], const int32_t dilation[3],
                     int8_t input_zp, int8_t weight_zp, uint32_t acc_type, const char *debug_name) {
    return guarded([&] {
        p->impl->makeConv3D(input, output, weights, biases, vec(pad, 6), vec(stride, 3), vec(dilation, 3), input_zp,
                            weight_zp, acc_type, nameOr(debug_name, "CONV3D"));
        return MLEL_SUCCESS;
    });
}

/* ---- planner ---- */

int mlel_allocate_intervals(const mlel_live_interval *intervals, size_t interval_count,
                            const mlel_unseen_allocation *unseen, size_t unseen_count, uint64_t alignment,
                            uint64_t *offsets_out, uint64_t *unseen_offsets_out, uint64_t *memory_size_out) {
    return guarded([&] {
        std::vector<LiveInterval> iv;
        for (size_t k = 0; k < interval_count; ++k) {
            iv.push_back({intervals[k].id, intervals[k].first, intervals[k].last, intervals[k].size,
                          intervals[k].order});
        }
        std::vector<UnseenAllocation> us;
        for (size_t k = 0; k < unseen_count; ++k) {
            us.push_back({unseen[k].id, unseen[k].size});
        }
        const AllocationPlan plan = allocateIntervals(std::move(iv), us, alignment);
        for (size_t k = 0; k < interval_count; ++k) {
            offsets_out[k] = plan.offsets.at(intervals[k].id);
        }
        for (size_t k = 0; k < unseen_count; ++k) {
            unseen_offsets_out[k] = plan.offsets.at(unseen[k].id);
        }
        *memory_size_out = plan.memorySize;
        return MLEL_SUCCESS;
    });
}

/* ---- session ---- */

int mlel_session_create(mlel_pipeline *p, mlel_session **out) {
    return guarded([&] {
        *out = new mlel_session(p->impl);
        return MLEL_SUCCESS;
    });
}

void mlel_session_destroy(mlel_session *s) { delete s; }

int mlel_session_memory_requirements(const mlel_session *s, uint64_t *size, uint64_t *alignment) {
    *size = s->impl.memorySize();
    *alignment = s->impl.alignment();
    return MLEL_SUCCESS;
}

int mlel_session_tensor_offset(const mlel_session *s, mlel_tensor_id tensor, uint64_t *offset) {
    if (!s->impl.tensorOffset(tensor, offset)) {
        setLastError("tensor has no session storage");
        return MLEL_ERROR_UNKNOWN;
    }
    return MLEL_SUCCESS;
}

int mlel_session_bind_memory(mlel_session *s, void *memory, uint64_t offset) {
    return guarded([&] {
        if (memory == nullptr && s->impl.memorySize() > 0) {
            throw std::runtime_error("session memory must not be null");
        }
        if ((reinterpret_cast<uintptr_t>(memory) + offset) % kSessionAlignment != 0) {
            throw std::runtime_error("session memory must be aligned to the reported alignment");
        }
        s->impl.bindMemory(memory, offset);
        return MLEL_SUCCESS;
    });
}

int mlel_session_set_external(mlel_session *s, uint32_t set, uint32_t binding, uint32_t array_index,
                              void *device_ptr) {
    return guarded([&] {
        s->impl.setExternal(set, binding, array_index, device_ptr);
        return MLEL_SUCCESS;
    });
}

int mlel_session_dispatch(mlel_session *s, void *cuda_stream) {
    return guarded([&] { return s->impl.dispatch(static_cast<cudaStream_t>(cuda_stream)); });
}

int mlel_session_dispatch_graph(mlel_session *s, void *cuda_stream) {
    return guarded([&] { return s->impl.dispatchGraph(static_cast<cudaStream_t>(cuda_stream)); });
}

int mlel_session_dispatch_profiled(mlel_session *s, void *cuda_stream, float *ms_out, uint32_t capacity) {
    return guarded(
        [&] { return s->impl.dispatchProfiled(static_cast<cudaStream_t>(cuda_stream), ms_out, capacity); });
}

const char *mlel_session_planner_name(const mlel_session *s) { return plannerName(s->impl.planner()); }

int mlel_session_plan(const mlel_session *s, uint32_t *count, mlel_planned_tensor *out) {
    return guarded([&]() -> int {
        const auto &planned = s->impl.plannedTensors();
        if (out == nullptr) {
            *count = uint32_t(planned.size());
            return MLEL_SUCCESS;
        }
        const size_t n = std::min<size_t>(*count, planned.size());
        for (size_t k = 0; k < n; ++k) {
            const auto &p = planned[k];
            out[k] = {p.tensor, p.seen ? 1u : 0u, p.offset, p.size, p.first, p.last};
        }
        const bool cut = *count < planned.size();
        *count = uint32_t(n);
        return int(cut ? MLEL_INCOMPLETE : MLEL_SUCCESS);
    });
}

/* ---- pipeline properties ---- */

namespace {
constexpr const char *kCreationLog = "Graph pipeline created"; // graph/graph_layer.cpp:51

// writeTextProperty, graph/graph_layer.cpp:1427-1448
int writeTextProperty(const std::string &text, void *data, size_t *dataSize, int *isText) {
    if (isText != nullptr) {
        *isText = 1;
    }
    const size_t required = text.size() + 1;
    if (data == nullptr) {
        *dataSize = required;
        return MLEL_SUCCESS;
    }
    const size_t n = std::min(*dataSize, required);
    std::memcpy(data, text.c_str(), n); // c_str() holds the terminating zero as its last byte
    *dataSize = n;
    return n < required ? MLEL_INCOMPLETE : MLEL_SUCCESS;
}
} // namespace

int mlel_pipeline_available_properties(const mlel_pipeline *p, uint32_t *count, uint32_t *properties) {
    return guarded([&]() -> int {
        std::vector<uint32_t> all{MLEL_PIPELINE_PROPERTY_CREATION_LOG};
        if (p->impl->profiler() != nullptr) {
            all.push_back(MLEL_PIPELINE_PROPERTY_PROFILING);
        }
        if (properties == nullptr) {
            *count = uint32_t(all.size());
            return MLEL_SUCCESS;
        }
        const size_t n = std::min<size_t>(*count, all.size());
        std::copy(all.begin(), all.begin() + long(n), properties);
        const bool cut = *count < all.size();
        *count = uint32_t(n);
        return int(cut ? MLEL_INCOMPLETE : MLEL_SUCCESS);
    });
}

int mlel_pipeline_get_property(mlel_pipeline *p, uint32_t property, void *data, size_t *data_size, int *is_text) {
    return guarded([&]() -> int {
        if (data_size == nullptr) {
            throw std::runtime_error("get_property: data_size must not be null");
        }
        if (property == MLEL_PIPELINE_PROPERTY_CREATION_LOG) {
            return writeTextProperty(kCreationLog, data, data_size, is_text);
        }
        if (property == MLEL_PIPELINE_PROPERTY_PROFILING && p->impl->profiler() != nullptr) {
            return writeTextProperty(p->impl->profiler()->makeJson(), data, data_size, is_text);
        }
        setLastError("unknown pipeline property");
        return MLEL_ERROR_UNKNOWN;
    });
}

int mlel_pipeline_clear_profile(mlel_pipeline *p) {
    return guarded([&] {
        if (p->impl->profiler() != nullptr) {
            p->impl->profiler()->clear();
        }
        return MLEL_SUCCESS;
    });
}

int mlel_measure_int8_mma_peak(int batches, void *cuda_stream, float *ms, double *ops) {
    return guarded([&] { return int8MmaPeak(batches, static_cast<cudaStream_t>(cuda_stream), ms, ops); });
}

int mlel_session_launch_count(const mlel_session *s) {
    int n = -1;
    guarded([&] {
        n = s->impl.launchCount();
        return MLEL_SUCCESS;
    });
    return n;
}

int mlel_session_run_host(mlel_session *s, const mlel_host_io *inputs, uint32_t n_in, const mlel_host_io *outputs,
                          uint32_t n_out, void *cuda_stream) {
    return guarded([&] { return s->impl.runHost(inputs, n_in, outputs, n_out, static_cast<cudaStream_t>(cuda_stream)); });
}

/* ---- direct kernel entry points ---- */

namespace {
ConvAttr convAttrOf(const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2], int32_t inZp,
                    int32_t wZp) {
    ConvAttr a{};
    for (int k = 0; k < 4; ++k) {
        a.pad[k] = pad[k];
    }
    a.stride[0] = stride[0], a.stride[1] = stride[1], a.dilation[0] = dilation[0], a.dilation[1] = dilation[1];
    a.inZp = inZp, a.wZp = wZp;
    return a;
}

// Builds a one-operator table and runs it through the same dispatcher the session uses, so the
// direct entry points take exactly the kernel a graph would.
int runSingle(OpDesc &op, const std::vector<const mlel_tensor *> &tensors, cudaStream_t stream) {
    std::vector<TView> views;
    for (const auto *t : tensors) {
        views.push_back(t != nullptr ? viewOf(*t) : TView{});
    }
    return launchOp(op, views.data(), stream);
}

FusedRescale fusedRescaleOf(int32_t multId, int32_t shiftId, int32_t inDtype, int32_t inZp, int32_t outZp,
                            int doubleRound, int perChannel, int32_t clampMin, int32_t clampMax) {
    FusedRescale f;
    f.multTensor = multId;
    f.shiftTensor = shiftId;
    f.inDtype = inDtype;
    f.outDtype = MLEL_I8;
    f.attr = RescaleAttr{inZp, outZp, 1, doubleRound, perChannel};
    if (clampMin <= clampMax) {
        f.lo = clampMin < -128 ? -128 : clampMin;
        f.hi = clampMax > 127 ? 127 : clampMax;
    }
    return f;
}
} // namespace

int mlel_cuda_conv2d(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                     const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                     const int32_t dilation[2], int32_t input_zp, int32_t weight_zp, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_CONV2D;
        op.in = {0, 1, 2};
        op.out = {3};
        for (int k = 0; k < 4; ++k) {
            op.i[k] = pad[k];
        }
        op.i[4] = stride[0], op.i[5] = stride[1], op.i[6] = dilation[0], op.i[7] = dilation[1];
        op.i[8] = input_zp, op.i[9] = weight_zp;
        return runSingle(op, {input, weights, biases, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_depthwise_conv2d(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                               const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                               const int32_t dilation[2], int32_t input_zp, int32_t weight_zp, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_DEPTHWISE_CONV2D;
        op.in = {0, 1, 2};
        op.out = {3};
        for (int k = 0; k < 4; ++k) {
            op.i[k] = pad[k];
        }
        op.i[4] = stride[0], op.i[5] = stride[1], op.i[6] = dilation[0], op.i[7] = dilation[1];
        op.i[8] = input_zp, op.i[9] = weight_zp;
        return runSingle(op, {input, weights, biases, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_matmul(const mlel_tensor *a, const mlel_tensor *b, const mlel_tensor *output, int32_t a_zp,
                     int32_t b_zp, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_MATMUL;
        op.in = {0, 1};
        op.out = {2};
        op.i[0] = a_zp, op.i[1] = b_zp;
        return runSingle(op, {a, b, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_rescale(const mlel_tensor *input, const mlel_tensor *output, const mlel_tensor *multiplier,
                      const mlel_tensor *shift, int32_t input_zp, int32_t output_zp, int scale32, int double_round,
                      int per_channel, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_RESCALE;
        op.in = {0, 1, 2};
        op.out = {3};
        op.i[0] = input_zp, op.i[1] = output_zp, op.i[2] = scale32, op.i[3] = double_round, op.i[4] = per_channel;
        return runSingle(op, {input, multiplier, shift, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_avg_pool2d(const mlel_tensor *input, const mlel_tensor *output, const int32_t kernel[2], const int32_t stride[2],
                         const int32_t pad[4], int32_t input_zp, int32_t output_zp, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_AVG_POOL2D;
        op.in = {0};
        op.out = {1};
        op.i[0] = kernel[0], op.i[1] = kernel[1], op.i[2] = stride[0], op.i[3] = stride[1];
        for (int k = 0; k < 4; ++k) {
            op.i[4 + k] = pad[k];
        }
        op.i[8] = input_zp, op.i[9] = output_zp;
        return runSingle(op, {input, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_max_pool2d(const mlel_tensor *input, const mlel_tensor *output, const int32_t kernel[2], const int32_t stride[2],
                         const int32_t pad[4], void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_MAX_POOL2D;
        op.in = {0};
        op.out = {1};
        op.i[0] = kernel[0], op.i[1] = kernel[1], op.i[2] = stride[0], op.i[3] = stride[1];
        for (int k = 0; k < 4; ++k) {
            op.i[4 + k] = pad[k];
        }
        return runSingle(op, {input, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_table(const mlel_tensor *input, const mlel_tensor *table, const mlel_tensor *output, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_TABLE;
        op.in = {0, 1};
        op.out = {2};
        return runSingle(op, {input, table, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_transpose(const mlel_tensor *input, const mlel_tensor *output, const uint32_t *perms, uint32_t rank,
                        void *cuda_stream) {
    return guarded([&] {
        if (rank > uint32_t(kMaxRank) || perms == nullptr) {
            setLastError("mlel_cuda_transpose: bad permutation");
            return int(MLEL_ERROR_UNKNOWN);
        }
        OpDesc op;
        op.kind = OP_TRANSPOSE;
        op.in = {0};
        op.out = {1};
        for (uint32_t k = 0; k < rank; ++k) {
            op.i[k] = int32_t(perms[k]);
        }
        return runSingle(op, {input, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_concat(const mlel_tensor *const *inputs, uint32_t input_count, const mlel_tensor *output, uint32_t axis,
                     void *cuda_stream) {
    return guarded([&] {
        // one pass per input, each writing at the offset accumulated along `axis` (concat.comp:20-34)
        uint32_t offset = 0;
        for (uint32_t k = 0; k < input_count; ++k) {
            if (inputs == nullptr || inputs[k] == nullptr || axis >= uint32_t(inputs[k]->desc.rank)) {
                setLastError("mlel_cuda_concat: bad input");
                return int(MLEL_ERROR_UNKNOWN);
            }
            OpDesc op;
            op.kind = OP_CONCAT;
            op.in = {0};
            op.out = {1};
            op.i[0] = int32_t(axis), op.i[1] = int32_t(offset);
            const int rc = runSingle(op, {inputs[k], output}, static_cast<cudaStream_t>(cuda_stream));
            if (rc != MLEL_SUCCESS) {
                return rc;
            }
            offset += uint32_t(inputs[k]->desc.dims[axis]);
        }
        return int(MLEL_SUCCESS);
    });
}

int mlel_cuda_clamp(const mlel_tensor *input, const mlel_tensor *output, double min_value, double max_value,
                    void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_CLAMP;
        op.in = {0};
        op.out = {1};
        op.d[0] = min_value, op.d[1] = max_value;
        return runSingle(op, {input, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_binary(const char *op_name, const mlel_tensor *input1, const mlel_tensor *input2, const mlel_tensor *output,
                     void *cuda_stream) {
    return guarded([&] {
        const auto it = kBinary.find(op_name != nullptr ? op_name : "");
        if (it == kBinary.end()) {
            throw UnsupportedError(std::string("unknown elementwise binary operator ") + (op_name != nullptr ? op_name : ""));
        }
        OpDesc op;
        op.kind = OP_BINARY;
        op.sub = it->second;
        op.in = {0, 1};
        op.out = {2};
        return runSingle(op, {input1, input2, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_reduce(const char *op_name, const mlel_tensor *input, const mlel_tensor *output, uint32_t axis,
                     void *cuda_stream) {
    return guarded([&] {
        const auto it = kReduce.find(op_name != nullptr ? op_name : "");
        if (it == kReduce.end()) {
            throw UnsupportedError(std::string("unknown reduce operator ") + (op_name != nullptr ? op_name : ""));
        }
        OpDesc op;
        op.kind = OP_REDUCE;
        op.sub = it->second;
        op.in = {0};
        op.out = {1};
        op.i[0] = int32_t(axis);
        return runSingle(op, {input, output}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_interleave_columns(const void *staging, void *output, uint64_t rows, uint32_t blocks, uint32_t pitch_bytes,
                                 const int32_t *first_byte, const int32_t *byte_count, void *cuda_stream) {
    return guarded([&] {
        return interleaveColumns(staging, output, int64_t(rows), int32_t(blocks), int32_t(pitch_bytes), first_byte,
                                 byte_count, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_matmul_rescale(const mlel_tensor *a, const mlel_tensor *b, const mlel_tensor *output, int32_t a_zp,
                             int32_t b_zp, const mlel_tensor *multiplier, const mlel_tensor *shift,
                             int32_t rescale_in_zp, int32_t output_zp, int double_round, int per_channel,
                             int32_t clamp_min, int32_t clamp_max, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_FUSED_MATMUL;
        op.in = {0, 1};
        op.out = {2};
        op.i[0] = a_zp, op.i[1] = b_zp;
        op.epi.hasMain = true;
        op.epi.main = fusedRescaleOf(3, 4, MLEL_I32, rescale_in_zp, output_zp, double_round, per_channel, clamp_min,
                                     clamp_max);
        return runSingle(op, {a, b, output, multiplier, shift}, static_cast<cudaStream_t>(cuda_stream));
    });
}

int mlel_cuda_conv2d_rescale(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                             const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                             const int32_t dilation[2], int32_t input_zp, int32_t weight_zp,
                             const mlel_tensor *multiplier, const mlel_tensor *shift, int32_t rescale_in_zp,
                             int32_t output_zp, int double_round, int per_channel, int32_t clamp_min,
                             int32_t clamp_max, void *cuda_stream) {
    return guarded([&] {
        OpDesc op;
        op.kind = OP_FUSED_CONV2D;
        op.in = {0, 1, 2};
        op.out = {3};
        for (int k = 0; k < 4; ++k) {
            op.i[k] = pad[k];
        }
        op.i[4] = stride[0], op.i[5] = stride[1], op.i[6] = dilation[0], op.i[7] = dilation[1];
        op.i[8] = input_zp, op.i[9] = weight_zp;
        op.epi.hasMain = true;
        op.epi.main = fusedRescaleOf(4, 5, MLEL_I32, rescale_in_zp, output_zp, double_round, per_channel, clamp_min,
                                     clamp_max);
        return runSingle(op, {input, weights, biases, output, multiplier, shift},
                         static_cast<cudaStream_t>(cuda_stream));
    });
}

} // extern "C"
