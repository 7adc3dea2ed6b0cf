/*
 * C ABI of the B200 (sm_100a) implementation of the ML Emulation Layer's TOSA data-graph
 * execution path.
 *
 * The reference reaches this path through Vulkan entry points of VkLayer_Graph
 * (graph/graph_layer.cpp) and, below them, through the C++ class GraphPipeline
 * (graph/compute_graph_op.hpp:1204-1549).  Vulkan handles have no meaning on a CUDA-only
 * machine, so this ABI keeps the same objects and call order with plain pointers:
 *
 *   VkPipeline (data graph)          -> mlel_pipeline*
 *   VkDataGraphPipelineSessionARM    -> mlel_session*
 *   VkTensorDescriptionARM           -> mlel_tensor_desc
 *   VkDeviceMemory + offset          -> device pointer (+ offset)
 *   VkCommandBuffer / queue order    -> cudaStream_t (passed as void*)
 *
 * Every function returns MLEL_SUCCESS (0) or a negative mlel_status; mlel_last_error()
 * gives the message of the last failure on the calling thread.  No exception crosses the
 * ABI.  A pipeline is immutable once a session exists; a session must be used from one
 * stream at a time.  All device work runs on the CUDA device that is current when the
 * pipeline's first session is created.
 */
#ifndef MLEL_B200_H
#define MLEL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLEL_MAX_RANK 6 /* graph/shaders/graph_op/common.comp:11 */

typedef enum mlel_status {
    MLEL_SUCCESS = 0,
    MLEL_ERROR_UNKNOWN = -13,            /* value of VK_ERROR_UNKNOWN: malformed input */
    MLEL_ERROR_FEATURE_NOT_PRESENT = -8, /* value of VK_ERROR_FEATURE_NOT_PRESENT: op/type not supported */
    MLEL_INCOMPLETE = 5,                 /* value of VK_INCOMPLETE: caller's array too short */
    MLEL_ERROR_OUT_OF_DEVICE_MEMORY = -2,
    MLEL_ERROR_DEVICE = -4               /* a CUDA call failed (value of VK_ERROR_DEVICE_LOST) */
} mlel_status;

/* Element types.  Integer tensor formats are always signed in the graph layer
 * (graph/graph_ext_inst_context.cpp:355-402). */
typedef enum mlel_dtype {
    MLEL_BOOL = 0,
    MLEL_I8 = 1,
    MLEL_I16 = 2,
    MLEL_I32 = 3,
    MLEL_I64 = 4,
    MLEL_U8 = 5,
    MLEL_U16 = 6,
    MLEL_U32 = 7,
    MLEL_F16 = 8,
    MLEL_BF16 = 9,
    MLEL_F32 = 10
} mlel_dtype;

/* Replaces VkTensorDescriptionARM.  strides are in bytes; strides[0] == 0 means packed
 * row-major (tensor/tensor_arm.cpp:82-92). */
typedef struct mlel_tensor_desc {
    int32_t dtype;
    int32_t rank;
    int64_t dims[MLEL_MAX_RANK];
    int64_t strides[MLEL_MAX_RANK];
} mlel_tensor_desc;

/* A tensor operand of a direct kernel call: a descriptor plus a device address. */
typedef struct mlel_tensor {
    void *data;
    mlel_tensor_desc desc;
} mlel_tensor;

typedef struct mlel_pipeline mlel_pipeline;
typedef struct mlel_session mlel_session;
typedef int32_t mlel_tensor_id; /* index of a tensor descriptor inside its pipeline */

const char *mlel_last_error(void);
int mlel_elem_size(int32_t dtype);
/* Device-side error word of the current device: 0, or the code a kernel recorded when one of its
 * bounded waits ran out (the kernel then returns instead of hanging).  Synchronises the device. */
int mlel_device_error(void);

/* ---- pipeline construction: replaces vkCreateDataGraphPipelinesARM, graph/graph_layer.cpp:815-964 ---- */

/* flags for mlel_pipeline_create */
#define MLEL_PIPELINE_NO_FUSION 1u      /* run one kernel per TOSA op, exactly the reference's op list */
#define MLEL_PIPELINE_NO_TENSOR_CORE 2u /* keep contractions on the one-thread-per-output kernels */

int mlel_pipeline_create(uint32_t flags, mlel_pipeline **out);
void mlel_pipeline_destroy(mlel_pipeline *pipeline); /* vkDestroyPipeline, graph_layer.cpp:1280-1295 */

/* GraphPipeline::makeDescriptorSetBinding, graph/compute_graph_op.cpp:2441-2450 */
int mlel_pipeline_bind_external(mlel_pipeline *p, uint32_t set, uint32_t binding, uint32_t array_index,
                                const mlel_tensor_desc *desc, mlel_tensor_id *out);
/* GraphPipeline::getTensor(set, binding, arrayIndex), compute_graph_op.cpp:2452-2455 */
int mlel_pipeline_get_external(mlel_pipeline *p, uint32_t set, uint32_t binding, uint32_t array_index,
                               mlel_tensor_id *out);
/* GraphPipeline::makeConstTensor (data is copied), compute_graph_op.cpp:2398-2407 */
int mlel_pipeline_add_constant(mlel_pipeline *p, uint32_t id, const mlel_tensor_desc *desc, const void *host_data,
                               mlel_tensor_id *out);
/* GraphPipeline::getConstTensor, compute_graph_op.cpp:2409-2411 */
int mlel_pipeline_get_constant(mlel_pipeline *p, uint32_t id, mlel_tensor_id *out);
/* GraphPipeline::makeConstCompositeTensor, compute_graph_op.cpp:2413-2425 */
int mlel_pipeline_make_composite_constant(mlel_pipeline *p, const mlel_tensor_desc *desc, const void *host_data,
                                          mlel_tensor_id *out);
/* GraphPipeline::makeTensor (session memory), compute_graph_op.cpp:2457-2469 */
int mlel_pipeline_make_tensor(mlel_pipeline *p, const mlel_tensor_desc *desc, mlel_tensor_id *out);
/* GraphPipeline::makeInput / makeOutput, compute_graph_op.cpp:2513-2521 */
int mlel_pipeline_mark_input(mlel_pipeline *p, mlel_tensor_id tensor);
int mlel_pipeline_mark_output(mlel_pipeline *p, mlel_tensor_id tensor);

/* Lowers a SPIR-V module in assembly text form (the form of the reference's tests/shader
 * fixtures) through the TOSA.001000.1 registry.  External bindings and graph constants must
 * have been registered first, as vkCreateDataGraphPipelinesARM does (graph_layer.cpp:874-901)
 * before it runs the graph pass (graph/graph_pass_ext_inst.cpp:25-82). */
int mlel_pipeline_lower_spvasm(mlel_pipeline *p, const char *text);

/* Registry queries: graph/graph_ext_inst_registry.cpp:36-59, graph/graph_tosa_1_0_ext_inst.cpp:41-108 */
int mlel_ext_inst_set_registered(const char *import_name);
int mlel_tosa_op_count(void);
const char *mlel_tosa_op_name(int index);
int mlel_tosa_op_supported(const char *op_name);
/* The registry as one query, by names (the numeric opcodes live in a header the reference does not vendor):
 * index of the handler of `op_name` in the instruction set imported as `import_name` ("TOSA.001000.1"), the same
 * index mlel_tosa_op_name uses; -1 when the set is not registered or has no such operator
 * (graph/graph_ext_inst_registry.cpp:53-59 selects the decoder by import string, graph_tosa_1_0_ext_inst.cpp:41-108
 * the handler). */
int mlel_tosa_lookup(const char *import_name, const char *op_name);

/* Introspection of the lowered graph (the reference logs the same at Info severity). */
int mlel_pipeline_op_count(const mlel_pipeline *p);
const char *mlel_pipeline_op_name(const mlel_pipeline *p, int index);
int mlel_pipeline_exec_count(mlel_pipeline *p);               /* kernels per dispatch after fusion */
const char *mlel_pipeline_exec_name(mlel_pipeline *p, int index);
int mlel_pipeline_tensor_desc(const mlel_pipeline *p, mlel_tensor_id tensor, mlel_tensor_desc *out);

/* ---- TOSA operators: one call per GraphPipeline::make<Op>, graph/compute_graph_op.hpp:1249-1483.
 * Argument order and meaning are the reference's; tensors are ids of this pipeline. ---- */
int mlel_make_conv2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                     mlel_tensor_id biases, const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2],
                     int8_t input_zp, int8_t weight_zp, uint32_t acc_type, const char *debug_name);
int mlel_make_depthwise_conv2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                               mlel_tensor_id biases, const int32_t pad[4], const int32_t stride[2],
                               const int32_t dilation[2], int8_t input_zp, int8_t weight_zp, uint32_t acc_type,
                               const char *debug_name);
int mlel_make_matmul(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2, mlel_tensor_id output,
                     int32_t input1_zp, int32_t input2_zp, const char *debug_name);
int mlel_make_rescale(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, int32_t input_zp,
                      int32_t output_zp, mlel_tensor_id multiplier, mlel_tensor_id shift, int scale32,
                      int double_round, int per_channel, int input_unsigned, int output_unsigned,
                      const char *debug_name);
int mlel_make_avg_pool2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const int32_t kernel[2],
                         const int32_t stride[2], const int32_t pad[4], uint32_t acc_type, int8_t input_zp,
                         int8_t output_zp, const char *debug_name);
int mlel_make_max_pool2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const int32_t kernel[2],
                         const int32_t stride[2], const int32_t pad[4], uint32_t nan_mode, const char *debug_name);
int mlel_make_table(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id table,
                    const char *debug_name);
int mlel_make_transpose(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const uint32_t *perms,
                        uint32_t perm_count, const char *debug_name);
int mlel_make_concat(mlel_pipeline *p, const mlel_tensor_id *inputs, uint32_t input_count, mlel_tensor_id output,
                     uint32_t axis, const char *debug_name);
int mlel_make_clamp(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, double min_value,
                    double max_value, uint32_t nan_mode, const char *debug_name);
/* makeAdd, makeSub, makeBitwise*, makeLogical*, makeIntdiv, makeMaximum, makeMinimum, makeEqual,
 * makeGreater, makeGreaterEqual: `op_name` is the TOSA name ("ADD", "LOGICAL_LEFT_SHIFT", ...). */
int mlel_make_binary(mlel_pipeline *p, const char *op_name, mlel_tensor_id input1, mlel_tensor_id input2,
                     mlel_tensor_id output, uint32_t nan_mode, const char *debug_name);
/* makeAbs, makeBitwiseNot, makeClz, makeLogicalNot (integer unary operators) */
int mlel_make_unary(mlel_pipeline *p, const char *op_name, mlel_tensor_id input, mlel_tensor_id output,
                    const char *debug_name);
int mlel_make_mul(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2, mlel_tensor_id output,
                  uint32_t shift, const char *debug_name);
/* makeReduceSum/Max/Min/Product/All/Any: `op_name` is "REDUCE_SUM", ... */
int mlel_make_reduce(mlel_pipeline *p, const char *op_name, mlel_tensor_id input, mlel_tensor_id output,
                     uint32_t axis, uint32_t nan_mode, const char *debug_name);
int mlel_make_cast(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const char *debug_name);
int mlel_make_reshape(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const char *debug_name);
int mlel_make_slice(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const uint32_t *start,
                    uint32_t start_count, const char *debug_name);
int mlel_make_pad(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id padding,
                  double pad_const, int32_t pad_const_int, const char *debug_name);
int mlel_make_arithmetic_right_shift(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2,
                                     mlel_tensor_id output, int round, const char *debug_name);
int mlel_make_negate(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, int32_t input_zp,
                     int32_t output_zp, const char *debug_name);
int mlel_make_select(mlel_pipeline *p, mlel_tensor_id input1, mlel_tensor_id input2, mlel_tensor_id input3,
                     mlel_tensor_id output, const char *debug_name);
/* makeFft2D / makeRfft2D: fp32 tensors [N, H, W]; RFFT2D's outputs are [N, H, W / 2 + 1].  The inverse transform
 * is not scaled (fft2d.comp). */
int mlel_make_fft2d(mlel_pipeline *p, mlel_tensor_id input_real, mlel_tensor_id input_imag, mlel_tensor_id output_real,
                    mlel_tensor_id output_imag, int inverse, const char *debug_name);
int mlel_make_rfft2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output_real, mlel_tensor_id output_imag,
                     const char *debug_name);
/* makeArgmax: the output has the input's shape without `axis` and holds int32 indices. */
int mlel_make_argmax(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, uint32_t axis, uint32_t nan_mode,
                     const char *debug_name);
/* makeGather: values [N,K,C], indices int32 [N,W] -> output [N,W,C]. */
int mlel_make_gather(mlel_pipeline *p, mlel_tensor_id values, mlel_tensor_id indices, mlel_tensor_id output,
                     const char *debug_name);
/* makeScatter: input [N,W,C] written into a copy of values [N,K,C] at rows indices [N,W] -> output [N,K,C]. */
int mlel_make_scatter(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id values, mlel_tensor_id indices,
                      mlel_tensor_id output, const char *debug_name);
int mlel_make_reverse(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, uint32_t axis,
                      const char *debug_name);
/* makeTile: the multiples are implied by the output's shape. */
int mlel_make_tile(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const char *debug_name);
/* makeResize: scale = {y_n, y_d, x_n, x_d}; mode 1 = NEAREST, 2 = BILINEAR (integer variants). */
int mlel_make_resize(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, const int32_t scale[4],
                     const int32_t offset[2], const int32_t border[2], uint32_t mode, const char *debug_name);
int mlel_make_transpose_conv2d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                               mlel_tensor_id biases, const int32_t out_pad[4], const int32_t stride[2],
                               int8_t input_zp, int8_t weight_zp, uint32_t acc_type, const char *debug_name);
/* makeConv3D: pad = {front, back, top, bottom, left, right}; stride and dilation = {d, y, x}. */
int mlel_make_conv3d(mlel_pipeline *p, mlel_tensor_id input, mlel_tensor_id output, mlel_tensor_id weights,
                     mlel_tensor_id biases, const int32_t pad[6], const int32_t stride[3], const int32_t dilation[3],
                     int8_t input_zp, int8_t weight_zp, uint32_t acc_type, const char *debug_name);

/* ---- interval memory planner: details::allocateIntervals, graph/interval_memory_planner.cpp:170-216 ---- */
typedef struct mlel_live_interval {
    uint64_t id;
    uint32_t first;
    uint32_t last;
    uint64_t size;
    uint64_t order;
} mlel_live_interval;
typedef struct mlel_unseen_allocation {
    uint64_t id;
    uint64_t size;
} mlel_unseen_allocation;
/* offsets_out[i] receives the offset of intervals[i]; unseen_offsets_out[j] that of unseen[j]. */
int mlel_allocate_intervals(const mlel_live_interval *intervals, size_t interval_count,
                            const mlel_unseen_allocation *unseen, size_t unseen_count, uint64_t alignment,
                            uint64_t *offsets_out, uint64_t *unseen_offsets_out, uint64_t *memory_size_out);

/* ---- session: graph/graph_layer.cpp:215-298, 1297-1420, 1844-1917 ---- */
/* vkCreateDataGraphPipelineSessionARM: plans session memory with the interval planner. */
int mlel_session_create(mlel_pipeline *p, mlel_session **out);
void mlel_session_destroy(mlel_session *s);
/* vkGetDataGraphPipelineSessionMemoryRequirementsARM */
int mlel_session_memory_requirements(const mlel_session *s, uint64_t *size, uint64_t *alignment);
/* Planned offset of one session tensor inside the bound memory (for inspection and tests). */
int mlel_session_tensor_offset(const mlel_session *s, mlel_tensor_id tensor, uint64_t *offset);
/* vkBindDataGraphPipelineSessionMemoryARM: `memory` is a device pointer owned by the caller. */
int mlel_session_bind_memory(mlel_session *s, void *memory, uint64_t offset);
/* Descriptor-set update of one application tensor (vkUpdateDescriptorSets + vkCmdBindDescriptorSets). */
int mlel_session_set_external(mlel_session *s, uint32_t set, uint32_t binding, uint32_t array_index,
                              void *device_ptr);
/* vkCmdDispatchDataGraphARM + queue submission: enqueues every kernel of the graph on `stream`. */
int mlel_session_dispatch(mlel_session *s, void *cuda_stream);
/* Same, replayed from a CUDA graph captured on first use.  One graph is kept per set of bound addresses (up to
 * 64 sets), so a host that alternates between a few input and output buffers replays a graph for each. */
int mlel_session_dispatch_graph(mlel_session *s, void *cuda_stream);
/* Dispatch with a CUDA event pair around every launched kernel, the counterpart of the reference's
 * per-operator timestamp profiling (VMEL_GRAPH_PROFILING, graph/graph_profiler.cpp:157-191).
 * Synchronises the stream; ms_out[i] receives the device time of kernel i (see
 * mlel_pipeline_exec_name); `capacity` must be at least mlel_session_launch_count(). */
int mlel_session_dispatch_profiled(mlel_session *s, void *cuda_stream, float *ms_out, uint32_t capacity);
/* ---- session memory planners: graph/graph_layer.cpp:282-297, graph/memory_planner.cpp ----
 * The environment variable VMEL_MEMORY_PLANNER, read when a session is created, selects "Linear"
 * (every tensor its own storage, memory_planner.cpp:52-98), "BestFit" (largest first into the
 * best-fitting reusable slot, memory_planner.cpp:239-381) or, by default, the interval planner. */
typedef struct mlel_planned_tensor {
    mlel_tensor_id tensor;
    uint32_t seen;   /* 0: no launched kernel touches it (kept only when fusion is off) */
    uint64_t offset; /* inside the bound session memory */
    uint64_t size;   /* rounded up to the session alignment */
    uint32_t first;  /* live range over {0 = graph inputs, 1..n = launched kernels, n + 1 = outputs} */
    uint32_t last;
} mlel_planned_tensor;
/* "Interval", "Linear" or "BestFit": the planner this session was planned with. */
const char *mlel_session_planner_name(const mlel_session *s);
/* Two-call enumeration: with `out` NULL *count receives the number of planned tensors; otherwise up to
 * *count records are written, *count receives the number written, MLEL_INCOMPLETE if there were more. */
int mlel_session_plan(const mlel_session *s, uint32_t *count, mlel_planned_tensor *out);

/* ---- pipeline properties: vkGetDataGraphPipelineAvailablePropertiesARM and
 * vkGetDataGraphPipelinePropertiesARM, graph/graph_layer.cpp:1427-1524 ----
 * The profiling property exists only for pipelines created while VMEL_GRAPH_PROFILING was truthy
 * (graph/graph_profiler.cpp:29-38, 107).  Every dispatch of such a pipeline's sessions is then timed kernel
 * by kernel with CUDA events, and the property returns the reference's JSON document
 * (graph/graph_profiler.cpp:563-620: "timestamp_period_ns", "samples", "by_operator") after waiting for the
 * recorded dispatches; ticks are nanoseconds since the pipeline's first profiled dispatch. */
#define MLEL_PIPELINE_PROPERTY_CREATION_LOG 0u     /* VK_DATA_GRAPH_PIPELINE_PROPERTY_CREATION_LOG_ARM */
#define MLEL_PIPELINE_PROPERTY_PROFILING 0x7ffffffeu /* the layer-private property, graph_layer.cpp:108-114 */
/* Two-call enumeration as above. */
int mlel_pipeline_available_properties(const mlel_pipeline *p, uint32_t *count, uint32_t *properties);
/* With `data` NULL *data_size receives the size needed (text plus its terminating zero).  Otherwise at most
 * *data_size bytes are written and *data_size receives the number written; MLEL_INCOMPLETE if the text was
 * cut short.  *is_text is set to 1.  Unknown property, or profiling not enabled: MLEL_ERROR_UNKNOWN. */
int mlel_pipeline_get_property(mlel_pipeline *p, uint32_t property, void *data, size_t *data_size, int *is_text);
/* Forgets the samples taken so far (the reference drops them with their command buffers). */
int mlel_pipeline_clear_profile(mlel_pipeline *p);

/* ---- measurement helper (no counterpart in the reference) ----
 * Runs tcgen05.mma kind::i8 (M 128, N 256, K 32) back to back on every SM, on operands that stay in shared
 * memory: `batches` batches of 64 instructions per SM.  *ms receives the device time, *ops the number of int8
 * operations (two per multiply-accumulate) it stands for: ops / ms is what the int8 tensor pipe sustains, the
 * denominator of tensor-bound roofline fractions.  Synchronises the stream. */
int mlel_measure_int8_mma_peak(int batches, void *cuda_stream, float *ms, double *ops);

/* Kernel selection of the tensor-core contractions (no counterpart in the reference; process-wide, takes
 * effect for kernels enqueued afterwards, results are the same bits whatever is chosen):
 *   "pair_kernel"       which contractions with more than 128 output channels run on the paired two-CTA kernel:
 *                       1 (default) matrix products, 2 convolutions as well, 0 none;
 *   "pair_tile_pixels"  0 (default: chosen per problem), 128, 192 or 256 pixels per tile of the paired kernel;
 *   "oc_tile_pixels"    the same for the channel-major single-CTA kernel;
 *   "oc_tile_rule"      0..8, default 3.  From 1 on: a layer whose 192-pixel tiles would leave a quarter of the SMs
 *                       without work takes 128-pixel tiles if those fit in one round.  r >= 2: a layer with at least r
 *                       rounds of 192-pixel tiles per SM takes 256-pixel tiles.  0: 192 pixels for every layer above
 *                       128 pixels;
 *   "dependent_launch"  1 (default) launches the tensor-core kernels with programmatic dependent launch;
 *   "tile_progress"     7 (default): a convolution whose input the convolution before it wrote starts on that launch's
 *                       finished pixel tiles; bit 0 read by tiles, bit 1 publish, bit 2 channel tiles first; 0 off.
 * Another key or value: MLEL_ERROR_UNKNOWN. */
int mlel_set_tuning(const char *key, int value);

/* Self-test of the bounded waits (no counterpart in the reference).  Every wait inside the tensor-core kernels has
 * a limit (about two seconds), after which the kernel records a code that mlel_device_error() reports, leaves its
 * loops and releases its tensor memory.  This runs a one-thread kernel that waits, with a limit of about a
 * millisecond, on a barrier nobody arrives at: *recorded_code receives the code that wait recorded (99), or 0 if
 * it did not give up.  The code is cleared again, so mlel_device_error() is 0 afterwards.  Synchronises the stream. */
int mlel_selftest_wait_timeout(void *cuda_stream, int *recorded_code);

/* Diagnostic (no counterpart in the reference): how often the library has enqueued tensor-core kernel
 * `kernel` since it was loaded -- 0 the pixel-major tcgen05 kernel, 1 the channel-major one, 2 the paired
 * (two-CTA) one; -1 for another index.  Tests use it to see which kernel took a case. */
long long mlel_tensor_core_launches(int kernel);

/* Number of kernels one dispatch launches. */
int mlel_session_launch_count(const mlel_session *s);
/* Host-buffer convenience used for end-to-end timing: copies `n_in` host inputs to their bound
 * device tensors, dispatches, copies `n_out` outputs back, and synchronises the stream. */
typedef struct mlel_host_io {
    uint32_t set, binding, array_index;
    void *host_ptr;
    uint64_t bytes;
} mlel_host_io;
int mlel_session_run_host(mlel_session *s, const mlel_host_io *inputs, uint32_t n_in, const mlel_host_io *outputs,
                          uint32_t n_out, void *cuda_stream);

/* ---- direct kernel entry points: one per reference shader, graph/shaders/graph_op/tosa/<op>.comp.
 * Operands are device tensors; work is enqueued on `cuda_stream`. ---- */
int mlel_cuda_conv2d(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                     const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                     const int32_t dilation[2], int32_t input_zp, int32_t weight_zp, void *cuda_stream);
int mlel_cuda_depthwise_conv2d(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                               const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                               const int32_t dilation[2], int32_t input_zp, int32_t weight_zp, void *cuda_stream);
int mlel_cuda_matmul(const mlel_tensor *a, const mlel_tensor *b, const mlel_tensor *output, int32_t a_zp,
                     int32_t b_zp, void *cuda_stream);
int mlel_cuda_rescale(const mlel_tensor *input, const mlel_tensor *output, const mlel_tensor *multiplier,
                      const mlel_tensor *shift, int32_t input_zp, int32_t output_zp, int scale32, int double_round,
                      int per_channel, void *cuda_stream);

/* The other operators of the path, one entry per reference shader (avgpool2d.comp, maxpool2d.comp, table.comp,
 * transpose.comp, concat.comp, clamp.comp, elementwise_binary.comp, reduce.comp), with the argument meaning of
 * the matching GraphPipeline::make<Op> (graph/compute_graph_op.hpp:1249-1483).  Each takes the kernel a graph
 * would take for the same tensors.  `op_name` of mlel_cuda_binary / mlel_cuda_reduce is the TOSA name
 * ("ADD", "MAXIMUM", ... / "REDUCE_SUM", "REDUCE_MAX", ...).  mlel_cuda_concat runs one pass per input, as the
 * reference does. */
int mlel_cuda_avg_pool2d(const mlel_tensor *input, const mlel_tensor *output, const int32_t kernel[2], const int32_t stride[2],
                         const int32_t pad[4], int32_t input_zp, int32_t output_zp, void *cuda_stream);
int mlel_cuda_max_pool2d(const mlel_tensor *input, const mlel_tensor *output, const int32_t kernel[2], const int32_t stride[2],
                         const int32_t pad[4], void *cuda_stream);
int mlel_cuda_table(const mlel_tensor *input, const mlel_tensor *table, const mlel_tensor *output, void *cuda_stream);
int mlel_cuda_transpose(const mlel_tensor *input, const mlel_tensor *output, const uint32_t *perms, uint32_t rank,
                        void *cuda_stream);
int mlel_cuda_concat(const mlel_tensor *const *inputs, uint32_t input_count, const mlel_tensor *output, uint32_t axis,
                     void *cuda_stream);
int mlel_cuda_clamp(const mlel_tensor *input, const mlel_tensor *output, double min_value, double max_value,
                    void *cuda_stream);
int mlel_cuda_binary(const char *op_name, const mlel_tensor *input1, const mlel_tensor *input2, const mlel_tensor *output,
                     void *cuda_stream);
int mlel_cuda_reduce(const char *op_name, const mlel_tensor *input, const mlel_tensor *output, uint32_t axis,
                     void *cuda_stream);

/* Fused int8 contraction + RESCALE (+ CLAMP): what the fusion pass substitutes for
 * MATMUL -> RESCALE [-> CLAMP] (matmul.comp + rescale.comp + clamp.comp in one kernel).
 * a: [N,H,C] int8, b: [N,C,W] int8, out: [N,H,W] int8. clamp_min > clamp_max disables CLAMP. */
int mlel_cuda_matmul_rescale(const mlel_tensor *a, const mlel_tensor *b, const mlel_tensor *output, int32_t a_zp,
                             int32_t b_zp, const mlel_tensor *multiplier, const mlel_tensor *shift,
                             int32_t rescale_in_zp, int32_t output_zp, int double_round, int per_channel,
                             int32_t clamp_min, int32_t clamp_max, void *cuda_stream);
/* CONV2D -> RESCALE [-> CLAMP] in one kernel (conv2d.comp + rescale.comp + clamp.comp). */
int mlel_cuda_conv2d_rescale(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                             const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                             const int32_t dilation[2], int32_t input_zp, int32_t weight_zp,
                             const mlel_tensor *multiplier, const mlel_tensor *shift, int32_t rescale_in_zp,
                             int32_t output_zp, int double_round, int per_channel, int32_t clamp_min,
                             int32_t clamp_max, void *cuda_stream);

/* Join of an output-channel-sharded MATMUL (no counterpart in the reference, which has no multi-device path):
 * after an all-gather, `staging` holds `blocks` column blocks one after another, block g as `rows` rows of
 * `pitch_bytes` bytes of which the first byte_count[g] are valid; this writes rows of sum(byte_count) bytes to
 * `output` with block g at byte first_byte[g] of every row (first_byte[0] = 0, first_byte[g + 1] = first_byte[g] +
 * byte_count[g]; at most 64 blocks).  Moves 16 bytes per thread when every block starts and ends on a 16-byte
 * boundary. */
int mlel_cuda_interleave_columns(const void *staging, void *output, uint64_t rows, uint32_t blocks, uint32_t pitch_bytes,
                                 const int32_t *first_byte, const int32_t *byte_count, void *cuda_stream);

/* CONV2D (int8 input, int8 OHWI weights with zero point 0, int32 bias, int32 output; same result as
 * mlel_cuda_conv2d) for callers that must not allocate device memory, such as a layer's dispatch hook
 * or code that runs inside another runtime's fixed memory budget.  It has no counterpart in the
 * reference.  All working memory is a 32 MiB array built into the library, so the call makes no
 * cudaMalloc/cudaFree and uses no allocating library routine; problems that need more
 * (pixels * kPad + OC * kPad + 4 * OC bytes, kPad = KH*KW*IC rounded up to 16) are rejected with
 * MLEL_ERROR_UNKNOWN.  Also rejected, with a message: tensors that are not packed, an output channel count
 * that is not a multiple of 16, KH*KW*IC above 65536, a weight zero point other than 0, an input zero point
 * outside the int8 range, and an output size that does not follow from the other arguments.
 * The array is shared by every call on the device: calls whose GPU work may overlap
 * must be serialised by the caller.  The first call on a device resolves the array's address and should
 * be made outside stream capture. */
int mlel_cuda_conv2d_static_scratch(const mlel_tensor *input, const mlel_tensor *weights, const mlel_tensor *biases,
                                    const mlel_tensor *output, const int32_t pad[4], const int32_t stride[2],
                                    const int32_t dilation[2], int32_t input_zp, int32_t weight_zp,
                                    void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* MLEL_B200_H */
