/* kxc_b200_plan.h — whole-graph entry point of libkxc_b200.so.
 *
 * A plan is the library-side counterpart of the reference's ExecutionPlan: a list of KernelExec
 * nodes `{op_name, input value ids, output value id}` (include/base/execution_plan.h:42-50,
 * built per Relay Call by src/relay/transforms/multi_device.cc:298-325). The reference's nodes do
 * not carry the call attributes (src/base/execution_plan.cc:695-708), so each node here takes them
 * in a plain-C struct equivalent to the Relay Attrs object the op's FRelayToTE hook receives
 * (include/relay/op_attr_types.h:19-20).
 *
 * Running a plan replaces `CompiledKernel::operator()` on the function the reference lowers the whole
 * graph into (`kxc_kernel_main`): same packed argument order — function inputs, then constants in
 * the order they were added (the lowering DFS order const_0, const_1, ...; src/relay/backend/lower.cc:534-565),
 * then outputs — same int32 return convention (src/codegen/compiled_kernel.cc:41-55).
 *
 * Supported ops: nn_conv2d, nn_relu, add, nn_max_pool2d, nn_global_avg_pool2d, nn_flatten, nn_dense,
 * nn_gemm — the set a ResNet-class graph uses (test/resnet18_ir_dump.cpp:281-448). finalize() fuses
 * conv -> [add] -> [relu] into one kernel and keeps activations channel-innermost in the plan's own
 * arena; only the graph's inputs and outputs use the reference's NCHW fp32 layout.
 */
#ifndef KXC_B200_PLAN_H_
#define KXC_B200_PLAN_H_

#include "kxc_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Threading: a plan owns ONE activation arena and ONE set of captured CUDA graphs, so it supports one run in
 * flight at a time. kxc_b200_plan_run / _run_timed calls on the same plan are serialised by a mutex inside the
 * plan on the host side, and the caller must not enqueue two runs of one plan on DIFFERENT streams without
 * ordering them (they would share the arena on the GPU). Different plans are independent: a host that runs the
 * same graph from several threads (src/runtime/kernel_runner.cc:17-30, src/runtime/runtime_session.cc:115-161)
 * creates one plan per thread; the weights are packed per plan. Building calls (add_*, finalize) are not
 * thread-safe per plan. */
typedef struct kxc_b200_plan kxc_b200_plan;

/* Attribute structs: the fields of Conv2DAttrsNode (include/relay/op.h:104-120), MaxPool2DAttrsNode
 * (:154-164) and GemmAttrsNode (:367-374) that the compute hooks read. */
typedef struct kxc_b200_conv2d_attrs {
    int32_t strides[2];
    int32_t padding[2];  /* symmetric (h, w): Conv2DCompute reads padding[0], padding[1] only */
    int32_t dilation[2];
    int32_t groups;
} kxc_b200_conv2d_attrs;

typedef struct kxc_b200_pool2d_attrs {
    int32_t pool_size[2];
    int32_t strides[2];
    int32_t padding[4];  /* top, left, bottom, right */
    int32_t ceil_mode;
} kxc_b200_pool2d_attrs;

typedef struct kxc_b200_gemm_attrs {
    float alpha, beta;
    int32_t transA, transB;
} kxc_b200_gemm_attrs;

/* SoftmaxAttrsNode (include/relay/op.h): accepted for "softmax" as the LAST node of the graph, last axis only (see
 * kxc_b200_softmax); it runs as one more launch on the plan's fp32 result. */
typedef struct kxc_b200_softmax_attrs {
    int32_t axis; /* negative values count from the end */
} kxc_b200_softmax_attrs;

/* FlattenAttrsNode (include/relay/op.h:353-358), optional for "nn_flatten" (NULL = axis 1). The reference honours the
 * axis (src/relay/op/tensor/transform.cc:145-165, src/relay/type_infer.cc:446-450); a plan flattens at axis 1 only
 * (negative values count from the end) and refuses anything else at finalize with KXC_B200_ERR_UNSUPPORTED rather than
 * produce another shape than the reference would. */
typedef struct kxc_b200_flatten_attrs {
    int32_t axis;
} kxc_b200_flatten_attrs;

/* precision: KXC_B200_PREC_BF16 (bf16 activations/weights, fp32 accumulate), KXC_B200_PREC_TF32 (fp32
 * activations, tf32-rounded operands, fp32 accumulate), KXC_B200_PREC_TF32X3 (full fp32 activations; every
 * convolution / dense node splits both operands into tf32 high and low parts and runs three tensor-core passes,
 * lo*hi + hi*lo + hi*hi, into one fp32 result: fp32-class accuracy, the mode that meets the reference's 1e-3
 * acceptance metric of test/onnx_importer_test.cpp:161-177 on a whole network) — all three on the tensor cores —
 * or KXC_B200_PREC_FP32: CUDA-core kernels in the reference's operation order on NCHW fp32 values, bit-identical
 * to the reference's CPU lowering of the same graph. */
int32_t kxc_b200_plan_create(int32_t precision, kxc_b200_plan** out);
int32_t kxc_b200_plan_destroy(kxc_b200_plan* plan);

/* Values are dense fp32 tensors named by caller-chosen non-negative ids. Inputs and constants must be
 * added in packed-argument order. */
int32_t kxc_b200_plan_add_input(kxc_b200_plan* plan, int32_t value_id, int32_t rank, const int64_t* shape);
int32_t kxc_b200_plan_add_constant(kxc_b200_plan* plan, int32_t value_id, int32_t rank, const int64_t* shape);
/* One KernelExec node. `attrs` points to the op's attribute struct (NULL for ops without attributes). */
int32_t kxc_b200_plan_add_kernel(kxc_b200_plan* plan, const char* op_name, const void* attrs, int32_t num_inputs,
                                 const int32_t* input_ids, int32_t output_id);
int32_t kxc_b200_plan_set_output(kxc_b200_plan* plan, int32_t value_id);
/* Shape inference, fusion, layout assignment, arena allocation, tensor-map construction. */
int32_t kxc_b200_plan_finalize(kxc_b200_plan* plan);
/* Shape of a value after finalize (rank <= 6); returns the rank or a negative error. */
int32_t kxc_b200_plan_value_shape(kxc_b200_plan* plan, int32_t value_id, int64_t* shape_out);
/* Number of kernels one run launches (after fusion), excluding the one-time weight packing. */
int32_t kxc_b200_plan_num_launches(kxc_b200_plan* plan);

/* packed_args = { inputs..., constants..., output }: device pointers, fp32. Asynchronous on `stream`.
 * Constants are packed into the plan's own tensor-core layout on the first run and whenever a
 * constant pointer changes (constants are immutable in the reference, include/relay/relay.h:120-125). */
int32_t kxc_b200_plan_run(kxc_b200_plan* plan, void** packed_args, void* stream);

/* Replay one run as a CUDA graph (off by default). With it on, the first run with a given packed-argument
 * list executes normally (it packs the constants), the second captures the launches on `stream`, and later
 * runs with the same pointers replay the captured graph with one launch call. Passing different pointers
 * re-captures. The reference has no counterpart (its kernels are host loops). */
int32_t kxc_b200_plan_set_cuda_graph(kxc_b200_plan* plan, int32_t enable);

/* NVTX ranges (ProfileOptions::enable_nvtx, include/base/profiling.h:66): with it on, every run is one range
 * "kxc_b200_plan_run" holding one range per launch, named as kxc_b200_plan_launch_info names that launch (a CUDA-graph
 * replay is a single range "cuda graph replay"). Call after finalize. Costs nothing while no NVTX tool is attached. */
int32_t kxc_b200_plan_set_nvtx(kxc_b200_plan* plan, int32_t enable);

/* Measurement support (no reference counterpart: the reference only prints one wall-clock elapsed_ms,
 * test/onnx_importer_test.cpp:261-281). launch_info: a label, the algorithmic FLOPs and the compulsory
 * HBM bytes of launch `index`. run_timed: one run with a CUDA event between launches on `stream`;
 * synchronises and returns each launch's duration in milliseconds. */
int32_t kxc_b200_plan_launch_info(kxc_b200_plan* plan, int32_t index, char* name, int32_t name_size, double* flops,
                                  double* bytes);
int32_t kxc_b200_plan_run_timed(kxc_b200_plan* plan, void** packed_args, void* stream, float* launch_ms, int32_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* KXC_B200_PLAN_H_ */
