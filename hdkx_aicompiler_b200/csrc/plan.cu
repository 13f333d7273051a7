// Whole-graph executor behind kxc_b200_plan_* (include/kxc_b200_plan.h).
//
// The caller describes the graph the way the reference's ExecutionPlan does — one KernelExec node
// per Relay call, values named by ids (include/base/execution_plan.h:42-50) — and finalize() turns
// it into a short list of launches:
//   * conv -> [add residual] -> [relu] chains become ONE tensor-core kernel (fused epilogue);
//   * activations stay in the plan's arena, channel-innermost (NHWC), in the operand type of the
//     chosen precision; arena blocks are reused once a value's last consumer has run;
//   * graph inputs are converted once (a few-channel stride-2 first convolution gets the packed
//     "stem" layout below), graph outputs are written in the reference's NCHW/row-major fp32 layout
//     straight from the last kernel's epilogue;
//   * constants are packed into the tensor-core weight layout on the first run.
//
// Stem layout. A 7x7 stride-2 convolution over 3 channels has K = 147, far too ragged for 64-channel
// K blocks. The input is instead packed as [N][H+2p][Wp][4] with a zero border, and one K block is
// "8 consecutive pixels x 4 channels" (32 elements) starting at column 2*ow: a TMA tensor map whose
// column dimension has a stride of 2 pixels makes consecutive output columns overlapping 32-element
// rows, so the A tile of filter row kh is again a single TMA box. Weights are packed to
// [O][KH][8][4] with zeros in the unused slots; K = KH*32.
#include "kxc_b200_plan.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"
#include "conv_direct.cuh"
#include "conv_rowstack.cuh"
#include "conv_stem.cuh"
#include "conv_tc.cuh"
#include "layout.cuh"
#include "nhwc_kernels.cuh"

using namespace kxc_b200;

namespace {

enum class VKind { Input, Constant, Intermediate };
enum class SKind { InputNHWC, InputStem, Conv, Gemm, MaxPool, Gap, Eltwise, ToNCHW };

struct Value {
    int id = -1;
    VKind kind = VKind::Intermediate;
    std::vector<int64_t> shape;  // logical (NCHW / [M,K]) shape, the reference's view
    int arg_index = -1;          // inputs/constants: position in packed_args
    int producer = -1;           // node index
    std::vector<int> consumers;  // node indices
    int alias_of = -1;           // value id whose storage this one shares (flatten)
    // storage of the internal (NHWC / row-major, operand dtype) copy
    size_t offset = 0, bytes = 0;
    bool has_storage = false;
    int first_step = -1, last_step = -1;
};

struct Node {
    std::string op;
    std::vector<int> in;
    int out = -1;
    kxc_b200_conv2d_attrs conv{};
    kxc_b200_pool2d_attrs pool{};
    kxc_b200_gemm_attrs gemm{};
    int flatten_axis = 1;
    bool fused_into_other = false;
};

struct PackedWeight {
    int const_id = -1;
    void* ptr = nullptr;       // plan-owned, tensor-core layout
    void* ptr_lo = nullptr;    // TF32X3 plans: the tf32 rounding of what `ptr`'s rounding dropped
    size_t bytes = 0;
    const void* source = nullptr;  // user pointer it was packed from
    int mode = 0;              // 0 conv OHWI, 1 stem (igemm), 2 dense [N,K], 3 dense from [K,N], 4 stem (direct kernel),
                               // 5 stem, filter rows stacked by parity (fused-input kernel)
    int O = 0, C = 0, KH = 0, KW = 0, cpad = 0;
};

struct Step {
    SKind kind;
    // generic references (value ids)
    int in0 = -1, in1 = -1, out = -1;
    int weight = -1;      // index into packed weights
    int bias_const = -1;  // constant value id (fp32 user pointer), -1 = none
    bool relu = false;
    bool out_is_graph_output = false;
    int direct = 0;  // 0 = implicit-GEMM kernel; 1 = direct 3x3 kernel; 2 = direct stem kernel
    int fused_pool = 0;  // direct stem kernel only: the following max_pool2d(3x3, s2, p1) is computed in its epilogue
    int direct_input = 0;  // fused stem kernel reads the NCHW fp32 graph input itself: no packed copy, no conversion step
    // second output (two-output implicit-GEMM kernel): a 1x1 convolution of the same stride over the same input
    int weight2 = -1, bias2_const = -1, out2 = -1;
    bool relu2 = false;
    // conv / gemm
    TcParams params{};
    TcConfig cfg{};
    // TF32X3 plans: the two correction passes (x_lo * w_hi, x_hi * w_lo) that run before `params` (x_hi * w_hi);
    // src_input = the graph input this step reads through its NHWC copy (-1: an intermediate)
    TcParams params_lohi{}, params_hilo{};
    int src_input = -1;
    // pooling / misc geometry
    int N = 0, C = 0, H = 0, W = 0, OH = 0, OW = 0;
    kxc_b200_pool2d_attrs pool{};
    int Hp = 0, Wp = 0, pad_h = 0, pad_w = 0, cpad = 0;
    int64_t numel = 0;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int64_t numel_of(const std::vector<int64_t>& s) {
    int64_t n = 1;
    for (auto d : s) n *= d;
    return n;
}

}  // namespace

struct kxc_b200_plan {
    int precision = KXC_B200_PREC_BF16;
    TcDType dtype = kTcBF16;
    // KXC_B200_PREC_TF32X3: activations stay full fp32 in the arena; every convolution / dense step splits its
    // input into tf32 high and low parts (x3_scratch) and runs three tensor-core passes into the same fp32 output
    bool x3 = false;
    void* x3_scratch = nullptr;
    size_t x3_half_bytes = 0;  // the low part starts this many bytes into x3_scratch
    std::map<int, Value> values;
    std::vector<int> inputs, constants;
    std::vector<Node> nodes;
    int output_id = -1;
    bool finalized = false;
    std::vector<Step> steps;
    std::vector<PackedWeight> weights;
    void* arena = nullptr;
    size_t arena_bytes = 0;
    void* weight_arena = nullptr;
    int device = -1;
    // KXC_B200_PREC_FP32 plans: reference-layout (NCHW fp32) values, CUDA-core kernels in the reference's
    // operation order, bit-exact end to end (see the "exact mode" section at the end of this file)
    struct XStep {
        std::string op;
        int in0 = -1, in1 = -1, weight = -1, bias = -1, out = -1;
        bool relu = false;
        int node = -1;
    };
    std::vector<XStep> xsteps;
    // optional CUDA-graph replay of one run (launch-bound small batches): the graph captured for a given
    // packed-argument list is replayed whenever the caller passes the same pointers again; a few argument
    // lists are remembered so that double-buffered inputs and outputs do not re-capture on every call
    bool use_graph = false;
    static constexpr int kGraphSlots = 4;
    struct GraphSlot {
        std::vector<void*> args;
        cudaGraphExec_t exec = nullptr;
    };
    GraphSlot graph_slots[kGraphSlots];
    int graph_next_slot = 0;
    // optional last node softmax(last axis) on the graph's fp32 result: the plan proper writes into tail_buf and one
    // more launch writes the caller's output
    int tail_in = -1, tail_out = -1, tail_axis = -1;
    void* tail_buf = nullptr;
    int64_t tail_rows = 0, tail_len = 0;
    // optional NVTX ranges: one per launch, named like kxc_b200_plan_launch_info names it, inside one range per run
    bool nvtx = false;
    std::vector<std::string> nvtx_names;
    // one run in flight per plan: run / run_timed calls from several host threads are serialised here (the arena,
    // the packed weights and the captured graphs are per plan)
    std::mutex run_mu;

    ~kxc_b200_plan() {
        for (auto& g : graph_slots)
            if (g.exec) cudaGraphExecDestroy(g.exec);
        if (tail_buf) cudaFree(tail_buf);
        if (x3_scratch) cudaFree(x3_scratch);
        if (arena) cudaFree(arena);
        if (weight_arena) cudaFree(weight_arena);
    }

    Value* find(int id) {
        auto it = values.find(id);
        return it == values.end() ? nullptr : &it->second;
    }
    int root_of(int id) {
        Value* v = find(id);
        while (v && v->alias_of >= 0) v = find(v->alias_of);
        return v ? v->id : -1;
    }
    void* storage(int id) {
        Value* v = find(root_of(id));
        return static_cast<uint8_t*>(arena) + v->offset;
    }
    int eb() const { return tc_elem_bytes(dtype); }
};

namespace {

int32_t infer_shapes(kxc_b200_plan* pl) {
    for (size_t ni = 0; ni < pl->nodes.size(); ++ni) {
        Node& n = pl->nodes[ni];
        std::vector<Value*> in;
        for (int id : n.in) {
            Value* v = pl->find(id);
            if (!v)
                return fail(KXC_B200_ERR_INVALID, "plan: node %zu (%s) reads undefined value %d", ni, n.op.c_str(), id);
            in.push_back(v);
        }
        Value* out = pl->find(n.out);
        if (!out) return fail(KXC_B200_ERR_INVALID, "plan: node %zu has no output value", ni);
        const std::string& op = n.op;
        if (op == "nn_conv2d") {
            // Conv2DInferType, src/relay/type_infer.cc:346-400
            if (in.size() < 2 || in.size() > 3) return fail(KXC_B200_ERR_INVALID, "nn_conv2d expects 2 or 3 inputs (data, weight[, bias])");
            if (in[0]->shape.size() != 4 || in[1]->shape.size() != 4)
                return fail(KXC_B200_ERR_INVALID, "nn_conv2d currently expects NCHW/OIHW rank-4 tensors");
            if (in.size() == 3 && in[2]->shape.size() != 1) return fail(KXC_B200_ERR_INVALID, "nn_conv2d bias must be rank-1");
            if (n.conv.groups != 1) return fail(KXC_B200_ERR_UNSUPPORTED, "nn_conv2d: groups=%d", n.conv.groups);
            if (in[0]->shape[1] != in[1]->shape[1]) return fail(KXC_B200_ERR_INVALID, "nn_conv2d: channel mismatch");
            const int64_t OH = conv_out_dim(in[0]->shape[2], in[1]->shape[2], n.conv.strides[0], n.conv.padding[0], n.conv.dilation[0]);
            const int64_t OW = conv_out_dim(in[0]->shape[3], in[1]->shape[3], n.conv.strides[1], n.conv.padding[1], n.conv.dilation[1]);
            if (OH <= 0 || OW <= 0) return fail(KXC_B200_ERR_INVALID, "nn_conv2d: empty output");
            out->shape = {in[0]->shape[0], in[1]->shape[0], OH, OW};
        } else if (op == "nn_relu") {
            if (in.size() != 1) return fail(KXC_B200_ERR_INVALID, "nn_relu expects exactly 1 input");
            out->shape = in[0]->shape;
        } else if (op == "add") {
            if (in.size() != 2) return fail(KXC_B200_ERR_INVALID, "add expects exactly 2 inputs");
            if (in[0]->shape != in[1]->shape)
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: add with broadcasting is not supported inside a plan (use kxc_b200_add)");
            out->shape = in[0]->shape;
        } else if (op == "nn_max_pool2d") {
            if (in.size() != 1 || in[0]->shape.size() != 4) return fail(KXC_B200_ERR_INVALID, "nn_max_pool2d expects NCHW rank-4 input");
            const auto& a = n.pool;
            const int64_t OH = pool_out_dim(in[0]->shape[2], a.pool_size[0], a.strides[0], a.padding[0], a.padding[2], a.ceil_mode != 0);
            const int64_t OW = pool_out_dim(in[0]->shape[3], a.pool_size[1], a.strides[1], a.padding[1], a.padding[3], a.ceil_mode != 0);
            if (OH <= 0 || OW <= 0) return fail(KXC_B200_ERR_INVALID, "nn_max_pool2d: empty output");
            out->shape = {in[0]->shape[0], in[0]->shape[1], OH, OW};
        } else if (op == "nn_global_avg_pool2d") {
            if (in.size() != 1 || in[0]->shape.size() != 4) return fail(KXC_B200_ERR_INVALID, "nn_global_avg_pool2d expects NCHW rank-4 input");
            out->shape = {in[0]->shape[0], in[0]->shape[1], 1, 1};
        } else if (op == "nn_flatten") {
            if (in.size() != 1 || in[0]->shape.empty()) return fail(KXC_B200_ERR_INVALID, "nn_flatten expects exactly 1 input");
            {   // FlattenInferType (src/relay/type_infer.cc:446-450) honours the axis; only axis 1 is implemented here
                const int rank = (int)in[0]->shape.size();
                const int axis = n.flatten_axis < 0 ? n.flatten_axis + rank : n.flatten_axis;
                if (axis != 1)
                    return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_flatten with axis %d (only axis 1 is supported inside a plan)", n.flatten_axis);
            }
            int64_t rest = 1;
            for (size_t i = 1; i < in[0]->shape.size(); ++i) rest *= in[0]->shape[i];
            out->shape = {in[0]->shape[0], rest};
        } else if (op == "nn_dense" || op == "nn_gemm") {
            const bool gemm = op == "nn_gemm";
            if ((int)in.size() != (gemm ? 3 : 2)) return fail(KXC_B200_ERR_INVALID, "%s expects exactly %d inputs", op.c_str(), gemm ? 3 : 2);
            if (in[0]->shape.size() != 2 || in[1]->shape.size() != 2) return fail(KXC_B200_ERR_INVALID, "%s expects rank-2 operands", op.c_str());
            if (gemm && n.gemm.transA != 0) return fail(KXC_B200_ERR_UNSUPPORTED, "nn_gemm currently does not support transA=1");
            const bool transB = !gemm || n.gemm.transB == 1;
            const int64_t K = in[0]->shape[1];
            const int64_t Nn = transB ? in[1]->shape[0] : in[1]->shape[1];
            if ((transB ? in[1]->shape[1] : in[1]->shape[0]) != K) return fail(KXC_B200_ERR_INVALID, "%s: inner dimensions differ", op.c_str());
            out->shape = {in[0]->shape[0], Nn};
        } else {
            return fail(KXC_B200_ERR_UNSUPPORTED, "plan: op '%s' is not supported", op.c_str());
        }
    }
    return KXC_B200_OK;
}

// The single consumer node of value `id`, or -1.
int sole_consumer(kxc_b200_plan* pl, int id) {
    Value* v = pl->find(id);
    if (!v || v->consumers.size() != 1 || id == pl->output_id) return -1;
    return v->consumers[0];
}

int32_t setup_stem(kxc_b200_plan* pl, Step& st, int N, int C, int H, int W, int O, int KH, int KW, int pad_h, int pad_w,
                   const void* packed_in, const void* packed_w, TcOutMode out_mode) {
    const TcDType dt = pl->dtype;
    const int eb = tc_elem_bytes(dt);
    TcParams& p = st.params;
    const int OH = (int)conv_out_dim(H, KH, 2, pad_h, 1), OW = (int)conv_out_dim(W, KW, 2, pad_w, 1);
    p.N = N; p.OH = OH; p.OW = OW; p.Cout = O;
    p.taps_h = KH; p.taps_w = 1; p.stride = 2;
    p.pad_h = 0; p.pad_w = 0; p.dil_h = 1; p.dil_w = 1;
    p.cblocks = 1; p.kb_elems = 32;
    tc_pick_tile(N, OH, OW, &p.BW, &p.BH, &p.BNI);
    p.tiles_w = (OW + p.BW - 1) / p.BW;
    p.tiles_h = (OH + p.BH - 1) / p.BH;
    p.tiles_n = (N + p.BNI - 1) / p.BNI;
    const int bn = O <= 64 ? 64 : (O <= 128 ? 128 : 256);
    p.tiles_c = (O + bn - 1) / bn;
    st.cfg = TcConfig{dt, 32 * eb, bn, out_mode};
    const size_t px = (size_t)4 * eb;  // bytes per packed pixel
    const uint32_t box[4] = {32u, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BNI};
    uint8_t* base = const_cast<uint8_t*>(static_cast<const uint8_t*>(packed_in));
    for (int hp = 0; hp < 2; ++hp) {
        const uint64_t dims[4] = {32, (uint64_t)OW, (uint64_t)((st.Hp - hp + 1) / 2), (uint64_t)N};
        const uint64_t strides[3] = {2 * px, (uint64_t)2 * st.Wp * px, (uint64_t)st.Hp * st.Wp * px};
        CUtensorMap m;
        KXC_TRY(tc_make_tmap(&m, dt, 4, base + (size_t)hp * st.Wp * px, dims, strides, box, 32 * eb));
        p.tmA[hp * 2] = m;
        p.tmA[hp * 2 + 1] = m;
    }
    const uint64_t ktot = (uint64_t)KH * 32;
    const uint64_t bdims[2] = {ktot, (uint64_t)O};
    const uint64_t bstr[1] = {ktot * eb};
    const uint32_t bbox[2] = {32u, (uint32_t)bn};
    KXC_TRY(tc_make_tmap(&p.tmB, dt, 2, const_cast<void*>(packed_w), bdims, bstr, bbox, 32 * eb));
    KXC_TRY(tc_status_word(&p.status));
    return KXC_B200_OK;
}

}  // namespace

// The 128 -> 128 channel 3x3 layers: the row-stacked CTA-pair kernel with resident weights or the implicit-GEMM kernel.
// Measured per launch at 28 x 28 (ms, row-stacked against implicit GEMM): without a residual 0.191 / 0.215 at 1024 images
// and 0.033 / 0.037 at 128; with a residual 0.235 / 0.227 at 1024, 0.127 / 0.121-0.125 at 512, 0.067-0.068 / 0.070-0.072
// at 256 and 0.037-0.039 / 0.040-0.041 at 128. So: always without a residual, with one up to 256 images of 28 x 28. KXC_B200_ROWSTACK128 = 0: never, 2: always (A/B runs); read at every
// plan build.
static bool rowstack128_wanted(bool has_residual, long long pixels) {
    const char* e = getenv("KXC_B200_ROWSTACK128");
    if (e != nullptr && e[0] == '0') return false;
    if (e != nullptr && e[0] == '2') return true;
    return !has_residual || pixels <= 256ll * 28 * 28;
}

static int32_t finalize_exact(kxc_b200_plan* pl);
static int32_t run_exact(kxc_b200_plan* pl, void** packed_args, void* stream, cudaEvent_t* events);

extern "C" int32_t kxc_b200_plan_create(int32_t precision, kxc_b200_plan** out) {
    if (!out) return fail(KXC_B200_ERR_INVALID, "plan_create: null out pointer");
    if (precision != KXC_B200_PREC_BF16 && precision != KXC_B200_PREC_TF32 && precision != KXC_B200_PREC_FP32 &&
        precision != KXC_B200_PREC_TF32X3)
        return fail(KXC_B200_ERR_UNSUPPORTED, "plan_create: precision must be KXC_B200_PREC_BF16, _TF32, _TF32X3 or _FP32");
    auto* pl = new (std::nothrow) kxc_b200_plan();
    if (!pl) return fail(KXC_B200_ERR_NOMEM, "plan_create: out of host memory");
    pl->precision = precision;
    pl->dtype = precision == KXC_B200_PREC_BF16 ? kTcBF16 : kTcTF32;
    pl->x3 = precision == KXC_B200_PREC_TF32X3;
    *out = pl;
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_destroy(kxc_b200_plan* plan) {
    delete plan;
    return KXC_B200_OK;
}

static int32_t add_value(kxc_b200_plan* pl, int32_t id, VKind kind, int32_t rank, const int64_t* shape) {
    if (!pl || pl->finalized) return fail(KXC_B200_ERR_INVALID, "plan: null or already finalized");
    if (id < 0 || rank < 0 || rank > 6 || (rank > 0 && !shape)) return fail(KXC_B200_ERR_INVALID, "plan: bad value declaration");
    if (pl->find(id)) return fail(KXC_B200_ERR_INVALID, "plan: value %d declared twice", id);
    Value v;
    v.id = id;
    v.kind = kind;
    v.shape.assign(shape, shape + rank);
    for (auto d : v.shape)
        if (d < 0) return fail(KXC_B200_ERR_INVALID, "plan: negative extent");
    v.arg_index = (int)(pl->inputs.size() + pl->constants.size());
    pl->values[id] = v;
    (kind == VKind::Input ? pl->inputs : pl->constants).push_back(id);
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_add_input(kxc_b200_plan* plan, int32_t value_id, int32_t rank, const int64_t* shape) {
    if (plan && !plan->constants.empty()) return fail(KXC_B200_ERR_INVALID, "plan: inputs must be added before constants");
    return add_value(plan, value_id, VKind::Input, rank, shape);
}
extern "C" int32_t kxc_b200_plan_add_constant(kxc_b200_plan* plan, int32_t value_id, int32_t rank, const int64_t* shape) {
    return add_value(plan, value_id, VKind::Constant, rank, shape);
}

extern "C" int32_t kxc_b200_plan_add_kernel(kxc_b200_plan* plan, const char* op_name, const void* attrs, int32_t num_inputs,
                                            const int32_t* input_ids, int32_t output_id) {
    if (!plan || plan->finalized || !op_name || num_inputs < 0 || (num_inputs > 0 && !input_ids) || output_id < 0)
        return fail(KXC_B200_ERR_INVALID, "plan_add_kernel: bad arguments");
    if (plan->find(output_id)) return fail(KXC_B200_ERR_INVALID, "plan: value %d already defined", output_id);
    if (std::string(op_name) == "softmax") {
        // SoftmaxCompute (src/relay/op/nn/softmax.cc:44-70), accepted as the graph's last node
        if (num_inputs != 1) return fail(KXC_B200_ERR_INVALID, "softmax expects exactly 1 input");
        if (plan->tail_out >= 0) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: only one softmax (the last node) is supported");
        if (!plan->find(input_ids[0])) return fail(KXC_B200_ERR_INVALID, "plan: node 'softmax' reads undefined value %d", input_ids[0]);
        plan->tail_in = input_ids[0];
        plan->tail_out = output_id;
        plan->tail_axis = attrs ? static_cast<const kxc_b200_softmax_attrs*>(attrs)->axis : -1;
        Value v;
        v.id = output_id;
        v.kind = VKind::Intermediate;
        v.producer = -1;
        plan->values[output_id] = v;
        return KXC_B200_OK;
    }
    if (plan->tail_out >= 0)
        for (int32_t i = 0; i < num_inputs; ++i)
            if (input_ids[i] == plan->tail_out) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: softmax is supported as the last node only");
    Node n;
    n.op = op_name;
    n.in.assign(input_ids, input_ids + num_inputs);
    n.out = output_id;
    if (n.op == "nn_conv2d") {
        if (!attrs) return fail(KXC_B200_ERR_INVALID, "nn_conv2d expects Conv2DAttrs");
        n.conv = *static_cast<const kxc_b200_conv2d_attrs*>(attrs);
        if (n.conv.strides[0] <= 0 || n.conv.strides[1] <= 0 || n.conv.dilation[0] <= 0 || n.conv.dilation[1] <= 0 ||
            n.conv.padding[0] < 0 || n.conv.padding[1] < 0)
            return fail(KXC_B200_ERR_INVALID, "nn_conv2d: bad strides/padding/dilation");
    } else if (n.op == "nn_max_pool2d") {
        if (!attrs) return fail(KXC_B200_ERR_INVALID, "nn_max_pool2d expects MaxPool2DAttrs");
        n.pool = *static_cast<const kxc_b200_pool2d_attrs*>(attrs);
        if (n.pool.pool_size[0] <= 0 || n.pool.pool_size[1] <= 0 || n.pool.strides[0] <= 0 || n.pool.strides[1] <= 0)
            return fail(KXC_B200_ERR_INVALID, "nn_max_pool2d: bad pool_size/strides");
    } else if (n.op == "nn_gemm") {
        if (!attrs) return fail(KXC_B200_ERR_INVALID, "nn_gemm expects GemmAttrs");
        n.gemm = *static_cast<const kxc_b200_gemm_attrs*>(attrs);
    } else if (n.op == "nn_flatten") {
        if (attrs) n.flatten_axis = static_cast<const kxc_b200_flatten_attrs*>(attrs)->axis;
    }
    for (int id : n.in)
        if (!plan->find(id)) return fail(KXC_B200_ERR_INVALID, "plan: node '%s' reads undefined value %d", op_name, id);
    Value v;
    v.id = output_id;
    v.kind = VKind::Intermediate;
    v.producer = (int)plan->nodes.size();
    plan->values[output_id] = v;
    for (int id : n.in) plan->find(id)->consumers.push_back((int)plan->nodes.size());
    plan->nodes.push_back(n);
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_set_output(kxc_b200_plan* plan, int32_t value_id) {
    if (!plan || plan->finalized) return fail(KXC_B200_ERR_INVALID, "plan_set_output: bad plan");
    Value* v = plan->find(value_id);
    if (!v || v->kind != VKind::Intermediate) return fail(KXC_B200_ERR_INVALID, "plan_set_output: value %d is not produced by a kernel", value_id);
    plan->output_id = value_id;
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_value_shape(kxc_b200_plan* plan, int32_t value_id, int64_t* shape_out) {
    if (!plan || !plan->finalized) return -KXC_B200_ERR_INVALID;
    Value* v = plan->find(value_id);
    if (!v) return -KXC_B200_ERR_INVALID;
    for (size_t i = 0; i < v->shape.size(); ++i) shape_out[i] = v->shape[i];
    return (int32_t)v->shape.size();
}

extern "C" int32_t kxc_b200_plan_num_launches(kxc_b200_plan* plan) {
    if (!plan || !plan->finalized) return -KXC_B200_ERR_INVALID;
    const int tail = plan->tail_out >= 0 ? 1 : 0;
    if (plan->precision == KXC_B200_PREC_FP32) return (int32_t)plan->xsteps.size() + tail;
    return (int32_t)plan->steps.size() + tail;
}

static int32_t finalize_core(kxc_b200_plan* pl);

extern "C" int32_t kxc_b200_plan_finalize(kxc_b200_plan* pl) {
    if (!pl || pl->finalized) return fail(KXC_B200_ERR_INVALID, "plan_finalize: null or already finalized");
    if (pl->tail_out < 0) return finalize_core(pl);
    if (pl->output_id != pl->tail_out) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: softmax is supported as the last node only");
    Value* src = pl->find(pl->tail_in);
    if (!src || src->kind != VKind::Intermediate)
        return fail(KXC_B200_ERR_UNSUPPORTED, "plan: softmax must follow a kernel of the plan (use kxc_b200_softmax on its own)");
    pl->output_id = pl->tail_in;  // the plan proper ends at the softmax's operand
    KXC_TRY(finalize_core(pl));
    const std::vector<int64_t> shape = pl->find(pl->tail_in)->shape;
    const int rank = (int)shape.size();
    const int axis = pl->tail_axis < 0 ? pl->tail_axis + rank : pl->tail_axis;
    pl->finalized = false;  // until the checks below pass
    if (rank < 1 || axis != rank - 1)
        return fail(KXC_B200_ERR_UNSUPPORTED, "softmax: only the last axis is supported (the reference's reduction over an inner axis "
                                             "reads the wrong elements)");
    pl->find(pl->tail_out)->shape = shape;
    pl->tail_len = shape[rank - 1];
    pl->tail_rows = 1;
    for (int i = 0; i < rank - 1; ++i) pl->tail_rows *= shape[i];
    const size_t bytes = (size_t)(pl->tail_rows * pl->tail_len) * sizeof(float);
    if (bytes > 0) KXC_CUDA_TRY(cudaMalloc(&pl->tail_buf, bytes));
    pl->finalized = true;
    return KXC_B200_OK;
}

static int32_t finalize_core(kxc_b200_plan* pl) {
    if (!pl || pl->finalized) return fail(KXC_B200_ERR_INVALID, "plan_finalize: null or already finalized");
    KXC_TRY(require_device());
    if (pl->output_id < 0) return fail(KXC_B200_ERR_INVALID, "plan_finalize: no output set");
    if (pl->inputs.size() != 1) return fail(KXC_B200_ERR_UNSUPPORTED, "plan_finalize: exactly one graph input is supported");
    KXC_TRY(infer_shapes(pl));
    if (!pl->find(pl->output_id)->consumers.empty())
        return fail(KXC_B200_ERR_UNSUPPORTED, "plan_finalize: the output value must not feed other kernels");
    if (pl->precision == KXC_B200_PREC_FP32) return finalize_exact(pl);
    KXC_CUDA_TRY(cudaGetDevice(&pl->device));
    const TcDType dt = pl->dtype;
    const int eb = pl->eb();
    const int lanes = 16 / eb;

    auto is_const = [&](int id) { return pl->find(id)->kind == VKind::Constant; };
    auto is_input = [&](int id) { return pl->find(id)->kind == VKind::Input; };

    // ---- build steps (fusing conv -> [add] -> [relu] and add -> relu) ----
    std::map<int, int> input_copy;  // (input value id * 2 + stem) -> step index producing the internal copy
    std::vector<std::pair<int, Step>> pending;  // (emit position = node index, step)
    for (size_t ni = 0; ni < pl->nodes.size(); ++ni) {
        Node& n = pl->nodes[ni];
        if (n.fused_into_other) continue;
        Step st{};
        int emit_at = (int)ni;
        if (n.op == "nn_conv2d") {
            Value* data = pl->find(n.in[0]);
            Value* w = pl->find(n.in[1]);
            if (!is_const(n.in[1]) || (n.in.size() == 3 && !is_const(n.in[2])))
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_conv2d weight and bias must be constants");
            if (is_const(n.in[0])) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_conv2d over a constant input");
            st.kind = SKind::Conv;
            st.in0 = n.in[0];
            st.bias_const = n.in.size() == 3 ? n.in[2] : -1;
            int cur = n.out;
            int c = sole_consumer(pl, cur);
            if (c >= 0 && pl->nodes[c].op == "add" && !pl->nodes[c].fused_into_other) {
                Node& a = pl->nodes[c];
                const int other = a.in[0] == cur ? a.in[1] : a.in[0];
                Value* ov = pl->find(other);
                if (other != cur && ov->kind == VKind::Intermediate && ov->producer < c && ov->shape == pl->find(cur)->shape) {
                    st.in1 = other;
                    a.fused_into_other = true;
                    cur = a.out;
                    emit_at = c;
                    c = sole_consumer(pl, cur);
                }
            }
            if (c >= 0 && pl->nodes[c].op == "nn_relu" && !pl->nodes[c].fused_into_other) {
                st.relu = true;
                pl->nodes[c].fused_into_other = true;
                cur = pl->nodes[c].out;
                emit_at = c;
            }
            st.N = (int)data->shape[0]; st.C = (int)data->shape[1]; st.H = (int)data->shape[2]; st.W = (int)data->shape[3];
            {   // stem conv -> relu -> max_pool2d(3x3, s2, p1): pool inside the direct stem kernel's epilogue
                const int pc = sole_consumer(pl, cur);
                const char* e1 = getenv("KXC_B200_STEM_DIRECT");
                const char* e2 = getenv("KXC_B200_STEM_POOL_FUSE");  // "0" keeps the separate pooling kernel
                if (pc >= 0 && pl->nodes[pc].op == "nn_max_pool2d" && !pl->nodes[pc].fused_into_other && st.relu && st.in1 < 0 &&
                    is_input(n.in[0]) && pl->nodes[pc].out != pl->output_id && (!e1 || atoi(e1) != 0) && (!e2 || atoi(e2) != 0) &&
                    n.conv.strides[0] == 2 && n.conv.strides[1] == 2 && n.conv.dilation[0] == 1 && n.conv.dilation[1] == 1) {
                    const auto& pa = pl->nodes[pc].pool;
                    const int KHc = (int)w->shape[2], KWc = (int)w->shape[3];
                    const int OHc = (int)conv_out_dim(st.H, KHc, 2, n.conv.padding[0], 1);
                    const int OWc = (int)conv_out_dim(st.W, KWc, 2, n.conv.padding[1], 1);
                    const int Wpc = (std::max(st.W + 2 * n.conv.padding[1], 2 * (OWc - 1) + 8) + 3) / 4 * 4;
                    const bool pool_ok = pa.pool_size[0] == 3 && pa.pool_size[1] == 3 && pa.strides[0] == 2 && pa.strides[1] == 2 &&
                                         pa.padding[0] == 1 && pa.padding[1] == 1 && pa.padding[2] == 1 && pa.padding[3] == 1 &&
                                         pa.ceil_mode == 0;
                    if (pool_ok && st.C <= 4 && KWc <= 8 && st.W >= 8 &&
                        stem_direct_applicable(dt, st.C, (int)w->shape[0], KHc, KWc, OWc, Wpc) && stem_pool_applicable(OHc, OWc, 3, 2, 1)) {
                        st.fused_pool = 1;
                        pl->nodes[pc].fused_into_other = true;
                        cur = pl->nodes[pc].out;
                        emit_at = pc;
                        const char* e3 = getenv("KXC_B200_STEM_FUSED_INPUT");  // "0" keeps the pack kernel + packed-input kernel
                        if ((!e3 || atoi(e3) != 0) && n.conv.padding[0] == KHc / 2 && n.conv.padding[1] == KWc / 2 &&
                            stem_pool_nchw_applicable(dt, st.C, (int)w->shape[0], KHc, KWc, st.W, OHc, OWc, Wpc))
                            st.direct_input = 1;
                    }
                }
            }
            st.out = cur;
            st.pool = {};  // unused
            // weight record
            PackedWeight pw;
            pw.const_id = n.in[1];
            pw.O = (int)w->shape[0]; pw.C = (int)w->shape[1]; pw.KH = (int)w->shape[2]; pw.KW = (int)w->shape[3];
            const bool stem = !pl->x3 && is_input(n.in[0]) && st.C <= 4 && n.conv.strides[0] == 2 && n.conv.strides[1] == 2 &&
                              n.conv.dilation[0] == 1 && n.conv.dilation[1] == 1 && pw.KW <= 8 && st.W >= 8;
            if (stem) {
                pw.mode = 1;
                pw.cpad = 4;
                pw.bytes = (size_t)pw.O * pw.KH * 32 * eb;
            } else {
                pw.mode = 0;
                pw.cpad = tc_channel_pad(dt, st.C);
                if (!is_input(n.in[0]) && pw.cpad != st.C)
                    return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_conv2d over %d channels: intermediate channel counts must be 16/32/64k for bf16 (8/16/32k for tf32)", st.C);
                pw.bytes = (size_t)pw.O * pw.KH * pw.KW * pw.cpad * eb;
            }
            st.cpad = pw.cpad;
            st.weight = (int)pl->weights.size();
            pl->weights.push_back(pw);
            // stash conv attrs in the pool struct slots we do not otherwise use
            st.pad_h = n.conv.padding[0]; st.pad_w = n.conv.padding[1];
            st.pool.strides[0] = n.conv.strides[0]; st.pool.strides[1] = n.conv.strides[1];
            st.pool.pool_size[0] = n.conv.dilation[0]; st.pool.pool_size[1] = n.conv.dilation[1];
            st.Hp = stem ? 1 : 0;  // marks stem until geometry is filled below
        } else if (n.op == "add" || n.op == "nn_relu") {
            st.kind = SKind::Eltwise;
            st.in0 = n.in[0];
            st.in1 = n.op == "add" ? n.in[1] : -1;
            st.relu = n.op == "nn_relu";
            int cur = n.out;
            if (n.op == "add") {
                const int c = sole_consumer(pl, cur);
                if (c >= 0 && pl->nodes[c].op == "nn_relu" && !pl->nodes[c].fused_into_other) {
                    st.relu = true;
                    pl->nodes[c].fused_into_other = true;
                    cur = pl->nodes[c].out;
                    emit_at = c;
                }
            }
            st.out = cur;
            st.numel = numel_of(pl->find(cur)->shape);
            if (is_const(st.in0) || is_input(st.in0) || (st.in1 >= 0 && (is_const(st.in1) || is_input(st.in1))))
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: elementwise ops over graph inputs/constants are not supported");
        } else if (n.op == "nn_max_pool2d") {
            Value* x = pl->find(n.in[0]);
            if (x->kind != VKind::Intermediate) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: pooling over a graph input/constant");
            st.kind = SKind::MaxPool;
            st.in0 = n.in[0]; st.out = n.out; st.pool = n.pool;
            st.N = (int)x->shape[0]; st.C = (int)x->shape[1]; st.H = (int)x->shape[2]; st.W = (int)x->shape[3];
            st.OH = (int)pl->find(n.out)->shape[2]; st.OW = (int)pl->find(n.out)->shape[3];
            if (st.C % lanes) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: pooling needs a channel count that is a multiple of %d", lanes);
        } else if (n.op == "nn_global_avg_pool2d") {
            Value* x = pl->find(n.in[0]);
            if (x->kind != VKind::Intermediate) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: pooling over a graph input/constant");
            st.kind = SKind::Gap;
            st.in0 = n.in[0]; st.out = n.out;
            st.N = (int)x->shape[0]; st.C = (int)x->shape[1]; st.H = (int)x->shape[2]; st.W = (int)x->shape[3];
            if (st.C % lanes) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: pooling needs a channel count that is a multiple of %d", lanes);
        } else if (n.op == "nn_flatten") {
            Value* x = pl->find(n.in[0]);
            bool trailing_ones = true;
            for (size_t i = 2; i < x->shape.size(); ++i) trailing_ones = trailing_ones && x->shape[i] == 1;
            if (x->kind != VKind::Intermediate || !trailing_ones)
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_flatten is supported on [N,C,1,1] / [N,C] intermediates only");
            pl->find(n.out)->alias_of = n.in[0];
            continue;
        } else if (n.op == "nn_dense" || n.op == "nn_gemm") {
            const bool gemm = n.op == "nn_gemm";
            if (gemm && ((double)n.gemm.alpha != 1.0 || (double)n.gemm.beta != 1.0))
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_gemm with alpha/beta != 1 (use kxc_b200_nn_gemm)");
            if (!is_const(n.in[1]) || (gemm && !is_const(n.in[2])) || pl->find(n.in[0])->kind != VKind::Intermediate)
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: dense needs an intermediate lhs and constant weight/bias");
            st.kind = SKind::Gemm;
            st.in0 = n.in[0]; st.out = n.out;
            st.bias_const = gemm ? n.in[2] : -1;
            Value* a = pl->find(n.in[0]);
            Value* b = pl->find(n.in[1]);
            const bool transB = !gemm || n.gemm.transB == 1;
            PackedWeight pw;
            pw.const_id = n.in[1];
            pw.mode = transB ? 2 : 3;
            pw.O = (int)pl->find(n.out)->shape[1];
            pw.C = (int)a->shape[1];
            pw.cpad = tc_channel_pad(dt, pw.C);
            if (pw.cpad != pw.C) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: dense reduction length %d must be 16/32/64k (bf16) or 8/16/32k (tf32)", pw.C);
            pw.bytes = (size_t)pw.O * pw.cpad * eb;
            (void)b;
            st.N = (int)a->shape[0]; st.C = pw.C;
            st.weight = (int)pl->weights.size();
            pl->weights.push_back(pw);
        } else {
            return fail(KXC_B200_ERR_UNSUPPORTED, "plan: op '%s' is not supported", n.op.c_str());
        }
        pending.push_back({emit_at, st});
    }
    std::stable_sort(pending.begin(), pending.end(), [](const auto& a, const auto& b) { return a.first < b.first; });

    // ---- a block's first convolution and the 1x1 convolution of its residual branch read the same tensor with
    // the same stride: compute both in one launch (the 1x1's only tap is the other filter's centre tap) ----
    {
        const char* e = getenv("KXC_B200_DUAL_CONV");  // "0" keeps two launches (A/B runs)
        const bool enabled = dt == kTcBF16 && !(e && atoi(e) == 0);
        auto geom = [&](const Step& st, int* kh, int* kw, int* stride, int* o) {
            const PackedWeight& pw = pl->weights[st.weight];
            *kh = pw.KH; *kw = pw.KW; *o = pw.O; *stride = st.pool.strides[0];
        };
        for (size_t a = 0; enabled && a < pending.size(); ++a) {
            Step& A = pending[a].second;
            if (A.kind != SKind::Conv || A.in1 >= 0 || A.fused_pool || A.weight2 >= 0 || is_input(A.in0) || A.Hp == 1) continue;
            int akh, akw, as, ao;
            geom(A, &akh, &akw, &as, &ao);
            if (akh * akw == 1 || A.pool.strides[0] != A.pool.strides[1]) continue;
            if (!tc_dual_applicable(dt, kOutNHWC_BF16, A.cpad, ao, akh, akw, as, A.pad_h, A.pad_w, A.pool.pool_size[0], A.pool.pool_size[1])) continue;
            if (direct3x3_applicable(dt, A.C, ao, akh, akw, as, A.pad_h, A.pad_w, 1, 1, (int)pl->find(A.out)->shape[3])) continue;
            if (pl->root_of(A.out) == pl->root_of(pl->output_id)) continue;
            {   // The two accumulators limit the tile to 128 channels and single CTAs. Measured at 1024 images: for
                // Cout = 128 one launch instead of two saves 25 % (0.260 -> 0.195 ms), for Cout >= 256 losing the 256-wide
                // paired tile costs more than the second launch (0.145 -> 0.164 ms); with few tiles (128 images per
                // GPU) the second launch's fixed cost dominates again (0.042 -> 0.031 ms).
                const Value* ov = pl->find(A.out);
                int bw, bh, bni;
                tc_pick_tile(A.N, (int)ov->shape[2], (int)ov->shape[3], &bw, &bh, &bni);
                const long long m_tiles = (long long)(((int)ov->shape[3] + bw - 1) / bw) * (((int)ov->shape[2] + bh - 1) / bh) *
                                          ((A.N + bni - 1) / bni);
                if (ao > 128 && m_tiles > 256) continue;
            }
            for (size_t b = 0; b < pending.size(); ++b) {
                if (b == a) continue;
                Step& B = pending[b].second;
                if (B.kind != SKind::Conv || B.in0 != A.in0 || B.in1 >= 0 || B.fused_pool || B.weight2 >= 0) continue;
                int bkh, bkw, bs, bo;
                geom(B, &bkh, &bkw, &bs, &bo);
                if (bkh != 1 || bkw != 1 || bs != as || B.pool.strides[0] != B.pool.strides[1] || bo != ao || B.pad_h != 0 || B.pad_w != 0 ||
                    B.cpad != A.cpad || pl->root_of(B.out) == pl->root_of(pl->output_id))
                    continue;
                // B's result now appears where A is emitted: every user of it must come later
                const int at = std::min(pending[a].first, pending[b].first);
                bool ok = true;
                for (size_t c = 0; c < pending.size(); ++c) {
                    if (c == a || c == b) continue;
                    const Step& U = pending[c].second;
                    if ((U.in0 == B.out || U.in1 == B.out || U.in0 == A.out || U.in1 == A.out) && pending[c].first <= std::max(pending[a].first, pending[b].first)) ok = false;
                }
                if (!ok) continue;
                A.weight2 = B.weight;
                A.bias2_const = B.bias_const;
                A.out2 = B.out;
                A.relu2 = B.relu;
                // emit at the later of the two positions: both only need the shared input, which is alive until then
                pending[a].first = std::max(pending[a].first, pending[b].first);
                (void)at;
                pending.erase(pending.begin() + b);
                if (b < a) --a;
                break;
            }
        }
        std::stable_sort(pending.begin(), pending.end(), [](const auto& x, const auto& y) { return x.first < y.first; });
    }

    // input conversion steps go first
    for (auto& pr : pending) {
        Step& st = pr.second;
        if (st.kind != SKind::Conv || !is_input(st.in0) || st.direct_input) continue;
        const bool stem = st.Hp == 1;
        const int key = st.in0 * 2 + (stem ? 1 : 0);
        if (input_copy.count(key)) continue;
        Step cv{};
        cv.kind = stem ? SKind::InputStem : SKind::InputNHWC;
        cv.in0 = st.in0;
        cv.N = st.N; cv.C = st.C; cv.H = st.H; cv.W = st.W;
        cv.cpad = st.cpad;
        if (stem) {
            const PackedWeight& pw = pl->weights[st.weight];
            const int OW = (int)conv_out_dim(st.W, pw.KW, 2, st.pad_w, 1);
            cv.pad_h = st.pad_h; cv.pad_w = st.pad_w;
            cv.Hp = st.H + 2 * st.pad_h;
            cv.Hp += cv.Hp & 1;
            cv.Wp = std::max(st.W + 2 * st.pad_w, 2 * (OW - 1) + 8);
            cv.Wp = (cv.Wp + 3) / 4 * 4;  // the pack kernel writes four pixels per thread; rows stay 16-byte multiples
        }
        // the internal copy is a synthetic value with a negative id
        const int copy_id = -(int)(input_copy.size() + 2);  // -1 means "no value"
        Value v;
        v.id = copy_id;
        v.kind = VKind::Intermediate;
        v.bytes = stem ? (size_t)cv.N * cv.Hp * cv.Wp * 4 * eb : (size_t)cv.N * cv.H * cv.W * cv.cpad * eb;
        pl->values[copy_id] = v;
        cv.out = copy_id;
        input_copy[key] = copy_id;
        pl->steps.push_back(cv);
    }
    for (auto& pr : pending) {
        Step st = pr.second;
        if (st.kind == SKind::Conv && is_input(st.in0) && st.direct_input) {
            // geometry of the packed layout the kernel builds in shared memory (same as the InputStem step's)
            const PackedWeight& pw = pl->weights[st.weight];
            const int OW = (int)conv_out_dim(st.W, pw.KW, 2, st.pad_w, 1);
            st.Hp = st.H + 2 * st.pad_h;
            st.Hp += st.Hp & 1;
            st.Wp = (std::max(st.W + 2 * st.pad_w, 2 * (OW - 1) + 8) + 3) / 4 * 4;
            st.src_input = st.in0;
            st.in0 = -1;
        } else if (st.kind == SKind::Conv && is_input(st.in0)) {
            const bool stem = st.Hp == 1;
            const int copy_id = input_copy[st.in0 * 2 + (stem ? 1 : 0)];
            st.src_input = st.in0;
            st.in0 = copy_id;
            if (stem) {
                for (auto& s2 : pl->steps)
                    if (s2.out == copy_id) { st.Hp = s2.Hp; st.Wp = s2.Wp; }
            }
        } else if (st.kind == SKind::Conv) {
            st.Hp = 0;
        }
        pl->steps.push_back(st);
    }
    // graph output: written directly by a conv/gemm epilogue, else converted by one extra step
    {
        Step& last = pl->steps.back();
        bool direct = false;
        for (auto& st : pl->steps) {
            if (st.out >= 0 && pl->root_of(st.out) == pl->root_of(pl->output_id) && pl->root_of(st.out) == st.out &&
                ((st.kind == SKind::Conv && st.in1 < 0) || st.kind == SKind::Gemm) && pl->find(pl->output_id)->alias_of < 0) {
                st.out_is_graph_output = true;
                direct = true;
            }
        }
        (void)last;
        if (!direct) {
            Value* ov = pl->find(pl->output_id);
            Step cv{};
            cv.kind = SKind::ToNCHW;
            cv.in0 = pl->output_id;
            cv.out_is_graph_output = true;
            if (ov->shape.size() == 4) {
                cv.N = (int)ov->shape[0]; cv.C = (int)ov->shape[1]; cv.H = (int)ov->shape[2]; cv.W = (int)ov->shape[3];
            } else if (ov->shape.size() == 2) {
                cv.N = (int)ov->shape[0]; cv.C = (int)ov->shape[1]; cv.H = 1; cv.W = 1;
            } else {
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: output rank %zu", ov->shape.size());
            }
            pl->steps.push_back(cv);
        }
    }

    // ---- storage sizes and liveness ----
    for (size_t si = 0; si < pl->steps.size(); ++si) {
        Step& st = pl->steps[si];
        auto touch = [&](int id) {
            if (id == -1) return;
            Value* v = pl->find(pl->root_of(id));
            if (!v || v->kind != VKind::Intermediate) return;
            if (v->first_step < 0) v->first_step = (int)si;
            v->last_step = (int)si;
        };
        touch(st.in0);
        touch(st.in1);
        if (st.out != -1 && !st.out_is_graph_output) {
            Value* v = pl->find(st.out);
            if (v->id >= 0) v->bytes = (size_t)numel_of(v->shape) * eb;
            touch(st.out);
        }
        if (st.out2 != -1) {
            Value* v = pl->find(st.out2);
            v->bytes = (size_t)numel_of(v->shape) * eb;
            touch(st.out2);
        }
    }
    // greedy arena assignment with reuse of dead blocks
    struct Block { size_t off, size; };
    std::vector<Block> free_blocks;
    size_t top = 0;
    for (size_t si = 0; si < pl->steps.size(); ++si) {
        Step& st = pl->steps[si];
        for (int which = 0; which < 2; ++which) {
            const int oid = which == 0 ? ((st.out != -1 && !st.out_is_graph_output) ? st.out : -1) : st.out2;
            if (oid == -1) continue;
            Value* v = pl->find(oid);
            if (v->alias_of < 0 && !v->has_storage) {
                const size_t need = align_up(std::max<size_t>(v->bytes, 16), 1024);
                int best = -1;
                for (size_t b = 0; b < free_blocks.size(); ++b)
                    if (free_blocks[b].size >= need && (best < 0 || free_blocks[b].size < free_blocks[best].size)) best = (int)b;
                if (best >= 0) {
                    v->offset = free_blocks[best].off;
                    if (free_blocks[best].size > need) {
                        free_blocks[best].off += need;
                        free_blocks[best].size -= need;
                    } else {
                        free_blocks.erase(free_blocks.begin() + best);
                    }
                } else {
                    v->offset = top;
                    top += need;
                }
                v->has_storage = true;
                v->bytes = need;
            }
        }
        for (auto& kv : pl->values) {
            Value& v = kv.second;
            if (v.kind == VKind::Intermediate && v.has_storage && v.alias_of < 0 && v.last_step == (int)si) {
                free_blocks.push_back({v.offset, v.bytes});
                // merge adjacent free blocks
                std::sort(free_blocks.begin(), free_blocks.end(), [](const Block& a, const Block& b) { return a.off < b.off; });
                for (size_t b = 0; b + 1 < free_blocks.size();) {
                    if (free_blocks[b].off + free_blocks[b].size == free_blocks[b + 1].off) {
                        free_blocks[b].size += free_blocks[b + 1].size;
                        free_blocks.erase(free_blocks.begin() + b + 1);
                    } else {
                        ++b;
                    }
                }
            }
        }
    }
    pl->arena_bytes = std::max<size_t>(top, 1024);
    KXC_CUDA_TRY(cudaMalloc(&pl->arena, pl->arena_bytes));
    size_t wtop = 0;
    for (auto& w : pl->weights) wtop += align_up(w.bytes, 1024) * (pl->x3 ? 2 : 1);
    KXC_CUDA_TRY(cudaMalloc(&pl->weight_arena, std::max<size_t>(wtop, 1024)));
    wtop = 0;
    for (auto& w : pl->weights) {
        w.ptr = static_cast<uint8_t*>(pl->weight_arena) + wtop;
        wtop += align_up(w.bytes, 1024);
        if (pl->x3) {
            w.ptr_lo = static_cast<uint8_t*>(pl->weight_arena) + wtop;
            wtop += align_up(w.bytes, 1024);
        }
    }
    if (pl->x3) {
        // high / low halves of the largest convolution or dense input
        size_t half = 0;
        for (auto& st : pl->steps) {
            if (st.kind == SKind::Conv) half = std::max(half, align_up((size_t)st.N * st.H * st.W * st.cpad * 4, 1024));
            if (st.kind == SKind::Gemm) half = std::max(half, align_up((size_t)st.N * pl->weights[st.weight].cpad * 4, 1024));
        }
        pl->x3_half_bytes = half;
        KXC_CUDA_TRY(cudaMalloc(&pl->x3_scratch, std::max<size_t>(2 * half, 1024)));
    }

    // ---- tensor maps and launch parameters ----
    for (auto& st : pl->steps) {
        if (st.kind == SKind::Conv) {
            PackedWeight& pw = pl->weights[st.weight];
            Value* ov = pl->find(st.out);
            const int stem_oh = (int)conv_out_dim(st.H, pw.KH, 2, st.pad_h, 1), stem_ow = (int)conv_out_dim(st.W, pw.KW, 2, st.pad_w, 1);
            if (st.direct_input) {
                pw.mode = 5;
                if (stem_stacked_weight_bytes() > pw.bytes) return fail(KXC_B200_ERR_INVALID, "plan: stacked stem weights do not fit their slot");
            }
            if (pw.mode == 1 && !st.out_is_graph_output) {
                // the direct stem kernel writes bf16 NHWC only; its packed weights take the same number of bytes
                const char* e = getenv("KXC_B200_STEM_DIRECT");  // "0" keeps the implicit-GEMM stem for A/B runs
                if ((!e || atoi(e) != 0) && stem_direct_applicable(dt, st.C, pw.O, pw.KH, pw.KW, stem_ow, st.Wp) &&
                    stem_direct_weight_bytes(pw.KH) <= pw.bytes)
                    pw.mode = 4;
            }
            TcOutMode om = st.out_is_graph_output ? kOutNCHW_F32 : (dt == kTcBF16 ? kOutNHWC_BF16 : kOutNHWC_F32);
            if (st.in1 >= 0 && st.out_is_graph_output)
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: a residual convolution cannot be the graph output");
            if (!st.out_is_graph_output && (pw.O % lanes))
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: %d output channels must be a multiple of %d", pw.O, lanes);
            if (st.fused_pool && pw.mode != 4 && pw.mode != 5) return fail(KXC_B200_ERR_UNSUPPORTED, "plan: fused stem pooling needs the direct stem kernel");
            if (pw.mode == 5) {
                st.direct = 4;
                KXC_TRY(stem_pool_nchw_setup(&st.params, pw.ptr, st.N, st.C, st.H, st.W, stem_oh, stem_ow, st.pad_h, st.pad_w, st.Hp, st.Wp));
                st.cfg = TcConfig{dt, 64, 64, om};
            } else if (pw.mode == 4) {
                st.direct = 2;
                KXC_TRY(stem_direct_setup(&st.params, pl->storage(st.in0), pw.ptr, st.N, stem_oh, stem_ow, pw.KH, st.Hp, st.Wp));
                st.cfg = TcConfig{dt, 64, 64, om};
            } else if (pw.mode == 1) {
                KXC_TRY(setup_stem(pl, st, st.N, st.C, st.H, st.W, pw.O, pw.KH, pw.KW, st.pad_h, st.pad_w, pl->storage(st.in0), pw.ptr, om));
            } else {
                if (st.pool.strides[0] != st.pool.strides[1])
                    return fail(KXC_B200_ERR_UNSUPPORTED, "plan: nn_conv2d with different strides in h and w");
                const char* dmode = getenv("KXC_B200_DIRECT3X3");  // "0" selects the implicit-GEMM kernel for A/B runs
                const int direct_mode = dmode ? atoi(dmode) : 1;
                const char* rmode = getenv("KXC_B200_ROWSTACK");  // "0" keeps the tap-by-tap direct kernel (A/B runs)
                if (direct_mode > 0 && (!rmode || atoi(rmode) != 0) && !st.out_is_graph_output &&
                    rowstack3x3_applicable(dt, st.C, pw.O, pw.KH, pw.KW, st.pool.strides[0], st.pad_h, st.pad_w, st.pool.pool_size[0],
                                           st.pool.pool_size[1], st.H, st.W)) {
                    st.direct = 3;
                    KXC_TRY(rowstack3x3_setup(&st.params, pl->storage(st.in0), pw.ptr, st.N, st.H, st.W));
                    st.cfg = TcConfig{dt, 128, 64, om};
                } else if (rowstack128_wanted(st.in1 >= 0, (long long)st.N * st.H * st.W) && !st.out_is_graph_output && !pl->x3 &&
                           st.weight2 < 0 &&
                           rowstack128_applicable(dt, st.C, pw.O, pw.KH, pw.KW, st.pool.strides[0], st.pad_h, st.pad_w,
                                                  st.pool.pool_size[0], st.pool.pool_size[1])) {
                    st.direct = 5;
                    KXC_TRY(rowstack128_setup(&st.params, pl->storage(st.in0), pw.ptr, st.N, st.H, st.W));
                    st.cfg = TcConfig{dt, 128, 192, om};
                    st.cfg.ctas = 2;
                } else if (direct_mode > 0 && !st.out_is_graph_output &&
                    direct3x3_applicable(dt, st.C, pw.O, pw.KH, pw.KW, st.pool.strides[0], st.pad_h, st.pad_w, st.pool.pool_size[0],
                                         st.pool.pool_size[1], (int)ov->shape[3])) {
                    st.direct = 1;
                    KXC_TRY(direct3x3_setup(&st.params, pl->storage(st.in0), pw.ptr, st.N, st.H, st.W));
                    st.cfg = TcConfig{dt, 128, 64, om};
                } else if (st.weight2 >= 0) {
                    KXC_TRY(tc_setup_dual(&st.params, &st.cfg, pl->storage(st.in0), pw.ptr, pl->weights[st.weight2].ptr, st.N, st.H, st.W,
                                          st.cpad, pw.O, pw.KH, pw.KW, st.pool.strides[0], st.pad_h, st.pad_w));
                    st.params.out2 = pl->storage(st.out2);
                    st.params.relu2 = st.relu2 ? 1 : 0;
                } else
                KXC_TRY(tc_setup_conv(&st.params, &st.cfg, dt, om, pl->storage(st.in0), pw.ptr, st.N, st.H, st.W, st.cpad, pw.O,
                                      pw.KH, pw.KW, st.pool.strides[0], st.pad_h, st.pad_w, st.pool.pool_size[0], st.pool.pool_size[1]));
            }
            st.params.relu = st.relu ? 1 : 0;
            st.params.round_out_tf32 = (!st.out_is_graph_output && dt == kTcTF32 && !pl->x3) ? 1 : 0;
            st.params.residual = st.in1 >= 0 ? pl->storage(st.in1) : nullptr;
            st.params.out = st.out_is_graph_output ? nullptr : pl->storage(st.out);
            if (pl->x3) {
                // three passes, small terms first; each later pass adds the previous sum through its residual input
                uint8_t* hi = static_cast<uint8_t*>(pl->x3_scratch);
                uint8_t* lo = hi + pl->x3_half_bytes;
                const void* act_hi = st.src_input >= 0 ? pl->storage(st.in0) : hi;  // a graph input's NHWC copy already holds the high part
                TcConfig c2{};
                KXC_TRY(tc_setup_conv(&st.params, &st.cfg, dt, om, act_hi, pw.ptr, st.N, st.H, st.W, st.cpad, pw.O, pw.KH, pw.KW,
                                      st.pool.strides[0], st.pad_h, st.pad_w, st.pool.pool_size[0], st.pool.pool_size[1]));
                KXC_TRY(tc_setup_conv(&st.params_lohi, &c2, dt, om, lo, pw.ptr, st.N, st.H, st.W, st.cpad, pw.O, pw.KH, pw.KW,
                                      st.pool.strides[0], st.pad_h, st.pad_w, st.pool.pool_size[0], st.pool.pool_size[1]));
                KXC_TRY(tc_setup_conv(&st.params_hilo, &c2, dt, om, act_hi, pw.ptr_lo, st.N, st.H, st.W, st.cpad, pw.O, pw.KH, pw.KW,
                                      st.pool.strides[0], st.pad_h, st.pad_w, st.pool.pool_size[0], st.pool.pool_size[1]));
                st.params.relu = st.relu ? 1 : 0;
                st.params.out = st.out_is_graph_output ? nullptr : pl->storage(st.out);
                st.params.residual = st.params.out;  // pass 3 adds the sum of passes 1 and 2
                st.params_lohi.out = st.params.out;
                st.params_lohi.residual = st.in1 >= 0 ? pl->storage(st.in1) : nullptr;
                st.params_hilo.out = st.params.out;
                st.params_hilo.residual = st.params.out;
            }
            if (st.direct == 3) KXC_TRY(rowstack3x3_bind(&st.params));
            if (st.direct == 5) KXC_TRY(rowstack128_bind(&st.params));
            if (st.direct == 0 && pw.mode == 0 && !st.out_is_graph_output) KXC_TRY(tc_bind_store(&st.params, st.cfg));
            (void)ov;
        } else if (st.kind == SKind::Gemm) {
            const PackedWeight& pw = pl->weights[st.weight];
            TcOutMode om = st.out_is_graph_output ? kOutNHWC_F32 : (dt == kTcBF16 ? kOutNHWC_BF16 : kOutNHWC_F32);
            if (!st.out_is_graph_output && (pw.O % lanes))
                return fail(KXC_B200_ERR_UNSUPPORTED, "plan: %d dense outputs must be a multiple of %d", pw.O, lanes);
            KXC_TRY(tc_setup_conv(&st.params, &st.cfg, dt, om, pl->x3 ? pl->x3_scratch : pl->storage(st.in0), pw.ptr, st.N, 1, 1, pw.cpad,
                                  pw.O, 1, 1, 1, 0, 0, 1, 1));
            st.params.relu = 0;
            st.params.round_out_tf32 = (!st.out_is_graph_output && dt == kTcTF32 && !pl->x3) ? 1 : 0;
            st.params.residual = nullptr;
            st.params.out = st.out_is_graph_output ? nullptr : pl->storage(st.out);
            if (pl->x3) {
                uint8_t* hi = static_cast<uint8_t*>(pl->x3_scratch);
                uint8_t* lo = hi + pl->x3_half_bytes;
                TcConfig c2{};
                KXC_TRY(tc_setup_conv(&st.params_lohi, &c2, dt, om, lo, pw.ptr, st.N, 1, 1, pw.cpad, pw.O, 1, 1, 1, 0, 0, 1, 1));
                KXC_TRY(tc_setup_conv(&st.params_hilo, &c2, dt, om, hi, pw.ptr_lo, st.N, 1, 1, pw.cpad, pw.O, 1, 1, 1, 0, 0, 1, 1));
                st.params.residual = st.params.out;
                st.params_lohi.out = st.params.out;
                st.params_lohi.residual = nullptr;
                st.params_hilo.out = st.params.out;
                st.params_hilo.residual = st.params.out;
            }
        }
    }
    pl->finalized = true;
    return KXC_B200_OK;
}

namespace {
// NVTX range around the host side of one launch (a no-op unless the plan asked for ranges; without a tool attached
// the NVTX calls themselves return at once).
struct LaunchRange {
    bool on;
    LaunchRange(const kxc_b200_plan* pl, size_t index) : on(pl->nvtx && index < pl->nvtx_names.size()) {
        if (on) nvtxRangePushA(pl->nvtx_names[index].c_str());
    }
    explicit LaunchRange(const char* name, bool enable) : on(enable) {
        if (on) nvtxRangePushA(name);
    }
    ~LaunchRange() {
        if (on) nvtxRangePop();
    }
    LaunchRange(const LaunchRange&) = delete;
    LaunchRange& operator=(const LaunchRange&) = delete;
};
}  // namespace

static int32_t plan_run_core(kxc_b200_plan* pl, void** packed_args, void* stream, cudaEvent_t* events);

static int32_t plan_run_impl(kxc_b200_plan* pl, void** packed_args, void* stream, cudaEvent_t* events) {
    if (!pl || !pl->finalized || pl->tail_out < 0 || !packed_args) return plan_run_core(pl, packed_args, stream, events);
    const size_t nargs = pl->inputs.size() + pl->constants.size();
    if (!packed_args[nargs]) return fail(KXC_B200_ERR_INVALID, "plan_run: packed_args[%zu] is null", nargs);
    if (pl->tail_rows * pl->tail_len == 0) return KXC_B200_OK;
    std::vector<void*> args(packed_args, packed_args + nargs + 1);
    args[nargs] = pl->tail_buf;
    KXC_TRY(plan_run_core(pl, args.data(), stream, events));  // records events[0 .. core launches]
    const size_t ncore = pl->precision == KXC_B200_PREC_FP32 ? pl->xsteps.size() : pl->steps.size();
    {
        LaunchRange range(pl, ncore);
        kxc_b200_softmax_desc d{};
        d.rank = 2;
        d.shape[0] = pl->tail_rows;
        d.shape[1] = pl->tail_len;
        d.axis = 1;
        void* io[2] = {pl->tail_buf, packed_args[nargs]};
        KXC_TRY(kxc_b200_softmax(io, &d, stream));
    }
    if (events) KXC_CUDA_TRY(cudaEventRecord(events[ncore + 1], static_cast<cudaStream_t>(stream)));
    return KXC_B200_OK;
}

static int32_t plan_run_core(kxc_b200_plan* pl, void** packed_args, void* stream, cudaEvent_t* events) {
    if (!pl || !pl->finalized) return fail(KXC_B200_ERR_INVALID, "plan_run: plan is not finalized");
    if (pl->precision == KXC_B200_PREC_FP32) return run_exact(pl, packed_args, stream, events);
    if (!packed_args) return fail(KXC_B200_ERR_INVALID, "plan_run: null packed_args");
    KXC_TRY(require_device());
    int dev = -1;
    KXC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != pl->device) return fail(KXC_B200_ERR_INVALID, "plan_run: plan was finalized on device %d, current device is %d", pl->device, dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const TcDType dt = pl->dtype;
    const size_t nargs = pl->inputs.size() + pl->constants.size();
    for (size_t i = 0; i <= nargs; ++i)
        if (!packed_args[i]) return fail(KXC_B200_ERR_INVALID, "plan_run: packed_args[%zu] is null", i);
    void* out_ptr = packed_args[nargs];
    auto arg_of = [&](int id) -> void* { return packed_args[pl->find(id)->arg_index]; };

    // (re)pack constants whose source pointer changed
    for (auto& w : pl->weights) {
        const void* src = arg_of(w.const_id);
        if (src == w.source) continue;
        switch (w.mode) {
            case 0: KXC_TRY(pack_weights_ohwi(src, w.ptr, dt, w.O, w.C, w.KH, w.KW, w.cpad, s)); break;
            case 1: KXC_TRY(stem_pack_weights(static_cast<const float*>(src), w.ptr, dt, w.O, w.C, w.KH, w.KW, s)); break;
            case 4: KXC_TRY(stem_direct_pack_weights(static_cast<const float*>(src), w.ptr, w.O, w.C, w.KH, w.KW, s)); break;
            case 5: KXC_TRY(stem_stacked_pack_weights(static_cast<const float*>(src), w.ptr, w.O, w.C, w.KW, s)); break;
            case 2: KXC_TRY(convert_rows(static_cast<const float*>(src), w.ptr, dt, w.O, w.C, w.cpad, s)); break;
            case 3: KXC_TRY(nchw_to_nhwc(src, w.ptr, dt, 1, w.C, w.O, w.cpad, s)); break;
        }
        if (pl->x3) {
            switch (w.mode) {
                case 0: KXC_TRY(pack_weights_ohwi(src, w.ptr_lo, dt, w.O, w.C, w.KH, w.KW, w.cpad, s, true)); break;
                case 2: KXC_TRY(convert_rows(static_cast<const float*>(src), w.ptr_lo, dt, w.O, w.C, w.cpad, s, true)); break;
                case 3: KXC_TRY(nchw_to_nhwc(src, w.ptr_lo, dt, 1, w.C, w.O, w.cpad, s, true)); break;
                default: return fail(KXC_B200_ERR_UNSUPPORTED, "plan: weight layout %d has no TF32X3 form", w.mode);
            }
        }
        w.source = src;
    }

    // Tensor-core launches alternate the direction in which they walk their work items (KXC_B200_TILE_ORDER=0: all
    // forward): a launch then begins with the images its producer finished last, whose lines are still in L2.
    static const bool alternate_order = [] {
        const char* e = getenv("KXC_B200_TILE_ORDER");
        return !(e != nullptr && e[0] == '0');
    }();
    int tc_index = 0;
    size_t step_index = 0;
    if (events) KXC_CUDA_TRY(cudaEventRecord(events[0], s));
    for (auto& st : pl->steps) {
        if (step_index > 0 && events) KXC_CUDA_TRY(cudaEventRecord(events[step_index], s));
        LaunchRange range(pl, step_index);
        ++step_index;
        switch (st.kind) {
            case SKind::InputNHWC:
                KXC_TRY(nchw_to_nhwc(arg_of(st.in0), pl->storage(st.out), dt, st.N, st.C, st.H * st.W, st.cpad, s));
                break;
            case SKind::InputStem:
                KXC_TRY(stem_pack(static_cast<const float*>(arg_of(st.in0)), pl->storage(st.out), dt, st.N, st.C, st.H, st.W, st.Hp,
                                  st.Wp, st.pad_h, st.pad_w, s));
                break;
            case SKind::Conv:
            case SKind::Gemm: {
                TcParams p = st.params;
                p.bias = st.bias_const >= 0 ? static_cast<const float*>(arg_of(st.bias_const)) : nullptr;
                p.bias2 = st.bias2_const >= 0 ? static_cast<const float*>(arg_of(st.bias2_const)) : nullptr;
                if (st.out_is_graph_output) p.out = out_ptr;
                p.reverse = (alternate_order && !pl->x3 && (tc_index++ & 1)) ? 1 : 0;
                tc_finish_params(&p);
                if (st.weight2 >= 0 && ((reinterpret_cast<uintptr_t>(p.bias2) | reinterpret_cast<uintptr_t>(p.out2)) & 15u)) p.vec_ok = 0;
                if (pl->x3) {
                    uint8_t* hi = static_cast<uint8_t*>(pl->x3_scratch);
                    uint8_t* lo = hi + pl->x3_half_bytes;
                    const bool gemm = st.kind == SKind::Gemm;
                    const int cpad = gemm ? pl->weights[st.weight].cpad : st.cpad;
                    if (st.src_input >= 0) {
                        KXC_TRY(nchw_to_nhwc(arg_of(st.src_input), lo, dt, st.N, st.C, st.H * st.W, cpad, s, true));
                    } else {
                        const int64_t rows = gemm ? (int64_t)st.N : (int64_t)st.N * st.H * st.W;
                        const float* src = static_cast<const float*>(pl->storage(st.in0));
                        KXC_TRY(convert_rows(src, hi, dt, rows, cpad, cpad, s, false));
                        KXC_TRY(convert_rows(src, lo, dt, rows, cpad, cpad, s, true));
                    }
                    TcParams q = st.params_lohi;
                    if (st.out_is_graph_output) q.out = out_ptr;
                    tc_finish_params(&q);
                    KXC_TRY(tc_launch(st.cfg, q, s));
                    q = st.params_hilo;
                    if (st.out_is_graph_output) { q.out = out_ptr; q.residual = out_ptr; }
                    tc_finish_params(&q);
                    KXC_TRY(tc_launch(st.cfg, q, s));
                    if (st.out_is_graph_output) p.residual = out_ptr;
                    tc_finish_params(&p);
                    KXC_TRY(tc_launch(st.cfg, p, s));
                } else if (st.direct == 4) {
                    p.aux_in = arg_of(st.src_input);
                    KXC_TRY(stem_pool_nchw_launch(p, s));
                } else if (st.direct == 2) {
                    KXC_TRY(st.fused_pool ? stem_pool_launch(p, s) : stem_direct_launch(p, s));
                } else if (st.direct == 3) {
                    KXC_TRY(rowstack3x3_launch(p, s));
                } else if (st.direct == 5) {
                    KXC_TRY(rowstack128_launch(p, s));
                } else if (st.direct == 1) {
                    KXC_TRY(direct3x3_launch(p, s));
                } else {
                    KXC_TRY(tc_launch(st.cfg, p, s));
                }
                break;
            }
            case SKind::MaxPool:
                KXC_TRY(maxpool_nhwc(pl->storage(st.in0), pl->storage(st.out), dt, st.N, st.H, st.W, st.C, st.OH, st.OW,
                                     st.pool.pool_size[0], st.pool.pool_size[1], st.pool.strides[0], st.pool.strides[1],
                                     st.pool.padding[0], st.pool.padding[1], s));
                break;
            case SKind::Gap:
                KXC_TRY(gap_nhwc(pl->storage(st.in0), pl->storage(st.out), dt, st.N, st.H * st.W, st.C, s));
                break;
            case SKind::Eltwise:
                KXC_TRY(eltwise_nhwc(pl->storage(st.in0), st.in1 >= 0 ? pl->storage(st.in1) : nullptr, pl->storage(st.out), dt,
                                     st.numel, st.relu ? 1 : 0, s));
                break;
            case SKind::ToNCHW:
                KXC_TRY(nhwc_to_nchw_f32(pl->storage(st.in0), static_cast<float*>(out_ptr), dt, st.N, st.C, st.H * st.W, s));
                break;
        }
    }
    if (events) KXC_CUDA_TRY(cudaEventRecord(events[step_index], s));
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_set_cuda_graph(kxc_b200_plan* pl, int32_t enable) {
    if (!pl) return fail(KXC_B200_ERR_INVALID, "plan_set_cuda_graph: null plan");
    pl->use_graph = enable != 0;
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_set_nvtx(kxc_b200_plan* pl, int32_t enable) {
    if (!pl || !pl->finalized) return fail(KXC_B200_ERR_INVALID, "plan_set_nvtx: plan is not finalized");
    if (enable && pl->nvtx_names.empty()) {
        const int n = kxc_b200_plan_num_launches(pl);
        char name[192];
        for (int i = 0; i < n; ++i) {
            KXC_TRY(kxc_b200_plan_launch_info(pl, i, name, (int32_t)sizeof(name), nullptr, nullptr));
            pl->nvtx_names.emplace_back(name);
        }
    }
    pl->nvtx = enable != 0;
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_run(kxc_b200_plan* pl, void** packed_args, void* stream) {
    LaunchRange run_range("kxc_b200_plan_run", pl && pl->nvtx);
    if (!pl) return plan_run_impl(pl, packed_args, stream, nullptr);
    std::lock_guard<std::mutex> run_lock(pl->run_mu);
    if (!pl->finalized || !packed_args || !pl->use_graph) return plan_run_impl(pl, packed_args, stream, nullptr);
    const size_t nargs = pl->inputs.size() + pl->constants.size() + 1;
    bool packed = true;  // weights must already be packed from these constants: packing stays outside the graph
    for (auto& w : pl->weights) packed = packed && (w.source == packed_args[pl->find(w.const_id)->arg_index]);
    if (!packed) return plan_run_impl(pl, packed_args, stream, nullptr);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the legacy default stream cannot be captured: run eagerly there
    if (s == nullptr || s == cudaStreamLegacy) return plan_run_impl(pl, packed_args, stream, nullptr);
    kxc_b200_plan::GraphSlot* slot = nullptr;
    for (auto& g : pl->graph_slots)
        if (g.exec != nullptr && g.args.size() == nargs && std::equal(g.args.begin(), g.args.end(), packed_args)) slot = &g;
    if (slot == nullptr) {
        slot = &pl->graph_slots[pl->graph_next_slot];
        pl->graph_next_slot = (pl->graph_next_slot + 1) % kxc_b200_plan::kGraphSlots;
        if (slot->exec) {
            cudaGraphExecDestroy(slot->exec);
            slot->exec = nullptr;
        }
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();  // capture not possible on this stream right now: fall back to eager launches
            return plan_run_impl(pl, packed_args, stream, nullptr);
        }
        const int32_t rc = plan_run_impl(pl, packed_args, stream, nullptr);
        const cudaError_t e = cudaStreamEndCapture(s, &graph);
        if (rc != KXC_B200_OK) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        if (e != cudaSuccess) return fail(KXC_B200_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
        const cudaError_t ie = cudaGraphInstantiate(&slot->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) {
            slot->exec = nullptr;
            return fail(KXC_B200_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(ie));
        }
        slot->args.assign(packed_args, packed_args + nargs);
    }
    LaunchRange replay("cuda graph replay", pl->nvtx);
    KXC_CUDA_TRY(cudaGraphLaunch(slot->exec, s));
    return KXC_B200_OK;
}

extern "C" int32_t kxc_b200_plan_run_timed(kxc_b200_plan* pl, void** packed_args, void* stream, float* launch_ms,
                                           int32_t capacity) {
    if (!pl || !pl->finalized) return fail(KXC_B200_ERR_INVALID, "plan_run_timed: plan is not finalized");
    const int n = kxc_b200_plan_num_launches(pl);
    if (!launch_ms || capacity < n) return fail(KXC_B200_ERR_INVALID, "plan_run_timed: need room for %d durations", n);
    std::lock_guard<std::mutex> run_lock(pl->run_mu);
    std::vector<cudaEvent_t> ev(n + 1);
    for (auto& e : ev) KXC_CUDA_TRY(cudaEventCreate(&e));
    int32_t rc = plan_run_impl(pl, packed_args, stream, ev.data());
    if (rc == KXC_B200_OK) {
        cudaError_t e = cudaEventSynchronize(ev[n]);
        if (e != cudaSuccess) rc = fail(KXC_B200_ERR_CUDA, "plan_run_timed: %s", cudaGetErrorString(e));
        for (int i = 0; i < n && rc == KXC_B200_OK; ++i)
            if (cudaEventElapsedTime(&launch_ms[i], ev[i], ev[i + 1]) != cudaSuccess) rc = fail(KXC_B200_ERR_CUDA, "plan_run_timed: elapsed time");
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return rc;
}

// ---- measurement support ------------------------------------------------------------------------
extern "C" int32_t kxc_b200_plan_launch_info(kxc_b200_plan* pl, int32_t index, char* name, int32_t name_size,
                                             double* flops, double* bytes) {
    if (pl && pl->finalized && pl->tail_out >= 0 &&
        index == (int)(pl->precision == KXC_B200_PREC_FP32 ? pl->xsteps.size() : pl->steps.size())) {
        if (name && name_size > 0) snprintf(name, (size_t)name_size, "softmax rows%lld len%lld", (long long)pl->tail_rows, (long long)pl->tail_len);
        if (flops) *flops = 0.0;
        if (bytes) *bytes = 2.0 * (double)pl->tail_rows * (double)pl->tail_len * 4.0;
        return KXC_B200_OK;
    }
    if (pl && pl->finalized && pl->precision == KXC_B200_PREC_FP32) {
        if (index < 0 || index >= (int)pl->xsteps.size()) return fail(KXC_B200_ERR_INVALID, "plan_launch_info: bad index");
        const auto& xs = pl->xsteps[index];
        double fl = 0.0;
        if (xs.op == "nn_conv2d") {
            const auto& o = pl->find(xs.out)->shape;
            const auto& w = pl->find(xs.weight)->shape;
            fl = 2.0 * (double)numel_of(o) * (double)(w[1] * w[2] * w[3]);
        }
        if (name && name_size > 0) snprintf(name, (size_t)name_size, "%s (fp32, reference order)%s", xs.op.c_str(), xs.relu ? " +relu" : "");
        if (flops) *flops = fl;
        if (bytes) *bytes = 0.0;
        return KXC_B200_OK;
    }
    if (!pl || !pl->finalized || index < 0 || index >= (int)pl->steps.size())
        return fail(KXC_B200_ERR_INVALID, "plan_launch_info: bad plan or index");
    const Step& st = pl->steps[index];
    const double eb = pl->eb();
    double fl = 0.0, by = 0.0;
    char buf[160];
    switch (st.kind) {
        case SKind::Conv: {
            const PackedWeight& w = pl->weights[st.weight];
            const TcParams& p = st.params;
            const double out_elems = (double)p.N * p.OH * p.OW * w.O;
            fl = 2.0 * out_elems * w.C * w.KH * w.KW;  // padded taps counted, as the reference executes them
            if (st.weight2 >= 0) fl += 2.0 * out_elems * w.C;  // the 1x1 convolution computed by the same launch
            const double in_bytes = w.mode == 5 ? (double)st.N * st.C * st.H * st.W * 4.0
                                                : ((w.mode == 1 || w.mode == 4) ? (double)st.N * st.Hp * st.Wp * 4 * eb : (double)st.N * st.H * st.W * st.cpad * eb);
            by = in_bytes + (double)w.bytes + out_elems * (st.fused_pool ? 0.25 : 1.0) * (st.out_is_graph_output ? 4.0 : eb) +
                 (st.in1 >= 0 ? out_elems * eb : 0.0) + 4.0 * w.O;
            snprintf(buf, sizeof(buf), "%s c%d h%d w%d -> o%d k%dx%d s%d%s%s tile %dx%dx%d bn%d%s", st.direct == 4 ? "conv_stem_pool_nchw" : st.direct == 2 ? (st.fused_pool ? "conv_stem_pool" : "conv_stem_direct") : (st.direct == 3 ? "conv_rowstack" : (st.direct == 5 ? "conv_rowstack128" : (st.direct ? "conv_direct" : "conv_igemm"))), w.C, st.H, st.W, w.O, w.KH, w.KW,
                     p.stride, st.in1 >= 0 ? " +res" : "", st.relu ? " +relu" : "", p.BNI, p.BH, p.BW, st.cfg.bn,
                     st.cfg.ctas == 2 ? " pair" : (st.weight2 >= 0 ? " +1x1 second output" : (st.cfg.mt == 2 ? " x2 tiles" : "")));
            break;
        }
        case SKind::Gemm: {
            const PackedWeight& w = pl->weights[st.weight];
            fl = 2.0 * st.N * (double)w.O * w.C;
            by = (double)st.N * w.C * eb + (double)w.bytes + (double)st.N * w.O * (st.out_is_graph_output ? 4.0 : eb) + 4.0 * w.O;
            snprintf(buf, sizeof(buf), "dense_igemm m%d k%d -> n%d bn%d%s", st.N, w.C, w.O, st.cfg.bn, st.cfg.ctas == 2 ? " pair" : "");
            break;
        }
        case SKind::MaxPool:
            by = ((double)st.N * st.H * st.W * st.C + (double)st.N * st.OH * st.OW * st.C) * eb;
            snprintf(buf, sizeof(buf), "maxpool_nhwc c%d h%d w%d k%dx%d s%d", st.C, st.H, st.W, st.pool.pool_size[0], st.pool.pool_size[1], st.pool.strides[0]);
            break;
        case SKind::Gap:
            by = ((double)st.N * st.H * st.W * st.C + (double)st.N * st.C) * eb;
            snprintf(buf, sizeof(buf), "gap_nhwc c%d h%d w%d", st.C, st.H, st.W);
            break;
        case SKind::Eltwise:
            by = (double)st.numel * eb * (st.in1 >= 0 ? 3.0 : 2.0);
            snprintf(buf, sizeof(buf), "eltwise_nhwc n%lld", (long long)st.numel);
            break;
        case SKind::InputStem:
            by = (double)st.N * st.C * st.H * st.W * 4.0 + (double)st.N * st.Hp * st.Wp * 4 * eb;
            snprintf(buf, sizeof(buf), "stem_pack c%d h%d w%d -> %dx%dx4", st.C, st.H, st.W, st.Hp, st.Wp);
            break;
        case SKind::InputNHWC:
            by = (double)st.N * st.C * st.H * st.W * 4.0 + (double)st.N * st.H * st.W * st.cpad * eb;
            snprintf(buf, sizeof(buf), "input_nhwc c%d h%d w%d", st.C, st.H, st.W);
            break;
        case SKind::ToNCHW:
            by = (double)st.N * st.C * st.H * st.W * (4.0 + eb);
            snprintf(buf, sizeof(buf), "nhwc_to_nchw c%d h%d w%d", st.C, st.H, st.W);
            break;
    }
    if (name && name_size > 0) snprintf(name, (size_t)name_size, "%s", buf);
    if (flops) *flops = fl;
    if (bytes) *bytes = by;
    return KXC_B200_OK;
}

// ---- exact mode (KXC_B200_PREC_FP32) -------------------------------------------------------------
// Values keep the reference's own layout (NCHW / row-major fp32), so graph inputs, constants and the
// output are used in place and nn_flatten is always a view. Every kernel is one of the bit-exact ones
// (reference reduction order, separately rounded multiply and add); the fused epilogue performs the
// same three IEEE operations, in the same order, that the reference's three loop nests perform. A whole
// graph therefore reproduces the reference's CPU lowering bit for bit.
static int32_t finalize_exact(kxc_b200_plan* pl) {
    KXC_CUDA_TRY(cudaGetDevice(&pl->device));
    pl->dtype = kTcTF32;  // 4-byte elements; no rounding kernel is used in this mode
    for (size_t ni = 0; ni < pl->nodes.size(); ++ni) {
        Node& n = pl->nodes[ni];
        if (n.fused_into_other) continue;
        kxc_b200_plan::XStep xs;
        xs.op = n.op;
        xs.node = (int)ni;
        xs.in0 = n.in[0];
        int cur = n.out;
        if (n.op == "nn_conv2d") {
            xs.weight = n.in[1];
            xs.bias = n.in.size() == 3 ? n.in[2] : -1;
            int c = sole_consumer(pl, cur);
            if (c >= 0 && pl->nodes[c].op == "add" && !pl->nodes[c].fused_into_other) {
                Node& a = pl->nodes[c];
                const int other = a.in[0] == cur ? a.in[1] : a.in[0];
                Value* ov = pl->find(other);
                // the residual must already exist when this convolution runs
                if (other != cur && (ov->kind != VKind::Intermediate || ov->producer < (int)ni) && ov->shape == pl->find(cur)->shape) {
                    xs.in1 = other;
                    a.fused_into_other = true;
                    cur = a.out;
                    c = sole_consumer(pl, cur);
                }
            }
            if (c >= 0 && pl->nodes[c].op == "nn_relu" && !pl->nodes[c].fused_into_other) {
                xs.relu = true;
                pl->nodes[c].fused_into_other = true;
                cur = pl->nodes[c].out;
            }
        } else if (n.op == "add") {
            xs.in1 = n.in[1];
            const int c = sole_consumer(pl, cur);
            if (c >= 0 && pl->nodes[c].op == "nn_relu" && !pl->nodes[c].fused_into_other) {
                xs.relu = true;
                pl->nodes[c].fused_into_other = true;
                cur = pl->nodes[c].out;
            }
        } else if (n.op == "nn_dense" || n.op == "nn_gemm") {
            xs.weight = n.in[1];
            xs.bias = n.op == "nn_gemm" ? n.in[2] : -1;
        } else if (n.op == "nn_flatten") {
            if (n.out != pl->output_id) {
                pl->find(n.out)->alias_of = n.in[0];
                continue;
            }
        }
        xs.out = cur;
        pl->xsteps.push_back(xs);
    }
    // storage: one arena block per materialised intermediate (no reuse: sizes are modest in this mode)
    size_t top = 0;
    for (auto& xs : pl->xsteps) {
        if (pl->root_of(xs.out) == pl->root_of(pl->output_id)) continue;
        Value* v = pl->find(xs.out);
        v->offset = top;
        v->bytes = align_up(std::max<size_t>((size_t)numel_of(v->shape) * 4, 16), 1024);
        v->has_storage = true;
        top += v->bytes;
    }
    pl->arena_bytes = std::max<size_t>(top, 1024);
    KXC_CUDA_TRY(cudaMalloc(&pl->arena, pl->arena_bytes));
    pl->finalized = true;
    return KXC_B200_OK;
}

static int32_t run_exact(kxc_b200_plan* pl, void** packed_args, void* stream, cudaEvent_t* events) {
    if (!packed_args) return fail(KXC_B200_ERR_INVALID, "plan_run: null packed_args");
    KXC_TRY(require_device());
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t nargs = pl->inputs.size() + pl->constants.size();
    for (size_t i = 0; i <= nargs; ++i)
        if (!packed_args[i]) return fail(KXC_B200_ERR_INVALID, "plan_run: packed_args[%zu] is null", i);
    void* out_ptr = packed_args[nargs];
    auto ptr_of = [&](int id) -> void* {
        if (id < 0) return nullptr;
        const int root = pl->root_of(id);
        Value* v = pl->find(root);
        if (v->kind != VKind::Intermediate) return packed_args[v->arg_index];
        if (root == pl->root_of(pl->output_id)) return out_ptr;
        return static_cast<uint8_t*>(pl->arena) + v->offset;
    };
    size_t idx = 0;
    if (events) KXC_CUDA_TRY(cudaEventRecord(events[0], s));
    for (auto& xs : pl->xsteps) {
        if (idx > 0 && events) KXC_CUDA_TRY(cudaEventRecord(events[idx], s));
        LaunchRange range(pl, idx);
        ++idx;
        const Node& n = pl->nodes[xs.node];
        const auto& ish = pl->find(xs.in0)->shape;
        const auto& osh = pl->find(xs.out)->shape;
        if (xs.op == "nn_conv2d") {
            const auto& w = pl->find(xs.weight)->shape;
            ConvDims d{(int)ish[0], (int)ish[1], (int)ish[2], (int)ish[3], (int)w[0], (int)w[2], (int)w[3],
                       n.conv.strides[0], n.conv.strides[1], n.conv.padding[0], n.conv.padding[1], n.conv.dilation[0],
                       n.conv.dilation[1], (int)osh[2], (int)osh[3]};
            KXC_TRY(conv2d_fp32_exact(static_cast<const float*>(ptr_of(xs.in0)), static_cast<const float*>(ptr_of(xs.weight)),
                                      static_cast<const float*>(ptr_of(xs.bias)), static_cast<const float*>(ptr_of(xs.in1)),
                                      static_cast<float*>(ptr_of(xs.out)), d, xs.relu ? 1 : 0, s));
        } else if (xs.op == "add") {
            kxc_b200_add_desc d{};
            const auto& bsh = pl->find(xs.in1)->shape;
            d.rank_a = (int)ish.size(); d.rank_b = (int)bsh.size(); d.relu = xs.relu ? 1 : 0;
            for (size_t i = 0; i < ish.size(); ++i) d.shape_a[i] = ish[i];
            for (size_t i = 0; i < bsh.size(); ++i) d.shape_b[i] = bsh[i];
            void* a[3] = {ptr_of(xs.in0), ptr_of(xs.in1), ptr_of(xs.out)};
            KXC_TRY(kxc_b200_add(a, &d, stream));
        } else if (xs.op == "nn_relu") {
            void* a[2] = {ptr_of(xs.in0), ptr_of(xs.out)};
            KXC_TRY(kxc_b200_nn_relu(a, numel_of(osh), stream));
        } else if (xs.op == "nn_max_pool2d") {
            const auto& pa = n.pool;
            kxc_b200_pool2d_desc d{(int)ish[0], (int)ish[1], (int)ish[2], (int)ish[3], pa.pool_size[0], pa.pool_size[1], pa.strides[0],
                                   pa.strides[1], pa.padding[0], pa.padding[1], pa.padding[2], pa.padding[3], pa.ceil_mode};
            void* a[2] = {ptr_of(xs.in0), ptr_of(xs.out)};
            KXC_TRY(kxc_b200_nn_max_pool2d(a, &d, stream));
        } else if (xs.op == "nn_global_avg_pool2d") {
            void* a[2] = {ptr_of(xs.in0), ptr_of(xs.out)};
            KXC_TRY(kxc_b200_nn_global_avg_pool2d(a, (int)ish[0], (int)ish[1], (int)ish[2], (int)ish[3], stream));
        } else if (xs.op == "nn_flatten") {
            void* a[2] = {ptr_of(xs.in0), ptr_of(xs.out)};
            KXC_TRY(kxc_b200_nn_flatten(a, numel_of(osh), stream));
        } else if (xs.op == "nn_dense" || xs.op == "nn_gemm") {
            const bool gemm = xs.op == "nn_gemm";
            kxc_b200_gemm_desc g{(int)ish[0], (int)osh[1], (int)ish[1], gemm ? n.gemm.alpha : 1.0f, gemm ? n.gemm.beta : 1.0f, 0,
                                 gemm ? n.gemm.transB : 1, gemm ? 1 : 0, KXC_B200_PREC_FP32};
            KXC_TRY(gemm_fp32_exact(static_cast<const float*>(ptr_of(xs.in0)), static_cast<const float*>(ptr_of(xs.weight)),
                                    static_cast<const float*>(ptr_of(xs.bias)), static_cast<float*>(ptr_of(xs.out)), g, s));
        } else {
            return fail(KXC_B200_ERR_UNSUPPORTED, "plan: op '%s' is not supported", xs.op.c_str());
        }
    }
    if (events) KXC_CUDA_TRY(cudaEventRecord(events[idx], s));
    return KXC_B200_OK;
}
