// Reference-side binding of libkxc_b200.so (see kxc_b200_adapter.h). Compiled against the reference's public headers.
#include "kxc_b200_adapter.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <any>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <unordered_map>
#include <utility>

#include "base/device.h"
#include "base/device_api.h"
#include "relay/op_macros.h"
#include "relay/transforms/infer_type.h"

#include "kxc_b200.h"

namespace kxc {
namespace b200 {

namespace {

// `Device` names both a class and a factory function in the reference (include/base/device.h:31,62)
using DeviceT = class Device;

[[noreturn]] void Fail(const std::string& what) { throw std::runtime_error("kxc_b200 adapter: " + what); }

void CheckRc(int32_t rc, const std::string& what) {
    if (rc != 0) Fail(what + " returned error code " + std::to_string(rc) + ": " + kxc_b200_last_error());
}
void CheckCuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) Fail(std::string(what) + ": " + cudaGetErrorString(e));
}
void CheckNccl(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) Fail(std::string(what) + ": " + ncclGetErrorString(r));
}

std::vector<int64_t> ShapeOf(const Expr& e) {
    const auto* tt = e.checked_type().As<TensorTypeNode>();
    if (!tt) Fail("expression without a tensor type (run InferTypePass first)");
    std::vector<int64_t> s;
    for (size_t i = 0; i < tt->shape.size(); ++i) s.push_back(tt->shape[i]);
    return s;
}
std::string DTypeOf(const Expr& e) {
    const auto* tt = e.checked_type().As<TensorTypeNode>();
    return tt ? tt->dtype : std::string("float32");
}
int64_t Numel(const std::vector<int64_t>& s) {
    int64_t n = 1;
    for (auto d : s) n *= d;
    return n;
}
Expr SelfExpr(const CallNode& call) { return Expr(ObjectRef(const_cast<CallNode*>(&call))); }

size_t DTypeBytes(const std::string& dtype) {
    if (dtype == "float32" || dtype == "int32") return 4;
    if (dtype == "float64" || dtype == "int64") return 8;
    if (dtype == "int8" || dtype == "uint8" || dtype == "bool") return 1;
    Fail("unsupported dtype " + dtype);
}

// ---- per-operator hooks --------------------------------------------------------------------------------------------
using ConvFn = int32_t (*)(void**, const kxc_b200_conv2d_desc*, void*);
using ReluFn = int32_t (*)(void**, int64_t, void*);
using AddFn = int32_t (*)(void**, const kxc_b200_add_desc*, void*);
using PoolFn = int32_t (*)(void**, const kxc_b200_pool2d_desc*, void*);
using GapFn = int32_t (*)(void**, int32_t, int32_t, int32_t, int32_t, void*);
using GemmFn = int32_t (*)(void**, const kxc_b200_gemm_desc*, void*);
using SoftmaxFn = int32_t (*)(void**, const kxc_b200_softmax_desc*, void*);

int32_t AddNode(kxc_b200_plan* plan, const char* op, const void* attrs, const std::vector<int32_t>& in, int32_t out) {
    return kxc_b200_plan_add_kernel(plan, op, attrs, (int32_t)in.size(), in.data(), out);
}

kxc_b200_conv2d_attrs ConvAttrs(const CallNode& call) {
    const auto* a = call.attrs.As<relay::Conv2DAttrsNode>();
    if (!a) Fail("nn_conv2d without Conv2DAttrs");
    kxc_b200_conv2d_attrs c{};
    c.strides[0] = (int32_t)a->strides[0];
    c.strides[1] = (int32_t)a->strides[1];
    c.padding[0] = a->padding.size() > 0 ? (int32_t)a->padding[0] : 0;  // Conv2DCompute reads padding[0], padding[1] only
    c.padding[1] = a->padding.size() > 1 ? (int32_t)a->padding[1] : 0;
    c.dilation[0] = (int32_t)a->dilation[0];
    c.dilation[1] = (int32_t)a->dilation[1];
    c.groups = a->groups;
    return c;
}
kxc_b200_pool2d_attrs PoolAttrs(const CallNode& call) {
    const auto* a = call.attrs.As<relay::MaxPool2DAttrsNode>();
    if (!a) Fail("pooling call without MaxPool2DAttrs");
    kxc_b200_pool2d_attrs p{};
    p.pool_size[0] = (int32_t)a->pool_size[0];
    p.pool_size[1] = (int32_t)a->pool_size[1];
    p.strides[0] = (int32_t)a->strides[0];
    p.strides[1] = (int32_t)a->strides[1];
    for (int i = 0; i < 4; ++i) p.padding[i] = a->padding.size() == 4 ? (int32_t)a->padding[i] : (a->padding.size() == 2 ? (int32_t)a->padding[i & 1] : 0);
    p.ceil_mode = a->ceil_mode ? 1 : 0;
    return p;
}
kxc_b200_pool2d_desc PoolDesc(const CallNode& call) {
    const auto x = ShapeOf(call.args[0]);
    const auto a = PoolAttrs(call);
    return kxc_b200_pool2d_desc{(int32_t)x[0], (int32_t)x[1], (int32_t)x[2], (int32_t)x[3], a.pool_size[0], a.pool_size[1], a.strides[0],
                                a.strides[1], a.padding[0], a.padding[1], a.padding[2], a.padding[3], a.ceil_mode};
}
kxc_b200_gemm_attrs GemmAttrsOf(const CallNode& call) {
    kxc_b200_gemm_attrs g{1.0f, 1.0f, 0, 1};
    if (const auto* a = call.attrs.As<relay::GemmAttrsNode>()) g = kxc_b200_gemm_attrs{a->alpha, a->beta, a->transA, a->transB};
    return g;
}

std::unordered_map<std::string, FB200Launch> BuildHooks() {
    std::unordered_map<std::string, FB200Launch> h;
    h["nn_conv2d"] = FB200Launch{
        "kxc_b200_nn_conv2d",
        [](kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& in, int32_t out) {
            const auto a = ConvAttrs(call);
            return AddNode(plan, "nn_conv2d", &a, in, out);
        },
        [](void* entry, const CallNode& call, void** args, int precision, void* stream) {
            const auto a = ConvAttrs(call);
            const auto x = ShapeOf(call.args[0]), w = ShapeOf(call.args[1]);
            kxc_b200_conv2d_desc d{(int32_t)x[0], (int32_t)x[1], (int32_t)x[2], (int32_t)x[3], (int32_t)w[0], (int32_t)w[2], (int32_t)w[3],
                                   a.strides[0], a.strides[1], a.padding[0], a.padding[1], a.dilation[0], a.dilation[1],
                                   call.args.size() == 3 ? KXC_B200_BIAS : 0, precision};
            return reinterpret_cast<ConvFn>(entry)(args, &d, stream);
        }};
    h["nn_relu"] = FB200Launch{
        "kxc_b200_nn_relu",
        [](kxc_b200_plan* plan, const CallNode&, const std::vector<int32_t>& in, int32_t out) { return AddNode(plan, "nn_relu", nullptr, in, out); },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            return reinterpret_cast<ReluFn>(entry)(args, Numel(ShapeOf(call.args[0])), stream);
        }};
    h["add"] = FB200Launch{
        "kxc_b200_add",
        [](kxc_b200_plan* plan, const CallNode&, const std::vector<int32_t>& in, int32_t out) { return AddNode(plan, "add", nullptr, in, out); },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            const auto a = ShapeOf(call.args[0]), b = ShapeOf(call.args[1]);
            kxc_b200_add_desc d{};
            d.rank_a = (int32_t)a.size();
            d.rank_b = (int32_t)b.size();
            for (size_t i = 0; i < a.size() && i < 6; ++i) d.shape_a[i] = a[i];
            for (size_t i = 0; i < b.size() && i < 6; ++i) d.shape_b[i] = b[i];
            return reinterpret_cast<AddFn>(entry)(args, &d, stream);
        }};
    h["nn_max_pool2d"] = FB200Launch{
        "kxc_b200_nn_max_pool2d",
        [](kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& in, int32_t out) {
            const auto a = PoolAttrs(call);
            return AddNode(plan, "nn_max_pool2d", &a, in, out);
        },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            const auto d = PoolDesc(call);
            return reinterpret_cast<PoolFn>(entry)(args, &d, stream);
        }};
    h["nn_avg_pool2d"] = FB200Launch{
        "kxc_b200_nn_avg_pool2d",
        [](kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& in, int32_t out) {
            const auto a = PoolAttrs(call);
            return AddNode(plan, "nn_avg_pool2d", &a, in, out);  // refused by plan_finalize: per-node execution only
        },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            const auto d = PoolDesc(call);
            return reinterpret_cast<PoolFn>(entry)(args, &d, stream);
        }};
    h["nn_global_avg_pool2d"] = FB200Launch{
        "kxc_b200_nn_global_avg_pool2d",
        [](kxc_b200_plan* plan, const CallNode&, const std::vector<int32_t>& in, int32_t out) {
            return AddNode(plan, "nn_global_avg_pool2d", nullptr, in, out);
        },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            const auto x = ShapeOf(call.args[0]);
            return reinterpret_cast<GapFn>(entry)(args, (int32_t)x[0], (int32_t)x[1], (int32_t)x[2], (int32_t)x[3], stream);
        }};
    h["nn_flatten"] = FB200Launch{
        "kxc_b200_nn_flatten",
        [](kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& in, int32_t out) {
            const auto* a = call.attrs.As<relay::FlattenAttrsNode>();
            if (a && a->axis != 1) return (int32_t)KXC_B200_ERR_UNSUPPORTED;  // plans flatten at axis 1 only
            return AddNode(plan, "nn_flatten", nullptr, in, out);
        },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            return reinterpret_cast<ReluFn>(entry)(args, Numel(ShapeOf(call.args[0])), stream);  // same signature: (args, numel, stream)
        }};
    auto gemm_launch = [](bool has_c) {
        return [has_c](void* entry, const CallNode& call, void** args, int precision, void* stream) {
            const auto a = ShapeOf(call.args[0]), b = ShapeOf(call.args[1]);
            const auto g = has_c ? GemmAttrsOf(call) : kxc_b200_gemm_attrs{1.0f, 1.0f, 0, 1};
            const int64_t n = g.transB ? b[0] : b[1];
            kxc_b200_gemm_desc d{(int32_t)a[0], (int32_t)n, (int32_t)a[1], g.alpha, g.beta, g.transA, g.transB, has_c ? 1 : 0, precision};
            return reinterpret_cast<GemmFn>(entry)(args, &d, stream);
        };
    };
    h["nn_dense"] = FB200Launch{
        "kxc_b200_nn_gemm",
        [](kxc_b200_plan* plan, const CallNode&, const std::vector<int32_t>& in, int32_t out) { return AddNode(plan, "nn_dense", nullptr, in, out); },
        gemm_launch(false)};
    h["nn_gemm"] = FB200Launch{
        "kxc_b200_nn_gemm",
        [](kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& in, int32_t out) {
            const auto g = GemmAttrsOf(call);
            return AddNode(plan, "nn_gemm", &g, in, out);
        },
        gemm_launch(true)};
    h["softmax"] = FB200Launch{
        "kxc_b200_softmax",
        [](kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& in, int32_t out) {
            const auto* a = call.attrs.As<relay::SoftmaxAttrsNode>();
            kxc_b200_softmax_attrs s{a ? a->axis : -1};
            return AddNode(plan, "softmax", &s, in, out);
        },
        [](void* entry, const CallNode& call, void** args, int, void* stream) {
            const auto x = ShapeOf(call.args[0]);
            const auto* a = call.attrs.As<relay::SoftmaxAttrsNode>();
            kxc_b200_softmax_desc d{};
            d.rank = (int32_t)x.size();
            for (size_t i = 0; i < x.size() && i < 6; ++i) d.shape[i] = x[i];
            d.axis = a ? a->axis : -1;
            return reinterpret_cast<SoftmaxFn>(entry)(args, &d, stream);
        }};
    return h;
}

const char* kAttrName = "FB200Launch";

std::string OpNameOf(const CallNode& call) {
    const auto* op = call.op.As<relay::OpNode>();
    if (!op) Fail("call of something that is not a registered operator");
    return op->name;
}

// Value numbering of RelayToExecPlanBuilder (src/relay/transforms/multi_device.cc:244-325): parameters first, then a
// memoised walk of the body in which a constant or a call gets the next id when it is first reached (a call after its
// arguments). The same walk gives the lowering order of the constants (src/relay/backend/lower.cc:534-565).
struct Numbering {
    std::unordered_map<const Object*, int> id_of;
    std::vector<const ConstantNode*> constants;
    std::vector<const CallNode*> calls;  // post order
    int next = 0;
    explicit Numbering(const Function& func) {
        for (const auto& p : func->params) id_of[p.get()] = next++;
        Visit(func->body);
    }
    int Visit(const Expr& e) {
        if (!e.defined()) Fail("undefined expression in the function body");
        auto it = id_of.find(e.get());
        if (it != id_of.end()) return it->second;
        if (const auto* c = e.As<ConstantNode>()) {
            constants.push_back(c);
            return id_of[e.get()] = next++;
        }
        if (const auto* call = e.As<CallNode>()) {
            for (const auto& a : call->args) Visit(a);
            calls.push_back(call);
            return id_of[e.get()] = next++;
        }
        if (e.As<VarNode>()) return id_of[e.get()] = next++;  // a free variable: numbered like the builder does
        Fail("only Var / Constant / Call expressions are supported");
    }
};

// ---- trampolines: real one-argument entry points for CompiledKernelNode::func_ptr --------------------------------------
struct Slot {
    kxc_b200_plan* plan = nullptr;
    void* stream = nullptr;
    bool used = false;
};
constexpr int kSlots = 64;
Slot g_slots[kSlots];
std::mutex g_slot_mutex;

template <int I>
int32_t Trampoline(void** packed_args) {
    return kxc_b200_plan_run(g_slots[I].plan, packed_args, g_slots[I].stream);
}
using EntryFn = int32_t (*)(void**);
template <int... I>
constexpr std::array<EntryFn, sizeof...(I)> MakeTrampolines(std::integer_sequence<int, I...>) {
    return {{&Trampoline<I>...}};
}
const std::array<EntryFn, kSlots> kTrampolines = MakeTrampolines(std::make_integer_sequence<int, kSlots>{});

void* LibraryHandle() {
    // The library is already mapped (this file links against it); a second dlopen hands out a counted handle that
    // CompiledKernelNode's destructor may dlclose (src/codegen/compiled_kernel.cc:21-27).
    void* h = dlopen("libkxc_b200.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) Fail(std::string("dlopen(libkxc_b200.so): ") + dlerror());
    return h;
}

Array<int> EffectiveWorkerSet(const Array<int>& worker_set, int fallback_worker) {
    if (!worker_set.empty()) return worker_set;
    return {fallback_worker >= 0 ? fallback_worker : 0};
}

int ResolveWorkerForValue(const ExecutionPlan& plan, int value_id) {
    if (!plan.defined() || !plan->value_virtual_devices.count(value_id)) return 0;
    const VirtualDevice& vd = plan->value_virtual_devices.at(value_id);
    if (!vd.defined()) return 0;
    if (vd->device_obj.defined()) {
        const auto* dev = static_cast<const class Device*>(vd->device_obj.get());
        if (dev) return dev->device_id();
    }
    return 0;
}

ncclDataType_t NcclType(const std::string& dtype) {
    if (dtype == "float32") return ncclFloat32;
    if (dtype == "float64") return ncclFloat64;
    if (dtype == "int32") return ncclInt32;
    if (dtype == "int64") return ncclInt64;
    if (dtype == "int8") return ncclInt8;
    if (dtype == "uint8" || dtype == "bool") return ncclUint8;
    Fail("no NCCL type for dtype " + dtype);
}

}  // namespace

void RegisterB200Ops() {
    static std::once_flag once;
    std::call_once(once, [] {
        for (auto& kv : BuildHooks()) relay::OpRegEntry(relay::Op::Get(kv.first)).set_attr<FB200Launch>(kAttrName, kv.second);
    });
}

const FB200Launch* GetB200Launch(const std::string& op_name) {
    RegisterB200Ops();
    const relay::Op& op = relay::Op::Get(op_name);
    auto it = op->attrs.find(kAttrName);
    if (it == op->attrs.end()) return nullptr;
    return std::any_cast<FB200Launch>(&it->second);
}

std::vector<runtime::NDArray> ConstantsInLoweringOrder(const Function& func) {
    Numbering num(func);
    std::vector<runtime::NDArray> out;
    for (const auto* c : num.constants) out.push_back(c->data);
    return out;
}

codegen::CompiledKernel CompileForB200(const Function& func_in, int precision, void* stream) {
    RegisterB200Ops();
    Function func = relay::InferTypePass(func_in);
    Numbering num(func);
    kxc_b200_plan* plan = nullptr;
    CheckRc(kxc_b200_plan_create(precision, &plan), "kxc_b200_plan_create");
    try {
        for (const auto& p : func->params) {
            const auto* tt = p->type_annotation.As<TensorTypeNode>();
            if (!tt) Fail("function parameter without a tensor type");
            std::vector<int64_t> s;
            for (size_t i = 0; i < tt->shape.size(); ++i) s.push_back(tt->shape[i]);
            CheckRc(kxc_b200_plan_add_input(plan, num.id_of.at(p.get()), (int32_t)s.size(), s.data()), "kxc_b200_plan_add_input");
        }
        for (const auto* c : num.constants) {
            std::vector<int64_t> s(c->data->shape.begin(), c->data->shape.end());
            CheckRc(kxc_b200_plan_add_constant(plan, num.id_of.at(c), (int32_t)s.size(), s.data()), "kxc_b200_plan_add_constant");
        }
        for (const auto* call : num.calls) {
            const std::string name = OpNameOf(*call);
            const FB200Launch* hooks = GetB200Launch(name);
            if (!hooks) Fail("operator " + name + " has no FB200Launch attribute");
            std::vector<int32_t> in;
            for (const auto& a : call->args) in.push_back(num.id_of.at(a.get()));
            CheckRc(hooks->add_to_plan(plan, *call, in, num.id_of.at(call)), "FB200Launch(" + name + ")");
        }
        CheckRc(kxc_b200_plan_set_output(plan, num.id_of.at(func->body.get())), "kxc_b200_plan_set_output");
        CheckRc(kxc_b200_plan_finalize(plan), "kxc_b200_plan_finalize");
    } catch (...) {
        kxc_b200_plan_destroy(plan);
        throw;
    }
    int slot = -1;
    {
        std::lock_guard<std::mutex> lock(g_slot_mutex);
        for (int i = 0; i < kSlots && slot < 0; ++i)
            if (!g_slots[i].used) slot = i;
        if (slot < 0) {
            kxc_b200_plan_destroy(plan);
            Fail("all " + std::to_string(kSlots) + " kernel slots are in use");
        }
        g_slots[slot] = Slot{plan, stream, true};
    }
    auto* node = new codegen::CompiledKernelNode();
    node->kernel_name = "kxc_kernel_main";
    node->backend = codegen::CodeGenBackend::kCUDA;
    node->func_ptr = reinterpret_cast<void*>(kTrampolines[slot]);
    node->so_path = "libkxc_b200.so";
    node->lib_handle = LibraryHandle();
    return codegen::CompiledKernel(static_cast<const Object*>(node));
}

std::map<int, const CallNode*> BindKernelSymbols(const ExecutionPlan& plan, const Function& typed_func) {
    RegisterB200Ops();
    Numbering num(typed_func);
    std::unordered_map<int, const CallNode*> call_of;
    for (const auto* call : num.calls) call_of[num.id_of.at(call)] = call;
    std::map<int, const CallNode*> side;
    for (const auto& ref : plan->nodes) {
        if (!ref.defined() || ref.get()->GetTypeId() != KernelExecNode::_type_index) continue;
        auto* k = const_cast<KernelExecNode*>(static_cast<const KernelExecNode*>(ref.get()));
        if (k->output_values.empty()) continue;
        const int out = k->output_values[0];
        auto it = call_of.find(out);
        if (it == call_of.end()) Fail("plan value " + std::to_string(out) + " has no Relay call");
        const CallNode* call = it->second;
        if (OpNameOf(*call) != k->op_name) Fail("plan node " + k->op_name + " does not match the Relay call " + OpNameOf(*call));
        if (call->args.size() != k->input_values.size()) Fail("plan node " + k->op_name + ": argument count differs from the Relay call");
        for (size_t i = 0; i < call->args.size(); ++i)
            if (num.id_of.at(call->args[i].get()) != k->input_values[i]) Fail("plan node " + k->op_name + ": value ids differ from the Relay call");
        const FB200Launch* hooks = GetB200Launch(k->op_name);
        if (!hooks) Fail("operator " + k->op_name + " has no FB200Launch attribute");
        k->kernel_symbol = hooks->kernel_symbol;
        side[out] = call;
    }
    return side;
}

// ---- device-resident values ------------------------------------------------------------------------------------------
class DeviceValues {
  public:
    struct Buf {
        void* ptr = nullptr;
        size_t bytes = 0;
        std::vector<int64_t> shape;
        std::string dtype;
        int device = 0;
    };
    explicit DeviceValues(std::vector<int> devices) : devices_(std::move(devices)) {}
    ~DeviceValues() {
        for (auto& kv : bufs_)
            if (kv.second.ptr) GetDeviceAPI(DeviceTypeCode::kGPU)->FreeDataSpace(DeviceT(DeviceTypeCode::kGPU, kv.second.device), kv.second.ptr);
    }
    Buf* Find(const disco::DRef& ref, int worker) {
        auto it = bufs_.find({ref.reg_id(), worker});
        return it == bufs_.end() ? nullptr : &it->second;
    }
    // (re)allocates the value on the worker's GPU through the reference's own DeviceAPI
    Buf& Alloc(const disco::DRef& ref, int worker, const std::vector<int64_t>& shape, const std::string& dtype) {
        Buf& b = bufs_[{ref.reg_id(), worker}];
        const size_t bytes = (size_t)Numel(shape) * DTypeBytes(dtype);
        DeviceAPI* api = GetDeviceAPI(DeviceTypeCode::kGPU);
        const DeviceT dev(DeviceTypeCode::kGPU, devices_.at(worker));
        if (b.ptr && b.bytes < bytes) {
            api->FreeDataSpace(dev, b.ptr);
            b.ptr = nullptr;
        }
        if (!b.ptr) {
            b.ptr = api->AllocDataSpace(dev, bytes > 0 ? bytes : 1, 256);
            b.bytes = bytes;
        }
        b.shape = shape;
        b.dtype = dtype;
        b.device = devices_.at(worker);
        return b;
    }
    // the device copy of a value; a host NDArray held in the session's register is uploaded on first use
    Buf& Ensure(const disco::DiscoSession& session, const disco::DRef& ref, int worker) {
        if (Buf* b = Find(ref, worker)) return *b;
        runtime::NDArray host = session.Get(worker, ref);
        if (!host.defined()) Fail("value in register " + std::to_string(ref.reg_id()) + " is undefined on worker " + std::to_string(worker));
        std::vector<int64_t> shape(host->shape.begin(), host->shape.end());
        const std::string dtype = DTypeString(host->dl_tensor.dtype);
        Buf& b = Alloc(ref, worker, shape, dtype);
        GetDeviceAPI(DeviceTypeCode::kGPU)->CopyDataFromTo(DeviceT(DeviceTypeCode::kCPU, 0), host->dl_tensor.data, DeviceT(DeviceTypeCode::kGPU, b.device),
                                                           b.ptr, host.NBytes());
        return b;
    }
    // writes the device value back into the session's register (what CpuCCLBackend leaves there)
    void Download(const disco::DiscoSession& session, const disco::DRef& ref, int worker) {
        Buf* b = Find(ref, worker);
        if (!b) Fail("no device value to download");
        Array<int64_t> shape;
        for (auto d : b->shape) shape.push_back(d);
        runtime::NDArray host(shape, b->dtype);
        GetDeviceAPI(DeviceTypeCode::kGPU)->CopyDataFromTo(DeviceT(DeviceTypeCode::kGPU, b->device), b->ptr, DeviceT(DeviceTypeCode::kCPU, 0),
                                                           host->dl_tensor.data, host.NBytes());
        session.Set(worker, ref, host);
    }

  private:
    static std::string DTypeString(const DLDataType& t) {
        if (t.code == kDLFloat && t.bits == 32) return "float32";
        if (t.code == kDLFloat && t.bits == 64) return "float64";
        if (t.code == kDLInt && t.bits == 32) return "int32";
        if (t.code == kDLInt && t.bits == 64) return "int64";
        if (t.code == kDLInt && t.bits == 8) return "int8";
        if (t.code == kDLUint && t.bits == 8) return "uint8";
        Fail("unsupported NDArray dtype");
    }
    std::vector<int> devices_;
    std::map<std::pair<int, int>, Buf> bufs_;
};

// ---- NCCL backend ----------------------------------------------------------------------------------------------------------
struct NcclCCLBackend::Impl {
    std::vector<int> devices;
    std::vector<ncclComm_t> comms;
    std::vector<cudaStream_t> streams;
    DeviceValues values;
    explicit Impl(std::vector<int> d) : devices(d), values(d) {}
    int n() const { return (int)devices.size(); }
    void SyncAll() {
        for (int w = 0; w < n(); ++w) {
            CheckCuda(cudaSetDevice(devices[w]), "cudaSetDevice");
            CheckCuda(cudaStreamSynchronize(streams[w]), "cudaStreamSynchronize");
        }
    }
};

NcclCCLBackend::NcclCCLBackend(std::vector<int> devices) : impl_(new Impl(std::move(devices))) {
    const int n = impl_->n();
    if (n <= 0) Fail("NcclCCLBackend needs at least one device");
    impl_->comms.resize(n);
    impl_->streams.resize(n);
    CheckNccl(ncclCommInitAll(impl_->comms.data(), n, impl_->devices.data()), "ncclCommInitAll");
    for (int w = 0; w < n; ++w) {
        CheckCuda(cudaSetDevice(impl_->devices[w]), "cudaSetDevice");
        CheckCuda(cudaStreamCreateWithFlags(&impl_->streams[w], cudaStreamNonBlocking), "cudaStreamCreate");
    }
}

NcclCCLBackend::~NcclCCLBackend() {
    for (int w = 0; w < impl_->n(); ++w) {
        cudaSetDevice(impl_->devices[w]);
        cudaStreamSynchronize(impl_->streams[w]);
        cudaStreamDestroy(impl_->streams[w]);
        ncclCommDestroy(impl_->comms[w]);
    }
}

DeviceValues& NcclCCLBackend::values() { return impl_->values; }
int NcclCCLBackend::device_of(int worker) const { return impl_->devices.at(worker); }
void* NcclCCLBackend::stream_of(int worker) const { return impl_->streams.at(worker); }

void NcclCCLBackend::Copy(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, int src_worker, int dst_worker) {
    auto& s = impl_->values.Ensure(session, src, src_worker);
    auto& d = impl_->values.Alloc(dst, dst_worker, s.shape, s.dtype);
    if (src_worker == dst_worker) {
        CheckCuda(cudaSetDevice(s.device), "cudaSetDevice");
        CheckCuda(cudaMemcpyAsync(d.ptr, s.ptr, s.bytes, cudaMemcpyDeviceToDevice, impl_->streams[src_worker]), "cudaMemcpyAsync");
    } else {
        const size_t count = (size_t)Numel(s.shape);
        CheckNccl(ncclGroupStart(), "ncclGroupStart");
        CheckNccl(ncclSend(s.ptr, count, NcclType(s.dtype), dst_worker, impl_->comms[src_worker], impl_->streams[src_worker]), "ncclSend");
        CheckNccl(ncclRecv(d.ptr, count, NcclType(s.dtype), src_worker, impl_->comms[dst_worker], impl_->streams[dst_worker]), "ncclRecv");
        CheckNccl(ncclGroupEnd(), "ncclGroupEnd");
    }
    impl_->SyncAll();
    impl_->values.Download(session, dst, dst_worker);
}

void NcclCCLBackend::AllReduce(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, const std::string& reduce_kind,
                               bool in_group) {
    (void)in_group;  // CpuCCLBackend::AllReduce sums over all workers whatever the flag says (ccl_cpu.cc:187-211)
    if (reduce_kind != "sum") Fail("NcclCCLBackend supports only sum allreduce, like CpuCCLBackend");
    const int n = impl_->n();
    std::vector<DeviceValues::Buf*> s(n), d(n);
    for (int w = 0; w < n; ++w) s[w] = &impl_->values.Ensure(session, src, w);
    for (int w = 0; w < n; ++w) d[w] = &impl_->values.Alloc(dst, w, s[w]->shape, s[w]->dtype);
    CheckNccl(ncclGroupStart(), "ncclGroupStart");
    for (int w = 0; w < n; ++w)
        CheckNccl(ncclAllReduce(s[w]->ptr, d[w]->ptr, (size_t)Numel(s[w]->shape), NcclType(s[w]->dtype), ncclSum, impl_->comms[w], impl_->streams[w]),
                  "ncclAllReduce");
    CheckNccl(ncclGroupEnd(), "ncclGroupEnd");
    impl_->SyncAll();
    for (int w = 0; w < n; ++w) impl_->values.Download(session, dst, w);
}

void NcclCCLBackend::BroadcastFromWorker0(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, bool in_group) {
    const int n = impl_->n();
    const int groups = in_group ? session.num_groups() : 1;
    const int per = n / groups;
    CheckNccl(ncclGroupStart(), "ncclGroupStart");
    for (int g = 0; g < groups; ++g) {
        const int root = g * per;
        // a group whose own root holds nothing broadcasts worker 0's value, as CpuCCLBackend does (ccl_cpu.cc:213-236)
        const int from = (impl_->values.Find(src, root) || session.Get(root, src).defined()) ? root : 0;
        auto& s = impl_->values.Ensure(session, src, from);
        for (int i = 0; i < per; ++i) {
            const int w = root + i;
            auto& d = impl_->values.Alloc(dst, w, s.shape, s.dtype);
            const size_t count = (size_t)Numel(s.shape);
            if (w == from) {
                CheckCuda(cudaSetDevice(s.device), "cudaSetDevice");
                CheckCuda(cudaMemcpyAsync(d.ptr, s.ptr, s.bytes, cudaMemcpyDeviceToDevice, impl_->streams[w]), "cudaMemcpyAsync");
            } else {
                CheckNccl(ncclSend(s.ptr, count, NcclType(s.dtype), w, impl_->comms[from], impl_->streams[from]), "ncclSend");
                CheckNccl(ncclRecv(d.ptr, count, NcclType(s.dtype), from, impl_->comms[w], impl_->streams[w]), "ncclRecv");
            }
        }
    }
    CheckNccl(ncclGroupEnd(), "ncclGroupEnd");
    impl_->SyncAll();
    for (int w = 0; w < n; ++w) impl_->values.Download(session, dst, w);
}

void NcclCCLBackend::ScatterFromWorker0(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, bool in_group) {
    const int n = impl_->n();
    const int groups = in_group ? session.num_groups() : 1;
    const int per = n / groups;
    CheckNccl(ncclGroupStart(), "ncclGroupStart");
    for (int g = 0; g < groups; ++g) {
        const int root = g * per;
        const int from = (impl_->values.Find(src, root) || session.Get(root, src).defined()) ? root : 0;
        auto& s = impl_->values.Ensure(session, src, from);
        if (s.shape.empty() || s.shape[0] % per != 0) Fail("Scatter expects first dimension divisible by receiver count");
        std::vector<int64_t> shard = s.shape;
        shard[0] /= per;
        const size_t count = (size_t)Numel(shard), bytes = count * DTypeBytes(s.dtype);
        for (int i = 0; i < per; ++i) {
            const int w = root + i;
            auto& d = impl_->values.Alloc(dst, w, shard, s.dtype);
            const char* piece = static_cast<const char*>(s.ptr) + (size_t)i * bytes;
            if (w == from) {
                CheckCuda(cudaSetDevice(s.device), "cudaSetDevice");
                CheckCuda(cudaMemcpyAsync(d.ptr, piece, bytes, cudaMemcpyDeviceToDevice, impl_->streams[w]), "cudaMemcpyAsync");
            } else {
                CheckNccl(ncclSend(piece, count, NcclType(s.dtype), w, impl_->comms[from], impl_->streams[from]), "ncclSend");
                CheckNccl(ncclRecv(d.ptr, count, NcclType(s.dtype), from, impl_->comms[w], impl_->streams[w]), "ncclRecv");
            }
        }
    }
    CheckNccl(ncclGroupEnd(), "ncclGroupEnd");
    impl_->SyncAll();
    for (int w = 0; w < n; ++w) impl_->values.Download(session, dst, w);
}

void NcclCCLBackend::GatherToWorker0(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, bool in_group) {
    // shards concatenated on dim 0 in worker order into the group's first worker: ConcatFirstDim (ccl_cpu.cc:134-174, :274-294)
    const int n = impl_->n();
    const int groups = in_group ? session.num_groups() : 1;
    const int per = n / groups;
    std::vector<int> roots;
    CheckNccl(ncclGroupStart(), "ncclGroupStart");
    for (int g = 0; g < groups; ++g) {
        const int root = g * per;
        roots.push_back(root);
        std::vector<DeviceValues::Buf*> shards;
        std::vector<int64_t> full;
        for (int i = 0; i < per; ++i) {
            auto& s = impl_->values.Ensure(session, src, root + i);
            if (i == 0) full = s.shape;
            else {
                if (s.shape.size() != full.size() || s.dtype != shards[0]->dtype) Fail("Gather expects shards of one rank and dtype");
                full[0] += s.shape[0];
            }
            shards.push_back(&s);
        }
        auto& d = impl_->values.Alloc(dst, root, full, shards[0]->dtype);
        size_t offset = 0;
        for (int i = 0; i < per; ++i) {
            const int w = root + i;
            const size_t count = (size_t)Numel(shards[i]->shape), bytes = count * DTypeBytes(shards[i]->dtype);
            char* where = static_cast<char*>(d.ptr) + offset;
            if (w == root) {
                CheckCuda(cudaSetDevice(d.device), "cudaSetDevice");
                CheckCuda(cudaMemcpyAsync(where, shards[i]->ptr, bytes, cudaMemcpyDeviceToDevice, impl_->streams[root]), "cudaMemcpyAsync");
            } else {
                CheckNccl(ncclSend(shards[i]->ptr, count, NcclType(shards[i]->dtype), root, impl_->comms[w], impl_->streams[w]), "ncclSend");
                CheckNccl(ncclRecv(where, count, NcclType(shards[i]->dtype), w, impl_->comms[root], impl_->streams[root]), "ncclRecv");
            }
            offset += bytes;
        }
    }
    CheckNccl(ncclGroupEnd(), "ncclGroupEnd");
    impl_->SyncAll();
    for (int root : roots) impl_->values.Download(session, dst, root);
}

void NcclCCLBackend::SendToWorker(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, int receiver_worker) {
    Copy(session, src, dst, 0, receiver_worker);
}

void NcclCCLBackend::RecvFromWorker(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, int sender_worker) {
    Copy(session, src, dst, sender_worker, 0);
}

void NcclCCLBackend::SyncWorker(const disco::DiscoSession& session, int worker_id) {
    CheckCuda(cudaSetDevice(impl_->devices.at(worker_id)), "cudaSetDevice");
    CheckCuda(cudaStreamSynchronize(impl_->streams.at(worker_id)), "cudaStreamSynchronize");
    session.SyncWorker(worker_id);
}

// ---- plan executor ------------------------------------------------------------------------------------------------------------
B200PlanExecutor::B200PlanExecutor(disco::DiscoSession session, std::shared_ptr<NcclCCLBackend> backend, int precision)
    : session_(std::move(session)), backend_(std::move(backend)), precision_(precision) {
    if (!session_.defined()) Fail("B200PlanExecutor requires a defined DiscoSession");
    if (!backend_) Fail("B200PlanExecutor requires a CCL backend");
    RegisterB200Ops();
}

void B200PlanExecutor::ExecuteKernel(const ExecutionPlan& plan, const KernelExecNode* kernel, const CallNode* call) {
    if (!kernel || kernel->output_values.empty()) return;
    if (!call) Fail("kernel node " + kernel->op_name + " has no attribute record (run BindKernelSymbols)");
    if (kernel->kernel_symbol.empty()) Fail("kernel node " + kernel->op_name + " has no kernel_symbol bound");
    const FB200Launch* hooks = GetB200Launch(kernel->op_name);
    if (!hooks) Fail("operator " + kernel->op_name + " has no FB200Launch attribute");
    void* entry = dlsym(RTLD_DEFAULT, kernel->kernel_symbol.c_str());
    if (!entry) Fail("symbol " + kernel->kernel_symbol + " not found: " + dlerror());
    for (int id : kernel->input_values)
        if (!values_.count(id)) Fail("Kernel input value is not available");
    const int out_id = kernel->output_values[0];
    disco::DRef out = values_.count(out_id) ? values_.at(out_id) : session_.NewDRef();
    const std::vector<int64_t> out_shape = ShapeOf(SelfExpr(*call));
    const std::string out_dtype = DTypeOf(SelfExpr(*call));
    for (int worker : EffectiveWorkerSet(kernel->worker_set, ResolveWorkerForValue(plan, kernel->input_values.empty() ? out_id : kernel->input_values[0]))) {
        CheckCuda(cudaSetDevice(backend_->device_of(worker)), "cudaSetDevice");
        std::vector<void*> args;
        for (int id : kernel->input_values) args.push_back(backend_->values().Ensure(session_, values_.at(id), worker).ptr);
        args.push_back(backend_->values().Alloc(out, worker, out_shape, out_dtype).ptr);
        const int32_t rc = hooks->launch(entry, *call, args.data(), precision_, backend_->stream_of(worker));
        if (rc != 0)  // the message CompiledKernel::operator() gives (src/codegen/compiled_kernel.cc:50-54)
            throw std::runtime_error("Kernel " + kernel->kernel_symbol + " returned error code " + std::to_string(rc) + ": " + kxc_b200_last_error());
    }
    for (int id : kernel->output_values) values_.Set(id, out);
}

void B200PlanExecutor::ExecuteComm(const ExecutionPlan& plan, const CommExecNode* comm) {
    if (!comm || comm->output_values.empty()) return;
    if (comm->input_values.empty()) Fail("Communication node requires at least one input");
    const int input_id = comm->input_values[0];
    if (!values_.count(input_id)) Fail("Communication input value is missing");
    disco::DRef src = values_.at(input_id);
    const int output_id = comm->output_values[0];
    disco::DRef dst = values_.count(output_id) ? values_.at(output_id) : session_.NewDRef();
    bool in_group = true;
    int root_worker = 0;
    std::string reduce_kind = "sum";
    if (const auto* a = comm->attrs.defined() ? comm->attrs.As<relay::CollectiveAttrsNode>() : nullptr) {
        in_group = a->in_group;
        root_worker = a->root_worker;
        reduce_kind = a->reduce_kind;
    }
    for (int w = 0; w < session_.num_workers(); ++w) backend_->SyncWorker(session_, w);  // kernels that produced the operands have finished
    if (comm->op_name == "device.copy") backend_->Copy(session_, src, dst, ResolveWorkerForValue(plan, input_id), ResolveWorkerForValue(plan, output_id));
    else if (comm->op_name == "device.allreduce") backend_->AllReduce(session_, src, dst, reduce_kind, in_group);
    else if (comm->op_name == "device.broadcast_from_worker0") backend_->BroadcastFromWorker0(session_, src, dst, in_group);
    else if (comm->op_name == "device.scatter_from_worker0") backend_->ScatterFromWorker0(session_, src, dst, in_group);
    else if (comm->op_name == "device.gather_to_worker0") backend_->GatherToWorker0(session_, src, dst, in_group);
    else if (comm->op_name == "device.send_to_worker") backend_->SendToWorker(session_, src, dst, root_worker);
    else if (comm->op_name == "device.recv_from_worker") backend_->RecvFromWorker(session_, src, dst, root_worker);
    else Fail("Unsupported communication op in executor: " + comm->op_name);
    for (int id : comm->output_values) values_.Set(id, dst);
}

disco::DRef B200PlanExecutor::ExecuteForOutput(const ExecutionPlan& plan, const std::map<int, const CallNode*>& attrs_of,
                                               const Map<int, disco::DRef>& initial_values) {
    if (!plan.defined()) Fail("Execute requires a defined ExecutionPlan");
    values_ = initial_values;
    for (size_t i = 0; i < plan->nodes.size(); ++i) {
        const auto& ref = plan->nodes[i];
        if (!ref.defined()) continue;
        if (ref.get()->GetTypeId() == KernelExecNode::_type_index) {
            const auto* k = static_cast<const KernelExecNode*>(ref.get());
            auto it = k->output_values.empty() ? attrs_of.end() : attrs_of.find(k->output_values[0]);
            ExecuteKernel(plan, k, it == attrs_of.end() ? nullptr : it->second);
        } else if (ref.get()->GetTypeId() == CommExecNode::_type_index) {
            ExecuteComm(plan, static_cast<const CommExecNode*>(ref.get()));
        } else if (ref.get()->GetTypeId() == BarrierExecNode::_type_index) {
            const auto* b = static_cast<const BarrierExecNode*>(ref.get());
            for (int worker : EffectiveWorkerSet(b->worker_set, 0)) backend_->SyncWorker(session_, worker);
        } else {
            Fail("ExecutionPlan contains unknown node type");
        }
    }
    const int output = plan->output_value;
    if (output < 0 || !values_.count(output)) Fail("ExecutionPlan output value is missing after execution");
    disco::DRef out = values_.at(output);
    for (int w = 0; w < session_.num_workers(); ++w) {
        backend_->SyncWorker(session_, w);
        if (backend_->values().Find(out, w)) backend_->values().Download(session_, out, w);
    }
    return out;
}

}  // namespace b200
}  // namespace kxc
