// Driver for the reference-side binding (kxc_b200_adapter.h): loads graphs with the reference's own importer, runs them
// through the reference's own entry points (CompiledKernel::operator(), an ExecutionPlan walk, the CCLBackend interface)
// with the kernels of libkxc_b200.so behind them, and writes the results for the tests to compare.
//
//   adapter_demo registry                                       operators with an FB200Launch attribute (no GPU needed)
//   adapter_demo graph <spec.json> <params.bin> <in> <out> <p>  whole graph as ONE CompiledKernel (p = fp32|tf32|bf16|tf32x3)
//   adapter_demo plan  <spec.json> <params.bin> <in> <out> <p>  the reference's ExecutionPlan, node by node via kernel_symbol
//   adapter_demo ccl   <workers>                                NcclCCLBackend against CpuCCLBackend, one GPU per worker
#include <dlfcn.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include "base/device.h"
#include "base/device_api.h"
#include "base/disco/session.h"
#include "frontend/onnx_importer.h"
#include "relay/transforms/infer_type.h"
#include "relay/transforms/multi_device.h"

#include "kxc_b200.h"
#include "kxc_b200_adapter.h"

using namespace kxc;
using DeviceT = class Device;

namespace {

int Precision(const std::string& p) {
    if (p == "fp32") return KXC_B200_PREC_FP32;
    if (p == "tf32") return KXC_B200_PREC_TF32;
    if (p == "bf16") return KXC_B200_PREC_BF16;
    if (p == "tf32x3") return KXC_B200_PREC_TF32X3;
    throw std::runtime_error("unknown precision " + p);
}

std::vector<char> ReadFile(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot read " + path);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
void WriteFile(const std::string& path, const void* data, size_t bytes) {
    std::ofstream f(path, std::ios::binary);
    f.write(static_cast<const char*>(data), (std::streamsize)bytes);
    if (!f) throw std::runtime_error("cannot write " + path);
}
size_t TypeBytes(const Type& t) {
    const auto* tt = t.As<TensorTypeNode>();
    if (!tt) throw std::runtime_error("non-tensor type");
    size_t n = 4;
    for (size_t i = 0; i < tt->shape.size(); ++i) n *= (size_t)tt->shape[i];
    return n;
}

int Registry() {
    b200::RegisterB200Ops();
    int missing = 0;
    for (const char* name : {"nn_conv2d", "nn_relu", "add", "nn_max_pool2d", "nn_avg_pool2d", "nn_global_avg_pool2d", "nn_flatten", "nn_dense",
                             "nn_gemm", "softmax"}) {
        const b200::FB200Launch* h = b200::GetB200Launch(name);
        void* sym = h ? dlsym(RTLD_DEFAULT, h->kernel_symbol.c_str()) : nullptr;
        std::cout << name << " -> " << (h ? h->kernel_symbol : std::string("-")) << (sym ? " (resolved)" : " (MISSING)") << "\n";
        // the attribute sits beside the reference's own FInferType / FRelayToTE attributes on the same OpNode
        const auto& attrs = relay::Op::Get(name)->attrs;
        if (!h || !sym || !attrs.count("FRelayToTE") || !attrs.count("FInferType")) ++missing;
    }
    std::cout << (missing ? "registry FAILED" : "registry ok") << "\n";
    return missing ? 1 : 0;
}

int Graph(const std::string& spec, const std::string& params, const std::string& in_path, const std::string& out_path, int precision) {
    frontend::ImportedONNXModel m = frontend::LoadONNXImportSpec(spec, params);
    Function func = relay::InferTypePass(m.function);
    std::vector<runtime::NDArray> consts = b200::ConstantsInLoweringOrder(func);
    DeviceAPI* api = GetDeviceAPI(DeviceTypeCode::kGPU);
    const class Device gpu(DeviceTypeCode::kGPU, 0), cpu(DeviceTypeCode::kCPU, 0);
    api->SetDevice(gpu);
    // packed argument list of the reference's kxc_kernel_main: inputs, constants in lowering order, output
    std::vector<void*> args;
    std::vector<char> input = ReadFile(in_path);
    const size_t in_bytes = TypeBytes(func->params[0]->type_annotation);
    if (input.size() != in_bytes) throw std::runtime_error("input file has " + std::to_string(input.size()) + " bytes, expected " + std::to_string(in_bytes));
    void* d_in = api->AllocDataSpace(gpu, in_bytes, 256);
    api->CopyDataFromTo(cpu, input.data(), gpu, d_in, in_bytes);
    args.push_back(d_in);
    for (const auto& c : consts) {
        void* d = api->AllocDataSpace(gpu, c.NBytes(), 256);
        api->CopyDataFromTo(cpu, c->dl_tensor.data, gpu, d, c.NBytes());
        args.push_back(d);
    }
    const size_t out_bytes = TypeBytes(func->body.checked_type());
    void* d_out = api->AllocDataSpace(gpu, out_bytes, 256);
    args.push_back(d_out);

    codegen::CompiledKernel kernel = b200::CompileForB200(func, precision, nullptr);
    if (!kernel.IsReady()) throw std::runtime_error("kernel not ready");
    kernel(args);  // CompiledKernel::operator(): int32_t (*)(void**) behind it, throws on a non-zero return
    api->StreamSync(gpu, nullptr);
    std::vector<char> out(out_bytes);
    api->CopyDataFromTo(gpu, d_out, cpu, out.data(), out_bytes);
    WriteFile(out_path, out.data(), out_bytes);
    // error convention: a failing kernel surfaces as the reference's own exception
    std::vector<void*> bad = args;
    bad.back() = nullptr;
    try {
        kernel(bad);
        std::cout << "error path FAILED: no exception\n";
        return 1;
    } catch (const std::runtime_error& e) {
        const std::string msg = e.what();
        std::cout << "error path: " << msg << "\n";
        if (msg.find("Kernel kxc_kernel_main returned error code") == std::string::npos) return 1;
    }
    for (void* p : args) api->FreeDataSpace(gpu, p);
    std::cout << "graph ok: " << consts.size() << " constants, " << out_bytes << " output bytes\n";
    return 0;
}

int Plan(const std::string& spec, const std::string& params, const std::string& in_path, const std::string& out_path, int precision) {
    frontend::ImportedONNXModel m = frontend::LoadONNXImportSpec(spec, params);
    Function func = relay::InferTypePass(m.function);
    ExecutionPlan plan = relay::LowerRelayToExecPlanPass(func);
    std::map<int, const CallNode*> side = b200::BindKernelSymbols(plan, func);
    // the bound plan survives the reference's own serializer and reader
    ExecutionPlan again = DeserializeExecutionPlanFromJson(SerializeExecutionPlanToJson(plan));
    int kernels = 0;
    for (size_t i = 0; i < again->nodes.size(); ++i) {
        if (!again->nodes[i].defined() || again->nodes[i].get()->GetTypeId() != KernelExecNode::_type_index) continue;
        const auto* k = static_cast<const KernelExecNode*>(again->nodes[i].get());
        std::cout << "node " << i << " " << k->op_name << " -> " << k->kernel_symbol << "\n";
        if (k->kernel_symbol.empty()) return 1;
        ++kernels;
    }
    disco::DiscoSession session = disco::DiscoSession::ThreadedSession(1);
    auto backend = std::make_shared<b200::NcclCCLBackend>(std::vector<int>{0});
    Map<int, disco::DRef> initial;
    {
        const auto* tt = func->params[0]->type_annotation.As<TensorTypeNode>();
        runtime::NDArray x(tt->shape, tt->dtype);
        std::vector<char> input = ReadFile(in_path);
        if (input.size() != x.NBytes()) throw std::runtime_error("input file size mismatch");
        x.CopyFromBytes(input.data(), input.size());
        disco::DRef r = session.NewDRef();
        session.Set(0, r, x);
        initial.Set(plan->input_value_ids[0], r);
    }
    std::vector<runtime::NDArray> consts = b200::ConstantsInLoweringOrder(func);
    if (consts.size() != plan->constant_value_ids.size()) throw std::runtime_error("constant count differs from the plan's");
    for (size_t i = 0; i < consts.size(); ++i) {
        disco::DRef r = session.NewDRef();
        session.Set(0, r, consts[i]);
        initial.Set(plan->constant_value_ids[i], r);
    }
    b200::B200PlanExecutor executor(session, backend, precision);
    disco::DRef out = executor.ExecuteForOutput(plan, side, initial);
    runtime::NDArray y = session.Get(0, out);
    if (!y.defined()) throw std::runtime_error("no output in the session register");
    WriteFile(out_path, y->dl_tensor.data, y.NBytes());
    std::cout << "plan ok: " << kernels << " kernel nodes, " << y.NBytes() << " output bytes\n";
    return 0;
}

bool SameArray(const runtime::NDArray& a, const runtime::NDArray& b) {
    if (!a.defined() || !b.defined()) return a.defined() == b.defined();
    if (a->shape != b->shape || a.NBytes() != b.NBytes()) return false;
    return std::memcmp(a->dl_tensor.data, b->dl_tensor.data, a.NBytes()) == 0;
}

int Ccl(int n) {
    disco::DiscoSession session = disco::DiscoSession::ThreadedSession(n);
    std::shared_ptr<disco::CCLBackend> cpu = disco::CreateCpuCCLBackend();
    std::vector<int> devices;
    for (int i = 0; i < n; ++i) devices.push_back(i);
    std::shared_ptr<disco::CCLBackend> nccl = std::make_shared<b200::NcclCCLBackend>(devices);
    // per-worker shards [3, 5] of small integers (sums stay exact in any order), a [3n, 5] tensor on worker 0
    disco::DRef shard = session.NewDRef(), full = session.NewDRef();
    for (int w = 0; w < n; ++w) {
        runtime::NDArray a({3, 5}, "float32");
        auto* p = static_cast<float*>(a->dl_tensor.data);
        for (int i = 0; i < 15; ++i) p[i] = (float)(100 * w + i);
        session.Set(w, shard, a);
    }
    {
        runtime::NDArray a({3 * n, 5}, "float32");
        auto* p = static_cast<float*>(a->dl_tensor.data);
        for (int i = 0; i < 15 * n; ++i) p[i] = (float)(7 * i - 3);
        session.Set(0, full, a);
    }
    int bad = 0;
    auto check = [&](const char* what, const std::function<void(disco::CCLBackend&, const disco::DRef&)>& run, const std::vector<int>& workers) {
        disco::DRef a = session.NewDRef(), b = session.NewDRef();
        run(*cpu, a);
        run(*nccl, b);
        bool same = true;
        for (int w : workers) same = same && SameArray(session.Get(w, a), session.Get(w, b)) && session.Get(w, a).defined();
        std::cout << what << (same ? " ok" : " DIFFERS") << "\n";
        if (!same) ++bad;
    };
    std::vector<int> all;
    for (int w = 0; w < n; ++w) all.push_back(w);
    check("gather_to_worker0", [&](disco::CCLBackend& be, const disco::DRef& d) { be.GatherToWorker0(session, shard, d, true); }, {0});
    check("scatter_from_worker0", [&](disco::CCLBackend& be, const disco::DRef& d) { be.ScatterFromWorker0(session, full, d, true); }, all);
    check("broadcast_from_worker0", [&](disco::CCLBackend& be, const disco::DRef& d) { be.BroadcastFromWorker0(session, full, d, true); }, all);
    check("allreduce(sum)", [&](disco::CCLBackend& be, const disco::DRef& d) { be.AllReduce(session, shard, d, "sum", true); }, all);
    check("copy 0 -> last", [&](disco::CCLBackend& be, const disco::DRef& d) { be.Copy(session, shard, d, 0, n - 1); }, {n - 1});
    check("send_to_worker(last)", [&](disco::CCLBackend& be, const disco::DRef& d) { be.SendToWorker(session, shard, d, n - 1); }, {n - 1});
    check("recv_from_worker(last)", [&](disco::CCLBackend& be, const disco::DRef& d) { be.RecvFromWorker(session, shard, d, n - 1); }, {0});
    std::cout << (bad ? "ccl FAILED" : "ccl ok") << " workers=" << n << "\n";
    return bad ? 1 : 0;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        const std::string cmd = argc > 1 ? argv[1] : "";
        if (cmd == "registry") return Registry();
        if (cmd == "graph" && argc == 7) return Graph(argv[2], argv[3], argv[4], argv[5], Precision(argv[6]));
        if (cmd == "plan" && argc == 7) return Plan(argv[2], argv[3], argv[4], argv[5], Precision(argv[6]));
        if (cmd == "ccl" && argc == 3) return Ccl(std::atoi(argv[2]));
        std::cerr << "usage: adapter_demo registry | graph|plan <spec.json> <params.bin> <in> <out> <precision> | ccl <workers>\n";
        return 2;
    } catch (const std::exception& e) {
        std::cerr << "adapter_demo: " << e.what() << "\n";
        return 1;
    }
}
