// ref_emit: drives the UNMODIFIED reference compiler (KDZZZZZZ/hdkx-aicompiler) to lower a small
// Relay graph to C source text, which the Python side (oracle/ref_oracle.py) compiles with gcc
// -ffp-contract=off into the "reference" CPU checker.
//
// TEST INFRASTRUCTURE ONLY. Nothing the product ships links, loads or executes this program.
//
// The lowering sequence is the one the reference's own numeric tests use
// (test/op_numeric_llvm_test.cpp:44-50, test/onnx_importer_test.cpp:131-136):
//   InferTypePass -> RunRelayPassPipeline{fold_constant, simplify_expr} -> InferTypePass
//   -> LowerToTIR (src/relay/backend/lower.cc:470) -> RunTIRPassPipeline{fold_constant, simplify_expr}
//   -> codegen::CodeGenC::Generate (src/codegen/codegen_c.cc:54), same `int32_t f(void** packed_args)`
//   ABI as the LLVM backend (src/codegen/codegen_llvm.cc:56-63).
//
// Usage: ref_emit <symbol> "<stmt>;<stmt>;..."  (C text on stdout)
//   in   NAME DTYPE d0,d1,...
//   conv2d OUT DATA WEIGHT BIAS|- sh,sw ph,pw dh,dw
//   relu OUT X | add OUT A B | flatten OUT X | global_avg_pool2d OUT X
//   max_pool2d OUT X kh,kw sh,sw pt,pl,pb,pr ceil   (avg_pool2d likewise)
//   dense OUT X W | gemm OUT A B C alpha beta transA transB
//   softmax OUT X axis | reduce_mean OUT X a0,a1,... keepdims
//   matmul OUT A B | transpose OUT X a0,a1,...|- | reshape OUT X d0,d1,... | cast OUT X code
// The function's parameters are the `in` tensors in declaration order; its result is the last OUT.
// Each op may appear once per function: CodeGenC names buffers after the op (codegen_c.cc:38-46).
//
// Usage: ref_emit --import <spec.json> <params.bin>   (JSON on stdout)
// Usage: ref_emit --plan <spec.json> <params.bin> | ref_emit --plan-check <plan.json>   (ExecutionPlan JSON on stdout)
//   The reference's ExecutionPlan of an imported graph in its own JSON form, and its reader applied to such a file.
//
//   --import loads a "kxc.onnx_import.v1" graph with the reference's own importer (LoadONNXImportSpec,
//   src/frontend/onnx_importer.cc:410-520), runs its InferTypePass and prints the resulting Relay function as the
//   reference sees it: inputs, calls in post order (operator name, arguments, attributes as its Attrs objects hold
//   them, inferred output shape) and the result. The Python side feeds that one description to both the CPU checker
//   and the GPU executor, so both compute the graph the reference's importer built.

#include <cstdint>
#include <cstdlib>
#include <functional>
#include <iostream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "codegen/codegen_c.h"
#include "frontend/onnx_importer.h"
#include "relay/op.h"
#include "relay/relay.h"
#include "relay/transforms/infer_type.h"
#include "base/execution_plan.h"
#include "relay/transforms/lower.h"
#include "relay/transforms/multi_device.h"
#include "relay/transforms/pipeline.h"
#include "tir/transforms/pipeline.h"

namespace {

std::vector<std::string> SplitWs(const std::string& s) {
    std::istringstream is(s);
    std::vector<std::string> out;
    std::string tok;
    while (is >> tok) out.push_back(tok);
    return out;
}

std::vector<int64_t> Ints(const std::string& s) {
    std::vector<int64_t> out;
    std::string cur;
    for (char c : s + ",") {
        if (c == ',') {
            if (!cur.empty()) out.push_back(std::atoll(cur.c_str()));
            cur.clear();
        } else {
            cur.push_back(c);
        }
    }
    return out;
}

kxc::Array<int64_t> ToArray(const std::vector<int64_t>& v) {
    kxc::Array<int64_t> a;
    for (auto x : v) a.push_back(x);
    return a;
}

std::string JsonInts(const std::vector<int64_t>& v) {
    std::string s = "[";
    for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
    return s + "]";
}
std::string JsonInts(const kxc::Array<int64_t>& a) {
    std::vector<int64_t> v;
    for (size_t i = 0; i < a.size(); ++i) v.push_back(a[i]);
    return JsonInts(v);
}

std::string AttrsJson(const std::string& op, const kxc::ObjectRef& attrs) {
    using namespace kxc::relay;
    std::ostringstream os;
    if (op == "nn_conv2d") {
        const auto* a = attrs.As<Conv2DAttrsNode>();
        if (!a) throw std::runtime_error("nn_conv2d without Conv2DAttrs");
        os << "{\"strides\":" << JsonInts(a->strides) << ",\"padding\":" << JsonInts(a->padding) << ",\"dilation\":"
           << JsonInts(a->dilation) << ",\"groups\":" << a->groups << "}";
    } else if (op == "nn_max_pool2d" || op == "nn_avg_pool2d") {
        const auto* a = attrs.As<MaxPool2DAttrsNode>();
        if (!a) throw std::runtime_error(op + " without MaxPool2DAttrs");
        os << "{\"pool_size\":" << JsonInts(a->pool_size) << ",\"strides\":" << JsonInts(a->strides) << ",\"padding\":"
           << JsonInts(a->padding) << ",\"dilation\":" << JsonInts(a->dilation) << ",\"ceil_mode\":" << (a->ceil_mode ? 1 : 0) << "}";
    } else if (op == "nn_gemm") {
        const auto* a = attrs.As<GemmAttrsNode>();
        if (!a) throw std::runtime_error("nn_gemm without GemmAttrs");
        std::ostringstream f;
        f.precision(9);
        f << "{\"alpha\":" << a->alpha << ",\"beta\":" << a->beta << ",\"transA\":" << a->transA << ",\"transB\":" << a->transB << "}";
        os << f.str();
    } else if (op == "nn_flatten") {
        const auto* a = attrs.As<FlattenAttrsNode>();
        os << "{\"axis\":" << (a ? a->axis : 1) << "}";
    } else {
        os << "{}";
    }
    return os.str();
}

int DumpImported(const std::string& json_path, const std::string& params_path) {
    kxc::frontend::ImportedONNXModel m = kxc::frontend::LoadONNXImportSpec(json_path, params_path);
    kxc::Function func = kxc::relay::InferTypePass(m.function);
    std::map<const void*, std::string> param_of;  // constant storage -> parameter name
    for (const auto& kv : m.params) param_of[kv.second->dl_tensor.data] = kv.first;
    std::map<const kxc::Object*, int> id_of;
    std::ostringstream nodes;
    int next_id = 0;
    auto shape_of = [](const kxc::Expr& e) -> std::string {
        const auto* tt = e.checked_type().As<kxc::TensorTypeNode>();
        if (!tt) throw std::runtime_error("non-tensor value in the imported function");
        return JsonInts(tt->shape);
    };
    std::function<std::string(const kxc::Expr&)> ref = [&](const kxc::Expr& e) -> std::string {
        if (const auto* v = e.As<kxc::VarNode>()) return "{\"var\":\"" + v->vid->name_hint + "\"}";
        if (const auto* c = e.As<kxc::ConstantNode>()) {
            auto it = param_of.find(c->data->dl_tensor.data);
            if (it == param_of.end()) throw std::runtime_error("constant that is not a parameter of the spec");
            return "{\"param\":\"" + it->second + "\"}";
        }
        const auto* call = e.As<kxc::CallNode>();
        if (!call) throw std::runtime_error("unsupported expression kind in the imported function");
        auto done = id_of.find(call);
        if (done != id_of.end()) return "{\"node\":" + std::to_string(done->second) + "}";
        const auto* op = call->op.As<kxc::relay::OpNode>();
        if (!op) throw std::runtime_error("call of a non-operator");
        std::string args;
        for (size_t i = 0; i < call->args.size(); ++i) args += (i ? "," : "") + ref(call->args[i]);
        const int id = next_id++;
        id_of[call] = id;
        nodes << (id ? ",\n" : "") << "  {\"id\":" << id << ",\"op\":\"" << op->name << "\",\"args\":[" << args
              << "],\"attrs\":" << AttrsJson(op->name, call->attrs) << ",\"shape\":" << shape_of(e) << "}";
        return "{\"node\":" + std::to_string(id) + "}";
    };
    const std::string result = ref(func->body);
    std::cout << "{\"inputs\":[";
    for (size_t i = 0; i < func->params.size(); ++i) {
        const auto* tt = func->params[i]->type_annotation.As<kxc::TensorTypeNode>();
        std::cout << (i ? "," : "") << "{\"name\":\"" << func->params[i]->vid->name_hint << "\",\"shape\":"
                  << (tt ? JsonInts(tt->shape) : std::string("[]")) << ",\"dtype\":\"" << (tt ? tt->dtype : "") << "\"}";
    }
    std::cout << "],\n \"nodes\":[\n" << nodes.str() << "\n ],\n \"result\":" << result << "}\n";
    return 0;
}

}  // namespace

// --plan: the reference's own ExecutionPlan for an imported graph (LowerRelayToExecPlanPass,
// src/relay/transforms/multi_device.cc:244-), serialized by its own SerializeExecutionPlanToJson.
int DumpPlan(const std::string& json_path, const std::string& params_path) {
    kxc::frontend::ImportedONNXModel m = kxc::frontend::LoadONNXImportSpec(json_path, params_path);
    kxc::Function func = kxc::relay::InferTypePass(m.function);
    kxc::ExecutionPlan plan = kxc::relay::LowerRelayToExecPlanPass(func);
    std::cout << kxc::SerializeExecutionPlanToJson(plan) << "\n";
    return 0;
}

// --plan-check: feed a plan JSON (for instance one whose kernel_symbol fields were filled in) to the reference's
// DeserializeExecutionPlanFromJson and print what it serializes back.
int CheckPlan(const std::string& path) {
    kxc::ExecutionPlan plan = kxc::LoadExecutionPlanFromJsonFile(path);
    std::cout << kxc::SerializeExecutionPlanToJson(plan) << "\n";
    return 0;
}

int main(int argc, char** argv) {
    if ((argc == 4 && std::string(argv[1]) == "--plan") || (argc == 3 && std::string(argv[1]) == "--plan-check")) {
        try {
            return argc == 4 ? DumpPlan(argv[2], argv[3]) : CheckPlan(argv[2]);
        } catch (const std::exception& e) {
            std::cerr << "ref_emit: " << e.what() << "\n";
            return 1;
        }
    }
    if (argc == 4 && std::string(argv[1]) == "--import") {
        try {
            return DumpImported(argv[2], argv[3]);
        } catch (const std::exception& e) {
            std::cerr << "ref_emit: " << e.what() << "\n";
            return 1;
        }
    }
    if (argc != 3) {
        std::cerr << "usage: ref_emit <symbol> \"<stmt>;...\"\n";
        return 2;
    }
    try {
        const std::string symbol = argv[1];
        std::map<std::string, kxc::Expr> env;
        kxc::Array<kxc::Var> params;
        kxc::Expr last;

        std::string prog = argv[2];
        std::string stmt;
        std::istringstream ps(prog);
        auto get = [&](const std::string& n) -> kxc::Expr {
            auto it = env.find(n);
            if (it == env.end()) throw std::runtime_error("unknown value: " + n);
            return it->second;
        };
        while (std::getline(ps, stmt, ';')) {
            auto t = SplitWs(stmt);
            if (t.empty()) continue;
            const std::string& op = t[0];
            if (op == "in") {
                kxc::Var v(t[1], kxc::TensorType(ToArray(Ints(t[3])), t[2]));
                params.push_back(v);
                env[t[1]] = v;
                continue;
            }
            kxc::Expr out;
            if (op == "conv2d") {
                auto s = Ints(t[5]), p = Ints(t[6]), d = Ints(t[7]);
                kxc::Array<kxc::Expr> args;
                args.push_back(get(t[2]));
                args.push_back(get(t[3]));
                if (t[4] != "-") args.push_back(get(t[4]));
                auto attrs = kxc::relay::Conv2DAttrs::Create(
                    {s[0], s[1]}, {p[0], p[1], p[0], p[1]}, {d[0], d[1]}, 1, 0, {}, "NCHW", "OIHW", "", "");
                out = kxc::Call(kxc::relay::Op::Get("nn_conv2d"), args, attrs);
            } else if (op == "relu") {
                out = kxc::Call(kxc::relay::Op::Get("nn_relu"), {get(t[2])}, kxc::relay::ReluAttrs::Create());
            } else if (op == "add") {
                out = kxc::Call(kxc::relay::Op::Get("add"), {get(t[2]), get(t[3])});
            } else if (op == "flatten") {
                out = kxc::Call(kxc::relay::Op::Get("nn_flatten"), {get(t[2])},
                                kxc::relay::FlattenAttrs::Create(1));
            } else if (op == "global_avg_pool2d") {
                out = kxc::Call(kxc::relay::Op::Get("nn_global_avg_pool2d"), {get(t[2])},
                                kxc::relay::GlobalAvgPool2DAttrs::Create());
            } else if (op == "max_pool2d" || op == "avg_pool2d") {
                auto k = Ints(t[3]), s = Ints(t[4]), p = Ints(t[5]);
                bool ceil = std::atoi(t[6].c_str()) != 0;
                auto attrs = kxc::relay::MaxPool2DAttrs::Create({s[0], s[1]}, {p[0], p[1], p[2], p[3]}, {1, 1},
                                                                {k[0], k[1]}, "NCHW", ceil);
                out = kxc::Call(kxc::relay::Op::Get(op == "max_pool2d" ? "nn_max_pool2d" : "nn_avg_pool2d"),
                                {get(t[2])}, attrs);
            } else if (op == "softmax") {
                out = kxc::Call(kxc::relay::Op::Get("softmax"), {get(t[2])}, kxc::relay::SoftmaxAttrs::Create(std::atoi(t[3].c_str())));
            } else if (op == "reduce_mean") {
                out = kxc::Call(kxc::relay::Op::Get("reduce_mean"), {get(t[2])},
                                kxc::relay::ReduceMeanAttrs::Create(Ints(t[3]), std::atoi(t[4].c_str())));
            } else if (op == "matmul") {
                out = kxc::Call(kxc::relay::Op::Get("matmul"), {get(t[2]), get(t[3])});
            } else if (op == "transpose") {
                out = kxc::Call(kxc::relay::Op::Get("transpose"), {get(t[2])},
                                kxc::relay::TransposeAttrs::Create(t[3] == "-" ? std::vector<int64_t>{} : Ints(t[3])));
            } else if (op == "reshape") {
                out = kxc::Call(kxc::relay::Op::Get("reshape"), {get(t[2])}, kxc::relay::ReshapeAttrs::Create(Ints(t[3]), 0));
            } else if (op == "cast") {
                out = kxc::Call(kxc::relay::Op::Get("cast"), {get(t[2])}, kxc::relay::CastAttrs::Create(std::atoi(t[3].c_str())));
            } else if (op == "dense") {
                out = kxc::Call(kxc::relay::Op::Get("nn_dense"), {get(t[2]), get(t[3])},
                                kxc::relay::DenseAttrs::Create(0, ""));
            } else if (op == "gemm") {
                auto attrs = kxc::relay::GemmAttrs::Create(std::atof(t[5].c_str()), std::atof(t[6].c_str()),
                                                           std::atoi(t[7].c_str()), std::atoi(t[8].c_str()));
                out = kxc::Call(kxc::relay::Op::Get("nn_gemm"), {get(t[2]), get(t[3]), get(t[4])}, attrs);
            } else {
                throw std::runtime_error("unknown statement: " + op);
            }
            env[t[1]] = out;
            last = out;
        }
        if (!last.defined()) throw std::runtime_error("no op in program");

        kxc::Function func(params, last);
        func = kxc::relay::InferTypePass(func);
        func = kxc::relay::RunRelayPassPipeline(func, {kxc::String("fold_constant"), kxc::String("simplify_expr")});
        func = kxc::relay::InferTypePass(func);
        kxc::tir::PrimFunc pf = kxc::relay::LowerToTIR(func);
        pf = kxc::tir::RunTIRPassPipeline(pf, {kxc::String("fold_constant"), kxc::String("simplify_expr")});
        std::cout << kxc::codegen::CodeGenC().Generate(pf, symbol);
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "ref_emit: " << e.what() << "\n";
        return 1;
    }
}
