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
// The function's parameters are the `in` tensors in declaration order; its result is the last OUT.
// Each op may appear once per function: CodeGenC names buffers after the op (codegen_c.cc:38-46).

#include <cstdint>
#include <cstdlib>
#include <iostream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "codegen/codegen_c.h"
#include "relay/op.h"
#include "relay/relay.h"
#include "relay/transforms/infer_type.h"
#include "relay/transforms/lower.h"
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

}  // namespace

int main(int argc, char** argv) {
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
