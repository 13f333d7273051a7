// kxc_b200_adapter.h — the reference-side binding of libkxc_b200.so: the translation unit a maintainer of the
// hdkx-aicompiler ("kxc") tree adds to route its kernel slots to the B200 library. It is compiled against the
// reference's own public headers and linked with the reference's objects; nothing in the reference is modified.
//
// What it binds (reference file:line of the slot each piece fills):
//   * an `FB200Launch` attribute on the registered Relay ops, next to their FInferType / FRelayToTE attributes
//     (include/relay/op_macros.h:27-32, lookup pattern of src/relay/backend/lower.cc:120-129);
//   * CompileForB200(): Relay Function -> kxc_b200_plan -> codegen::CompiledKernel whose func_ptr is a real
//     `int32_t f(void** packed_args)` (src/codegen/compiled_kernel.cc:41-55), packed_args = inputs ++ constants in
//     lowering DFS order ++ output (src/relay/backend/lower.cc:534-565), all DEVICE pointers
//     (DeviceAPI::AllocDataSpace of a kGPU device, src/base/device/cuda_device_api.cc:89-105);
//   * B200PlanExecutor: the interpreter loop of ExecutionPlanExecutor::Execute with a real ExecuteKernel
//     (src/base/disco/executor.cc:48-92, :122-157 is the placeholder it replaces): every KernelExecNode is bound to
//     the C-ABI symbol that runs it (KernelExecNode::kernel_symbol, include/base/execution_plan.h:42-50), resolved
//     with dlsym and launched on the worker's GPU;
//   * NcclCCLBackend: a CCLBackend (include/base/disco/ccl_backend.h:16-35) whose collectives run over NCCL on device
//     buffers, with the semantics of CpuCCLBackend (src/base/disco/ccl_cpu.cc:176-317); the reference's own
//     NcclCCLBackend is a stub whose methods throw (src/base/disco/ccl_nccl.cc:13-40).
#pragma once

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "base/disco/ccl_backend.h"
#include "base/disco/executor.h"
#include "base/execution_plan.h"
#include "codegen/compiled_kernel.h"
#include "relay/op.h"
#include "relay/relay.h"

#include "kxc_b200_plan.h"

namespace kxc {
namespace b200 {

// Per-operator hooks, stored on the OpNode under the attribute name "FB200Launch".
struct FB200Launch {
    // the C-ABI entry point that runs ONE node of this operator (what KernelExecNode::kernel_symbol is bound to)
    std::string kernel_symbol;
    // appends the call as one KernelExec node of a whole-graph plan
    std::function<int32_t(kxc_b200_plan* plan, const CallNode& call, const std::vector<int32_t>& input_ids, int32_t output_id)> add_to_plan;
    // runs the call as one kernel: `entry` is the dlsym'd kernel_symbol, packed_args = device pointers, inputs then output
    std::function<int32_t(void* entry, const CallNode& call, void** packed_args, int precision, void* stream)> launch;
};

// Registers FB200Launch on every operator the library implements (idempotent). Called by the functions below.
void RegisterB200Ops();
// The hook of a registered operator, or nullptr.
const FB200Launch* GetB200Launch(const std::string& op_name);

// Relay Function (InferTypePass is run here) -> CompiledKernel on the current CUDA device. `precision` is a
// KXC_B200_PREC_* value. Constants are passed by the caller at run time, in lowering order, like for the reference's
// own kernels; ConstantsInLoweringOrder gives that order.
codegen::CompiledKernel CompileForB200(const Function& func, int precision, void* stream = nullptr);
std::vector<runtime::NDArray> ConstantsInLoweringOrder(const Function& func);

// Fills the reserved kernel_symbol of every KernelExecNode of `plan` (in place) and returns the side table
// value id -> Relay call that carries the attributes the plan JSON drops (src/base/execution_plan.cc:695-708).
std::map<int, const CallNode*> BindKernelSymbols(const ExecutionPlan& plan, const Function& typed_func);

// Device-resident values of a session: (register, worker) -> device buffer. Host NDArrays in the session's registers
// are uploaded on first use; Download() writes a device value back into its register.
class DeviceValues;

class NcclCCLBackend final : public disco::CCLBackend {
  public:
    // one NCCL communicator per worker, worker i on CUDA device devices[i] (all driven by the calling thread)
    explicit NcclCCLBackend(std::vector<int> devices);
    ~NcclCCLBackend() override;
    void Copy(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, int src_worker, int dst_worker) override;
    void AllReduce(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, const std::string& reduce_kind,
                   bool in_group) override;
    void BroadcastFromWorker0(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, bool in_group) override;
    void ScatterFromWorker0(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, bool in_group) override;
    void GatherToWorker0(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, bool in_group) override;
    void SendToWorker(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, int receiver_worker) override;
    void RecvFromWorker(const disco::DiscoSession& session, const disco::DRef& src, const disco::DRef& dst, int sender_worker) override;
    void SyncWorker(const disco::DiscoSession& session, int worker_id) override;

    DeviceValues& values();
    int device_of(int worker) const;
    void* stream_of(int worker) const;

  private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

// ExecutionPlanExecutor with a real ExecuteKernel: same node walk, kernels dispatched through kernel_symbol.
class B200PlanExecutor {
  public:
    B200PlanExecutor(disco::DiscoSession session, std::shared_ptr<NcclCCLBackend> backend, int precision);
    // `attrs_of` is the side table of BindKernelSymbols. initial_values: value id -> DRef of host NDArrays per worker
    // (plan inputs and constants), as for ExecutionPlanExecutor::Execute.
    disco::DRef ExecuteForOutput(const ExecutionPlan& plan, const std::map<int, const CallNode*>& attrs_of,
                                 const Map<int, disco::DRef>& initial_values);

  private:
    void ExecuteKernel(const ExecutionPlan& plan, const KernelExecNode* kernel, const CallNode* call);
    void ExecuteComm(const ExecutionPlan& plan, const CommExecNode* comm);
    disco::DiscoSession session_;
    std::shared_ptr<NcclCCLBackend> backend_;
    int precision_;
    Map<int, disco::DRef> values_;
};

}  // namespace b200
}  // namespace kxc
