// Common Setup/Execute state machine of the operators: argument checks, error codes and the
// Setup -> Execute contract of OperationBase in the reference
// (src/atb/operation/operation_base.cpp:369-449 CheckVariantPack/SetupCheck, :600-668 Setup,
//  :752-862 ExecuteCheck, :1095-1133 Execute).  The kernel-graph / runner machinery of the
// reference collapses into two virtual hooks: PlanImpl (host, at Setup) and LaunchImpl (enqueue).
#ifndef ATB_B200_OPERATION_BASE_H
#define ATB_B200_OPERATION_BASE_H
#include <atomic>
#include <string>
#include <vector>
#include "atb/atb_infer.h"
#include "../../include/atb_b200.h"

namespace atb {

class ContextImpl : public Context {
public:
    Status SetExecuteStream(aclrtStream stream) override;
    aclrtStream GetExecuteStream() const override;
    Status SetAsyncTilingCopyStatus(bool enable) override;
    bool GetAsyncTilingCopyStatus() const override;
    Status SetExecuteStreams(const std::vector<aclrtStream> &streams) override;
    std::vector<aclrtStream> GetExecuteStreams() override;
    Status SetExecuteType(ExecuteType type) override;
    ExecuteType GetExecuteType() override;
    Status SetLaunchMode(LaunchMode mode) override;
    LaunchMode GetLaunchMode() override;
    // Extension (atb_b200_context_set_gather): the ranks' gathered output buffers for the next
    // PagedAttention Execute calls on this context, or none.
    void SetGatherPeers(const atb_b200_pa_peers *peers)
    {
        hasPeers_ = peers != nullptr;
        if (hasPeers_) {
            peers_ = *peers;
        }
    }
    const atb_b200_pa_peers *GatherPeers() const { return hasPeers_ ? &peers_ : nullptr; }

private:
    atb_b200_pa_peers peers_{};
    bool hasPeers_ = false;
    std::vector<aclrtStream> streams_{nullptr};
    bool asyncTilingCopy_ = false;
    LaunchMode mode_ = KERNEL_LAUNCH_MODE;
};

// One allowed combination of tensor dtypes (inputs then outputs), the role of a column of the
// reference's ops_configs/atb_ops_info.ini section.
using DtypeComb = std::vector<aclDataType>;

class OperationBase : public Operation {
public:
    explicit OperationBase(const std::string &name) : name_(name) {}
    std::string GetName() const override { return name_; }
    Status InferShape(const SVector<TensorDesc> &inTensorDescs, SVector<TensorDesc> &outTensorDescs) const override;
    Status Setup(const VariantPack &variantPack, uint64_t &workspaceSize, Context *context) override;
    Status Execute(const VariantPack &variantPack, uint8_t *workspace, uint64_t workspaceSize,
                   Context *context) override;

protected:
    virtual Status InferShapeCheckImpl(const SVector<TensorDesc> &inTensorDescs) const = 0;
    virtual Status InferShapeImpl(const SVector<TensorDesc> &inTensorDescs,
                                  SVector<TensorDesc> &outTensorDescs) const = 0;
    virtual Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &outTensors) const = 0;
    virtual const std::vector<DtypeComb> &DtypeCombs() const = 0;
    // Host planning from the tensors' descs and hostData; returns the workspace size.
    virtual Status PlanImpl(const VariantPack &variantPack, uint64_t &workspaceSize) = 0;
    // Optional: called at the end of a successful Setup when the context already has a stream, so an
    // operation can start moving its plan to the device before Execute.
    virtual void AfterPlanImpl(aclrtStream) {}
    // Enqueue on `stream` with the device pointers of this call.
    virtual Status LaunchImpl(const VariantPack &variantPack, uint8_t *workspace, uint64_t workspaceSize,
                              aclrtStream stream) = 0;
    // The context of the last successful Setup (the one Execute insists on).
    Context *SetupContext() const { return context_; }

private:
    Status CheckVariantPack(const VariantPack &variantPack) const;
    bool CheckIniMatch(const VariantPack &variantPack) const;

    std::string name_;
    std::atomic<bool> setupSuccess_{false};
    Context *context_ = nullptr;
    uint64_t workspaceSize_ = 0;
    uint64_t executeCount_ = 0;   // names the tensor-dump directories (ATB_SAVE_TENSOR_DIR)
    std::vector<TensorDesc> setupInDescs_, setupOutDescs_;
};

void AtbLog(LogLevel level, const std::string &msg);
#define ATB_B200_LOG(level, msg) ::atb::AtbLog(::atb::LogLevel::level, (msg))

bool TensorDescEqual(const TensorDesc &a, const TensorDesc &b);
// rsv[] bytes of a param struct must all be zero (forward-compatibility padding).
bool RsvIsZero(const uint8_t *rsv, size_t n);

} // namespace atb
#endif
