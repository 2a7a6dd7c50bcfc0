// The operator interface: InferShape / Setup (plan + workspace size) / Execute (enqueue on the
// context's stream).  Interface of include/atb/operation.h:34-120 of the reference.
#ifndef ATB_OPERATION_H
#define ATB_OPERATION_H
#include <cstdint>
#include <string>
#include "atb/context.h"
#include "atb/svector.h"
#include "atb/types.h"

namespace atb {
class Operation {
public:
    Operation() = default;
    virtual ~Operation() = default;
    virtual std::string GetName() const = 0;
    virtual Status InferShape(const SVector<TensorDesc> &inTensorDescs, SVector<TensorDesc> &outTensorDescs) const = 0;
    virtual uint32_t GetInputNum() const = 0;
    virtual uint32_t GetOutputNum() const = 0;
    // Reads hostData (e.g. contextLens) and plans the launch; writes the workspace size needed.
    virtual Status Setup(const VariantPack &variantPack, uint64_t &workspaceSize, Context *context) = 0;
    // Enqueues the kernels on the context's stream; completion is the caller's stream sync.
    virtual Status Execute(const VariantPack &variantPack, uint8_t *workspace, uint64_t workspaceSize,
                           Context *context) = 0;
};

// Instantiated for infer::PagedAttentionParam and infer::ReshapeAndCacheParam.
template <typename OpParam> Status CreateOperation(const OpParam &opParam, Operation **operation);
Status DestroyOperation(Operation *operation);
} // namespace atb
#endif
