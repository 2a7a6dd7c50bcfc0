// Operator-level C functions of include/atb_b200.h: flat handles around atb::Operation / Context
// for callers that cannot use the C++ classes (ctypes, cgo, JNI ...).
#include <cstring>
#include "../../include/atb_b200.h"
#include "atb/atb_infer.h"
#include "atb_operation_base.h"

namespace {
using namespace atb;

Tensor ToTensor(const atb_b200_tensor &t)
{
    Tensor r;
    r.desc.dtype = static_cast<aclDataType>(t.dtype);
    r.desc.format = static_cast<aclFormat>(t.format);
    r.desc.shape.dimNum = t.dim_num;
    for (int i = 0; i < 8; ++i) {
        r.desc.shape.dims[i] = t.dims[i];
    }
    r.deviceData = t.device_data;
    r.hostData = t.host_data;
    r.dataSize = t.data_size;
    return r;
}

bool ToPack(const atb_b200_tensor *in, uint32_t nIn, const atb_b200_tensor *out, uint32_t nOut, VariantPack &vp)
{
    if ((nIn > 0 && in == nullptr) || (nOut > 0 && out == nullptr) || nIn > MAX_SVECTOR_SIZE || nOut > MAX_SVECTOR_SIZE) {
        return false;
    }
    for (uint32_t i = 0; i < nIn; ++i) {
        vp.inTensors.push_back(ToTensor(in[i]));
    }
    for (uint32_t i = 0; i < nOut; ++i) {
        vp.outTensors.push_back(ToTensor(out[i]));
    }
    return true;
}
} // namespace

extern "C" {

int atb_b200_context_create(void **context)
{
    if (context == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    Context *c = nullptr;
    Status st = CreateContext(&c);
    *context = c;
    return st;
}

int atb_b200_context_set_stream(void *context, void *stream)
{
    if (context == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    return static_cast<Context *>(context)->SetExecuteStream(stream);
}

int atb_b200_context_set_gather(void *context, const atb_b200_pa_peers *peers)
{
    ContextImpl *ci = dynamic_cast<ContextImpl *>(static_cast<Context *>(context));
    if (ci == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (peers != nullptr && (peers->world < 1 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world)) {
        return ERROR_INVALID_PARAM;
    }
    ci->SetGatherPeers(peers);
    return NO_ERROR;
}

int atb_b200_context_destroy(void *context) { return DestroyContext(static_cast<Context *>(context)); }

int atb_b200_operation_create_paged_attention(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::PagedAttentionParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::PagedAttentionParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_reshape_and_cache(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::ReshapeAndCacheParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::ReshapeAndCacheParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_kv_cache(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::KvCacheParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::KvCacheParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_block_copy(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::BlockCopyParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::BlockCopyParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_reshape_and_cache_with_stride(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::ReshapeAndCacheWithStrideParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::ReshapeAndCacheWithStrideParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_multi_latent_attention(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::MultiLatentAttentionParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::MultiLatentAttentionParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_norm_rope_reshape(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::NormRopeReshapeParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::NormRopeReshapeParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_create_paged_cache_load(const void *param, uint64_t param_bytes, void **operation)
{
    if (param == nullptr || operation == nullptr || param_bytes != sizeof(infer::PagedCacheLoadParam)) {
        return ERROR_INVALID_PARAM;
    }
    infer::PagedCacheLoadParam p;
    std::memcpy(&p, param, sizeof(p));
    Operation *op = nullptr;
    Status st = CreateOperation(p, &op);
    *operation = op;
    return st;
}

int atb_b200_operation_input_num(void *operation, uint32_t *n)
{
    if (operation == nullptr || n == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    *n = static_cast<Operation *>(operation)->GetInputNum();
    return NO_ERROR;
}

int atb_b200_operation_output_num(void *operation, uint32_t *n)
{
    if (operation == nullptr || n == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    *n = static_cast<Operation *>(operation)->GetOutputNum();
    return NO_ERROR;
}

int atb_b200_operation_name(void *operation, char *buf, uint64_t cap)
{
    if (operation == nullptr || buf == nullptr || cap == 0) {
        return ERROR_INVALID_PARAM;
    }
    try {
        const std::string name = static_cast<Operation *>(operation)->GetName();
        const uint64_t n = name.size() < cap - 1 ? name.size() : cap - 1;
        std::memcpy(buf, name.data(), n);
        buf[n] = '\0';
    } catch (...) {
        return ERROR_INTERNAL_ERROR;
    }
    return NO_ERROR;
}

int atb_b200_operation_infer_shape(void *operation, const atb_b200_tensor *in, uint32_t n_in, atb_b200_tensor *out,
                                   uint32_t n_out)
{
    if (operation == nullptr || (n_in > 0 && in == nullptr) || out == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    try {
        SVector<TensorDesc> inDescs, outDescs;
        for (uint32_t i = 0; i < n_in; ++i) {
            inDescs.push_back(ToTensor(in[i]).desc);
        }
        Status st = static_cast<Operation *>(operation)->InferShape(inDescs, outDescs);
        if (st != NO_ERROR) {
            return st;
        }
        if (outDescs.size() != n_out) {
            return ERROR_INVALID_PARAM;
        }
        for (uint32_t i = 0; i < n_out; ++i) {
            out[i].dtype = outDescs.at(i).dtype;
            out[i].format = outDescs.at(i).format;
            out[i].dim_num = outDescs.at(i).shape.dimNum;
            for (int k = 0; k < 8; ++k) {
                out[i].dims[k] = outDescs.at(i).shape.dims[k];
            }
        }
        return NO_ERROR;
    } catch (...) {
        return ERROR_INTERNAL_ERROR;
    }
}

int atb_b200_operation_setup(void *operation, const atb_b200_tensor *in, uint32_t n_in, const atb_b200_tensor *out,
                             uint32_t n_out, uint64_t *workspace_bytes, void *context)
{
    if (operation == nullptr || workspace_bytes == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    try {
        VariantPack vp;
        if (!ToPack(in, n_in, out, n_out, vp)) {
            return ERROR_INVALID_PARAM;
        }
        uint64_t ws = 0;
        Status st = static_cast<Operation *>(operation)->Setup(vp, ws, static_cast<Context *>(context));
        *workspace_bytes = ws;
        return st;
    } catch (...) {
        return ERROR_INTERNAL_ERROR;
    }
}

int atb_b200_operation_execute(void *operation, const atb_b200_tensor *in, uint32_t n_in, const atb_b200_tensor *out,
                               uint32_t n_out, void *workspace, uint64_t workspace_bytes, void *context)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    try {
        VariantPack vp;
        if (!ToPack(in, n_in, out, n_out, vp)) {
            return ERROR_INVALID_PARAM;
        }
        return static_cast<Operation *>(operation)->Execute(vp, static_cast<uint8_t *>(workspace), workspace_bytes,
                                                            static_cast<Context *>(context));
    } catch (...) {
        return ERROR_INTERNAL_ERROR;
    }
}

int atb_b200_operation_destroy(void *operation) { return DestroyOperation(static_cast<Operation *>(operation)); }

} // extern "C"
