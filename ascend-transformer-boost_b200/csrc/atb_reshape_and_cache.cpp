// atb::CreateOperation<infer::ReshapeAndCacheParam> and the ReshapeAndCacheOperation behind it.
// Rules follow src/ops/ops_infer/reshape_and_cache/reshape_and_cache_operation.cpp of the reference
// (CreateOperation :43-99, GetInputNum/GetOutputNum :124-145, InferShapeImpl :147-158,
//  SetupCheckImpl :176-215, DimCheck :217-252, DimCheckSISO :254-278, KVCacheDimCheck910B :280-319).
// The fractal-NZ cache layout and the head-compression modes belong to other SoCs and are rejected.
#include <new>
#include "../../include/atb_b200.h"
#include "atb_operation_base.h"

namespace atb {
namespace {

using Param = infer::ReshapeAndCacheParam;

uint64_t ElemSize(aclDataType t) { return t == ACL_INT8 ? 1 : 2; }

class ReshapeAndCacheOperation : public OperationBase {
public:
    explicit ReshapeAndCacheOperation(const Param &p) : OperationBase("ReshapeAndCacheOperation"), param_(p)
    {
        for (aclDataType t : {ACL_FLOAT16, ACL_INT8, ACL_BF16}) {
            if (siso()) {
                combs_.push_back({t, t, ACL_INT32, t});
            } else {
                combs_.push_back({t, t, t, t, ACL_INT32, t, t});
            }
        }
    }
    uint32_t GetInputNum() const override { return siso() ? 3 : 5; }
    uint32_t GetOutputNum() const override { return siso() ? 1 : 2; }

protected:
    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override { return siso() ? DimCheckSiso(in) : DimCheck(in); }

    Status InferShapeImpl(const SVector<TensorDesc> &in, SVector<TensorDesc> &out) const override
    {
        if (siso()) {
            out.at(0) = in.at(1);
        } else {
            out.at(0) = in.at(2);
            out.at(1) = in.at(3);
        }
        return NO_ERROR;
    }

    Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &outTensors) const override
    {
        SVector<TensorDesc> descs;
        for (size_t i = 0; i < inTensors.size(); ++i) {
            descs.push_back(inTensors.at(i).desc);
        }
        Status st = InferShapeCheckImpl(descs);
        if (st != NO_ERROR) {
            return st;
        }
        const size_t kc = siso() ? 1 : 2;
        if (!TensorDescEqual(descs.at(kc), outTensors.at(0).desc) ||
            (!siso() && !TensorDescEqual(descs.at(3), outTensors.at(1).desc))) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: intensor & outtensor descs should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status PlanImpl(const VariantPack &, uint64_t &workspaceSize) override
    {
        workspaceSize = 0;
        return NO_ERROR;
    }

    Status LaunchImpl(const VariantPack &vp, uint8_t *, uint64_t, aclrtStream stream) override
    {
        const Tensor &key = vp.inTensors.at(0);
        const Tensor &keyCache = vp.inTensors.at(siso() ? 1 : 2);
        const Tensor &slots = vp.inTensors.at(siso() ? 2 : 4);
        const Tensor *value = siso() ? nullptr : &vp.inTensors.at(1);
        const Tensor *valueCache = siso() ? nullptr : &vp.inTensors.at(3);
        // outputs alias the cache inputs in every caller; write through the output pointers, which is
        // where the result is expected
        void *kcOut = vp.outTensors.at(0).deviceData;
        void *vcOut = siso() ? nullptr : vp.outTensors.at(1).deviceData;
        if (kcOut != keyCache.deviceData || (!siso() && vcOut != valueCache->deviceData)) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: output caches must alias the input caches (in-place update)");
            return ERROR_INVALID_TENSOR_ADDR;
        }
        const Dims &k = key.desc.shape, &c = keyCache.desc.shape;
        const int64_t es = static_cast<int64_t>(ElemSize(key.desc.dtype));
        const int64_t kRow = k.dims[1] * k.dims[2] * es;
        const int64_t vRow = siso() ? 0 : value->desc.shape.dims[1] * value->desc.shape.dims[2] * es;
        const int64_t numSlots = c.dims[0] * c.dims[1];
        if (key.deviceData == nullptr || kcOut == nullptr || slots.deviceData == nullptr ||
            (!siso() && (value->deviceData == nullptr || vcOut == nullptr))) {
            return ERROR_INVALID_PARAM;
        }
        const int rc = atb_b200_reshape_and_cache(key.deviceData, siso() ? nullptr : value->deviceData, kcOut, vcOut,
                                                  static_cast<const int32_t *>(slots.deviceData),
                                                  static_cast<int32_t>(k.dims[0]), kRow, vRow, numSlots, stream);
        return rc == 0 ? NO_ERROR : ERROR_RT_FAIL;
    }

private:
    bool siso() const { return param_.kvCacheCfg == Param::K_CACHE_V_BYPASS; }

    Status DimCheck(const SVector<TensorDesc> &in) const
    {
        if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 3 || in.at(2).shape.dimNum != 4 ||
            in.at(3).shape.dimNum != 4 || in.at(4).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        const Dims &k = in.at(0).shape, &v = in.at(1).shape, &kc = in.at(2).shape, &vc = in.at(3).shape;
        if (k.dims[0] != v.dims[0] || k.dims[1] != v.dims[1]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: numTokens / numHead of key and value should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kc.dims[0] != vc.dims[0] || kc.dims[1] != vc.dims[1]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: numBlocks / blockSize of the caches should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (k.dims[1] != kc.dims[2] || v.dims[1] != vc.dims[2]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: numHeads should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (k.dims[2] != kc.dims[3] || v.dims[2] != vc.dims[3]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: key/keyCache and value/valueCache headSize should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (in.at(4).shape.dims[0] != k.dims[0]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: slotMapping length should equal numTokens");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status DimCheckSiso(const SVector<TensorDesc> &in) const
    {
        if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 4 || in.at(2).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        const Dims &k = in.at(0).shape, &kc = in.at(1).shape;
        if (k.dims[0] != in.at(2).shape.dims[0] || k.dims[1] != kc.dims[2] || k.dims[2] != kc.dims[3]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCache: key, keyCache and slotMapping dims do not match");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Param param_;
    std::vector<DtypeComb> combs_;
};

} // namespace

template <> Status CreateOperation(const infer::ReshapeAndCacheParam &opParam, Operation **operation)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "ReshapeAndCacheParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.compressType < Param::COMPRESS_TYPE_UNDEFINED || opParam.compressType > Param::COMPRESS_TYPE_KVHEAD_ROPE) {
        ATB_B200_LOG(ERROR, "wrong compress head");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.kvCacheCfg < Param::K_CACHE_V_CACHE || opParam.kvCacheCfg > Param::K_CACHE_V_CACHE_NZ) {
        ATB_B200_LOG(ERROR, "wrong kvcache config");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.compressType != Param::COMPRESS_TYPE_UNDEFINED || opParam.kvCacheCfg == Param::K_CACHE_V_CACHE_NZ) {
        ATB_B200_LOG(ERROR, "ReshapeAndCache: head compression and the NZ cache layout are not supported by this build");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) ReshapeAndCacheOperation(opParam);
    if (*operation == nullptr) {
        return ERROR_OUT_OF_HOST_MEMORY;
    }
    return NO_ERROR;
}

} // namespace atb
