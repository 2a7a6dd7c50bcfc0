// atb::CreateOperation<infer::BlockCopyParam>, <infer::PagedCacheLoadParam> and
// <infer::ReshapeAndCacheWithStrideParam>: the cache-management
// operations next to ReshapeAndCache.  Checks follow the reference:
//   BlockCopy       src/ops/ops_infer/block_copy/block_copy_operation.cpp (CreateOperation :29-46,
//                   GetInputNum/GetOutputNum :58-67, InferShapeCheckImpl :69-95, SetupCheckImpl :105-150)
//   PagedCacheLoad  src/ops/ops_infer/paged_cache_load/paged_cache_load_operation.cpp (CreateOperation :51-77,
//                   GetInputNum :95-102, InferShapeImpl :109-115, SetupCheckImpl :122-146, DimCheck :149-196,
//                   KVCacheDimCheck910BND :252-297)
//   ReshapeAndCacheWithStride  src/ops/ops_infer/reshape_and_cache_with_stride/
//                   reshape_and_cache_with_stride_operation.cpp (CreateOperation :51-88, GetInputNum :115-127,
//                   SetupCheckImpl :164-194, DimCheck :196-232, DimCheckSISO :234-260)
// The fractal-NZ cache layout of PagedCacheLoad and the head-compression modes belong to other hardware
// and are rejected.
#include <new>
#include "../../include/atb_b200.h"
#include "atb_operation_base.h"

namespace atb {
namespace {

uint64_t ElemSize(aclDataType t) { return t == ACL_INT8 ? 1 : 2; }

bool ShapeEqual(const Dims &a, const Dims &b)
{
    if (a.dimNum != b.dimNum) {
        return false;
    }
    for (uint64_t i = 0; i < a.dimNum; ++i) {
        if (a.dims[i] != b.dims[i]) {
            return false;
        }
    }
    return true;
}

// ---------------------------------------------------------------------------------------------------
class BlockCopyOperation : public OperationBase {
public:
    explicit BlockCopyOperation(const infer::BlockCopyParam &p) : OperationBase("BlockCopyOperation"), param_(p)
    {
        for (aclDataType t : {ACL_FLOAT16, ACL_BF16, ACL_INT8}) {
            combs_.push_back({t, t, ACL_INT32, ACL_INT32, ACL_INT32});
        }
    }
    uint32_t GetInputNum() const override { return 5; } // keyCache, valueCache, srcBlockIndices, dstBlockIndices, cumSum
    uint32_t GetOutputNum() const override { return 0; } // the caches are updated in place

protected:
    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        const int64_t blockCount = in.at(0).shape.dims[0];
        if (!ShapeEqual(in.at(0).shape, in.at(1).shape)) {
            ATB_B200_LOG(ERROR, "BlockCopy: kCache shape is not equal vCache shape");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (in.at(0).shape.dimNum != 4) {
            ATB_B200_LOG(ERROR, "BlockCopy: cache shape is not 4");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        if (in.at(2).shape.dimNum != 1 || in.at(3).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "BlockCopy: indices shape is not 1");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        if (!ShapeEqual(in.at(4).shape, in.at(2).shape)) {
            ATB_B200_LOG(ERROR, "BlockCopy: cumSum shape is not equal srcBlockIndices shape");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (in.at(2).shape.dims[0] > blockCount || in.at(3).shape.dims[0] > blockCount) {
            ATB_B200_LOG(ERROR, "BlockCopy: indices shape[0] is greater than blockCount");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status InferShapeImpl(const SVector<TensorDesc> &, SVector<TensorDesc> &) const override { return NO_ERROR; }

    Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &) const override
    {
        SVector<TensorDesc> descs;
        for (size_t i = 0; i < inTensors.size(); ++i) {
            descs.push_back(inTensors.at(i).desc);
        }
        Status st = InferShapeCheckImpl(descs);
        if (st != NO_ERROR) {
            return st;
        }
        if (!TensorDescEqual(descs.at(0), descs.at(1))) {
            ATB_B200_LOG(ERROR, "BlockCopy: kCache desc is not equal vCache desc");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (descs.at(0).format != ACL_FORMAT_ND || descs.at(1).format != ACL_FORMAT_ND) {
            return ERROR_INVALID_TENSOR_FORMAT;
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
        const Tensor &kc = vp.inTensors.at(0), &vc = vp.inTensors.at(1);
        const Tensor &src = vp.inTensors.at(2), &dst = vp.inTensors.at(3), &cum = vp.inTensors.at(4);
        if (kc.deviceData == nullptr || vc.deviceData == nullptr || src.deviceData == nullptr ||
            dst.deviceData == nullptr || cum.deviceData == nullptr) {
            return ERROR_INVALID_PARAM;
        }
        const Dims &s = kc.desc.shape;
        const int64_t blockBytes = s.dims[1] * s.dims[2] * s.dims[3] * static_cast<int64_t>(ElemSize(kc.desc.dtype));
        const int rc = atb_b200_block_copy(kc.deviceData, vc.deviceData, static_cast<const int32_t *>(src.deviceData),
                                           static_cast<const int32_t *>(dst.deviceData),
                                           static_cast<const int32_t *>(cum.deviceData),
                                           static_cast<int32_t>(src.desc.shape.dims[0]),
                                           static_cast<int32_t>(dst.desc.shape.dims[0]), blockBytes, blockBytes, s.dims[0],
                                           stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    infer::BlockCopyParam param_;
    std::vector<DtypeComb> combs_;
};

// ---------------------------------------------------------------------------------------------------
class PagedCacheLoadOperation : public OperationBase {
public:
    using Param = infer::PagedCacheLoadParam;
    explicit PagedCacheLoadOperation(const Param &p) : OperationBase("PagedCacheLoadOperation"), param_(p)
    {
        for (aclDataType t : {ACL_FLOAT16, ACL_BF16, ACL_INT8}) {
            // keyCache, valueCache, blockTables, contextLens, key, value, seqStarts -> key, value
            combs_.push_back({t, t, ACL_INT32, ACL_INT32, t, t, ACL_INT32, t, t});
        }
    }
    uint32_t GetInputNum() const override { return 7; }
    uint32_t GetOutputNum() const override { return 2; }

protected:
    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        if (in.at(0).shape.dimNum != 4 || in.at(1).shape.dimNum != 4 || in.at(2).shape.dimNum != 2 ||
            in.at(3).shape.dimNum != 1 || in.at(4).shape.dimNum != 3 || in.at(5).shape.dimNum != 3 ||
            in.at(6).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        const Dims &kc = in.at(0).shape, &vc = in.at(1).shape;
        if (kc.dims[0] != vc.dims[0]) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: numBlocks should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (in.at(4).shape.dims[0] != in.at(5).shape.dims[0]) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: sumcontextlens should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kc.dims[1] != vc.dims[1]) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: blockSizes should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kc.dims[2] != vc.dims[2]) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: numHeads should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kc.dims[1] == 0) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: blockSize cannot be zero");
            return ERROR_INVALID_TENSOR_DIM;
        }
        const int64_t batch = in.at(2).shape.dims[0];
        if (in.at(3).shape.dims[0] != batch + (param_.isSeqLensCumsumMode ? 1 : 0)) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: the rows of blockTables should match the length of SeqLens");
            return ERROR_INVALID_TENSOR_DIM;
        }
        const int64_t alignK = in.at(0).dtype == ACL_INT8 ? 32 : 16, alignV = in.at(1).dtype == ACL_INT8 ? 32 : 16;
        if (kc.dims[2] * kc.dims[3] % alignK != 0 || vc.dims[2] * vc.dims[3] % alignV != 0) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: num_heads*head_size should be aligned to 16 (fp16/bf16) or 32 (int8)");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (param_.hasSeqStarts && in.at(6).shape.dims[0] != batch) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: the length of seqStarts should match the rows of blockTables");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status InferShapeImpl(const SVector<TensorDesc> &in, SVector<TensorDesc> &out) const override
    {
        out.at(0) = in.at(4);
        out.at(1) = in.at(5);
        return NO_ERROR;
    }

    Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &outTensors) const override
    {
        SVector<TensorDesc> descs;
        for (size_t i = 0; i < inTensors.size(); ++i) {
            descs.push_back(inTensors.at(i).desc);
        }
        const Dims &ok = outTensors.at(0).desc.shape, &ov = outTensors.at(1).desc.shape;
        if (ok.dimNum != 3 || ov.dimNum != 3 || descs.at(0).shape.dimNum != 4 || descs.at(1).shape.dimNum != 4 ||
            ok.dims[1] != descs.at(0).shape.dims[2] || ok.dims[2] != descs.at(0).shape.dims[3] ||
            ov.dims[1] != descs.at(1).shape.dims[2] || ov.dims[2] != descs.at(1).shape.dims[3]) {
            ATB_B200_LOG(ERROR, "PagedCacheLoad: the last dimensions of outTensors need to match the caches");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return InferShapeCheckImpl(descs);
    }

    Status PlanImpl(const VariantPack &vp, uint64_t &workspaceSize) override
    {
        const int32_t batch = static_cast<int32_t>(vp.inTensors.at(2).desc.shape.dims[0]);
        workspaceSize = atb_b200_paged_cache_load_workspace_bytes(batch, param_.isSeqLensCumsumMode ? 1 : 0);
        if (workspaceSize > 0) {
            workspaceSize += 256; // room to align the caller's pointer
        }
        return NO_ERROR;
    }

    Status LaunchImpl(const VariantPack &vp, uint8_t *workspace, uint64_t workspaceSize, aclrtStream stream) override
    {
        const Tensor &kc = vp.inTensors.at(0), &vc = vp.inTensors.at(1), &bt = vp.inTensors.at(2);
        const Tensor &lens = vp.inTensors.at(3), &starts = vp.inTensors.at(6);
        const Tensor &key = vp.outTensors.at(0), &value = vp.outTensors.at(1);
        if (kc.deviceData == nullptr || vc.deviceData == nullptr || bt.deviceData == nullptr ||
            lens.deviceData == nullptr || key.deviceData == nullptr || value.deviceData == nullptr ||
            (param_.hasSeqStarts && starts.deviceData == nullptr)) {
            return ERROR_INVALID_PARAM;
        }
        const Dims &k = kc.desc.shape, &v = vc.desc.shape;
        uint8_t *ws = nullptr;
        uint64_t usable = 0;
        if (workspace != nullptr && workspaceSize >= 256) {
            ws = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
            usable = workspaceSize - static_cast<uint64_t>(ws - workspace);
        }
        const int rc = atb_b200_paged_cache_load(
            kc.deviceData, vc.deviceData, static_cast<const int32_t *>(bt.deviceData),
            static_cast<const int32_t *>(lens.deviceData),
            param_.hasSeqStarts ? static_cast<const int32_t *>(starts.deviceData) : nullptr, key.deviceData,
            value.deviceData, static_cast<int32_t>(bt.desc.shape.dims[0]), static_cast<int32_t>(bt.desc.shape.dims[1]),
            static_cast<int32_t>(k.dims[1]), k.dims[2] * k.dims[3] * static_cast<int64_t>(ElemSize(kc.desc.dtype)),
            v.dims[2] * v.dims[3] * static_cast<int64_t>(ElemSize(vc.desc.dtype)), k.dims[0], key.desc.shape.dims[0],
            param_.isSeqLensCumsumMode ? 1 : 0, ws, usable, stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    Param param_;
    std::vector<DtypeComb> combs_;
};

// ---------------------------------------------------------------------------------------------------
// ReshapeAndCacheWithStride: key (and value) are strided views described by host tensors
// kStrides / vStrides (int64 element strides per dimension) and kOffset / vOffset (int64 element offset
// from the tensor's address).  As in the reference, only the token stride matters: a token's row of
// heads x headSize elements is contiguous, and the KEY's token stride is applied to the value as well
// (tiling/reshape_and_cache_tiling.cpp:64-72, op_kernel/reshape_and_cache_nd.cpp:78-79, 111-112).
class ReshapeAndCacheWithStrideOperation : public OperationBase {
public:
    using Param = infer::ReshapeAndCacheWithStrideParam;
    explicit ReshapeAndCacheWithStrideOperation(const Param &p)
        : OperationBase("ReshapeAndCacheWithStrideOperation"), param_(p)
    {
        for (aclDataType t : {ACL_FLOAT16, ACL_BF16, ACL_INT8}) {
            if (siso()) {
                combs_.push_back({t, t, ACL_INT32, ACL_INT64, ACL_INT64, t});
            } else {
                combs_.push_back({t, t, t, t, ACL_INT32, ACL_INT64, ACL_INT64, ACL_INT64, ACL_INT64, t, t});
            }
        }
    }
    uint32_t GetInputNum() const override { return siso() ? 5 : 9; }
    uint32_t GetOutputNum() const override { return siso() ? 1 : 2; }

protected:
    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        if (siso()) {
            if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 4 || in.at(2).shape.dimNum != 1 ||
                in.at(3).shape.dimNum != 1 || in.at(4).shape.dimNum != 1) {
                ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: invalid intensor dimNum");
                return ERROR_INVALID_TENSOR_DIM_NUM;
            }
            const Dims &k = in.at(0).shape, &kc = in.at(1).shape;
            if (k.dims[0] != in.at(2).shape.dims[0] || k.dims[1] != kc.dims[2] || k.dims[2] != kc.dims[3]) {
                ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: key, keyCache and slotMapping dims do not match");
                return ERROR_INVALID_TENSOR_DIM;
            }
            return NO_ERROR;
        }
        if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 3 || in.at(2).shape.dimNum != 4 ||
            in.at(3).shape.dimNum != 4) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        for (size_t i = 4; i < 9; ++i) {
            if (in.at(i).shape.dimNum != 1) {
                ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: invalid intensor dimNum");
                return ERROR_INVALID_TENSOR_DIM_NUM;
            }
        }
        const Dims &k = in.at(0).shape, &v = in.at(1).shape, &kc = in.at(2).shape, &vc = in.at(3).shape;
        if (k.dims[0] != v.dims[0] || k.dims[1] != v.dims[1]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: numTokens / numHead of key and value should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kc.dims[0] != vc.dims[0] || kc.dims[1] != vc.dims[1]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: numBlocks / blockSize of the caches should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (k.dims[1] != kc.dims[2] || v.dims[1] != vc.dims[2]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: numHeads should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (k.dims[2] != kc.dims[3] || v.dims[2] != vc.dims[3]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: key/keyCache and value/valueCache headSize should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (in.at(4).shape.dims[0] != k.dims[0]) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: slotMapping length should equal numTokens");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

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
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: intensor & outtensor descs should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    // The strides and offsets are host data, read at Setup like contextLens of PagedAttention
    // (reshape_and_cache_with_stride_ops_runner.cpp:79-104 of the reference).
    Status PlanImpl(const VariantPack &vp, uint64_t &workspaceSize) override
    {
        workspaceSize = 0;
        const Tensor &kStrides = vp.inTensors.at(siso() ? 3 : 5);
        const Tensor &kOffset = vp.inTensors.at(siso() ? 4 : 7);
        const Tensor *vOffset = siso() ? nullptr : &vp.inTensors.at(8);
        const Tensor *vStrides = siso() ? nullptr : &vp.inTensors.at(6);
        if (kStrides.hostData == nullptr || kOffset.hostData == nullptr ||
            (!siso() && (vOffset->hostData == nullptr || vStrides->hostData == nullptr))) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: strides / offsets hostData is null");
            return ERROR_INVALID_PARAM;
        }
        if (kStrides.desc.shape.dims[0] < 1 || kOffset.desc.shape.dims[0] < 1 ||
            (!siso() && vOffset->desc.shape.dims[0] < 1)) {
            return ERROR_INVALID_TENSOR_DIM;
        }
        tokenStride_ = static_cast<const int64_t *>(kStrides.hostData)[0];
        kOffset_ = static_cast<const int64_t *>(kOffset.hostData)[0];
        vOffset_ = siso() ? 0 : static_cast<const int64_t *>(vOffset->hostData)[0];
        if (tokenStride_ < 0 || kOffset_ < 0 || vOffset_ < 0) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: strides and offsets must not be negative");
            return ERROR_INVALID_PARAM;
        }
        return NO_ERROR;
    }

    Status LaunchImpl(const VariantPack &vp, uint8_t *, uint64_t, aclrtStream stream) override
    {
        const Tensor &key = vp.inTensors.at(0);
        const Tensor &keyCache = vp.inTensors.at(siso() ? 1 : 2);
        const Tensor &slots = vp.inTensors.at(siso() ? 2 : 4);
        const Tensor *value = siso() ? nullptr : &vp.inTensors.at(1);
        const Tensor *valueCache = siso() ? nullptr : &vp.inTensors.at(3);
        void *kcOut = vp.outTensors.at(0).deviceData;
        void *vcOut = siso() ? nullptr : vp.outTensors.at(1).deviceData;
        if (kcOut != keyCache.deviceData || (!siso() && vcOut != valueCache->deviceData)) {
            ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: the output tensors must alias the cache inputs");
            return ERROR_INVALID_TENSOR_ADDR;
        }
        if (key.deviceData == nullptr || kcOut == nullptr || slots.deviceData == nullptr ||
            (!siso() && (value->deviceData == nullptr || vcOut == nullptr))) {
            return ERROR_INVALID_PARAM;
        }
        const int64_t es = static_cast<int64_t>(ElemSize(key.desc.dtype));
        const Dims &k = key.desc.shape, &kc = keyCache.desc.shape;
        const int64_t kRow = k.dims[1] * k.dims[2] * es;
        const int64_t vRow = siso() ? 0 : value->desc.shape.dims[1] * value->desc.shape.dims[2] * es;
        const uint8_t *kPtr = static_cast<const uint8_t *>(key.deviceData) + kOffset_ * es;
        const uint8_t *vPtr = siso() ? nullptr : static_cast<const uint8_t *>(value->deviceData) + vOffset_ * es;
        const int rc = atb_b200_reshape_and_cache_strided(kPtr, vPtr, kcOut, vcOut,
                                                          static_cast<const int32_t *>(slots.deviceData),
                                                          static_cast<int32_t>(k.dims[0]), kRow, vRow, tokenStride_ * es,
                                                          tokenStride_ * es, kc.dims[0] * kc.dims[1], stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    bool siso() const { return param_.kvCacheCfg == Param::K_CACHE_V_BYPASS; }
    Param param_;
    std::vector<DtypeComb> combs_;
    int64_t tokenStride_ = 0, kOffset_ = 0, vOffset_ = 0; // elements, from the host tensors at Setup
};

// ---------------------------------------------------------------------------------------------------
// NormRopeReshape: RMSNorm of the latent row, RoPE of the rope row, both written into the token's slot of
// the MLA latent cache (src/ops/ops_infer/norm_rope_reshape/norm_rope_reshape_operation.cpp of the
// reference: CreateOperation :35-55, GetInputNum/GetOutputNum :66-74, InferShapeImpl :76-81,
// InferShapeCheckImpl :83-98, SetupCheckImpl :100-113, CheckDim910B :122-135, NormRopeReshapeCheckImpl910B :137-184).
class NormRopeReshapeOperation : public OperationBase {
public:
    using Param = infer::NormRopeReshapeParam;
    explicit NormRopeReshapeOperation(const Param &p) : OperationBase("NormRopeReshapeOperation"), param_(p)
    {
        for (aclDataType t : {ACL_FLOAT16, ACL_BF16}) {
            // x, gamma, keyRope, cos, sin, slotMapping, keyCacheIn -> keyCacheOut
            combs_.push_back({t, t, t, t, t, ACL_INT32, t, t});
        }
    }
    uint32_t GetInputNum() const override { return 7; }
    uint32_t GetOutputNum() const override { return 1; }

protected:
    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 1 || in.at(2).shape.dimNum != 2 ||
            in.at(3).shape.dimNum != 2 || in.at(4).shape.dimNum != 2 || in.at(5).shape.dimNum != 1 ||
            in.at(6).shape.dimNum != 4) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        const Dims &x = in.at(0).shape, &g = in.at(1).shape, &kr = in.at(2).shape, &c = in.at(3).shape;
        const Dims &s = in.at(4).shape, &slots = in.at(5).shape, &kc = in.at(6).shape;
        if (g.dims[0] != x.dims[2]) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: gamma should have as many elements as a row of x");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (x.dims[0] != kr.dims[0] || x.dims[0] != c.dims[0] || x.dims[0] != s.dims[0] || x.dims[0] != slots.dims[0]) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: x, keyRope, cos, sin and slotMapping should have one row per token");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kr.dims[1] != c.dims[1] || kr.dims[1] != s.dims[1]) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: keyRope, cos and sin should have the same width");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kc.dims[3] != x.dims[2] + kr.dims[1]) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: the cache row should be as wide as x plus keyRope");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (x.dims[2] % 16 != 0) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: the last dimension of x should be a multiple of 16");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (x.dims[1] != 1 || kc.dims[2] != 1 || kr.dims[1] % 2 != 0) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: one latent head per token and an even rope width are required");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status InferShapeImpl(const SVector<TensorDesc> &in, SVector<TensorDesc> &out) const override
    {
        out.at(0) = in.at(6);
        return NO_ERROR;
    }

    Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &outTensors) const override
    {
        SVector<TensorDesc> descs;
        for (size_t i = 0; i < inTensors.size(); ++i) {
            descs.push_back(inTensors.at(i).desc);
        }
        const TensorDesc &o = outTensors.at(0).desc;
        if (o.dtype != descs.at(6).dtype) {
            return ERROR_INVALID_TENSOR_DTYPE;
        }
        if (o.format != descs.at(6).format) {
            return ERROR_INVALID_TENSOR_FORMAT;
        }
        if (!ShapeEqual(o.shape, descs.at(6).shape)) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: keyCacheOut should have the shape of keyCacheIn");
            return o.shape.dimNum != descs.at(6).shape.dimNum ? ERROR_INVALID_TENSOR_SIZE : ERROR_INVALID_TENSOR_DIM;
        }
        return InferShapeCheckImpl(descs);
    }

    Status PlanImpl(const VariantPack &, uint64_t &workspaceSize) override
    {
        workspaceSize = 0;
        return NO_ERROR;
    }

    Status LaunchImpl(const VariantPack &vp, uint8_t *, uint64_t, aclrtStream stream) override
    {
        const Tensor &cacheIn = vp.inTensors.at(6);
        void *cacheOut = vp.outTensors.at(0).deviceData;
        if (cacheOut != cacheIn.deviceData) {
            ATB_B200_LOG(ERROR, "NormRopeReshape: the output tensor must alias keyCacheIn (only the tokens' slots are written)");
            return ERROR_INVALID_TENSOR_ADDR;
        }
        for (size_t i = 0; i < 6; ++i) {
            if (vp.inTensors.at(i).deviceData == nullptr) {
                return ERROR_INVALID_PARAM;
            }
        }
        if (cacheOut == nullptr) {
            return ERROR_INVALID_PARAM;
        }
        const Dims &x = vp.inTensors.at(0).desc.shape, &kc = cacheIn.desc.shape;
        const int rc = atb_b200_norm_rope_reshape(
            vp.inTensors.at(0).deviceData, vp.inTensors.at(1).deviceData, vp.inTensors.at(2).deviceData,
            vp.inTensors.at(3).deviceData, vp.inTensors.at(4).deviceData,
            static_cast<const int32_t *>(vp.inTensors.at(5).deviceData), cacheOut, static_cast<int32_t>(x.dims[0]),
            static_cast<int32_t>(x.dims[2]), static_cast<int32_t>(vp.inTensors.at(2).desc.shape.dims[1]),
            vp.inTensors.at(0).desc.dtype == ACL_BF16 ? ATB_B200_BF16 : ATB_B200_FP16, param_.epsilon,
            kc.dims[0] * kc.dims[1], stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    Param param_;
    std::vector<DtypeComb> combs_;
};

// ---------------------------------------------------------------------------------------------------
// KvCache: appends the new K (or V) rows of every sequence to a contiguous per-layer cache.  Rules of
// src/ops/ops_infer/kv_cache/kv_cache_operation.cpp:42-141 of the reference (ND layout).
class KvCacheOperation : public OperationBase {
public:
    explicit KvCacheOperation(const infer::KvCacheParam &p) : OperationBase("KvCacheOperation"), param_(p)
    {
        for (aclDataType t : {ACL_FLOAT16, ACL_BF16, ACL_INT8}) {
            combs_.push_back({t, ACL_INT32, t, ACL_INT32, ACL_INT32});
        }
    }
    uint32_t GetInputNum() const override { return 5; } // newKv, layerId, past, tokenOffset, seqLen
    uint32_t GetOutputNum() const override { return 0; } // past is updated in place

protected:
    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status DimCheck(const SVector<TensorDesc> &in, Status dimNumError) const
    {
        if ((in.at(0).shape.dimNum != 2 && in.at(0).shape.dimNum != 4) || in.at(1).shape.dimNum != 1 ||
            in.at(2).shape.dimNum != 4 || in.at(3).shape.dimNum != 1 || in.at(4).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "KvCache: invalid intensor dimNums");
            return dimNumError;
        }
        const Dims &kv = in.at(0).shape, &past = in.at(2).shape;
        const int64_t hiddenSize = past.dims[3];
        if (in.at(2).dtype == ACL_INT8 ? hiddenSize % 32 != 0 : hiddenSize % 16 != 0) {
            ATB_B200_LOG(ERROR, "KvCache: hiddenSize should be a multiple of 16 (int8: 32)");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (hiddenSize != (kv.dimNum == 2 ? kv.dims[1] : kv.dims[2] * kv.dims[3])) {
            ATB_B200_LOG(ERROR, "KvCache: hiddenSizes should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (past.dims[1] != in.at(3).shape.dims[0] || past.dims[1] != in.at(4).shape.dims[0]) {
            ATB_B200_LOG(ERROR, "KvCache: batches should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        return DimCheck(in, ERROR_INVALID_TENSOR_DIM_NUM);
    }

    Status InferShapeImpl(const SVector<TensorDesc> &, SVector<TensorDesc> &) const override { return NO_ERROR; }

    Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &) const override
    {
        SVector<TensorDesc> descs;
        for (size_t i = 0; i < inTensors.size(); ++i) {
            descs.push_back(inTensors.at(i).desc);
        }
        return DimCheck(descs, ERROR_INVALID_TENSOR_DIM); // the reference's Setup reports the dim count this way
    }

    Status PlanImpl(const VariantPack &, uint64_t &workspaceSize) override
    {
        workspaceSize = 0;
        return NO_ERROR;
    }

    Status LaunchImpl(const VariantPack &vp, uint8_t *, uint64_t, aclrtStream stream) override
    {
        const Tensor &kv = vp.inTensors.at(0), &layer = vp.inTensors.at(1), &past = vp.inTensors.at(2);
        const Tensor &off = vp.inTensors.at(3), &len = vp.inTensors.at(4);
        if (kv.deviceData == nullptr || layer.deviceData == nullptr || past.deviceData == nullptr ||
            off.deviceData == nullptr || len.deviceData == nullptr) {
            return ERROR_INVALID_PARAM;
        }
        const Dims &k = kv.desc.shape, &p = past.desc.shape;
        const int64_t tokens = k.dimNum == 2 ? k.dims[0] : k.dims[0] * k.dims[1];
        const int rc = atb_b200_kv_cache(kv.deviceData, static_cast<const int32_t *>(layer.deviceData), past.deviceData,
                                         static_cast<const int32_t *>(off.deviceData),
                                         static_cast<const int32_t *>(len.deviceData), tokens,
                                         static_cast<int32_t>(p.dims[0]), static_cast<int32_t>(p.dims[1]),
                                         static_cast<int32_t>(p.dims[2]),
                                         p.dims[3] * static_cast<int64_t>(ElemSize(past.desc.dtype)), stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    infer::KvCacheParam param_;
    std::vector<DtypeComb> combs_;
};

} // namespace

template <> Status CreateOperation(const infer::KvCacheParam &opParam, Operation **operation)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "KvCacheParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) KvCacheOperation(opParam);
    return *operation == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

template <> Status CreateOperation(const infer::NormRopeReshapeParam &opParam, Operation **operation)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "NormRopeReshapeParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    if (!(opParam.epsilon > 0.f)) {
        ATB_B200_LOG(ERROR, "NormRopeReshape: invalid epsilon, it should be a positive value");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.rotaryCoeff != 2 || opParam.precisionMode != 0) {
        ATB_B200_LOG(ERROR, "NormRopeReshape: only rotaryCoeff 2 and precisionMode 0 are supported");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) NormRopeReshapeOperation(opParam);
    return *operation == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

template <> Status CreateOperation(const infer::ReshapeAndCacheWithStrideParam &opParam, Operation **operation)
{
    using Param = infer::ReshapeAndCacheWithStrideParam;
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStrideParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.compressType < Param::COMPRESS_TYPE_UNDEFINED || opParam.compressType > Param::COMPRESS_TYPE_KVHEAD_ROPE) {
        ATB_B200_LOG(ERROR, "wrong compress head");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.kvCacheCfg < Param::K_CACHE_V_CACHE || opParam.kvCacheCfg > Param::K_CACHE_V_BYPASS) {
        ATB_B200_LOG(ERROR, "wrong kvcache config");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.compressType != Param::COMPRESS_TYPE_UNDEFINED) {
        ATB_B200_LOG(ERROR, "ReshapeAndCacheWithStride: head compression is not supported by this build");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) ReshapeAndCacheWithStrideOperation(opParam);
    return *operation == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

template <> Status CreateOperation(const infer::BlockCopyParam &opParam, Operation **operation)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "BlockCopyParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) BlockCopyOperation(opParam);
    return *operation == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

template <> Status CreateOperation(const infer::PagedCacheLoadParam &opParam, Operation **operation)
{
    using Param = infer::PagedCacheLoadParam;
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "PagedCacheLoadParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.kvCacheCfg < Param::K_CACHE_V_CACHE_NZ || opParam.kvCacheCfg > Param::K_CACHE_V_CACHE_ND) {
        ATB_B200_LOG(ERROR, "wrong kvcache config");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.kvCacheCfg == Param::K_CACHE_V_CACHE_NZ) {
        ATB_B200_LOG(ERROR, "PagedCacheLoad: the NZ cache layout is not supported by this build");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) PagedCacheLoadOperation(opParam);
    return *operation == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

} // namespace atb
