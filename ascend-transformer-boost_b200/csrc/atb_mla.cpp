// atb::CreateOperation<infer::MultiLatentAttentionParam>: decode attention of DeepSeek-style MLA over the split
// latent cache (query and cache each given as a 512-wide latent tensor and a 64-wide rope tensor), the operator the
// reference's DeepSeek graphs call in decode.  Rules follow
// src/ops/ops_infer/multi_latent_attention/multi_latent_attention_operation.cpp of the reference
// (CreateOperation :58-91, ParamCheck :93-146, ParamRangeCheck :148-170, GetInputNum/GetOutputNum :240-270,
//  InferShapeImpl :272-286, QKVDimCheck :337-379, DimCheck :579-640) and its host-tensor handling
// (multi_latent_attention/param.cpp: contextLens is host data).  Built here: cacheMode KROPE_CTKV with calcType
// UNDEFINED (one query token per sequence), CALC_TYPE_SPEC (several: MTP; no mask, MASK_TYPE_SPEC or MASK_TYPE_MASK_FREE)
// and the _RING forms of both (log-sum-exp as a second output); prefill, the other masks and the NZ / int8 caches are
// rejected.  The device path is the tcgen05 MLA kernel with a
// second tensor map for the rope rows.
#include <cmath>
#include <cstdlib>
#include <new>
#include "../../include/atb_b200.h"
#include "atb_operation_base.h"

namespace atb {
namespace {

using Param = infer::MultiLatentAttentionParam;

class MultiLatentAttentionOperation : public OperationBase {
public:
    explicit MultiLatentAttentionOperation(const Param &p) : OperationBase("MultiLatentAttentionOperation"), param_(p)
    {
        for (aclDataType h : {ACL_FLOAT16, ACL_BF16}) {
            // qNope, qRope, ctKV, kRope, blockTables, contextLens [, mask] [, qSeqLens] -> attnOut [, lse]
            DtypeComb c = {h, h, h, h, ACL_INT32, ACL_INT32};
            if (HasMask()) {
                c.push_back(h);
            }
            if (Spec()) {
                c.push_back(ACL_INT32);
            }
            c.push_back(h);
            if (Ring()) {
                c.push_back(h);
            }
            combs_.push_back(c);
        }
    }
    ~MultiLatentAttentionOperation() override
    {
        if (plan_ != nullptr) {
            atb_b200_pa_plan_destroy(plan_);
        }
    }
    uint32_t GetInputNum() const override { return 6u + (HasMask() ? 1u : 0u) + (Spec() ? 1u : 0u); }
    uint32_t GetOutputNum() const override { return Ring() ? 2 : 1; }

protected:
    // CALC_TYPE_RING: the log-sum-exp of every (token, head) is a second output [tokens, heads, 1]
    bool Ring() const
    {
        return param_.calcType == Param::CALC_TYPE_RING || param_.calcType == Param::CALC_TYPE_SPEC_AND_RING;
    }
    // CALC_TYPE_SPEC: several query tokens per sequence (MTP), qSeqLens as host data after the optional mask
    bool Spec() const
    {
        return param_.calcType == Param::CALC_TYPE_SPEC || param_.calcType == Param::CALC_TYPE_SPEC_AND_RING;
    }
    bool HasMask() const { return param_.maskType != Param::UNDEFINED; }
    size_t MaskPos() const { return 6; }
    size_t QLensPos() const { return 6 + (HasMask() ? 1 : 0); }

    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 3 || in.at(2).shape.dimNum != 4 ||
            in.at(3).shape.dimNum != 4 || in.at(4).shape.dimNum != 2 || in.at(5).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        const Dims &q = in.at(0).shape, &qr = in.at(1).shape, &kv = in.at(2).shape, &kr = in.at(3).shape;
        const int64_t numTokens = q.dims[0], batch = in.at(4).shape.dims[0];
        if (batch > 8192) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: batch should be <= 8192");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (!Spec() && numTokens != batch) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: numTokens and batch should be same in decoder stage");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (Spec()) {
            const Dims &ql = in.at(QLensPos()).shape;
            if (ql.dimNum != 1) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: invalid qSeqlen dimNum");
                return ERROR_INVALID_TENSOR_DIM_NUM;
            }
            if (ql.dims[0] != batch || numTokens < batch) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: dim 0 of qSeqlen should be equal to dim 0 of contextLens");
                return ERROR_INVALID_TENSOR_DIM;
            }
        }
        if (HasMask()) {
            // MASK_TYPE_SPEC: one row per query token [num_tokens, max_seq_len]; MASK_TYPE_MASK_FREE: the reference's
            // fixed causal pattern, any 2-D tensor (its content is implied, it is not read)
            const Dims &m = in.at(MaskPos()).shape;
            if (m.dimNum != 2) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: invalid mask dimNum");
                return ERROR_INVALID_TENSOR_DIM_NUM;
            }
            if (param_.maskType == Param::MASK_TYPE_SPEC && m.dims[0] < numTokens) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: the spec mask should have one row per query token");
                return ERROR_INVALID_TENSOR_DIM;
            }
        }
        if (in.at(5).shape.dims[0] != batch) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: dim 0 of block_tables and contextLens should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kv.dims[1] != 128) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: decoder blockSize should be 128");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (qr.dims[0] != numTokens) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: dim 0 of query and queryRope should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kr.dims[0] != kv.dims[0] || kr.dims[1] != kv.dims[1]) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: dim 0 and dim 1 of kvCache and kvCacheRope should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (kv.dims[2] != param_.kvHeadNum || kr.dims[2] != param_.kvHeadNum) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: dim 2 of kvCache and kvCacheRope should equal kvHeadNum");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (q.dims[1] != param_.headNum || qr.dims[1] != param_.headNum) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: dim 1 of query and queryRope should equal headNum");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (q.dims[2] != 512 || kv.dims[3] != 512) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: head_size of query and kvCache should be 512");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (qr.dims[2] != 64 || kr.dims[3] != 64) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: head_size of queryRope and kvCacheRope should be 64");
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status InferShapeImpl(const SVector<TensorDesc> &in, SVector<TensorDesc> &out) const override
    {
        out.at(0) = in.at(0);
        out.at(0).dtype = in.at(1).dtype;
        if (Ring()) {
            out.at(1) = out.at(0);
            out.at(1).shape.dims[2] = 1;
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
        const Dims &o = outTensors.at(0).desc.shape, &q = descs.at(0).shape;
        if (o.dimNum != 3 || o.dims[0] != q.dims[0] || o.dims[1] != q.dims[1] || o.dims[2] != q.dims[2]) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: attnOut should have the shape of query");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (Ring()) {
            const Dims &l = outTensors.at(1).desc.shape;
            if (l.dimNum != 3 || l.dims[0] != q.dims[0] || l.dims[1] != q.dims[1] || l.dims[2] != 1) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: lse should be [tokens, heads, 1]");
                return ERROR_INVALID_TENSOR_DIM;
            }
        }
        return NO_ERROR;
    }

    Status PlanImpl(const VariantPack &vp, uint64_t &workspaceSize) override
    {
        const Tensor &cl = vp.inTensors.at(5);
        if (cl.hostData == nullptr) {
            ATB_B200_LOG(ERROR, "MultiLatentAttention: contextLens hostData is null");
            return ERROR_INVALID_PARAM;
        }
        const Dims &q = vp.inTensors.at(0).desc.shape, &kv = vp.inTensors.at(2).desc.shape;
        atb_b200_pa_desc d{};
        d.batch = static_cast<int32_t>(q.dims[0]);
        d.num_heads = param_.headNum;
        d.kv_heads = 1;
        d.head_dim_k = 576;
        d.head_dim_v = 512;
        d.v_row_dim = 512;
        d.rope_dim = 64;
        d.block_size = static_cast<int32_t>(kv.dims[1]);
        d.num_blocks = static_cast<int32_t>(kv.dims[0]);
        d.max_blocks_per_seq = static_cast<int32_t>(vp.inTensors.at(4).desc.shape.dims[1]);
        d.q_dtype = vp.inTensors.at(0).desc.dtype == ACL_BF16 ? ATB_B200_BF16 : ATB_B200_FP16;
        d.kv_dtype = d.q_dtype;
        d.qk_scale = param_.qkScale;
        d.kernel = ATB_B200_KERNEL_AUTO;
        d.sm_count = 0; // the current device's SM count; ATB_B200_SM_COUNT overrides (planning without a GPU)
        if (const char *sm = std::getenv("ATB_B200_SM_COUNT")) {
            d.sm_count = std::atoi(sm);
        }
        const int32_t *lens = static_cast<const int32_t *>(cl.hostData);
        const bool specMask = param_.maskType == Param::MASK_TYPE_SPEC;
        if (Spec()) {
            // Every query token becomes a planned row of its own with its sequence's block-table row.  Without a mask
            // it sees the whole context; MASK_FREE is the causal rule (token j of q sees ctx - (q - 1 - j) tokens),
            // expressed through the row's length; MASK_TYPE_SPEC adds the caller's mask row of that token.
            const Tensor &ql = vp.inTensors.at(QLensPos());
            if (ql.hostData == nullptr) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: qSeqlen hostData is null");
                return ERROR_INVALID_PARAM;
            }
            const int32_t *qLens = static_cast<const int32_t *>(ql.hostData);
            const int64_t batch = cl.desc.shape.dims[0];
            const bool causal = param_.maskType == Param::MASK_TYPE_MASK_FREE;
            tokenLens_.clear();
            btRows_.clear();
            maskRows_.clear();
            for (int64_t b = 0; b < batch; ++b) {
                if (qLens[b] < 0 || lens[b] < 0 || (causal && qLens[b] > lens[b])) {
                    ATB_B200_LOG(ERROR, "MultiLatentAttention: qSeqlen should be in [0, contextLens]");
                    return ERROR_INVALID_PARAM;
                }
                for (int32_t j = 0; j < qLens[b]; ++j) {
                    maskRows_.push_back(static_cast<int32_t>(tokenLens_.size()));
                    tokenLens_.push_back(causal ? lens[b] - (qLens[b] - 1 - j) : lens[b]);
                    btRows_.push_back(static_cast<int32_t>(b));
                }
            }
            if (static_cast<int64_t>(tokenLens_.size()) != q.dims[0]) {
                ATB_B200_LOG(ERROR, "MultiLatentAttention: the sum of qSeqlen should equal the query tokens");
                return ERROR_INVALID_PARAM;
            }
            // The same number n of query tokens for every sequence (the usual MTP batch): one planned row per SEQUENCE,
            // the kernel's rows are the n x heads (token, head) pairs and the cache is read once per 64 of them.
            int32_t n = batch > 0 ? qLens[0] : 0;
            for (int64_t b = 1; b < batch; ++b) {
                n = qLens[b] == n ? n : 0;
            }
            // Worth it when the pairs fill the kernel's 64 rows better than the heads alone do (16 or 32 heads per GPU
            // under tensor parallelism); with 64 or 128 heads the per-token plan is as good (measured: 269 vs 280 us
            // on the 128-head benchmark configuration).  The environment can force either form.
            const int64_t H = param_.headNum;
            const bool packs = n > 1 && (n * H + 63) / 64 < n * ((H + 63) / 64);
            const bool fuse = std::getenv("ATB_B200_SPEC_FUSE") != nullptr ||
                              (packs && std::getenv("ATB_B200_SPEC_EXPAND") == nullptr);
            fusedTokens_ = (n > 1 && fuse) ? n : 0;
            if (fusedTokens_ > 1) {
                d.batch = static_cast<int32_t>(batch);
                d.num_heads = n * param_.headNum;
                d.q_per_seq = n;
                d.score_mods = (specMask ? ATB_B200_SCORE_MASK : 0) | (causal ? ATB_B200_SCORE_CAUSAL : 0);
            } else {
                lens = tokenLens_.data();
                d.score_mods = ATB_B200_SCORE_ROWS | (specMask ? ATB_B200_SCORE_MASK : 0);
            }
            if (specMask) {
                const int64_t maskLen = vp.inTensors.at(MaskPos()).desc.shape.dims[1];
                for (int32_t t = 0; t < d.batch; ++t) {
                    if (lens[t] > maskLen) {
                        ATB_B200_LOG(ERROR, "MultiLatentAttention: the mask is shorter than a sequence's context");
                        return ERROR_INVALID_TENSOR_DIM;
                    }
                }
            }
        }
        int rc;
        if (plan_ != nullptr && d.batch == desc_.batch && d.num_blocks == desc_.num_blocks &&
            d.max_blocks_per_seq == desc_.max_blocks_per_seq && d.q_dtype == desc_.q_dtype && d.sm_count == desc_.sm_count &&
            d.score_mods == desc_.score_mods && d.num_heads == desc_.num_heads && d.q_per_seq == desc_.q_per_seq) {
            rc = atb_b200_pa_plan_update(plan_, lens);
        } else {
            if (plan_ != nullptr) {
                atb_b200_pa_plan_destroy(plan_);
                plan_ = nullptr;
            }
            rc = atb_b200_pa_plan_create(&d, lens, &plan_);
            desc_ = d;
        }
        if (rc != 0) {
            return rc;
        }
        if (Spec() && fusedTokens_ <= 1) {
            rc = atb_b200_pa_plan_set_rows(plan_, btRows_.data(), static_cast<int32_t>(cl.desc.shape.dims[0]),
                                           specMask ? maskRows_.data() : nullptr,
                                           specMask ? vp.inTensors.at(MaskPos()).desc.shape.dims[0] : 0);
            if (rc != 0) {
                return rc;
            }
        }
        atb_b200_pa_plan_info info{};
        atb_b200_pa_plan_get_info(plan_, &info);
        workspaceSize = info.workspace_bytes + 256; // room to align the caller's pointer
        return NO_ERROR;
    }

    void AfterPlanImpl(aclrtStream stream) override { (void)atb_b200_pa_plan_prefetch(plan_, stream); }

    Status LaunchImpl(const VariantPack &vp, uint8_t *workspace, uint64_t workspaceSize, aclrtStream stream) override
    {
        atb_b200_pa_tensors t{};
        t.q = vp.inTensors.at(0).deviceData;
        t.q_rope = vp.inTensors.at(1).deviceData;
        t.k_cache = vp.inTensors.at(2).deviceData;
        t.v_cache = t.k_cache;
        t.k_rope_cache = vp.inTensors.at(3).deviceData;
        t.block_tables = static_cast<const int32_t *>(vp.inTensors.at(4).deviceData);
        t.out = vp.outTensors.at(0).deviceData;
        if (Spec() && param_.maskType == Param::MASK_TYPE_SPEC) {
            const Tensor &m = vp.inTensors.at(MaskPos());
            t.mask = m.deviceData;
            // one mask row per query token; planned per sequence, a sequence's rows are fusedTokens_ consecutive ones
            t.mask_batch_stride = m.desc.shape.dims[1] * (fusedTokens_ > 1 ? fusedTokens_ : 1);
            t.mask_q_stride = fusedTokens_ > 1 ? m.desc.shape.dims[1] : 0;
            t.mask_head_stride = 0;
            t.mask_tokens = m.desc.shape.dims[1];
            if (t.mask == nullptr) {
                return ERROR_INVALID_PARAM;
            }
        }
        if (Ring()) {
            t.lse_out = vp.outTensors.at(1).deviceData;
            if (t.lse_out == nullptr) {
                return ERROR_INVALID_PARAM;
            }
        }
        if (t.q == nullptr || t.q_rope == nullptr || t.k_cache == nullptr || t.k_rope_cache == nullptr ||
            t.block_tables == nullptr || t.out == nullptr) {
            return ERROR_INVALID_PARAM;
        }
        uint8_t *ws = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
        const uint64_t usable = workspaceSize - static_cast<uint64_t>(ws - workspace);
        const int rc = atb_b200_pa_launch(plan_, &t, ws, usable, stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    Param param_;
    std::vector<DtypeComb> combs_;
    atb_b200_pa_plan *plan_ = nullptr;
    atb_b200_pa_desc desc_{};
    std::vector<int32_t> tokenLens_, btRows_, maskRows_; // CALC_TYPE_SPEC: one entry per query token
    int32_t fusedTokens_ = 0; // CALC_TYPE_SPEC planned per sequence: query tokens per sequence (else 0)
};

} // namespace

template <> Status CreateOperation(const infer::MultiLatentAttentionParam &opParam, Operation **operation)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (opParam.qkScale <= 0 || opParam.qkScale > 1) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: qkScale should be > 0 and <= 1");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.maskType < Param::UNDEFINED || opParam.maskType > Param::MASK_TYPE_SWA_NORM ||
        opParam.calcType < Param::CALC_TYPE_UNDEFINED || opParam.calcType > Param::CALC_TYPE_PREFILL ||
        opParam.cacheMode > Param::NZCACHE) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: invalid maskType / calcType / cacheMode");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.headNum != 8 && opParam.headNum != 16 && opParam.headNum != 32 && opParam.headNum != 64 &&
        opParam.headNum != 128) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: headNum should be {8,16,32,64,128}");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.kvHeadNum != 1) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: kvHeadNum should be 1, only support MQA");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.cacheMode == Param::KVCACHE) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: dont support cacheMode KVCACHE yet");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.maskUseStatusType < Param::MASK_USE_STATUS_TYPE_UNDEFINED ||
        opParam.maskUseStatusType >= Param::MASK_USE_STATUS_TYPE_MAX) {
        return ERROR_INVALID_PARAM;
    }
    const bool spec = opParam.calcType == Param::CALC_TYPE_SPEC || opParam.calcType == Param::CALC_TYPE_SPEC_AND_RING;
    if (!spec && opParam.maskType != Param::UNDEFINED) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: only mtp(CALC_TYPE_SPEC) support mask");
        return ERROR_INVALID_PARAM;
    }
    if (opParam.calcType == Param::CALC_TYPE_PREFILL || opParam.maskType == Param::MASK_TYPE_CAUSAL_MASK ||
        opParam.maskType == Param::MASK_TYPE_SWA_NORM || opParam.cacheMode != Param::KROPE_CTKV ||
        opParam.maskUseStatusType != Param::MASK_USE_STATUS_TYPE_UNDEFINED) {
        ATB_B200_LOG(ERROR, "MultiLatentAttention: prefill, the CAUSAL_MASK / SWA_NORM masks, maskUseStatus and the NZ / int8 "
                            "caches are not supported by this build");
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "MultiLatentAttentionParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) MultiLatentAttentionOperation(opParam);
    return *operation == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

} // namespace atb
