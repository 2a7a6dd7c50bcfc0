// atb::CreateOperation<infer::PagedAttentionParam> and the PagedAttentionOperation behind it.
// Parameter rules, tensor order and shape checks follow
// src/ops/ops_infer/paged_attention/paged_attention_operation.cpp of the reference
// (CreateOperation :92-143, *ParamCheck :145-365, GetInputNum :408-444, InferShapeImpl :451-472,
//  SetupCheckImpl :492-525, KVCacheDimCheck910B :585-632, SetupDimCheck :926-963).  Built: NORM / ALIBI / SPEC
// masks, batchRunStatus, parallel decoding (CALC_TYPE_SPEC), logN scaling, qScale, the BNSD cache layout,
// int8 caches with per-channel dequantisation, int8 Q / K / V (TYPE_QUANT_QKV_ONLINE / OFFLINE, without a mask).
// Head compression, MASK_TYPE_MASK_FREE and the NZ layouts
// (other SoC classes) are rejected at CreateOperation with ERROR_INVALID_PARAM.
#include <cmath>
#include <cstdlib>
#include <new>
#include <vector>
#include "../../include/atb_b200.h"
#include "atb_operation_base.h"

namespace atb {
namespace {

using Param = infer::PagedAttentionParam;

bool ParamCheck(const Param &p)
{
    if (p.headNum <= 0) {
        ATB_B200_LOG(ERROR, "headNum should be greater than zero");
        return false;
    }
    if (p.kvHeadNum < 0) {
        ATB_B200_LOG(ERROR, "kvHeadNum should be no less than zero");
        return false;
    }
    if (p.kvHeadNum != 0 && p.headNum % p.kvHeadNum != 0) {
        ATB_B200_LOG(ERROR, "headNum mod kvHeadNum should be zero");
        return false;
    }
    if (p.compressType >= Param::COMPRESS_TYPE_MAX || p.compressType < Param::COMPRESS_TYPE_UNDEFINED ||
        p.scaleType >= Param::SCALE_TYPE_MAX || p.scaleType < Param::SCALE_TYPE_TOR) {
        ATB_B200_LOG(ERROR, "enum parameter out of range");
        return false;
    }
    if (p.quantType == Param::TYPE_DEQUANT_FUSION && p.calcType != Param::CALC_TYPE_UNDEFINED) {
        ATB_B200_LOG(ERROR, "dequant only supports calcType CALC_TYPE_UNDEFINED");
        return false;
    }
    if (p.mlaVHeadSize > 0) {
        if (p.maskType == Param::MASK_TYPE_ALIBI || p.compressType != Param::COMPRESS_TYPE_UNDEFINED ||
            p.quantType == Param::TYPE_DEQUANT_FUSION || p.scaleType != Param::SCALE_TYPE_TOR ||
            p.inputLayout != infer::TYPE_BSND) {
            ATB_B200_LOG(ERROR, "mla mode does not support alibi, compress, dequant_fusion, logN or BNSD");
            return false;
        }
        if (p.kvHeadNum != 1) {
            ATB_B200_LOG(ERROR, "kvHeadNum should be 1, mla mode only supports MQA");
            return false;
        }
        if (p.mlaVHeadSize > 576) {
            ATB_B200_LOG(ERROR, "mlaVHeadSize should be no greater than 576");
            return false;
        }
    }
    if (p.scaleType == Param::SCALE_TYPE_LOGN &&
        (p.quantType != Param::TYPE_QUANT_UNQUANT || p.calcType != Param::CALC_TYPE_UNDEFINED ||
         p.compressType != Param::COMPRESS_TYPE_UNDEFINED)) {
        ATB_B200_LOG(ERROR, "logN func does not support quant, calcType or compressType features");
        return false;
    }
    if (p.inputLayout == infer::TYPE_BNSD &&
        (p.calcType != Param::CALC_TYPE_UNDEFINED || p.compressType != Param::COMPRESS_TYPE_UNDEFINED ||
         p.quantType != Param::TYPE_QUANT_UNQUANT || p.scaleType != Param::SCALE_TYPE_TOR)) {
        ATB_B200_LOG(ERROR, "BNSD feature cannot coexist with calcType, compressType, quantType or scaleType features");
        return false;
    }
    if (p.inputLayout != infer::TYPE_BSND && p.inputLayout != infer::TYPE_BNSD) {
        ATB_B200_LOG(ERROR, "inputLayout should be TYPE_BSND or TYPE_BNSD");
        return false;
    }
    if (p.calcType != Param::CALC_TYPE_UNDEFINED && p.calcType != Param::CALC_TYPE_SPEC) {
        ATB_B200_LOG(ERROR, "calcType should be in the range of its enum value");
        return false;
    }
    if (p.calcType == Param::CALC_TYPE_SPEC) {
        if (p.batchRunStatusEnable) {
            ATB_B200_LOG(ERROR, "SPEC func does not support dynamic batch");
            return false;
        }
        if (p.mlaVHeadSize == 0 && p.maskType != Param::MASK_TYPE_NORM && p.maskType != Param::MASK_TYPE_SPEC) {
            ATB_B200_LOG(ERROR, "SPEC func only support norm mask and spec mask");
            return false;
        }
        if (p.mlaVHeadSize > 0) {
            ATB_B200_LOG(ERROR, "PagedAttention: parallel decoding over the MLA cache is not supported by this build");
            return false;
        }
    } else if (p.maskType == Param::MASK_TYPE_SPEC) {
        ATB_B200_LOG(ERROR, "MASK_TYPE_SPEC needs calcType CALC_TYPE_SPEC");
        return false;
    }
    const bool qkvQuant = p.quantType == Param::TYPE_QUANT_QKV_OFFLINE || p.quantType == Param::TYPE_QUANT_QKV_ONLINE;
    if (qkvQuant) {
        // QuantParamCheck of the reference (paged_attention_operation.cpp:249-276)
        if (p.outDataType != ACL_FLOAT16 && p.outDataType != ACL_BF16) {
            ATB_B200_LOG(ERROR, "outDataType only support ACL_FLOAT16 and ACL_BF16");
            return false;
        }
        if (p.hasQuantOffset) {
            ATB_B200_LOG(ERROR, "QKVQuant only support when hasQuantOffset is False");
            return false;
        }
        if (p.calcType != Param::CALC_TYPE_UNDEFINED) {
            ATB_B200_LOG(ERROR, "QKVQuant only support when calcType is CALC_TYPE_UNDEFINED");
            return false;
        }
        if (p.maskType != Param::UNDEFINED || p.batchRunStatusEnable || p.mlaVHeadSize > 0 ||
            p.inputLayout != infer::TYPE_BSND) {
            ATB_B200_LOG(ERROR, "PagedAttention: QKVQuant with a mask, batchRunStatus, mla or BNSD is not supported by "
                                "this build");
            return false;
        }
    }
    // Features outside the decode path of this build.
    if ((p.maskType != Param::UNDEFINED && p.maskType != Param::MASK_TYPE_NORM && p.maskType != Param::MASK_TYPE_ALIBI &&
         p.maskType != Param::MASK_TYPE_SPEC) ||
        p.compressType != Param::COMPRESS_TYPE_UNDEFINED ||
        (p.quantType != Param::TYPE_QUANT_UNQUANT && p.quantType != Param::TYPE_DEQUANT_FUSION && !qkvQuant)) {
        ATB_B200_LOG(ERROR, "PagedAttention: MASK_FREE / NORM_COMPRESS masks and compress are not supported by this build");
        return false;
    }
    return true;
}

int ToKernelDtype(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT16:
            return ATB_B200_FP16;
        case ACL_BF16:
            return ATB_B200_BF16;
        case ACL_INT8:
            return ATB_B200_INT8;
        default:
            return -1;
    }
}

class PagedAttentionOperation : public OperationBase {
public:
    explicit PagedAttentionOperation(const Param &p) : OperationBase("PagedAttentionOperation"), param_(p)
    {
        const bool mla = p.mlaVHeadSize > 0;
        const aclDataType halfs[2] = {ACL_FLOAT16, ACL_BF16};
        for (aclDataType h : halfs) {
            if (QkvQuant()) {
                // int8 query and caches, fp32 scales per head, output of the type the param names
                if (h != p.outDataType) {
                    continue;
                }
                DtypeComb c = {ACL_INT8, ACL_INT8, ACL_INT8, ACL_INT32, ACL_INT32, ACL_FLOAT, ACL_FLOAT};
                if (p.quantType == Param::TYPE_QUANT_QKV_OFFLINE) {
                    c.push_back(ACL_FLOAT); // pScale
                }
                c.push_back(h);
                combs_.push_back(c);
            } else if (p.quantType == Param::TYPE_DEQUANT_FUSION) {
                // descale tensors: fp32, the int64-packed fp32 encoding, or (extension) fp16
                for (aclDataType sc : {ACL_FLOAT, ACL_INT64, ACL_FLOAT16}) {
                    DtypeComb c = {h, ACL_INT8, ACL_INT8, ACL_INT32, ACL_INT32};
                    if (p.maskType != Param::UNDEFINED) {
                        c.push_back(h);
                    }
                    if (p.batchRunStatusEnable) {
                        c.push_back(ACL_INT32);
                    }
                    c.push_back(sc);
                    if (p.hasQuantOffset) {
                        c.push_back(ACL_INT32);
                    }
                    c.push_back(sc);
                    if (p.hasQuantOffset) {
                        c.push_back(ACL_INT32);
                    }
                    c.push_back(h);
                    combs_.push_back(c);
                }
            } else {
                DtypeComb c = {h, h};
                if (!mla) {
                    c.push_back(h);
                }
                c.push_back(ACL_INT32);
                c.push_back(ACL_INT32);
                if (p.maskType != Param::UNDEFINED) {
                    c.push_back(h);
                }
                if (p.batchRunStatusEnable) {
                    c.push_back(ACL_INT32);
                }
                if (p.calcType == Param::CALC_TYPE_SPEC) {
                    c.push_back(ACL_INT32); // qSeqLens
                }
                if (p.scaleType == Param::SCALE_TYPE_LOGN) {
                    c.push_back(ACL_FLOAT);
                }
                c.push_back(h);
                combs_.push_back(c);
            }
        }
    }
    ~PagedAttentionOperation() override
    {
        if (plan_ != nullptr) {
            atb_b200_pa_plan_destroy(plan_);
        }
        for (void *p : scratch_) {
            FreeDevice(p);
        }
    }

    uint32_t GetInputNum() const override
    {
        uint32_t n = 5; // query, keyCache, valueCache, blockTables, contextLens
        if (param_.maskType != Param::UNDEFINED) {
            n += 1; // mask
        }
        if (param_.scaleType == Param::SCALE_TYPE_LOGN) {
            n += 1; // logN, always the last input
        }
        if (param_.calcType == Param::CALC_TYPE_SPEC) {
            n += 1; // qSeqLens
        }
        if (param_.batchRunStatusEnable) {
            n += 1; // batchRunStatus
        }
        if (param_.quantType == Param::TYPE_DEQUANT_FUSION) {
            n += param_.hasQuantOffset ? 4 : 2;
        }
        if (QkvQuant()) {
            n += param_.quantType == Param::TYPE_QUANT_QKV_OFFLINE ? 3 : 2; // kDescale, vDescale, [pScale]
        }
        if (param_.mlaVHeadSize > 0) {
            n -= 1; // no valueCache
        }
        return n;
    }
    uint32_t GetOutputNum() const override { return 1; }

protected:
    // optional inputs follow contextLens in the reference's order: mask, batchRunStatus, kDescale ..., logN (last)
    bool HasMask() const { return param_.maskType != Param::UNDEFINED; }
    bool QkvQuant() const
    {
        return param_.quantType == Param::TYPE_QUANT_QKV_OFFLINE || param_.quantType == Param::TYPE_QUANT_QKV_ONLINE;
    }
    size_t ClPos() const { return param_.mlaVHeadSize > 0 ? 3 : 4; }
    size_t MaskPos() const { return ClPos() + 1; }
    size_t StatusPos() const { return ClPos() + 1 + (HasMask() ? 1 : 0); }
    size_t ScalePos() const { return StatusPos() + (param_.batchRunStatusEnable ? 1 : 0); }
    bool Spec() const { return param_.calcType == Param::CALC_TYPE_SPEC; }
    // qSeqLens follows the quantisation tensors (none of which exist together with SPEC in this build)
    size_t QLensPos() const { return ScalePos(); }

    // The mask shapes of the reference's documentation for this SoC class: plain [batch, 1, tokens] or [1, tokens];
    // alibi [batch, heads, 1, tokens] or [heads, 1, tokens].  Fills the element strides the kernels index with.
    Status MaskLayout(const Dims &m, int64_t qTokens, int64_t *batchStride, int64_t *headStride, int64_t *tokens) const
    {
        const int64_t len = m.dims[m.dimNum - 1];
        *tokens = len;
        if (Spec()) {
            // parallel decoding: MASK_TYPE_SPEC [num_tokens, max_seq_len], one row per query token; MASK_TYPE_NORM the
            // square causal mask [max_seq_len, max_seq_len], a token reads row contextLen - qSeqLen + j
            *headStride = 0;
            *batchStride = len;
            const bool ok = m.dimNum == 2 && (param_.maskType == Param::MASK_TYPE_SPEC ? m.dims[0] >= qTokens : m.dims[0] == len);
            if (!ok) {
                ATB_B200_LOG(ERROR, "PagedAttention: with CALC_TYPE_SPEC the mask should be [num_tokens, max_seq_len] "
                                    "(spec mask) or [max_seq_len, max_seq_len] (norm mask)");
                return m.dimNum == 2 ? ERROR_INVALID_TENSOR_DIM : ERROR_INVALID_TENSOR_DIM_NUM;
            }
            return NO_ERROR;
        }
        if (param_.maskType == Param::MASK_TYPE_NORM) {
            *headStride = 0;
            if (m.dimNum == 3 && m.dims[1] == 1 && m.dims[0] >= qTokens) {
                *batchStride = len;
                return NO_ERROR;
            }
            if (m.dimNum == 2 && m.dims[0] == 1) {
                *batchStride = 0;
                return NO_ERROR;
            }
            ATB_B200_LOG(ERROR, "PagedAttention: norm mask should be [batch, 1, max_seq_len] or [1, max_seq_len]");
            return m.dimNum == 2 || m.dimNum == 3 ? ERROR_INVALID_TENSOR_DIM : ERROR_INVALID_TENSOR_DIM_NUM;
        }
        *headStride = len;
        if (m.dimNum == 4 && m.dims[1] == param_.headNum && m.dims[2] == 1 && m.dims[0] >= qTokens) {
            *batchStride = static_cast<int64_t>(param_.headNum) * len;
            return NO_ERROR;
        }
        if (m.dimNum == 3 && m.dims[0] == param_.headNum && m.dims[1] == 1) {
            *batchStride = 0;
            return NO_ERROR;
        }
        ATB_B200_LOG(ERROR, "PagedAttention: alibi mask should be [batch, head_num, 1, max_seq_len] or "
                            "[head_num, 1, max_seq_len]");
        return m.dimNum == 3 || m.dimNum == 4 ? ERROR_INVALID_TENSOR_DIM : ERROR_INVALID_TENSOR_DIM_NUM;
    }

    const std::vector<DtypeComb> &DtypeCombs() const override { return combs_; }

    Status InferShapeCheckImpl(const SVector<TensorDesc> &in) const override
    {
        const bool mla = param_.mlaVHeadSize > 0;
        const size_t btPos = mla ? 2 : 3, clPos = mla ? 3 : 4;
        if (!mla && in.at(2).shape.dimNum != 4) {
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        if (in.at(0).shape.dimNum != 3 || in.at(1).shape.dimNum != 4 || in.at(btPos).shape.dimNum != 2 ||
            in.at(clPos).shape.dimNum != 1) {
            ATB_B200_LOG(ERROR, "PagedAttention: invalid intensor dimNum");
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        const Dims &q = in.at(0).shape, &k = in.at(1).shape;
        if (q.dims[1] != param_.headNum) {
            ATB_B200_LOG(ERROR, "PagedAttention: query dim 1 should equal headNum");
            return ERROR_INVALID_TENSOR_DIM;
        }
        const int64_t kvHeads = param_.kvHeadNum == 0 ? param_.headNum : param_.kvHeadNum;
        // TYPE_BNSD: cache blocks are [kv_heads, block_size, head_size] instead of [block_size, kv_heads, head_size]
        const bool bnsd = param_.inputLayout == infer::TYPE_BNSD;
        const int hDim = bnsd ? 1 : 2, sDim = bnsd ? 2 : 1;
        if (k.dims[hDim] != kvHeads) {
            ATB_B200_LOG(ERROR, "PagedAttention: the head dim of keyCache should equal kvHeadNum");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (HasMask()) {
            int64_t bs = 0, hs = 0, len = 0;
            const Status st = MaskLayout(in.at(MaskPos()).shape, q.dims[0], &bs, &hs, &len);
            if (st != NO_ERROR) {
                return st;
            }
        }
        if (param_.scaleType == Param::SCALE_TYPE_LOGN) {
            const Dims &ln = in.at(in.size() - 1).shape;
            if (ln.dimNum != 1) {
                ATB_B200_LOG(ERROR, "PagedAttention: invalid logN intensor dimNum");
                return ERROR_INVALID_TENSOR_DIM_NUM;
            }
            if (ln.dims[0] != in.at(clPos).shape.dims[0]) {
                ATB_B200_LOG(ERROR, "PagedAttention: intensor contextLens and intensor logn has different batch size");
                return ERROR_INVALID_TENSOR_DIM;
            }
        }
        if (param_.batchRunStatusEnable) {
            // dynamic batch: the control tensors may describe more sequences than there are query tokens
            if (q.dims[0] > in.at(btPos).shape.dims[0] || q.dims[0] > in.at(clPos).shape.dims[0]) {
                ATB_B200_LOG(ERROR, "PagedAttention: numTokens in q should be no greater than blockTables and contextLens");
                return ERROR_INVALID_TENSOR_DIM;
            }
            if (in.at(StatusPos()).shape.dimNum != 1 || in.at(StatusPos()).shape.dims[0] < q.dims[0]) {
                ATB_B200_LOG(ERROR, "PagedAttention: batchRunStatus should hold one value per query token");
                return ERROR_INVALID_TENSOR_DIM;
            }
        } else if (Spec()) {
            // several query tokens per sequence: the control tensors have one row per sequence
            const int64_t batch = in.at(clPos).shape.dims[0];
            const Dims &ql = in.at(QLensPos()).shape;
            if (ql.dimNum != 1 || ql.dims[0] != batch || in.at(btPos).shape.dims[0] != batch || q.dims[0] < batch) {
                ATB_B200_LOG(ERROR, "PagedAttention: blockTables, contextLens and qSeqLens should have one row per "
                                    "sequence, and the query at least one token per sequence");
                return ERROR_INVALID_TENSOR_DIM;
            }
            if (k.dims[sDim] > 128) {
                ATB_B200_LOG(ERROR, "PagedAttention: blockSize should be no greater than 128 with CALC_TYPE_SPEC");
                return ERROR_INVALID_TENSOR_DIM;
            }
        } else if (in.at(btPos).shape.dims[0] != q.dims[0] || in.at(clPos).shape.dims[0] != q.dims[0]) {
            ATB_B200_LOG(ERROR, "PagedAttention: blockTables / contextLens rows should equal query tokens");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (!mla) {
            const Dims &v = in.at(2).shape;
            if (k.dims[0] != v.dims[0] || k.dims[1] != v.dims[1] || k.dims[2] != v.dims[2]) {
                ATB_B200_LOG(ERROR, "PagedAttention: keyCache and valueCache block dims should be the same");
                return ERROR_INVALID_TENSOR_DIM;
            }
        }
        const int64_t headSize = k.dims[3], blockSize = k.dims[sDim];
        if (headSize != q.dims[2]) {
            ATB_B200_LOG(ERROR, "PagedAttention: headSize of keyCache and query should be same");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (QkvQuant()) {
            if (headSize != in.at(2).shape.dims[3] || headSize > 256 || headSize * blockSize > 128 * 128) {
                ATB_B200_LOG(ERROR, "PagedAttention: QKVQuant needs equal head sizes <= 256 and block_size * head_size <= 128*128");
                return ERROR_INVALID_TENSOR_DIM;
            }
            const size_t n = param_.quantType == Param::TYPE_QUANT_QKV_OFFLINE ? 3u : 2u;
            for (size_t i = ScalePos(); i < ScalePos() + n; ++i) {
                if (in.at(i).shape.dimNum != 1 || in.at(i).shape.dims[0] != param_.headNum) {
                    ATB_B200_LOG(ERROR, "PagedAttention: QKVQuant scales should have headNum elements");
                    return ERROR_INVALID_TENSOR_DIM;
                }
            }
        } else if (param_.quantType == Param::TYPE_DEQUANT_FUSION) {
            if (headSize != in.at(2).shape.dims[3]) {
                return ERROR_INVALID_TENSOR_DIM;
            }
            if (headSize > 256 || headSize * blockSize > 128 * 128) {
                ATB_B200_LOG(ERROR, "PagedAttention: head_size <= 256 and block_size * head_size <= 128*128 required");
                return ERROR_INVALID_TENSOR_DIM;
            }
            const int64_t want = kvHeads * headSize;
            for (size_t i = ScalePos(); i < ScalePos() + (param_.hasQuantOffset ? 4u : 2u); ++i) {
                if (in.at(i).shape.dimNum != 1 || in.at(i).shape.dims[0] != want) {
                    ATB_B200_LOG(ERROR, "PagedAttention: descale / offset should have kvHeadNum*headSize elements");
                    return ERROR_INVALID_TENSOR_DIM;
                }
            }
        } else {
            if (param_.mlaVHeadSize > headSize) {
                ATB_B200_LOG(ERROR, "PagedAttention: mlaVHeadSize should be no greater than headSizeK");
                return ERROR_INVALID_TENSOR_DIM;
            }
            const int64_t headSizeV = mla ? param_.mlaVHeadSize : in.at(2).shape.dims[3];
            if (headSize > 576 || headSizeV > 576) {
                return ERROR_INVALID_TENSOR_DIM;
            }
            if (mla && q.dims[0] > 8192) {
                return ERROR_INVALID_TENSOR_DIM;
            }
            if ((headSize > 256 || headSizeV > 256) && blockSize > 128) {
                return ERROR_INVALID_TENSOR_DIM;
            }
            if (headSize % 4 != 0 || headSizeV % 4 != 0) {
                ATB_B200_LOG(ERROR, "PagedAttention: head sizes must be multiples of 4");
                return ERROR_INVALID_TENSOR_DIM;
            }
        }
        return NO_ERROR;
    }

    Status InferShapeImpl(const SVector<TensorDesc> &in, SVector<TensorDesc> &out) const override
    {
        out.at(0) = in.at(0);
        out.at(0).shape.dims[2] = param_.mlaVHeadSize > 0 ? param_.mlaVHeadSize : in.at(2).shape.dims[3];
        if (QkvQuant()) {
            out.at(0).dtype = param_.outDataType; // the query is int8 here
        }
        return NO_ERROR;
    }

    Status SetupCheckImpl(const SVector<Tensor> &inTensors, const SVector<Tensor> &outTensors) const override
    {
        if (inTensors.at(1).desc.shape.dimNum != 4) {
            return ERROR_INVALID_TENSOR_DIM_NUM;
        }
        SVector<TensorDesc> descs;
        for (size_t i = 0; i < inTensors.size(); ++i) {
            descs.push_back(inTensors.at(i).desc);
        }
        Status st = InferShapeCheckImpl(descs);
        if (st != NO_ERROR) {
            return st;
        }
        const Dims &o = outTensors.at(0).desc.shape, &q = inTensors.at(0).desc.shape;
        const int64_t dv = param_.mlaVHeadSize > 0 ? param_.mlaVHeadSize : inTensors.at(2).desc.shape.dims[3];
        if (o.dimNum != 3 || o.dims[2] != dv) {
            ATB_B200_LOG(ERROR, "PagedAttention: headSize of attnOut error");
            return ERROR_INVALID_TENSOR_DIM;
        }
        if (o.dims[0] != q.dims[0] || o.dims[1] != q.dims[1]) {
            return ERROR_INVALID_TENSOR_DIM;
        }
        return NO_ERROR;
    }

    Status PlanImpl(const VariantPack &vp, uint64_t &workspaceSize) override
    {
        const bool mla = param_.mlaVHeadSize > 0;
        const size_t btPos = mla ? 2 : 3, clPos = mla ? 3 : 4;
        const Tensor &cl = vp.inTensors.at(clPos);
        if (cl.hostData == nullptr) {
            ATB_B200_LOG(ERROR, "PagedAttention: contextLens hostData is null");
            return ERROR_INVALID_PARAM;
        }
        const Dims &q = vp.inTensors.at(0).desc.shape, &k = vp.inTensors.at(1).desc.shape;
        atb_b200_pa_desc d{};
        d.batch = static_cast<int32_t>(q.dims[0]);
        d.num_heads = param_.headNum;
        d.kv_heads = param_.kvHeadNum == 0 ? param_.headNum : param_.kvHeadNum;
        d.head_dim_k = static_cast<int32_t>(k.dims[3]);
        d.head_dim_v = mla ? static_cast<int32_t>(param_.mlaVHeadSize)
                           : static_cast<int32_t>(vp.inTensors.at(2).desc.shape.dims[3]);
        d.v_row_dim = mla ? d.head_dim_k : d.head_dim_v;
        d.kv_layout = param_.inputLayout == infer::TYPE_BNSD ? ATB_B200_KV_BNSD : ATB_B200_KV_BSND;
        d.block_size = static_cast<int32_t>(k.dims[d.kv_layout == ATB_B200_KV_BNSD ? 2 : 1]);
        d.num_blocks = static_cast<int32_t>(k.dims[0]);
        d.max_blocks_per_seq = static_cast<int32_t>(vp.inTensors.at(btPos).desc.shape.dims[1]);
        d.q_dtype = ToKernelDtype(vp.inTensors.at(0).desc.dtype);
        d.kv_dtype = ToKernelDtype(vp.inTensors.at(1).desc.dtype);
        float scale = param_.qkScale;
        if (std::fabs(param_.qScale) > 1e-6f && std::fabs(param_.qScale - 1.f) > 1e-6f) {
            scale *= param_.qScale; // the reference multiplies Q by qScale in a separate node
        }
        d.qk_scale = scale;
        if (QkvQuant()) {
            d.qkv_quant = param_.quantType == Param::TYPE_QUANT_QKV_OFFLINE ? ATB_B200_QUANT_OFFLINE : ATB_B200_QUANT_ONLINE;
            d.out_dtype = ToKernelDtype(param_.outDataType);
        }
        d.kernel = ATB_B200_KERNEL_AUTO;
        if (const char *force = std::getenv("ATB_B200_FORCE_KERNEL")) {
            d.kernel = std::atoi(force);
        }
        d.sm_count = 0; // the current device's SM count; ATB_B200_SM_COUNT overrides (planning without a GPU)
        if (const char *sm = std::getenv("ATB_B200_SM_COUNT")) {
            d.sm_count = std::atoi(sm);
        }
        d.score_mods = (HasMask() ? ATB_B200_SCORE_MASK : 0) |
                       (param_.scaleType == Param::SCALE_TYPE_LOGN ? ATB_B200_SCORE_LOGN : 0) |
                       (Spec() ? ATB_B200_SCORE_ROWS : 0);
        const int32_t *lens = static_cast<const int32_t *>(cl.hostData);
        if (Spec()) {
            // Parallel decoding: every query token becomes a planned row of its own, with its sequence's length and
            // block-table row (qSeqLens is host data: src/ops/ops_infer/paged_attention/param.cpp of the reference).
            const Tensor &ql = vp.inTensors.at(QLensPos());
            if (ql.hostData == nullptr) {
                ATB_B200_LOG(ERROR, "PagedAttention: qSeqLens hostData is null");
                return ERROR_INVALID_PARAM;
            }
            const int32_t *qLens = static_cast<const int32_t *>(ql.hostData);
            const int64_t batch = cl.desc.shape.dims[0];
            const bool normMask = param_.maskType == Param::MASK_TYPE_NORM;
            effectiveLens_.clear();
            btRows_.clear();
            maskRows_.clear();
            for (int64_t b = 0; b < batch; ++b) {
                if (qLens[b] < 0 || (normMask && qLens[b] > lens[b])) {
                    ATB_B200_LOG(ERROR, "PagedAttention: qSeqLens should be in [0, contextLens]");
                    return ERROR_INVALID_PARAM;
                }
                for (int32_t j = 0; j < qLens[b]; ++j) {
                    maskRows_.push_back(normMask ? lens[b] - qLens[b] + j : static_cast<int32_t>(effectiveLens_.size()));
                    effectiveLens_.push_back(lens[b]);
                    btRows_.push_back(static_cast<int32_t>(b));
                }
            }
            if (static_cast<int64_t>(effectiveLens_.size()) != q.dims[0]) {
                ATB_B200_LOG(ERROR, "PagedAttention: the sum of qSeqLens should equal the query tokens");
                return ERROR_INVALID_PARAM;
            }
            // The same number n of query tokens for every sequence (MTP): one planned row per SEQUENCE whose CTA
            // columns are the n x heads-per-kv-head (token, head) pairs, so the cache is read once.  Tried first; a shape
            // the fused form does not cover (more than 8 pairs, head size, int8) falls back to one row per token.
            int32_t n = batch > 0 ? qLens[0] : 0;
            for (int64_t b = 1; b < batch; ++b) {
                n = qLens[b] == n ? n : 0;
            }
            fusedTokens_ = 0;
            if (n > 1 && !fusedRefused_ && std::getenv("ATB_B200_SPEC_EXPAND") == nullptr) {
                atb_b200_pa_desc f = d;
                f.batch = static_cast<int32_t>(batch);
                f.num_heads = n * param_.headNum;
                f.q_per_seq = n;
                f.score_mods = ATB_B200_SCORE_MASK | (normMask ? ATB_B200_SCORE_ROWS : 0);
                const int64_t maskLen = vp.inTensors.at(MaskPos()).desc.shape.dims[1];
                for (int64_t b = 0; b < batch; ++b) {
                    if (lens[b] > maskLen) {
                        ATB_B200_LOG(ERROR, "PagedAttention: the mask is shorter than a sequence's context");
                        return ERROR_INVALID_TENSOR_DIM;
                    }
                }
                int rc = MakePlan(f, lens);
                if (rc == 0 && normMask) {
                    // row of a sequence's first query token in the square mask; block-table rows are the identity
                    btRows_.resize(batch);
                    maskRows_.resize(batch);
                    for (int64_t b = 0; b < batch; ++b) {
                        btRows_[b] = static_cast<int32_t>(b);
                        maskRows_[b] = lens[b] - n;
                    }
                    rc = atb_b200_pa_plan_set_rows(plan_, btRows_.data(), static_cast<int32_t>(batch), maskRows_.data(),
                                                   vp.inTensors.at(MaskPos()).desc.shape.dims[0]);
                }
                if (rc == 0) {
                    fusedTokens_ = n;
                    atb_b200_pa_plan_info info{};
                    atb_b200_pa_plan_get_info(plan_, &info);
                    workspaceSize = info.workspace_bytes + 256;
                    return NO_ERROR;
                }
                if (rc != ERROR_INVALID_TENSOR_DIM) {
                    return rc;
                }
                fusedRefused_ = true; // these shapes have no fused form: do not try again on later Setups
            }
            lens = effectiveLens_.data();
        }
        if (HasMask()) {
            int64_t bs = 0, hs = 0, len = 0;
            (void)MaskLayout(vp.inTensors.at(MaskPos()).desc.shape, q.dims[0], &bs, &hs, &len);
            for (int32_t b = 0; b < d.batch; ++b) {
                if (lens[b] > len) {
                    ATB_B200_LOG(ERROR, "PagedAttention: the mask is shorter than a sequence's context");
                    return ERROR_INVALID_TENSOR_DIM;
                }
            }
        }
        if (param_.batchRunStatusEnable) {
            // Dynamic batch: the status tensor is host data like contextLens
            // (src/ops/ops_infer/paged_attention/param.cpp:39-50 of the reference).  The reference's kernels
            // skip a sequence through its zero context length; here a sequence whose status is 0 is also
            // planned as empty, so it is skipped whatever length the caller left in contextLens.
            const Tensor &status = vp.inTensors.at(StatusPos());
            if (status.hostData == nullptr) {
                ATB_B200_LOG(ERROR, "PagedAttention: batchRunStatus hostData is null");
                return ERROR_INVALID_PARAM;
            }
            const int32_t *run = static_cast<const int32_t *>(status.hostData);
            effectiveLens_.assign(lens, lens + d.batch);
            for (int32_t b = 0; b < d.batch; ++b) {
                if (run[b] == 0) {
                    effectiveLens_[b] = 0;
                }
            }
            lens = effectiveLens_.data();
        }
        int rc = MakePlan(d, lens);
        if (rc != 0) {
            return rc;
        }
        if (Spec()) {
            const Dims &m = vp.inTensors.at(MaskPos()).desc.shape;
            rc = atb_b200_pa_plan_set_rows(plan_, btRows_.data(), static_cast<int32_t>(cl.desc.shape.dims[0]),
                                           maskRows_.data(), m.dims[0]);
            if (rc != 0) {
                return rc;
            }
        }
        atb_b200_pa_plan_info info{};
        atb_b200_pa_plan_get_info(plan_, &info);
        workspaceSize = info.workspace_bytes + 256; // room to align the caller's pointer
        return NO_ERROR;
    }

    void AfterPlanImpl(aclrtStream stream) override
    {
        // start uploading the plan now; if this fails Execute uploads it itself
        (void)atb_b200_pa_plan_prefetch(plan_, stream);
    }

    Status LaunchImpl(const VariantPack &vp, uint8_t *workspace, uint64_t workspaceSize, aclrtStream stream) override
    {
        const bool mla = param_.mlaVHeadSize > 0;
        const size_t btPos = mla ? 2 : 3;
        atb_b200_pa_tensors t{};
        t.q = vp.inTensors.at(0).deviceData;
        t.k_cache = vp.inTensors.at(1).deviceData;
        t.v_cache = mla ? t.k_cache : vp.inTensors.at(2).deviceData;
        t.block_tables = static_cast<const int32_t *>(vp.inTensors.at(btPos).deviceData);
        t.out = vp.outTensors.at(0).deviceData;
        if (param_.quantType == Param::TYPE_DEQUANT_FUSION) {
            // runner order: kDescale, [kOffset], vDescale, [vOffset]
            size_t i = ScalePos();
            const Tensor &ks = vp.inTensors.at(i++);
            const Tensor *ko = param_.hasQuantOffset ? &vp.inTensors.at(i++) : nullptr;
            const Tensor &vs = vp.inTensors.at(i++);
            const Tensor *vo = param_.hasQuantOffset ? &vp.inTensors.at(i++) : nullptr;
            Status st = ScaleAsFloat(ks, 0, stream, &t.k_descale);
            if (st != NO_ERROR) {
                return st;
            }
            st = ScaleAsFloat(vs, 1, stream, &t.v_descale);
            if (st != NO_ERROR) {
                return st;
            }
            t.k_offset = ko ? static_cast<const int32_t *>(ko->deviceData) : nullptr;
            t.v_offset = vo ? static_cast<const int32_t *>(vo->deviceData) : nullptr;
        }
        if (QkvQuant()) {
            size_t i = ScalePos();
            t.k_descale = static_cast<const float *>(vp.inTensors.at(i++).deviceData);
            t.v_descale = static_cast<const float *>(vp.inTensors.at(i++).deviceData);
            if (param_.quantType == Param::TYPE_QUANT_QKV_OFFLINE) {
                t.p_scale = static_cast<const float *>(vp.inTensors.at(i++).deviceData);
            }
            if (t.k_descale == nullptr || t.v_descale == nullptr ||
                (param_.quantType == Param::TYPE_QUANT_QKV_OFFLINE && t.p_scale == nullptr)) {
                return ERROR_INVALID_PARAM;
            }
        }
        if (HasMask()) {
            const Tensor &m = vp.inTensors.at(MaskPos());
            t.mask = m.deviceData;
            (void)MaskLayout(m.desc.shape, vp.inTensors.at(0).desc.shape.dims[0], &t.mask_batch_stride,
                             &t.mask_head_stride, &t.mask_tokens);
            if (fusedTokens_ > 1) {
                // fused parallel decoding: consecutive tokens of a sequence are consecutive mask rows; with the spec mask
                // a sequence's first row is sequence x tokens-per-sequence (the norm mask's comes from the plan's rows)
                t.mask_q_stride = t.mask_tokens;
                if (param_.maskType == Param::MASK_TYPE_SPEC) {
                    t.mask_batch_stride = fusedTokens_ * t.mask_tokens;
                }
            }
        }
        if (param_.scaleType == Param::SCALE_TYPE_LOGN) {
            t.logn = static_cast<const float *>(vp.inTensors.at(vp.inTensors.size() - 1).deviceData);
        }
        if (t.q == nullptr || t.k_cache == nullptr || t.v_cache == nullptr || t.block_tables == nullptr ||
            t.out == nullptr || (HasMask() && t.mask == nullptr) ||
            (param_.scaleType == Param::SCALE_TYPE_LOGN && t.logn == nullptr)) {
            return ERROR_INVALID_PARAM;
        }
        uint8_t *ws = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
        const uint64_t usable = workspaceSize - static_cast<uint64_t>(ws - workspace);
        // kv heads sharded over the GPUs of a node: the context carries the ranks' gathered buffers and the kernel
        // stores this rank's heads into all of them (attnOut itself is then left untouched)
        const ContextImpl *ci = dynamic_cast<const ContextImpl *>(SetupContext());
        const atb_b200_pa_peers *peers = ci != nullptr ? ci->GatherPeers() : nullptr;
        const int rc = peers != nullptr ? atb_b200_pa_launch_gathered(plan_, &t, peers, ws, usable, stream)
                                        : atb_b200_pa_launch(plan_, &t, ws, usable, stream);
        return rc == 0 ? NO_ERROR : (rc == ERROR_INVALID_PARAM ? ERROR_INVALID_PARAM : ERROR_RT_FAIL);
    }

private:
    // Re-plans in place when only the lengths changed, else builds a new plan for `d`.
    int MakePlan(const atb_b200_pa_desc &d, const int32_t *lens)
    {
        if (plan_ != nullptr && SameDesc(d)) {
            return atb_b200_pa_plan_update(plan_, lens);
        }
        if (plan_ != nullptr) {
            atb_b200_pa_plan_destroy(plan_);
            plan_ = nullptr;
        }
        desc_ = d;
        const int rc = atb_b200_pa_plan_create(&d, lens, &plan_);
        if (rc == 0) {
            // once per plan shape: say when a shape misses the tiled kernels (the CUDA-core kernel is a
            // correctness path, far from the memory roofline)
            atb_b200_pa_plan_info info{};
            if (atb_b200_pa_plan_get_info(plan_, &info) == 0 && info.kernel == ATB_B200_KERNEL_GENERIC) {
                ATB_B200_LOG(INFO, "PagedAttentionOperation: this shape (heads per kv head " +
                                       std::to_string(d.num_heads / d.kv_heads) + ", head dims " +
                                       std::to_string(d.head_dim_k) + "/" + std::to_string(d.head_dim_v) + ", block size " +
                                       std::to_string(d.block_size) + ") runs on the untuned CUDA-core kernel");
            }
        }
        return rc;
    }

    bool SameDesc(const atb_b200_pa_desc &d) const
    {
        return d.batch == desc_.batch && d.num_heads == desc_.num_heads && d.kv_heads == desc_.kv_heads &&
               d.head_dim_k == desc_.head_dim_k && d.head_dim_v == desc_.head_dim_v && d.v_row_dim == desc_.v_row_dim &&
               d.block_size == desc_.block_size && d.num_blocks == desc_.num_blocks &&
               d.max_blocks_per_seq == desc_.max_blocks_per_seq && d.q_dtype == desc_.q_dtype &&
               d.kv_dtype == desc_.kv_dtype && d.qk_scale == desc_.qk_scale && d.kernel == desc_.kernel &&
               d.score_mods == desc_.score_mods && d.kv_layout == desc_.kv_layout && d.q_per_seq == desc_.q_per_seq &&
               d.qkv_quant == desc_.qkv_quant && d.out_dtype == desc_.out_dtype;
    }
    // fp32 scales are used in place; the int64-packed and fp16 encodings are converted once per
    // launch into a small device buffer owned by the operation.
    Status ScaleAsFloat(const Tensor &t, int which, aclrtStream stream, const float **out);
    static void FreeDevice(void *p);

    Param param_;
    std::vector<DtypeComb> combs_;
    atb_b200_pa_plan *plan_ = nullptr;
    // contextLens with the sequences batchRunStatus switches off set to 0; with CALC_TYPE_SPEC one entry per query token
    std::vector<int32_t> effectiveLens_;
    bool fusedRefused_ = false;
    int32_t fusedTokens_ = 0;                // CALC_TYPE_SPEC planned per sequence: query tokens per sequence (else 0)
    std::vector<int32_t> btRows_, maskRows_; // CALC_TYPE_SPEC: block-table row and mask row of every query token
    atb_b200_pa_desc desc_{};
    void *scratch_[2] = {nullptr, nullptr};
    uint64_t scratchElems_[2] = {0, 0};
};

} // namespace

// implemented in atb_scale_convert.cu (needs device code)
extern "C" int atb_b200_internal_convert_scales(const void *src, int src_kind, float *dst, uint64_t n, void *stream);
extern "C" int atb_b200_internal_device_alloc(void **p, uint64_t bytes);
extern "C" void atb_b200_internal_device_free(void *p);

namespace {
Status PagedAttentionOperation::ScaleAsFloat(const Tensor &t, int which, aclrtStream stream, const float **out)
{
    if (t.deviceData == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (t.desc.dtype == ACL_FLOAT) {
        *out = static_cast<const float *>(t.deviceData);
        return NO_ERROR;
    }
    const uint64_t n = Utils::GetTensorNumel(t.desc);
    if (scratchElems_[which] < n) {
        FreeDevice(scratch_[which]);
        scratch_[which] = nullptr;
        if (atb_b200_internal_device_alloc(&scratch_[which], n * sizeof(float)) != 0) {
            scratchElems_[which] = 0;
            return ERROR_OUT_OF_DEVICE_MEMORY;
        }
        scratchElems_[which] = n;
    }
    const int kind = t.desc.dtype == ACL_INT64 ? 1 : 2; // 1: fp32 bits in int64 words, 2: fp16
    if (atb_b200_internal_convert_scales(t.deviceData, kind, static_cast<float *>(scratch_[which]), n, stream) != 0) {
        return ERROR_RT_FAIL;
    }
    *out = static_cast<const float *>(scratch_[which]);
    return NO_ERROR;
}

void PagedAttentionOperation::FreeDevice(void *p)
{
    if (p != nullptr) {
        atb_b200_internal_device_free(p);
    }
}
} // namespace

template <> Status CreateOperation(const infer::PagedAttentionParam &opParam, Operation **operation)
{
    if (operation == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    if (!RsvIsZero(opParam.rsv, sizeof(opParam.rsv))) {
        ATB_B200_LOG(ERROR, "PagedAttentionParam.rsv must be zero");
        return ERROR_INVALID_PARAM;
    }
    if (!ParamCheck(opParam)) {
        return ERROR_INVALID_PARAM;
    }
    *operation = new (std::nothrow) PagedAttentionOperation(opParam);
    if (*operation == nullptr) {
        return ERROR_OUT_OF_HOST_MEMORY;
    }
    return NO_ERROR;
}

} // namespace atb
