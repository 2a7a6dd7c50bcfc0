// Parameter structs of the two operators on the decode path, byte-compatible with
// include/atb/infer_op_params.h of the reference: ReshapeAndCacheParam :488-526 (24 bytes),
// PagedAttentionParam :1859-1963 (120 bytes); sizes pinned by tests/unittest/ops/test_op_param_size.cpp:47,51.
#ifndef ATB_INFER_OP_PARAMS_H
#define ATB_INFER_OP_PARAMS_H
#include <cstdint>
#include <acl/acl.h>

namespace atb {
namespace infer {
enum InputLayout : int { TYPE_BSND = 0, TYPE_BNSD };

struct ReshapeAndCacheParam {
    enum CompressType : int { COMPRESS_TYPE_UNDEFINED = 0, COMPRESS_TYPE_KVHEAD, COMPRESS_TYPE_KVHEAD_ROPE };
    enum KvCacheCfg : int {
        K_CACHE_V_CACHE = 0, // key/value + both caches (5 inputs, 2 outputs)
        K_CACHE_V_BYPASS,    // key + key cache only (3 inputs, 1 output), e.g. the MLA combined cache
        K_CACHE_V_CACHE_NZ   // fractal layout of another SoC; rejected here
    };
    CompressType compressType = COMPRESS_TYPE_UNDEFINED;
    KvCacheCfg kvCacheCfg = K_CACHE_V_CACHE;
    uint8_t rsv[16] = {0};
};

struct PagedAttentionParam {
    int32_t headNum = 0;   // query heads
    float qkScale = 1.0;   // multiplies Q*K^T
    int32_t kvHeadNum = 0; // 0 = same as headNum
    enum MaskType : int {
        UNDEFINED = 0,
        MASK_TYPE_NORM,
        MASK_TYPE_ALIBI,
        MASK_TYPE_SPEC,
        MASK_TYPE_MASK_FREE,
        MASK_TYPE_NORM_COMPRESS
    };
    MaskType maskType = UNDEFINED;
    bool batchRunStatusEnable = false;
    enum QuantType : int {
        TYPE_QUANT_UNDEFINED = 0,
        TYPE_QUANT_UNQUANT = 0,
        TYPE_DEQUANT_FUSION = 1, // int8 K/V cache with per-channel descale (+ optional offset) inputs
        TYPE_QUANT_QKV_OFFLINE = 2,
        TYPE_QUANT_QKV_ONLINE = 3
    };
    QuantType quantType = TYPE_QUANT_UNQUANT;
    aclDataType outDataType = ACL_DT_UNDEFINED;
    bool hasQuantOffset = false;
    enum CompressType : int {
        COMPRESS_TYPE_UNDEFINED = 0,
        COMPRESS_TYPE_KVHEAD,
        COMPRESS_TYPE_KVHEAD_ROPE,
        COMPRESS_TYPE_MAX
    };
    CompressType compressType = COMPRESS_TYPE_UNDEFINED;
    enum CalcType : int { CALC_TYPE_UNDEFINED = 0, CALC_TYPE_SPEC };
    CalcType calcType = CALC_TYPE_UNDEFINED;
    enum ScaleType : int { SCALE_TYPE_TOR = 0, SCALE_TYPE_LOGN, SCALE_TYPE_MAX };
    ScaleType scaleType = SCALE_TYPE_TOR;
    InputLayout inputLayout = TYPE_BSND;
    uint32_t mlaVHeadSize = 0; // >0: combined K/V cache, V = first mlaVHeadSize columns of each K row
    float qScale = 0;
    uint8_t rsv[64] = {0};
};

// ReshapeAndCache whose key / value are strided views (e.g. slices of a fused QKV projection output):
// include/atb/infer_op_params.h:531-568 of the reference.  Inputs key, value, keyCache, valueCache,
// slotMapping, kStrides, vStrides, kOffset, vOffset (the last four int64 host tensors: element strides
// per dimension and the element offset of the view); K_CACHE_V_BYPASS: key, keyCache, slotMapping,
// kStrides, kOffset.
struct ReshapeAndCacheWithStrideParam {
    enum CompressType : int { COMPRESS_TYPE_UNDEFINED = 0, COMPRESS_TYPE_KVHEAD, COMPRESS_TYPE_KVHEAD_ROPE };
    enum KvCacheCfg : int { K_CACHE_V_CACHE = 0, K_CACHE_V_BYPASS };
    CompressType compressType = COMPRESS_TYPE_UNDEFINED;
    KvCacheCfg kvCacheCfg = K_CACHE_V_CACHE;
    uint8_t rsv[16] = {0};
};

// KvCache (include/atb/infer_op_params.h:423-431 of the reference): appends new K or V rows to a contiguous per-layer
// cache.  Inputs newKv [tokens, hidden] (or [batch, seq, heads, headSize]), layerId [1], past [layers, batch, maxSeqLen,
// hidden], tokenOffset [batch], seqLen [batch] (all int32 device tensors); no outputs, past is updated in place.
struct KvCacheParam {
    uint8_t rsv[8] = {0};
};

// MultiLatentAttention (include/atb/infer_op_params.h:2899-2950 of the reference): attention over the MLA latent
// cache given as separate latent (512) and rope (64) tensors.  Decode form built here: inputs qNope [tokens, heads,
// 512], qRope [tokens, heads, 64], ctKV [blocks, 128, 1, 512], kRope [blocks, 128, 1, 64], blockTables, contextLens
// (host data mandatory); output attnOut [tokens, heads, 512].
struct MultiLatentAttentionParam {
    int32_t headNum = 0;
    float qkScale = 1.0;
    int32_t kvHeadNum = 0;
    enum MaskType : int { UNDEFINED = 0, MASK_TYPE_SPEC, MASK_TYPE_MASK_FREE, MASK_TYPE_CAUSAL_MASK, MASK_TYPE_SWA_NORM };
    MaskType maskType = UNDEFINED;
    enum CalcType : int {
        CALC_TYPE_UNDEFINED = 0, // decode, one query token per sequence
        CALC_TYPE_SPEC,          // several query tokens per sequence (parallel decoding)
        CALC_TYPE_RING,          // also returns the log-sum-exp
        CALC_TYPE_SPEC_AND_RING,
        CALC_TYPE_PREFILL,
    };
    CalcType calcType = CALC_TYPE_UNDEFINED;
    enum CacheMode : uint8_t {
        KVCACHE = 0,  // combined cache (not supported by the reference either)
        KROPE_CTKV,   // separate latent and rope caches
        INT8_NZCACHE, // layouts of another SoC
        NZCACHE,
    };
    CacheMode cacheMode = KVCACHE;
    uint32_t windowSize = 0;
    enum MaskUseStatusType : int {
        MASK_USE_STATUS_TYPE_UNDEFINED = 0,
        MASK_USE_STATUS_TYPE_BATCH_MASK,
        MASK_USE_STATUS_TYPE_MAX
    };
    MaskUseStatusType maskUseStatusType = MASK_USE_STATUS_TYPE_UNDEFINED;
    uint8_t rsv[32] = {0};
};

// Fused RMSNorm + RoPE + ReshapeAndCache of the MLA latent cache (include/atb/infer_op_params.h:2697-2716 of
// the reference).  Inputs x [tokens, 1, dx], gamma [dx], keyRope [tokens, dr], cos [tokens, dr],
// sin [tokens, dr], slotMapping [tokens], keyCacheIn [blocks, blockSize, 1, dx + dr]; output keyCacheOut.
struct NormRopeReshapeParam {
    uint32_t precisionMode = 0;
    uint32_t rotaryCoeff = 2; // 2: rotate halves (the only mode of the reference kernel and of this one)
    float epsilon = 1e-5;
    uint8_t rsv[16] = {0};
};

// BlockCopy: copy the cache blocks named by srcBlockIndices onto the blocks named by dstBlockIndices
// (include/atb/infer_op_params.h:1205-1215 of the reference).  Inputs keyCache, valueCache,
// srcBlockIndices [n], dstBlockIndices [m], cumSum [n] (running total of destinations per source);
// no outputs, the caches are updated in place.
struct BlockCopyParam {
    uint8_t rsv[16] = {0};
};

// PagedCacheLoad: the reverse of ReshapeAndCache (include/atb/infer_op_params.h:3070-3100 of the
// reference).  Inputs keyCache, valueCache, blockTables, contextLens, key, value, seqStarts; outputs
// key, value ([sum of lengths, heads, headSize]).
struct PagedCacheLoadParam {
    enum KvCacheCfg : int8_t {
        K_CACHE_V_CACHE_NZ = 0, // fractal layout of another SoC (the reference's default); rejected here
        K_CACHE_V_CACHE_ND,     // [numBlocks, blockSize, heads, headSize] caches
    };
    KvCacheCfg kvCacheCfg = K_CACHE_V_CACHE_NZ;
    bool isSeqLensCumsumMode = false; // contextLens holds running totals [batch + 1] instead of lengths
    bool hasSeqStarts = false;        // seqStarts[i] / blockSize = first block-table column of sequence i
    uint8_t rsv[61] = {0};
};

static_assert(sizeof(ReshapeAndCacheWithStrideParam) == 24, "ABI: ReshapeAndCacheWithStrideParam is 24 bytes");
static_assert(sizeof(KvCacheParam) == 8, "ABI: KvCacheParam is 8 bytes");
static_assert(sizeof(MultiLatentAttentionParam) == 64, "ABI: MultiLatentAttentionParam is 64 bytes");
static_assert(sizeof(NormRopeReshapeParam) == 28, "ABI: NormRopeReshapeParam is 28 bytes");
static_assert(sizeof(BlockCopyParam) == 16, "ABI: BlockCopyParam is 16 bytes");
static_assert(sizeof(PagedCacheLoadParam) == 64, "ABI: PagedCacheLoadParam is 64 bytes");
static_assert(sizeof(ReshapeAndCacheParam) == 24, "ABI: ReshapeAndCacheParam is 24 bytes");
static_assert(sizeof(PagedAttentionParam) == 120, "ABI: PagedAttentionParam is 120 bytes");
} // namespace infer
} // namespace atb
#endif
