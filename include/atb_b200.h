/*
 * C ABI of libatb_b200.so: the boundary a foreign-function binding targets.  Plain pointers and
 * sizes only.  Every function returns 0 (ATB_B200_OK) or an atb::ErrorType value.
 *
 * Two levels:
 *   1. kernel level  - plan on the host from context_lens, then enqueue the CUDA kernels; this is
 *      what the reference's kernel-host layer does in PagedAttentionTiling + kernel launch.
 *   2. operator level - handles around the C++ atb::Operation objects, mirroring the reference's
 *      C-style wrappers (include/atb/atb_acl.h) for callers that cannot use the C++ classes.
 *
 * All device pointers are CUDA device memory of the current device; `stream` is a cudaStream_t.
 * Launch functions only enqueue work; completion is the caller's stream synchronisation.
 */
#ifndef ATB_B200_H
#define ATB_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATB_B200_OK 0

/* element types of query / cache tensors */
enum { ATB_B200_FP16 = 0, ATB_B200_BF16 = 1, ATB_B200_INT8 = 2 };

/* kernel families; AUTO lets the planner choose */
enum {
    ATB_B200_KERNEL_AUTO = 0,
    ATB_B200_KERNEL_GENERIC = 1, /* CUDA-core kernel, any shape */
    ATB_B200_KERNEL_TMA_MMA = 2, /* TMA page gather + warp-level tensor-core tiles, D = 128 */
    ATB_B200_KERNEL_MLA_TC5 = 3  /* TMA + tcgen05/TMEM tiles for the 576/512 latent cache */
};

/*
 * Shape of one paged-attention decode call (one query token per sequence).
 * Replaces AtbOps::OpParam::PagedAttention (src/kernels/include/atbops/params/pagedattention.h:21-87
 * of the reference) plus the shapes its tiling reads from the tensors
 * (src/kernels/mixkernels/pagedattention/tiling/paged_attention_tiling.cpp:194-244).
 */
typedef struct atb_b200_pa_desc {
    int32_t batch;          /* sequences = query tokens */
    int32_t num_heads;      /* query heads */
    int32_t kv_heads;       /* key/value heads; num_heads % kv_heads == 0 */
    int32_t head_dim_k;     /* width of a query / key row */
    int32_t head_dim_v;     /* width of the output row (MLA: mlaVHeadSize) */
    int32_t v_row_dim;      /* allocated width of a value-cache row (MLA combined cache: head_dim_k) */
    int32_t block_size;     /* tokens per cache block */
    int32_t num_blocks;     /* blocks in the cache */
    int32_t max_blocks_per_seq; /* row length of block_tables */
    int32_t q_dtype;        /* ATB_B200_FP16 | ATB_B200_BF16; also the output type (ATB_B200_INT8 with qkv_quant) */
    int32_t kv_dtype;       /* same as q_dtype, or ATB_B200_INT8 */
    float qk_scale;         /* multiplies Q*K^T */
    int32_t kernel;         /* ATB_B200_KERNEL_*; AUTO unless forcing a path */
    int32_t sm_count;       /* 0 = query the current device (148 on B200) */
    int32_t rope_dim;       /* 0, or 64 for the split MLA cache (MultiLatentAttention, cacheMode KROPE_CTKV of the
                               reference): the last rope_dim elements of every query / key row live in the separate
                               tensors q_rope / k_rope_cache, q and k_cache hold the first head_dim_k - rope_dim
                               (= head_dim_v = v_row_dim) elements */
    int32_t score_mods;     /* ATB_B200_SCORE_* bits: what is applied to Q*K^T besides qk_scale (PagedAttentionParam
                               maskType NORM / ALIBI, scaleType SCALE_TYPE_LOGN of the reference) */
    int32_t kv_layout;      /* ATB_B200_KV_BSND (0): caches [num_blocks, block_size, kv_heads, dim];
                               ATB_B200_KV_BNSD (1): [num_blocks, kv_heads, block_size, dim] (inputLayout TYPE_BNSD of
                               the reference; fp16 / bf16 caches, no split MLA cache) */
    int32_t q_per_seq;      /* 0 / 1: one query token per planned row.  n > 1 (parallel decoding with the same number of
                               query tokens for every sequence): batch = sequences, q and out hold n consecutive tokens
                               per sequence ([batch * n, heads, dim]), num_heads = n x the real head count, and one CTA
                               serves the n x heads-per-kv-head (token, head) pairs of a kv head from one read of the
                               cache (at most 8 pairs; fp16 / bf16, head_dim 128); the MLA kernel takes any n: its
                               rows are the n x heads (token, head) pairs.  A mask is indexed per (sequence, token):
                               see mask_q_stride */
    int32_t qkv_quant;      /* 0, or ATB_B200_QUANT_ONLINE / ATB_B200_QUANT_OFFLINE (quantType TYPE_QUANT_QKV_ONLINE /
                               OFFLINE of the reference): q_dtype and kv_dtype are ATB_B200_INT8, k_descale and v_descale
                               hold ONE fp32 scale per query head ([num_heads]: of Q.K^T and of P.V), the probabilities
                               are quantised to int8 - online against each tile's own maximum, offline with p_scale
                               [num_heads] - and both contractions run on the integer tensor cores; head_dim 128 */
    int32_t out_dtype;      /* qkv_quant only: ATB_B200_FP16 | ATB_B200_BF16, the type of `out` */
} atb_b200_pa_desc;

enum { ATB_B200_QUANT_ONLINE = 1, ATB_B200_QUANT_OFFLINE = 2 };

enum { ATB_B200_KV_BSND = 0, ATB_B200_KV_BNSD = 1 };

enum {
    ATB_B200_SCORE_MASK = 1, /* score(b, h, t) += mask[b * mask_batch_stride + h * mask_head_stride + t] */
    ATB_B200_SCORE_LOGN = 2, /* the scale of sequence b is qk_scale * logn[b] */
    ATB_B200_SCORE_CAUSAL = 8, /* q_per_seq = n > 1 only: query token j of a sequence sees its first context_len - (n - 1 - j)
                                  cached tokens (the causal rule of parallel decoding, MASK_TYPE_MASK_FREE of the
                                  reference's MultiLatentAttention) without reading a mask */
    ATB_B200_SCORE_ROWS = 4  /* query token b reads row bt_rows[b] of block_tables and (with a mask) row mask_rows[b]
                                of the mask instead of row b: parallel decoding (CALC_TYPE_SPEC of the reference),
                                where several query tokens share one sequence's cache.  The rows are set with
                                atb_b200_pa_plan_set_rows; until then they are the identity. */
};

/* Device pointers of one call.  v_cache == k_cache for the MLA combined cache. */
typedef struct atb_b200_pa_tensors {
    const void *q;              /* [batch, num_heads, head_dim_k] */
    const void *k_cache;        /* [num_blocks, block_size, kv_heads, head_dim_k] */
    const void *v_cache;        /* [num_blocks, block_size, kv_heads, v_row_dim] */
    const int32_t *block_tables; /* [batch, max_blocks_per_seq] */
    const float *k_descale;     /* [kv_heads*head_dim_k] fp32, int8 cache only, may be NULL (=1) */
    const float *v_descale;     /* [kv_heads*head_dim_v] */
    const int32_t *k_offset;    /* optional int32 offsets added before scaling */
    const int32_t *v_offset;
    void *out;                  /* [batch, num_heads, head_dim_v], q_dtype */
    const void *q_rope;         /* rope_dim > 0 only: [batch, num_heads, rope_dim] */
    const void *k_rope_cache;   /* rope_dim > 0 only: [num_blocks, block_size, kv_heads, rope_dim] */
    /* ATB_B200_SCORE_MASK only: additive mask in q_dtype, indexed in elements as stated at the enum.  The alibi mask
       [batch, heads, 1, tokens] has strides (heads*tokens, tokens), [heads, 1, tokens] (0, tokens); the plain mask
       [batch, 1, tokens] (tokens, 0), [1, tokens] (0, 0).  mask_tokens = its last dimension, at least the longest
       context of the plan. */
    const void *mask;
    int64_t mask_batch_stride;
    int64_t mask_head_stride;
    int64_t mask_tokens;
    int64_t mask_q_stride;      /* q_per_seq > 1 only: elements between the mask rows of consecutive query tokens of a
                                   sequence; token j of sequence b reads mask[row(b) * mask_batch_stride + j *
                                   mask_q_stride + h * mask_head_stride + t], row(b) = b or mask_rows[b] */
    const float *logn;          /* ATB_B200_SCORE_LOGN only: [batch] fp32 */
    void *lse_out;              /* optional, MLA kernel only: [batch, num_heads] in q_dtype, the natural-log
                                   log-sum-exp of the scaled scores of every (token, head) (the second output of
                                   MultiLatentAttention with CALC_TYPE_RING); NULL = not wanted */
    const float *p_scale;       /* ATB_B200_QUANT_OFFLINE only: [num_heads] fp32 */
} atb_b200_pa_tensors;

typedef struct atb_b200_pa_plan atb_b200_pa_plan; /* opaque */

typedef struct atb_b200_pa_plan_info {
    int32_t kernel;          /* family chosen */
    int32_t num_ctas;        /* grid of the attention kernel */
    int32_t num_items;       /* (sequence, token-range) work items */
    int32_t num_partials;    /* split-KV partial results written to the workspace */
    int32_t num_combine_seqs; /* sequences merged by the combine kernel */
    int32_t tile_tokens;     /* scheduling granule */
    uint64_t workspace_bytes;
    uint64_t plan_bytes;     /* bytes uploaded per launch */
    int32_t kernels_per_launch; /* 1 = attention only (it merges split sequences itself), 2 = + combine */
    int32_t reserved;
} atb_b200_pa_plan_info;

/*
 * Host-only planning: splits the sequences into balanced token ranges (split-KV) from the host
 * copy of context_lens.  No CUDA call is made unless desc->sm_count == 0.
 * Replaces PagedAttentionTiling (tiling/paged_attention_tiling.cpp:419-470 of the reference).
 */
int atb_b200_pa_plan_create(const atb_b200_pa_desc *desc, const int32_t *context_lens_host, atb_b200_pa_plan **plan);
/* Re-plan in place for new context_lens of the same batch (one decode step later). */
int atb_b200_pa_plan_update(atb_b200_pa_plan *plan, const int32_t *context_lens_host);
/*
 * ATB_B200_SCORE_ROWS only: which row of block_tables (bt_rows[b] in [0, bt_row_count)) and of the mask
 * (mask_rows[b] in [0, mask_row_count); may be NULL without a mask) query token b uses; both host arrays of
 * desc->batch entries, copied.  Call after plan_create / plan_update and before plan_prefetch / launch of the step.
 * The caller passes block_tables with bt_row_count rows and a mask with mask_row_count rows of mask_tokens elements
 * (mask_batch_stride = the row length).  Replaces the qSeqLens handling of the reference's tiling
 * (paged_attention_tiling.cpp; qSeqLens is host data there too, ops_infer/paged_attention/param.cpp).
 */
int atb_b200_pa_plan_set_rows(atb_b200_pa_plan *plan, const int32_t *bt_rows, int32_t bt_row_count,
                              const int32_t *mask_rows, int64_t mask_row_count);
int atb_b200_pa_plan_get_info(const atb_b200_pa_plan *plan, atb_b200_pa_plan_info *info);
/* Copies the plan's work items (4 int32 each: seq, tok_begin, tok_end, partial slot or -1) and the
 * per-CTA-group item offsets into caller arrays (either may be NULL); for tests and debugging. */
int atb_b200_pa_plan_dump(const atb_b200_pa_plan *plan, int32_t *items, int32_t max_items, int32_t *group_begin,
                          int32_t max_groups);
void atb_b200_pa_plan_destroy(atb_b200_pa_plan *plan);

/*
 * Enqueue plan upload + attention kernel (+ combine kernel when any sequence was split).
 * `workspace` must hold plan->workspace_bytes, 256-byte aligned.  Replaces the launch of
 * paged_attention_mask / paged_multi_latent_attention_mask
 * (src/kernels/mixkernels/pagedattention/op_kernel/paged_attention_mask_mix.cce:24,
 *  paged_MLAttention_combine_cache_mask_mix.cce:24 of the reference).
 */
int atb_b200_pa_launch(atb_b200_pa_plan *plan, const atb_b200_pa_tensors *tensors, void *workspace,
                       uint64_t workspace_bytes, void *stream);

/*
 * Optional: upload the plan ahead of the launch.  Copies the plan into device memory owned by the plan
 * on a private stream and makes `stream` wait for that copy at the point of this call, so the copy
 * overlaps whatever the caller enqueues before it and no longer sits between ReshapeAndCache and the
 * attention kernel.  Call it after plan_create / plan_update and before the work that precedes the
 * launch; the next atb_b200_pa_launch on the same stream then uses that copy.  Without it the launch
 * uploads the plan itself.  (The reference uploads its tiling at Execute: operation_base.cpp:716.)
 */
int atb_b200_pa_plan_prefetch(atb_b200_pa_plan *plan, void *stream);

/*
 * KV heads sharded over the GPUs of one node (one process per GPU): every rank computes the query
 * heads of its kv heads and the outputs are exchanged.  Instead of a separate all-gather
 * (AllGatherOperation after attention in a reference model graph,
 * src/ops/ops_infer/all_gather/all_gather_hccl_runner.cpp:47), the attention kernel stores its
 * output rows into the gathered buffer [batch, total_heads, head_dim_v] of EVERY rank through
 * peer-mapped memory (plain stores over NVLink), and a one-CTA kernel then publishes / awaits a
 * per-rank completion flag.  When the call's work has completed on the stream, the local gathered
 * buffer holds all ranks' heads.
 *
 * peer_out[r] / peer_flags[r]: rank r's gathered buffer and flag array (8 x uint32, zero before the
 * first call) as mapped in THIS process (atb_b200_peer_buffer_*).  `epoch` starts at 1 and grows by
 * one per call on every rank.  A rank may run one step ahead of a slow peer, so alternate between
 * two gathered buffers from call to call.  The wait is bounded; a peer that never arrives sets the
 * status word instead of hanging the GPU, and the call has still returned ATB_B200_OK (it only enqueues):
 * read atb_b200_pa_plan_device_status before trusting the gathered buffer whenever a rank may have
 * stalled (status 1 = the buffer is incomplete).  Only the TMA kernels (head_dim 128) support this path.
 */
typedef struct atb_b200_pa_peers {
    int32_t world;        /* ranks, 1..8 */
    int32_t rank;         /* this rank */
    int32_t total_heads;  /* query heads of the whole model */
    int32_t head_offset;  /* first global head computed by this rank */
    void *peer_out[8];
    uint32_t *peer_flags[8];
    uint32_t epoch;
    uint32_t poll_limit;  /* polls (about 0.2 us each) before the wait for the peers gives up; 0 = 2^22 (about a second).
                             Match it to the host skew between the ranks: a rank that enqueues its kernel later than
                             this makes every other rank give up. */
} atb_b200_pa_peers;

int atb_b200_pa_launch_gathered(atb_b200_pa_plan *plan, const atb_b200_pa_tensors *tensors,
                                const atb_b200_pa_peers *peers, void *workspace, uint64_t workspace_bytes,
                                void *stream);

/* Device buffers other processes of the node can map (CUDA IPC): create returns the local pointer
 * and a 64-byte handle to hand to the peers (over any host channel); open maps a peer's buffer. */
int atb_b200_peer_buffer_create(uint64_t bytes, void **local_ptr, uint8_t handle[64]);
int atb_b200_peer_buffer_open(const uint8_t handle[64], void **peer_ptr);
int atb_b200_peer_buffer_close(void *peer_ptr);
int atb_b200_peer_buffer_destroy(void *local_ptr);

/*
 * ReshapeAndCache: cache[slot_mapping[i]] = key[i] (and value) for slot >= 0; byte-exact copy.
 * row bytes = heads * head_dim * sizeof(elem).  value/value_cache NULL = K-only variant.
 * Replaces the reshape_and_cache / reshape_and_cache_siso kernels
 * (src/kernels/mixkernels/reshape_and_cache/op_kernel/reshape_and_cache_nd.cpp:146,
 *  reshape_and_cache_nd_siso.cpp:80 of the reference).
 */
int atb_b200_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                               const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                               int64_t v_row_bytes, int64_t num_slots, void *stream);

/* Device-side status word of the last launch into `workspace` (0 = ok; 1 = a bounded wait in a
 * kernel gave up).  Synchronises `stream`. */
int atb_b200_pa_plan_device_status(atb_b200_pa_plan *plan, void *workspace, void *stream, int32_t *status);

/* Optional event probe for kernel tuning (the role of the reference's Probe hooks,
 * src/atb/utils/probe.h:19-58): `device_events` is a zeroed device array of (capacity & 0xffffff) uint64;
 * CTA number (capacity >> 24) of the MLA kernel appends (tag << 56 | index << 40 | SM cycle counter) records,
 * element 0 counts them.  CTA number 255 selects the other form: every CTA b of the MLA kernel stores the global
 * nanosecond timer at its start and at its end in elements 1 + 2b and 2 + 2b (capacity >= 2 * grid + 2), which shows how
 * evenly the plan loads the SMs.  NULL switches it off. */
int atb_b200_pa_plan_set_trace(atb_b200_pa_plan *plan, void *device_events, uint32_t capacity);

/* Optional timing of the attention kernel alone: with enable = n > 0 every n-th launch (the first one included)
 * records a pair of CUDA events on the launch stream around that kernel (a ring of 256 pairs); 0 switches it
 * off.  An event between ReshapeAndCache and the attention kernel costs their programmatic overlap, so a
 * stride above 1 keeps the timed steps close to untimed ones.  kernel_ms returns the duration of the timed
 * launch `launches_back` timed launches ago (0 = the latest) and synchronises on its second event. */
int atb_b200_pa_plan_set_profiling(atb_b200_pa_plan *plan, int enable);
int atb_b200_pa_plan_kernel_ms(atb_b200_pa_plan *plan, int32_t launches_back, float *ms);

/*
 * Paged decode attention without any allocation.  No counterpart in the reference: there the
 * caller always owns a workspace.  This one is for callers that may not allocate at all - a server
 * that hands its whole device memory to its own pool and forbids cudaMalloc afterwards, a
 * latency-bound host thread that must not take an allocator lock, a plugin inside a runtime whose
 * allocator has to stay the only one.  One call plans the split on the stack (about 80 KB of
 * stack), uploads the plan from there and runs the same attention and combine kernels as
 * atb_b200_pa_launch, with their workspace taken from a scratch array built into the library
 * (8 MiB + 320 KiB of device memory on every GPU that loads the library, held until exit).
 *
 * Limits - a call beyond any of them is refused with ERROR_INVALID_PARAM and a message on stderr,
 * nothing is truncated: batch <= 1024; CTA groups <= 1024; split-KV partials x num_heads <= 65536;
 * partials x num_heads x head_dim_v <= 2097152 floats.  (The five benchmark shapes need at most a
 * quarter of that.)
 *
 * The scratch is shared by every call and keeps the last call's contents; a call writes all it
 * later reads (the uploaded plan carries a zeroed status word).  Calls whose kernels can overlap on
 * the GPU - different streams without ordering, several host threads - race on it: keep them on one
 * stream or order them yourself.
 *
 * The first call on each device looks the scratch's device address up (cudaGetSymbolAddress, with
 * that device current) and caches it; make that first call outside of any stream capture.  The
 * call uses no cudaMalloc, cudaFree, cudaHostAlloc, event creation or other allocating routine.
 */
int atb_b200_pa_decode_static_scratch(const atb_b200_pa_desc *desc, const int32_t *context_lens_host,
                                      const atb_b200_pa_tensors *tensors, void *stream);

/* Device status of the last atb_b200_pa_decode_static_scratch call on this GPU whose kernels have run: 0, 1 (a bounded
 * wait gave up) or 2 (a block id outside the cache), as atb_b200_pa_plan_device_status reports for the planned entry
 * points.  Copies the word from the scratch on `stream` and waits for that stream; allocates nothing; refused on a
 * capturing stream.  Like the entry point itself it has no counterpart in the reference. */
int atb_b200_pa_static_scratch_status(void *stream, int32_t *status_out);

/* ---------------------------------------------------------------- operator level */

/* Mirrors atb::Tensor (include/atb/types.h:118-127 of the reference). */
typedef struct atb_b200_tensor {
    int32_t dtype;      /* aclDataType value */
    int32_t format;     /* aclFormat value */
    int64_t dims[8];
    uint64_t dim_num;
    void *device_data;
    void *host_data;
    uint64_t data_size;
} atb_b200_tensor;

int atb_b200_context_create(void **context);
int atb_b200_context_set_stream(void *context, void *stream);
int atb_b200_context_destroy(void *context);
/* Extension with no counterpart in the reference (there a model graph runs AllGatherOperation after attention,
 * src/ops/ops_infer/all_gather/all_gather_operation.cpp:79-89): while `peers` is set on a context, every
 * PagedAttention Execute on it takes the atb_b200_pa_launch_gathered path - the kernel stores this rank's heads
 * into every rank's gathered buffer and attnOut is left untouched.  The struct is copied; set it again before
 * every Execute (the epoch grows by one per step and the gathered buffers alternate), NULL switches it off. */
int atb_b200_context_set_gather(void *context, const atb_b200_pa_peers *peers);

/* `param` points at an atb::infer::PagedAttentionParam (120 bytes) / ReshapeAndCacheParam (24 bytes). */
int atb_b200_operation_create_paged_attention(const void *param, uint64_t param_bytes, void **operation);
int atb_b200_operation_create_reshape_and_cache(const void *param, uint64_t param_bytes, void **operation);
/* atb::CreateOperation<infer::BlockCopyParam> (16-byte param) and <infer::PagedCacheLoadParam> (64-byte param) */
int atb_b200_operation_create_block_copy(const void *param, uint64_t param_bytes, void **operation);
int atb_b200_operation_create_paged_cache_load(const void *param, uint64_t param_bytes, void **operation);
/* atb::CreateOperation<infer::ReshapeAndCacheWithStrideParam> (24-byte param) */
int atb_b200_operation_create_reshape_and_cache_with_stride(const void *param, uint64_t param_bytes, void **operation);
/*
 * KvCache (src/kernels/mixkernels/kvcache of the reference; golden tests/apitest/kernelstest/mix/test_kvcache.py:65-78):
 * the contiguous per-layer cache past [layers, batch, max_seqlen, hidden] receives, for every sequence b, its seq_len[b]
 * rows of new_kv [num_tokens, hidden] (sequences back to back) at positions [token_offset[b] - seq_len[b],
 * token_offset[b]) of layer layer_id[0].  layer_id, token_offset, seq_len are device int32 arrays; row_bytes = hidden x
 * element size.  Runs that do not fit the cache or new_kv are skipped.
 */
int atb_b200_kv_cache(const void *new_kv, const int32_t *layer_id, void *past, const int32_t *token_offset,
                      const int32_t *seq_len, int64_t num_tokens, int32_t layers, int32_t batch, int32_t max_seqlen,
                      int64_t row_bytes, void *stream);
/* atb::CreateOperation<infer::KvCacheParam> (8-byte param; tests/unittest/ops/test_op_param_size.cpp:36) */
int atb_b200_operation_create_kv_cache(const void *param, uint64_t param_bytes, void **operation);
/* atb::CreateOperation<infer::MultiLatentAttentionParam> (64-byte param; tests/unittest/ops/test_op_param_size.cpp:68) */
int atb_b200_operation_create_multi_latent_attention(const void *param, uint64_t param_bytes, void **operation);
/* atb::CreateOperation<infer::NormRopeReshapeParam> (28-byte param) */
int atb_b200_operation_create_norm_rope_reshape(const void *param, uint64_t param_bytes, void **operation);
int atb_b200_operation_input_num(void *operation, uint32_t *n);
int atb_b200_operation_output_num(void *operation, uint32_t *n);
/* Operation::GetName (include/atb/operation.h:46 of the reference): copies the NUL-terminated name into
 * buf (at most cap bytes, always terminated); ERROR_INVALID_PARAM when buf is null or cap is 0. */
int atb_b200_operation_name(void *operation, char *buf, uint64_t cap);
int atb_b200_operation_infer_shape(void *operation, const atb_b200_tensor *in, uint32_t n_in, atb_b200_tensor *out,
                                   uint32_t n_out);
int atb_b200_operation_setup(void *operation, const atb_b200_tensor *in, uint32_t n_in, const atb_b200_tensor *out,
                             uint32_t n_out, uint64_t *workspace_bytes, void *context);
int atb_b200_operation_execute(void *operation, const atb_b200_tensor *in, uint32_t n_in, const atb_b200_tensor *out,
                               uint32_t n_out, void *workspace, uint64_t workspace_bytes, void *context);
int atb_b200_operation_destroy(void *operation);

/* ---- cache-management siblings of ReshapeAndCache (kernel level) ------------------------------------
 *
 * BlockCopy: copy whole cache blocks in place, replaces the BlockCopyOperation kernel of the reference
 * (src/ops/ops_infer/block_copy/block_copy_operation.cpp:58-120, golden tests/apitest/kernelstest/mix/
 * test_blockcopy.py:65-81).  Source block src_blocks[i] goes to the destinations
 * dst_blocks[cum_sum[i-1] .. cum_sum[i]) (cum_sum = running total of destinations per source; all three
 * are device int32 arrays).  v_cache may be null.  Blocks outside [0, num_blocks) are skipped.  The
 * copies run in parallel: a block must not be both a source and a destination of one call. */
int atb_b200_block_copy(void *k_cache, void *v_cache, const int32_t *src_blocks, const int32_t *dst_blocks,
                        const int32_t *cum_sum, int32_t n_src, int32_t n_dst, int64_t k_block_bytes,
                        int64_t v_block_bytes, int64_t num_blocks, void *stream);

/* PagedCacheLoad (ND caches): gather every sequence's cached tokens into contiguous rows, the reverse of
 * ReshapeAndCache; replaces src/kernels/mixkernels/paged_cache_load/op_kernel/paged_cache_load_nd.cpp:139-226
 * of the reference.  context_lens (device int32) holds lengths [batch], or running totals [batch + 1] when
 * lens_are_cumulative; sequence i fills rows [start_i, start_i + len_i) of key / value ([out_rows, row bytes])
 * from the blocks block_tables[i][seq_starts[i] / block_size + t].  seq_starts may be null; v_cache and value
 * may both be null.  Block ids, table columns and rows out of range are skipped.  With plain lengths the call
 * needs atb_b200_paged_cache_load_workspace_bytes(batch, 0) bytes of device workspace for the running totals. */
uint64_t atb_b200_paged_cache_load_workspace_bytes(int32_t batch, int32_t lens_are_cumulative);
int atb_b200_paged_cache_load(const void *k_cache, const void *v_cache, const int32_t *block_tables,
                              const int32_t *context_lens, const int32_t *seq_starts, void *key, void *value,
                              int32_t batch, int32_t table_cols, int32_t block_size, int64_t k_row_bytes,
                              int64_t v_row_bytes, int64_t num_blocks, int64_t out_rows, int32_t lens_are_cumulative,
                              void *workspace, uint64_t workspace_bytes, void *stream);

/* ReshapeAndCache reading strided rows: token t's key row (k_row_bytes, contiguous) starts at
 * key + t * k_token_stride_bytes (value likewise), e.g. the K and V slices of a fused QKV projection output;
 * the rows are scattered to the cache slots like atb_b200_reshape_and_cache does.  key / value point at the
 * first element of token 0's row (the caller applies the view's element offset).  Replaces the strided mode
 * of the reference's ReshapeAndCache kernel (op_kernel/reshape_and_cache_nd.cpp:70-128, tiling
 * reshape_and_cache_tiling.cpp:60-75).  value and value_cache may both be null. */
int atb_b200_reshape_and_cache_strided(const void *key, const void *value, void *key_cache, void *value_cache,
                                       const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                                       int64_t v_row_bytes, int64_t k_token_stride_bytes, int64_t v_token_stride_bytes,
                                       int64_t num_slots, void *stream);

/* Fused RMSNorm + RoPE + cache write of the MLA latent cache (NormRopeReshapeOperation of the reference,
 * src/ops/ops_infer/norm_rope_reshape/norm_rope_reshape_operation.cpp; golden tests/apitest/kernelstest/mix/
 * test_rms_norm_and_rope_and_reshape_and_cache.py:24-72): token t's cache row (slot slot_mapping[t], dx + dr wide)
 * becomes [ x[t] * rsqrt(mean(x[t]^2) + epsilon) * gamma | key_rope[t] * cos[t] + rotate_half(key_rope[t]) * sin[t] ].
 * x [tokens, dx], gamma [dx], key_rope / cos_table / sin_table [tokens, dr], all of `dtype` (ATB_B200_FP16 | BF16);
 * negative slots are skipped, slots >= num_slots dropped. */
int atb_b200_norm_rope_reshape(const void *x, const void *gamma, const void *key_rope, const void *cos_table,
                               const void *sin_table, const int32_t *slot_mapping, void *key_cache,
                               int32_t num_tokens, int32_t dx, int32_t dr, int32_t dtype, float epsilon,
                               int64_t num_slots, void *stream);

const char *atb_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif
