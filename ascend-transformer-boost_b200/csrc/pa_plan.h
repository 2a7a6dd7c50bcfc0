// Work decomposition shared by the host planner and the device kernels.
//
// The attention grid is n_cta_groups x cols CTAs.  A column is one kv head (or one chunk of the
// query heads of one kv head); a CTA group owns a contiguous slice of the global sequence of
// 64-token tiles, cut so that every group streams the same number of tiles (split-KV with exact
// balance).  All columns of a group walk the same token ranges, so the 8 kv-head slices of one
// cache page are read at about the same time.  A sequence cut into several ranges yields one fp32
// partial result per range; the range that finishes last merges them with their log-sum-exp weights
// (the CUDA-core and the MLA kernels leave that to the combine kernel).
//
// Stands in for the core-split / split-KV tiling of the reference
// (src/kernels/mixkernels/pagedattention/tiling/paged_attention_tiling_dependency.cpp:186-212, 406-521).
#ifndef ATB_B200_PA_PLAN_H
#define ATB_B200_PA_PLAN_H
#include <stdint.h>

namespace atb_b200 {

constexpr int kTileTokens = 64; // scheduling granule: token ranges start at multiples of it

// One contiguous token range of one sequence.  `slot` is the index of the partial result the range
// writes, or -1 when the range is the whole sequence and the kernel writes the final output.
struct PaItem {
    int32_t seq;
    int32_t tok_begin;
    int32_t tok_end;
    int32_t slot;
};

// Device view of a plan, passed by value to the kernels.
struct PaDevPlan {
    const int32_t *group_begin;   // [n_cta_groups + 1] offsets into items
    const PaItem *items;          // [n_items]
    const int32_t *seq_part_base; // [batch] first partial slot of a split sequence
    const int32_t *seq_nparts;    // [batch] 0 (empty), 1 (direct) or the number of partials
    const int32_t *combine_seqs;  // [n_combine_seqs] sequences with nparts > 1
    float *part_o;                // [n_partials, num_heads, dv] normalised partial outputs
    float *part_lse;              // [n_partials, num_heads] log2-domain log-sum-exp
    int32_t *status;              // device status word (0 = ok)
    int32_t *counters;            // [batch * cols] arrivals per (sequence, column), zero before the launch;
                                  // non-null = the last range to finish merges the partials itself
    int32_t *done_ctas;           // CTAs that have finished (zero before the launch); used by the
                                  // cross-GPU completion exchange
    int32_t n_cta_groups;
    int32_t cols;
};

// Kernel arguments common to all attention kernels.
struct PaArgs {
    const void *q;
    const void *k_cache;
    const void *v_cache;
    const int32_t *block_tables;
    const float *k_descale;
    const float *v_descale;
    const int32_t *k_offset;
    const int32_t *v_offset;
    const float *p_scale; // int8 query, offline quantisation of P: one scale per query head (else null)
    void *out;
    PaDevPlan plan;
    int32_t batch, num_heads, kv_heads, group; // group = num_heads / kv_heads
    int32_t dk, dv, v_row_dim, block_size, max_blocks, num_blocks;
    int32_t heads_per_cta, chunks_per_kvh;     // generic kernel: head chunking inside a kv head
    float scale_log2;                          // qk_scale * log2(e)
    // kv heads sharded over several GPUs: every rank's gathered output [tokens, out_total_heads, dv]
    // (peer-mapped memory); 0 peers = write `out` only
    void *out_peers[8];
    int32_t n_out_peers, out_total_heads, out_head_offset;
    // completion exchange: flag array (8 x uint32) of every rank, this rank, the step number
    uint32_t *peer_flags[8];
    int32_t xchg_rank;
    uint32_t xchg_epoch;
    uint32_t xchg_poll_limit; // polls before the wait for the peers gives up (0 = 2^22)
    // split MLA cache: rope parts of the query rows and of the cache rows (null = combined rows)
    const void *q_rope;
    const void *k_rope;
    // additive mask in the query dtype (score(b, h, t) += mask[b * mask_bs + h * mask_hs + t]) and per-sequence
    // factors of the scale; both null on the plain path
    const void *mask;
    int64_t mask_bs, mask_hs, mask_qs; // mask_qs: between the rows of a sequence's consecutive query tokens
    const int32_t *seq_lens;           // causal parallel decoding: context length of every sequence (else null)
    int32_t q_per_seq;                 // > 1: a CTA's columns are (query token, head) pairs of one sequence
    const float *logn;
    // parallel decoding: the block-table row and the mask row of every query token (null: the token's own index)
    const int32_t *bt_rows;
    const int32_t *mask_rows;
    void *lse_out;   // optional [batch, num_heads] natural-log LSE in the query dtype (MLA kernel + combine)
    int32_t kv_bnsd; // 1: caches laid out [num_blocks, kv_heads, block_size, dim]
    // optional event probe of one CTA (CTA number = trace_cap >> 24, capacity = its low 24 bits):
    // trace[0] = number of events, then (tag << 56 | index << 40 | cycles)
    unsigned long long *trace;
    uint32_t trace_cap;
};

__device__ __forceinline__ void probe(const PaArgs &a, unsigned tag, unsigned idx)
{
#ifdef __CUDA_ARCH__
    if (a.trace != nullptr && (a.trace_cap >> 24) != 255u && blockIdx.x == (a.trace_cap >> 24)) {
        const unsigned long long n = atomicAdd(a.trace, 1ull);
        if (n + 1 < (a.trace_cap & 0xffffffu)) {
            a.trace[n + 1] = ((unsigned long long)tag << 56) | ((unsigned long long)(idx & 0xffffu) << 40) |
                             ((unsigned long long)clock64() & 0xffffffffffull);
        }
    }
#endif
}

enum PaDeviceStatus : int32_t { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadBlockId = 2 };

} // namespace atb_b200
#endif
