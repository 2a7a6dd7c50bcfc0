// Per-thread bodies of the cache-management kernels (BlockCopy, PagedCacheLoad), written once for
// device and host: cache_ops.cu wraps them in __global__ kernels, and the CPU tests run the same
// index arithmetic over an emulated grid to check every address before a GPU ever sees it.
// Pure byte movement: bit-exact for every element type.
#ifndef ATB_B200_CACHE_OPS_BODY_H
#define ATB_B200_CACHE_OPS_BODY_H
#include <cstdint>

#if defined(__CUDACC__)
#define ATB_B200_HD __host__ __device__ __forceinline__
#else
#define ATB_B200_HD inline
#endif

namespace atb_b200 {

struct alignas(16) Bytes16 {
    uint64_t lo, hi;
};

// Thread `tid` of `nthreads` copies its share of bytes [begin, end) of src to dst.  With vec16 the
// caller guarantees that both pointers, begin and end are multiples of 16.
ATB_B200_HD void copy_range(uint8_t *dst, const uint8_t *src, int64_t begin, int64_t end, int tid, int nthreads,
                            bool vec16)
{
    if (vec16) {
        Bytes16 *d = reinterpret_cast<Bytes16 *>(dst);
        const Bytes16 *s = reinterpret_cast<const Bytes16 *>(src);
        for (int64_t i = begin / 16 + tid; i < end / 16; i += nthreads) {
            d[i] = s[i];
        }
    } else {
        for (int64_t i = begin + tid; i < end; i += nthreads) {
            dst[i] = src[i];
        }
    }
}

// Bytes [begin, end) of chunk `c` of `chunks` of a run of `bytes` bytes; chunk sizes are multiples of 16.
ATB_B200_HD void chunk_range(int64_t bytes, int32_t chunks, int32_t c, int64_t *begin, int64_t *end)
{
    int64_t per = (bytes + chunks - 1) / chunks;
    per = (per + 15) / 16 * 16;
    *begin = (int64_t)c * per;
    *end = *begin + per < bytes ? *begin + per : bytes;
}

// ---------------------------------------------------------------------------------------------------
// BlockCopy: destination block dst[j] receives source block src[i], where i is the source whose share
// [cum[i-1], cum[i]) of the destination list contains j (cum = running total of destinations per
// source).  One CTA per (destination, chunk).  Blocks outside the cache are skipped.
struct BlockCopyArgs {
    uint8_t *k_cache, *v_cache;        // v_cache may be null
    const int32_t *src, *dst, *cum;
    int32_t n_src, n_dst;
    int64_t k_block_bytes, v_block_bytes;
    int64_t num_blocks;
    int32_t chunks;
    bool vec16;
};

ATB_B200_HD void block_copy_body(const BlockCopyArgs &a, int64_t cta, int tid, int nthreads)
{
    const int32_t j = (int32_t)(cta / a.chunks), c = (int32_t)(cta % a.chunks);
    if (j >= a.n_dst) {
        return;
    }
    int32_t lo = 0, hi = a.n_src; // first i with cum[i] > j
    while (lo < hi) {
        const int32_t mid = lo + (hi - lo) / 2;
        if (a.cum[mid] > j) {
            hi = mid;
        } else {
            lo = mid + 1;
        }
    }
    if (lo >= a.n_src) {
        return; // j lies beyond the last running total
    }
    const int64_t s = a.src[lo], d = a.dst[j];
    if (s < 0 || s >= a.num_blocks || d < 0 || d >= a.num_blocks || s == d) {
        return;
    }
    int64_t begin, end;
    chunk_range(a.k_block_bytes, a.chunks, c, &begin, &end);
    if (begin < end) {
        copy_range(a.k_cache + d * a.k_block_bytes, a.k_cache + s * a.k_block_bytes, begin, end, tid, nthreads, a.vec16);
    }
    if (a.v_cache != nullptr) {
        chunk_range(a.v_block_bytes, a.chunks, c, &begin, &end);
        if (begin < end) {
            copy_range(a.v_cache + d * a.v_block_bytes, a.v_cache + s * a.v_block_bytes, begin, end, tid, nthreads,
                       a.vec16);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// PagedCacheLoad (ND caches): the reverse of ReshapeAndCache.  Sequence i owns output rows
// [cu[i], cu[i+1]); its tokens [t*block_size, ...) come from the cache block block_tables[i][off_i + t],
// off_i = seq_starts[i] / block_size.  One CTA per (sequence, table entry, chunk).  Negative or
// out-of-range block ids, table columns and output rows are skipped, never dereferenced.
struct PagedCacheLoadArgs {
    const uint8_t *k_cache, *v_cache;  // v_cache / value may be null
    const int32_t *block_tables;
    const int32_t *cu_lens;            // [batch + 1] running totals
    const int32_t *seq_starts;         // may be null
    uint8_t *key, *value;
    int32_t batch, table_cols, block_size;
    int64_t k_row_bytes, v_row_bytes;  // bytes of one token
    int64_t num_blocks, out_rows;
    int32_t chunks;
    bool vec16;
};

ATB_B200_HD void paged_cache_load_body(const PagedCacheLoadArgs &a, int64_t cta, int tid, int nthreads)
{
    const int32_t c = (int32_t)(cta % a.chunks);
    const int64_t entry = cta / a.chunks;
    const int32_t t = (int32_t)(entry % a.table_cols), i = (int32_t)(entry / a.table_cols);
    if (i >= a.batch) {
        return;
    }
    const int64_t start = a.cu_lens[i], len = (int64_t)a.cu_lens[i + 1] - start;
    const int64_t tok0 = (int64_t)t * a.block_size;
    if (len <= 0 || tok0 >= len) {
        return;
    }
    const int64_t ntok = len - tok0 < a.block_size ? len - tok0 : a.block_size;
    int64_t col = t;
    if (a.seq_starts != nullptr) {
        col += a.seq_starts[i] / a.block_size;
    }
    if (col < 0 || col >= a.table_cols) {
        return;
    }
    const int64_t blk = a.block_tables[(int64_t)i * a.table_cols + col];
    const int64_t row0 = start + tok0;
    if (blk < 0 || blk >= a.num_blocks || row0 < 0 || row0 + ntok > a.out_rows) {
        return;
    }
    int64_t begin, end;
    chunk_range(ntok * a.k_row_bytes, a.chunks, c, &begin, &end);
    if (begin < end) {
        copy_range(a.key + row0 * a.k_row_bytes, a.k_cache + blk * a.block_size * a.k_row_bytes, begin, end, tid, nthreads,
                   a.vec16);
    }
    if (a.v_cache != nullptr && a.value != nullptr) {
        chunk_range(ntok * a.v_row_bytes, a.chunks, c, &begin, &end);
        if (begin < end) {
            copy_range(a.value + row0 * a.v_row_bytes, a.v_cache + blk * a.block_size * a.v_row_bytes, begin, end, tid,
                       nthreads, a.vec16);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// ReshapeAndCache over strided inputs: token t's key row (heads x head size, contiguous) starts
// `k_src_stride` bytes after token t-1's, e.g. inside the output of a fused QKV projection; the row is
// scattered to cache slot slot_mapping[t] like ReshapeAndCache does.  One CTA per (token, chunk).
// Negative slots mean "do not store"; slots past the cache are dropped.
struct RacStridedArgs {
    const uint8_t *key, *value;        // first element of token 0's row (any view offset already applied)
    uint8_t *key_cache, *value_cache;  // value / value_cache may be null
    const int32_t *slot_mapping;
    int32_t num_tokens;
    int64_t k_row_bytes, v_row_bytes;
    int64_t k_src_stride, v_src_stride; // bytes between consecutive tokens' rows
    int64_t num_slots;
    int32_t chunks;
    bool vec16;
};

ATB_B200_HD void rac_strided_body(const RacStridedArgs &a, int64_t cta, int tid, int nthreads)
{
    const int32_t token = (int32_t)(cta / a.chunks), c = (int32_t)(cta % a.chunks);
    if (token >= a.num_tokens) {
        return;
    }
    const int64_t slot = a.slot_mapping[token];
    if (slot < 0 || slot >= a.num_slots) {
        return;
    }
    int64_t begin, end;
    chunk_range(a.k_row_bytes, a.chunks, c, &begin, &end);
    if (begin < end) {
        copy_range(a.key_cache + slot * a.k_row_bytes, a.key + token * a.k_src_stride, begin, end, tid, nthreads, a.vec16);
    }
    if (a.value != nullptr && a.value_cache != nullptr) {
        chunk_range(a.v_row_bytes, a.chunks, c, &begin, &end);
        if (begin < end) {
            copy_range(a.value_cache + slot * a.v_row_bytes, a.value + token * a.v_src_stride, begin, end, tid, nthreads,
                       a.vec16);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// KvCache (contiguous, per-layer cache [layers, batch, max_seqlen, hidden]): sequence b's seq_len[b] new rows,
// which follow those of the sequences before it in new_kv [tokens, hidden], go to positions
// [token_offset[b] - seq_len[b], token_offset[b]) of past[layer_id[0]][b] - one contiguous run on both sides.
// One CTA per (sequence, chunk).  A layer outside the cache, a negative length, a run that would start before
// position 0 or end past max_seqlen, and rows past the end of new_kv are skipped, never dereferenced.
struct KvCacheArgs {
    const uint8_t *new_kv;
    uint8_t *past;
    const int32_t *layer_id, *token_offset, *seq_len;
    int32_t layers, batch, max_seqlen;
    int64_t row_bytes;   // hidden size x element size
    int64_t n_tokens;    // rows of new_kv
    int32_t chunks;
    bool vec16;
};

ATB_B200_HD void kv_cache_body(const KvCacheArgs &a, int64_t cta, int tid, int nthreads)
{
    const int32_t b = (int32_t)(cta / a.chunks), c = (int32_t)(cta % a.chunks);
    if (b >= a.batch) {
        return;
    }
    const int64_t layer = a.layer_id[0], n = a.seq_len[b], off = a.token_offset[b];
    if (layer < 0 || layer >= a.layers || n <= 0 || off < n || off > a.max_seqlen) {
        return;
    }
    int64_t prefix = 0; // rows of the sequences before b (batch is small)
    for (int32_t i = 0; i < b; ++i) {
        prefix += a.seq_len[i] > 0 ? a.seq_len[i] : 0;
    }
    if (prefix + n > a.n_tokens) {
        return;
    }
    int64_t begin, end;
    chunk_range(n * a.row_bytes, a.chunks, c, &begin, &end);
    if (begin < end) {
        copy_range(a.past + ((layer * a.batch + b) * a.max_seqlen + off - n) * a.row_bytes, a.new_kv + prefix * a.row_bytes,
                   begin, end, tid, nthreads, a.vec16);
    }
}

// Running totals of the sequence lengths (one thread; batch is small): cu[0] = 0, cu[i+1] = cu[i] + lens[i].
ATB_B200_HD void prefix_lens_body(const int32_t *lens, int32_t *cu, int32_t batch)
{
    int32_t acc = 0;
    cu[0] = 0;
    for (int32_t i = 0; i < batch; ++i) {
        acc += lens[i] > 0 ? lens[i] : 0;
        cu[i + 1] = acc;
    }
}

} // namespace atb_b200
#endif
