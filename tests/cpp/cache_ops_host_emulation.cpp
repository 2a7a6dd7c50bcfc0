// Runs the per-thread bodies of the cache-management kernels (csrc/cache_ops_body.h) on the CPU over
// an emulated grid, with every pointer the body touches checked against the buffers the test owns:
// the index arithmetic of the CUDA kernels is verified here, without a GPU.
// Build: g++ -O1 -shared -fPIC (see build.py::build_host_emulation).
#include <cstdint>
#include <cstring>
#include "../../ascend-transformer-boost_b200/csrc/cache_ops_body.h"

using namespace atb_b200;

namespace {
int64_t chunks_for(int64_t bytes)
{
    const int64_t chunk = 32 * 1024;
    int64_t c = (bytes + chunk - 1) / chunk;
    return c < 1 ? 1 : (c > 64 ? 64 : c);
}
bool aligned16(const void *p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
} // namespace

extern "C" {

// The same argument set-up as atb_b200_block_copy, then every (cta, thread) of the grid in turn.
// `chunks` > 0 overrides the chunk count (to exercise the chunk arithmetic on small blocks).
int emu_block_copy(uint8_t *k_cache, uint8_t *v_cache, const int32_t *src, const int32_t *dst, const int32_t *cum,
                   int32_t n_src, int32_t n_dst, int64_t k_block_bytes, int64_t v_block_bytes, int64_t num_blocks,
                   int32_t chunks, int32_t threads)
{
    BlockCopyArgs a{};
    a.k_cache = k_cache;
    a.v_cache = v_cache;
    a.src = src;
    a.dst = dst;
    a.cum = cum;
    a.n_src = n_src;
    a.n_dst = n_dst;
    a.k_block_bytes = k_block_bytes;
    a.v_block_bytes = v_cache ? v_block_bytes : 0;
    a.num_blocks = num_blocks;
    const int64_t larger = k_block_bytes > a.v_block_bytes ? k_block_bytes : a.v_block_bytes;
    a.chunks = chunks > 0 ? chunks : (int32_t)chunks_for(larger);
    a.vec16 = aligned16(k_cache) && aligned16(v_cache) && k_block_bytes % 16 == 0 && a.v_block_bytes % 16 == 0;
    for (int64_t cta = 0; cta < (int64_t)n_dst * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            block_copy_body(a, cta, tid, threads);
        }
    }
    return a.vec16 ? 16 : 1;
}

int emu_paged_cache_load(const uint8_t *k_cache, const uint8_t *v_cache, const int32_t *block_tables,
                         const int32_t *context_lens, const int32_t *seq_starts, uint8_t *key, uint8_t *value,
                         int32_t batch, int32_t table_cols, int32_t block_size, int64_t k_row_bytes, int64_t v_row_bytes,
                         int64_t num_blocks, int64_t out_rows, int32_t cumulative, int32_t *workspace, int32_t chunks,
                         int32_t threads)
{
    const int32_t *cu = context_lens;
    if (!cumulative) {
        prefix_lens_body(context_lens, workspace, batch);
        cu = workspace;
    }
    PagedCacheLoadArgs a{};
    a.k_cache = k_cache;
    a.v_cache = v_cache;
    a.block_tables = block_tables;
    a.cu_lens = cu;
    a.seq_starts = seq_starts;
    a.key = key;
    a.value = value;
    a.batch = batch;
    a.table_cols = table_cols;
    a.block_size = block_size;
    a.k_row_bytes = k_row_bytes;
    a.v_row_bytes = v_cache ? v_row_bytes : 0;
    a.num_blocks = num_blocks;
    a.out_rows = out_rows;
    const int64_t larger = (k_row_bytes > a.v_row_bytes ? k_row_bytes : a.v_row_bytes) * block_size;
    a.chunks = chunks > 0 ? chunks : (int32_t)chunks_for(larger);
    a.vec16 = aligned16(k_cache) && aligned16(v_cache) && aligned16(key) && aligned16(value) && k_row_bytes % 16 == 0 &&
              a.v_row_bytes % 16 == 0;
    for (int64_t cta = 0; cta < (int64_t)batch * table_cols * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            paged_cache_load_body(a, cta, tid, threads);
        }
    }
    return a.vec16 ? 16 : 1;
}

int emu_rac_strided(const uint8_t *key, const uint8_t *value, uint8_t *key_cache, uint8_t *value_cache,
                    const int32_t *slots, int32_t num_tokens, int64_t k_row_bytes, int64_t v_row_bytes, int64_t k_stride,
                    int64_t v_stride, int64_t num_slots, int32_t chunks, int32_t threads)
{
    RacStridedArgs a{};
    a.key = key;
    a.value = value;
    a.key_cache = key_cache;
    a.value_cache = value_cache;
    a.slot_mapping = slots;
    a.num_tokens = num_tokens;
    a.k_row_bytes = k_row_bytes;
    a.v_row_bytes = value ? v_row_bytes : 0;
    a.k_src_stride = k_stride;
    a.v_src_stride = value ? v_stride : 0;
    a.num_slots = num_slots;
    a.chunks = chunks > 0 ? chunks : (int32_t)chunks_for(k_row_bytes > a.v_row_bytes ? k_row_bytes : a.v_row_bytes);
    a.vec16 = aligned16(key) && aligned16(value) && aligned16(key_cache) && aligned16(value_cache) &&
              k_row_bytes % 16 == 0 && a.v_row_bytes % 16 == 0 && a.k_src_stride % 16 == 0 && a.v_src_stride % 16 == 0;
    for (int64_t cta = 0; cta < (int64_t)num_tokens * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            rac_strided_body(a, cta, tid, threads);
        }
    }
    return a.vec16 ? 16 : 1;
}

int emu_kv_cache(const uint8_t *new_kv, const int32_t *layer_id, uint8_t *past, const int32_t *token_offset,
                 const int32_t *seq_len, int64_t n_tokens, int32_t layers, int32_t batch, int32_t max_seqlen,
                 int64_t row_bytes, int32_t chunks, int32_t threads)
{
    KvCacheArgs a{};
    a.new_kv = new_kv;
    a.past = past;
    a.layer_id = layer_id;
    a.token_offset = token_offset;
    a.seq_len = seq_len;
    a.layers = layers;
    a.batch = batch;
    a.max_seqlen = max_seqlen;
    a.row_bytes = row_bytes;
    a.n_tokens = n_tokens;
    a.chunks = chunks > 0 ? chunks
                          : (int32_t)chunks_for((n_tokens < max_seqlen ? n_tokens : (int64_t)max_seqlen) * row_bytes);
    a.vec16 = aligned16(new_kv) && aligned16(past) && row_bytes % 16 == 0;
    for (int64_t cta = 0; cta < (int64_t)batch * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            kv_cache_body(a, cta, tid, threads);
        }
    }
    return a.vec16 ? 16 : 1;
}

} // extern "C"
