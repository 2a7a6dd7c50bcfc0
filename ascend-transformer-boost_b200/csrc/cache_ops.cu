// BlockCopy, PagedCacheLoad and ReshapeAndCache over strided inputs: the cache-management siblings of
// ReshapeAndCache.
//   BlockCopy        copies whole cache blocks (beam search / prefix reuse); replaces
//                    src/kernels/mixkernels/blockcopy of the reference.
//   PagedCacheLoad   gathers a sequence's cached tokens back into contiguous rows; replaces
//                    src/kernels/mixkernels/paged_cache_load/op_kernel/paged_cache_load_nd.cpp.
//   ReshapeAndCache (strided)  the scatter of ReshapeAndCache reading rows that are `stride` apart (K/V
//                    slices of a fused QKV projection); replaces the strided mode of
//                    src/kernels/mixkernels/reshape_and_cache/op_kernel/reshape_and_cache_nd.cpp:70-128.
// HBM-bound byte movement: 16-byte vectors, one CTA per (block, chunk) so that a few hundred KB are
// in flight per SM.  The per-thread arithmetic lives in cache_ops_body.h, shared with the CPU tests.
#include <cuda_runtime.h>
#include "../../include/atb_b200.h"
#include "cache_ops_body.h"

namespace atb_b200 {
namespace {

constexpr int kErrInvalidParam = 1; // atb::ERROR_INVALID_PARAM
constexpr int kErrRtFail = 4;       // atb::ERROR_RT_FAIL
constexpr int kThreads = 256;
constexpr int64_t kChunkBytes = 32 * 1024; // target bytes one CTA moves per tensor

__global__ void __launch_bounds__(kThreads) block_copy_kernel(const BlockCopyArgs a)
{
    block_copy_body(a, blockIdx.x, threadIdx.x, blockDim.x);
}

__global__ void __launch_bounds__(kThreads) paged_cache_load_kernel(const PagedCacheLoadArgs a)
{
    paged_cache_load_body(a, blockIdx.x, threadIdx.x, blockDim.x);
}

__global__ void __launch_bounds__(kThreads) rac_strided_kernel(const RacStridedArgs a)
{
    rac_strided_body(a, blockIdx.x, threadIdx.x, blockDim.x);
}

__global__ void __launch_bounds__(kThreads) kv_cache_kernel(const KvCacheArgs a)
{
    kv_cache_body(a, blockIdx.x, threadIdx.x, blockDim.x);
}

__global__ void prefix_lens_kernel(const int32_t *lens, int32_t *cu, int32_t batch)
{
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        prefix_lens_body(lens, cu, batch);
    }
}

inline bool aligned16(const void *p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int32_t chunks_for(int64_t bytes)
{
    int64_t c = (bytes + kChunkBytes - 1) / kChunkBytes;
    return (int32_t)(c < 1 ? 1 : (c > 64 ? 64 : c));
}

} // namespace
} // namespace atb_b200

using namespace atb_b200;

extern "C" {

int atb_b200_block_copy(void *k_cache, void *v_cache, const int32_t *src_blocks, const int32_t *dst_blocks,
                        const int32_t *cum_sum, int32_t n_src, int32_t n_dst, int64_t k_block_bytes,
                        int64_t v_block_bytes, int64_t num_blocks, void *stream)
{
    if (k_cache == nullptr || src_blocks == nullptr || dst_blocks == nullptr || cum_sum == nullptr || n_src < 0 ||
        n_dst < 0 || k_block_bytes <= 0 || (v_cache != nullptr && v_block_bytes <= 0) || num_blocks <= 0) {
        return kErrInvalidParam;
    }
    if (n_src == 0 || n_dst == 0) {
        return 0;
    }
    BlockCopyArgs a{};
    a.k_cache = static_cast<uint8_t *>(k_cache);
    a.v_cache = static_cast<uint8_t *>(v_cache);
    a.src = src_blocks;
    a.dst = dst_blocks;
    a.cum = cum_sum;
    a.n_src = n_src;
    a.n_dst = n_dst;
    a.k_block_bytes = k_block_bytes;
    a.v_block_bytes = v_cache != nullptr ? v_block_bytes : 0;
    a.num_blocks = num_blocks;
    const int64_t larger = k_block_bytes > a.v_block_bytes ? k_block_bytes : a.v_block_bytes;
    a.chunks = chunks_for(larger);
    a.vec16 = aligned16(k_cache) && aligned16(v_cache) && k_block_bytes % 16 == 0 && a.v_block_bytes % 16 == 0;
    const int64_t ctas = (int64_t)n_dst * a.chunks;
    if (ctas > 0x7fffffff) {
        return kErrInvalidParam;
    }
    block_copy_kernel<<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : kErrRtFail;
}

uint64_t atb_b200_paged_cache_load_workspace_bytes(int32_t batch, int32_t lens_are_cumulative)
{
    if (batch <= 0 || lens_are_cumulative) {
        return 0;
    }
    return ((uint64_t)(batch + 1) * sizeof(int32_t) + 255) / 256 * 256;
}

int atb_b200_paged_cache_load(const void *k_cache, const void *v_cache, const int32_t *block_tables,
                              const int32_t *context_lens, const int32_t *seq_starts, void *key, void *value,
                              int32_t batch, int32_t table_cols, int32_t block_size, int64_t k_row_bytes,
                              int64_t v_row_bytes, int64_t num_blocks, int64_t out_rows, int32_t lens_are_cumulative,
                              void *workspace, uint64_t workspace_bytes, void *stream)
{
    if (k_cache == nullptr || block_tables == nullptr || context_lens == nullptr || key == nullptr || batch < 0 ||
        table_cols <= 0 || block_size <= 0 || k_row_bytes <= 0 || num_blocks <= 0 || out_rows < 0 ||
        ((v_cache == nullptr) != (value == nullptr)) || (v_cache != nullptr && v_row_bytes <= 0)) {
        return kErrInvalidParam;
    }
    if (batch == 0 || out_rows == 0) {
        return 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int32_t *cu = context_lens;
    if (!lens_are_cumulative) {
        if (workspace == nullptr || workspace_bytes < atb_b200_paged_cache_load_workspace_bytes(batch, 0) ||
            (reinterpret_cast<uintptr_t>(workspace) & 3u) != 0) {
            return kErrInvalidParam;
        }
        prefix_lens_kernel<<<1, 32, 0, s>>>(context_lens, static_cast<int32_t *>(workspace), batch);
        if (cudaGetLastError() != cudaSuccess) {
            return kErrRtFail;
        }
        cu = static_cast<const int32_t *>(workspace);
    }
    PagedCacheLoadArgs a{};
    a.k_cache = static_cast<const uint8_t *>(k_cache);
    a.v_cache = static_cast<const uint8_t *>(v_cache);
    a.block_tables = block_tables;
    a.cu_lens = cu;
    a.seq_starts = seq_starts;
    a.key = static_cast<uint8_t *>(key);
    a.value = static_cast<uint8_t *>(value);
    a.batch = batch;
    a.table_cols = table_cols;
    a.block_size = block_size;
    a.k_row_bytes = k_row_bytes;
    a.v_row_bytes = v_cache != nullptr ? v_row_bytes : 0;
    a.num_blocks = num_blocks;
    a.out_rows = out_rows;
    const int64_t larger = (k_row_bytes > a.v_row_bytes ? k_row_bytes : a.v_row_bytes) * block_size;
    a.chunks = chunks_for(larger);
    a.vec16 = aligned16(k_cache) && aligned16(v_cache) && aligned16(key) && aligned16(value) && k_row_bytes % 16 == 0 &&
              a.v_row_bytes % 16 == 0;
    const int64_t ctas = (int64_t)batch * table_cols * a.chunks;
    if (ctas > 0x7fffffff) {
        return kErrInvalidParam;
    }
    paged_cache_load_kernel<<<(unsigned)ctas, kThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : kErrRtFail;
}

int atb_b200_reshape_and_cache_strided(const void *key, const void *value, void *key_cache, void *value_cache,
                                       const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                                       int64_t v_row_bytes, int64_t k_token_stride_bytes, int64_t v_token_stride_bytes,
                                       int64_t num_slots, void *stream)
{
    if (key == nullptr || key_cache == nullptr || slot_mapping == nullptr || num_tokens < 0 || k_row_bytes <= 0 ||
        k_token_stride_bytes < 0 || num_slots <= 0 || ((value == nullptr) != (value_cache == nullptr)) ||
        (value != nullptr && (v_row_bytes <= 0 || v_token_stride_bytes < 0))) {
        return kErrInvalidParam;
    }
    if (num_tokens == 0) {
        return 0;
    }
    RacStridedArgs a{};
    a.key = static_cast<const uint8_t *>(key);
    a.value = static_cast<const uint8_t *>(value);
    a.key_cache = static_cast<uint8_t *>(key_cache);
    a.value_cache = static_cast<uint8_t *>(value_cache);
    a.slot_mapping = slot_mapping;
    a.num_tokens = num_tokens;
    a.k_row_bytes = k_row_bytes;
    a.v_row_bytes = value != nullptr ? v_row_bytes : 0;
    a.k_src_stride = k_token_stride_bytes;
    a.v_src_stride = value != nullptr ? v_token_stride_bytes : 0;
    a.num_slots = num_slots;
    a.chunks = chunks_for(k_row_bytes > a.v_row_bytes ? k_row_bytes : a.v_row_bytes);
    a.vec16 = aligned16(key) && aligned16(value) && aligned16(key_cache) && aligned16(value_cache) &&
              k_row_bytes % 16 == 0 && a.v_row_bytes % 16 == 0 && a.k_src_stride % 16 == 0 && a.v_src_stride % 16 == 0;
    const int64_t ctas = (int64_t)num_tokens * a.chunks;
    if (ctas > 0x7fffffff) {
        return kErrInvalidParam;
    }
    rac_strided_kernel<<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : kErrRtFail;
}

int atb_b200_kv_cache(const void *new_kv, const int32_t *layer_id, void *past, const int32_t *token_offset,
                      const int32_t *seq_len, int64_t num_tokens, int32_t layers, int32_t batch, int32_t max_seqlen,
                      int64_t row_bytes, void *stream)
{
    if (new_kv == nullptr || layer_id == nullptr || past == nullptr || token_offset == nullptr || seq_len == nullptr ||
        num_tokens < 0 || layers <= 0 || batch < 0 || max_seqlen <= 0 || row_bytes <= 0) {
        return kErrInvalidParam;
    }
    if (batch == 0 || num_tokens == 0) {
        return 0;
    }
    KvCacheArgs a{};
    a.new_kv = static_cast<const uint8_t *>(new_kv);
    a.past = static_cast<uint8_t *>(past);
    a.layer_id = layer_id;
    a.token_offset = token_offset;
    a.seq_len = seq_len;
    a.layers = layers;
    a.batch = batch;
    a.max_seqlen = max_seqlen;
    a.row_bytes = row_bytes;
    a.n_tokens = num_tokens;
    // the longest run a sequence can have: every row of new_kv, or a full cache row
    const int64_t longest = (num_tokens < max_seqlen ? num_tokens : (int64_t)max_seqlen) * row_bytes;
    // a sequence's run can be megabytes (prefill): cut it into ~32 KB chunks, up to 1024 per sequence, so that the
    // grid has enough CTAs in flight; chunks past the end of a shorter run return at once
    const int64_t want = (longest + kChunkBytes - 1) / kChunkBytes;
    a.chunks = (int32_t)(want < 1 ? 1 : (want > 1024 ? 1024 : want));
    a.vec16 = aligned16(new_kv) && aligned16(past) && row_bytes % 16 == 0;
    const int64_t ctas = (int64_t)batch * a.chunks;
    if (ctas > 0x7fffffff) {
        return kErrInvalidParam;
    }
    kv_cache_kernel<<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return cudaGetLastError() == cudaSuccess ? 0 : kErrRtFail;
}

} // extern "C"
