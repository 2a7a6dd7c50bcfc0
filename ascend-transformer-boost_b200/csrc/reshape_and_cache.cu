// ReshapeAndCache: scatter the new tokens' K/V rows into the block-paged cache.
// cache[slot] = row(token) for slot = slot_mapping[token] >= 0; negative slots are skipped, as in
// op_kernel/reshape_and_cache_nd.cpp:91-128 and reshape_and_cache_base.h:104-118 of the reference.
// Pure byte copy (bit-exact for fp16 / bf16 / int8); HBM- and latency-bound.
#include "kernels.h"

namespace atb_b200 {
namespace {

template <typename V>
__global__ void __launch_bounds__(256) reshape_and_cache_kernel(const uint8_t *__restrict__ key,
                                                                const uint8_t *__restrict__ value,
                                                                uint8_t *__restrict__ key_cache,
                                                                uint8_t *__restrict__ value_cache,
                                                                const int32_t *__restrict__ slot_mapping,
                                                                int64_t k_row_bytes, int64_t v_row_bytes,
                                                                int64_t num_slots)
{
    // lets a dependent kernel launched with programmatic stream serialisation (the attention kernel)
    // begin its prologue now; it still waits for this grid to finish before it reads the cache
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int token = blockIdx.x;
    const int64_t slot = slot_mapping[token];
    if (slot < 0 || slot >= num_slots) {
        return; // negative = "do not store"; out-of-range slots are dropped rather than written
    }
    const int64_t kv = k_row_bytes / (int64_t)sizeof(V);
    const int64_t vv = v_row_bytes / (int64_t)sizeof(V);
    const int64_t stride = (int64_t)blockDim.x * gridDim.y;
    const int64_t start = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
    if (key != nullptr) {
        const V *src = reinterpret_cast<const V *>(key + (int64_t)token * k_row_bytes);
        V *dst = reinterpret_cast<V *>(key_cache + slot * k_row_bytes);
        for (int64_t i = start; i < kv; i += stride) {
            dst[i] = src[i];
        }
    }
    if (value != nullptr) {
        const V *src = reinterpret_cast<const V *>(value + (int64_t)token * v_row_bytes);
        V *dst = reinterpret_cast<V *>(value_cache + slot * v_row_bytes);
        for (int64_t i = start; i < vv; i += stride) {
            dst[i] = src[i];
        }
    }
}

inline bool aligned(const void *p, uintptr_t a) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % a) == 0; }

} // namespace

cudaError_t launch_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                                     const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                                     int64_t v_row_bytes, int64_t num_slots, cudaStream_t stream)
{
    if (num_tokens <= 0) {
        return cudaSuccess;
    }
    if (key == nullptr || key_cache == nullptr) {
        k_row_bytes = 0;
        key = nullptr;
    }
    if (value == nullptr || value_cache == nullptr) {
        v_row_bytes = 0;
        value = nullptr;
    }
    const int64_t max_row = k_row_bytes > v_row_bytes ? k_row_bytes : v_row_bytes;
    auto fits = [&](int64_t w) {
        return k_row_bytes % w == 0 && v_row_bytes % w == 0 && aligned(key, w) && aligned(value, w) &&
               aligned(key_cache, w) && aligned(value_cache, w);
    };
    const uint8_t *k = static_cast<const uint8_t *>(key), *v = static_cast<const uint8_t *>(value);
    uint8_t *kc = static_cast<uint8_t *>(key_cache), *vc = static_cast<uint8_t *>(value_cache);
    if (fits(16)) {
        int64_t vecs = max_row / 16;
        dim3 grid(num_tokens, (unsigned)((vecs + 255) / 256 > 8 ? 8 : (vecs + 255) / 256 > 0 ? (vecs + 255) / 256 : 1));
        reshape_and_cache_kernel<uint4><<<grid, 256, 0, stream>>>(k, v, kc, vc, slot_mapping, k_row_bytes,
                                                                   v_row_bytes, num_slots);
    } else if (fits(4)) {
        dim3 grid(num_tokens, 1);
        reshape_and_cache_kernel<uint32_t><<<grid, 256, 0, stream>>>(k, v, kc, vc, slot_mapping, k_row_bytes,
                                                                      v_row_bytes, num_slots);
    } else if (fits(2)) {
        dim3 grid(num_tokens, 1);
        reshape_and_cache_kernel<uint16_t><<<grid, 256, 0, stream>>>(k, v, kc, vc, slot_mapping, k_row_bytes,
                                                                      v_row_bytes, num_slots);
    } else {
        dim3 grid(num_tokens, 1);
        reshape_and_cache_kernel<uint8_t><<<grid, 256, 0, stream>>>(k, v, kc, vc, slot_mapping, k_row_bytes,
                                                                     v_row_bytes, num_slots);
    }
    return cudaGetLastError();
}

} // namespace atb_b200
