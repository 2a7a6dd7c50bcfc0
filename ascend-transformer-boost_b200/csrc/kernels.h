// Host-side launchers of the CUDA kernels (internal to the library).
#ifndef ATB_B200_KERNELS_H
#define ATB_B200_KERNELS_H
#include <cuda_runtime.h>
#include "pa_plan.h"

namespace atb_b200 {

enum DType : int { kFp16 = 0, kBf16 = 1, kInt8 = 2 };

cudaError_t launch_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                                     const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                                     int64_t v_row_bytes, int64_t num_slots, cudaStream_t stream);

// CUDA-core decode attention for any head size / block size / head grouping.
bool pa_generic_supported(int dk, int dv, int q_dtype, int kv_dtype);
int pa_generic_heads_per_cta(int dk, int dv);
cudaError_t launch_pa_generic(const PaArgs &args, int q_dtype, int kv_dtype, cudaStream_t stream);

// TMA page gather + mma.sync tiles: D = 128, block_size 16 / 32 / 64 / 128 / 256, fp16 / bf16 cache.
bool pa_tma_mma_supported(int dk, int dv, int v_row_dim, int block_size, int group, int q_dtype, int kv_dtype);
cudaError_t launch_pa_tma_mma(const PaArgs &args, int q_dtype, int kv_dtype, int num_blocks, cudaStream_t stream);

// The same for an int8 cache with per-channel descale (and optional offsets).
bool pa_tma_mma_i8_supported(int dk, int dv, int v_row_dim, int block_size, int group, int q_dtype, int kv_dtype);
cudaError_t launch_pa_tma_mma_i8(const PaArgs &args, int q_dtype, int num_blocks, cudaStream_t stream);

// int8 query, int8 cache (QKV quantisation): both contractions on the integer tensor cores; k_descale, v_descale
// (and p_scale for the offline form) hold one fp32 value per query head.  `out_dtype` is fp16 or bf16.
bool pa_tma_mma_q8_supported(int dk, int dv, int v_row_dim, int block_size, int group, int out_dtype);
cudaError_t launch_pa_tma_mma_q8(const PaArgs &args, int out_dtype, int num_blocks, cudaStream_t stream);

// MLA combined cache (Dk 576, Dv 512, one kv head): TMA + tcgen05/TMEM, 64 query heads per CTA.
bool pa_mla_tc5_supported(int dk, int dv, int v_row_dim, int rope_dim, int block_size, int kv_heads, int q_dtype,
                          int kv_dtype);
cudaError_t launch_pa_mla_tc5(const PaArgs &args, int q_dtype, int num_blocks, cudaStream_t stream);

// The same cache as a cluster of two CTAs per 128 heads that split the 576 dims (bf16, no mask): heads in M, Q and P in
// tensor memory; the grid is 2 x n_cta_groups x cols CTAs.
bool pa_mla_pair_supported(int dk, int dv, int v_row_dim, int rope_dim, int block_size, int kv_heads, int q_dtype, int kv_dtype);
cudaError_t launch_pa_mla_pair(const PaArgs &args, int num_blocks, cudaStream_t stream);
int pa_mla_pair_max_pairs(); // CTA pairs resident at once on the current device (0: unknown)

// Merges the split-KV partials of every split sequence into the output.
cudaError_t launch_pa_combine(const PaArgs &args, int n_combine_seqs, int q_dtype, cudaStream_t stream);

} // namespace atb_b200
#endif
