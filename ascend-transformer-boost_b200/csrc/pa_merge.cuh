// Merge of the split-KV partials of one sequence inside an attention kernel, by the CTA that finishes the sequence
// last (the other CTAs have fenced their partials and counted themselves done).  Shared by the tiled kernels.
// Follows CombineScale of the reference (paged_attention_decoder_nd_common.cce:6568-6700): out = sum_i w_i O_i / sum_i w_i
// with w_i = 2^(lse_i - max lse).
#pragma once
#include "common.cuh"
#include "pa_plan.h"

namespace atb_b200 {

// 8 consecutive dims (from d0) of head h of the sequence whose partials start at index pbase; rows of row_dim floats.
// The partials come from L2: the loads are issued in batches of independent requests, or their latencies add up.
template <typename T>
__device__ __forceinline__ uint4 merge_partials8(const PaArgs &a, int pbase, int h, int d0, int row_dim, int n_parts)
{
    const float *lse = a.plan.part_lse + (int64_t)pbase * a.num_heads + h;
    const float *po = a.plan.part_o + ((int64_t)pbase * a.num_heads + h) * row_dim + d0;
    const int64_t lstride = a.num_heads, ostride = (int64_t)a.num_heads * row_dim;
    float mx = -INFINITY;
    for (int i0 = 0; i0 < n_parts; i0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = i0 + j < n_parts ? __ldcg(lse + (i0 + j) * lstride) : -INFINITY;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            mx = fmaxf(mx, v[j]);
        }
    }
    float wsum = 0.f;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i0 = 0; i0 < n_parts; i0 += 4) {
        float w[4];
        float4 pa[4], pb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const bool in = i0 + j < n_parts;
            const int i = in ? i0 + j : i0;
            w[j] = __ldcg(lse + i * lstride);
            pa[j] = __ldcg(reinterpret_cast<const float4 *>(po + i * ostride));
            pb[j] = __ldcg(reinterpret_cast<const float4 *>(po + i * ostride + 4));
            w[j] = in ? exp2f(w[j] - mx) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            wsum += w[j];
            acc[0] = fmaf(w[j], pa[j].x, acc[0]);
            acc[1] = fmaf(w[j], pa[j].y, acc[1]);
            acc[2] = fmaf(w[j], pa[j].z, acc[2]);
            acc[3] = fmaf(w[j], pa[j].w, acc[3]);
            acc[4] = fmaf(w[j], pb[j].x, acc[4]);
            acc[5] = fmaf(w[j], pb[j].y, acc[5]);
            acc[6] = fmaf(w[j], pb[j].z, acc[6]);
            acc[7] = fmaf(w[j], pb[j].w, acc[7]);
        }
    }
    const float inv = 1.f / wsum;
    uint4 pk;
    pk.x = Elem<T>::pack2(acc[0] * inv, acc[1] * inv);
    pk.y = Elem<T>::pack2(acc[2] * inv, acc[3] * inv);
    pk.z = Elem<T>::pack2(acc[4] * inv, acc[5] * inv);
    pk.w = Elem<T>::pack2(acc[6] * inv, acc[7] * inv);
    return pk;
}

} // namespace atb_b200
