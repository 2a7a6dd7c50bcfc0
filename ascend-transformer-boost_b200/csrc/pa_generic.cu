// CUDA-core paged decode attention for any head size, block size and head grouping: the path for
// shapes the tiled kernels do not cover (head_dim != 128, small block sizes, more than 8 query
// heads per kv head, Dk != Dv, offsets with unusual layouts).
//
// One CTA (4 warps) per (CTA group, column); a column is up to GH query heads of one kv head.  The
// warps take tokens round-robin, every lane owns 4 consecutive elements of each 128-wide slice of
// the row, scores are reduced with warp shuffles and each warp keeps its own online-softmax state
// (running max, sum, fp32 output), merged through shared memory at the end of the token range.
//
// Arithmetic follows the reference golden (tests/apitest/kernelstest/mix/test_paged_attention_common.py
// :229-276 of the reference): fp32 dot products, score * scale, fp32 softmax, fp32 P*V; the int8
// cache is dequantised as (float(x) + offset) * scale before use (:89-103).
#include "common.cuh"
#include "kernels.h"

namespace atb_b200 {
namespace {

constexpr int kWarps = 4;

template <typename TQ, typename TKV, int GH, int NPK, int NPV>
__global__ void __launch_bounds__(kWarps * 32) pa_generic_kernel(const PaArgs a)
{
    constexpr bool kInt8 = sizeof(TKV) == 1;
    extern __shared__ float smem[];
    float *sm_o = smem;                              // [kWarps][GH][NPV*128]
    float *sm_m = sm_o + kWarps * GH * NPV * 128;    // [kWarps][GH]
    float *sm_l = sm_m + kWarps * GH;                // [kWarps][GH]

    const int cols = a.plan.cols;
    const int grp = blockIdx.x / cols;
    const int col = blockIdx.x - grp * cols;
    const int kvh = col / a.chunks_per_kvh;
    const int chunk = col - kvh * a.chunks_per_kvh;
    const int head0 = kvh * a.group + chunk * GH;
    const int nh = min(GH, a.group - chunk * GH);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TQ *q = static_cast<const TQ *>(a.q);
    const TKV *kc = static_cast<const TKV *>(a.k_cache);
    const TKV *vc = static_cast<const TKV *>(a.v_cache);
    TQ *out = static_cast<TQ *>(a.out);

    // per-lane dequant constants of this kv head (int8 cache only)
    float ksc[NPK][4], kof[NPK][4], vsc[NPV][4], vof[NPV][4];
    if (kInt8) {
#pragma unroll
        for (int p = 0; p < NPK; ++p) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int e = p * 128 + lane * 4 + j;
                bool in = e < a.dk;
                ksc[p][j] = (in && a.k_descale) ? a.k_descale[kvh * a.dk + e] : 1.f;
                kof[p][j] = (in && a.k_offset) ? (float)a.k_offset[kvh * a.dk + e] : 0.f;
            }
        }
#pragma unroll
        for (int p = 0; p < NPV; ++p) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int e = p * 128 + lane * 4 + j;
                bool in = e < a.dv;
                vsc[p][j] = (in && a.v_descale) ? a.v_descale[kvh * a.dv + e] : 1.f;
                vof[p][j] = (in && a.v_offset) ? (float)a.v_offset[kvh * a.dv + e] : 0.f;
            }
        }
    }

    const int item_begin = a.plan.group_begin[grp], item_end = a.plan.group_begin[grp + 1];
    for (int it = item_begin; it < item_end; ++it) {
        const PaItem item = a.plan.items[it];
        float qr[GH][NPK][4];
#pragma unroll
        for (int g = 0; g < GH; ++g) {
#pragma unroll
            for (int p = 0; p < NPK; ++p) {
                int e = p * 128 + lane * 4;
                if (g < nh && e < a.dk) {
                    load4<TQ>(q + ((int64_t)item.seq * a.num_heads + head0 + g) * a.dk + e, qr[g][p]);
                } else {
                    qr[g][p][0] = qr[g][p][1] = qr[g][p][2] = qr[g][p][3] = 0.f;
                }
            }
        }
        float m[GH], l[GH], o[GH][NPV][4];
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.f;
#pragma unroll
            for (int p = 0; p < NPV; ++p) {
                o[g][p][0] = o[g][p][1] = o[g][p][2] = o[g][p][3] = 0.f;
            }
        }
        const int32_t *bt = a.block_tables + (int64_t)(a.bt_rows != nullptr ? a.bt_rows[item.seq] : item.seq) * a.max_blocks;
        // SCALE_TYPE_LOGN: the sequence's factor multiplies the scale; additive mask in the query dtype
        const float scale_l2 = a.logn != nullptr ? a.scale_log2 * __ldg(a.logn + item.seq) : a.scale_log2;
        const TQ *mrow = a.mask == nullptr ? nullptr
                                           : static_cast<const TQ *>(a.mask) +
                                                 (int64_t)(a.mask_rows != nullptr ? a.mask_rows[item.seq] : item.seq) * a.mask_bs +
                                                 (int64_t)head0 * a.mask_hs;
        for (int t = item.tok_begin + warp; t < item.tok_end; t += kWarps) {
            const int64_t blk = bt[t / a.block_size];
            if (blk < 0 || blk >= a.num_blocks) {
                // a block id outside the cache: record it and leave the token out instead of faulting
                if (lane == 0) {
                    atomicExch(a.plan.status, kStatusBadBlockId);
                }
                continue;
            }
            // row of (block, token, kv head): token-major blocks, or heads-major ones (BNSD)
            const int64_t row = a.kv_bnsd ? (blk * a.kv_heads + kvh) * a.block_size + (t % a.block_size)
                                          : (blk * a.block_size + (t % a.block_size)) * a.kv_heads + kvh;
            const TKV *kp = kc + row * a.dk;
            const TKV *vp = vc + row * a.v_row_dim;
            float kf[NPK][4], vf[NPV][4];
#pragma unroll
            for (int p = 0; p < NPK; ++p) {
                int e = p * 128 + lane * 4;
                if (e < a.dk) {
                    load4<TKV>(kp + e, kf[p]);
                } else {
                    kf[p][0] = kf[p][1] = kf[p][2] = kf[p][3] = 0.f;
                }
            }
#pragma unroll
            for (int p = 0; p < NPV; ++p) {
                int e = p * 128 + lane * 4;
                if (e < a.dv) {
                    load4<TKV>(vp + e, vf[p]);
                } else {
                    vf[p][0] = vf[p][1] = vf[p][2] = vf[p][3] = 0.f;
                }
            }
            if (kInt8) {
#pragma unroll
                for (int p = 0; p < NPK; ++p) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        kf[p][j] = (kf[p][j] + kof[p][j]) * ksc[p][j];
                    }
                }
#pragma unroll
                for (int p = 0; p < NPV; ++p) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        vf[p][j] = (vf[p][j] + vof[p][j]) * vsc[p][j];
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < GH; ++g) {
                float acc = 0.f;
#pragma unroll
                for (int p = 0; p < NPK; ++p) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc = fmaf(qr[g][p][j], kf[p][j], acc);
                    }
                }
                acc = warp_sum(acc);
                float s = acc * scale_l2;
                if (mrow != nullptr && g < nh) {
                    // a mask of -inf must not turn the running maximum into -inf (exp2(-inf - -inf) = NaN)
                    s = fmaxf(s + 1.4426950408889634f * Elem<TQ>::to_float(mrow[(int64_t)g * a.mask_hs + t]), -1e30f);
                }
                const float m_new = fmaxf(m[g], s);
                const float corr = exp2f(m[g] - m_new);
                const float pr = exp2f(s - m_new);
                m[g] = m_new;
                l[g] = l[g] * corr + pr;
#pragma unroll
                for (int p = 0; p < NPV; ++p) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        o[g][p][j] = fmaf(pr, vf[p][j], o[g][p][j] * corr);
                    }
                }
            }
        }
        // merge the warps' states
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            if (lane == 0) {
                sm_m[warp * GH + g] = m[g];
                sm_l[warp * GH + g] = l[g];
            }
#pragma unroll
            for (int p = 0; p < NPV; ++p) {
                float4 v = make_float4(o[g][p][0], o[g][p][1], o[g][p][2], o[g][p][3]);
                *reinterpret_cast<float4 *>(sm_o + ((warp * GH + g) * NPV + p) * 128 + lane * 4) = v;
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nh * a.dv; idx += kWarps * 32) {
            const int g = idx / a.dv, d = idx - g * a.dv;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                mm = fmaxf(mm, sm_m[w * GH + g]);
            }
            float ll = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float f = exp2f(sm_m[w * GH + g] - mm);
                ll += sm_l[w * GH + g] * f;
                acc += sm_o[(w * GH + g) * NPV * 128 + d] * f;
            }
            const float val = acc / ll;
            const int h = head0 + g;
            if (item.slot < 0) {
                out[((int64_t)item.seq * a.num_heads + h) * a.dv + d] = Elem<TQ>::from_float(val);
            } else {
                a.plan.part_o[((int64_t)item.slot * a.num_heads + h) * a.dv + d] = val;
                if (d == 0) {
                    a.plan.part_lse[(int64_t)item.slot * a.num_heads + h] = mm + log2f(ll);
                }
            }
        }
        __syncthreads();
    }
}

template <typename TQ, typename TKV, int GH, int NPK, int NPV>
cudaError_t launch_one(const PaArgs &args, cudaStream_t stream)
{
    const size_t smem = sizeof(float) * (kWarps * GH * NPV * 128 + 2 * kWarps * GH);
    auto kern = pa_generic_kernel<TQ, TKV, GH, NPK, NPV>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            return e;
        }
    }
    const int grid = args.plan.n_cta_groups * args.plan.cols;
    kern<<<grid, kWarps * 32, smem, stream>>>(args);
    return cudaGetLastError();
}

template <typename TQ, typename TKV> cudaError_t launch_sized(const PaArgs &a, cudaStream_t s)
{
    const int dmax = a.dk > a.dv ? a.dk : a.dv;
    if (dmax <= 128) {
        return launch_one<TQ, TKV, 8, 1, 1>(a, s);
    }
    if (dmax <= 256) {
        return launch_one<TQ, TKV, 4, 2, 2>(a, s);
    }
    if constexpr (sizeof(TKV) == 1) {
        return cudaErrorInvalidValue; // int8 caches are limited to head_dim <= 256
    } else {
        return launch_one<TQ, TKV, 2, 5, 5>(a, s);
    }
}

} // namespace

int pa_generic_heads_per_cta(int dk, int dv)
{
    const int dmax = dk > dv ? dk : dv;
    return dmax <= 128 ? 8 : (dmax <= 256 ? 4 : 2);
}

bool pa_generic_supported(int dk, int dv, int q_dtype, int kv_dtype)
{
    if (dk <= 0 || dv <= 0 || dk > 640 || dv > 640 || dk % 4 != 0 || dv % 4 != 0) {
        return false;
    }
    if (q_dtype != kFp16 && q_dtype != kBf16) {
        return false;
    }
    if (kv_dtype == kInt8) {
        return dk <= 256 && dv <= 256;
    }
    return kv_dtype == q_dtype;
}

cudaError_t launch_pa_generic(const PaArgs &args, int q_dtype, int kv_dtype, cudaStream_t stream)
{
    if (q_dtype == kFp16) {
        return kv_dtype == kInt8 ? launch_sized<__half, int8_t>(args, stream) : launch_sized<__half, __half>(args, stream);
    }
    return kv_dtype == kInt8 ? launch_sized<__nv_bfloat16, int8_t>(args, stream)
                             : launch_sized<__nv_bfloat16, __nv_bfloat16>(args, stream);
}

} // namespace atb_b200
