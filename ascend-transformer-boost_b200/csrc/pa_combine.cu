// Split-KV combine: merges the partial results of every sequence that was cut into several token
// ranges.  Each partial holds a normalised fp32 output and the log2-domain log-sum-exp of its
// range; the merge weight of partial i is 2^(lse_i - lse_max) / sum_j 2^(lse_j - lse_max), the
// same LSE merge as CombineScale in the reference
// (src/kernels/mixkernels/pagedattention/op_kernel/paged_attention_decoder_nd_common.cce:6568-6700).
#include "common.cuh"
#include "kernels.h"

namespace atb_b200 {
namespace {

constexpr int kMaxPartsShared = 512;

// One CTA per (split sequence, head); thread t owns output elements 4t..4t+3 (dv is a multiple of 4).
template <typename TQ>
__global__ void __launch_bounds__(160) pa_combine_kernel(const PaArgs a)
{
    __shared__ float w[kMaxPartsShared];
    // launched with programmatic stream serialisation right behind the attention kernel: wait for its
    // partials before reading anything
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int seq = a.plan.combine_seqs[blockIdx.x];
    const int h = blockIdx.y;
    const int base = a.plan.seq_part_base[seq];
    const int n = a.plan.seq_nparts[seq];
    const float *lse = a.plan.part_lse + (int64_t)base * a.num_heads + h;
    // Every load here is an L2 hit with ~1 us of latency and the kernel is nothing but such loads: they are issued in
    // batches (all log-sum-exps of up to kRegParts ranges at once, then four partial rows at once), never one by one.
    constexpr int kRegParts = 8;
    float lr[kRegParts];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kRegParts; ++i) {
        lr[i] = i < n ? lse[(int64_t)i * a.num_heads] : -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < kRegParts; ++i) {
        mx = fmaxf(mx, lr[i]);
    }
    for (int i = kRegParts; i < n; ++i) {
        mx = fmaxf(mx, lse[(int64_t)i * a.num_heads]);
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kRegParts; ++i) {
        lr[i] = exp2f(lr[i] - mx); // 0 for the ranges that do not exist
        sum += lr[i];
    }
    for (int i = kRegParts; i < n; ++i) {
        sum += exp2f(lse[(int64_t)i * a.num_heads] - mx);
    }
    const float inv = 1.f / sum;
    if (a.lse_out != nullptr && threadIdx.x == 0) {
        // log-sum-exp of the whole sequence from its ranges' (log2 domain), written as a natural log
        static_cast<TQ *>(a.lse_out)[(int64_t)seq * a.num_heads + h] =
            Elem<TQ>::from_float((mx + log2f(sum)) * 0.6931471805599453f);
    }
    const bool use_shared = n <= kMaxPartsShared;
    if (use_shared) {
#pragma unroll
        for (int i = 0; i < kRegParts; ++i) {
            if (threadIdx.x == 0 && i < n) {
                w[i] = lr[i] * inv;
            }
        }
        for (int i = kRegParts + threadIdx.x; i < n; i += blockDim.x) {
            w[i] = exp2f(lse[(int64_t)i * a.num_heads] - mx) * inv;
        }
        __syncthreads();
    }
    TQ *out = static_cast<TQ *>(a.out) + ((int64_t)seq * a.num_heads + h) * a.dv;
    const float *po = a.plan.part_o + ((int64_t)base * a.num_heads + h) * a.dv;
    const int64_t stride = (int64_t)a.num_heads * a.dv;
    for (int d = threadIdx.x * 4; d < a.dv; d += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i0 = 0; i0 < n; i0 += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                v[u] = *reinterpret_cast<const float4 *>(po + (int64_t)min(i0 + u, n - 1) * stride + d);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u;
                float wi = 0.f;
                if (i < n) {
                    wi = use_shared ? w[i] : exp2f(lse[(int64_t)i * a.num_heads] - mx) * inv;
                }
                acc.x = fmaf(wi, v[u].x, acc.x);
                acc.y = fmaf(wi, v[u].y, acc.y);
                acc.z = fmaf(wi, v[u].z, acc.z);
                acc.w = fmaf(wi, v[u].w, acc.w);
            }
        }
        uint2 pk;
        pk.x = Elem<TQ>::pack2(acc.x, acc.y);
        pk.y = Elem<TQ>::pack2(acc.z, acc.w);
        *reinterpret_cast<uint2 *>(out + d) = pk;
    }
}

} // namespace

cudaError_t launch_pa_combine(const PaArgs &args, int n_combine_seqs, int q_dtype, cudaStream_t stream)
{
    if (n_combine_seqs <= 0) {
        return cudaSuccess;
    }
    dim3 grid(n_combine_seqs, args.num_heads);
    const int threads = ((args.dv / 4 + 31) / 32 * 32) > 160 ? 160 : ((args.dv / 4 + 31) / 32 * 32);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (q_dtype == kFp16) {
        return cudaLaunchKernelEx(&cfg, pa_combine_kernel<__half>, args);
    }
    return cudaLaunchKernelEx(&cfg, pa_combine_kernel<__nv_bfloat16>, args);
}

} // namespace atb_b200
