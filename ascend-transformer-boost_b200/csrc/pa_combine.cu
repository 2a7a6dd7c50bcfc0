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
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) {
        mx = fmaxf(mx, lse[(int64_t)i * a.num_heads]);
    }
    float sum = 0.f;
    for (int i = 0; i < n; ++i) {
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
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            w[i] = exp2f(lse[(int64_t)i * a.num_heads] - mx) * inv;
        }
        __syncthreads();
    }
    TQ *out = static_cast<TQ *>(a.out) + ((int64_t)seq * a.num_heads + h) * a.dv;
    const float *po = a.plan.part_o + ((int64_t)base * a.num_heads + h) * a.dv;
    const int64_t stride = (int64_t)a.num_heads * a.dv;
    for (int d = threadIdx.x * 4; d < a.dv; d += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < n; ++i) {
            const float wi = use_shared ? w[i] : exp2f(lse[(int64_t)i * a.num_heads] - mx) * inv;
            const float4 v = *reinterpret_cast<const float4 *>(po + i * stride + d);
            acc.x = fmaf(wi, v.x, acc.x);
            acc.y = fmaf(wi, v.y, acc.y);
            acc.z = fmaf(wi, v.z, acc.z);
            acc.w = fmaf(wi, v.w, acc.w);
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
