// Fused RMSNorm + RoPE + cache write for the MLA latent cache: for every new token the normalised
// latent row (x * rsqrt(mean(x^2) + eps) * gamma, 512 wide) and the rotated rope row (64 wide) are
// written side by side into the token's cache slot, without a round trip of the new K through HBM.
// Replaces src/kernels/mixkernels/rms_norm_and_rope_and_reshape_and_cache of the reference; the
// arithmetic follows its CPU golden operation by operation in fp32
// (tests/apitest/kernelstest/mix/test_rms_norm_and_rope_and_reshape_and_cache.py:24-72):
//   rms  = 1 / sqrt(sum(x^2) / Dx + eps);  norm = (rms * x) * gamma
//   rope = k * cos + rotate_half(k) * sin,  rotate_half(k) = (-k[Dr/2:], k[:Dr/2])
// each rounded once to the storage type.  One CTA of 128 threads per token; a decode step has one
// token per sequence, so the kernel is latency-bound (about 2.4 KB read and 1.2 KB written per token).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "../../include/atb_b200.h"
#include "common.cuh"

namespace atb_b200 {
namespace {

constexpr int kErrInvalidParam = 1; // atb::ERROR_INVALID_PARAM
constexpr int kErrRtFail = 4;       // atb::ERROR_RT_FAIL
constexpr int kThreads = 128;

template <typename T>
__global__ void __launch_bounds__(kThreads) norm_rope_reshape_kernel(const T *__restrict__ x, const T *__restrict__ gamma,
                                                                     const T *__restrict__ key_rope,
                                                                     const T *__restrict__ cos_t,
                                                                     const T *__restrict__ sin_t,
                                                                     const int32_t *__restrict__ slot_mapping,
                                                                     T *__restrict__ key_cache, int32_t dx, int32_t dr,
                                                                     float epsilon, int64_t num_slots)
{
    __shared__ float warp_sums[kThreads / 32];
    const int token = blockIdx.x, tid = threadIdx.x;
    const int64_t slot = slot_mapping[token];
    if (slot < 0 || slot >= num_slots) {
        return; // negative = "do not store"; slots past the cache are dropped (the whole CTA leaves together)
    }
    const T *xr = x + (int64_t)token * dx;
    // explicit round-to-nearest operations: no fused multiply-add, so every product and sum rounds as in the golden
    float ss = 0.f;
    for (int i = tid; i < dx; i += kThreads) {
        const float v = Elem<T>::to_float(xr[i]);
        ss = __fadd_rn(ss, __fmul_rn(v, v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    }
    if ((tid & 31) == 0) {
        warp_sums[tid >> 5] = ss;
    }
    __syncthreads();
    float total = warp_sums[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) {
        total = __fadd_rn(total, warp_sums[w]);
    }
    const float rms = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)dx), epsilon)));
    T *row = key_cache + slot * (int64_t)(dx + dr);
    for (int i = tid; i < dx; i += kThreads) {
        const float v = Elem<T>::to_float(xr[i]);
        row[i] = Elem<T>::from_float(__fmul_rn(__fmul_rn(rms, v), Elem<T>::to_float(gamma[i])));
    }
    const int half = dr / 2;
    const T *kr = key_rope + (int64_t)token * dr, *cr = cos_t + (int64_t)token * dr, *sr = sin_t + (int64_t)token * dr;
    for (int j = tid; j < dr; j += kThreads) {
        const float k = Elem<T>::to_float(kr[j]);
        const float partner = j < half ? -Elem<T>::to_float(kr[j + half]) : Elem<T>::to_float(kr[j - half]);
        const float v = __fadd_rn(__fmul_rn(k, Elem<T>::to_float(cr[j])), __fmul_rn(partner, Elem<T>::to_float(sr[j])));
        row[dx + j] = Elem<T>::from_float(v);
    }
}

} // namespace
} // namespace atb_b200

using namespace atb_b200;

extern "C" int atb_b200_norm_rope_reshape(const void *x, const void *gamma, const void *key_rope, const void *cos_table,
                                          const void *sin_table, const int32_t *slot_mapping, void *key_cache,
                                          int32_t num_tokens, int32_t dx, int32_t dr, int32_t dtype, float epsilon,
                                          int64_t num_slots, void *stream)
{
    if (x == nullptr || gamma == nullptr || key_rope == nullptr || cos_table == nullptr || sin_table == nullptr ||
        slot_mapping == nullptr || key_cache == nullptr || num_tokens < 0 || dx <= 0 || dr <= 0 || dr % 2 != 0 ||
        num_slots <= 0 || !(epsilon > 0.f) || (dtype != ATB_B200_FP16 && dtype != ATB_B200_BF16)) {
        return kErrInvalidParam;
    }
    if (num_tokens == 0) {
        return 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ATB_B200_FP16) {
        norm_rope_reshape_kernel<__half><<<num_tokens, kThreads, 0, s>>>(
            static_cast<const __half *>(x), static_cast<const __half *>(gamma), static_cast<const __half *>(key_rope),
            static_cast<const __half *>(cos_table), static_cast<const __half *>(sin_table), slot_mapping,
            static_cast<__half *>(key_cache), dx, dr, epsilon, num_slots);
    } else {
        norm_rope_reshape_kernel<__nv_bfloat16><<<num_tokens, kThreads, 0, s>>>(
            static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(gamma),
            static_cast<const __nv_bfloat16 *>(key_rope), static_cast<const __nv_bfloat16 *>(cos_table),
            static_cast<const __nv_bfloat16 *>(sin_table), slot_mapping, static_cast<__nv_bfloat16 *>(key_cache), dx, dr,
            epsilon, num_slots);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : kErrRtFail;
}
