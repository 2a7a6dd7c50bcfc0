// Paged decode attention over an int8 KV cache with per-channel dequantisation
// (quantType TYPE_DEQUANT_FUSION), head_dim 128 / block_size 16, 32, 64, 128 or 256, up to 8 query heads per kv head.
//
// Same structure as the fp16/bf16 kernel in pa_tma_mma.cu (TMA page gather into a shared-memory
// ring, four consumer warps with independent online-softmax states, split-KV partials), with the
// cache kept int8 all the way into registers:
//   * a stage is 64 tokens x 128 B of K plus the same of V (16 KB), six stages deep;
//   * the per-channel scales commute with the contractions, so K is never multiplied:
//     sum_d q_d (k_td + off_d) s_d = sum_d (q_d s_d) k_td + const(head), and the constant does not
//     change the softmax; Q is pre-scaled by kDescale once per token range.  Likewise
//     out_d = vDescale_d * (sum_t p_t v_td / l + vOffset_d), applied when the range is written;
//   * int8 -> fp16 is exact and done with byte permutes: (x ^ 0x80) placed in the mantissa of
//     1024.0 gives 1152 + x; the bias is never subtracted from the operands (three ALU instructions
//     per four cache bytes): it cancels in the softmax for K and is taken out of the accumulated
//     output once per token range for V.  ldmatrix moves byte pairs, so the k index of Q.K^T and
//     the row index of V^T.P^T are permuted consistently between the two operands;
//   * the tensor-core tiles run in fp16 for both fp16 and bf16 queries (P in fp16 is at least as
//     precise as the golden's rounding of P to the query dtype).
//
// kQ8 (quantType TYPE_QUANT_QKV_ONLINE / OFFLINE: the query is int8 too) runs both contractions on the integer
// tensor cores: S^T = K . Q^T as mma m16n8k32 s8 x s8 -> s32 straight from the ldmatrix registers (no conversion
// at all), the probabilities of a warp's 16 tokens quantised to int8 - online: 127 * 2^(s - max of those 16),
// i.e. relative to the tile's own maximum, weight 2^(tile max - running max) applied to the tile's int32 P.V
// result; offline: p * pScale[head] - and O^T += V^T . P^T as m16n8k16 s8 (one byte permute per cache register).
// One dequantisation scale per query head for each contraction, applied to the scores and to the output row.
// Follows the golden of tests/apitest/kernelstest/mix/test_paged_attention_common.py:104-110, 142-227, whose
// tiles are 128 tokens or more where these are 16: the results differ by the quantisation noise of P only.
//
// The reference dequantises K/V to fp16/bf16 through a global-memory scratch before its matmuls
// (DequantKV, src/kernels/mixkernels/pagedattention/op_kernel/paged_attention_decoder_nd_common.cce:8306-8420);
// its golden computes (float(x) + offset) * scale in fp32
// (tests/apitest/kernelstest/mix/test_paged_attention_common.py:89-103).  Results agree within 1e-2.
#include <cuda.h>
#include <mutex>
#include "common.cuh"
#include "kernels.h"
#include "pa_merge.cuh"
#include "tma_encode.h"
#include "pa_exchange.cuh"

namespace atb_b200 {
namespace {

constexpr int kStageTokens = 64;
constexpr int kStages = 6;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileBytes = kStageTokens * 128;      // 64 tokens x 128 int8
constexpr int kStageBytes = 2 * kTileBytes;         // K, V
constexpr int kXbufFloats = 32 * 32;                // one warp's O fragments
constexpr int kFinalStride = 132;                   // padded [head][dim] row (floats)
constexpr int kSmemBytes = kStages * kStageBytes + (kXbufFloats + 8 * kFinalStride + 64) * 4 + 2 * kStages * 8 + 1024;

// Four int8 in a register -> two half2 holding 1152 + x.  (x ^ 0x80) is x + 128 as an unsigned byte; placed under
// the high byte 0x64 it reads as the half 1024 + 128 + x, exactly.  The 1152 is never subtracted from the operands:
//   * in Q.K^T it adds 1152 * sum_d q_d to every score of a head, the same for every token, which the softmax
//     cancels (like the kOffset term);
//   * in P.V it adds 1152 * sum_t p_t to every output dim of a head; the kernel keeps that sum of the ROUNDED
//     probabilities (the values the tensor cores multiply) and subtracts it once per token range.
// Products of two 11-bit significands are exact in the fp32 accumulators, so nothing is lost but ~4 of their 24 bits.
constexpr float kI8Bias = 1152.f;
// lo = (byte0, byte1), hi = (byte2, byte3)
__device__ __forceinline__ void i8x4_to_h2x2(uint32_t w, uint32_t &lo, uint32_t &hi)
{
    const uint32_t x = w ^ 0x80808080u;
    lo = __byte_perm(x, 0x64646464u, 0x4140);
    hi = __byte_perm(x, 0x64646464u, 0x4342);
}
// even = (byte0, byte2), odd = (byte1, byte3)
__device__ __forceinline__ void i8x4_to_h2x2_even_odd(uint32_t w, uint32_t &even, uint32_t &odd)
{
    const uint32_t x = w ^ 0x80808080u;
    even = __byte_perm(x, 0x64646464u, 0x4240);
    odd = __byte_perm(x, 0x64646464u, 0x4341);
}

__device__ __forceinline__ void mma_s8_16832(int32_t (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8_16816(int32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
// rint(fp16(x)) as the golden rounds a probability before it becomes an int8
__device__ __forceinline__ int32_t quant_p(float x) { return __half2int_rn(__float2half_rn(x)); }

// Writes 8 output elements of (sequence, local head h) to the output tensor - or, when the heads are
// sharded over several GPUs, into the gathered [tokens, all heads, 128] buffer of every rank.
template <typename T>
__device__ __forceinline__ void store_out_row(const PaArgs &a, int seq, int h, int d0, const uint4 &pk)
{
    if (a.n_out_peers == 0) {
        *reinterpret_cast<uint4 *>(static_cast<T *>(a.out) + ((int64_t)seq * a.num_heads + h) * 128 + d0) = pk;
    } else {
        const int64_t off = ((int64_t)seq * a.out_total_heads + a.out_head_offset + h) * 128 + d0;
#pragma unroll 1
        for (int r = 0; r < a.n_out_peers; ++r) {
            *reinterpret_cast<uint4 *>(static_cast<T *>(a.out_peers[r]) + off) = pk;
        }
    }
}

// T: query / output type; kQ8: the query is int8 as well (T is the output type only), see the file comment.
template <typename T, bool kQ8>
__global__ void __launch_bounds__(kThreads, 2)
pa_tma_mma_i8_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const PaArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stages = base;
    float *xbuf0 = reinterpret_cast<float *>(base + kStages * kStageBytes);
    float *xbuf1 = xbuf0 + kXbufFloats; // also the final [8][132] tile
    float *sm_m = xbuf1 + 8 * kFinalStride;
    float *sm_l = sm_m + 32;
    uint64_t *full = reinterpret_cast<uint64_t *>(sm_l + 32);
    uint64_t *empty = full + kStages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cols = a.plan.cols;
    const int grp = blockIdx.x / cols;
    // a column is (kv head, chunk of 8 query heads): groups of more than 8 heads per kv head take several
    // columns, whose CTAs read the same K/V tiles at about the same time (once from HBM, again from L2)
    const int col = blockIdx.x - grp * cols;
    const int kvh = col / a.chunks_per_kvh;
    const int head0 = kvh * a.group + (col - kvh * a.chunks_per_kvh) * 8; // first query head of this CTA

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        fence_barrier_init();
    }
    __syncthreads();
    // launched with programmatic stream serialisation: everything above overlapped the tail of the
    // previous kernel in the stream; wait for it (and its memory) before reading any input
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int item_begin = a.plan.group_begin[grp], item_end = a.plan.group_begin[grp + 1];
    uint32_t stage = 0, phase = 0;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer warp
        if (lane == 0) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
        }
        bool alive = true;
        for (int it = item_begin; it < item_end && alive; ++it) {
            const PaItem item = a.plan.items[it];
            const int n_st = (item.tok_end - item.tok_begin + kStageTokens - 1) / kStageTokens;
            const int32_t *bt = a.block_tables + (int64_t)item.seq * a.max_blocks;
            // A 64-token stage is one TMA box per operand half when the cache block holds >= 64 tokens,
            // and 64 / block_size boxes (one per block) otherwise.  The lanes look the block ids of up
            // to 32 boxes up at once; boxes past the end of the range get id -1 (zero-filled tile).
            const int box_tok = min(a.block_size, kStageTokens);
            const int bps = kStageTokens / box_tok;          // boxes per stage: 1, 2 or 4
            const int box_bytes = box_tok * 128;
            const int st_per_batch = 32 / bps;
            for (int st0 = 0; st0 < n_st && alive; st0 += st_per_batch) {
                int blk = -1;
                {
                    const int tok = item.tok_begin + (st0 + lane / bps) * kStageTokens + (lane % bps) * box_tok;
                    if (tok < item.tok_end) {
                        blk = bt[tok / a.block_size];
                        if ((unsigned)blk >= (unsigned)a.num_blocks) {
                            // a caller error: report it, and load a zero tile instead of whatever lies there
                            atomicExch(a.plan.status, kStatusBadBlockId);
                            blk = -1;
                        }
                    }
                }
                const int cnt = min(st_per_batch, n_st - st0);
                for (int j = 0; j < cnt; ++j) {
                    if (lane == 0) {
                        if (!mbar_wait(&empty[stage], phase ^ 1u)) {
                            atomicExch(a.plan.status, kStatusWaitTimeout);
                            alive = false;
                        } else {
                            mbar_expect_tx(&full[stage], kStageBytes);
                        }
                    }
                    alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
                    if (!alive) {
                        break;
                    }
                    for (int bx = 0; bx < bps; ++bx) {
                        const int b = __shfl_sync(0xffffffffu, blk, j * bps + bx);
                        if (lane == 0) {
                            const int tok_in_blk = (item.tok_begin + (st0 + j) * kStageTokens + bx * box_tok) % a.block_size;
                            uint8_t *dst = stages + stage * kStageBytes + bx * box_bytes;
                            // a block id outside the cache makes the tile out of bounds: TMA fills zeros
                            tma_load_4d(dst, &kmap, &full[stage], 0, kvh, tok_in_blk, b);
                            tma_load_4d(dst + kTileBytes, &vmap, &full[stage], 0, kvh, tok_in_blk, b);
                        }
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int g = lane >> 2, c = lane & 3;
    const T *q = static_cast<const T *>(a.q);
    const uint32_t stages_u32 = smem_u32(stages);
    const int group = min(8, kvh * a.group + a.group - head0); // query heads of this CTA

    for (int it = item_begin; it < item_end; ++it) {
        const PaItem item = a.plan.items[it];
        // B fragments of Q^T, pre-multiplied by kDescale.  ldmatrix hands a thread the 4 consecutive
        // int8 dims 4c..4c+3 of each 16-dim chunk, so those dims take the mma's k slots
        // {2c, 2c+1, 2c+8, 2c+9} for both operands.  (kQ8: the int8 query bytes themselves, 4 dims per register.)
        uint32_t qf[8][2];
        float kd0 = 0.f, kd1 = 0.f;   // kQ8: score scale of this thread's two heads (columns 2c, 2c + 1), log2 domain
        float ps0 = 127.f, ps1 = 127.f; // kQ8 offline: their pScale
        if constexpr (kQ8) {
            const bool valid = g < group;
            const int8_t *qp = static_cast<const int8_t *>(a.q) + ((int64_t)item.seq * a.num_heads + head0 + (valid ? g : 0)) * 128;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                qf[2 * kk][0] = valid ? *reinterpret_cast<const uint32_t *>(qp + kk * 32 + 4 * c) : 0u;
                qf[2 * kk][1] = valid ? *reinterpret_cast<const uint32_t *>(qp + kk * 32 + 16 + 4 * c) : 0u;
            }
            const int h0 = head0 + min(2 * c, group - 1), h1 = head0 + min(2 * c + 1, group - 1);
            kd0 = a.k_descale[h0] * a.scale_log2;
            kd1 = a.k_descale[h1] * a.scale_log2;
            if (a.p_scale != nullptr) {
                ps0 = a.p_scale[h0];
                ps1 = a.p_scale[h1];
            }
        } else {
            const bool valid = g < group;
            const T *qp = q + ((int64_t)item.seq * a.num_heads + head0 + (valid ? g : 0)) * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                float f[4] = {0.f, 0.f, 0.f, 0.f};
                if (valid) {
                    load4<T>(qp + ks * 16 + 4 * c, f);
                    if (a.k_descale != nullptr) {
                        const float4 sc = *reinterpret_cast<const float4 *>(a.k_descale + kvh * 128 + ks * 16 + 4 * c);
                        f[0] *= sc.x;
                        f[1] *= sc.y;
                        f[2] *= sc.z;
                        f[3] *= sc.w;
                    }
                }
                qf[ks][0] = Elem<__half>::pack2(f[0], f[1]);
                qf[ks][1] = Elem<__half>::pack2(f[2], f[3]);
            }
        }
        if (!kQ8 && it + 1 < item_end && warp == 0 && c == 0 && g < group) {
            // the next range's query row of this head: on its way into L2 while this range streams
            const char *nq = reinterpret_cast<const char *>(q) + ((int64_t)a.plan.items[it + 1].seq * a.num_heads + head0 + g) * 128 * (int64_t)sizeof(*q);
            for (int b = 0; b < 128 * (int)sizeof(*q); b += 128) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(nq + b));
            }
        }
        float o[8][4];
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
        }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        float lr0 = 0.f, lr1 = 0.f; // sums of the probabilities as rounded for the tensor cores (bias of V)

        const int n_st = (item.tok_end - item.tok_begin + kStageTokens - 1) / kStageTokens;
        for (int st = 0; st < n_st; ++st) {
            const int valid_tokens = item.tok_end - (item.tok_begin + st * kStageTokens + warp * 16);
            if (!mbar_wait(&full[stage], phase)) {
                if (lane == 0) {
                    atomicExch(a.plan.status, kStatusWaitTimeout);
                }
                return;
            }
            if (valid_tokens > 0) {
                const uint32_t kbase = stages_u32 + stage * kStageBytes;
                const uint32_t vbase = kbase + kTileBytes;
                if (!kQ8 && valid_tokens < 16) {
                    // rows past the end of the sequence may hold anything (even NaN bit patterns):
                    // clear this warp's unused V rows so that 0 * V stays 0 (integer products need no such care)
                    uint8_t *vs = stages + stage * kStageBytes + kTileBytes;
                    const int rows = 16 - valid_tokens;
                    for (int i = lane; i < rows * 8; i += 32) { // 8 x 16-byte chunks per 128-byte row
                        const int r = warp * 16 + valid_tokens + (i >> 3);
                        *reinterpret_cast<uint4 *>(vs + r * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
                // ---- S^T = K . Q^T  (16 tokens x 8 heads, k = 128)
                float s[4];
                if constexpr (kQ8) {
                    int32_t si[4] = {0, 0, 0, 0};
                    const int t = warp * 16 + (lane & 15);
                    const uint32_t row_addr = kbase + t * 128;
                    const int sw = t & 7;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        // one ldmatrix.x4 = 16 tokens x 32 int8 dims = the A fragment of one k = 32 step as it is
                        const int ch = kk * 2 + (lane >> 4);
                        uint32_t r[4];
                        ldmatrix_x4(r, row_addr + ((ch ^ sw) << 4));
                        mma_s8_16832(si, r, qf[2 * kk][0], qf[2 * kk][1]);
                    }
                    s[0] = (float)si[0] * kd0;
                    s[1] = (float)si[1] * kd1;
                    s[2] = (float)si[2] * kd0;
                    s[3] = (float)si[3] * kd1;
                } else {
                    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
                    // one ldmatrix.x4 = 16 tokens x 32 int8 dims = two k steps:
                    // r[0] (token g, chunk 2kk), r[1] (token g+8, chunk 2kk), r[2], r[3] the same for chunk 2kk+1
                    const int t = warp * 16 + (lane & 15);
                    const uint32_t row_addr = kbase + t * 128;
                    const int sw = t & 7;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const int ch = kk * 2 + (lane >> 4);
                        uint32_t r[4];
                        ldmatrix_x4(r, row_addr + ((ch ^ sw) << 4));
                        uint32_t af[4];
                        i8x4_to_h2x2(r[0], af[0], af[2]);
                        i8x4_to_h2x2(r[1], af[1], af[3]);
                        mma_16816<__half>(s0, af, qf[2 * kk][0], qf[2 * kk][1]);
                        i8x4_to_h2x2(r[2], af[0], af[2]);
                        i8x4_to_h2x2(r[3], af[1], af[3]);
                        mma_16816<__half>(s1, af, qf[2 * kk + 1][0], qf[2 * kk + 1][1]);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        s[i] = (s0[i] + s1[i]) * a.scale_log2;
                    }
                }
                if (g >= valid_tokens) {
                    s[0] = s[1] = -INFINITY;
                }
                if (g + 8 >= valid_tokens) {
                    s[2] = s[3] = -INFINITY;
                }
                float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
                }
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1); // finite: token 0 of the slice is valid
                const float corr0 = fast_exp2(m0 - mn0), corr1 = fast_exp2(m1 - mn1);
                if constexpr (kQ8) {
                    // weight of this tile against the running maximum, and the probabilities against the tile's own
                    const float w0 = fast_exp2(mx0 - mn0), w1 = fast_exp2(mx1 - mn1);
                    const float e0 = fast_exp2(s[0] - mx0), e1 = fast_exp2(s[1] - mx1);
                    const float e2 = fast_exp2(s[2] - mx0), e3 = fast_exp2(s[3] - mx1);
                    l0 = l0 * corr0 + (e0 + e2) * w0;
                    l1 = l1 * corr1 + (e1 + e3) * w1;
                    m0 = mn0;
                    m1 = mn1;
                    const bool offline = a.p_scale != nullptr;
                    // online: 127 * 2^(s - tile max), weight w on the tile's result; offline: p * pScale, weight 1
                    const float f0 = offline ? w0 * ps0 : 127.f, f1 = offline ? w1 * ps1 : 127.f;
                    const float u0 = offline ? 1.f : w0, u1 = offline ? 1.f : w1;
                    const int32_t q0 = quant_p(e0 * f0), q1 = quant_p(e1 * f1), q2 = quant_p(e2 * f0), q3 = quant_p(e3 * f1);
                    if (__any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f)) {
#pragma unroll
                        for (int mt = 0; mt < 8; ++mt) {
                            o[mt][0] *= corr0;
                            o[mt][1] *= corr1;
                            o[mt][2] *= corr0;
                            o[mt][3] *= corr1;
                        }
                    }
                    // P^T as the B operand: after the transposes a thread holds, for head g, tokens 2c, 2c+1 (and
                    // 8+2c, 9+2c) in 16-bit slots; their low bytes are the operand's k slots 4c..4c+3
                    const uint32_t ta = movmatrix_trans((uint32_t)q0 | ((uint32_t)q1 << 16));
                    const uint32_t tb = movmatrix_trans((uint32_t)q2 | ((uint32_t)q3 << 16));
                    const uint32_t bq = __byte_perm(ta, tb, 0x6420);
                    // ---- O^T += w * (V^T . P^T)  (128 dims x 8 heads, k = 16 tokens; the thread's registers hold
                    // tokens {2c, 2c+1} / {8+2c, 9+2c} x dims {2g, 2g+1}: even bytes are dim 2g = mma row g, odd
                    // bytes dim 2g+1 = row g+8, the same row order as the float path)
                    const int t = warp * 16 + (lane & 15);
                    const uint32_t row_addr = vbase + t * 128;
                    const int sw = t & 7;
#pragma unroll
                    for (int mm = 0; mm < 4; ++mm) {
                        const int ch = mm * 2 + (lane >> 4);
                        uint32_t r[4];
                        ldmatrix_x4_trans(r, row_addr + ((ch ^ sw) << 4));
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            int32_t d[4] = {0, 0, 0, 0};
                            mma_s8_16816(d, __byte_perm(r[2 * hf], r[2 * hf + 1], 0x6420),
                                         __byte_perm(r[2 * hf], r[2 * hf + 1], 0x7531), bq);
                            float *oo = o[2 * mm + hf];
                            oo[0] = fmaf((float)d[0], u0, oo[0]);
                            oo[1] = fmaf((float)d[1], u1, oo[1]);
                            oo[2] = fmaf((float)d[2], u0, oo[2]);
                            oo[3] = fmaf((float)d[3], u1, oo[3]);
                        }
                    }
                } else {
                    const float p0 = fast_exp2(s[0] - mn0), p1 = fast_exp2(s[1] - mn1);
                    const float p2 = fast_exp2(s[2] - mn0), p3 = fast_exp2(s[3] - mn1);
                    l0 = l0 * corr0 + p0 + p2;
                    l1 = l1 * corr1 + p1 + p3;
                    m0 = mn0;
                    m1 = mn1;
                    const uint32_t pk01 = Elem<__half>::pack2(p0, p1), pk23 = Elem<__half>::pack2(p2, p3);
                    {
                        const float2 r01 = Elem<__half>::unpack2(pk01), r23 = Elem<__half>::unpack2(pk23);
                        lr0 = lr0 * corr0 + r01.x + r23.x;
                        lr1 = lr1 * corr1 + r01.y + r23.y;
                    }
                    if (__any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f)) {
    #pragma unroll
                        for (int mt = 0; mt < 8; ++mt) {
                            o[mt][0] *= corr0;
                            o[mt][1] *= corr1;
                            o[mt][2] *= corr0;
                            o[mt][3] *= corr1;
                        }
                    }
                    const uint32_t b0 = movmatrix_trans(pk01);
                    const uint32_t b1 = movmatrix_trans(pk23);
                    // ---- O^T += V^T . P^T  (128 dims x 8 heads, k = 16 tokens)
                    {
                        // one ldmatrix.x4.trans = 16 tokens x 32 int8 dims = two 16-dim row tiles.  A thread
                        // receives (token 2c, dims 2g,2g+1 | token 2c+1, dims 2g,2g+1) per 8-token matrix, so
                        // within a row tile the mma row g holds dim 2g and the row g+8 holds dim 2g+1.
                        const int t = warp * 16 + (lane & 15);
                        const uint32_t row_addr = vbase + t * 128;
                        const int sw = t & 7;
    #pragma unroll
                        for (int mm = 0; mm < 4; ++mm) {
                            const int ch = mm * 2 + (lane >> 4);
                            uint32_t r[4];
                            ldmatrix_x4_trans(r, row_addr + ((ch ^ sw) << 4));
                            uint32_t af[4];
                            i8x4_to_h2x2_even_odd(r[0], af[0], af[1]);
                            i8x4_to_h2x2_even_odd(r[1], af[2], af[3]);
                            mma_16816<__half>(o[2 * mm], af, b0, b1);
                            i8x4_to_h2x2_even_odd(r[2], af[0], af[1]);
                            i8x4_to_h2x2_even_odd(r[3], af[2], af[3]);
                            mma_16816<__half>(o[2 * mm + 1], af, b0, b1);
                        }
                    }
                }
                }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[stage]);
            }
            if (++stage == kStages) {
                stage = 0;
                phase ^= 1u;
            }
        }

        // ---- end of the token range: merge the four warps and write the result
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
            lr0 += __shfl_xor_sync(0xffffffffu, lr0, off);
            lr1 += __shfl_xor_sync(0xffffffffu, lr1, off);
        }
        // take the bias of the V operand out of this warp's accumulators: 1152 x (sum of its rounded probabilities)
#pragma unroll
        for (int mt = 0; mt < (kQ8 ? 0 : 8); ++mt) {
            o[mt][0] = fmaf(-kI8Bias, lr0, o[mt][0]);
            o[mt][1] = fmaf(-kI8Bias, lr1, o[mt][1]);
            o[mt][2] = fmaf(-kI8Bias, lr0, o[mt][2]);
            o[mt][3] = fmaf(-kI8Bias, lr1, o[mt][3]);
        }
        if (g == 0) {
            sm_m[warp * 8 + 2 * c] = m0;
            sm_m[warp * 8 + 2 * c + 1] = m1;
            sm_l[warp * 8 + 2 * c] = l0;
            sm_l[warp * 8 + 2 * c + 1] = l1;
        }
        named_bar_sync(1, kConsumerWarps * 32);
        float f0, f1;
        {
            float M0 = -INFINITY, M1 = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                M0 = fmaxf(M0, sm_m[w * 8 + 2 * c]);
                M1 = fmaxf(M1, sm_m[w * 8 + 2 * c + 1]);
            }
            float L0 = 0.f, L1 = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                L0 += sm_l[w * 8 + 2 * c] * exp2f(sm_m[w * 8 + 2 * c] - M0);
                L1 += sm_l[w * 8 + 2 * c + 1] * exp2f(sm_m[w * 8 + 2 * c + 1] - M1);
            }
            f0 = exp2f(m0 - M0) / L0;
            f1 = exp2f(m1 - M1) / L1;
        }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            o[mt][0] *= f0;
            o[mt][1] *= f1;
            o[mt][2] *= f0;
            o[mt][3] *= f1;
        }
        if (warp >= 2) {
            float *xb = (warp == 2) ? xbuf0 : xbuf1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    xb[(mt * 4 + i) * 32 + lane] = o[mt][i];
                }
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (warp < 2) {
            const float *xb = (warp == 0) ? xbuf0 : xbuf1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    o[mt][i] += xb[(mt * 4 + i) * 32 + lane];
                }
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (warp == 1) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    xbuf0[(mt * 4 + i) * 32 + lane] = o[mt][i];
                }
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (warp == 0) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const float v0 = o[mt][0] + xbuf0[(mt * 4 + 0) * 32 + lane];
                const float v1 = o[mt][1] + xbuf0[(mt * 4 + 1) * 32 + lane];
                const float v2 = o[mt][2] + xbuf0[(mt * 4 + 2) * 32 + lane];
                const float v3 = o[mt][3] + xbuf0[(mt * 4 + 3) * 32 + lane];
                xbuf1[(2 * c) * kFinalStride + mt * 16 + 2 * g] = v0;
                xbuf1[(2 * c + 1) * kFinalStride + mt * 16 + 2 * g] = v1;
                xbuf1[(2 * c) * kFinalStride + mt * 16 + 2 * g + 1] = v2;
                xbuf1[(2 * c + 1) * kFinalStride + mt * 16 + 2 * g + 1] = v3;
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        {
            const int hl = threadIdx.x >> 4;       // head within the group
            const int d0 = (threadIdx.x & 15) * 8; // 8 consecutive dims
            if (hl < group) {
                const float *src = xbuf1 + hl * kFinalStride + d0;
                float4 va = *reinterpret_cast<const float4 *>(src);
                float4 vb = *reinterpret_cast<const float4 *>(src + 4);
                if constexpr (kQ8) {
                    // one P.V scale per query head; online quantisation put 127 into every probability
                    const float sc = a.v_descale[head0 + hl] * (a.p_scale != nullptr ? 1.f : 1.f / 127.f);
                    va.x *= sc; va.y *= sc; va.z *= sc; va.w *= sc;
                    vb.x *= sc; vb.y *= sc; vb.z *= sc; vb.w *= sc;
                }
                if (!kQ8 && a.v_offset != nullptr) {
                    const int4 oa = *reinterpret_cast<const int4 *>(a.v_offset + kvh * 128 + d0);
                    const int4 ob = *reinterpret_cast<const int4 *>(a.v_offset + kvh * 128 + d0 + 4);
                    va.x += (float)oa.x; va.y += (float)oa.y; va.z += (float)oa.z; va.w += (float)oa.w;
                    vb.x += (float)ob.x; vb.y += (float)ob.y; vb.z += (float)ob.z; vb.w += (float)ob.w;
                }
                if (!kQ8 && a.v_descale != nullptr) {
                    const float4 sa = *reinterpret_cast<const float4 *>(a.v_descale + kvh * 128 + d0);
                    const float4 sb = *reinterpret_cast<const float4 *>(a.v_descale + kvh * 128 + d0 + 4);
                    va.x *= sa.x; va.y *= sa.y; va.z *= sa.z; va.w *= sa.w;
                    vb.x *= sb.x; vb.y *= sb.y; vb.z *= sb.z; vb.w *= sb.w;
                }
                const int h = head0 + hl;
                if (item.slot < 0) {
                    uint4 pk;
                    pk.x = Elem<T>::pack2(va.x, va.y);
                    pk.y = Elem<T>::pack2(va.z, va.w);
                    pk.z = Elem<T>::pack2(vb.x, vb.y);
                    pk.w = Elem<T>::pack2(vb.z, vb.w);
                    store_out_row<T>(a, item.seq, h, d0, pk);
                } else {
                    float *dst = a.plan.part_o + ((int64_t)item.slot * a.num_heads + h) * 128 + d0;
                    *reinterpret_cast<float4 *>(dst) = va;
                    *reinterpret_cast<float4 *>(dst + 4) = vb;
                    if (d0 == 0) {
                        float M = -INFINITY, L = 0.f;
#pragma unroll
                        for (int w = 0; w < kConsumerWarps; ++w) {
                            M = fmaxf(M, sm_m[w * 8 + hl]);
                        }
#pragma unroll
                        for (int w = 0; w < kConsumerWarps; ++w) {
                            L += sm_l[w * 8 + hl] * exp2f(sm_m[w * 8 + hl] - M);
                        }
                        a.plan.part_lse[(int64_t)item.slot * a.num_heads + h] = M + log2f(L);
                    }
                }
            }
        }
        if (item.slot >= 0 && a.plan.counters != nullptr) {
            // In-kernel merge: the range that arrives last for this (sequence, kv head) finds every
            // partial already written (fence + counter) and combines them with their LSE weights.
            __threadfence();
            named_bar_sync(1, kConsumerWarps * 32);
            const int n_parts = a.plan.seq_nparts[item.seq];
            if (threadIdx.x == 0) {
                const int old = atomicAdd(&a.plan.counters[item.seq * cols + col], 1);
                sm_l[0] = (old == n_parts - 1) ? 1.f : 0.f;
            }
            named_bar_sync(1, kConsumerWarps * 32);
            const bool last = sm_l[0] != 0.f;
            if (last) {
                __threadfence();
                const int hl = threadIdx.x >> 4;
                const int d0 = (threadIdx.x & 15) * 8;
                if (hl < group) {
                    const int h = head0 + hl;
                    const int pbase = a.plan.seq_part_base[item.seq];
                    const uint4 pk = merge_partials8<T>(a, pbase, h, d0, 128, n_parts);
                    store_out_row<T>(a, item.seq, h, d0, pk);
                }
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
    }
    if (a.n_out_peers > 0) {
        // heads sharded over several GPUs: make this CTA's peer stores visible, then let the last CTA
        // of the grid exchange completion flags with the other ranks
        __threadfence_system();
        named_bar_sync(1, kConsumerWarps * 32);
        if (warp == 0) {
            exchange_tail(a, lane);
        }
    }
}


// 4-D view [num_blocks][block_size][kv_heads][128] of an int8 cache; one box = 64 tokens x 128
// bytes of one kv head (128-byte rows, 128-byte swizzle).
bool encode_cache_map(CUtensorMap *map, const void *base, int kv_heads, int block_size, int num_blocks)
{
    TmaEncodeFn fn = tma_encode_fn();
    if (fn == nullptr) {
        return false;
    }
    cuuint64_t dims[4] = {128, (cuuint64_t)kv_heads, (cuuint64_t)block_size, (cuuint64_t)num_blocks};
    cuuint64_t strides[3] = {128, (cuuint64_t)kv_heads * 128, (cuuint64_t)block_size * kv_heads * 128};
    cuuint32_t box[4] = {128, 1, (cuuint32_t)(block_size < kStageTokens ? block_size : kStageTokens), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <typename T, bool kQ8>
cudaError_t launch_typed(const PaArgs &args, const CUtensorMap &km, const CUtensorMap &vm, cudaStream_t s)
{
    auto kern = pa_tma_mma_i8_kernel<T, kQ8>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) {
            return e;
        }
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (dev >= 0 && dev < 64) {
            configured[dev] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(args.plan.n_cta_groups * args.plan.cols));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, km, vm, args);
}

} // namespace

bool pa_tma_mma_i8_supported(int dk, int dv, int v_row_dim, int block_size, int group, int q_dtype, int kv_dtype)
{
    return dk == 128 && dv == 128 && v_row_dim == 128 && (block_size == 16 || block_size == 32 || block_size == 64 || block_size == 128 || block_size == 256) && group >= 1 &&
           (q_dtype == kFp16 || q_dtype == kBf16) && kv_dtype == kInt8;
}

cudaError_t launch_pa_tma_mma_i8(const PaArgs &args, int q_dtype, int num_blocks, cudaStream_t stream)
{
    CUtensorMap km, vm;
    if (!encode_cache_map(&km, args.k_cache, args.kv_heads, args.block_size, num_blocks) ||
        !encode_cache_map(&vm, args.v_cache, args.kv_heads, args.block_size, num_blocks)) {
        return cudaErrorInvalidValue;
    }
    return q_dtype == kFp16 ? launch_typed<__half, false>(args, km, vm, stream)
                            : launch_typed<__nv_bfloat16, false>(args, km, vm, stream);
}

bool pa_tma_mma_q8_supported(int dk, int dv, int v_row_dim, int block_size, int group, int out_dtype)
{
    return pa_tma_mma_i8_supported(dk, dv, v_row_dim, block_size, group, out_dtype, kInt8);
}

cudaError_t launch_pa_tma_mma_q8(const PaArgs &args, int out_dtype, int num_blocks, cudaStream_t stream)
{
    CUtensorMap km, vm;
    if (args.k_descale == nullptr || args.v_descale == nullptr ||
        !encode_cache_map(&km, args.k_cache, args.kv_heads, args.block_size, num_blocks) ||
        !encode_cache_map(&vm, args.v_cache, args.kv_heads, args.block_size, num_blocks)) {
        return cudaErrorInvalidValue;
    }
    return out_dtype == kFp16 ? launch_typed<__half, true>(args, km, vm, stream)
                              : launch_typed<__nv_bfloat16, true>(args, km, vm, stream);
}

} // namespace atb_b200
