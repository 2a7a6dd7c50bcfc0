// Paged decode attention for head_dim 64, 128 or 256 / block_size 16, 32, 64, 128 or 256 (MHA and GQA, fp16 / bf16
// cache; 8 query heads of one kv head per CTA, larger groups as several CTA columns): the HBM-bound hot kernel.
//
// One CTA per (CTA group, kv head), two CTAs per SM.  A producer warp walks the CTA's token ranges,
// looks the physical block of every 64-token stage up in block_tables and issues TMA tile loads
// (cp.async.bulk.tensor, 128-byte swizzle) of the K and V rows of this kv head into a 3-stage
// shared-memory ring guarded by full/empty mbarriers.  Four consumer warps each own 16 tokens of a
// stage: S^T[tokens x heads] = K . Q^T on the tensor cores (mma.sync m16n8k16, the 8 query heads of
// the group in the N dimension, so nothing is padded at group 8), fp32 online softmax with warp
// shuffles, P^T transposed in registers (movmatrix) into the B operand of O^T[dims x heads] =
// V^T . P^T.  Every warp keeps an independent (max, sum, O) state; the states are merged through
// shared memory once per token range, which then writes either the final output row or a
// normalised fp32 partial plus its log-sum-exp for the combine kernel.
//
// Does the work of UnpadAttentionDecoderAic/Aiv (ProcessQK, SoftmaxStage1/2, ProcessPV) in
// src/kernels/mixkernels/pagedattention/op_kernel/paged_attention_decoder_nd_common.cce:4945-8562
// of the reference; the math follows its CPU golden (fp32 scores and softmax, P rounded to the
// query dtype before P.V, fp32 accumulation).
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
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kHalfBytes = kStageTokens * 128;      // 64 tokens x 64 elements x 2 B: one TMA box

// Sizes that follow from the head dimension kD (64, 128 or 256).  A row is kD / 64 boxes of 64 elements.  Other head
// sizes (multiples of 16 below 256) run the next larger geometry: the part of a box past the end of the cache row is out
// of the tensor's bounds, which TMA fills with zeros without fetching anything, the query's missing dims are set to
// zero, and only the real dims of the output are written (kPad: global rows are a.dk elements, not kD).
template <int kD> struct Geo {
    static_assert(kD == 64 || kD == 128 || kD == 256, "head dimensions of the tiled kernel");
    static constexpr int kHalves = kD / 64;                       // boxes per K (or V) row
    static constexpr int kStageBytes = 2 * kHalves * kHalfBytes;  // K boxes, then V boxes
    static constexpr int kStages = kD == 64 ? 6 : 3;              // 96 KB (two CTAs per SM); 192 KB at kD = 256 (one)
    static constexpr int kSteps = kD / 16;                        // k steps of Q.K^T = row tiles of V^T.P^T
    static constexpr int kXbufFloats = kSteps * 4 * 32;           // one warp's O fragments
    static constexpr int kFinalStride = kD + 4;                   // padded [head][dim] row (floats)
    static constexpr int kSmemBytes =
        kStages * kStageBytes + (kXbufFloats + 8 * kFinalStride + 64) * 4 + 2 * kStages * 8 + 1024;
    static constexpr int kCtasPerSm = kD == 256 ? 1 : 2;
};

// Writes 8 output elements of (sequence, local head h) to the output tensor - or, when the heads are
// sharded over several GPUs, into the gathered [tokens, all heads, 128] buffer of every rank.
template <typename T>
__device__ __forceinline__ void store_out_row(const PaArgs &a, int row_dim, int seq, int h, int d0, const uint4 &pk)
{
    if (a.n_out_peers == 0) {
        *reinterpret_cast<uint4 *>(static_cast<T *>(a.out) + ((int64_t)seq * a.num_heads + h) * row_dim + d0) = pk;
    } else {
        const int64_t off = ((int64_t)seq * a.out_total_heads + a.out_head_offset + h) * row_dim + d0;
#pragma unroll 1
        for (int r = 0; r < a.n_out_peers; ++r) {
            *reinterpret_cast<uint4 *>(static_cast<T *>(a.out_peers[r]) + off) = pk;
        }
    }
}

// kMods: the variant that applies an additive mask and / or per-sequence logN factors to the scores; the plain
// variant carries none of that code.
template <typename T, bool kMods, int kD, bool kPad>
__global__ void __launch_bounds__(kThreads, Geo<kD>::kCtasPerSm)
pa_tma_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const PaArgs a)
{
    constexpr int kHalves = Geo<kD>::kHalves, kStageBytes = Geo<kD>::kStageBytes, kStages = Geo<kD>::kStages;
    constexpr int kSteps = Geo<kD>::kSteps, kXbufFloats = Geo<kD>::kXbufFloats, kFinalStride = Geo<kD>::kFinalStride;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stages = base;
    float *xbuf0 = reinterpret_cast<float *>(base + kStages * kStageBytes);
    float *xbuf1 = xbuf0 + kXbufFloats; // also the final [8][kD + 4] tile
    const int dr = kPad ? a.dk : kD;    // elements per row of the query, the output and the partials
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
    const int chunk0 = (col - kvh * a.chunks_per_kvh) * 8; // first head of this CTA within its kv head's group

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
            const int bt_row = (kMods && a.bt_rows != nullptr) ? a.bt_rows[item.seq] : item.seq;
            const int32_t *bt = a.block_tables + (int64_t)bt_row * a.max_blocks;
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
                            // coordinates (dim, kv head, token, block); heads-major blocks swap the middle two
                            const int c1 = a.kv_bnsd ? tok_in_blk : kvh, c2 = a.kv_bnsd ? kvh : tok_in_blk;
#pragma unroll
                            for (int hf = 0; hf < kHalves; ++hf) {
                                tma_load_4d(dst + hf * kHalfBytes, &kmap, &full[stage], 64 * hf, c1, c2, b);
                            }
#pragma unroll
                            for (int hf = 0; hf < kHalves; ++hf) {
                                tma_load_4d(dst + (kHalves + hf) * kHalfBytes, &vmap, &full[stage], 64 * hf, c1, c2, b);
                            }
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
    const int group = min(8, a.group - chunk0); // query heads (columns) of this CTA
    // Column x of this CTA (0..7) -> head index in the [.., num_heads, 128] tensors.  With q_per_seq query tokens per
    // sequence those tensors hold q_per_seq x real-heads rows per sequence and a column is a (token, head) pair:
    // token x / gr, head kvh * gr + x % gr, gr = real heads per kv head (at most 8 pairs: one chunk).
    const int qps = kMods ? a.q_per_seq : 1;
    const int gr = a.group / qps, heads_real = a.num_heads / qps;
    const int hbase = kvh * gr + chunk0;
    auto head_of = [&](int x) { return qps > 1 ? (x / gr) * heads_real + hbase + x % gr : hbase + x; };

    for (int it = item_begin; it < item_end; ++it) {
        const PaItem item = a.plan.items[it];
        uint32_t qf[kSteps][2];
        {
            const bool valid = g < group;
            const T *qp = q + ((int64_t)item.seq * a.num_heads + head_of(valid ? g : 0)) * dr;
#pragma unroll
            for (int ks = 0; ks < kSteps; ++ks) {
                const bool in = valid && (!kPad || ks * 16 < dr);   // dr is a multiple of 16
                qf[ks][0] = in ? *reinterpret_cast<const uint32_t *>(qp + ks * 16 + 2 * c) : 0u;
                qf[ks][1] = in ? *reinterpret_cast<const uint32_t *>(qp + ks * 16 + 8 + 2 * c) : 0u;
            }
            if (it + 1 < item_end && warp == 0 && c == 0 && valid) {
                // the next range's query row of this head: on its way into L2 while this range streams (the cache
                // stream evicts it otherwise, and the range start would wait for DRAM)
                const char *nq = reinterpret_cast<const char *>(q + ((int64_t)a.plan.items[it + 1].seq * a.num_heads + head_of(g)) * dr);
                for (int b = 0; b < dr * 2; b += 128) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(nq + b));
                }
            }
        }
        float o[kSteps][4];
#pragma unroll
        for (int mt = 0; mt < kSteps; ++mt) {
            o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
        }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        float scale_l2 = a.scale_log2;
        const T *mrow0 = nullptr, *mrow1 = nullptr; // mask rows of this thread's two heads (columns 2c, 2c + 1)
        if (kMods) {
            if (a.logn != nullptr) {
                scale_l2 *= __ldg(a.logn + item.seq);
            }
            if (a.mask != nullptr) {
                const T *mb = static_cast<const T *>(a.mask) +
                              (int64_t)(a.mask_rows != nullptr ? a.mask_rows[item.seq] : item.seq) * a.mask_bs;
                const int x0 = min(2 * c, group - 1), x1 = min(2 * c + 1, group - 1); // padding columns read a real one's row
                mrow0 = mb + (int64_t)(x0 / gr) * a.mask_qs + (int64_t)(hbase + x0 % gr) * a.mask_hs;
                mrow1 = mb + (int64_t)(x1 / gr) * a.mask_qs + (int64_t)(hbase + x1 % gr) * a.mask_hs;
            }
        }
        // causal parallel decoding: the query token of column x sees the sequence's first len - (qps - 1 - x / gr) tokens
        int lim0 = 0x7fffffff, lim1 = 0x7fffffff;
        if (kMods && a.seq_lens != nullptr) {
            const int len = a.seq_lens[item.seq];
            lim0 = len - (qps - 1 - min(2 * c, group - 1) / gr);
            lim1 = len - (qps - 1 - min(2 * c + 1, group - 1) / gr);
        }
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
                const uint32_t vbase = kbase + kHalves * kHalfBytes;
                if (valid_tokens < 16) {
                    // rows past the end of the sequence may hold anything (even NaN bit patterns):
                    // clear this warp's unused V rows so that 0 * V stays 0
                    uint8_t *vs = stages + stage * kStageBytes + kHalves * kHalfBytes;
                    const int rows = 16 - valid_tokens;
                    constexpr int kRowChunks = kD / 8; // 16-byte chunks per row (8 per box)
                    for (int i = lane; i < rows * kRowChunks; i += 32) {
                        const int r = warp * 16 + valid_tokens + i / kRowChunks;
                        const int ch = i % kRowChunks;
                        *reinterpret_cast<uint4 *>(vs + (ch >> 3) * kHalfBytes + r * 128 + ((ch & 7) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
                // ---- S^T = K . Q^T  (16 tokens x 8 heads, k = kD)
                float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const int t = warp * 16 + (lane & 15);
                    const uint32_t row_addr = kbase + t * 128;
                    const int sw = t & 7;
#pragma unroll
                    for (int ks = 0; ks < kSteps; ++ks) {
                        const int ch = ks * 2 + (lane >> 4);
                        uint32_t af[4];
                        ldmatrix_x4(af, row_addr + (ch >> 3) * kHalfBytes + (((ch & 7) ^ sw) << 4));
                        if (ks & 1) {
                            mma_16816<T>(s1, af, qf[ks][0], qf[ks][1]);
                        } else {
                            mma_16816<T>(s0, af, qf[ks][0], qf[ks][1]);
                        }
                    }
                }
                float s[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[i] = (s0[i] + s1[i]) * scale_l2;
                }
                if (kMods && mrow0 != nullptr) {
                    // tokens past the end are not read; a mask of -inf is kept finite so that a fully masked
                    // start of a sequence cannot turn the running maximum into -inf
                    constexpr float kLog2e = 1.4426950408889634f;
                    const int64_t t0 = (int64_t)item.tok_begin + st * kStageTokens + warp * 16 + g;
                    if (g < valid_tokens) {
                        s[0] = fmaxf(s[0] + kLog2e * Elem<T>::to_float(mrow0[t0]), -1e30f);
                        s[1] = fmaxf(s[1] + kLog2e * Elem<T>::to_float(mrow1[t0]), -1e30f);
                    }
                    if (g + 8 < valid_tokens) {
                        s[2] = fmaxf(s[2] + kLog2e * Elem<T>::to_float(mrow0[t0 + 8]), -1e30f);
                        s[3] = fmaxf(s[3] + kLog2e * Elem<T>::to_float(mrow1[t0 + 8]), -1e30f);
                    }
                }
                if (kMods && a.seq_lens != nullptr) {
                    // finite, like a mask of -inf: a range may hold nothing but tokens this column does not see
                    const int t0 = item.tok_begin + st * kStageTokens + warp * 16 + g;
                    s[0] = t0 < lim0 ? s[0] : -1e30f;
                    s[1] = t0 < lim1 ? s[1] : -1e30f;
                    s[2] = t0 + 8 < lim0 ? s[2] : -1e30f;
                    s[3] = t0 + 8 < lim1 ? s[3] : -1e30f;
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
                const float p0 = fast_exp2(s[0] - mn0), p1 = fast_exp2(s[1] - mn1);
                const float p2 = fast_exp2(s[2] - mn0), p3 = fast_exp2(s[3] - mn1);
                l0 = l0 * corr0 + p0 + p2;
                l1 = l1 * corr1 + p1 + p3;
                m0 = mn0;
                m1 = mn1;
                if (__any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f)) {
#pragma unroll
                    for (int mt = 0; mt < kSteps; ++mt) {
                        o[mt][0] *= corr0;
                        o[mt][1] *= corr1;
                        o[mt][2] *= corr0;
                        o[mt][3] *= corr1;
                    }
                }
                const uint32_t b0 = movmatrix_trans(Elem<T>::pack2(p0, p1));
                const uint32_t b1 = movmatrix_trans(Elem<T>::pack2(p2, p3));
                // ---- O^T += V^T . P^T  (kD dims x 8 heads, k = 16 tokens)
                {
                    const int j = lane >> 3;
                    const int tok = warp * 16 + (j >> 1) * 8 + (lane & 7);
                    const uint32_t row_addr = vbase + tok * 128;
                    const int sw = tok & 7;
#pragma unroll
                    for (int mt = 0; mt < kSteps; ++mt) {
                        const int ch = mt * 2 + (j & 1);
                        uint32_t af[4];
                        ldmatrix_x4_trans(af, row_addr + (ch >> 3) * kHalfBytes + (((ch & 7) ^ sw) << 4));
                        mma_16816<T>(o[mt], af, b0, b1);
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
        for (int mt = 0; mt < kSteps; ++mt) {
            o[mt][0] *= f0;
            o[mt][1] *= f1;
            o[mt][2] *= f0;
            o[mt][3] *= f1;
        }
        if (warp >= 2) {
            float *xb = (warp == 2) ? xbuf0 : xbuf1;
#pragma unroll
            for (int mt = 0; mt < kSteps; ++mt) {
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
            for (int mt = 0; mt < kSteps; ++mt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    o[mt][i] += xb[(mt * 4 + i) * 32 + lane];
                }
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (warp == 1) {
#pragma unroll
            for (int mt = 0; mt < kSteps; ++mt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    xbuf0[(mt * 4 + i) * 32 + lane] = o[mt][i];
                }
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (warp == 0) {
#pragma unroll
            for (int mt = 0; mt < kSteps; ++mt) {
                const float v0 = o[mt][0] + xbuf0[(mt * 4 + 0) * 32 + lane];
                const float v1 = o[mt][1] + xbuf0[(mt * 4 + 1) * 32 + lane];
                const float v2 = o[mt][2] + xbuf0[(mt * 4 + 2) * 32 + lane];
                const float v3 = o[mt][3] + xbuf0[(mt * 4 + 3) * 32 + lane];
                xbuf1[(2 * c) * kFinalStride + mt * 16 + g] = v0;
                xbuf1[(2 * c + 1) * kFinalStride + mt * 16 + g] = v1;
                xbuf1[(2 * c) * kFinalStride + mt * 16 + g + 8] = v2;
                xbuf1[(2 * c + 1) * kFinalStride + mt * 16 + g + 8] = v3;
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        // kD / 8 chunks of 8 dims per head row, 8 head rows: a thread per chunk (two at kD = 256, half the threads at 64)
        for (int idx = threadIdx.x; idx < dr; idx += kConsumerWarps * 32) {
            const int hl = idx / (dr / 8);       // head within the group
            const int d0 = (idx % (dr / 8)) * 8; // 8 consecutive dims
            if (hl < group) {
                const float *src = xbuf1 + hl * kFinalStride + d0;
                const float4 va = *reinterpret_cast<const float4 *>(src);
                const float4 vb = *reinterpret_cast<const float4 *>(src + 4);
                const int h = head_of(hl);
                if (item.slot < 0) {
                    uint4 pk;
                    pk.x = Elem<T>::pack2(va.x, va.y);
                    pk.y = Elem<T>::pack2(va.z, va.w);
                    pk.z = Elem<T>::pack2(vb.x, vb.y);
                    pk.w = Elem<T>::pack2(vb.z, vb.w);
                    store_out_row<T>(a, dr, item.seq, h, d0, pk);
                } else {
                    float *dst = a.plan.part_o + ((int64_t)item.slot * a.num_heads + h) * dr + d0;
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
                for (int idx = threadIdx.x; idx < dr; idx += kConsumerWarps * 32) {
                    const int hl = idx / (dr / 8);
                    const int d0 = (idx % (dr / 8)) * 8;
                    if (hl >= group) {
                        continue;
                    }
                    const int h = head_of(hl);
                    const int pbase = a.plan.seq_part_base[item.seq];
                    const uint4 pk = merge_partials8<T>(a, pbase, h, d0, dr, n_parts);
                    store_out_row<T>(a, dr, item.seq, h, d0, pk);
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


// 4-D view [num_blocks][block_size][kv_heads][dim] of a cache; one box = 64 tokens x 64 elements
// of one kv head (128-byte rows, 128-byte swizzle).
bool encode_cache_map(CUtensorMap *map, const void *base, int elem_dtype, int kv_heads, int block_size, int num_blocks,
                      bool bnsd, int dim)
{
    TmaEncodeFn fn = tma_encode_fn();
    if (fn == nullptr) {
        return false;
    }
    const cuuint64_t es = 2;
    const cuuint64_t D = (cuuint64_t)dim;
    cuuint64_t dims[4] = {D, (cuuint64_t)kv_heads, (cuuint64_t)block_size, (cuuint64_t)num_blocks};
    cuuint64_t strides[3] = {D * es, (cuuint64_t)kv_heads * D * es, (cuuint64_t)block_size * kv_heads * D * es};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)(block_size < kStageTokens ? block_size : kStageTokens), 1};
    if (bnsd) {
        // [num_blocks][kv_heads][block_size][128]: coordinates (dim, token, kv head, block), strides still ascending;
        // a box is the same 64-element x box_tokens tile in shared memory
        dims[1] = (cuuint64_t)block_size;
        dims[2] = (cuuint64_t)kv_heads;
        strides[0] = D * es;
        strides[1] = (cuuint64_t)block_size * D * es;
        box[1] = box[2];
        box[2] = 1;
    }
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, elem_dtype == kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <typename T, int kD, bool kPad>
cudaError_t launch_typed(const PaArgs &args, const CUtensorMap &km, const CUtensorMap &vm, cudaStream_t s)
{
    constexpr int kSmemBytes = Geo<kD>::kSmemBytes;
    const bool mods = args.mask != nullptr || args.logn != nullptr || args.bt_rows != nullptr || args.q_per_seq > 1 ||
                      args.seq_lens != nullptr;
    auto kern = mods ? pa_tma_mma_kernel<T, true, kD, kPad> : pa_tma_mma_kernel<T, false, kD, kPad>;
    static bool configured_plain[64] = {}, configured_mods[64] = {};
    bool *configured = mods ? configured_mods : configured_plain;
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

// The geometry (64, 128 or 256) a head size runs on; 0 if the tiled kernel has none for it.
static int tiled_geometry(int dk)
{
    if (dk < 16 || dk > 256 || dk % 16 != 0) {
        return 0;
    }
    return dk <= 64 ? 64 : dk <= 128 ? 128 : 256;
}

bool pa_tma_mma_supported(int dk, int dv, int v_row_dim, int block_size, int group, int q_dtype, int kv_dtype)
{
    return tiled_geometry(dk) != 0 && dv == dk && v_row_dim == dk && (block_size == 16 || block_size == 32 || block_size == 64 || block_size == 128 || block_size == 256) && group >= 1 &&
           (q_dtype == kFp16 || q_dtype == kBf16) && kv_dtype == q_dtype;
}

cudaError_t launch_pa_tma_mma(const PaArgs &args, int q_dtype, int kv_dtype, int num_blocks, cudaStream_t stream)
{
    (void)kv_dtype;
    CUtensorMap km, vm;
    if (!encode_cache_map(&km, args.k_cache, q_dtype, args.kv_heads, args.block_size, num_blocks, args.kv_bnsd != 0, args.dk) ||
        !encode_cache_map(&vm, args.v_cache, q_dtype, args.kv_heads, args.block_size, num_blocks, args.kv_bnsd != 0, args.dk)) {
        return cudaErrorInvalidValue;
    }
    const bool f16 = q_dtype == kFp16;
    const int geo = tiled_geometry(args.dk);
    const bool pad = geo != args.dk;
#define ATB_B200_LAUNCH_TILED(D)                                                                                              \
    (pad ? (f16 ? launch_typed<__half, D, true>(args, km, vm, stream) : launch_typed<__nv_bfloat16, D, true>(args, km, vm, stream)) \
         : (f16 ? launch_typed<__half, D, false>(args, km, vm, stream) : launch_typed<__nv_bfloat16, D, false>(args, km, vm, stream)))
    switch (geo) {
        case 64:
            return ATB_B200_LAUNCH_TILED(64);
        case 128:
            return ATB_B200_LAUNCH_TILED(128);
        case 256:
            return ATB_B200_LAUNCH_TILED(256);
        default:
            return cudaErrorInvalidValue;
    }
#undef ATB_B200_LAUNCH_TILED
}

} // namespace atb_b200
