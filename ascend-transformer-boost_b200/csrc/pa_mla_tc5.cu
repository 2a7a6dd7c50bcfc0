// Paged decode attention over the MLA combined latent cache (one kv head, K row = 576 = 512 latent
// + 64 rope, V = the first 512 columns of the same row) on the 5th-generation tensor cores.
//
// One CTA per (CTA group, 64 query heads), one CTA per SM.  Warp roles:
//   warp 4  - TMA producer: 64-token K tiles (9 boxes of 64 tokens x 64 elements, 128-byte swizzle)
//             into a 3-stage shared-memory ring (3 x 72 KB: the whole shared memory);
//   warp 5  - one elected thread issues tcgen05.mma (M = 64 heads):
//               S[64 x 64 tokens]  = Q . K^T          36 MMAs, A = Q read from TENSOR MEMORY (the 64 x 576
//                                                      query block is stored there once per token range,
//                                                      which frees 72 KB of shared memory for the third
//                                                      stage), B = K tile, accumulator in TMEM
//               O[64 x 512]       += P . V            8 MMAs of N = 256; V is the same shared-memory
//                                                      tile read MN-major, so the cache row crosses
//                                                      the memory system once
//             and owns the TMEM allocation;
//   warps 0-3 - softmax: tcgen05.ld one S row per thread (no cross-thread reductions), running max /
//             sum in the exp2 domain, P -> bf16/fp16 into shared memory for the P.V MMA; O stays in
//             TMEM for the whole token range and is rescaled only when a row's maximum grows by more
//             than 2^8 (the final division by the row sum absorbs the stale scale).
// TMEM: an M = 64 operand occupies 16 of the 32 lanes of each warp's quadrant, so O (512 columns)
// lives in the lower half-quadrants; the upper ones hold the two S buffers (columns 0..127) and Q
// (bf16/fp16 pairs, columns 128..415).
//
// Replaces MLAttentionDecoderAic / paged_multi_latent_attention_mask of the reference
// (src/kernels/mixkernels/pagedattention/op_kernel/paged_MLAttention_combine_cache_mask_mix.cce:24-150,
//  paged_attention_decoder_nd_common.cce:2861-3897), which never splits the KV range
// (tiling/paged_attention_tiling_dependency.cpp:230); here token ranges are split and merged like the
// other kernels.  Math as the golden: fp32 scores and softmax, P rounded to the query dtype.
#include <cuda.h>
#include <mutex>
#include <type_traits>
#include "common.cuh"
#include "kernels.h"
#include "tc5.cuh"
#include "tma_encode.h"

namespace atb_b200 {
namespace {

constexpr int kHeadsPerCta = 64;
constexpr int kTok = 64;                 // tokens per stage
constexpr int kDk = 576, kDv = 512;
constexpr int kAtoms = kDk / 64;         // 9 boxes of 64 elements per row
constexpr int kAtomBytes = 64 * 128;     // 64 rows x 128 B
constexpr int kTileBytes = kAtoms * kAtomBytes; // 73728
constexpr int kStages = 3;
constexpr int kPBytes = 64 * 128;        // P: 64 heads x 64 tokens x 2 B
constexpr int kNumBars = 16;
constexpr int kSmemBytes = kStages * kTileBytes + kPBytes + kNumBars * 8 + 64 + 1024;
constexpr uint32_t kQCol = 128;          // first TMEM column of Q (upper half-quadrants)
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

enum Bar { kQFull = 0, kQEmpty, kKvFull0, kKvFull1, kKvFull2, kKvEmpty0, kKvEmpty1, kKvEmpty2, kSFull0, kSFull1, kSEmpty0, kSEmpty1, kPFull, kPvDone };

// One 256-bit read-only load from a 32-byte aligned global address.
__device__ __forceinline__ void ld_global_nc_v8(const void *p, uint32_t *w)
{
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
}

// One 256-bit store (eight 32-bit words) to a 32-byte aligned global address.
__device__ __forceinline__ void st_global_v8(void *p, const uint32_t *w)
{
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}

// kMask: the variant for parallel decoding with a mask or the causal rule: it adds the query token's mask row to the
// scores (MASK_TYPE_SPEC) and / or hides the tokens behind the query token (q_per_seq > 1: the rows of a CTA are (token,
// head) pairs, row r belongs to query token (head0 + r) / real heads).  The plain variant carries none of that code.
// Both follow bt_rows when the plan gives every query token its block-table row.
// kTrace: the build that carries the event probe (atb_b200_pa_plan_set_trace); the product build has none of it in
// the issuing thread's loop.
template <typename T, bool kMask, bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
pa_mla_tc5_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap rmap, const PaArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *kv_smem = base;
    uint8_t *p_smem = kv_smem + kStages * kTileBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(p_smem + kPBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cols = a.plan.cols;
    const int grp = blockIdx.x / cols;
    const int col = blockIdx.x - grp * cols;
    const int head0 = col * kHeadsPerCta;
    const int nh = min(kHeadsPerCta, a.num_heads - head0);
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

    if (threadIdx.x == 0) {
        mbar_init(&bars[kQFull], 4);   // the four softmax warps have stored Q into TMEM
        mbar_init(&bars[kQEmpty], 1);  // the last Q.K^T of the range has completed
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars[kKvFull0 + s], 1);
            mbar_init(&bars[kKvEmpty0 + s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[kSFull0 + s], 1);
            mbar_init(&bars[kSEmpty0 + s], 4);
        }
        mbar_init(&bars[kPFull], 4);
        mbar_init(&bars[kPvDone], 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // launched with programmatic stream serialisation: the set-up above overlapped the tail of the
    // previous kernel in the stream; wait for it (and its memory) before reading any input
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // probe with CTA selector 255: every CTA records when it started and ended (global nanosecond timer) instead of
    // one CTA recording its events
    const bool time_all = kTrace && a.trace != nullptr && (a.trace_cap >> 24) == 255u && 2 * gridDim.x + 2 <= (a.trace_cap & 0xffffffu);
    unsigned long long t_start = 0;
    if (time_all && threadIdx.x == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    }
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base;                 // lanes 0-15 of every quadrant, columns 0..511
    const uint32_t tmem_s = tmem_base + (16u << 16);   // lanes 16-31 of every quadrant, columns 0..127

    const int item_begin = a.plan.group_begin[grp], item_end = a.plan.group_begin[grp + 1];

    auto wait = [&](int bar, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < (1u << 21); ++i) {
            if (mbar_try_wait(&bars[bar], parity)) {
                return true;
            }
            if (i > 32) {
                __nanosleep(64);
                if (*abort_flag) {
                    return false;
                }
            }
        }
        *abort_flag = 1;
        atomicExch(a.plan.status, kStatusWaitTimeout);
        return false;
    };

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&rmap);
        }
        // The rope part of a row (elements 512..575) is either the tail of the combined cache row or, with the
        // split cache, a row of a tensor of its own; rmap describes whichever holds it.
        const int rope_x0 = a.k_rope != nullptr ? 0 : kDv;
        uint32_t g = 0; // global stage counter
        bool alive = true;
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_st = (item.tok_end - item.tok_begin + kTok - 1) / kTok;
            const int32_t *bt = a.block_tables + (int64_t)(a.bt_rows != nullptr ? a.bt_rows[item.seq] : item.seq) * a.max_blocks;
            for (int st0 = 0; st0 < n_st && alive; st0 += 32) {
                int blk = 0;
                if (st0 + lane < n_st) {
                    blk = bt[(item.tok_begin + (st0 + lane) * kTok) / a.block_size];
                    if ((unsigned)blk >= (unsigned)a.num_blocks) {
                        // a caller error: report it, and load a zero tile instead of whatever lies there
                        atomicExch(a.plan.status, kStatusBadBlockId);
                        blk = -1;
                    }
                }
                const int cnt = min(32, n_st - st0);
                for (int j = 0; j < cnt && alive; ++j, ++g) {
                    const int b = __shfl_sync(0xffffffffu, blk, j);
                    if (lane == 0) {
                        const int s = g % kStages;
                        if (!wait(kKvEmpty0 + s, ((g / kStages) & 1) ^ 1u)) {
                            alive = false;
                        } else {
                            const int tok_in_blk = (item.tok_begin + (st0 + j) * kTok) % a.block_size;
                            uint8_t *dst = kv_smem + s * kTileBytes;
                            if constexpr (kTrace) {
                                probe(a, 1, g);
                            }
                            mbar_expect_tx(&bars[kKvFull0 + s], kTileBytes);
                            for (int at = 0; at < kAtoms - 1; ++at) {
                                tma_load_4d(dst + at * kAtomBytes, &kmap, &bars[kKvFull0 + s], at * 64, 0, tok_in_blk, b);
                            }
                            tma_load_4d(dst + (kAtoms - 1) * kAtomBytes, &rmap, &bars[kKvFull0 + s], rope_x0, 0, tok_in_blk, b);
                        }
                    }
                    alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(kFmt, 0, kTok, kHeadsPerCta);
            constexpr uint32_t idesc_pv = instr_desc(kFmt, 1, 256, kHeadsPerCta);
            const uint32_t kv_addr = smem_u32(kv_smem), p_addr = smem_u32(p_smem);
            const uint32_t tmem_q = tmem_base + (16u << 16) + kQCol;
            uint32_t g = 0;
            bool alive = true;
            // Issue order is decided by what is ready, P.V first: a P.V releases its K tile to the
            // producer, so it must never queue behind a Q.K^T that is still waiting for its tile.
            auto ready = [&](int bar, uint32_t parity) { return mbar_test_wait(&bars[bar], parity); };
            for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
                const PaItem item = a.plan.items[it];
                const int n_st = (item.tok_end - item.tok_begin + kTok - 1) / kTok;
                if (!wait(kQFull, i & 1)) {
                    break;
                }
                int next_qk = 0, next_pv = 0;
                uint32_t idle = 0;
                while (next_pv < n_st) {
                    const uint32_t gp = g + next_pv, gq = g + next_qk;
                    if (next_pv < next_qk && ready(kPFull, gp & 1)) {
                        if constexpr (kTrace) {
                            probe(a, 3, gp);
                        }
                        tc_fence_after();
                        const int s = gp % kStages;
                        const uint32_t vb = kv_addr + s * kTileBytes;
                        const uint64_t da0 = smem_desc(p_addr, 16, 1024);
                        // V^T operand: 64-element boxes along N are 8192 B apart, 8-token groups 1024 B apart
                        const uint64_t dv0 = smem_desc(vb, kAtomBytes, 1024);
                        const bool acc = next_pv != 0;
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
                                tc_mma(tmem_o + half * 256, da0 + ((ks * 32) >> 4),
                                       dv0 + (((4 * half) * kAtomBytes + ks * 2048) >> 4), idesc_pv, acc || ks != 0);
                            }
                        }
                        tc_commit(&bars[kKvEmpty0 + s]);
                        tc_commit(&bars[kPvDone]);
                        ++next_pv;
                        idle = 0;
                    } else if (next_qk < n_st && next_qk < next_pv + 2 &&
                               ready(kKvFull0 + (gq % kStages), (gq / kStages) & 1) &&
                               ready(kSEmpty0 + (gq & 1), ((gq >> 1) & 1) ^ 1u)) {
                        if constexpr (kTrace) {
                            probe(a, 2, gq);
                        }
                        tc_fence_after();
                        const int s = gq & 1;                                   // S buffer
                        const uint32_t kb = kv_addr + (gq % kStages) * kTileBytes; // K tile slot
                        // The issuing thread is the bottleneck of a tile: all 36 MMAs unrolled, one descriptor built and
                        // the others derived by adding to its address field (16-byte units; shared memory addresses stay
                        // below the field's 256 KB range, so nothing carries into the next field).
                        const uint64_t db0 = smem_desc(kb, 16, 1024);
                        const uint32_t ds = tmem_s + s * 64;
#pragma unroll
                        for (int at = 0; at < kAtoms; ++at) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
                                // 16 elements of Q = 8 TMEM columns (two 16-bit values per column)
                                tc_mma_ts(ds, tmem_q + at * 32 + ks * 8, db0 + ((at * kAtomBytes + ks * 32) >> 4), idesc_qk,
                                          (at | ks) != 0);
                            }
                        }
                        tc_commit(&bars[kSFull0 + s]);
                        if (next_qk + 1 == n_st) {
                            tc_commit(&bars[kQEmpty]); // Q of this range is no longer needed
                        }
                        ++next_qk;
                        idle = 0;
                    } else {
                        ++idle;
                        if (idle > (1u << 22) || *abort_flag) {
                            *abort_flag = 1;
                            atomicExch(a.plan.status, kStatusWaitTimeout);
                            alive = false;
                            break;
                        }
                    }
                }
                g += n_st;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / epilogue warps 0..3
        const bool s_lane = lane >= 16;                 // upper half-quadrant: the S rows
        const int row = warp * 16 + (lane & 15);        // head within the CTA
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        uint32_t g = 0;
        bool alive = true;
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_st = (item.tok_end - item.tok_begin + kTok - 1) / kTok;
            // ---- Q block of this range -> TMEM (upper half-quadrants, two 16-bit values per column).
            // The previous range's Q.K^T MMAs must be done with the old Q; O is dead here (its first
            // P.V overwrites it), so the lower lanes of these columns may be written with anything.
            if (!wait(kQEmpty, (i & 1) ^ 1u)) {
                alive = false;
                break;
            }
            tc_fence_after();
            {
                const bool has_row = s_lane && row < nh;
                const int64_t qidx = (int64_t)item.seq * a.num_heads + head0 + (has_row ? row : 0);
                // combined rows: 576 elements; split cache: 512 latent elements here, 64 rope elements in q_rope
                const bool split = a.q_rope != nullptr;
                // rows are 1152 / 1024 / 128 bytes: with 32-byte aligned tensors every atom of every row is aligned too
                const bool q_wide = ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.q_rope)) & 31u) == 0;
                const uint4 *qrow = reinterpret_cast<const uint4 *>(static_cast<const T *>(a.q) + qidx * (split ? kDv : kDk));
                const uint4 *qrope = split ? reinterpret_cast<const uint4 *>(static_cast<const T *>(a.q_rope) + qidx * (kDk - kDv))
                                           : qrow + kDv / 8;
                // 64 elements = 128 B = 32 columns per atom; three atoms' loads are in flight together (this runs
                // between two token ranges with the pipeline drained: every exposed load latency is kernel time)
                static_assert(kAtoms % 3 == 0, "the Q block is stored three atoms at a time");
#pragma unroll 1
                for (int c0 = 0; c0 < kAtoms; c0 += 3) {
                    uint32_t t[3][32];
#pragma unroll
                    for (int u = 0; u < 3; ++u) {
                        const uint4 *src = c0 + u < kAtoms - 1 ? qrow + (c0 + u) * 8 : qrope;
                        if (q_wide) {
                            // 32-byte loads: four per 128-byte atom of the row
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (has_row) {
                                    ld_global_nc_v8(src + 2 * j, &t[u][8 * j]);
                                } else {
#pragma unroll
                                    for (int k = 0; k < 8; ++k) {
                                        t[u][8 * j + k] = 0u;
                                    }
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const uint4 v = has_row ? __ldg(src + j) : make_uint4(0, 0, 0, 0);
                                t[u][4 * j] = v.x;
                                t[u][4 * j + 1] = v.y;
                                t[u][4 * j + 2] = v.z;
                                t[u][4 * j + 3] = v.w;
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 3; ++u) {
                        tmem_st32(tmem_base + lane_base + kQCol + (c0 + u) * 32, t[u]);
                    }
                }
                if (has_row && it + 1 < item_end) {
                    // the next range's Q rows: into L2 now, so that its range start finds them there
                    const int64_t nidx = (int64_t)a.plan.items[it + 1].seq * a.num_heads + head0 + row;
                    const char *nrow = reinterpret_cast<const char *>(static_cast<const T *>(a.q) + nidx * (split ? kDv : kDk));
                    const int lines = split ? kDv / 64 : kDk / 64;
                    for (int c = 0; c < lines; ++c) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(nrow + c * 128));
                    }
                    if (split) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const T *>(a.q_rope) + nidx * (kDk - kDv)));
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kQFull]);
                }
            }
            float m_used = -INFINITY, l = 0.f;
            const T *mrow = nullptr; // this row's mask row, at the first token of the range
            int row_limit = 0x7fffffff; // first token of the range this row does not see (causal rule)
            if (kMask) {
                const int jq = a.q_per_seq > 1 ? min(head0 + row, a.num_heads - 1) / (a.num_heads / a.q_per_seq) : 0;
                if (a.mask != nullptr) {
                    mrow = static_cast<const T *>(a.mask) +
                           (int64_t)(a.mask_rows != nullptr ? a.mask_rows[item.seq] : item.seq) * a.mask_bs +
                           (int64_t)jq * a.mask_qs + item.tok_begin;
                }
                if (a.seq_lens != nullptr) {
                    row_limit = a.seq_lens[item.seq] - (a.q_per_seq - 1 - jq) - item.tok_begin;
                }
            }
            for (int st = 0; st < n_st && alive; ++st, ++g) {
                const int sb = g & 1;
                const int valid = min(kTok, item.tok_end - (item.tok_begin + st * kTok));
                if (!wait(kSFull0 + sb, (g >> 1) & 1)) {
                    alive = false;
                    break;
                }
                if (threadIdx.x == 16) {
                    if constexpr (kTrace) {
                        probe(a, 4, g);
                    }
                }
                tc_fence_after();
                uint32_t r0[32], r1[32];
                tmem_ld32(tmem_base + lane_base + sb * 64, r0);
                tmem_ld32(tmem_base + lane_base + sb * 64 + 32, r1);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kSEmpty0 + sb]);
                }
                // scores in the exp2 domain, tokens past the end of the range masked
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float v0 = __uint_as_float(r0[j]) * a.scale_log2;
                    float v1 = __uint_as_float(r1[j]) * a.scale_log2;
                    if (kMask) {
                        // the same mask value for every head (row); -inf is kept finite so that a fully masked
                        // start of a range cannot make the running maximum -inf.  Tokens past the end are not read.
                        constexpr float kLog2e = 1.4426950408889634f;
                        if (mrow != nullptr) {
                            if (j < valid) {
                                v0 = fmaxf(v0 + kLog2e * Elem<T>::to_float(mrow[st * kTok + j]), -1e30f);
                            }
                            if (j + 32 < valid) {
                                v1 = fmaxf(v1 + kLog2e * Elem<T>::to_float(mrow[st * kTok + j + 32]), -1e30f);
                            }
                        }
                        // hidden by the causal rule: finite like a mask of -inf (a range may hold nothing else)
                        v0 = (st * kTok + j < row_limit) ? v0 : -1e30f;
                        v1 = (st * kTok + j + 32 < row_limit) ? v1 : -1e30f;
                    }
                    v0 = (j < valid) ? v0 : -INFINITY;
                    v1 = (j + 32 < valid) ? v1 : -INFINITY;
                    r0[j] = __float_as_uint(v0);
                    r1[j] = __float_as_uint(v1);
                    mx = fmaxf(mx, fmaxf(v0, v1));
                }
                // lazy rescale: keep the old reference maximum unless it is exceeded by more than 2^8
                float factor = 1.f;
                if (s_lane && mx > m_used + 8.f) {
                    factor = exp2f(m_used - mx); // 0 on the first tile
                    m_used = mx;
                    l *= factor;
                }
                const bool rescale_row = s_lane && factor != 1.f && st > 0;
                const bool rescale_any = __any_sync(0xffffffffu, rescale_row);
                float lsum = 0.f;
                uint32_t pk[32];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float p0 = fast_exp2(__uint_as_float(r0[2 * j]) - m_used);
                    const float p1 = fast_exp2(__uint_as_float(r0[2 * j + 1]) - m_used);
                    const float p2 = fast_exp2(__uint_as_float(r1[2 * j]) - m_used);
                    const float p3 = fast_exp2(__uint_as_float(r1[2 * j + 1]) - m_used);
                    lsum += (p0 + p1) + (p2 + p3);
                    pk[j] = Elem<T>::pack2(p0, p1);
                    pk[16 + j] = Elem<T>::pack2(p2, p3);
                }
                l += lsum;
                if (threadIdx.x == 16) {
                    if constexpr (kTrace) {
                        probe(a, 5, g);
                    }
                }
                // P(g) overwrites P(g-1) and a rescale touches O: both need P.V(g-1) to have finished
                if (g > 0 && !wait(kPvDone, (g - 1) & 1)) {
                    alive = false;
                    break;
                }
                if (threadIdx.x == 16) {
                    if constexpr (kTrace) {
                        probe(a, 6, g);
                    }
                }
                if (rescale_any) {
                    // O rows live in lanes 0..15; the multiplier comes from the row's S lane.  The S lanes
                    // of columns 0..127 are rewritten with their own values, so the next S tile must be
                    // complete before they are touched.
                    if (st + 1 < n_st && !wait(kSFull0 + (sb ^ 1), ((g + 1) >> 1) & 1)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const float f_o = __shfl_sync(0xffffffffu, factor, (lane & 15) + 16);
                    const float mul = s_lane ? 1.f : f_o;
#pragma unroll 1
                    for (int c0 = 0; c0 < kDv; c0 += 32) {
                        uint32_t t[32];
                        tmem_ld32(tmem_base + lane_base + c0, t);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            t[j] = __float_as_uint(__uint_as_float(t[j]) * mul);
                        }
                        tmem_st32(tmem_base + lane_base + c0, t);
                    }
                    tmem_wait_st();
                }
                if (s_lane) {
                    // row of P: 64 tokens = 8 chunks of 16 B, 128-byte swizzle
                    uint8_t *prow = p_smem + row * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        *reinterpret_cast<uint4 *>(prow + ((ch ^ (row & 7)) << 4)) =
                            make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                    }
                }
                if (valid < kTok) {
                    // rows of V past the end of the range may hold anything: clear them (0 * NaN != 0)
                    uint8_t *vt = kv_smem + (g % kStages) * kTileBytes;
                    const int rows = kTok - valid;
                    for (int idx = threadIdx.x; idx < rows * 8 * 8; idx += 128) {
                        const int at = idx / (rows * 8), rem = idx - at * (rows * 8);
                        const int rr = valid + (rem >> 3), ch = rem & 7;
                        *reinterpret_cast<uint4 *>(vt + at * kAtomBytes + rr * 128 + (ch << 4)) = make_uint4(0, 0, 0, 0);
                    }
                }
                fence_proxy_async();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kPFull]);
                }
                if (threadIdx.x == 16) {
                    if constexpr (kTrace) {
                        probe(a, 7, g);
                    }
                }
            }
            if (!alive) {
                break;
            }
            // ---- end of the token range: O / l -> output row or split-KV partial
            if (!wait(kPvDone, (g - 1) & 1)) {
                alive = false;
                break;
            }
            tc_fence_after();
            const float l_row = __shfl_sync(0xffffffffu, l, (lane & 15) + 16);
            const float m_row = __shfl_sync(0xffffffffu, m_used, (lane & 15) + 16);
            const float inv = 1.f / l_row;
            const int h = head0 + row;
            const bool writer = !s_lane && row < nh;
            T *out_row = static_cast<T *>(a.out) + ((int64_t)item.seq * a.num_heads + h) * kDv;
            const bool out_wide = (reinterpret_cast<uintptr_t>(a.out) & 31u) == 0; // rows are 1 KB: all are aligned then
            float *part_row = a.plan.part_o + ((int64_t)(item.slot < 0 ? 0 : item.slot) * a.num_heads + h) * kDv;
#pragma unroll 1
            for (int c0 = 0; c0 < kDv; c0 += 32) {
                uint32_t t[32];
                tmem_ld32(tmem_base + lane_base + c0, t);
                tmem_wait_ld();
                if (writer) {
                    // 32-byte stores: a lane writes whole sectors of its row (the rows of a warp are 1 or 2 KB apart,
                    // so no two lanes share a line)
                    if (item.slot < 0) {
                        uint32_t w[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            w[j] = Elem<T>::pack2(__uint_as_float(t[2 * j]) * inv, __uint_as_float(t[2 * j + 1]) * inv);
                        }
                        if (out_wide) {
                            st_global_v8(out_row + c0, w);
                            st_global_v8(out_row + c0 + 16, w + 8);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                *reinterpret_cast<uint4 *>(out_row + c0 + 8 * j) =
                                    make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            t[j] = __float_as_uint(__uint_as_float(t[j]) * inv);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            st_global_v8(part_row + c0 + 8 * j, t + 8 * j); // the workspace is 256-byte aligned
                        }
                    }
                }
            }
            if (writer && item.slot >= 0) {
                a.plan.part_lse[(int64_t)item.slot * a.num_heads + h] = m_row + log2f(l_row);
            } else if (writer && a.lse_out != nullptr) {
                // whole sequence in this range: its log-sum-exp, natural log (m_row is in the log2 domain)
                static_cast<T *>(a.lse_out)[(int64_t)item.seq * a.num_heads + h] =
                    Elem<T>::from_float((m_row + log2f(l_row)) * 0.6931471805599453f);
            }
            // the next range's first P.V overwrites O: all reads of O must be done first.  It cannot start
            // before the next P tile is signalled by these same warps, which orders it after this point.
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (time_all && threadIdx.x == 0) {
        unsigned long long t_end;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
        a.trace[1 + 2 * blockIdx.x] = t_start;
        a.trace[2 + 2 * blockIdx.x] = t_end;
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}


template <typename T>
cudaError_t launch_typed(const PaArgs &args, const CUtensorMap &km, const CUtensorMap &rm, cudaStream_t s)
{
    const bool masked = args.mask != nullptr || args.seq_lens != nullptr;
    const bool traced = args.trace != nullptr;
    auto kern = traced ? (masked ? pa_mla_tc5_kernel<T, true, true> : pa_mla_tc5_kernel<T, false, true>)
                       : (masked ? pa_mla_tc5_kernel<T, true, false> : pa_mla_tc5_kernel<T, false, false>);
    static bool configured_all[4][64] = {};
    bool *configured = configured_all[(traced ? 2 : 0) + (masked ? 1 : 0)];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) {
            return e;
        }
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
    return cudaLaunchKernelEx(&cfg, kern, km, rm, args);
}

} // namespace

bool pa_mla_tc5_supported(int dk, int dv, int v_row_dim, int rope_dim, int block_size, int kv_heads, int q_dtype,
                          int kv_dtype)
{
    // combined cache: rows of 576; split cache: latent rows of 512 plus rope rows of 64 in a tensor of their own
    const bool rows_ok = (rope_dim == 0 && v_row_dim == kDk) || (rope_dim == kDk - kDv && v_row_dim == kDv);
    return dk == kDk && dv == kDv && rows_ok && kv_heads == 1 && block_size >= kTok && block_size % kTok == 0 &&
           block_size <= 256 && (q_dtype == kFp16 || q_dtype == kBf16) && kv_dtype == q_dtype;
}

cudaError_t launch_pa_mla_tc5(const PaArgs &args, int q_dtype, int num_blocks, cudaStream_t stream)
{
    TmaEncodeFn fn = tma_encode_fn();
    if (fn == nullptr) {
        return cudaErrorInvalidValue;
    }
    const CUtensorMapDataType dt = q_dtype == kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    // cache [num_blocks][block_size][1][row]; box = 64 elements x 64 tokens of one block
    auto encode = [&](CUtensorMap *map, const void *base, int row) {
        cuuint64_t dims[4] = {(cuuint64_t)row, 1, (cuuint64_t)args.block_size, (cuuint64_t)num_blocks};
        cuuint64_t strides[3] = {(cuuint64_t)row * 2, (cuuint64_t)row * 2, (cuuint64_t)args.block_size * row * 2};
        cuuint32_t box[4] = {64, 1, kTok, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        return fn(map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const bool split = args.k_rope != nullptr;
    CUtensorMap km, rm;
    if (!encode(&km, args.k_cache, split ? kDv : kDk) ||
        !encode(&rm, split ? args.k_rope : args.k_cache, split ? kDk - kDv : kDk)) {
        return cudaErrorInvalidValue;
    }
    return q_dtype == kFp16 ? launch_typed<__half>(args, km, rm, stream) : launch_typed<__nv_bfloat16>(args, km, rm, stream);
}

} // namespace atb_b200
