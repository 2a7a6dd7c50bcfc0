// Paged decode attention over the MLA latent cache (one kv head, K row = 512 latent + 64 rope dims, V = the latent
// part), bf16, as a pair of CTAs (a thread-block cluster of two) per (token range, 64 query heads).
//
// Both contractions run TRANSPOSED, with the 128 tokens of a tile in the M dimension of tcgen05.mma, so that every
// instruction is a full-rate M = 128 MMA:
//     S^T[128 tokens x 64 heads] = K[tokens x dims] . Q^T          A = K tile (shared memory), B = Q (shared memory)
//     O^T[dims x 64 heads]      += V^T[dims x tokens] . P^T         A = V^T = the same K tile read MN-major, B = P^T
// A 128-token tile of the cache is 144 KB and would fit shared memory once, next to Q, with nothing left to load
// the next tile into.  So the two CTAs of the pair split the 576 DIMS: rank 0 owns dims 0..255 (4 atoms of 64), rank 1
// dims 256..575 (5 atoms, the rope part last).  Each loads only its atoms of every tile (64 / 80 KB: two stages fit),
// computes the partial S^T over its dims and the O^T rows of its own dims (rank 0: V dims 0..255, rank 1: 256..511).
// Once per tile rank 1 sends its partial S^T to rank 0 through distributed shared memory; rank 0 adds the two,
// applies the softmax and writes P^T (bf16) into both CTAs' shared memory.
//
// The softmax of the transposed scores is element-wise: a thread owns one token (one TMEM lane) and all 64 heads.
// Instead of the running row maximum it subtracts a per-head reference, the score of the range's first token, and
// clamps the exponent at +100: bf16 has the exponent range of fp32, so P keeps its relative precision wherever the
// reference lies, the first token contributes exactly 1 to the row sum (never 0), and a score more than 2^100 times
// above the reference - which no softmax input reaches - would only be weighted as 2^100.  Row sums are kept per thread
// and reduced across the 128 tokens once per range.
//
// Warp roles in each CTA: warps 0-3 softmax (rank 0) or partial-S^T forwarding (rank 1), and the read-out of O^T;
// warp 4 TMA producer; warp 5 MMA issuer and owner of the tensor-memory allocation.  Every wait is bounded; a wait
// that runs out sets the status word and an abort flag that drains every loop of the CTA; its peer then runs out of
// its own waits.  Both CTAs always reach the final cluster barrier.
//
// Replaces MLAttentionDecoderAic / paged_multi_latent_attention_mask of the reference
// (src/kernels/mixkernels/pagedattention/op_kernel/paged_MLAttention_combine_cache_mask_mix.cce:24-150,
//  paged_attention_decoder_nd_common.cce:2861-3897).  Math as the golden: fp32 scores and softmax, P rounded to bf16.
#include <cuda.h>
#include "common.cuh"
#include "kernels.h"
#include "tc5.cuh"
#include "tma_encode.h"

namespace atb_b200 {
namespace {

constexpr int kHeads = 64;                     // query heads per cluster
constexpr int kTile = 128;                     // tokens per tile = M of both contractions
constexpr int kBox = 64;                       // tokens per TMA box (token ranges start at multiples of it)
constexpr int kDk = 576, kDv = 512;
constexpr int kAtomBytes = kTile * 128;        // 128 tokens x 64 dims: 16 KB
constexpr int kQAtomBytes = kHeads * 128;      // 64 heads x 64 dims: 8 KB
constexpr int kMaxAtoms = 5;
constexpr int kStages = 2;
constexpr int kPBytes = kTile * 128;           // P^T: 128 tokens x 64 heads, bf16
constexpr int kRecvStride = kHeads + 4;        // floats per token row of the receive buffer: 272 B, so that the 16-byte
                                               // accesses of a quarter warp (8 rows) fall into 8 different bank groups
constexpr int kRecvBytes = kTile * kRecvStride * 4; // rank 0: the peer's partial S^T, [token][head] fp32
constexpr int kBigBytes = kMaxAtoms * kQAtomBytes + kStages * kMaxAtoms * kAtomBytes + kPBytes; // 216 KB (rank 1)
static_assert(4 * kQAtomBytes + kStages * 4 * kAtomBytes + kPBytes + kRecvBytes <= kBigBytes, "rank 0 fits the same area");
constexpr int kSmallBytes = 4096;              // barriers, tmem slot, flags, reference scores, row-sum scratch
constexpr int kSmemBytes = kBigBytes + kSmallBytes + 1024;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 256;            // S^T buffers at columns 0 and 64, O^T blocks at 128 and 192
constexpr float kMaxExponent = 100.f;

enum Bar {
    kQFull = 0, kQEmpty, kStFull0, kStFull1, kStEmpty0, kStEmpty1, kSFull0, kSFull1, kSEmpty0, kSEmpty1,
    kPFull, kPvDone, kPHalf0, kPHalf1, kPHalfPeer0, kPHalfPeer1, kRecvFull0, kRecvFull1, kRecvFull2, kRecvFull3,
    kRecvEmpty0, kRecvEmpty1, kRecvEmpty2, kRecvEmpty3, kMref, kWsum, kLinv, kOFree, kNumBars
};

struct Small {
    uint64_t bars[32];
    uint32_t tmem_slot;
    int abort_flag;
    int v_clean;               // rank 1: warps that have cleared the stale V rows, 4 per tile, counted over the kernel
    alignas(16) float mref[2][kHeads]; // (read 16 bytes at a time) reference score per head, log2 domain (double-buffered over ranges)
    float wsum[2][4][kHeads];  // per-warp row sums of a range (double-buffered over ranges)
    float linv[2][kHeads];     // 1 / row sum (both ranks), double-buffered over ranges
    float lfull[2][kHeads];    // row sum (rank 0), for the log-sum-exp
};
static_assert(sizeof(Small) <= kSmallBytes, "small shared-memory area");

// kTrace: the build with the timing probe (atb_b200_pa_plan_set_trace with CTA selector 255): every CTA stores the
// global timer at its start and end in trace[1 + 2b], trace[2 + 2b], and 16 cycle counters of its issuing thread and of
// thread 0 from trace[2 + 2 * grid + 16b] on.  The product build carries none of it.
template <bool kTrace>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
pa_mla_split_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap rmap,
                    const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qrmap, const PaArgs a)
{
    using T = __nv_bfloat16;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Small *sm = reinterpret_cast<Small *>(base + kBigBytes);
    uint64_t *bars = sm->bars;
    volatile int *abort_flag = &sm->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t peer = rank ^ 1u;
    const int n_atoms = rank == 0 ? 4 : 5;                 // atoms of 64 dims this CTA owns
    const int atom0 = rank == 0 ? 0 : 4;                   // first global atom (of 9)
    uint8_t *q_smem = base;
    uint8_t *st_smem = base + n_atoms * kQAtomBytes;
    uint8_t *p_smem = st_smem + kStages * n_atoms * kAtomBytes;
    float *recv = reinterpret_cast<float *>(p_smem + kPBytes);  // rank 0 only

    const int cols = a.plan.cols;
    const int pair = blockIdx.x >> 1;
    const int grp = pair / cols;
    const int col = pair - grp * cols;
    const int head0 = col * kHeads;
    const int nh = min(kHeads, a.num_heads - head0);

    if (threadIdx.x == 0) {
        mbar_init(&bars[kQFull], 1);
        mbar_init(&bars[kQEmpty], 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[kStFull0 + s], 1);
            mbar_init(&bars[kStEmpty0 + s], 1);
            mbar_init(&bars[kSFull0 + s], 1);
            mbar_init(&bars[kSEmpty0 + s], 4);
        }
        // P^T of a tile is written by rank 0's four warps (into both CTAs).  Rank 1's own warps report their cleared V rows
        // on a plain counter (v_clean): they run up to two tiles ahead of the P.V that needs them, which the parity of an
        // mbarrier cannot express
        mbar_init(&bars[kPFull], 4);
        sm->v_clean = 0;
        mbar_init(&bars[kPvDone], 1);
        for (int k = 0; k < 2; ++k) {
            mbar_init(&bars[kPHalf0 + k], 1);     // P.V has consumed tokens 64k..64k+63 of P^T (this CTA)
            mbar_init(&bars[kPHalfPeer0 + k], 1); // the same on the peer, relayed
        }
        for (int w = 0; w < 4; ++w) {
            mbar_init(&bars[kRecvFull0 + w], 1);  // rank 0: warp w of rank 1 has sent its 32 token rows
            mbar_init(&bars[kRecvEmpty0 + w], 1); // rank 1: warp w of rank 0 has read them
        }
        mbar_init(&bars[kMref], 1);
        mbar_init(&bars[kWsum], 4);
        mbar_init(&bars[kLinv], 2);
        mbar_init(&bars[kOFree], 4);
        sm->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(&sm->tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // the peer's barriers must exist before anything arrives on them
    cluster_sync_all();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint32_t tmem_base = sm->tmem_slot;
    const bool tracing = kTrace && a.trace != nullptr && (a.trace_cap >> 24) == 255u &&
                         2 + 18 * gridDim.x <= (a.trace_cap & 0xffffffu);
    unsigned long long t_start = 0;
    if (tracing && threadIdx.x == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    }
    unsigned long long *acct = tracing ? a.trace + 2 + 2 * gridDim.x + 16 * blockIdx.x : nullptr;
    long long acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    auto tick = [&]() -> long long { return kTrace ? clock64() : 0; };
    const int item_begin = a.plan.group_begin[grp], item_end = a.plan.group_begin[grp + 1];

    // bounded waits; `cluster` = the barrier is arrived on by the peer CTA
    auto wait = [&](int bar, uint32_t parity, bool cluster) -> bool {
        for (uint32_t i = 0; i < (1u << 21); ++i) {
            const bool ok = cluster ? mbar_try_wait_cluster(&bars[bar], parity) : mbar_try_wait(&bars[bar], parity);
            if (ok) {
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
    auto peer_bar = [&](int bar) { return map_to_cta(smem_u32(&bars[bar]), peer); };

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&rmap);
            tma_prefetch_desc(&qmap);
            tma_prefetch_desc(&qrmap);
        }
        const bool split_cache = a.k_rope != nullptr;
        uint32_t g = 0;
        bool alive = true;
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
            const int32_t *bt = a.block_tables + (int64_t)(a.bt_rows != nullptr ? a.bt_rows[item.seq] : item.seq) * a.max_blocks;
            if (lane == 0) {
                // the query block of this range: this CTA's atoms of the 64 head rows
                if (!wait(kQEmpty, (i & 1) ^ 1u, false)) {
                    alive = false;
                } else {
                    mbar_expect_tx(&bars[kQFull], n_atoms * kQAtomBytes);
                    for (int at = 0; at < n_atoms; ++at) {
                        const int ga = atom0 + at;
                        if (ga < 8) {
                            tma_load_3d(q_smem + at * kQAtomBytes, &qmap, &bars[kQFull], ga * 64, head0, item.seq);
                        } else {
                            tma_load_3d(q_smem + at * kQAtomBytes, &qrmap, &bars[kQFull], split_cache ? 0 : kDv, head0, item.seq);
                        }
                    }
                }
            }
            alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
            for (int t = 0; t < n_tiles && alive; ++t, ++g) {
                if (lane == 0) {
                    const int s = g & 1;
                    if (!wait(kStEmpty0 + s, ((g >> 1) & 1) ^ 1u, false)) {
                        alive = false;
                    } else {
                        const int tok0 = item.tok_begin + t * kTile;
                        const int n_box = (item.tok_end - tok0 > kBox) ? 2 : 1;
                        uint8_t *dst = st_smem + s * n_atoms * kAtomBytes;
                        mbar_expect_tx(&bars[kStFull0 + s], n_box * n_atoms * kBox * 128);
                        for (int bx = 0; bx < n_box; ++bx) {
                            const int tok = tok0 + bx * kBox;
                            int blk = bt[tok / a.block_size];
                            if ((unsigned)blk >= (unsigned)a.num_blocks) {
                                // a caller error: report it, and load a zero tile instead of whatever lies there
                                atomicExch(a.plan.status, kStatusBadBlockId);
                                blk = -1;
                            }
                            const int tok_in_blk = tok % a.block_size;
                            for (int at = 0; at < n_atoms; ++at) {
                                const int ga = atom0 + at;
                                uint8_t *d = dst + at * kAtomBytes + bx * kBox * 128;
                                if (ga < 8) {
                                    tma_load_4d(d, &kmap, &bars[kStFull0 + s], ga * 64, 0, tok_in_blk, blk);
                                } else {
                                    tma_load_4d(d, &rmap, &bars[kStFull0 + s], split_cache ? 0 : kDv, 0, tok_in_blk, blk);
                                }
                            }
                        }
                    }
                }
                alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc_ab(1, 0, 0, kHeads, kTile); // A = K tile, B = Q, both K-major
            constexpr uint32_t idesc_pv = instr_desc_ab(1, 1, 1, kHeads, kTile); // A = V^T, B = P^T, both MN-major
            const uint32_t q_addr = smem_u32(q_smem), st_addr = smem_u32(st_smem), p_addr = smem_u32(p_smem);
            uint32_t g = 0;
            bool alive = true;
            auto ready = [&](int bar, uint32_t parity) { return mbar_test_wait(&bars[bar], parity); };
            for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
                const PaItem item = a.plan.items[it];
                const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
                if (!wait(kQFull, i & 1, false)) {
                    break;
                }
                int next_qk = 0, next_pv = 0;
                bool o_free = false;
                uint32_t idle = 0;
                while (next_pv < n_tiles) {
                    const uint32_t gp = g + next_pv, gq = g + next_qk;
                    if (next_pv < next_qk && mbar_test_wait_cluster(&bars[kPFull], gp & 1) &&
                        (rank == 0 || *reinterpret_cast<volatile int *>(&sm->v_clean) >= 4 * (int)(gp + 1)) &&
                        (o_free || next_pv > 0 || ready(kOFree, (i & 1) ^ 1u))) {
                        // the first P.V of a range overwrites O^T: the previous range's read-out must be over
                        o_free = true;
                        const long long t0 = tick();
                        tc_fence_after();
                        fence_proxy_async_all(); // P^T was written by ordinary stores (on rank 1: by the peer CTA's)
                        const uint32_t vb = st_addr + (gp & 1) * n_atoms * kAtomBytes;
                        const uint64_t dp0 = smem_desc(p_addr, kAtomBytes, 1024);
                        // tokens 0..63 first, then 64..127: each half of P^T is handed back to the softmax warps as soon as
                        // its MMAs have completed
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
#pragma unroll
                            for (int mb = 0; mb < 2; ++mb) {
                                // V^T rows of 128 dims = two atoms kAtomBytes apart; 8-token groups 1024 B apart
                                const uint64_t dv0 = smem_desc(vb + 2 * mb * kAtomBytes, kAtomBytes, 1024);
#pragma unroll
                                for (int ks = 4 * half; ks < 4 * half + 4; ++ks) {
                                    tc_mma(tmem_base + 128 + mb * 64, dv0 + ((ks * 2048) >> 4), dp0 + ((ks * 2048) >> 4), idesc_pv,
                                           next_pv != 0 || ks != 0);
                                }
                            }
                            tc_commit(&bars[kPHalf0 + half]);
                        }
                        tc_commit(&bars[kStEmpty0 + (gp & 1)]);
                        tc_commit(&bars[kPvDone]);
                        ++next_pv;
                        idle = 0;
                        acc[1] += tick() - t0;
                    } else if (next_qk < n_tiles && next_qk < next_pv + 2 &&
                               ready(kStFull0 + (gq & 1), (gq >> 1) & 1) && ready(kSEmpty0 + (gq & 1), ((gq >> 1) & 1) ^ 1u)) {
                        const long long t0 = tick();
                        tc_fence_after();
                        const uint32_t kb = st_addr + (gq & 1) * n_atoms * kAtomBytes;
                        const uint32_t ds = tmem_base + (gq & 1) * 64;
                        for (int at = 0; at < n_atoms; ++at) {
                            const uint64_t da0 = smem_desc(kb + at * kAtomBytes, 16, 1024);
                            const uint64_t db0 = smem_desc(q_addr + at * kQAtomBytes, 16, 1024);
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
                                tc_mma(ds, da0 + ((ks * 32) >> 4), db0 + ((ks * 32) >> 4), idesc_qk, (at | ks) != 0);
                            }
                        }
                        tc_commit(&bars[kSFull0 + (gq & 1)]);
                        if (next_qk + 1 == n_tiles) {
                            tc_commit(&bars[kQEmpty]); // the query block of this range is no longer needed
                        }
                        ++next_qk;
                        idle = 0;
                        acc[0] += tick() - t0;
                    } else {
                        if (kTrace) {
                            // why nothing could be issued: 3 look-ahead exhausted (P^T missing), 4 K tile missing, 5 S^T buffer busy
                            if (!(next_qk < n_tiles && next_qk < next_pv + 2)) {
                                acc[3]++;
                            } else if (!ready(kStFull0 + (gq & 1), (gq >> 1) & 1)) {
                                acc[4]++;
                            } else {
                                acc[5]++;
                            }
                        }
                        ++idle;
                        if (idle > (1u << 22) || *abort_flag) {
                            *abort_flag = 1;
                            atomicExch(a.plan.status, kStatusWaitTimeout);
                            alive = false;
                            break;
                        }
                    }
                }
                g += n_tiles;
            }
            if (tracing) {
                for (int k = 0; k < 8; ++k) {
                    acct[k] = (unsigned long long)acc[k];
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ warps 0..3: one token (TMEM lane) per thread
        const int tok_l = warp * 32 + lane;                            // row of the tile
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        uint32_t g = 0;
        bool alive = true;
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
            float lsum[kHeads];
            if (rank == 0) {
#pragma unroll
                for (int h = 0; h < kHeads; ++h) {
                    lsum[h] = 0.f;
                }
            }
            for (int t = 0; t < n_tiles && alive; ++t, ++g) {
                const int sb = g & 1;
                const int valid = min(kTile, item.tok_end - (item.tok_begin + t * kTile));
                long long t0 = tick();
                if (!wait(kSFull0 + sb, (g >> 1) & 1, false)) {
                    alive = false;
                    break;
                }
                acc[0] += tick() - t0;
                t0 = tick();
                tc_fence_after();
                uint32_t sv[kHeads];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + lane_base + sb * 64 + c * 16, r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        sv[c * 16 + j] = r[j];
                    }
                }
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kSEmpty0 + sb]);
                }
                // rows of V past the end of the range may hold anything: clear them (0 * NaN != 0); the K rows only
                // feed the scores of those tokens, which get probability 0 below
                if (valid < kTile) {
                    uint8_t *stg = st_smem + sb * n_atoms * kAtomBytes;
                    if (tok_l >= valid) {
                        for (int at = 0; at < 4; ++at) {
#pragma unroll
                            for (int ch = 0; ch < 8; ++ch) {
                                *reinterpret_cast<uint4 *>(stg + at * kAtomBytes + tok_l * 128 + (ch << 4)) = make_uint4(0, 0, 0, 0);
                            }
                        }
                    }
                    fence_proxy_async();
                }
                const int half = warp >> 1;                       // which 64 tokens of the tile this warp owns
                if (rank == 1) {
                    // ---- forward the partial scores to rank 0: recv[token][head], the thread's own row, 16 bytes per store
                    acc[2] += tick() - t0;
                    t0 = tick();
                    if (!wait(kRecvEmpty0 + warp, (g & 1) ^ 1u, true)) {
                        alive = false;
                        break;
                    }
                    acc[1] += tick() - t0;
                    t0 = tick();
                    // rank 0 keeps 4 atoms, so its receive buffer lies at another offset than this CTA's layout suggests
                    const uint32_t dst = map_to_cta(smem_u32(base + 4 * kQAtomBytes + kStages * 4 * kAtomBytes + kPBytes), 0) +
                                         tok_l * (kRecvStride * 4);
#pragma unroll
                    for (int c = 0; c < kHeads / 4; ++c) {
                        st_cluster_v4(dst + c * 16, sv[4 * c], sv[4 * c + 1], sv[4 * c + 2], sv[4 * c + 3]);
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive_cluster(peer_bar(kRecvFull0 + warp));
                        __threadfence_block();
                        atomicAdd(&sm->v_clean, 1);          // this warp's V rows of tile g are clean
                    }
                    acc[4] += tick() - t0;
                    t0 = tick();
                    // relay "P.V of the previous tile has consumed this half of P^T here" so that rank 0 may overwrite it
                    if ((warp & 1) == 0 && g > 0) {
                        if (!wait(kPHalf0 + half, (g - 1) & 1, false)) {
                            alive = false;
                            break;
                        }
                        if (lane == 0) {
                            mbar_arrive_cluster(peer_bar(kPHalfPeer0 + half));
                        }
                    }
                    acc[3] += tick() - t0;
                    continue;
                }
                // ---- rank 0: add the peer's partial, scale, reference, exponentials
                acc[2] += tick() - t0;
                t0 = tick();
                if (!wait(kRecvFull0 + warp, g & 1, true)) {
                    alive = false;
                    break;
                }
                acc[1] += tick() - t0;
                t0 = tick();
                {
                    const float4 *row = reinterpret_cast<const float4 *>(recv + tok_l * kRecvStride);
#pragma unroll
                    for (int c = 0; c < kHeads / 4; ++c) {
                        const float4 r = row[c];
                        sv[4 * c] = __float_as_uint(__uint_as_float(sv[4 * c]) + r.x);
                        sv[4 * c + 1] = __float_as_uint(__uint_as_float(sv[4 * c + 1]) + r.y);
                        sv[4 * c + 2] = __float_as_uint(__uint_as_float(sv[4 * c + 2]) + r.z);
                        sv[4 * c + 3] = __float_as_uint(__uint_as_float(sv[4 * c + 3]) + r.w);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(peer_bar(kRecvEmpty0 + warp));
                }
                float *mref = sm->mref[i & 1];
                if (t == 0) {
                    if (threadIdx.x == 0) {
#pragma unroll
                        for (int h = 0; h < kHeads; ++h) {
                            mref[h] = __uint_as_float(sv[h]) * a.scale_log2;
                        }
                        mbar_arrive(&bars[kMref]);
                    }
                    if (!wait(kMref, i & 1, false)) {
                        alive = false;
                        break;
                    }
                }
                const bool live = tok_l < valid;
                uint32_t pk[kHeads / 2];
#pragma unroll
                for (int c = 0; c < kHeads / 4; ++c) {
                    const float4 m = reinterpret_cast<const float4 *>(mref)[c];
                    const float p0 = live ? fast_exp2(fminf(fmaf(__uint_as_float(sv[4 * c]), a.scale_log2, -m.x), kMaxExponent)) : 0.f;
                    const float p1 = live ? fast_exp2(fminf(fmaf(__uint_as_float(sv[4 * c + 1]), a.scale_log2, -m.y), kMaxExponent)) : 0.f;
                    const float p2 = live ? fast_exp2(fminf(fmaf(__uint_as_float(sv[4 * c + 2]), a.scale_log2, -m.z), kMaxExponent)) : 0.f;
                    const float p3 = live ? fast_exp2(fminf(fmaf(__uint_as_float(sv[4 * c + 3]), a.scale_log2, -m.w), kMaxExponent)) : 0.f;
                    lsum[4 * c] += p0;
                    lsum[4 * c + 1] += p1;
                    lsum[4 * c + 2] += p2;
                    lsum[4 * c + 3] += p3;
                    pk[2 * c] = Elem<T>::pack2(p0, p1);
                    pk[2 * c + 1] = Elem<T>::pack2(p2, p3);
                }
                // this half of P^T(g) overwrites that of P^T(g-1): both CTAs' P.V(g-1) must have consumed it
                acc[2] += tick() - t0;
                t0 = tick();
                if (g > 0 && (!wait(kPHalf0 + half, (g - 1) & 1, false) || !wait(kPHalfPeer0 + half, (g - 1) & 1, true))) {
                    alive = false;
                    break;
                }
                acc[3] += tick() - t0;
                t0 = tick();
                {
                    // row of P^T: 64 heads = 8 chunks of 16 B, 128-byte swizzle; the same row into the peer's buffer
                    uint8_t *prow = p_smem + tok_l * 128;
                    // rank 1 keeps 5 atoms, so its P^T buffer lies at another offset than this CTA's
                    const uint32_t peer_p = map_to_cta(smem_u32(base + 5 * kQAtomBytes + kStages * 5 * kAtomBytes), 1) + tok_l * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        const int pos = (ch ^ (tok_l & 7)) << 4;
                        *reinterpret_cast<uint4 *>(prow + pos) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                        st_cluster_v4(peer_p + pos, pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                    }
                }
                fence_proxy_async_all();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kPFull]);
                    mbar_arrive_cluster(peer_bar(kPFull));
                }
                acc[4] += tick() - t0;
                acc[6]++;
            }
            if (!alive) {
                break;
            }
            // ---- end of the token range: row sums -> 1 / l for both CTAs, then O^T / l -> output row or partial
            const long long t_ep = tick();
            float *linv = sm->linv[i & 1];
            if (rank == 0) {
#pragma unroll
                for (int h = 0; h < kHeads; ++h) {
                    float s = lsum[h];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) {
                        s += __shfl_xor_sync(0xffffffffu, s, off);
                    }
                    if (lane == 0) {
                        sm->wsum[i & 1][warp][h] = s;
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kWsum]);
                }
                if (!wait(kWsum, i & 1, false)) {
                    alive = false;
                    break;
                }
                if (warp < 2) {
                    const int h = warp * 32 + lane;
                    const float l = sm->wsum[i & 1][0][h] + sm->wsum[i & 1][1][h] + sm->wsum[i & 1][2][h] + sm->wsum[i & 1][3][h];
                    const float inv = 1.f / l;
                    linv[h] = inv;
                    sm->lfull[i & 1][h] = l;
                    st_cluster_f32(map_to_cta(smem_u32(&linv[h]), 1), inv);
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&bars[kLinv]);
                        mbar_arrive_cluster(peer_bar(kLinv));
                    }
                }
            }
            if (!wait(kLinv, i & 1, true)) {
                alive = false;
                break;
            }
            // every P.V of the range has completed here
            if (!wait(kPvDone, (g - 1) & 1, false)) {
                alive = false;
                break;
            }
            tc_fence_after();
            if (rank == 0 && warp < 2) {
                const int h = warp * 32 + lane;
                if (h < nh) {
                    const float lse2 = sm->mref[i & 1][h] + log2f(sm->lfull[i & 1][h]);
                    if (item.slot >= 0) {
                        a.plan.part_lse[(int64_t)item.slot * a.num_heads + head0 + h] = lse2;
                    } else if (a.lse_out != nullptr) {
                        // whole sequence in this range: its log-sum-exp, natural log
                        static_cast<T *>(a.lse_out)[(int64_t)item.seq * a.num_heads + head0 + h] =
                            Elem<T>::from_float(lse2 * 0.6931471805599453f);
                    }
                }
            }
#pragma unroll 1
            for (int mb = 0; mb < 2; ++mb) {
                const int dim = (int)rank * 256 + mb * 128 + tok_l;   // the TMEM lane is a V dim here
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + lane_base + 128 + mb * 64 + c * 16, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int h = c * 16 + j;
                        if (h < nh) {
                            const float o = __uint_as_float(r[j]) * linv[h];
                            if (item.slot < 0) {
                                static_cast<T *>(a.out)[((int64_t)item.seq * a.num_heads + head0 + h) * kDv + dim] = Elem<T>::from_float(o);
                            } else {
                                a.plan.part_o[((int64_t)item.slot * a.num_heads + head0 + h) * kDv + dim] = o;
                            }
                        }
                    }
                }
            }
            // the next range's first P.V overwrites O^T: tell the issuer the read-out is over
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars[kOFree]);
            }
            acc[5] += tick() - t_ep;
            acc[7]++;
        }
        if (tracing && threadIdx.x == 0) {
            for (int k = 0; k < 8; ++k) {
                acct[8 + k] = (unsigned long long)acc[k];
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tracing && threadIdx.x == 0) {
        unsigned long long t_end;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
        a.trace[1 + 2 * blockIdx.x] = t_start;
        a.trace[2 + 2 * blockIdx.x] = t_end;
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    // a CTA's shared memory must outlive the peer's last access to it
    cluster_sync_all();
}

} // namespace

bool pa_mla_split_supported(int dk, int dv, int v_row_dim, int rope_dim, int block_size, int kv_heads, int q_dtype,
                            int kv_dtype)
{
    const bool rows_ok = (rope_dim == 0 && v_row_dim == kDk) || (rope_dim == kDk - kDv && v_row_dim == kDv);
    return dk == kDk && dv == kDv && rows_ok && kv_heads == 1 && block_size >= kBox && block_size % kBox == 0 &&
           block_size <= 256 && q_dtype == kBf16 && kv_dtype == kBf16;
}

// CTA pairs that can be resident at once on the current device (pairs are placed within a GPC, so this may be less
// than SMs / 2); 0 if the query fails.  Cached per device.
int pa_mla_split_max_pairs()
{
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return 0;
    }
    if (cached[dev] == 0) {
        if (cudaFuncSetAttribute(pa_mla_split_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
            return 0;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 148);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, pa_mla_split_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return 0;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

cudaError_t launch_pa_mla_split(const PaArgs &args, int num_blocks, cudaStream_t stream)
{
    TmaEncodeFn fn = tma_encode_fn();
    if (fn == nullptr) {
        return cudaErrorInvalidValue;
    }
    const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    // cache [num_blocks][block_size][1][row]; box = 64 elements x 64 tokens of one block
    auto encode_cache = [&](CUtensorMap *map, const void *base, int row) {
        cuuint64_t dims[4] = {(cuuint64_t)row, 1, (cuuint64_t)args.block_size, (cuuint64_t)num_blocks};
        cuuint64_t strides[3] = {(cuuint64_t)row * 2, (cuuint64_t)row * 2, (cuuint64_t)args.block_size * row * 2};
        cuuint32_t box[4] = {64, 1, kBox, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        return fn(map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    // query [tokens][num_heads][row]; box = 64 elements x 64 heads of one token (rows past num_heads read as zero)
    auto encode_q = [&](CUtensorMap *map, const void *base, int row) {
        cuuint64_t dims[3] = {(cuuint64_t)row, (cuuint64_t)args.num_heads, (cuuint64_t)args.batch};
        cuuint64_t strides[2] = {(cuuint64_t)row * 2, (cuuint64_t)args.num_heads * row * 2};
        cuuint32_t box[3] = {64, kHeads, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        return fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const bool split = args.k_rope != nullptr;
    CUtensorMap km, rm, qm, qrm;
    if (!encode_cache(&km, args.k_cache, split ? kDv : kDk) ||
        !encode_cache(&rm, split ? args.k_rope : args.k_cache, split ? kDk - kDv : kDk) ||
        !encode_q(&qm, args.q, split ? kDv : kDk) ||
        !encode_q(&qrm, split ? args.q_rope : args.q, split ? kDk - kDv : kDk)) {
        return cudaErrorInvalidValue;
    }
    const bool traced = args.trace != nullptr;
    auto kern = traced ? pa_mla_split_kernel<true> : pa_mla_split_kernel<false>;
    static bool configured_all[2][64] = {};
    bool *configured = configured_all[traced ? 1 : 0];
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
    cfg.gridDim = dim3((unsigned)(2 * args.plan.n_cta_groups * args.plan.cols));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, km, rm, qm, qrm, args);
}

} // namespace atb_b200
