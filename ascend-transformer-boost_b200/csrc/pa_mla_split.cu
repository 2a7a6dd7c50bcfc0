// Paged decode attention over the MLA latent cache (one kv head, K row = 512 latent + 64 rope dims, V = the latent
// part), bf16, as a pair of CTAs (a thread-block cluster of two) per (token range, 64 query heads).
//
// Both contractions run TRANSPOSED, with the 128 tokens of a tile in the M dimension of tcgen05.mma, so that every
// instruction is a full-rate M = 128 MMA:
//     S^T[128 tokens x 64 heads] = K[tokens x dims] . Q^T          A = K tile (shared memory), B = Q (shared memory)
//     O^T[dims x 64 heads]      += V^T[dims x tokens] . P^T         A = V^T = the same K tile read MN-major, B = P^T
// A 128-token tile of the cache is 144 KB and would fit shared memory once, next to Q, with nothing left to load
// the next tile into.  So the two CTAs of the pair split the 576 DIMS evenly: rank r owns latent dims 256r..256r+255
// (4 atoms of 64 dims, 128-byte swizzle) and rope dims 32r..32r+31 (a half atom, 64-byte swizzle).  Each loads only
// its dims of every tile (72 KB: two stages fit), computes the partial S^T over its dims and the O^T rows of its own
// latent dims.  The softmax is split by HEADS: rank r owns heads 32r..32r+31.  Once per tile each CTA sends the partial
// scores of the peer's heads into the peer's shared memory (distributed shared memory, 16-byte stores that a warp
// lays out as 512 contiguous bytes), adds what it received to its own partial, applies the softmax and writes its
// heads' part of P^T (bf16) into both CTAs' copies of P^T.
//
// The softmax of the transposed scores is element-wise: a thread owns one token (one TMEM lane) and 16 heads.
// Instead of the running row maximum it subtracts a per-head reference, the score of the range's first token, and
// clamps the exponent at +100: bf16 has the exponent range of fp32, so P keeps its relative precision wherever the
// reference lies, the first token contributes exactly 1 to the row sum (never 0), and a score more than 2^100 times
// above the reference - which no softmax input reaches - would only be weighted as 2^100.  Row sums are kept per thread
// and reduced across the 128 tokens once per range.
//
// Warp roles in each CTA: warps 0-7 partial-score exchange, softmax and the read-out of O^T (warp w reads TMEM lane
// quarter w % 4 and the heads 16 (w / 4).. of either half); warp 8 TMA producer; warp 9 MMA issuer and owner of the
// tensor-memory allocation.  P^T is single-buffered: P.V hands it back in two halves of 64 tokens (one commit each),
// and a warp passes its own CTA's hand-back on to the peer, whose copy of P^T it also writes.  Every wait is bounded;
// a wait that runs out sets the status word and an abort flag that drains every loop of the CTA; its peer then runs
// out of its own waits.  Both CTAs always reach the final cluster barrier.
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
constexpr int kMine = kHeads / 2;              // heads whose softmax one CTA computes
constexpr int kTile = 128;                     // tokens per tile = M of both contractions
constexpr int kBox = 64;                       // tokens per TMA box (token ranges start at multiples of it)
constexpr int kDk = 576, kDv = 512;
constexpr int kFullAtoms = 4;                  // atoms of 64 dims (128-byte rows) per CTA: its half of the latent part
constexpr int kAtomBytes = kTile * 128;        // 128 tokens x 64 dims: 16 KB
constexpr int kHalfAtomBytes = kTile * 64;     // 128 tokens x 32 rope dims: 8 KB, 64-byte swizzle
constexpr int kQAtomBytes = kHeads * 128;      // 64 heads x 64 dims: 8 KB
constexpr int kQHalfBytes = kHeads * 64;       // 64 heads x 32 rope dims: 4 KB
constexpr int kQBytes = kFullAtoms * kQAtomBytes + kQHalfBytes;      // 36 KB
constexpr int kStageBytes = kFullAtoms * kAtomBytes + kHalfAtomBytes; // 72 KB
constexpr int kStages = 2;
constexpr int kPBytes = kTile * 128;           // P^T: 128 tokens x 64 heads, bf16
constexpr int kRecvBytes = kMine * kTile * 4;  // the peer's partial S^T of this CTA's heads: [head / 4][token][4] fp32
constexpr int kBigBytes = kQBytes + kStages * kStageBytes + kPBytes + kRecvBytes; // 212 KB
constexpr int kSmallBytes = 4096;              // barriers, tmem slot, flags, reference scores, row-sum scratch
constexpr int kSmemBytes = kBigBytes + kSmallBytes + 1024;
constexpr int kSoftmaxWarps = 8;
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
constexpr uint32_t kTmemCols = 256;            // S^T buffers at columns 0 and 64, O^T blocks at 128 and 192
constexpr float kMaxExponent = 100.f;
static_assert(kQBytes % 1024 == 0 && kStageBytes % 1024 == 0 && (kFullAtoms * kAtomBytes) % 1024 == 0, "swizzle atoms stay aligned");

enum Bar {
    kQFull = 0, kQEmpty, kStEmpty0, kStEmpty1, kSFull0, kSFull1, kSEmpty0, kSEmpty1,
    kPFull, kPvDone, kPHalf0, kPHalf1, kMref, kWsum, kLinv, kOFree,
    kStFull0,                                  // one per stage and atom (the rope half last): stage s, atom k at kStFull0 + 5 s + k
    kRecvFull0 = kStFull0 + 2 * (kFullAtoms + 1), kRecvEmpty0 = kRecvFull0 + kSoftmaxWarps,
    kNumBars = kRecvEmpty0 + kSoftmaxWarps
};

struct Small {
    uint64_t bars[kNumBars];
    uint32_t tmem_slot;
    int abort_flag;
    alignas(16) float mref[2][kMine]; // reference score of this CTA's heads, log2 domain (double-buffered over ranges)
    float wsum[2][4][kMine];   // row sums of this CTA's heads per token quarter (double-buffered over ranges)
    float lfull[2][kMine];     // row sum of this CTA's heads, for the log-sum-exp
    unsigned long long pdone[4]; // timing probe: when the last warp finished a tile's P^T
    float linv[2][kHeads];     // 1 / row sum of all heads (each CTA fills its half in both), double-buffered over ranges
};
static_assert(sizeof(Small) <= kSmallBytes, "small shared-memory area");

// kTrace: the build with the timing probe (atb_b200_pa_plan_set_trace with CTA selector 255): every CTA stores the
// global timer at its start and end in trace[1 + 2b], trace[2 + 2b], and 8 cycle counters of its issuing thread and 24
// of thread 0 from trace[2 + 2 * grid + 32b] on.  The product build carries none of it.
// adds the cycles since the last mark to counter k (timing-probe build only)
#define TK(k)                                 \
    do {                                      \
        if (kTrace > 1) {                     \
            const long long now_ = clock64(); \
            acc[k] += now_ - t0;              \
            t0 = now_;                        \
        }                                     \
    } while (0)

template <int kTrace>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
pa_mla_split_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap khmap,
                    const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qhmap, const PaArgs a)
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
    uint8_t *q_smem = base;
    uint8_t *st_smem = base + kQBytes;
    uint8_t *p_smem = st_smem + kStages * kStageBytes;
    uint8_t *recv = p_smem + kPBytes;

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
            for (int k = 0; k <= kFullAtoms; ++k) {
                mbar_init(&bars[kStFull0 + 5 * s + k], 1);
            }
            mbar_init(&bars[kStEmpty0 + s], 1);
            mbar_init(&bars[kSFull0 + s], 1);
            mbar_init(&bars[kSEmpty0 + s], kSoftmaxWarps);
        }
        // P^T of a tile is written by the eight softmax warps of BOTH CTAs, each half of the heads into both copies: the
        // own warps arrive, the peer's stores count their bytes
        mbar_init(&bars[kPFull], kSoftmaxWarps);
        mbar_init(&bars[kPvDone], 1);
        for (int k = 0; k < 2; ++k) {
            mbar_init(&bars[kPHalf0 + k], 2);     // P.V has consumed tokens 64k..64k+63 of P^T, in this CTA and in the peer
        }
        for (int w = 0; w < kSoftmaxWarps; ++w) {
            mbar_init(&bars[kRecvFull0 + w], 1);  // the partial scores sent by warp w of the peer have landed (byte count)
            mbar_init(&bars[kRecvEmpty0 + w], 1); // warp w of the peer has read what this CTA's warp w sent
        }
        mbar_init(&bars[kMref], 2);
        mbar_init(&bars[kWsum], kSoftmaxWarps);
        mbar_init(&bars[kLinv], 2);
        mbar_init(&bars[kOFree], kSoftmaxWarps);
        sm->abort_flag = 0;
        for (int k = 0; k < 4; ++k) {
            sm->pdone[k] = 0;
        }
        fence_barrier_init();
    }
    if (warp == kSoftmaxWarps + 1) {
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
    const bool tracing = kTrace != 0 && a.trace != nullptr && (a.trace_cap >> 24) >= 254u &&
                         2 + 34 * gridDim.x + 1024 <= (a.trace_cap & 0xffffffu);
    unsigned long long t_start = 0;
    if (tracing && threadIdx.x == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    }
    unsigned long long *acct = tracing ? a.trace + 2 + 2 * gridDim.x + 32 * blockIdx.x : nullptr;
    long long acc[24] = {};
    // CTAs 0 and 1 also record a timeline: 8 clock values for each of their first 64 tiles
    unsigned long long *tl = tracing && blockIdx.x < 2 ? a.trace + 2 + 34 * gridDim.x + 512 * blockIdx.x : nullptr;
    auto mark = [&](uint32_t tile, int ev) {
        if (kTrace && tl != nullptr && tile < 64) {
            tl[8 * tile + ev] = (unsigned long long)clock64();
        }
    };
    auto tick = [&]() -> long long { return kTrace > 1 ? clock64() : 0; };
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

    if (warp == kSoftmaxWarps) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&khmap);
            tma_prefetch_desc(&qmap);
            tma_prefetch_desc(&qhmap);
        }
        // the rope half of this CTA: 32 dims of the rope tensor, or of the combined row behind the latent part
        const int rope_x = (a.k_rope != nullptr ? 0 : kDv) + 32 * (int)rank;
        const int atom_x = kFullAtoms * 64 * (int)rank;
        uint32_t g = 0;
        bool alive = true;
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
            const int32_t *bt = a.block_tables + (int64_t)(a.bt_rows != nullptr ? a.bt_rows[item.seq] : item.seq) * a.max_blocks;
            if (lane == 0) {
                // the query block of this range: this CTA's dims of the 64 head rows
                if (!wait(kQEmpty, (i & 1) ^ 1u, false)) {
                    alive = false;
                } else {
                    mbar_expect_tx(&bars[kQFull], kQBytes);
                    for (int at = 0; at < kFullAtoms; ++at) {
                        tma_load_3d(q_smem + at * kQAtomBytes, &qmap, &bars[kQFull], atom_x + at * 64, head0, item.seq);
                    }
                    tma_load_3d(q_smem + kFullAtoms * kQAtomBytes, &qhmap, &bars[kQFull], rope_x, head0, item.seq);
                }
            }
            alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
            for (int t = 0; t < n_tiles && alive; ++t, ++g) {
                if (lane == 0) {
                    const int s = g & 1;
                    // where the tile's boxes lie, and their lines on the way into L2, while the stage is still in use: the
                    // loads below then find the block ids in registers and the data in L2
                    const int tok0 = item.tok_begin + t * kTile;
                    const int n_box = (item.tok_end - tok0 > kBox) ? 2 : 1;
                    int blk[2], tib[2];
#pragma unroll
                    for (int bx = 0; bx < 2; ++bx) {
                        const int tok = tok0 + bx * kBox;
                        blk[bx] = bx < n_box ? bt[tok / a.block_size] : 0;
                        tib[bx] = tok % a.block_size;
                        if ((unsigned)blk[bx] >= (unsigned)a.num_blocks) {
                            // a caller error: report it, and load a zero tile instead of whatever lies there
                            atomicExch(a.plan.status, kStatusBadBlockId);
                            blk[bx] = -1;
                        }
                    }
#pragma unroll
                    for (int bx = 0; bx < 2; ++bx) {
                        if (bx < n_box && blk[bx] >= 0) {
                            for (int at = 0; at < kFullAtoms; ++at) {
                                tma_prefetch_4d(&kmap, atom_x + at * 64, 0, tib[bx], blk[bx]);
                            }
                            tma_prefetch_4d(&khmap, rope_x, 0, tib[bx], blk[bx]);
                        }
                    }
                    if (!wait(kStEmpty0 + s, ((g >> 1) & 1) ^ 1u, false)) {
                        alive = false;
                    } else {
                        mark(g, 0);
                        uint8_t *dst = st_smem + s * kStageBytes;
                        // atom by atom, each with a barrier of its own: Q.K^T starts on the first while the others are on
                        // their way
                        for (int at = 0; at < kFullAtoms; ++at) {
                            uint64_t *full = &bars[kStFull0 + 5 * s + at];
                            mbar_expect_tx(full, n_box * kBox * 128);
#pragma unroll
                            for (int bx = 0; bx < 2; ++bx) {
                                if (bx < n_box) {
                                    tma_load_4d(dst + at * kAtomBytes + bx * kBox * 128, &kmap, full, atom_x + at * 64, 0, tib[bx], blk[bx]);
                                }
                            }
                        }
                        {
                            uint64_t *full = &bars[kStFull0 + 5 * s + kFullAtoms];
                            mbar_expect_tx(full, n_box * kBox * 64);
#pragma unroll
                            for (int bx = 0; bx < 2; ++bx) {
                                if (bx < n_box) {
                                    tma_load_4d(dst + kFullAtoms * kAtomBytes + bx * kBox * 64, &khmap, full, rope_x, 0, tib[bx], blk[bx]);
                                }
                            }
                        }
                        mark(g, 1);
                    }
                }
                alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
            }
        }
    } else if (warp == kSoftmaxWarps + 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc_ab(1, 0, 0, kHeads, kTile); // A = K tile, B = Q, both K-major
            constexpr uint32_t idesc_pv = instr_desc_ab(1, 1, 1, kHeads, kTile); // A = V^T, B = P^T, both MN-major
            const uint32_t q_addr = smem_u32(q_smem), st_addr = smem_u32(st_smem), p_addr = smem_u32(p_smem);
            const uint64_t dp0 = smem_desc(p_addr, kAtomBytes, 1024);
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
                const long long t_range = tick();
                // P.V of the oldest tile whose P^T is complete: asked for at every point where this thread would wait
                auto try_pv = [&]() -> bool {
                    const uint32_t gp = g + next_pv;
                    if (!(next_pv < next_qk && mbar_test_wait_cluster(&bars[kPFull], gp & 1))) {
                        return false;
                    }
                    // the first P.V of a range overwrites O^T: the previous range's read-out must be over
                    if (!(o_free || next_pv > 0 || ready(kOFree, (i & 1) ^ 1u))) {
                        return false;
                    }
                    o_free = true;
                    const long long t0 = tick();
                    mark(gp, 6);
                    if (kTrace && tl != nullptr && gp < 64) {
                        tl[8 * gp + 5] = sm->pdone[gp & 3];   // the last of this CTA's warps
                        sm->pdone[gp & 3] = 0;
                    }
                    tc_fence_after();
                    fence_proxy_async();     // P^T was written by ordinary stores, half of it by the peer CTA's
                    const uint32_t vb = st_addr + (gp & 1) * kStageBytes;
                    // V^T rows of 128 dims = two atoms kAtomBytes apart; 8-token groups 1024 B apart
                    const uint64_t dv0 = smem_desc(vb, kAtomBytes, 1024);
                    // tokens 0..63 first, then 64..127: each half of P^T is handed back to the softmax warps of both CTAs as
                    // soon as its MMAs have completed
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
#pragma unroll
                        for (int mb = 0; mb < 2; ++mb) {
#pragma unroll
                            for (int ks = 4 * half; ks < 4 * half + 4; ++ks) {
                                tc_mma(tmem_base + 128 + mb * 64, dv0 + ((2 * mb * kAtomBytes + ks * 2048) >> 4), dp0 + ((ks * 2048) >> 4),
                                       idesc_pv, next_pv != 0 || ks != 0);
                            }
                        }
                        tc_commit_pair(&bars[kPHalf0 + half]);
                    }
                    tc_commit(&bars[kStEmpty0 + (gp & 1)]);
                    tc_commit(&bars[kPvDone]);
                    ++next_pv;
                    mark(gp, 7);
                    acc[1] += tick() - t0;
                    return true;
                };
                uint32_t idle = 0;
                while (next_pv < n_tiles && alive) {
                    if (try_pv()) {
                        idle = 0;
                        continue;
                    }
                    const uint32_t gq = g + next_qk;
                    const int stg = gq & 1;
                    const uint32_t ph = (gq >> 1) & 1;
                    if (next_qk < n_tiles && next_qk < next_pv + 2 && ready(kSEmpty0 + stg, ph ^ 1u) && ready(kStFull0 + 5 * stg, ph)) {
                        // Q.K^T atom by atom as the atoms land; a P.V that becomes ready in between goes first
                        const long long t0 = tick();
                        mark(gq, 2);
                        tc_fence_after();
                        const uint64_t da0 = smem_desc(st_addr + stg * kStageBytes, 16, 1024);
                        const uint64_t db0 = smem_desc(q_addr, 16, 1024);
                        const uint32_t ds = tmem_base + stg * 64;
#pragma unroll
                        for (int at = 0; at <= kFullAtoms; ++at) {
                            if (at > 0) {
                                try_pv();
                                uint32_t spins = 0;
                                while (!ready(kStFull0 + 5 * stg + at, ph)) {
                                    if (try_pv()) {
                                        spins = 0;
                                    } else if (++spins > (1u << 22) || *abort_flag) {
                                        *abort_flag = 1;
                                        atomicExch(a.plan.status, kStatusWaitTimeout);
                                        alive = false;
                                        break;
                                    }
                                }
                                if (!alive) {
                                    break;
                                }
                                tc_fence_after();
                            }
                            if (at < kFullAtoms) {
#pragma unroll
                                for (int ks = 0; ks < 4; ++ks) {
                                    tc_mma(ds, da0 + ((at * kAtomBytes + ks * 32) >> 4), db0 + ((at * kQAtomBytes + ks * 32) >> 4), idesc_qk,
                                           (at | ks) != 0);
                                }
                            } else {
                                // the 32 rope dims: rows of 64 bytes, 64-byte swizzle, 8-row groups 512 B apart
                                const uint64_t dra = smem_desc_sw64(st_addr + stg * kStageBytes + kFullAtoms * kAtomBytes, 16, 512);
                                const uint64_t drb = smem_desc_sw64(q_addr + kFullAtoms * kQAtomBytes, 16, 512);
#pragma unroll
                                for (int ks = 0; ks < 2; ++ks) {
                                    tc_mma(ds, dra + ((ks * 32) >> 4), drb + ((ks * 32) >> 4), idesc_qk, true);
                                }
                            }
                        }
                        if (!alive) {
                            break;
                        }
                        tc_commit(&bars[kSFull0 + stg]);
                        if (next_qk + 1 == n_tiles) {
                            tc_commit(&bars[kQEmpty]); // the query block of this range is no longer needed
                        }
                        ++next_qk;
                        mark(gq, 3);
                        idle = 0;
                        acc[0] += tick() - t0;
                    } else {
                        ++idle;
                        if (idle > (1u << 22) || *abort_flag) {
                            *abort_flag = 1;
                            atomicExch(a.plan.status, kStatusWaitTimeout);
                            alive = false;
                        }
                    }
                }
                g += n_tiles;
                acc[6] += tick() - t_range;
            }
            if (tracing) {
                for (int k = 0; k < 8; ++k) {
                    acct[k] = (unsigned long long)acc[k];
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ warps 0..7: one token (TMEM lane) and 16 + 16
        // heads per thread: 16 of this CTA's heads (softmax here) and 16 of the peer's (partial scores sent over)
        const int q4 = warp & 3;                                       // TMEM lane quarter this warp may read
        const int hh = warp >> 2;                                      // which 16 of each CTA's 32 heads
        const int tok_l = q4 * 32 + lane;                              // row of the tile
        const int half = q4 >> 1;                                      // which 64 tokens of P^T this warp writes
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const int my_col = kMine * (int)rank + 16 * hh;                // first of this thread's own heads
        const int peer_col = kMine * (int)peer + 16 * hh;              // first of the heads it forwards
        // [head / 4][token][4 floats]: a warp's 16-byte accesses are 512 contiguous bytes
        const uint32_t recv_off = (uint32_t)(4 * hh) * (kTile * 16) + (uint32_t)tok_l * 16;
        const uint32_t peer_recv = map_to_cta(smem_u32(recv), peer) + recv_off;
        const uint32_t peer_p = map_to_cta(smem_u32(p_smem), peer);
        const uint32_t peer_pfull = peer_bar(kPFull);
        uint32_t g = 0;
        bool alive = true;
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
            float lsum[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                lsum[j] = 0.f;
            }
            float *mref = sm->mref[i & 1];
            for (int t = 0; t < n_tiles && alive; ++t, ++g) {
                const int sb = g & 1;
                const int valid = min(kTile, item.tok_end - (item.tok_begin + t * kTile));
                long long t0 = tick();
                (void)t0;
                if (!wait(kSFull0 + sb, (g >> 1) & 1, false)) {
                    alive = false;
                    break;
                }
                TK(0);
                if (threadIdx.x == 0) {
                    mark(g, 4);
                }
                tc_fence_after();
                uint32_t mine[16], theirs[16];
                tmem_ld16(tmem_base + lane_base + sb * 64 + peer_col, theirs);
                tmem_ld16(tmem_base + lane_base + sb * 64 + my_col, mine);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kSEmpty0 + sb]);
                }
                TK(1);
                // ---- the peer's heads: partial scores into its receive buffer; the stores count their bytes on the peer's
                // barrier, and this warp expects as many from the peer's warp of the same number
                if (lane == 0) {
                    mbar_expect_tx(&bars[kRecvFull0 + warp], 32 * 4 * 16);
                }
                if (!wait(kRecvEmpty0 + warp, (g & 1) ^ 1u, false)) {
                    alive = false;
                    break;
                }
                TK(2);
                {
                    const uint32_t full = peer_bar(kRecvFull0 + warp);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        st_async_v4(peer_recv + c * (kTile * 16), theirs[4 * c], theirs[4 * c + 1], theirs[4 * c + 2], theirs[4 * c + 3], full);
                    }
                }
                TK(3);
                // rows of V past the end of the range may hold anything: clear them (0 * NaN != 0); the K rows only
                // feed the scores of those tokens, which get probability 0 below.  Two warps share a token row.
                if (valid < kTile) {
                    uint8_t *stg = st_smem + sb * kStageBytes;
                    if (tok_l >= valid) {
                        for (int at = 2 * hh; at < 2 * hh + 2; ++at) {
#pragma unroll
                            for (int ch = 0; ch < 8; ++ch) {
                                *reinterpret_cast<uint4 *>(stg + at * kAtomBytes + tok_l * 128 + (ch << 4)) = make_uint4(0, 0, 0, 0);
                            }
                        }
                    }
                    fence_proxy_async();
                }
                TK(4);
                // ---- this CTA's heads: add the peer's partial, scale, reference, exponentials
                if (!wait(kRecvFull0 + warp, g & 1, true)) {
                    alive = false;
                    break;
                }
                TK(5);
                float s[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 r = *reinterpret_cast<const float4 *>(recv + recv_off + c * (kTile * 16));
                    s[4 * c] = __uint_as_float(mine[4 * c]) + r.x;
                    s[4 * c + 1] = __uint_as_float(mine[4 * c + 1]) + r.y;
                    s[4 * c + 2] = __uint_as_float(mine[4 * c + 2]) + r.z;
                    s[4 * c + 3] = __uint_as_float(mine[4 * c + 3]) + r.w;
                }
                TK(6);
                if (t == 0) {
                    // the reference of a head: the score of the range's first token
                    if (tok_l == 0) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            mref[16 * hh + j] = s[j] * a.scale_log2;
                        }
                        mbar_arrive(&bars[kMref]);
                    }
                    if (!wait(kMref, i & 1, false)) {
                        alive = false;
                        break;
                    }
                }
                TK(7);
                const bool live = tok_l < valid;
                uint32_t pk[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 m = reinterpret_cast<const float4 *>(mref + 16 * hh)[c];
                    float p0 = fast_exp2(fminf(fmaf(s[4 * c], a.scale_log2, -m.x), kMaxExponent));
                    float p1 = fast_exp2(fminf(fmaf(s[4 * c + 1], a.scale_log2, -m.y), kMaxExponent));
                    float p2 = fast_exp2(fminf(fmaf(s[4 * c + 2], a.scale_log2, -m.z), kMaxExponent));
                    float p3 = fast_exp2(fminf(fmaf(s[4 * c + 3], a.scale_log2, -m.w), kMaxExponent));
                    if (!live) {
                        p0 = p1 = p2 = p3 = 0.f;
                    }
                    lsum[4 * c] += p0;
                    lsum[4 * c + 1] += p1;
                    lsum[4 * c + 2] += p2;
                    lsum[4 * c + 3] += p3;
                    pk[2 * c] = Elem<T>::pack2(p0, p1);
                    pk[2 * c + 1] = Elem<T>::pack2(p2, p3);
                }
                // what was received has been consumed (the arithmetic above depends on it): the peer may send the next tile's
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster_relaxed(peer_bar(kRecvEmpty0 + warp));
                }
                TK(8);
                // this half of P^T(g) overwrites that of P^T(g-1): both CTAs' P.V(g-1) must have consumed it
                if (g > 0 && !wait(kPHalf0 + half, (g - 1) & 1, false)) {
                    alive = false;
                    break;
                }
                TK(9);
                {
                    // row of P^T: 64 heads = 8 chunks of 16 B, 128-byte swizzle; this thread's 16 heads are two of them, and go
                    // to the same place in the peer's copy (first: those stores take longest to land)
                    const int ch = my_col / 8;
                    const uint32_t off0 = (uint32_t)tok_l * 128 + (uint32_t)((ch ^ (tok_l & 7)) << 4);
                    const uint32_t off1 = (uint32_t)tok_l * 128 + (uint32_t)(((ch + 1) ^ (tok_l & 7)) << 4);
                    st_async_v4(peer_p + off0, pk[0], pk[1], pk[2], pk[3], peer_pfull);
                    st_async_v4(peer_p + off1, pk[4], pk[5], pk[6], pk[7], peer_pfull);
                    *reinterpret_cast<uint4 *>(p_smem + off0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4 *>(p_smem + off1) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
                TK(11);
                fence_proxy_async();   // this CTA's copy: ordinary stores, read by the tensor core
                __syncwarp();
                if (lane == 0) {
                    if (warp == 0) {
                        mbar_expect_tx(&bars[kPFull], kPBytes / 2);   // the peer's half of the tile's P^T
                    } else {
                        mbar_arrive(&bars[kPFull]);
                    }
                }
                TK(12);
                if (kTrace && tl != nullptr && lane == 0) {
                    atomicMax(&sm->pdone[g & 3], (unsigned long long)clock64());
                }
                acc[14]++;
            }
            if (!alive) {
                break;
            }
            // ---- end of the token range: row sums -> 1 / l in both CTAs, then O^T / l -> output row or partial
            const long long t_ep = tick();
            long long t0 = t_ep;
            (void)t0;
            float *linv = sm->linv[i & 1];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float v = lsum[j];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    v += __shfl_xor_sync(0xffffffffu, v, off);
                }
                if (lane == 0) {
                    sm->wsum[i & 1][q4][16 * hh + j] = v;
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars[kWsum]);
            }
            TK(16);
            if (!wait(kWsum, i & 1, false)) {
                alive = false;
                break;
            }
            TK(17);
            if (warp == 0) {
                const int h = lane;                                   // one of this CTA's heads
                const float l = sm->wsum[i & 1][0][h] + sm->wsum[i & 1][1][h] + sm->wsum[i & 1][2][h] + sm->wsum[i & 1][3][h];
                const float inv = 1.f / l;
                linv[kMine * rank + h] = inv;
                sm->lfull[i & 1][h] = l;
                st_cluster_f32(map_to_cta(smem_u32(&linv[kMine * rank + h]), peer), inv);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kLinv]);
                    mbar_arrive_cluster(peer_bar(kLinv));
                }
            }
            TK(18);
            if (!wait(kLinv, i & 1, true)) {
                alive = false;
                break;
            }
            TK(19);
            // every P.V of the range has completed here
            if (!wait(kPvDone, (g - 1) & 1, false)) {
                alive = false;
                break;
            }
            TK(20);
            tc_fence_after();
            if (warp == 0) {
                const int h = kMine * (int)rank + lane;
                if (h < nh) {
                    const float lse2 = mref[lane] + log2f(sm->lfull[i & 1][lane]);
                    if (item.slot >= 0) {
                        a.plan.part_lse[(int64_t)item.slot * a.num_heads + head0 + h] = lse2;
                    } else if (a.lse_out != nullptr) {
                        // whole sequence in this range: its log-sum-exp, natural log
                        static_cast<T *>(a.lse_out)[(int64_t)item.seq * a.num_heads + head0 + h] =
                            Elem<T>::from_float(lse2 * 0.6931471805599453f);
                    }
                }
            }
            {
                // the TMEM lane is a V dim here: a warp's store covers 32 consecutive dims of one head
                const int dim0 = (int)rank * 256 + tok_l;
                float *po = item.slot >= 0 ? a.plan.part_o + ((int64_t)item.slot * a.num_heads + head0 + 32 * hh) * kDv + dim0 : nullptr;
                T *oo = static_cast<T *>(a.out) + ((int64_t)item.seq * a.num_heads + head0 + 32 * hh) * kDv + dim0;
                const int n_mine = min(32, nh - 32 * hh);   // heads of this warp that exist
#pragma unroll
                for (int mb = 0; mb < 2; ++mb) {
                    uint32_t r0[16], r1[16];
                    tmem_ld16(tmem_base + lane_base + 128 + mb * 64 + 32 * hh, r0);
                    tmem_ld16(tmem_base + lane_base + 128 + mb * 64 + 32 * hh + 16, r1);
                    tmem_wait_ld();
                    if (po != nullptr) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < n_mine) {
                                po[j * kDv + mb * 128] = __uint_as_float(j < 16 ? r0[j & 15] : r1[j & 15]) * linv[32 * hh + j];
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < n_mine) {
                                oo[j * kDv + mb * 128] =
                                    Elem<T>::from_float(__uint_as_float(j < 16 ? r0[j & 15] : r1[j & 15]) * linv[32 * hh + j]);
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
            TK(21);
            acc[13] += tick() - t_ep;
            acc[15]++;
        }
        if (tracing && threadIdx.x == 0) {
            for (int k = 0; k < 24; ++k) {
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
    if (warp == kSoftmaxWarps + 1) {
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
        if (cudaFuncSetAttribute(pa_mla_split_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
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
        if (cudaOccupancyMaxActiveClusters(&n, pa_mla_split_kernel<0>, &cfg) != cudaSuccess || n <= 0) {
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
    // cache [num_blocks][block_size][1][row]; box = 64 elements x 64 tokens of one block with the 128-byte swizzle, or
    // (the rope halves) 32 elements x 64 tokens with the 64-byte swizzle
    auto encode_cache = [&](CUtensorMap *map, const void *base, int row, bool half) {
        cuuint64_t dims[4] = {(cuuint64_t)row, 1, (cuuint64_t)args.block_size, (cuuint64_t)num_blocks};
        cuuint64_t strides[3] = {(cuuint64_t)row * 2, (cuuint64_t)row * 2, (cuuint64_t)args.block_size * row * 2};
        cuuint32_t box[4] = {half ? 32u : 64u, 1, kBox, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        return fn(map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  half ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    // query [tokens][num_heads][row]; box = 64 (32) elements x 64 heads of one token (rows past num_heads read as zero)
    auto encode_q = [&](CUtensorMap *map, const void *base, int row, bool half) {
        cuuint64_t dims[3] = {(cuuint64_t)row, (cuuint64_t)args.num_heads, (cuuint64_t)args.batch};
        cuuint64_t strides[2] = {(cuuint64_t)row * 2, (cuuint64_t)args.num_heads * row * 2};
        cuuint32_t box[3] = {half ? 32u : 64u, kHeads, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        return fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  half ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const bool split = args.k_rope != nullptr;
    CUtensorMap km, rm, qm, qrm;
    if (!encode_cache(&km, args.k_cache, split ? kDv : kDk, false) ||
        !encode_cache(&rm, split ? args.k_rope : args.k_cache, split ? kDk - kDv : kDk, true) ||
        !encode_q(&qm, args.q, split ? kDv : kDk, false) ||
        !encode_q(&qrm, split ? args.q_rope : args.q, split ? kDk - kDv : kDk, true)) {
        return cudaErrorInvalidValue;
    }
    // CTA selector 255: all cycle counters; 254: the CTA spans and the timeline only (perturbs the kernel far less)
    const int traced = args.trace == nullptr ? 0 : ((args.trace_cap >> 24) == 254u ? 1 : 2);
    auto kern = traced == 0 ? pa_mla_split_kernel<0> : (traced == 1 ? pa_mla_split_kernel<1> : pa_mla_split_kernel<2>);
    static bool configured_all[3][64] = {};
    bool *configured = configured_all[traced];
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
