// Paged decode attention over the MLA latent cache (one kv head, K row = 512 latent + 64 rope dims, V = the latent
// part), bf16, as a pair of CTAs (a thread-block cluster of two) per (token range, 128 query heads).
//
// Why a pair, and why 128 heads: a decode step of this shape is paced by a chain per tile of tokens (load, Q.K^T,
// softmax, P.V) that cannot be made short, so each link should carry as much work as the SM can hold.  With all 128
// heads of a DeepSeek-style model in the M dimension every tcgen05.mma runs at the full rate, and each K tile is
// fetched once for all heads.  One SM cannot hold that: the accumulator O[128 x 512] alone is all of tensor memory, and
// a 128-token tile of the cache is 144 KB of shared memory.  So the two CTAs of the pair split the 576 DIMS: rank r owns
// latent dims 256r..256r+255 (4 atoms of 64 dims, 128-byte swizzle) and rope dims 32r..32r+31 (a half atom, 64-byte
// swizzle).  Each loads only its dims of every tile (72 KB: two stages), computes the partial scores over its dims
// and the columns of O of its own latent dims:
//     S[128 heads x 128 tokens] = Q . K^T     A = Q, kept in TENSOR MEMORY for the whole token range (the rope part in
//                                             shared memory), B = K tile; 16 + 2 MMAs of N = 128
//     O[128 heads x 256 dims] += P . V        A = P, written to tensor memory by the softmax warps in place of S,
//                                             B = the same K tile read MN-major; 8 MMAs of N = 256
// The softmax is split by HEADS: rank r owns heads 64r..64r+63 (TMEM lane quarters 2r, 2r+1).  Per tile, the warps of
// the other two quarters send the partial scores of their rows into the peer's shared memory (distributed shared
// memory; 16-byte stores that count their bytes on a barrier of the receiving CTA and that a warp lays out as 512
// contiguous bytes); the owning warps add what they received to their own partial, apply the softmax, write P (bf16)
// into their lanes of tensor memory and send the same P to the peer, whose other-quarter warps copy it into their
// lanes.  Both CTAs then hold P for all 128 heads and multiply it with their own V dims.
//
// The softmax is element-wise: a thread owns one head (one TMEM lane) and 32 of the tile's tokens.  Instead of the
// running row maximum it subtracts a per-head reference, the score of the range's first token, and clamps the
// exponent at +100: bf16 has the exponent range of fp32, so P keeps its relative precision wherever the reference
// lies, the first token contributes exactly 1 to the row sum (never 0), and a score more than 2^100 times above the
// reference - which no softmax input reaches - would only be weighted as 2^100.  No rescaling of O, no cross-thread
// reduction per tile; row sums are kept per thread and added up once per range.  They add up P as rounded to bf16, the
// values P.V multiplies with: the weights of a row then sum to one exactly, and the rounding of a dominant P (which,
// unlike with a running maximum, is not 1.0 here) cancels between numerator and denominator.
//
// Tensor memory (512 columns): Q 0..127 (256 dims as bf16 pairs), S 128..255 (P over its first 64), O 256..511.  S has
// one buffer: per tile the MMA thread issues Q.K^T, waits for P, issues P.V and goes on to the next tile's Q.K^T, which
// the tensor core runs behind P.V in issue order.  Warps 0-15: exchange, softmax, Q into tensor memory, read-out of O
// (warp w: lane quarter w % 4, tokens 32 (w / 4).. of a tile); warp 16 TMA producer; warp 17 MMA issuer and owner of
// the tensor-memory allocation.  Every wait is bounded; a wait that runs out sets the status word and an abort flag
// that drains every loop of the CTA; its peer then runs out of its own waits.  Both CTAs always reach the final
// cluster barrier.
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

constexpr int kHeads = 128;                    // query heads per cluster = M of both contractions
constexpr int kOwn = kHeads / 2;               // heads whose softmax one CTA computes
constexpr int kTile = 128;                     // tokens per tile
constexpr int kBox = 64;                       // tokens per TMA box (token ranges start at multiples of it)
constexpr int kDk = 576, kDv = 512;
constexpr int kFullAtoms = 4;                  // atoms of 64 dims (128-byte rows) per CTA: its half of the latent part
constexpr int kAtomBytes = kTile * 128;        // 128 tokens x 64 dims: 16 KB
constexpr int kHalfAtomBytes = kTile * 64;     // 128 tokens x 32 rope dims: 8 KB, 64-byte swizzle
constexpr int kStageBytes = kFullAtoms * kAtomBytes + kHalfAtomBytes; // 72 KB
constexpr int kStages = 2;
constexpr int kQRopeBytes = kHeads * 64;       // 128 heads x 32 rope dims: 8 KB, 64-byte swizzle
constexpr int kRecvSBytes = kOwn * kTile * 4;  // the peer's partial scores of this CTA's heads: [token / 4][head][4] fp32
constexpr int kRecvPBytes = kOwn * kTile * 2;  // the peer's P of its heads: [token / 8][head][8] bf16
constexpr int kBigBytes = kStages * kStageBytes + kQRopeBytes + kRecvSBytes + kRecvPBytes; // 200 KB
constexpr int kSmallBytes = 6144;              // barriers, tmem slot, flags, reference scores, row-sum scratch
constexpr int kSmemBytes = kBigBytes + kSmallBytes + 1024;
constexpr int kSoftmaxWarps = 16;
constexpr int kParts = 2;                      // a tile's tokens go through Q.K^T, softmax and P.V in this many parts, each
                                               // with its own S / P columns and barriers, pipelined against one another
constexpr int kPartTok = kTile / kParts;       // tokens per part = N of a Q.K^T MMA
constexpr int kCgPerPart = 4 / kParts;         // a warp holds 32 tokens of a tile: warps (per lane quarter) per part
static_assert(kParts == 2 || kParts == 4, "a part is one or two warps' tokens");
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kQCol = 0, kSCol = 128, kOCol = 256;
constexpr float kMaxExponent = 100.f;
static_assert(kStageBytes % 1024 == 0 && (kFullAtoms * kAtomBytes) % 1024 == 0 && (kStages * kStageBytes) % 1024 == 0,
              "swizzle atoms stay aligned");

enum Bar {
    kQFull = 0, kQTmem, kQEmpty, kStEmpty0, kStEmpty1, kPvDone, kWsum, kLinv, kOFree,
    kSFull0,                                   // per part: its S is complete
    kPFull0 = kSFull0 + kParts,                // per part: P of all 128 heads is in tensor memory
    kQuadS0 = kPFull0 + kParts,                // per lane quarter and part: its warps have read their S
    kQuadM0 = kQuadS0 + 4 * kParts,            // 4: the reference scores of a quarter's heads are in shared memory
    kStFull0 = kQuadM0 + 4,                    // one per stage and atom (the rope half last): kStFull0 + 5 s + k
    kXSFull0 = kStFull0 + 2 * (kFullAtoms + 1), // per warp and 16 tokens (kXSFull0 + 16 c + w): partial scores from the peer's
                                               // warp of the same number have landed
    kXSEmpty0 = kXSFull0 + 2 * kSoftmaxWarps,  // per warp: the peer has read what this warp sent
    kXPFull0 = kXSEmpty0 + kSoftmaxWarps,      // per warp and 16 tokens: P from the peer's warp of the same number has landed
    kXPEmpty0 = kXPFull0 + 2 * kSoftmaxWarps,  // per warp: the peer has read the P this warp sent
    kNumBars = kXPEmpty0 + kSoftmaxWarps
};

struct Small {
    uint64_t bars[kNumBars];
    uint32_t tmem_slot;
    int abort_flag;
    float mref[2][kOwn];       // reference score of this CTA's heads, log2 domain (double-buffered over ranges)
    float wsum[2][4][kOwn];    // row sums of this CTA's heads per quarter of a tile's tokens (double-buffered)
    float lfull[2][kOwn];      // row sum of this CTA's heads, for the log-sum-exp
    float linv[2][kHeads];     // 1 / row sum of all heads (each CTA fills its half in both), double-buffered
};
static_assert(sizeof(Small) <= kSmallBytes, "small shared-memory area");

// One 256-bit store (eight 32-bit words) to a 32-byte aligned global address.
__device__ __forceinline__ void st_global_v8(void *p, const uint32_t *w)
{
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]),
                 "r"(w[6]), "r"(w[7])
                 : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                 "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}

// kTrace: the build with the timing probe (atb_b200_pa_plan_set_trace with CTA selector 254): every CTA stores the
// global timer at its start and end in trace[1 + 2b], trace[2 + 2b]; CTAs 0 and 1 also store a timeline of their first
// 64 tiles (16 clock values each) from trace[2 + 2 * grid + 1024 b] on.  The product build carries none of it.
template <bool kTrace>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
pa_mla_pair_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap khmap,
                   const __grid_constant__ CUtensorMap qhmap, const PaArgs a)
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
    uint8_t *st_smem = base;
    uint8_t *qr_smem = st_smem + kStages * kStageBytes;
    uint8_t *recv_s = qr_smem + kQRopeBytes;
    uint8_t *recv_p = recv_s + kRecvSBytes;

    const int cols = a.plan.cols;
    const int pair = blockIdx.x >> 1;
    const int grp = pair / cols;
    const int col = pair - grp * cols;
    const int head0 = col * kHeads;
    const int nh = min(kHeads, a.num_heads - head0);

    if (threadIdx.x == 0) {
        mbar_init(&bars[kQFull], 1);
        mbar_init(&bars[kQTmem], kSoftmaxWarps);
        mbar_init(&bars[kQEmpty], 1);
        for (int s = 0; s < 2; ++s) {
            for (int k = 0; k <= kFullAtoms; ++k) {
                mbar_init(&bars[kStFull0 + 5 * s + k], 1);
            }
            mbar_init(&bars[kStEmpty0 + s], 1);
        }
        for (int h = 0; h < kParts; ++h) {
            mbar_init(&bars[kSFull0 + h], 1);
            mbar_init(&bars[kPFull0 + h], kSoftmaxWarps / kParts);
        }
        mbar_init(&bars[kPvDone], 1);
        mbar_init(&bars[kWsum], kSoftmaxWarps / 2);
        mbar_init(&bars[kLinv], 4);               // two warps here, two in the peer
        mbar_init(&bars[kOFree], kSoftmaxWarps);
        for (int k = 0; k < 4 * kParts; ++k) {
            mbar_init(&bars[kQuadS0 + k], kCgPerPart);
        }
        for (int k = 0; k < 4; ++k) {
            mbar_init(&bars[kQuadM0 + k], 1);
        }
        for (int w = 0; w < kSoftmaxWarps; ++w) {
            for (int c = 0; c < 2; ++c) {
                mbar_init(&bars[kXSFull0 + c * kSoftmaxWarps + w], 1);
                mbar_init(&bars[kXPFull0 + c * kSoftmaxWarps + w], 1);
            }
            mbar_init(&bars[kXSEmpty0 + w], 1);
            mbar_init(&bars[kXPEmpty0 + w], 1);
        }
        sm->abort_flag = 0;
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
    const bool tracing = kTrace && a.trace != nullptr && (a.trace_cap >> 24) == 254u &&
                         2 + 2 * gridDim.x + 2048 <= (a.trace_cap & 0xffffffu);
    unsigned long long t_start = 0;
    if (tracing && threadIdx.x == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    }
    unsigned long long *tl = tracing && blockIdx.x < 2 ? a.trace + 2 + 2 * gridDim.x + 1024 * blockIdx.x : nullptr;
    auto mark = [&](uint32_t tile, int ev) {
        if (kTrace && tl != nullptr && tile < 64) {
            tl[16 * tile + ev] = (unsigned long long)clock64();
        }
    };
    const int item_begin = a.plan.group_begin[grp], item_end = a.plan.group_begin[grp + 1];

    // bounded waits; `cluster` = the barrier's phase completes with data published by the peer CTA
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
                // the rope dims of the query block of this range (the latent dims go to tensor memory by the other warps)
                if (!wait(kQEmpty, (i & 1) ^ 1u, false)) {
                    alive = false;
                } else {
                    mbar_expect_tx(&bars[kQFull], kQRopeBytes);
                    tma_load_3d(qr_smem, &qhmap, &bars[kQFull], rope_x, head0, item.seq);
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
            constexpr uint32_t idesc_qk = instr_desc_ab(1, 0, 0, kPartTok, kHeads);  // B = a part of a K tile, K-major
            constexpr uint32_t idesc_pv = instr_desc_ab(1, 0, 1, 256, kHeads);    // B = V, MN-major, N = 256 dims
            const uint32_t st_addr = smem_u32(st_smem);
            const uint64_t dqr = smem_desc_sw64(smem_u32(qr_smem), 16, 512);
            uint32_t g = 0;
            bool alive = true;
            for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
                const PaItem item = a.plan.items[it];
                const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
                if (!wait(kQFull, i & 1, false) || !wait(kQTmem, i & 1, false)) {
                    break;
                }
                // S = Q . K^T of one part of tile gg.  Each part of S has one buffer: the softmax warps are done with the
                // previous tile's (they have delivered its P), and P.V of that part runs before this in issue order
                auto qk = [&](uint32_t gg, int h, bool last) -> bool {
                    const int stg = gg & 1;
                    const uint32_t ph = (gg >> 1) & 1;
                    const uint32_t kb = st_addr + stg * kStageBytes + h * kPartTok * 128;   // the part's rows of every atom
                    const uint64_t db0 = smem_desc(kb, 16, 1024);
                    const uint32_t ds = tmem_base + kSCol + kPartTok * h;
                    if (h == 0) {
                        mark(gg, 2);
                    }
#pragma unroll
                    for (int at = 0; at <= kFullAtoms; ++at) {
                        // atom by atom as the atoms land (the later parts find them there)
                        if (h == 0 && !wait(kStFull0 + 5 * stg + at, ph, false)) {
                            return false;
                        }
                        tc_fence_after();
                        if (at < kFullAtoms) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
                                // 16 dims of Q = 8 TMEM columns (two bf16 per column)
                                tc_mma_ts(ds, tmem_base + kQCol + at * 32 + ks * 8, db0 + ((at * kAtomBytes + ks * 32) >> 4), idesc_qk,
                                          (at | ks) != 0);
                            }
                        } else {
                            // the 32 rope dims, both operands from shared memory: rows of 64 bytes, 64-byte swizzle
                            const uint64_t dkr = smem_desc_sw64(st_addr + stg * kStageBytes + kFullAtoms * kAtomBytes + h * kPartTok * 64, 16, 512);
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                tc_mma(ds, dqr + ((ks * 32) >> 4), dkr + ((ks * 32) >> 4), idesc_qk, true);
                            }
                        }
                    }
                    tc_commit(&bars[kSFull0 + h]);
                    if (h == 0) {
                        mark(gg, 1);   // (overwrites the producer's mark) first half issued
                    }
                    if (last && h == kParts - 1) {
                        tc_commit(&bars[kQEmpty]); // the query block of this range is no longer needed
                    }
                    if (h == kParts - 1) {
                        mark(gg, 3);
                    }
                    return true;
                };
                // O += P . V of one part, once P of all 128 heads for its tokens is in tensor memory
                auto pv = [&](uint32_t gg, int h, bool first) -> bool {
                    if (!wait(kPFull0 + h, gg & 1, false)) {
                        return false;
                    }
                    // the first P.V of a range overwrites O: the previous range's read-out must be over
                    if (first && h == 0 && !wait(kOFree, (i & 1) ^ 1u, false)) {
                        return false;
                    }
                    if (h == 0) {
                        mark(gg, 6);
                    }
                    tc_fence_after();
                    const int stg = gg & 1;
                    // V: 64-dim atoms kAtomBytes apart along N, 8-token groups 1024 B apart; 16 tokens of P = 8 TMEM columns
                    const uint64_t dv0 = smem_desc(st_addr + stg * kStageBytes + h * kPartTok * 128, kAtomBytes, 1024);
#pragma unroll
                    for (int ks = 0; ks < kPartTok / 16; ++ks) {
                        tc_mma_ts(tmem_base + kOCol, tmem_base + kSCol + kPartTok * h + ks * 8, dv0 + ((ks * 2048) >> 4), idesc_pv,
                                  !(first && h == 0) || ks != 0);
                    }
                    if (h == kParts - 1) {
                        tc_commit(&bars[kStEmpty0 + stg]);
                        tc_commit(&bars[kPvDone]);
                        mark(gg, 7);
                    }
                    return true;
                };
#pragma unroll
                for (int h = 0; h < kParts; ++h) {
                    alive = alive && qk(g, h, n_tiles == 1);
                }
                for (int t = 0; t < n_tiles && alive; ++t, ++g) {
                    const bool more = t + 1 < n_tiles, last = t + 2 == n_tiles;
#pragma unroll
                    for (int h = 0; h < kParts; ++h) {
                        alive = alive && pv(g, h, t == 0) && (!more || qk(g + 1, h, last));
                    }
                }
                if (!alive) {
                    *abort_flag = 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ warps 0..15: one head (TMEM lane) and 32 of a
        // tile's tokens per thread
        const int q4 = warp & 3;                                       // TMEM lane quarter this warp may access
        const int cg = warp >> 2;                                      // which 32 tokens of a tile
        const int part = cg / kCgPerPart;                              // which part of the tile: it has its own S, P and barriers
        const int head = q4 * 32 + lane;                               // row of S, P and O
        const bool own = (uint32_t)(q4 >> 1) == rank;                  // this CTA computes the softmax of this quarter's heads
        const int hidx = (q4 & 1) * 32 + lane;                         // index among the 64 heads of their owner
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        // partial scores: [token / 4][head][4 floats], P: [token / 8][head][8 bf16]: a warp's 16-byte accesses are 512
        // contiguous bytes
        const uint32_t xs_off = (uint32_t)(8 * cg) * (kOwn * 16) + (uint32_t)hidx * 16;
        const uint32_t xp_off = (uint32_t)(4 * cg) * (kOwn * 16) + (uint32_t)hidx * 16;
        const uint32_t peer_recv_s = map_to_cta(smem_u32(recv_s), peer) + xs_off;
        const uint32_t peer_recv_p = map_to_cta(smem_u32(recv_p), peer) + xp_off;
        const uint32_t peer_xsfull = peer_bar(kXSFull0 + warp), peer_xpfull = peer_bar(kXPFull0 + warp);
        const uint32_t peer_xsfull2 = peer_bar(kXSFull0 + kSoftmaxWarps + warp), peer_xpfull2 = peer_bar(kXPFull0 + kSoftmaxWarps + warp);
        const bool split_cache = a.k_rope != nullptr;
        const int q_row = split_cache ? kDv : kDk;                     // elements per query row
        uint32_t g = 0;
        bool alive = true;
        // This CTA's latent dims of the query block of range i2 (item it2) -> tensor memory: 64 dims (32 columns) per thread.
        // Called for the first range at once, and for every other one BEFORE the read-out of the range in front of it,
        // so that the MMA thread can start on the new range while the warps here are busy with the old one's output.
        auto store_q = [&](int it2, int i2) -> bool {
            const int seq = a.plan.items[it2].seq;
            uint32_t qv[32];
            if (head < nh) {
                const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const T *>(a.q) + ((int64_t)seq * a.num_heads + head0 + head) * q_row +
                                                                   256 * (int)rank + 64 * cg);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint4 v = __ldg(src + k);
                    qv[4 * k] = v.x;
                    qv[4 * k + 1] = v.y;
                    qv[4 * k + 2] = v.z;
                    qv[4 * k + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    qv[k] = 0u;
                }
            }
            // the previous range's Q.K^T must be done with Q
            if (!wait(kQEmpty, (i2 & 1) ^ 1u, false)) {
                return false;
            }
            tc_fence_after();
            tmem_st32(tmem_base + lane_base + kQCol + 32 * cg, qv);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars[kQTmem]);
            }
            return true;
        };
        for (int it = item_begin, i = 0; it < item_end && alive; ++it, ++i) {
            const PaItem item = a.plan.items[it];
            const int n_tiles = (item.tok_end - item.tok_begin + kTile - 1) / kTile;
            if (i == 0 && !store_q(it, 0)) {
                alive = false;
                break;
            }
            float lsum = 0.f, mref = 0.f;
            float *mref_s = sm->mref[i & 1];
            for (int t = 0; t < n_tiles && alive; ++t, ++g) {
                const int valid = min(kTile, item.tok_end - (item.tok_begin + t * kTile));
                if (!wait(kSFull0 + part, g & 1, false)) {
                    alive = false;
                    break;
                }
                if (threadIdx.x == 0) {
                    mark(g, 4);
                }
                tc_fence_after();
                uint32_t sv[32];
                tmem_ld32(tmem_base + lane_base + kSCol + 32 * cg, sv);
                tmem_wait_ld();
                if (threadIdx.x == 0) {
                    mark(g, 8);
                }
                tc_fence_before();
                __syncwarp();
                // P goes over S: nothing of it may be written before the warps of this quarter and part have read their S
                if (lane == 0) {
                    mbar_arrive(&bars[kQuadS0 + kParts * q4 + part]);
                }
                // rows of V past the end of the range may hold anything: clear them (0 * NaN != 0); the K rows only feed the
                // scores of those tokens, which get probability 0 below
                if (valid < kTile) {
                    uint8_t *stg = st_smem + (g & 1) * kStageBytes;
                    // the threads of this part: its rows of the four atoms
                    const int idx = ((cg % kCgPerPart) * 4 + q4) * 32 + lane;
                    const int row = kPartTok * part + (idx % kPartTok), at = idx / kPartTok;
                    if (row >= valid) {
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch) {
                            *reinterpret_cast<uint4 *>(stg + at * kAtomBytes + row * 128 + (ch << 4)) = make_uint4(0, 0, 0, 0);
                        }
                    }
                    fence_proxy_async();
                }
                uint32_t pk[16];
                if (!own) {
                    // ---- the peer's heads: partial scores into its receive buffer (the stores count their bytes on the
                    // peer's barriers, one per 16 tokens so that it can start on the first while the rest is under way),
                    // then its P for these lanes
                    if (lane == 0) {
                        mbar_expect_tx(&bars[kXPFull0 + warp], 32 * 2 * 16);
                        mbar_expect_tx(&bars[kXPFull0 + kSoftmaxWarps + warp], 32 * 2 * 16);
                    }
                    if (!wait(kXSEmpty0 + warp, (g & 1) ^ 1u, false)) {
                        alive = false;
                        break;
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        st_async_v4(peer_recv_s + k * (kOwn * 16), sv[4 * k], sv[4 * k + 1], sv[4 * k + 2], sv[4 * k + 3],
                                    k < 4 ? peer_xsfull : peer_xsfull2);
                    }
                    if (threadIdx.x == 0) {
                        mark(g, 9);
                    }
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        if (!wait(kXPFull0 + c * kSoftmaxWarps + warp, g & 1, true)) {
                            alive = false;
                            break;
                        }
#pragma unroll
                        for (int k = 2 * c; k < 2 * c + 2; ++k) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(recv_p + xp_off + k * (kOwn * 16));
                            pk[4 * k] = v.x;
                            pk[4 * k + 1] = v.y;
                            pk[4 * k + 2] = v.z;
                            pk[4 * k + 3] = v.w;
                        }
                    }
                    if (!alive) {
                        break;
                    }
                    if (threadIdx.x == 0) {
                        mark(g, 10);
                    }
                } else {
                    // ---- this CTA's heads: add the peer's partial, scale, reference, exponentials; 16 tokens at a time, and
                    // each 16 tokens of P to the peer (for these lanes of its tensor memory) as soon as they exist
                    if (lane == 0) {
                        mbar_expect_tx(&bars[kXSFull0 + warp], 32 * 4 * 16);
                        mbar_expect_tx(&bars[kXSFull0 + kSoftmaxWarps + warp], 32 * 4 * 16);
                    }
                    const int tok_first = 32 * cg;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        if (!wait(kXSFull0 + c * kSoftmaxWarps + warp, g & 1, true)) {
                            alive = false;
                            break;
                        }
                        if (threadIdx.x == 0 && c == 0) {
                            mark(g, 9);
                        }
                        float s[16];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float4 r = *reinterpret_cast<const float4 *>(recv_s + xs_off + (4 * c + k) * (kOwn * 16));
                            s[4 * k] = __uint_as_float(sv[16 * c + 4 * k]) + r.x;
                            s[4 * k + 1] = __uint_as_float(sv[16 * c + 4 * k + 1]) + r.y;
                            s[4 * k + 2] = __uint_as_float(sv[16 * c + 4 * k + 2]) + r.z;
                            s[4 * k + 3] = __uint_as_float(sv[16 * c + 4 * k + 3]) + r.w;
                        }
                        if (t == 0 && c == 0) {
                            // the reference of a head: the score of the range's first token, held by the warp of tokens 0..31
                            if (cg == 0) {
                                mref_s[hidx] = s[0] * a.scale_log2;
                                __syncwarp();
                                if (lane == 0) {
                                    mbar_arrive(&bars[kQuadM0 + q4]);
                                }
                            }
                            if (!wait(kQuadM0 + q4, i & 1, false)) {
                                alive = false;
                                break;
                            }
                            mref = mref_s[hidx];
                        }
                        if (tok_first + 16 * c + 16 <= valid) {
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const float p0 = fast_exp2(fminf(fmaf(s[2 * k], a.scale_log2, -mref), kMaxExponent));
                                const float p1 = fast_exp2(fminf(fmaf(s[2 * k + 1], a.scale_log2, -mref), kMaxExponent));
                                pk[8 * c + k] = Elem<T>::pack2(p0, p1);
                                const float2 pr = Elem<T>::unpack2(pk[8 * c + k]);   // the row sum of P as P.V sees it
                                lsum += pr.x + pr.y;
                            }
                        } else {
                            // the ragged end of a range: tokens past it get probability 0 whatever their scores are
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                float p0 = fast_exp2(fminf(fmaf(s[2 * k], a.scale_log2, -mref), kMaxExponent));
                                float p1 = fast_exp2(fminf(fmaf(s[2 * k + 1], a.scale_log2, -mref), kMaxExponent));
                                if (tok_first + 16 * c + 2 * k >= valid) {
                                    p0 = 0.f;
                                }
                                if (tok_first + 16 * c + 2 * k + 1 >= valid) {
                                    p1 = 0.f;
                                }
                                pk[8 * c + k] = Elem<T>::pack2(p0, p1);
                                const float2 pr = Elem<T>::unpack2(pk[8 * c + k]);
                                lsum += pr.x + pr.y;
                            }
                        }
                        if (c == 0) {
                            // the peer must have taken the previous tile's P out of its receive buffer
                            if (!wait(kXPEmpty0 + warp, (g & 1) ^ 1u, false)) {
                                alive = false;
                                break;
                            }
                        } else {
                            // what was received has been consumed (the arithmetic above depends on it): the peer may send the
                            // next tile's
                            __syncwarp();
                            if (lane == 0) {
                                mbar_arrive_cluster_relaxed(peer_bar(kXSEmpty0 + warp));
                            }
                        }
#pragma unroll
                        for (int k = 2 * c; k < 2 * c + 2; ++k) {
                            st_async_v4(peer_recv_p + k * (kOwn * 16), pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3],
                                        c == 0 ? peer_xpfull : peer_xpfull2);
                        }
                    }
                    if (!alive) {
                        break;
                    }
                    if (threadIdx.x == 0) {
                        mark(g, 11);
                    }
                }
                // ---- P into this thread's lane of tensor memory, over the first half of S
                if (!wait(kQuadS0 + kParts * q4 + part, g & 1, false)) {
                    alive = false;
                    break;
                }
                if (threadIdx.x == 0) {
                    mark(g, 12);
                }
                tc_fence_after();
                tmem_st16(tmem_base + lane_base + kSCol + kPartTok * part + 16 * (cg % kCgPerPart), pk);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kPFull0 + part]);
                    if (!own) {
                        mbar_arrive_cluster_relaxed(peer_bar(kXPEmpty0 + warp));   // the received P has been read
                    }
                }
                if (threadIdx.x == 0) {
                    mark(g, 5);
                }
            }
            if (!alive) {
                break;
            }
            // ---- end of the token range: row sums -> 1 / l in both CTAs, then O / l -> output row or partial
            if (threadIdx.x == 0) {
                mark(g - 1, 15);
            }
            if (it + 1 < item_end && !store_q(it + 1, i + 1)) {
                alive = false;
                break;
            }
            if (threadIdx.x == 0) {
                mark(g - 1, 14);
            }
            float *linv = sm->linv[i & 1];
            if (own) {
                sm->wsum[i & 1][cg][hidx] = lsum;
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[kWsum]);
                }
                if (cg == 0) {
                    if (!wait(kWsum, i & 1, false)) {
                        alive = false;
                        break;
                    }
                    const float l = sm->wsum[i & 1][0][hidx] + sm->wsum[i & 1][1][hidx] + sm->wsum[i & 1][2][hidx] + sm->wsum[i & 1][3][hidx];
                    const float inv = 1.f / l;
                    linv[kOwn * rank + hidx] = inv;
                    sm->lfull[i & 1][hidx] = l;
                    st_cluster_f32(map_to_cta(smem_u32(&linv[kOwn * rank + hidx]), peer), inv);
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
            if (threadIdx.x == 0) {
                mark(g - 1, 9);       // (overwrites the tile's own mark) every P.V of the range has completed
            }
            tc_fence_after();
            if (own && cg == 0 && head < nh) {
                const float lse2 = mref_s[hidx] + log2f(sm->lfull[i & 1][hidx]);
                if (item.slot >= 0) {
                    a.plan.part_lse[(int64_t)item.slot * a.num_heads + head0 + head] = lse2;
                } else if (a.lse_out != nullptr) {
                    // whole sequence in this range: its log-sum-exp, natural log
                    static_cast<T *>(a.lse_out)[(int64_t)item.seq * a.num_heads + head0 + head] = Elem<T>::from_float(lse2 * 0.6931471805599453f);
                }
            }
            {
                // this thread's head, 64 of this CTA's 256 dims: contiguous in the output row
                const float inv = linv[head];
                const int dim0 = 256 * (int)rank + 64 * cg;
                float *po = item.slot >= 0 ? a.plan.part_o + ((int64_t)item.slot * a.num_heads + head0 + head) * kDv + dim0 : nullptr;
                T *oo = static_cast<T *>(a.out) + ((int64_t)item.seq * a.num_heads + head0 + head) * kDv + dim0;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_base + kOCol + 64 * cg + 32 * hf, r);
                    tmem_wait_ld();
                    if (head < nh) {
                        // whole 32-byte sectors per store (the workspace is 256-byte aligned, output rows 32-byte aligned)
                        if (po != nullptr) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                uint32_t w[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    w[j] = __float_as_uint(__uint_as_float(r[8 * k + j]) * inv);
                                }
                                st_global_v8(po + 32 * hf + 8 * k, w);
                            }
                        } else {
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                uint32_t w[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    w[j] = Elem<T>::pack2(__uint_as_float(r[16 * k + 2 * j]) * inv, __uint_as_float(r[16 * k + 2 * j + 1]) * inv);
                                }
                                st_global_v8(oo + 32 * hf + 16 * k, w);
                            }
                        }
                    }
                }
            }
            // the next range's first P.V overwrites O: tell the issuer the read-out is over
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars[kOFree]);
            }
            if (threadIdx.x == 0) {
                mark(g - 1, 10);      // (overwrites the tile's own mark) read-out over
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

bool pa_mla_pair_supported(int dk, int dv, int v_row_dim, int rope_dim, int block_size, int kv_heads, int q_dtype, int kv_dtype)
{
    const bool rows_ok = (rope_dim == 0 && v_row_dim == kDk) || (rope_dim == kDk - kDv && v_row_dim == kDv);
    return dk == kDk && dv == kDv && rows_ok && kv_heads == 1 && block_size >= kBox && block_size % kBox == 0 &&
           block_size <= 256 && q_dtype == kBf16 && kv_dtype == kBf16;
}

// CTA pairs that can be resident at once on the current device (pairs are placed within a GPC, so this may be less
// than SMs / 2); 0 if the query fails.  Cached per device.
int pa_mla_pair_max_pairs()
{
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return 0;
    }
    if (cached[dev] == 0) {
        if (cudaFuncSetAttribute(pa_mla_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
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
        if (cudaOccupancyMaxActiveClusters(&n, pa_mla_pair_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return 0;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

cudaError_t launch_pa_mla_pair(const PaArgs &args, int num_blocks, cudaStream_t stream)
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
    // rope part of the query [tokens][num_heads][row]; box = 32 elements x 128 heads of one token (rows past num_heads
    // read as zero)
    auto encode_q = [&](CUtensorMap *map, const void *base, int row) {
        cuuint64_t dims[3] = {(cuuint64_t)row, (cuuint64_t)args.num_heads, (cuuint64_t)args.batch};
        cuuint64_t strides[2] = {(cuuint64_t)row * 2, (cuuint64_t)args.num_heads * row * 2};
        cuuint32_t box[3] = {32, kHeads, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        return fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const bool split = args.k_rope != nullptr;
    CUtensorMap km, rm, qrm;
    if (!encode_cache(&km, args.k_cache, split ? kDv : kDk, false) ||
        !encode_cache(&rm, split ? args.k_rope : args.k_cache, split ? kDk - kDv : kDk, true) ||
        !encode_q(&qrm, split ? args.q_rope : args.q, split ? kDk - kDv : kDk)) {
        return cudaErrorInvalidValue;
    }
    const bool traced = args.trace != nullptr;
    auto kern = traced ? pa_mla_pair_kernel<true> : pa_mla_pair_kernel<false>;
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
    return cudaLaunchKernelEx(&cfg, kern, km, rm, qrm, args);
}

} // namespace atb_b200
