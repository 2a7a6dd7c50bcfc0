#include "pa_planner.h"
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include "kernels.h"

namespace atb_b200 {
namespace {
constexpr int kErrInvalidParam = 1;     // atb::ERROR_INVALID_PARAM
constexpr int kErrInvalidTensorDim = 8; // atb::ERROR_INVALID_TENSOR_DIM

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
} // namespace

void HostPlan::write_blob(uint8_t *dst) const
{
    std::memset(dst, 0, blob_bytes);
    std::memcpy(dst + off_group_begin, group_begin.data(), group_begin.size() * sizeof(int32_t));
    if (!items.empty()) {
        std::memcpy(dst + off_items, items.data(), items.size() * sizeof(PaItem));
    }
    std::memcpy(dst + off_part_base, seq_part_base.data(), seq_part_base.size() * sizeof(int32_t));
    std::memcpy(dst + off_nparts, seq_nparts.data(), seq_nparts.size() * sizeof(int32_t));
    if (!combine_seqs.empty()) {
        std::memcpy(dst + off_combine, combine_seqs.data(), combine_seqs.size() * sizeof(int32_t));
    }
    if (!seq_lens.empty()) {
        std::memcpy(dst + off_lens, seq_lens.data(), seq_lens.size() * sizeof(int32_t));
    }
    if (!bt_rows.empty()) {
        std::memcpy(dst + off_rows, bt_rows.data(), bt_rows.size() * sizeof(int32_t));
        std::memcpy(dst + off_rows + bt_rows.size() * sizeof(int32_t), mask_rows.data(), mask_rows.size() * sizeof(int32_t));
    }
}

int plan_paged_attention(const atb_b200_pa_desc &d, const int32_t *context_lens, int sm_count, HostPlan *p)
{
    if (p == nullptr || (context_lens == nullptr && d.batch > 0) || sm_count <= 0) {
        return kErrInvalidParam;
    }
    if (d.batch < 0 || d.num_heads <= 0 || d.kv_heads <= 0 || d.num_heads % d.kv_heads != 0 || d.head_dim_k <= 0 ||
        d.head_dim_v <= 0 || d.v_row_dim < d.head_dim_v || d.block_size <= 0 || d.num_blocks <= 0 ||
        d.max_blocks_per_seq <= 0) {
        return kErrInvalidParam;
    }
    if (d.q_per_seq < 0 || (d.q_per_seq > 1 && (d.num_heads % d.q_per_seq != 0 ||
                                                (d.num_heads / d.q_per_seq) % d.kv_heads != 0))) {
        return kErrInvalidParam;
    }
    const int group = d.num_heads / d.kv_heads;
    if (d.qkv_quant != 0) {
        // int8 query and cache: the integer tensor-core variant of the tiled kernel only, plain scores
        if ((d.qkv_quant != ATB_B200_QUANT_ONLINE && d.qkv_quant != ATB_B200_QUANT_OFFLINE) || d.q_dtype != kInt8 ||
            d.kv_dtype != kInt8 || d.score_mods != 0 || d.rope_dim != 0 || d.kv_layout != ATB_B200_KV_BSND ||
            d.q_per_seq > 1) {
            return kErrInvalidParam;
        }
        if (!pa_tma_mma_q8_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.block_size, group, d.out_dtype) ||
            (d.kernel != ATB_B200_KERNEL_AUTO && d.kernel != ATB_B200_KERNEL_TMA_MMA)) {
            return kErrInvalidTensorDim;
        }
    } else if (d.q_dtype == kInt8) {
        return kErrInvalidParam;
    }
    const bool tma_ok = d.qkv_quant != 0 || pa_tma_mma_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.block_size, group, d.q_dtype,
                                             d.kv_dtype) ||
                        pa_tma_mma_i8_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.block_size, group, d.q_dtype,
                                                d.kv_dtype);
    const bool gen_ok = pa_generic_supported(d.head_dim_k, d.head_dim_v, d.q_dtype, d.kv_dtype);
    const bool mla_ok = pa_mla_tc5_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.rope_dim, d.block_size, d.kv_heads, d.q_dtype,
                                             d.kv_dtype);
    if (d.rope_dim != 0 && !mla_ok) {
        return kErrInvalidTensorDim; // the split latent / rope cache exists for the tcgen05 MLA kernel only
    }
    int kernel = d.kernel;
    if (d.rope_dim != 0) {
        if (kernel != ATB_B200_KERNEL_AUTO && kernel != ATB_B200_KERNEL_MLA_TC5) {
            return kErrInvalidTensorDim;
        }
        kernel = ATB_B200_KERNEL_MLA_TC5;
    }
    if (d.score_mods != 0) {
        // masks, logN scaling and per-token rows live in the fp16 / bf16 D = 128 kernel and in the CUDA-core kernel;
        // the MLA kernel takes per-token rows and a mask without a head stride, no logN
        if ((d.score_mods & ~(ATB_B200_SCORE_MASK | ATB_B200_SCORE_LOGN | ATB_B200_SCORE_ROWS | ATB_B200_SCORE_CAUSAL)) != 0 ||
            ((d.score_mods & ATB_B200_SCORE_CAUSAL) != 0 && d.q_per_seq <= 1)) {
            return kErrInvalidParam;
        }
        const bool tma_plain = tma_ok && d.kv_dtype != kInt8;
        const bool mla_mods = mla_ok && (d.score_mods & ATB_B200_SCORE_LOGN) == 0;
        if (kernel == ATB_B200_KERNEL_AUTO) {
            kernel = tma_plain ? ATB_B200_KERNEL_TMA_MMA : (mla_mods ? ATB_B200_KERNEL_MLA_TC5 : ATB_B200_KERNEL_GENERIC);
        }
        if ((kernel == ATB_B200_KERNEL_MLA_TC5 && !mla_mods) || (kernel == ATB_B200_KERNEL_TMA_MMA && !tma_plain)) {
            return kErrInvalidTensorDim;
        }
    }
    if (d.kv_layout != ATB_B200_KV_BSND) {
        // heads-major cache blocks: fp16 / bf16 caches in the D = 128 kernel and in the CUDA-core kernel
        if (d.kv_layout != ATB_B200_KV_BNSD || d.rope_dim != 0 || d.kv_dtype == kInt8 || d.v_row_dim != d.head_dim_v) {
            return kErrInvalidParam;
        }
        if (kernel == ATB_B200_KERNEL_AUTO) {
            kernel = tma_ok ? ATB_B200_KERNEL_TMA_MMA : ATB_B200_KERNEL_GENERIC;
        }
        if (kernel == ATB_B200_KERNEL_MLA_TC5) {
            return kErrInvalidTensorDim;
        }
    }
    if (d.q_per_seq > 1) {
        // (token, head) pairs as the columns of one CTA of the fp16 / bf16 D = 128 kernel (at most 8 pairs per kv head,
        // which is what its head limit already says about num_heads / kv_heads), or as the rows of the MLA kernel
        const bool tma_pairs = tma_ok && d.kv_dtype != kInt8 && d.rope_dim == 0 && group <= 8;
        const int want = tma_pairs ? ATB_B200_KERNEL_TMA_MMA : ATB_B200_KERNEL_MLA_TC5;
        if ((!tma_pairs && !mla_ok) || (d.score_mods & ATB_B200_SCORE_LOGN) != 0 ||
            (kernel != ATB_B200_KERNEL_AUTO && kernel != want)) {
            return kErrInvalidTensorDim;
        }
        kernel = want;
    }
    if (kernel == ATB_B200_KERNEL_AUTO) {
        kernel = tma_ok ? ATB_B200_KERNEL_TMA_MMA : (mla_ok ? ATB_B200_KERNEL_MLA_TC5 : ATB_B200_KERNEL_GENERIC);
    }
    if ((kernel == ATB_B200_KERNEL_TMA_MMA && !tma_ok) || (kernel == ATB_B200_KERNEL_GENERIC && !gen_ok) ||
        (kernel == ATB_B200_KERNEL_MLA_TC5 && !mla_ok) ||
        (kernel != ATB_B200_KERNEL_TMA_MMA && kernel != ATB_B200_KERNEL_GENERIC && kernel != ATB_B200_KERNEL_MLA_TC5)) {
        return kErrInvalidTensorDim;
    }

    p->desc = d;
    p->kernel = kernel;
    p->sm_count = sm_count;
    p->mla_pair = false;
    if (kernel == ATB_B200_KERNEL_TMA_MMA) {
        p->heads_per_cta = 8;
        p->chunks_per_kvh = (group + 7) / 8; // more than 8 heads per kv head: several columns over the same K/V tiles
        p->ctas_per_sm = d.head_dim_k > 128 ? 1 : 2; // the 3-stage ring of 256-wide rows takes 192 KB of shared memory
    } else if (kernel == ATB_B200_KERNEL_MLA_TC5) {
        p->heads_per_cta = 64;
        p->chunks_per_kvh = (group + 63) / 64;
        p->ctas_per_sm = 1;
        // opt-in (ATB_B200_MLA_PAIR=1), bf16 without a mask, the causal rule or fused query tokens: CTA pairs that split the
        // dims, 128 heads per pair
        const char *env = std::getenv("ATB_B200_MLA_PAIR");
        if (env != nullptr && env[0] == '1' && d.q_per_seq <= 1 && (d.score_mods & (ATB_B200_SCORE_MASK | ATB_B200_SCORE_CAUSAL)) == 0 &&
            pa_mla_pair_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.rope_dim, d.block_size, d.kv_heads, d.q_dtype, d.kv_dtype)) {
            p->mla_pair = true;
            p->heads_per_cta = 128;   // per pair
            p->chunks_per_kvh = (group + 127) / 128;
        }
    } else {
        p->heads_per_cta = pa_generic_heads_per_cta(d.head_dim_k, d.head_dim_v);
        p->chunks_per_kvh = (group + p->heads_per_cta - 1) / p->heads_per_cta;
        p->ctas_per_sm = 4;
    }
    p->cols = d.kv_heads * p->chunks_per_kvh;

    // ---- balanced cut of the global tile sequence into CTA groups
    const int64_t max_ctx = (int64_t)d.max_blocks_per_seq * d.block_size;
    int64_t total_tiles = 0, longest = 0;
    for (int b = 0; b < d.batch; ++b) {
        const int64_t ctx = context_lens[b];
        if (ctx < 0 || ctx > max_ctx) {
            return kErrInvalidParam; // a length the block table cannot describe
        }
        total_tiles += (ctx + kTileTokens - 1) / kTileTokens;
        longest = std::max(longest, ctx);
    }
    p->max_context = longest;
    const int slots = sm_count * p->ctas_per_sm;
    int64_t n_groups = std::max<int64_t>(1, slots / p->cols);
    if (p->mla_pair) {
        // one CTA pair per (group, column), all pairs resident at once
        const int pairs = p->cta_pairs > 0 ? p->cta_pairs : sm_count / 2;
        n_groups = std::max<int64_t>(1, pairs / p->cols);
    }
    if (n_groups < 4) {
        n_groups = 4; // many columns: still cut long sequences a little for balance
    }
    n_groups = std::min<int64_t>(n_groups, std::max<int64_t>(total_tiles, 1));

    // Group j owns the global tile positions [cut[j], cut[j+1]).  The ideal cut j*total/n is moved
    // onto a sequence boundary when that is at most one tile away (a one-tile fragment costs about
    // as much in per-range overhead as it saves in balance); cuts are absolute positions, so the
    // rounding never accumulates and every group stays within ~one tile of the mean.
    std::vector<int64_t> seq_start(d.batch + 1, 0);
    for (int b = 0; b < d.batch; ++b) {
        seq_start[b + 1] = seq_start[b] + ((int64_t)context_lens[b] + kTileTokens - 1) / kTileTokens;
    }
    const int64_t snap = (total_tiles / n_groups >= 8) ? 1 : 0;
    std::vector<int64_t> cut(n_groups + 1, 0);
    cut[n_groups] = total_tiles;
    {
        int b = 0;
        for (int64_t j = 1; j < n_groups; ++j) {
            int64_t pos = (j * total_tiles) / n_groups;
            while (b < d.batch && seq_start[b + 1] <= pos) {
                ++b;
            }
            if (b < d.batch && pos > seq_start[b]) {
                if (pos - seq_start[b] <= snap) {
                    pos = seq_start[b];
                } else if (seq_start[b + 1] - pos <= snap) {
                    pos = seq_start[b + 1];
                }
            }
            cut[j] = std::max(pos, cut[j - 1]);
        }
    }
    if (kernel == ATB_B200_KERNEL_MLA_TC5 && total_tiles > 0) {
        // The MLA kernel pays for every token range it starts (store the Q block into tensor memory, refill the
        // pipeline, drain it, write 64 x 512 floats) about as much as for kItemTiles tiles: measured 14.5 us per
        // range against 2.4 us per tile on a B200.  A group that straddles a sequence boundary holds two ranges, and
        // with equal tile counts those groups end last.  So balance cost = tiles + kItemTiles x ranges instead: the
        // smallest cap T for which a greedy left-to-right packing needs no more than n_groups groups.
        int64_t kItemTiles = 6;
        if (const char *env = std::getenv("ATB_B200_MLA_RANGE_TILES")) { // tuning knob: the weight of a range start
            const long v = std::strtol(env, nullptr, 10);
            if (v >= 0 && v <= 64) {
                kItemTiles = v;
            }
        }
        auto pack = [&](int64_t cap, std::vector<int64_t> *cuts) {
            int64_t groups = 1, cost = 0, pos = 0;
            if (cuts != nullptr) {
                cuts->assign(1, 0);
            }
            for (int b = 0; b < d.batch; ++b) {
                int64_t left = seq_start[b + 1] - seq_start[b];
                while (left > 0) {
                    if (cost + kItemTiles + 1 > cap) { // no room for another range of at least one tile
                        ++groups;
                        cost = 0;
                        if (cuts != nullptr) {
                            cuts->push_back(pos);
                        }
                    }
                    const int64_t take = std::min(left, cap - cost - kItemTiles);
                    cost += kItemTiles + take;
                    left -= take;
                    pos += take;
                }
            }
            return groups;
        };
        // one group that holds every range is always feasible: that is the upper end of the search
        int64_t lo = kItemTiles + 1, hi = total_tiles + kItemTiles * (int64_t)d.batch;
        while (lo < hi) {
            const int64_t mid = (lo + hi) / 2;
            if (pack(mid, nullptr) <= n_groups) {
                hi = mid;
            } else {
                lo = mid + 1;
            }
        }
        std::vector<int64_t> cuts;
        pack(lo, &cuts);
        for (int64_t j = 0; j <= n_groups; ++j) {
            cut[j] = j < (int64_t)cuts.size() ? cuts[j] : total_tiles; // unused groups at the end stay empty
        }
    }

    p->items.clear();
    p->group_begin.assign(1, 0);
    p->seq_part_base.assign(d.batch, 0);
    p->seq_nparts.assign(d.batch, 0);
    p->combine_seqs.clear();
    p->n_partials = 0;
    {
        int b = 0;
        for (int64_t j = 0; j < n_groups; ++j) {
            int64_t pos = cut[j];
            const int64_t end = cut[j + 1];
            while (pos < end) {
                while (seq_start[b + 1] <= pos) {
                    ++b;
                }
                const int64_t stop = std::min(end, seq_start[b + 1]);
                PaItem item;
                item.seq = b;
                item.tok_begin = (int32_t)((pos - seq_start[b]) * kTileTokens);
                item.tok_end = (int32_t)std::min<int64_t>(context_lens[b], (stop - seq_start[b]) * kTileTokens);
                item.slot = -1;
                p->items.push_back(item);
                p->seq_nparts[b] += 1;
                pos = stop;
            }
            p->group_begin.push_back((int32_t)p->items.size());
        }
    }
    // items of one sequence are consecutive in the list: number its partial slots
    for (size_t i = 0; i < p->items.size();) {
        const int b = p->items[i].seq;
        const int nparts = p->seq_nparts[b];
        if (nparts > 1) {
            p->seq_part_base[b] = p->n_partials;
            for (int k = 0; k < nparts; ++k) {
                p->items[i + k].slot = p->n_partials + k;
            }
            p->n_partials += nparts;
            p->combine_seqs.push_back(b);
        }
        i += nparts;
    }
    p->n_cta_groups = (int)p->group_begin.size() - 1;

    // ---- workspace layout
    uint64_t off = 0;
    p->off_group_begin = off;
    off = align_up(off + p->group_begin.size() * sizeof(int32_t), 16);
    p->off_items = off;
    off = align_up(off + p->items.size() * sizeof(PaItem), 16);
    p->off_part_base = off;
    off = align_up(off + (uint64_t)d.batch * sizeof(int32_t), 16);
    p->off_nparts = off;
    off = align_up(off + (uint64_t)d.batch * sizeof(int32_t), 16);
    p->off_combine = off;
    off = align_up(off + p->combine_seqs.size() * sizeof(int32_t), 16);
    p->off_status = off; // zeroed by every upload
    p->off_done = off + 4;
    off += 16;
    p->fused_combine = kernel == ATB_B200_KERNEL_TMA_MMA;
    p->off_counters = off;
    if (p->fused_combine && p->n_partials > 0) {
        off = align_up(off + (uint64_t)d.batch * p->cols * sizeof(int32_t), 16);
    }
    if ((d.score_mods & ATB_B200_SCORE_CAUSAL) != 0) {
        p->seq_lens.assign(context_lens, context_lens + d.batch);
        p->off_lens = off;
        off = align_up(off + (uint64_t)d.batch * sizeof(int32_t), 16);
    } else {
        p->seq_lens.clear();
    }
    if ((d.score_mods & ATB_B200_SCORE_ROWS) != 0) {
        // rows set for this batch size stay; otherwise token b reads row b
        if (p->bt_rows.size() != (size_t)d.batch) {
            p->bt_rows.resize(d.batch);
            p->mask_rows.resize(d.batch);
            for (int b = 0; b < d.batch; ++b) {
                p->bt_rows[b] = p->mask_rows[b] = b;
            }
        }
        p->off_rows = off;
        off = align_up(off + 2 * (uint64_t)d.batch * sizeof(int32_t), 16);
    } else {
        p->bt_rows.clear();
        p->mask_rows.clear();
    }
    p->blob_bytes = align_up(off, 256);
    p->off_lse = p->blob_bytes;
    p->off_part_o = align_up(p->off_lse + (uint64_t)p->n_partials * d.num_heads * sizeof(float), 256);
    p->workspace_bytes =
        align_up(p->off_part_o + (uint64_t)p->n_partials * d.num_heads * d.head_dim_v * sizeof(float), 256);
    return 0;
}

} // namespace atb_b200
