// Host planner of the paged-attention launch: kernel choice, balanced split-KV work list,
// workspace layout.  Pure host code (no CUDA calls), so it is unit-testable on a CPU-only machine.
#ifndef ATB_B200_PA_PLANNER_H
#define ATB_B200_PA_PLANNER_H
#include <cstdint>
#include <vector>
#include "../../include/atb_b200.h"
#include "pa_plan.h"

namespace atb_b200 {

struct HostPlan {
    atb_b200_pa_desc desc{};
    int kernel = 0;        // ATB_B200_KERNEL_*
    int cols = 1;          // CTAs per CTA group (kv heads x head chunks)
    int heads_per_cta = 8; // generic kernel: query heads one CTA handles
    int chunks_per_kvh = 1;
    int ctas_per_sm = 2;
    int sm_count = 148;
    int cta_pairs = 0;     // CTA pairs of the split MLA kernel resident at once (0: assume sm_count / 2)
    int n_cta_groups = 0;
    int n_partials = 0;
    int64_t max_context = 0; // longest context of the planned batch (tokens)
    std::vector<PaItem> items;
    std::vector<int32_t> group_begin;   // n_cta_groups + 1
    std::vector<int32_t> seq_part_base; // batch
    std::vector<int32_t> seq_nparts;    // batch
    std::vector<int32_t> combine_seqs;
    std::vector<int32_t> bt_rows, mask_rows; // per query token, ATB_B200_SCORE_ROWS only (else empty)
    std::vector<int32_t> seq_lens;           // context lengths, ATB_B200_SCORE_CAUSAL only (else empty)

    // Byte offsets inside the workspace (all 256-byte aligned).
    uint64_t off_group_begin = 0, off_items = 0, off_part_base = 0, off_nparts = 0, off_combine = 0;
    uint64_t off_done = 0;        // finished-CTA counter (zeroed by every upload)
    uint64_t off_counters = 0;    // arrival counters of the in-kernel merge (zeroed by every upload)
    uint64_t off_lens = 0;        // seq_lens (batch entries), ATB_B200_SCORE_CAUSAL only
    uint64_t off_rows = 0;        // bt_rows then mask_rows (batch entries each), ATB_B200_SCORE_ROWS only
    bool fused_combine = false;   // the attention kernel merges split sequences itself
    bool mla_pair = false;        // MLA on CTA pairs that split the dims, 128 heads per pair (pa_mla_pair.cu); grid = 2 x groups x cols
    uint64_t blob_bytes = 0;      // uploaded per launch
    uint64_t off_status = 0, off_lse = 0, off_part_o = 0;
    uint64_t workspace_bytes = 0;

    // Serialises the lists into `dst` (blob_bytes) in the layout the offsets describe.
    void write_blob(uint8_t *dst) const;
};

// Returns 0 or an atb::ErrorType value.  `sm_count` must be > 0.
// `plan->cta_pairs`, when set beforehand, bounds the grid of the split MLA kernel.
int plan_paged_attention(const atb_b200_pa_desc &desc, const int32_t *context_lens, int sm_count, HostPlan *plan);

} // namespace atb_b200
#endif
