// extern "C" boundary of libatb_b200.so (see include/atb_b200.h).
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include "../../include/atb_b200.h"
#include "kernels.h"
#include "pa_planner.h"

using namespace atb_b200;

namespace {
constexpr int kErrInvalidParam = 1; // atb::ERROR_INVALID_PARAM
constexpr int kErrRtFail = 4;       // atb::ERROR_RT_FAIL
constexpr int kErrOutOfHostMemory = 27;
} // namespace

struct atb_b200_pa_plan {
    HostPlan hp;
    // Pinned staging of the plan blob: a ring of slots, so the host can enqueue several steps ahead
    // of the GPU; a slot is rewritten only after the copy that last read it has completed.
    static constexpr int kStagingRing = 4;
    uint8_t *staging = nullptr; // kStagingRing slots of staging_cap bytes
    size_t staging_cap = 0;
    cudaEvent_t uploaded[kStagingRing] = {};
    bool upload_pending[kStagingRing] = {};
    uint64_t uploads = 0;
    // Prefetch path: plan-owned device copies of the blob, uploaded on a private stream ahead of
    // the launch so that the copy leaves the caller's stream (ring: a slot is refilled only after
    // the kernels that read it have completed).
    static constexpr int kDevRing = 4;
    cudaStream_t copy_stream = nullptr;
    uint8_t *dev_blob = nullptr;
    size_t dev_cap = 0;
    cudaEvent_t dev_uploaded[kDevRing] = {}, dev_consumed[kDevRing] = {};
    bool dev_consumed_pending[kDevRing] = {};
    int prefetched_slot = -1;
    void *prefetch_stream = nullptr; // the stream that was made to wait for the prefetched copy
    uint64_t prefetches = 0;
    const int32_t *last_status_ptr = nullptr;
    // status word of the last launch, read back when the device copy it lived in had to be freed
    int32_t saved_status = 0;
    bool has_saved_status = false;
    unsigned long long *trace = nullptr; // optional device event buffer (probe)
    uint32_t trace_cap = 0;
    // optional timing of the attention kernel: a ring of event pairs, one pair per launch
    static constexpr int kProfRing = 256;
    int profile_every = 0; // 0 = off, n = every n-th launch carries an event pair
    cudaEvent_t ev0[kProfRing] = {}, ev1[kProfRing] = {};
    uint64_t launches = 0;  // launches that recorded an event pair
    uint64_t launch_seq = 0; // all launches since profiling was switched on
    int32_t *status_host = nullptr;
};

extern "C" {

const char *atb_b200_version(void) { return "atb-b200 0.1 (API level of ascend-transformer-boost 8.5.0)"; }

int atb_b200_pa_plan_create(const atb_b200_pa_desc *desc, const int32_t *context_lens_host, atb_b200_pa_plan **plan)
{
    if (desc == nullptr || plan == nullptr) {
        return kErrInvalidParam;
    }
    int sm = desc->sm_count;
    if (sm <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm <= 0) {
            return kErrRtFail;
        }
    }
    atb_b200_pa_plan *p = new (std::nothrow) atb_b200_pa_plan();
    if (p == nullptr) {
        return kErrOutOfHostMemory;
    }
    if (desc->sm_count <= 0 && desc->head_dim_k == 576) {
        p->hp.cta_pairs = pa_mla_pair_max_pairs(); // planned for the current device: how many CTA pairs it can hold
    }
    int rc;
    try {
        rc = plan_paged_attention(*desc, context_lens_host, sm, &p->hp);
    } catch (...) {
        rc = kErrOutOfHostMemory;
    }
    if (rc != 0) {
        delete p;
        return rc;
    }
    *plan = p;
    return ATB_B200_OK;
}

int atb_b200_pa_plan_update(atb_b200_pa_plan *plan, const int32_t *context_lens_host)
{
    if (plan == nullptr) {
        return kErrInvalidParam;
    }
    plan->prefetched_slot = -1; // an upload of the old plan, if any, is simply never used
    try {
        const atb_b200_pa_desc d = plan->hp.desc;
        return plan_paged_attention(d, context_lens_host, plan->hp.sm_count, &plan->hp);
    } catch (...) {
        return kErrOutOfHostMemory;
    }
}

int atb_b200_pa_plan_set_rows(atb_b200_pa_plan *plan, const int32_t *bt_rows, int32_t bt_row_count,
                              const int32_t *mask_rows, int64_t mask_row_count)
{
    if (plan == nullptr || bt_rows == nullptr || (plan->hp.desc.score_mods & ATB_B200_SCORE_ROWS) == 0) {
        return kErrInvalidParam;
    }
    HostPlan &h = plan->hp;
    const bool masked = (h.desc.score_mods & ATB_B200_SCORE_MASK) != 0;
    if (masked && mask_rows == nullptr) {
        return kErrInvalidParam;
    }
    const int batch = h.desc.batch;
    for (int b = 0; b < batch; ++b) {
        if (bt_rows[b] < 0 || bt_rows[b] >= bt_row_count ||
            (masked && (mask_rows[b] < 0 || mask_rows[b] >= mask_row_count))) {
            return kErrInvalidParam;
        }
    }
    if (h.bt_rows.size() != (size_t)batch) {
        return kErrInvalidParam; // planned without the rows: the blob has no room for them
    }
    for (int b = 0; b < batch; ++b) {
        h.bt_rows[b] = bt_rows[b];
        h.mask_rows[b] = masked ? mask_rows[b] : 0;
    }
    plan->prefetched_slot = -1; // an upload made before the rows were set is not used
    return ATB_B200_OK;
}

int atb_b200_pa_plan_get_info(const atb_b200_pa_plan *plan, atb_b200_pa_plan_info *info)
{
    if (plan == nullptr || info == nullptr) {
        return kErrInvalidParam;
    }
    const HostPlan &h = plan->hp;
    info->kernel = h.kernel;
    info->num_ctas = h.n_cta_groups * h.cols * (h.mla_pair ? 2 : 1);
    info->num_items = (int32_t)h.items.size();
    info->num_partials = h.n_partials;
    info->num_combine_seqs = (int32_t)h.combine_seqs.size();
    info->tile_tokens = kTileTokens;
    info->workspace_bytes = h.workspace_bytes;
    info->plan_bytes = h.blob_bytes;
    info->kernels_per_launch = (h.n_partials > 0 && !h.fused_combine) ? 2 : 1;
    info->reserved = 0;
    return ATB_B200_OK;
}

int atb_b200_pa_plan_dump(const atb_b200_pa_plan *plan, int32_t *items, int32_t max_items, int32_t *group_begin,
                          int32_t max_groups)
{
    if (plan == nullptr) {
        return kErrInvalidParam;
    }
    const HostPlan &h = plan->hp;
    if (items != nullptr) {
        if ((size_t)max_items < h.items.size()) {
            return kErrInvalidParam;
        }
        std::memcpy(items, h.items.data(), h.items.size() * sizeof(PaItem));
    }
    if (group_begin != nullptr) {
        if ((size_t)max_groups < h.group_begin.size()) {
            return kErrInvalidParam;
        }
        std::memcpy(group_begin, h.group_begin.data(), h.group_begin.size() * sizeof(int32_t));
    }
    return ATB_B200_OK;
}

void atb_b200_pa_plan_destroy(atb_b200_pa_plan *plan)
{
    if (plan == nullptr) {
        return;
    }
    for (int i = 0; i < atb_b200_pa_plan::kStagingRing; ++i) {
        if (plan->uploaded[i] != nullptr) {
            cudaEventSynchronize(plan->uploaded[i]);
            cudaEventDestroy(plan->uploaded[i]);
        }
    }
    for (int i = 0; i < atb_b200_pa_plan::kProfRing; ++i) {
        if (plan->ev0[i] != nullptr) {
            cudaEventDestroy(plan->ev0[i]);
            cudaEventDestroy(plan->ev1[i]);
        }
    }
    if (plan->staging != nullptr) {
        cudaFreeHost(plan->staging);
    }
    if (plan->copy_stream != nullptr) {
        cudaStreamSynchronize(plan->copy_stream);
        for (int i = 0; i < atb_b200_pa_plan::kDevRing; ++i) {
            if (plan->dev_consumed_pending[i]) {
                cudaEventSynchronize(plan->dev_consumed[i]);
            }
            if (plan->dev_uploaded[i] != nullptr) {
                cudaEventDestroy(plan->dev_uploaded[i]);
                cudaEventDestroy(plan->dev_consumed[i]);
            }
        }
        cudaStreamDestroy(plan->copy_stream);
    }
    if (plan->dev_blob != nullptr) {
        cudaFree(plan->dev_blob);
    }
    if (plan->status_host != nullptr) {
        cudaFreeHost(plan->status_host);
    }
    delete plan;
}

int atb_b200_pa_plan_set_trace(atb_b200_pa_plan *plan, void *device_events, uint32_t capacity)
{
    if (plan == nullptr || (device_events != nullptr && capacity < 2)) {
        return kErrInvalidParam;
    }
    plan->trace = static_cast<unsigned long long *>(device_events);
    plan->trace_cap = device_events != nullptr ? capacity : 0;
    return ATB_B200_OK;
}

int atb_b200_pa_plan_set_profiling(atb_b200_pa_plan *plan, int enable)
{
    if (plan == nullptr) {
        return kErrInvalidParam;
    }
    if (enable && plan->ev0[0] == nullptr) {
        for (int i = 0; i < atb_b200_pa_plan::kProfRing; ++i) {
            if (cudaEventCreate(&plan->ev0[i]) != cudaSuccess || cudaEventCreate(&plan->ev1[i]) != cudaSuccess) {
                return kErrRtFail;
            }
        }
    }
    plan->profile_every = enable > 0 ? enable : 0;
    plan->launches = 0;
    plan->launch_seq = 0;
    return ATB_B200_OK;
}

int atb_b200_pa_plan_kernel_ms(atb_b200_pa_plan *plan, int32_t launches_back, float *ms)
{
    if (plan == nullptr || ms == nullptr || plan->ev0[0] == nullptr || launches_back < 0 ||
        launches_back >= atb_b200_pa_plan::kProfRing || (uint64_t)launches_back >= plan->launches) {
        return kErrInvalidParam;
    }
    const int i = (int)((plan->launches - 1 - (uint64_t)launches_back) % atb_b200_pa_plan::kProfRing);
    if (cudaEventSynchronize(plan->ev1[i]) != cudaSuccess ||
        cudaEventElapsedTime(ms, plan->ev0[i], plan->ev1[i]) != cudaSuccess) {
        return kErrRtFail;
    }
    return ATB_B200_OK;
}

// Writes the current blob into the next pinned staging slot (waiting, on the host, only for the copy
// that last read that slot) and returns it; `*slot_out` is the slot whose event the caller records.
static uint8_t *stage_blob(atb_b200_pa_plan *plan, int *slot_out)
{
    HostPlan &h = plan->hp;
    constexpr int kRing = atb_b200_pa_plan::kStagingRing;
    if (plan->staging_cap < h.blob_bytes) {
        for (int i = 0; i < kRing; ++i) {
            if (plan->upload_pending[i]) {
                cudaEventSynchronize(plan->uploaded[i]);
                plan->upload_pending[i] = false;
            }
        }
        if (plan->staging != nullptr) {
            cudaFreeHost(plan->staging);
            plan->staging = nullptr;
        }
        const size_t cap = ((size_t)h.blob_bytes * 2 + 255) / 256 * 256;
        if (cudaHostAlloc(reinterpret_cast<void **>(&plan->staging), cap * kRing, cudaHostAllocDefault) != cudaSuccess) {
            plan->staging_cap = 0;
            return nullptr;
        }
        plan->staging_cap = cap;
    }
    const int slot = (int)(plan->uploads % kRing);
    if (plan->uploaded[slot] == nullptr &&
        cudaEventCreateWithFlags(&plan->uploaded[slot], cudaEventDisableTiming) != cudaSuccess) {
        return nullptr;
    }
    if (plan->upload_pending[slot]) {
        cudaEventSynchronize(plan->uploaded[slot]); // the copy that last read this slot must be done
    }
    uint8_t *stage = plan->staging + (size_t)slot * plan->staging_cap;
    h.write_blob(stage);
    *slot_out = slot;
    return stage;
}

int atb_b200_pa_plan_prefetch(atb_b200_pa_plan *plan, void *stream_v)
{
    if (plan == nullptr) {
        return kErrInvalidParam;
    }
    HostPlan &h = plan->hp;
    if (h.items.empty()) {
        return ATB_B200_OK;
    }
    constexpr int kRing = atb_b200_pa_plan::kDevRing;
    if (plan->copy_stream == nullptr) {
        if (cudaStreamCreateWithFlags(&plan->copy_stream, cudaStreamNonBlocking) != cudaSuccess) {
            return kErrRtFail;
        }
        for (int i = 0; i < kRing; ++i) {
            if (cudaEventCreateWithFlags(&plan->dev_uploaded[i], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&plan->dev_consumed[i], cudaEventDisableTiming) != cudaSuccess) {
                return kErrRtFail;
            }
        }
    }
    if (plan->dev_cap < h.blob_bytes) {
        for (int i = 0; i < kRing; ++i) {
            if (plan->dev_consumed_pending[i]) {
                cudaEventSynchronize(plan->dev_consumed[i]);
                plan->dev_consumed_pending[i] = false;
            }
        }
        cudaStreamSynchronize(plan->copy_stream);
        if (plan->dev_blob != nullptr) {
            // the status word of the last launch may live in the copy about to be freed (its readers have
            // completed: see the waits above): keep its value for atb_b200_pa_plan_device_status
            const uint8_t *lo = plan->dev_blob, *hi = plan->dev_blob + plan->dev_cap * kRing;
            const uint8_t *sp = reinterpret_cast<const uint8_t *>(plan->last_status_ptr);
            if (sp != nullptr && sp >= lo && sp < hi) {
                plan->has_saved_status =
                    cudaMemcpy(&plan->saved_status, sp, sizeof(int32_t), cudaMemcpyDeviceToHost) == cudaSuccess;
                plan->last_status_ptr = nullptr;
            }
            cudaFree(plan->dev_blob);
            plan->dev_blob = nullptr;
        }
        const size_t cap = ((size_t)h.blob_bytes * 2 + 255) / 256 * 256;
        if (cudaMalloc(reinterpret_cast<void **>(&plan->dev_blob), cap * kRing) != cudaSuccess) {
            plan->dev_cap = 0;
            return 26; // ERROR_OUT_OF_DEVICE_MEMORY
        }
        plan->dev_cap = cap;
    }
    const int slot = (int)(plan->prefetches % kRing);
    if (plan->dev_consumed_pending[slot]) {
        cudaStreamWaitEvent(plan->copy_stream, plan->dev_consumed[slot], 0); // its last readers must be done
        plan->dev_consumed_pending[slot] = false;
    }
    int sslot = 0;
    uint8_t *stage = stage_blob(plan, &sslot);
    if (stage == nullptr) {
        return kErrOutOfHostMemory;
    }
    if (cudaMemcpyAsync(plan->dev_blob + (size_t)slot * plan->dev_cap, stage, h.blob_bytes, cudaMemcpyHostToDevice,
                        plan->copy_stream) != cudaSuccess) {
        return kErrRtFail;
    }
    cudaEventRecord(plan->uploaded[sslot], plan->copy_stream);
    plan->upload_pending[sslot] = true;
    plan->uploads++;
    cudaEventRecord(plan->dev_uploaded[slot], plan->copy_stream);
    // everything the caller enqueues on `stream` from here on runs after the upload
    if (cudaStreamWaitEvent(static_cast<cudaStream_t>(stream_v), plan->dev_uploaded[slot], 0) != cudaSuccess) {
        return kErrRtFail;
    }
    plan->prefetched_slot = slot;
    plan->prefetch_stream = stream_v;
    plan->prefetches++;
    return ATB_B200_OK;
}

static int pa_launch_impl(atb_b200_pa_plan *plan, const atb_b200_pa_tensors *t, const atb_b200_pa_peers *peers,
                          void *workspace, uint64_t workspace_bytes, void *stream_v);

int atb_b200_pa_launch(atb_b200_pa_plan *plan, const atb_b200_pa_tensors *t, void *workspace, uint64_t workspace_bytes,
                       void *stream_v)
{
    return pa_launch_impl(plan, t, nullptr, workspace, workspace_bytes, stream_v);
}

int atb_b200_pa_launch_gathered(atb_b200_pa_plan *plan, const atb_b200_pa_tensors *t, const atb_b200_pa_peers *peers,
                                void *workspace, uint64_t workspace_bytes, void *stream_v)
{
    if (plan == nullptr || peers == nullptr || plan->hp.desc.q_per_seq > 1 || peers->world < 1 || peers->world > 8 || peers->rank < 0 ||
        peers->rank >= peers->world || plan->hp.kernel != ATB_B200_KERNEL_TMA_MMA ||
        peers->head_offset < 0 || peers->head_offset + plan->hp.desc.num_heads > peers->total_heads) {
        return kErrInvalidParam;
    }
    for (int r = 0; r < peers->world; ++r) {
        if (peers->peer_out[r] == nullptr || peers->peer_flags[r] == nullptr) {
            return kErrInvalidParam;
        }
    }
    return pa_launch_impl(plan, t, peers, workspace, workspace_bytes, stream_v);
}

static int pa_launch_impl(atb_b200_pa_plan *plan, const atb_b200_pa_tensors *t, const atb_b200_pa_peers *peers,
                          void *workspace, uint64_t workspace_bytes, void *stream_v)
{
    if (plan == nullptr || t == nullptr || t->q == nullptr || t->k_cache == nullptr || t->v_cache == nullptr ||
        t->block_tables == nullptr || (t->out == nullptr && peers == nullptr) ||
        (plan->hp.desc.rope_dim != 0 && (t->q_rope == nullptr || t->k_rope_cache == nullptr))) {
        return kErrInvalidParam;
    }
    HostPlan &h = plan->hp;
    if ((h.desc.score_mods & ATB_B200_SCORE_MASK) != 0 &&
        (t->mask == nullptr || t->mask_tokens < h.max_context || t->mask_batch_stride < 0 || t->mask_head_stride < 0)) {
        return kErrInvalidParam; // no mask, or one shorter than the longest context
    }
    if ((h.desc.score_mods & ATB_B200_SCORE_MASK) != 0 && h.kernel == ATB_B200_KERNEL_MLA_TC5 && t->mask_head_stride != 0) {
        return kErrInvalidParam; // the MLA kernel adds one mask row to all heads
    }
    if ((h.desc.score_mods & ATB_B200_SCORE_LOGN) != 0 && t->logn == nullptr) {
        return kErrInvalidParam;
    }
    if (workspace_bytes < h.workspace_bytes || (h.workspace_bytes > 0 && workspace == nullptr) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
        return kErrInvalidParam;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (h.items.empty() && peers == nullptr) {
        return ATB_B200_OK; // every sequence is empty: outputs stay untouched
    }
    // ---- the plan blob: already on the device (prefetch), or uploaded now into the workspace
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    uint8_t *blob = ws;
    const int dev_slot = plan->prefetched_slot;
    if (dev_slot >= 0) {
        blob = plan->dev_blob + (size_t)dev_slot * plan->dev_cap;
        if (plan->prefetch_stream != stream_v) { // launched on another stream than the one that waited
            cudaStreamWaitEvent(stream, plan->dev_uploaded[dev_slot], 0);
        }
    } else {
        int sslot = 0;
        uint8_t *stage = stage_blob(plan, &sslot);
        if (stage == nullptr) {
            return kErrOutOfHostMemory;
        }
        if (cudaMemcpyAsync(ws, stage, h.blob_bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) {
            return kErrRtFail;
        }
        cudaEventRecord(plan->uploaded[sslot], stream);
        plan->upload_pending[sslot] = true;
        plan->uploads++;
    }

    const atb_b200_pa_desc &d = h.desc;
    PaArgs a{};
    a.q = t->q;
    a.k_cache = t->k_cache;
    a.v_cache = t->v_cache;
    a.block_tables = t->block_tables;
    a.k_descale = t->k_descale;
    a.v_descale = t->v_descale;
    a.k_offset = t->k_offset;
    a.v_offset = t->v_offset;
    a.p_scale = d.qkv_quant == ATB_B200_QUANT_OFFLINE ? t->p_scale : nullptr;
    if (d.qkv_quant != 0 && (t->k_descale == nullptr || t->v_descale == nullptr ||
                             (d.qkv_quant == ATB_B200_QUANT_OFFLINE && t->p_scale == nullptr))) {
        return kErrInvalidParam;
    }
    a.out = t->out;
    a.q_rope = d.rope_dim != 0 ? t->q_rope : nullptr;
    a.k_rope = d.rope_dim != 0 ? t->k_rope_cache : nullptr;
    if (d.rope_dim != 0 && (a.q_rope == nullptr || a.k_rope == nullptr)) {
        return kErrInvalidParam;
    }
    if ((d.score_mods & ATB_B200_SCORE_MASK) != 0) {
        a.mask = t->mask;
        a.mask_bs = t->mask_batch_stride;
        a.mask_hs = t->mask_head_stride;
        a.mask_qs = d.q_per_seq > 1 ? t->mask_q_stride : 0;
    }
    a.logn = (d.score_mods & ATB_B200_SCORE_LOGN) != 0 ? t->logn : nullptr;
    a.kv_bnsd = d.kv_layout == ATB_B200_KV_BNSD ? 1 : 0;
    a.q_per_seq = d.q_per_seq > 1 ? d.q_per_seq : 1;
    a.seq_lens = (d.score_mods & ATB_B200_SCORE_CAUSAL) != 0 ? reinterpret_cast<const int32_t *>(blob + h.off_lens) : nullptr;
    if (t->lse_out != nullptr && h.kernel != ATB_B200_KERNEL_MLA_TC5) {
        return kErrInvalidParam; // only the MLA kernel writes the log-sum-exp
    }
    a.lse_out = t->lse_out;
    if ((d.score_mods & ATB_B200_SCORE_ROWS) != 0) {
        a.bt_rows = reinterpret_cast<const int32_t *>(blob + h.off_rows);
        a.mask_rows = a.bt_rows + d.batch;
    }
    a.plan.group_begin = reinterpret_cast<const int32_t *>(blob + h.off_group_begin);
    a.plan.items = reinterpret_cast<const PaItem *>(blob + h.off_items);
    a.plan.seq_part_base = reinterpret_cast<const int32_t *>(blob + h.off_part_base);
    a.plan.seq_nparts = reinterpret_cast<const int32_t *>(blob + h.off_nparts);
    a.plan.combine_seqs = reinterpret_cast<const int32_t *>(blob + h.off_combine);
    a.plan.part_o = reinterpret_cast<float *>(ws + h.off_part_o);
    a.plan.part_lse = reinterpret_cast<float *>(ws + h.off_lse);
    a.plan.status = reinterpret_cast<int32_t *>(blob + h.off_status);
    a.plan.done_ctas = reinterpret_cast<int32_t *>(blob + h.off_done);
    a.plan.counters = (h.fused_combine && h.n_partials > 0) ? reinterpret_cast<int32_t *>(blob + h.off_counters) : nullptr;
    plan->last_status_ptr = a.plan.status;
    plan->has_saved_status = false;
    a.plan.n_cta_groups = h.n_cta_groups;
    a.plan.cols = h.cols;
    a.batch = d.batch;
    a.num_heads = d.num_heads;
    a.kv_heads = d.kv_heads;
    a.group = d.num_heads / d.kv_heads;
    a.dk = d.head_dim_k;
    a.dv = d.head_dim_v;
    a.v_row_dim = d.v_row_dim;
    a.block_size = d.block_size;
    a.max_blocks = d.max_blocks_per_seq;
    a.num_blocks = d.num_blocks;
    a.heads_per_cta = h.heads_per_cta;
    a.chunks_per_kvh = h.chunks_per_kvh;
    a.scale_log2 = d.qk_scale * 1.4426950408889634f;
    a.trace = plan->trace;
    a.trace_cap = plan->trace_cap;
    if (peers != nullptr) {
        a.n_out_peers = peers->world;
        a.out_total_heads = peers->total_heads;
        a.out_head_offset = peers->head_offset;
        for (int r = 0; r < peers->world; ++r) {
            a.out_peers[r] = peers->peer_out[r];
            a.peer_flags[r] = peers->peer_flags[r];
        }
        a.xchg_rank = peers->rank;
        a.xchg_epoch = peers->epoch;
        a.xchg_poll_limit = peers->poll_limit;
    }

    const int prof_i = (int)(plan->launches % atb_b200_pa_plan::kProfRing);
    const bool profiled = plan->profile_every > 0 && (plan->launch_seq++ % (uint64_t)plan->profile_every) == 0;
    if (profiled) {
        cudaEventRecord(plan->ev0[prof_i], stream);
    }
    cudaError_t e;
    if (h.kernel == ATB_B200_KERNEL_TMA_MMA) {
        e = d.qkv_quant != 0 ? launch_pa_tma_mma_q8(a, d.out_dtype, d.num_blocks, stream)
            : d.kv_dtype == kInt8 ? launch_pa_tma_mma_i8(a, d.q_dtype, d.num_blocks, stream)
                                  : launch_pa_tma_mma(a, d.q_dtype, d.kv_dtype, d.num_blocks, stream);
    } else if (h.kernel == ATB_B200_KERNEL_MLA_TC5) {
        e = h.mla_pair ? launch_pa_mla_pair(a, d.num_blocks, stream) : launch_pa_mla_tc5(a, d.q_dtype, d.num_blocks, stream);
    } else {
        e = launch_pa_generic(a, d.q_dtype, d.kv_dtype, stream);
    }
    if (profiled) {
        cudaEventRecord(plan->ev1[prof_i], stream);
        plan->launches++;
    }
    if (e != cudaSuccess) {
        std::fprintf(stderr, "[atb][ERROR] paged attention kernel launch failed: %s\n", cudaGetErrorString(e));
        return kErrRtFail;
    }
    if (a.plan.counters == nullptr) {
        e = launch_pa_combine(a, (int)h.combine_seqs.size(), d.q_dtype, stream);
        if (e != cudaSuccess) {
            std::fprintf(stderr, "[atb][ERROR] split-KV merge kernel launch failed: %s\n", cudaGetErrorString(e));
        }
    }
    if (dev_slot >= 0) {
        cudaEventRecord(plan->dev_consumed[dev_slot], stream);
        plan->dev_consumed_pending[dev_slot] = true;
        plan->prefetched_slot = -1;
    }
    return e == cudaSuccess ? ATB_B200_OK : kErrRtFail;
}

int atb_b200_pa_plan_device_status(atb_b200_pa_plan *plan, void *workspace, void *stream_v, int32_t *status)
{
    if (plan == nullptr || status == nullptr || workspace == nullptr) {
        return kErrInvalidParam;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (plan->status_host == nullptr &&
        cudaHostAlloc(reinterpret_cast<void **>(&plan->status_host), 64, cudaHostAllocDefault) != cudaSuccess) {
        return kErrOutOfHostMemory;
    }
    if (plan->last_status_ptr == nullptr && plan->has_saved_status) {
        if (cudaStreamSynchronize(stream) != cudaSuccess) {
            return kErrRtFail;
        }
        *status = plan->saved_status;
        return ATB_B200_OK;
    }
    const uint8_t *ws = static_cast<const uint8_t *>(workspace);
    const void *src = plan->last_status_ptr != nullptr ? static_cast<const void *>(plan->last_status_ptr)
                                                      : static_cast<const void *>(ws + plan->hp.off_status);
    if (cudaMemcpyAsync(plan->status_host, src, sizeof(int32_t), cudaMemcpyDeviceToHost, stream) !=
            cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        return kErrRtFail;
    }
    *status = *plan->status_host;
    return ATB_B200_OK;
}

int atb_b200_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                               const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                               int64_t v_row_bytes, int64_t num_slots, void *stream)
{
    if (slot_mapping == nullptr || num_tokens < 0 || k_row_bytes < 0 || v_row_bytes < 0 || num_slots < 0 ||
        ((key == nullptr) != (key_cache == nullptr)) || ((value == nullptr) != (value_cache == nullptr)) ||
        (key == nullptr && value == nullptr)) {
        return kErrInvalidParam;
    }
    cudaError_t e = launch_reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, num_tokens, k_row_bytes,
                                             v_row_bytes, num_slots, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? ATB_B200_OK : kErrRtFail;
}

} // extern "C"
