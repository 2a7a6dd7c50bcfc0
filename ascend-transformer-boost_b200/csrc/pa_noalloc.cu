// Paged decode attention for callers that must not allocate.
//
// Who needs this: an inference server that reserves all device memory up front and forbids
// cudaMalloc afterwards, a host thread with a latency bound that an allocator lock would break, or
// a plugin loaded into a runtime whose own allocator must be the only one touching the device.
// The regular entry points take a caller-provided workspace and keep a pinned staging buffer inside
// the plan object; this one takes neither.  It plans on the stack, uploads the plan with a plain
// cudaMemcpyAsync from that stack buffer, and points the attention and combine kernels at a scratch
// array that is part of the library image.
//
// The price is a fixed capacity (see the limits below; larger calls are refused, never truncated)
// and a single shared scratch: the array keeps the previous call's contents, so everything a call
// reads from it is written by that same call first (the plan, including its zeroed status word, is
// uploaded before the kernels run; partial results are fully written by the attention kernel before
// the combine kernel reads them).  Two calls whose kernels may be in flight at the same time - on
// different streams, or from different host threads - race on the array and give wrong results; a
// single stream, or explicit ordering between the streams, is required.
//
// Device address of the scratch: inside host code the array's name is only a handle, not something
// a kernel may dereference, so the first call on each device asks the runtime for the real address
// with cudaGetSymbolAddress while that device is current and caches it.  That first call per device
// therefore does a little extra work and should be made before any stream capture begins.  Later calls
// read the cached address with one atomic load (no lock).
//
// The plan travels to the device by cudaMemcpyAsync from the (pageable) stack buffer: the runtime
// stages such a copy before the call returns, which may make the host wait until the stream has
// reached the copy.  For the same reason a call on a stream that is being captured is refused
// (ERROR_INVALID_PARAM): a captured copy node would keep the address of a dead stack frame, and the
// split would stay frozen at the lengths seen at capture time.
//
// Device-side status (a bounded wait that gave up, a block id outside the cache) is written into the
// first word of the scratch (cleared by every call's plan upload); atb_b200_pa_static_scratch_status
// copies it back on the caller's stream, also without allocating.
#include <cuda_runtime.h>
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include "../../include/atb_b200.h"
#include "kernels.h"
#include "pa_plan.h"

namespace atb_b200 {
namespace {

// ---- capacity of the built-in scratch (held by every GPU that loads the library, until exit)
constexpr int kMaxBatch = 1024;                       // sequences per call
constexpr int kMaxGroups = 1024;                      // CTA groups of the work split
constexpr int kMaxItems = kMaxBatch + kMaxGroups;     // token ranges
constexpr uint64_t kBlobCap = 64 * 1024;              // uploaded plan
constexpr uint64_t kLseFloats = 64 * 1024;            // partials x query heads
constexpr uint64_t kPartFloats = 2 * 1024 * 1024;     // partials x query heads x head_dim_v
constexpr uint64_t kOffLse = kBlobCap;
constexpr uint64_t kOffPartO = kOffLse + kLseFloats * sizeof(float);
constexpr uint64_t kScratchBytes = kOffPartO + kPartFloats * sizeof(float); // 8 MiB + 320 KiB

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kErrInvalidParam = 1;
constexpr int kErrRtFail = 4;
constexpr int kErrInvalidTensorDim = 8;

std::mutex g_setup_mutex;
std::atomic<unsigned char *> g_scratch_ptr[64];

// Device address of g_static_scratch on the current device.  Looked up once per device under a
// mutex; every later call takes the cached pointer with a single atomic load.
int scratch_address(unsigned char **out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return kErrRtFail;
    }
    unsigned char *ptr = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        ptr = g_scratch_ptr[dev].load(std::memory_order_relaxed);
        if (ptr == nullptr) {
            const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch);
            if (e != cudaSuccess || ptr == nullptr) {
                std::fprintf(stderr, "[atb][ERROR] static scratch: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
                return kErrRtFail;
            }
            g_scratch_ptr[dev].store(ptr, std::memory_order_release);
        }
    }
    *out = ptr;
    return 0;
}

int refuse(const char *what, long long got, long long limit)
{
    std::fprintf(stderr, "[atb][ERROR] atb_b200_pa_decode_static_scratch: %s = %lld exceeds the built-in limit %lld\n",
                 what, got, limit);
    return kErrInvalidParam;
}

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

} // namespace
} // namespace atb_b200

using namespace atb_b200;

extern "C" int atb_b200_pa_decode_static_scratch(const atb_b200_pa_desc *desc, const int32_t *context_lens_host,
                                                 const atb_b200_pa_tensors *t, void *stream_v)
{
    if (desc == nullptr || t == nullptr || (context_lens_host == nullptr && desc->batch > 0) || t->q == nullptr ||
        t->k_cache == nullptr || t->v_cache == nullptr || t->block_tables == nullptr || t->out == nullptr) {
        return kErrInvalidParam;
    }
    const atb_b200_pa_desc &d = *desc;
    if (d.batch < 0 || d.num_heads <= 0 || d.kv_heads <= 0 || d.num_heads % d.kv_heads != 0 || d.head_dim_k <= 0 ||
        d.head_dim_v <= 0 || d.v_row_dim < d.head_dim_v || d.block_size <= 0 || d.num_blocks <= 0 ||
        d.max_blocks_per_seq <= 0) {
        return kErrInvalidParam;
    }
    if (d.rope_dim != 0 || d.score_mods != 0 || d.kv_layout != 0 || d.q_per_seq > 1 || d.qkv_quant != 0) {
        return kErrInvalidTensorDim; // the split latent / rope cache, masks, logN scaling and the heads-major
                                     // cache layout are served by the planned entry points only
    }
    if (d.batch > kMaxBatch) {
        return refuse("batch", d.batch, kMaxBatch);
    }
    {
        // a copy from this call's stack frame must not become a node of a captured graph
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream_v), &cap) != cudaSuccess) {
            return kErrRtFail;
        }
        if (cap != cudaStreamCaptureStatusNone) {
            std::fprintf(stderr, "[atb][ERROR] atb_b200_pa_decode_static_scratch: the stream is being captured; this entry "
                                 "point uploads its plan from the caller's stack and cannot be part of a graph\n");
            return kErrInvalidParam;
        }
    }
    const int group = d.num_heads / d.kv_heads;
    const bool tma_i8 = pa_tma_mma_i8_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.block_size, group, d.q_dtype,
                                                d.kv_dtype);
    const bool tma_ok = tma_i8 || pa_tma_mma_supported(d.head_dim_k, d.head_dim_v, d.v_row_dim, d.block_size, group,
                                                       d.q_dtype, d.kv_dtype);
    const bool gen_ok = pa_generic_supported(d.head_dim_k, d.head_dim_v, d.q_dtype, d.kv_dtype);
    int kernel = d.kernel == ATB_B200_KERNEL_AUTO ? (tma_ok ? ATB_B200_KERNEL_TMA_MMA : ATB_B200_KERNEL_GENERIC) : d.kernel;
    if ((kernel == ATB_B200_KERNEL_TMA_MMA && !tma_ok) || (kernel == ATB_B200_KERNEL_GENERIC && !gen_ok) ||
        (kernel != ATB_B200_KERNEL_TMA_MMA && kernel != ATB_B200_KERNEL_GENERIC)) {
        return kErrInvalidTensorDim;
    }
    int sm = d.sm_count;
    if (sm <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm <= 0) {
            return kErrRtFail;
        }
    }
    unsigned char *scratch = nullptr;
    int rc = scratch_address(&scratch);
    if (rc != 0) {
        return rc;
    }

    // ---- work split on the stack: same balanced cut as the regular planner, fixed capacity
    const int heads_per_cta = kernel == ATB_B200_KERNEL_TMA_MMA ? 8 : pa_generic_heads_per_cta(d.head_dim_k, d.head_dim_v);
    const int chunks_per_kvh = (group + heads_per_cta - 1) / heads_per_cta;
    const int ctas_per_sm = kernel == ATB_B200_KERNEL_TMA_MMA ? (d.head_dim_k > 128 ? 1 : 2) : 4;
    const int cols = d.kv_heads * chunks_per_kvh;
    const int64_t max_ctx = (int64_t)d.max_blocks_per_seq * d.block_size;
    int64_t seq_start[kMaxBatch + 1];
    seq_start[0] = 0;
    for (int b = 0; b < d.batch; ++b) {
        const int64_t ctx = context_lens_host[b];
        if (ctx < 0 || ctx > max_ctx) {
            return kErrInvalidParam;
        }
        seq_start[b + 1] = seq_start[b] + (ctx + kTileTokens - 1) / kTileTokens;
    }
    const int64_t total_tiles = seq_start[d.batch];
    if (total_tiles == 0) {
        return ATB_B200_OK; // every sequence is empty: outputs stay untouched
    }
    int64_t n_groups = std::max<int64_t>(1, (int64_t)sm * ctas_per_sm / cols);
    n_groups = std::max<int64_t>(n_groups, 4);
    n_groups = std::min<int64_t>(n_groups, total_tiles);
    if (n_groups > kMaxGroups) {
        return refuse("CTA groups", n_groups, kMaxGroups);
    }
    const int64_t snap = (total_tiles / n_groups >= 8) ? 1 : 0;

    alignas(16) unsigned char blob[kBlobCap];
    const uint64_t off_status = 0;          // fixed place: atb_b200_pa_static_scratch_status reads it
    uint64_t off = 16;
    const uint64_t off_group_begin = off;
    off = align_up(off + (uint64_t)(n_groups + 1) * sizeof(int32_t), 16);
    const uint64_t off_items = off;
    off = align_up(off + (uint64_t)(d.batch + n_groups) * sizeof(PaItem), 16);
    const uint64_t off_part_base = off;
    off = align_up(off + (uint64_t)d.batch * sizeof(int32_t), 16);
    const uint64_t off_nparts = off;
    off = align_up(off + (uint64_t)d.batch * sizeof(int32_t), 16);
    const uint64_t off_combine = off;
    off = align_up(off + (uint64_t)d.batch * sizeof(int32_t), 16);
    const uint64_t blob_bytes = align_up(off, 256);
    if (blob_bytes > kBlobCap) {
        return refuse("plan bytes", (long long)blob_bytes, (long long)kBlobCap);
    }
    std::memset(blob, 0, blob_bytes); // also clears the status word the kernels report into
    int32_t *group_begin = reinterpret_cast<int32_t *>(blob + off_group_begin);
    PaItem *items = reinterpret_cast<PaItem *>(blob + off_items);
    int32_t *part_base = reinterpret_cast<int32_t *>(blob + off_part_base);
    int32_t *nparts = reinterpret_cast<int32_t *>(blob + off_nparts);
    int32_t *combine = reinterpret_cast<int32_t *>(blob + off_combine);

    int n_items = 0;
    {
        int b_cut = 0, b = 0;
        int64_t prev_cut = 0;
        group_begin[0] = 0;
        for (int64_t j = 0; j < n_groups; ++j) {
            int64_t end = total_tiles;
            if (j + 1 < n_groups) {
                end = ((j + 1) * total_tiles) / n_groups;
                while (b_cut < d.batch && seq_start[b_cut + 1] <= end) {
                    ++b_cut;
                }
                if (b_cut < d.batch && end > seq_start[b_cut]) {
                    if (end - seq_start[b_cut] <= snap) {
                        end = seq_start[b_cut];
                    } else if (seq_start[b_cut + 1] - end <= snap) {
                        end = seq_start[b_cut + 1];
                    }
                }
                end = std::max(end, prev_cut);
            }
            int64_t pos = prev_cut;
            while (pos < end) {
                while (seq_start[b + 1] <= pos) {
                    ++b;
                }
                const int64_t stop = std::min(end, seq_start[b + 1]);
                if (n_items >= kMaxItems || n_items >= d.batch + n_groups) {
                    return kErrInvalidParam; // cannot happen: at most batch + groups ranges exist
                }
                PaItem &it = items[n_items++];
                it.seq = b;
                it.tok_begin = (int32_t)((pos - seq_start[b]) * kTileTokens);
                it.tok_end = (int32_t)std::min<int64_t>(context_lens_host[b], (stop - seq_start[b]) * kTileTokens);
                it.slot = -1;
                nparts[b] += 1;
                pos = stop;
            }
            group_begin[j + 1] = n_items;
            prev_cut = end;
        }
    }
    int n_partials = 0, n_combine = 0;
    for (int i = 0; i < n_items;) {
        const int b = items[i].seq;
        const int np = nparts[b];
        if (np > 1) {
            part_base[b] = n_partials;
            for (int k = 0; k < np; ++k) {
                items[i + k].slot = n_partials + k;
            }
            n_partials += np;
            combine[n_combine++] = b;
        }
        i += np;
    }
    if ((uint64_t)n_partials * d.num_heads > kLseFloats) {
        return refuse("partials x heads", (long long)n_partials * d.num_heads, (long long)kLseFloats);
    }
    if ((uint64_t)n_partials * d.num_heads * d.head_dim_v > kPartFloats) {
        return refuse("partials x heads x head_dim_v", (long long)n_partials * d.num_heads * d.head_dim_v,
                      (long long)kPartFloats);
    }

    // ---- upload the plan (the stack buffer may be reused as soon as the call returns) and launch
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (cudaMemcpyAsync(scratch, blob, blob_bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        return kErrRtFail;
    }
    PaArgs a{};
    a.q = t->q;
    a.k_cache = t->k_cache;
    a.v_cache = t->v_cache;
    a.block_tables = t->block_tables;
    a.k_descale = t->k_descale;
    a.v_descale = t->v_descale;
    a.k_offset = t->k_offset;
    a.v_offset = t->v_offset;
    a.out = t->out;
    a.plan.group_begin = reinterpret_cast<const int32_t *>(scratch + off_group_begin);
    a.plan.items = reinterpret_cast<const PaItem *>(scratch + off_items);
    a.plan.seq_part_base = reinterpret_cast<const int32_t *>(scratch + off_part_base);
    a.plan.seq_nparts = reinterpret_cast<const int32_t *>(scratch + off_nparts);
    a.plan.combine_seqs = reinterpret_cast<const int32_t *>(scratch + off_combine);
    a.plan.part_lse = reinterpret_cast<float *>(scratch + kOffLse);
    a.plan.part_o = reinterpret_cast<float *>(scratch + kOffPartO);
    a.plan.status = reinterpret_cast<int32_t *>(scratch + off_status);
    a.plan.n_cta_groups = (int32_t)n_groups;
    a.plan.cols = cols;
    a.batch = d.batch;
    a.num_heads = d.num_heads;
    a.kv_heads = d.kv_heads;
    a.group = group;
    a.dk = d.head_dim_k;
    a.dv = d.head_dim_v;
    a.v_row_dim = d.v_row_dim;
    a.block_size = d.block_size;
    a.max_blocks = d.max_blocks_per_seq;
    a.num_blocks = d.num_blocks;
    a.heads_per_cta = heads_per_cta;
    a.chunks_per_kvh = chunks_per_kvh;
    a.scale_log2 = d.qk_scale * 1.4426950408889634f;
    cudaError_t e;
    if (kernel == ATB_B200_KERNEL_TMA_MMA) {
        e = tma_i8 ? launch_pa_tma_mma_i8(a, d.q_dtype, d.num_blocks, stream)
                   : launch_pa_tma_mma(a, d.q_dtype, d.kv_dtype, d.num_blocks, stream);
    } else {
        e = launch_pa_generic(a, d.q_dtype, d.kv_dtype, stream);
    }
    if (e != cudaSuccess) {
        return kErrRtFail;
    }
    e = launch_pa_combine(a, n_combine, d.q_dtype, stream);
    return e == cudaSuccess ? ATB_B200_OK : kErrRtFail;
}

extern "C" int atb_b200_pa_static_scratch_status(void *stream, int32_t *status_out)
{
    if (status_out == nullptr) {
        return atb_b200::kErrInvalidParam;
    }
    unsigned char *scratch = nullptr;
    const int rc = atb_b200::scratch_address(&scratch);
    if (rc != 0) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        return atb_b200::kErrInvalidParam;
    }
    // the status word is the first word of the scratch; the destination may be pageable: the call waits for the copy
    if (cudaMemcpyAsync(status_out, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        return atb_b200::kErrRtFail;
    }
    return ATB_B200_OK;
}
