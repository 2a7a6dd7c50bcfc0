// Cross-GPU completion exchange at the tail of a sharded attention kernel.
//
// Every CTA makes its peer stores visible system-wide and counts itself done; the CTA that finishes
// last publishes "rank r finished step e" into every rank's flag array and waits until every rank
// has published the same step, so that when the kernel completes the local gathered output is whole.
// The wait is bounded (xchg_poll_limit polls of about 0.2 us each, 2^22 by default): if a peer never
// arrives the kernel records kStatusWaitTimeout and returns instead of hanging the GPU; the gathered
// output is then incomplete, which only the status word tells.  This replaces the separate AllGatherOperation a model graph of the
// reference runs after attention (src/ops/ops_infer/all_gather/all_gather_hccl_runner.cpp:47).
#ifndef ATB_B200_PA_EXCHANGE_CUH
#define ATB_B200_PA_EXCHANGE_CUH
#include "pa_plan.h"

namespace atb_b200 {

// Called by one full warp per CTA after all of the CTA's output stores have been issued and fenced.
__device__ __forceinline__ void exchange_tail(const PaArgs &a, int lane)
{
    int last = 0;
    if (lane == 0) {
        const int old = atomicAdd(a.plan.done_ctas, 1);
        last = (old == (int)gridDim.x - 1) ? 1 : 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) {
        return;
    }
    __threadfence_system();
    if (lane < a.n_out_peers) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[lane] + a.xchg_rank), "r"(a.xchg_epoch)
                     : "memory");
        const uint32_t *mine = a.peer_flags[a.xchg_rank] + lane;
        uint32_t seen = 0;
        bool ok = false;
        const uint32_t limit = a.xchg_poll_limit != 0 ? a.xchg_poll_limit : (1u << 22);
        for (uint32_t i = 0; i < limit; ++i) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int32_t)(seen - a.xchg_epoch) >= 0) {
                ok = true;
                break;
            }
            if (i > 256) {
                __nanosleep(200);
            }
        }
        if (!ok) {
            atomicExch(a.plan.status, kStatusWaitTimeout);
        }
    }
}

} // namespace atb_b200
#endif
