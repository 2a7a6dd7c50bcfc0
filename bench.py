"""Benchmark of the paged-decode hot path (ReshapeAndCache + PagedAttention) on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config i]

One step = one decode step over the whole batch: scatter the step's new K/V tokens into the paged
cache, then attention of every sequence's query token over its cached context.  The headline workload is
benchmark configuration 4, the largest one a single GPU holds (skewed long-context GQA decode: bf16,
batch 256, 64 q / 8 kv heads, head_dim 128, block_size 128, context_lens lognormal(7.6, 1.0) clipped to
[16, 32768], 3.4 GB of KV per step) with seeded synthetic tensors; on one GPU the other four
configurations are measured in the same process and reported in the line's `configs` array (`--only`
leaves them out, `--config i` picks another headline).  With N > 1 the kv heads are sharded over the ranks
(strong scaling, one process per GPU) and the per-shard outputs are gathered; the MLA configuration has
a single kv head and is sharded by sequence instead (contiguous chunks of the batch per rank).  At every
N the output is checked against the CPU oracle (`max_abs_err_vs_oracle`).

`--op block_copy | paged_cache_load | norm_rope_reshape` times one of the cache-management kernels instead
(1 GPU, its own JSON line with the achieved HBM bandwidth); the default is the decode hot path.

Prints ONE JSON line: `value` is whole-job KV GB/s with all inputs resident in HBM (device-timed),
`e2e` the same metric through the atb operator API with host buffers (H2D of the step's inputs,
re-planning, D2H of the output inside the timed region), `roofline` the attention kernel's achieved
HBM bandwidth against the measured copy peak, `cpu_baseline` the CPU oracle on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

L2_BYTES = 126 * 1000 * 1000
METRIC = "paged_decode_kv_bandwidth"
UNIT = "GB/s"
HEADLINE_CONFIG = 3          # configuration 4 (skewed long-context GQA): the largest one a single GPU holds
TOLERANCE = {"fp16": 2e-3, "bf16": 8e-3, "int8": 1e-2}   # max-abs error allowed against the oracle


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the attention kernel, from the ncu
# captures summarised under profiles/ (pa_tma_mma_c2_gqa_bf16.md, pa_tma_mma_i8_c3_int8kv.md,
# pa_mla_tc5_c5_mla.md).  Configuration 4 is too large for a full capture: its figure is configuration 2's
# (the same kernel) scaled by the tokens per launch, 819 968 / 193 274.  None where no capture exists.
NCU_TRAFFIC_BYTES = {"c2_gqa_bf16_llama3_8b": 806_130_000, "c3_int8kv_70b": 1_379_560_000,
                     "c5_mla_bf16_dsv3": 257_770_000, "c4_gqa_bf16_skewed": 3_420_040_000}


def ncu_traffic_bytes(case_name):
    return NCU_TRAFFIC_BYTES.get(case_name)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_threads():
    """Host threads the CPU arms use: all of the box's cores, stated explicitly because a launcher may
    export OMP_NUM_THREADS=1 (torch.distributed.run does), which OpenMP's default would follow."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference_arm(args, case, wl):
    """The reference's own CPU implementation of the path = its Python/torch golden, restated in C with
    OpenMP (oracle/pa_oracle.c) because the reference's C++ cannot be built without CANN; timed on
    all host threads on a bounded sample of the same workload."""
    import oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle.build()
    threads = host_threads()
    lens = wl.context_lens(case)
    # bounded sample: the first sequences of the batch, at most ~256k tokens, so a step stays well under a second
    budget, take = 65536 * 4, 0
    while take < case.batch and lens[:take + 1].sum() <= budget:
        take += 1
    take = max(take, 1)
    sub = wl.Case(case.name + f"/first{take}", batch=take, heads=case.heads, kv_heads=case.kv_heads, dk=case.dk,
                  dv=case.dv, block_size=case.block_size, q_dtype=case.q_dtype, kv_dtype=case.kv_dtype,
                  ctx=("list", [int(x) for x in lens[:take]]), mla=case.mla, seed=case.seed)
    h = wl.make_host_inputs(sub)
    kvb = wl.kv_bytes(sub, h["context_lens"])

    def step():
        oracle.reshape_and_cache(h["new_k"], h["new_v"], h["k_cache"], h["v_cache"], h["slot_mapping"])
        oracle.paged_attention(h["q"], h["k_cache"], h["v_cache"], h["block_tables"], h["context_lens"],
                               sub.qk_scale, sub.q_dtype, kv_dtype=sub.kvd, dv=sub.dv,
                               k_descale=h.get("k_descale"), v_descale=h.get("v_descale"), nthreads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = kvb / dt / 1e9
    sample = f"first {take} of {case.batch} sequences ({int(h['context_lens'].sum())} tokens) per step"
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": case.q_dtype, "data": "synthetic",
            "config": {"workload": case.name, "sample": sample},
            "tokens_per_s": take / dt,
            "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def oracle_on_device_inputs(case, wl, d, lens, threads):
    """The CPU oracle on the tensors the GPU run used (copied back from the device, so the cache holds what
    ReshapeAndCache wrote).  Returns (output in the host encoding, seconds)."""
    import oracle
    hk = wl.torch_to_host(d["k_cache"], case.kvd)
    hv = None if case.mla else wl.torch_to_host(d["v_cache"], case.kvd)
    hq = wl.torch_to_host(d["q"], case.q_dtype)
    kd = d["k_descale"].cpu().numpy() if "k_descale" in d else None
    vd = d["v_descale"].cpu().numpy() if "v_descale" in d else None
    t0 = time.perf_counter()
    out = oracle.paged_attention(hq, hk, hv, d["block_tables_host"], lens, case.qk_scale, case.q_dtype, kv_dtype=case.kvd,
                                 dv=case.dv, k_descale=kd, v_descale=vd, nthreads=threads)
    dt = time.perf_counter() - t0

    def again():
        t1 = time.perf_counter()
        oracle.paged_attention(hq, hk, hv, d["block_tables_host"], lens, case.qk_scale, case.q_dtype, kv_dtype=case.kvd,
                               dv=case.dv, k_descale=kd, v_descale=vd, nthreads=threads)
        return time.perf_counter() - t1
    return out, dt, again


class L2Flusher:
    """Empties the L2 between timed steps when a GPU's share of the cache is not well above it: writes a
    256 MB buffer, then reads another one, so that the step starts from a cold L2 that holds clean lines
    (after the write alone it would hold ~126 MB of dirty lines whose write-back the step would pay for)."""

    def __init__(self, dev):
        import torch
        self.w = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.r = torch.zeros(64 << 20, dtype=torch.int32, device=dev)

    def __call__(self):
        self.w.zero_()
        self.r.sum()


def measure_decode(args, case, rt, steps, with_cpu_baseline):
    """Times one configuration on this process's GPU (its shard of it when the job has several ranks):
    device-timed steps with resident inputs, the attention kernel's own time from event pairs inside the same
    steps, the end-to-end step through the operator API with host buffers, and the check against the CPU
    oracle.  Returns the result dictionary on rank 0, None elsewhere."""
    import ctypes
    import torch
    import torch.distributed as dist
    wl, capi, dev, world, rank = rt["wl"], rt["capi"], rt["dev"], rt["world"], rt["rank"]

    # kv heads are sharded over the ranks; the MLA cache has one kv head and is sharded by sequence
    by_sequence = world > 1 and case.kv_heads % world != 0
    if world == 1:
        shard = case
    elif by_sequence:
        shard = case.shard_sequences(rank, world)
    else:
        shard = case.shard_heads(rank, world)
    d = wl.make_device_inputs(shard, dev)
    lens = d["context_lens_host"]
    global_lens = wl.context_lens(case)
    kv_bytes_global = wl.kv_bytes(case, global_lens)
    B, H_local, Dv = shard.batch, shard.heads, shard.dv

    stream = torch.cuda.Stream()
    out = torch.zeros((B, H_local, Dv), dtype=d["q"].dtype, device=dev)
    gathered = torch.zeros((world, B, H_local, Dv), dtype=d["q"].dtype, device=dev) if world > 1 else None
    desc = capi.make_desc(B, shard.heads, shard.kv_heads, shard.dk, Dv, shard.block_size, d["num_blocks"],
                          d["block_tables"].shape[1], shard.q_dtype, shard.kvd, shard.qk_scale,
                          v_row_dim=shard.dk if shard.mla else Dv)
    plan = capi.PaPlan(desc, lens)
    info = plan.info
    ws = torch.empty(max(int(info.workspace_bytes), 256), dtype=torch.uint8, device=dev)
    tens = capi.pa_tensors(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], out, d.get("k_descale"),
                           d.get("v_descale"))
    launches_per_step = 1 + info.kernels_per_launch      # ReshapeAndCache + attention (+ combine)
    p2p = world > 1 and args.gather == "p2p" and info.kernel == capi.KERNEL_TMA_MMA
    exchange = None
    if p2p:
        exchange = capi.PeerExchange(B * case.heads * Dv * out.element_size(), case.heads, rank * H_local)
    torch.cuda.synchronize()

    # The timed loop calls the C ABI with pre-built arguments: at N = 8 a step lasts tens of
    # microseconds and per-call Python marshalling would otherwise bound the measurement.
    L = capi.lib()
    vp = ctypes.c_void_p
    rac_args = (vp(d["new_k"].data_ptr()), vp(d["new_v"].data_ptr()) if d["new_v"] is not None else None,
                vp(d["k_cache"].data_ptr()), vp(d["v_cache"].data_ptr()) if d["v_cache"] is not None else None,
                vp(d["slot_mapping"].data_ptr()), B,
                d["new_k"][0].numel() * d["new_k"].element_size(),
                d["new_v"][0].numel() * d["new_v"].element_size() if d["new_v"] is not None else 0,
                d["k_cache"].shape[0] * d["k_cache"].shape[1], vp(stream.cuda_stream))
    tens_ref, ws_ptr, ws_bytes, stream_ptr = ctypes.byref(tens), vp(ws.data_ptr()), ws.numel(), vp(stream.cuda_stream)
    plan_handle = plan.handle
    gathered_flat = gathered.view(-1) if gathered is not None else None
    out_flat = out.view(-1)
    last_gathered = [None]

    def step():
        rc = L.atb_b200_pa_plan_prefetch(plan_handle, stream_ptr)      # plan upload leaves the critical stream
        rc |= L.atb_b200_reshape_and_cache(*rac_args)
        if p2p:
            peers, last_gathered[0] = exchange.peers()
            rc |= L.atb_b200_pa_launch_gathered(plan_handle, tens_ref, ctypes.byref(peers), ws_ptr, ws_bytes, stream_ptr)
        else:
            rc |= L.atb_b200_pa_launch(plan_handle, tens_ref, ws_ptr, ws_bytes, stream_ptr)
            if world > 1:
                dist.all_gather_into_tensor(gathered_flat, out_flat)
        if rc != 0:
            raise RuntimeError(f"C ABI call failed with {rc}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # A step re-reads the same cache.  When this GPU's share of it is not well above the 126 MB L2
    # (small configurations, or kv heads sharded over many GPUs) the L2 is flushed before every step
    # and the steps are timed one by one so that the flush stays outside.
    flush_l2 = wl.kv_bytes(shard, lens) < 2 * L2_BYTES
    flush = L2Flusher(dev) if flush_l2 else None
    with torch.cuda.stream(stream):
        # value, ms_per_step and the attention kernel's own time all come from the SAME steps: every prof_stride-th
        # launch carries a CUDA-event pair around the attention kernel (atb_b200_pa_plan_set_profiling; an event
        # between ReshapeAndCache and attention costs their programmatic overlap, hence not every launch)
        prof_stride = 8 if steps >= 100 else (4 if steps >= 12 else 1)
        plan.set_profiling(prof_stride)
        for _ in range(args.warmup):
            step()
        barrier()
        sampler = ClockSampler(rt["local_rank"])
        if rank == 0:
            sampler.start()
            time.sleep(0.25)
        if flush_l2:
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            barrier()
            align = torch.zeros(1, device=dev) if world > 1 else None
            for a0, a1 in evs:
                flush()
                if world > 1:
                    # the ranks flush on their own clocks: line them up again (a collective on this stream, outside the
                    # timed region), or a step's wait for its peers would include their flushes
                    dist.all_reduce(align)
                a0.record(stream)
                step()
                a1.record(stream)
            barrier()
            ms = sum(a0.elapsed_time(a1) for a0, a1 in evs) / steps
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(stream)
            for _ in range(steps):
                step()
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1) / steps
        n_prof = max(1, min((steps + prof_stride - 1) // prof_stride, 256))
        kernel_ms = float(np.mean([plan.kernel_ms(i) for i in range(n_prof)]))
        clocks = sampler.stop() if rank == 0 else None
        plan.set_profiling(False)
    status = plan.device_status(ws.data_ptr(), stream.cuda_stream)
    if status != 0:
        raise RuntimeError(f"device status {status}")
    if world > 1:
        t = torch.tensor([ms, kernel_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, kernel_ms = float(t[0]), float(t[1])

    # ---- end to end through the operator API with host buffers (rank-local shard, same step)
    chunks = e2e_chunks(shard, lens, world, ms, args.e2e_chunks)
    if len(chunks) > 1:
        e2e = run_e2e_pipelined(args, shard, rt, d, lens, steps, chunks, out)
    else:
        e2e = run_e2e(args, case, shard, rt, d, lens, gathered, steps, p2p)
    if world > 1:
        t = torch.tensor([e2e["ms"]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e["ms"] = float(t[0])

    # ---- parity: every rank runs the CPU oracle on its own shard's tensors; the per-rank references are
    # all-gathered into the unsharded reference and every rank compares the WHOLE gathered output it holds
    threads = max(1, host_threads() // world)
    with torch.cuda.stream(stream):
        step()
        barrier()
    ref_local, oracle_s, oracle_again = oracle_on_device_inputs(shard, wl, d, lens, threads)
    if world == 1:
        got = wl.torch_to_host(out, case.q_dtype)
        err = float(np.abs(wl.to_f32(got, case.q_dtype) - wl.to_f32(ref_local, case.q_dtype)).max()) if got.size else 0.0
    else:
        # as raw bytes: NCCL moves uint8 whatever the element type
        ref_t = torch.from_numpy(np.ascontiguousarray(ref_local).view(np.uint8).reshape(-1)).to(dev)
        ref_all = torch.empty((world, ref_t.numel()), dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(ref_all.view(-1), ref_t)
        ref_all = ref_all.view(d["q"].dtype).view(world, B, H_local, Dv)
        if p2p:
            mine = exchange.local_tensor(last_gathered[0], (case.batch, case.heads, Dv), d["q"].dtype)
        elif by_sequence:
            mine = gathered.reshape(case.batch, case.heads, Dv)
        else:
            mine = gathered.permute(1, 0, 2, 3).reshape(case.batch, case.heads, Dv)
        if by_sequence:
            ref_full = ref_all.reshape(case.batch, case.heads, Dv)
        else:
            ref_full = ref_all.permute(1, 0, 2, 3).reshape(case.batch, case.heads, Dv)
        e = (mine.float() - ref_full.float()).abs().max().reshape(1)
        dist.all_reduce(e, op=dist.ReduceOp.MAX)
        err = float(e[0])

    res = None
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        value = kv_bytes_global / (ms * 1e-3) / 1e9
        achieved = wl.kv_bytes(shard, lens) / (kernel_ms * 1e-3) / 1e9
        sm_mhz = clocks.get("sm_mhz") if clocks else None
        res = {"workload": case.name, "value": value, "ms_per_step": ms, "steps": steps,
               "dtype": case.q_dtype if case.kvd != "int8" else "int8/" + case.q_dtype,
               "config": {"workload": case.name, "batch": case.batch, "q_heads": case.heads,
                          "kv_heads": case.kv_heads, "head_dim": case.dk, "block_size": case.block_size,
                          "context_tokens": int(global_lens.sum()), "kv_bytes_per_step": kv_bytes_global,
                          "parallelism": ((f"sequence shard x{world} (one kv head: contiguous chunks of the batch per "
                                           "rank), outputs gathered by NCCL all-gather") if by_sequence else
                                          (f"kv-head shard x{world}, outputs gathered by " +
                                           ("peer stores from the attention kernel" if p2p else "NCCL all-gather")))
                          if world > 1 else "single GPU",
                          "l2": ("KV cache per GPU (%.0f MB): L2 flushed before every step (256 MB written, then 256 MB "
                                 "read so that no dirty lines remain), steps timed one by one" if flush_l2 else
                                 "KV cache per GPU (%.0f MB) is larger than the 126 MB L2") %
                                (wl.kv_bytes(shard, lens) / 1e6),
                          "kernel": {1: "generic", 2: "tma_mma", 3: "mla_tc5"}.get(info.kernel, "?"),
                          "ctas": info.num_ctas, "partials": info.num_partials},
               "tokens_per_s": case.batch / (ms * 1e-3),
               "pct_of_8000_gbs": 100.0 * value / (8000.0 * world),
               "pct_of_measured_peak": 100.0 * value / (peak * world),
               "gpu_launches": launches_per_step * steps,
               "clocks": clocks,
               "e2e": {"value": kv_bytes_global / (e2e["ms"] * 1e-3) / 1e9, "unit": UNIT,
                       # at N > 1: summed over the ranks (every rank copies its shard's inputs in and 1/N of the result out)
                       "h2d_bytes_per_step": e2e["h2d"] * world, "d2h_bytes_per_step": e2e["d2h"] * world,
                       "ms_per_step": e2e["ms"], "tokens_per_s": case.batch / (e2e["ms"] * 1e-3),
                       "gather": e2e["gather"], **{k: e2e[k] for k in ("pipeline", "max_abs_diff_vs_kernel_level_path") if k in e2e}},
               "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT,
                            "frac": achieved / peak, "peak_kind": "of " + peak_kind,
                            "kernel": "pa attention kernel, per GPU", "kernel_ms": kernel_ms,
                            "kernel_samples": n_prof,
                            "kernel_ms_x_sm_mhz": kernel_ms * sm_mhz if sm_mhz else None,
                            "traffic": ncu_traffic_bytes(case.name) if world == 1 else None},
               "max_abs_err_vs_oracle": err,
               "oracle_check": ("whole workload; every rank compares the gathered output it holds with the all-gathered "
                                "per-shard oracle results, maximum over ranks") if world > 1 else "whole workload"}
        if case.mla:
            flops = wl.attn_flops(shard, lens)
            res["roofline"]["tensor_tflops"] = flops / (kernel_ms * 1e-3) / 1e12
        if with_cpu_baseline and world == 1:
            reps, t_total = 1, oracle_s
            while reps < 3 or (t_total < 10.0 and reps < 20):
                t_total += oracle_again()
                reps += 1
            dt = t_total / reps
            res["cpu_baseline"] = {"value": wl.kv_bytes(case, lens) / dt / 1e9, "unit": UNIT, "cores": threads,
                                   "kind": "port", "sample": f"whole workload, mean of {reps} runs ({dt * 1e3:.0f} ms each)"}
        elif world == 1:
            res["cpu_baseline"] = {"value": wl.kv_bytes(case, lens) / oracle_s / 1e9, "unit": UNIT, "cores": threads,
                                   "kind": "port", "sample": f"whole workload, one run ({oracle_s * 1e3:.0f} ms)"}
    if exchange is not None:
        exchange.close()
    del d, out, gathered, ws, plan
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--config", type=int, default=HEADLINE_CONFIG,
                    help="index into the benchmark configurations (default: the largest single-GPU one)")
    ap.add_argument("--only", action="store_true", help="measure the chosen configuration alone (no `configs` array)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=0,
                    help="sub-batches of the pipelined end-to-end step on one GPU (0: chosen from the step's copy and kernel times; 1: no pipelining)")
    ap.add_argument("--gather", default="p2p", choices=["p2p", "nccl"],
                    help="N>1: attention stores into every rank's gathered buffer (p2p) or a separate NCCL all-gather")
    ap.add_argument("--variant", default="plain", choices=["plain", "alibi", "mtp2", "mtp2_rows"],
                    help="single-GPU side measurements of the attention kernel's other forms: an alibi mask shared by all "
                         "sequences; two query tokens per sequence (parallel decoding, causal) planned per sequence "
                         "(mtp2: one read of the cache) or per token (mtp2_rows)")
    ap.add_argument("--op", default="decode", choices=["decode", "block_copy", "paged_cache_load", "norm_rope_reshape", "kv_cache"],
                    help="decode (default): the hot path; the others time one cache-management kernel on 1 GPU")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    pkg = entry.load_package()
    wl, capi = pkg.workloads, pkg.capi
    if args.op != "decode":
        run_cache_op_bench(args, capi)
        return
    if args.variant != "plain":
        run_variant_bench(args, wl, capi)
        return
    case = wl.CONFIGS[args.config]
    if args.impl == "reference":
        run_reference_arm(args, case, wl)
        return

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"      # the version banner goes to stdout, which carries the JSON line
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()
    rt = {"wl": wl, "capi": capi, "dev": dev, "world": world, "rank": rank, "local_rank": local_rank}

    res = measure_decode(args, case, rt, args.steps, with_cpu_baseline=not args.no_cpu_baseline)
    # the other configurations, measured in the same process (fewer steps; their CPU figure is the one oracle
    # run that checks them)
    others = []
    if world == 1 and not args.only:
        for i, c in enumerate(wl.CONFIGS):
            if i == args.config:
                continue
            r = measure_decode(args, c, rt, min(args.steps, 200), with_cpu_baseline=False)
            others.append({"workload": r["workload"], "value": r["value"], "ms_per_step": r["ms_per_step"],
                           "kernel_ms": r["roofline"]["kernel_ms"], "dtype": r["dtype"],
                           "roofline": {k: r["roofline"][k] for k in ("achieved", "frac", "kernel_ms", "kernel_ms_x_sm_mhz",
                                                                       "traffic", "tensor_tflops") if k in r["roofline"]},
                           "e2e": r["e2e"], "max_abs_err_vs_oracle": r["max_abs_err_vs_oracle"],
                           "tolerance": TOLERANCE["int8" if c.kvd == "int8" else c.q_dtype],
                           "tokens_per_s": r["tokens_per_s"], "cpu_baseline": r["cpu_baseline"],
                           "clocks": r["clocks"], "l2": r["config"]["l2"], "kernel": r["config"]["kernel"]})
    if rank == 0:
        line = {"metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": world, "steps": res["steps"],
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": res["dtype"], "data": "synthetic", "config": res["config"],
                "tokens_per_s": res["tokens_per_s"], "pct_of_8000_gbs": res["pct_of_8000_gbs"],
                "pct_of_measured_peak": res["pct_of_measured_peak"], "gpu_launches": res["gpu_launches"],
                "clocks": res["clocks"], "e2e": res["e2e"], "roofline": res["roofline"],
                "max_abs_err_vs_oracle": res["max_abs_err_vs_oracle"],
                "tolerance": TOLERANCE["int8" if case.kvd == "int8" else case.q_dtype],
                "oracle_check": res["oracle_check"]}
        if "cpu_baseline" in res:
            line["cpu_baseline"] = res["cpu_baseline"]
        if others:
            line["configs"] = others
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_variant_bench(args, wl, capi):
    """Attention kernel alone on one GPU in one of its other forms, on the chosen configuration's cache: `alibi` adds
    a [heads, 1, tokens] mask; `mtp2` / `mtp2_rows` run two query tokens per sequence (the second sees the whole context,
    the first one token less): `mtp2` as one planned row per sequence whose CTA columns are the (token, head) pairs,
    with the causal rule given as a [tokens, max_ctx] mask (MLA: as the kernel's own rule); `mtp2_rows` as one planned row
    per token (the form ragged token counts use).  KV bytes are counted once per sequence."""
    import torch
    case = wl.CONFIGS[args.config]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    capi.lib()
    d = wl.make_device_inputs(case, dev)
    lens = d["context_lens_host"]
    q_per_seq = 2 if args.variant.startswith("mtp2") else 1
    tokens = case.batch * q_per_seq
    q = d["q"].repeat_interleave(q_per_seq, dim=0).contiguous()
    out = torch.zeros((tokens, case.heads, case.dv), dtype=q.dtype, device=dev)
    mods, mask, strides, mask_tokens, plan_lens, fused, planned_rows, heads = 0, None, (0, 0), 0, lens, 0, tokens, case.heads
    if args.variant == "alibi":
        if case.mla:
            raise SystemExit("the MLA kernel takes no per-head mask")
        mask_tokens = int(lens.max())
        slopes = torch.exp2(-8.0 * (torch.arange(case.heads, device=dev) + 1) / case.heads)
        mask = (slopes[:, None, None] * (torch.arange(mask_tokens, device=dev) - mask_tokens + 1)[None, None, :]).to(q.dtype)
        mods, strides = capi.SCORE_MASK, (0, mask_tokens)
    elif args.variant == "mtp2" and case.mla:
        # the MLA kernel's rows are the (token, head) pairs; the causal rule needs no mask
        mods, fused, planned_rows, heads = capi.SCORE_CAUSAL, 2, case.batch, 2 * case.heads
    elif args.variant == "mtp2":
        mask_tokens = int(lens.max())
        mask = torch.zeros((tokens, mask_tokens), dtype=q.dtype, device=dev)
        first = torch.arange(case.batch, device=dev) * 2                 # a sequence's first token does not see the last key
        mask[first, torch.from_numpy(lens.astype(np.int64) - 1).to(dev)] = -10000.0
        mods, strides, fused, planned_rows, heads = capi.SCORE_MASK, (2 * mask_tokens, 0), 2, case.batch, 2 * case.heads
    else:
        mods = capi.SCORE_ROWS
        plan_lens = np.stack([np.maximum(lens - 1, 1), lens], axis=1).reshape(-1).astype(np.int32)
    desc = capi.make_desc(planned_rows, heads, case.kv_heads, case.dk, case.dv, case.block_size, d["num_blocks"],
                          d["block_tables"].shape[1], case.q_dtype, case.kvd, case.qk_scale,
                          v_row_dim=case.dk if case.mla else case.dv, score_mods=mods, q_per_seq=fused)
    plan = capi.PaPlan(desc, plan_lens)
    if args.variant == "mtp2_rows":
        plan.set_rows(np.repeat(np.arange(case.batch, dtype=np.int32), 2), case.batch)
    info = plan.info
    ws = torch.empty(max(int(info.workspace_bytes), 256), dtype=torch.uint8, device=dev)
    tens = capi.pa_tensors(q, d["k_cache"], d["v_cache"], d["block_tables"], out, d.get("k_descale"), d.get("v_descale"),
                           mask=mask, mask_strides=strides, mask_tokens=mask_tokens, mask_q_stride=mask_tokens if fused else 0)
    stream = torch.cuda.Stream()
    steps = min(args.steps, 500)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            plan.launch(tens, ws.data_ptr(), ws.numel(), stream.cuda_stream)
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        time.sleep(0.25)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            plan.launch(tens, ws.data_ptr(), ws.numel(), stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        clocks = sampler.stop()
    if plan.device_status(ws.data_ptr(), stream.cuda_stream) != 0:
        raise RuntimeError("device status")
    peak, peak_kind = measured_peak_gbs()
    kv = wl.kv_bytes(case, lens)
    value = kv / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                      "dtype": case.q_dtype if case.kvd != "int8" else "int8/" + case.q_dtype, "data": "synthetic",
                      "config": {"workload": case.name, "variant": args.variant, "query_tokens": tokens,
                                 "kv_bytes_per_step": kv, "step": "attention launch alone (with its in-stream plan upload)",
                                 "l2": "KV cache (%.0f MB) %s the 126 MB L2" % (kv / 1e6, "is larger than" if kv > 2 * L2_BYTES
                                                                               else "is not well above"),
                                 "kernel": {1: "generic", 2: "tma_mma", 3: "mla_tc5"}.get(info.kernel, "?"),
                                 "ctas": info.num_ctas, "partials": info.num_partials},
                      "gpu_launches": info.kernels_per_launch * steps, "clocks": clocks,
                      "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak,
                                   "peak_kind": "of " + peak_kind, "traffic": None}}))


def run_cache_op_bench(args, capi):
    """Times one cache-management kernel (1 GPU, device-resident inputs larger than L2, CUDA events on the
    launching stream) and prints its achieved HBM bandwidth: algorithmic bytes = bytes read + bytes written."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    capi.lib()
    rng = np.random.default_rng(2024)
    stream = torch.cuda.Stream()
    heads, d, bs = 8, 128, 128                         # the cache geometry of benchmark configuration 2
    steps = min(args.steps, 200)
    if args.op == "block_copy":
        nb = 4096                                      # 2 x 1 GiB of cache
        kc = torch.empty((nb, bs, heads, d), dtype=torch.bfloat16, device=dev).normal_()
        vc = torch.empty_like(kc).normal_()
        n_src, per = 512, 3                            # 512 sources copied to 3 blocks each
        perm = rng.permutation(nb)
        src = torch.from_numpy(perm[:n_src].astype(np.int32)).to(dev)
        dst = torch.from_numpy(perm[n_src:n_src + n_src * per].astype(np.int32)).to(dev)
        cum = torch.from_numpy((np.arange(1, n_src + 1) * per).astype(np.int32)).to(dev)
        block_bytes = kc[0].numel() * kc.element_size()
        moved = 2 * 2 * n_src * per * block_bytes      # K and V, read + write
        workload = f"{n_src} source blocks x {per} copies, block {block_bytes >> 10} KiB, K and V"

        def step():
            capi.block_copy(kc, vc, src, dst, cum, stream_ptr=stream.cuda_stream)
    elif args.op == "paged_cache_load":
        batch, ctx = 64, 3072
        blocks_per_seq = ctx // bs
        nb = 2 * batch * blocks_per_seq
        kc = torch.empty((nb, bs, heads, d), dtype=torch.bfloat16, device=dev).normal_()
        vc = torch.empty_like(kc).normal_()
        tables = torch.from_numpy(rng.permutation(nb)[:batch * blocks_per_seq].reshape(batch, -1).astype(np.int32)).to(dev)
        cu = torch.from_numpy((np.arange(batch + 1) * ctx).astype(np.int32)).to(dev)
        key = torch.empty((batch * ctx, heads, d), dtype=torch.bfloat16, device=dev)
        value = torch.empty_like(key)
        moved = 2 * 2 * key.numel() * key.element_size()
        workload = f"{batch} sequences x {ctx} tokens, {heads} heads x {d}, bf16, K and V"

        def step():
            capi.paged_cache_load(kc, vc, tables, cu, key, value, cumulative=True, stream_ptr=stream.cuda_stream)
    elif args.op == "kv_cache":
        layers, batch, max_seqlen, hidden = 2, 64, 4096, 1024          # a prefill: 64 sequences x ~3072 new rows of 2 KB
        lens_h = rng.integers(2048, 4097, size=batch).astype(np.int32)
        seq_len, token_offset = torch.from_numpy(lens_h).to(dev), torch.from_numpy(lens_h).to(dev)
        layer_id = torch.tensor([1], dtype=torch.int32, device=dev)
        new_kv = torch.empty((int(lens_h.sum()), hidden), dtype=torch.bfloat16, device=dev).normal_()
        past = torch.zeros((layers, batch, max_seqlen, hidden), dtype=torch.bfloat16, device=dev)
        moved = 2 * new_kv.numel() * new_kv.element_size()
        workload = f"{batch} sequences x 2048..4096 new rows of {hidden} bf16 into layer 1 of a [{layers}, {batch}, {max_seqlen}, {hidden}] cache"

        def step():
            capi.kv_cache(new_kv, layer_id, past, token_offset, seq_len, stream_ptr=stream.cuda_stream)
    else:
        tokens, dx, dr, nb = 4096, 512, 64, 4096       # a prefill-sized batch of new tokens: decode is latency-bound
        x = torch.empty((tokens, 1, dx), dtype=torch.bfloat16, device=dev).normal_()
        gamma = torch.empty(dx, dtype=torch.bfloat16, device=dev).uniform_(0.5, 1.5)
        kr = torch.empty((tokens, dr), dtype=torch.bfloat16, device=dev).normal_()
        cos, sin = torch.empty_like(kr).uniform_(-1, 1), torch.empty_like(kr).uniform_(-1, 1)
        slots = torch.from_numpy(rng.permutation(nb * bs)[:tokens].astype(np.int32)).to(dev)
        cache = torch.zeros((nb, bs, 1, dx + dr), dtype=torch.bfloat16, device=dev)
        moved = tokens * ((dx + 3 * dr) * 2 + (dx + dr) * 2 + 4) + dx * 2
        workload = f"{tokens} new tokens, latent {dx} + rope {dr}, bf16"
        L = capi.lib()

        def step():
            rc = L.atb_b200_norm_rope_reshape(x.data_ptr(), gamma.data_ptr(), kr.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                              slots.data_ptr(), cache.data_ptr(), tokens, dx, dr, 1, 1e-6, nb * bs,
                                              stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"C ABI call failed with {rc}")
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        time.sleep(0.25)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        clocks = sampler.stop()
    peak, peak_kind = measured_peak_gbs()
    achieved = moved / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "cache_op_bandwidth", "value": achieved, "unit": UNIT, "n_gpus": 1, "steps": steps,
                      "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": f"{args.op}: {workload}",
                                 "l2": "working set larger than the 126 MB L2" if moved > 252e6 else "fits in L2: latency-bound"},
                      "gpu_launches": steps, "clocks": clocks,
                      "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                                   "peak_kind": "of " + peak_kind, "kernel": args.op, "kernel_ms": ms, "traffic": None}}))


PCIE_GBS = 50.0   # what a pinned copy reaches on these hosts, for choosing the sub-batches of the end-to-end step only


def e2e_chunks(case, lens, world, step_ms, forced=0):
    """Sub-batches of the end-to-end step on one GPU: contiguous slices of the batch with about equal context tokens
    (equal kernel time).  Pipelining pays where the step's copies (query and new tokens in, output back) are a good part
    of its kernel time: two sub-batches then, four for steps above 300 us (smaller kernels lose more than the overlap
    gains).  [(b0, b1)]; one slice = the whole batch = no pipelining."""
    esz = 2
    io_bytes = case.batch * case.heads * (case.dk + case.dv) * esz          # queries in, outputs back
    copy_us = io_bytes / (PCIE_GBS * 1e3)
    n = 1
    if world == 1 and copy_us >= 0.25 * step_ms * 1e3:
        n = 4 if step_ms > 0.3 else 2
    if forced > 0 and world == 1:
        n = forced
    n = max(1, min(n, case.batch // 2))
    csum = np.concatenate([[0], np.cumsum(np.asarray(lens, dtype=np.int64))])
    cuts = [0]
    for j in range(1, n):
        b = int(np.searchsorted(csum, csum[-1] * j / n))
        cuts.append(min(max(b, cuts[-1] + 1), case.batch - (n - j)))
    cuts.append(case.batch)
    return [(cuts[j], cuts[j + 1]) for j in range(n)]


def run_e2e_pipelined(args, case, rt, d, lens, steps, chunks, check_out):
    """The end-to-end step of run_e2e on one GPU, as sub-batches in a pipeline: each sub-batch has its inputs packed in
    one pinned staging area (one H2D copy on a copy stream), its own ReshapeAndCache and PagedAttention operations
    (Setup re-plans from its host context_lens every step, Execute on the compute stream once its copy has landed) and
    its slice of the output read back on a third stream.  The copies of one sub-batch overlap the kernels of another;
    a step ends when the whole output is in pinned host memory.  The result of the last step is compared with
    `check_out` (the output of the kernel-level path on the same inputs)."""
    import ctypes
    import torch
    wl, capi, dev = rt["wl"], rt["capi"], rt["dev"]
    T = capi.atb_tensor
    s_h2d, s_run, s_d2h = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    names = ["q", "new_k", "block_tables", "slot_mapping", "context_lens"] + ([] if case.mla else ["new_v"])
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=d["q"].dtype, device=dev)
    out_host = torch.empty(tuple(out.shape), dtype=out.dtype).pin_memory()
    ctx = capi.Context(s_run.cuda_stream)
    L = capi.lib()
    arr = capi.Operation._arr
    need = ctypes.c_uint64(0)
    parts, h2d = [], 0
    for b0, b1 in chunks:
        offs, total = {}, 0
        for k in names:
            offs[k] = total
            total += (d[k][b0:b1].numel() * d[k].element_size() + 255) // 256 * 256
        host_pack = torch.empty(total, dtype=torch.uint8).pin_memory()
        dev_pack = torch.empty(total, dtype=torch.uint8, device=dev)
        devb = {}
        for k in names:
            src = d[k][b0:b1]
            n = src.numel() * src.element_size()
            host_pack[offs[k]:offs[k] + n] = src.cpu().contiguous().view(torch.uint8).view(-1)
            devb[k] = dev_pack[offs[k]:offs[k] + n].view(src.dtype).view(src.shape)
            h2d += n
        lens_host = host_pack[offs["context_lens"]:offs["context_lens"] + 4 * (b1 - b0)].view(torch.int32).numpy()
        rac_param = capi.ReshapeAndCacheParam()
        rac_param.kvCacheCfg = 1 if case.mla else 0
        rac = capi.Operation(rac_param)
        pa_kw = dict(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale)
        if case.kvd == "int8":
            pa_kw["quantType"] = 1
        if case.mla:
            pa_kw["mlaVHeadSize"] = case.dv
        pa = capi.Operation(capi.PagedAttentionParam(**pa_kw))
        if case.mla:
            rac_in = [T(devb["new_k"]), T(d["k_cache"]), T(devb["slot_mapping"])]
            rac_out = [T(d["k_cache"])]
            pa_in = [T(devb["q"]), T(d["k_cache"]), T(devb["block_tables"]), T(devb["context_lens"], host=lens_host)]
        else:
            rac_in = [T(devb["new_k"]), T(devb["new_v"]), T(d["k_cache"]), T(d["v_cache"]), T(devb["slot_mapping"])]
            rac_out = [T(d["k_cache"]), T(d["v_cache"])]
            pa_in = [T(devb["q"]), T(d["k_cache"]), T(d["v_cache"]), T(devb["block_tables"]),
                     T(devb["context_lens"], host=lens_host)]
        if case.kvd == "int8":
            pa_in += [T(d["k_descale"]), T(d["v_descale"])]
        pa_out = [T(out[b0:b1])]
        ws_bytes = pa.setup(pa_in, pa_out, ctx)
        ws = torch.empty(max(ws_bytes * 2, 256), dtype=torch.uint8, device=dev)
        parts.append(dict(host_pack=host_pack, dev_pack=dev_pack, rac=rac, pa=pa, keep=(rac_in, rac_out, pa_in, pa_out, devb, ws),
                          rac_i=arr(rac_in), n_ri=len(rac_in), rac_o=arr(rac_out), n_ro=len(rac_out), pa_i=arr(pa_in), n_pi=len(pa_in),
                          pa_o=arr(pa_out), n_po=len(pa_out), ws_ptr=ctypes.c_void_p(ws.data_ptr()), ws_len=ws.numel(),
                          out_dev=out[b0:b1], out_host=out_host[b0:b1], ev_in=torch.cuda.Event(), ev_done=torch.cuda.Event()))
    d2h = out_host.numel() * out_host.element_size()

    def step():
        # sub-batch by sub-batch: the first one's kernels are submitted before the others' copies are even queued
        for p in parts:
            with torch.cuda.stream(s_h2d):
                p["dev_pack"].copy_(p["host_pack"], non_blocking=True)
                p["ev_in"].record(s_h2d)
            s_run.wait_event(p["ev_in"])
            rc = L.atb_b200_operation_setup(p["rac"].handle, p["rac_i"], p["n_ri"], p["rac_o"], p["n_ro"], ctypes.byref(need), ctx.handle)
            rc |= L.atb_b200_operation_setup(p["pa"].handle, p["pa_i"], p["n_pi"], p["pa_o"], p["n_po"], ctypes.byref(need), ctx.handle)
            rc |= L.atb_b200_operation_execute(p["rac"].handle, p["rac_i"], p["n_ri"], p["rac_o"], p["n_ro"], None, 0, ctx.handle)
            rc |= L.atb_b200_operation_execute(p["pa"].handle, p["pa_i"], p["n_pi"], p["pa_o"], p["n_po"], p["ws_ptr"], p["ws_len"], ctx.handle)
            if rc != 0 or need.value > p["ws_len"]:
                raise RuntimeError(f"operator call failed ({rc})")
            p["ev_done"].record(s_run)
            s_d2h.wait_event(p["ev_done"])
            with torch.cuda.stream(s_d2h):
                p["out_host"].copy_(p["out_dev"], non_blocking=True)
        s_d2h.synchronize()                           # the caller consumes the result every step

    torch.cuda.synchronize()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if wl.kv_bytes(case, lens) < 2 * L2_BYTES:
        # the cache is not well above the L2: flush it before every step, outside the step's clock (as run_e2e does)
        flush = L2Flusher(dev)
        total = 0.0
        for _ in range(steps):
            flush()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            step()
            total += time.perf_counter() - t0
        ms = total * 1e3 / steps
    else:
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / steps
    diff = float((out_host.float() - check_out.detach().cpu().float()).abs().max())
    if not diff <= TOLERANCE[case.q_dtype if case.kvd != "int8" else "int8"]:
        raise RuntimeError(f"pipelined end-to-end output differs from the kernel-level path by {diff}")
    return {"ms": ms, "h2d": h2d, "d2h": d2h, "gather": "single GPU",
            "pipeline": f"{len(chunks)} sub-batches of about equal context tokens; the copies of one overlap the kernels of another",
            "max_abs_diff_vs_kernel_level_path": diff}


def run_e2e(args, full_case, case, rt, d, lens, gathered, steps, p2p):
    """The same step through atb::Operation Setup/Execute with HOST buffers: every step copies the
    query, the new K/V tokens, slot_mapping, block_tables and context_lens from pinned host memory
    (packed in one staging area, one H2D copy), re-plans from the host context_lens, runs
    ReshapeAndCache + PagedAttention and reads the output back to pinned host memory, then waits for
    it.  The KV cache itself is the path's resident state and stays in HBM.  The operator calls use
    pre-built tensor records (a C++ caller builds its VariantPack once, too).  `case` is this rank's
    shard of `full_case`; with sharded heads the operator stores into every rank's gathered buffer
    (atb_b200_context_set_gather); the gathered result is read back once by the ranks' hosts between them, rank r taking
    its r-th contiguous 1/N (d2h_bytes_per_step is this rank's share)."""
    import ctypes
    import torch
    import torch.distributed as dist
    wl, capi, dev, world, rank = rt["wl"], rt["capi"], rt["dev"], rt["world"], rt["rank"]
    T = capi.atb_tensor
    stream = torch.cuda.Stream()
    names = ["q", "new_k", "block_tables", "slot_mapping", "context_lens"] + ([] if case.mla else ["new_v"])
    # one pinned staging area and one device area holding all per-step inputs back to back
    offs, total = {}, 0
    for k in names:
        offs[k] = total
        total += (d[k].numel() * d[k].element_size() + 255) // 256 * 256
    host_pack = torch.empty(total, dtype=torch.uint8).pin_memory()
    dev_pack = torch.empty(total, dtype=torch.uint8, device=dev)
    devb, h2d = {}, 0
    for k in names:
        n = d[k].numel() * d[k].element_size()
        host_pack[offs[k]:offs[k] + n] = d[k].cpu().contiguous().view(torch.uint8).view(-1)
        devb[k] = dev_pack[offs[k]:offs[k] + n].view(d[k].dtype).view(d[k].shape)
        h2d += n
    lens_off = offs["context_lens"]
    lens_host = host_pack[lens_off:lens_off + 4 * case.batch].view(torch.int32).numpy()
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=d["q"].dtype, device=dev)
    exchange = None
    if p2p:
        exchange = capi.PeerExchange(case.batch * full_case.heads * case.dv * out.element_size(), full_case.heads,
                                     rank * case.heads)
        result_shape = (case.batch, full_case.heads, case.dv)
    elif world > 1:
        result_shape = tuple(gathered.shape)
    else:
        result_shape = tuple(out.shape)
    # Every rank holds the whole gathered result on its GPU; the ranks' hosts read it back once between them: rank r its
    # r-th contiguous 1/N of the buffer (at N = 1 the whole output)
    n_result = int(np.prod(result_shape))
    r0, r1 = rank * n_result // world, (rank + 1) * n_result // world
    out_host = torch.empty(r1 - r0, dtype=out.dtype).pin_memory()
    ctx = capi.Context(stream.cuda_stream)
    rac_param = capi.ReshapeAndCacheParam()
    rac_param.kvCacheCfg = 1 if case.mla else 0
    rac = capi.Operation(rac_param)
    pa_kw = dict(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale)
    if case.kvd == "int8":
        pa_kw["quantType"] = 1
    if case.mla:
        pa_kw["mlaVHeadSize"] = case.dv
    pa = capi.Operation(capi.PagedAttentionParam(**pa_kw))
    if case.mla:
        rac_in = [T(devb["new_k"]), T(d["k_cache"]), T(devb["slot_mapping"])]
        rac_out = [T(d["k_cache"])]
        pa_in = [T(devb["q"]), T(d["k_cache"]), T(devb["block_tables"]), T(devb["context_lens"], host=lens_host)]
    else:
        rac_in = [T(devb["new_k"]), T(devb["new_v"]), T(d["k_cache"]), T(d["v_cache"]), T(devb["slot_mapping"])]
        rac_out = [T(d["k_cache"]), T(d["v_cache"])]
        pa_in = [T(devb["q"]), T(d["k_cache"]), T(d["v_cache"]), T(devb["block_tables"]),
                 T(devb["context_lens"], host=lens_host)]
    if case.kvd == "int8":
        pa_in += [T(d["k_descale"]), T(d["v_descale"])]
    pa_out = [T(out)]
    ws_bytes = pa.setup(pa_in, pa_out, ctx)
    ws = torch.empty(max(ws_bytes * 2, 256), dtype=torch.uint8, device=dev)
    d2h = out_host.numel() * out_host.element_size()

    L = capi.lib()
    arr = capi.Operation._arr
    rac_i, rac_o, pa_i, pa_o = arr(rac_in), arr(rac_out), arr(pa_in), arr(pa_out)
    n_ri, n_ro, n_pi, n_po = len(rac_in), len(rac_out), len(pa_in), len(pa_out)
    need = ctypes.c_uint64(0)
    ws_ptr, ws_len = ctypes.c_void_p(ws.data_ptr()), ws.numel()
    gathered_flat = gathered.view(-1) if gathered is not None else None
    gathered_views = {}

    def step():
        dev_pack.copy_(host_pack, non_blocking=True)
        # Setup of both operators first (host planning; PagedAttention re-plans from the host
        # context_lens and starts uploading its plan), then the two Executes
        rc = L.atb_b200_operation_setup(rac.handle, rac_i, n_ri, rac_o, n_ro, ctypes.byref(need), ctx.handle)
        rc |= L.atb_b200_operation_setup(pa.handle, pa_i, n_pi, pa_o, n_po, ctypes.byref(need), ctx.handle)
        rc |= L.atb_b200_operation_execute(rac.handle, rac_i, n_ri, rac_o, n_ro, None, 0, ctx.handle)
        if p2p:
            peers, local_ptr = exchange.peers()
            rc |= L.atb_b200_context_set_gather(ctx.handle, ctypes.byref(peers))
        rc |= L.atb_b200_operation_execute(pa.handle, pa_i, n_pi, pa_o, n_po, ws_ptr, ws_len, ctx.handle)
        if rc != 0 or need.value > ws_len:
            raise RuntimeError(f"operator call failed ({rc})")
        if p2p:
            if local_ptr not in gathered_views:
                gathered_views[local_ptr] = exchange.local_tensor(local_ptr, result_shape, out.dtype).view(-1)[r0:r1]
            out_host.copy_(gathered_views[local_ptr], non_blocking=True)
        elif world > 1:
            dist.all_gather_into_tensor(gathered_flat, out.view(-1))
            out_host.copy_(gathered_flat[r0:r1], non_blocking=True)
        else:
            out_host.copy_(out.view(-1), non_blocking=True)
        stream.synchronize()                          # the caller consumes the result every step

    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if wl.kv_bytes(case, lens) < 2 * L2_BYTES:
            # this GPU's cache is not well above the L2: flush it before every step, outside the step's clock
            flush = L2Flusher(dev)
            total = 0.0
            for _ in range(steps):
                flush()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()                    # the ranks flush on their own clocks: start the step together
                t0 = time.perf_counter()
                step()
                total += time.perf_counter() - t0
            ms = total * 1e3 / steps
        else:
            t0 = time.perf_counter()
            for _ in range(steps):
                step()
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) * 1e3 / steps
    if exchange is not None:
        exchange.close()
    how = "single GPU" if world == 1 else (("peer stores from the attention kernel (operator-level gather)" if p2p
                                            else "NCCL all-gather") + f"; each rank's host reads 1/{world} of the gathered result")
    return {"ms": ms, "h2d": h2d, "d2h": d2h, "gather": how}


if __name__ == "__main__":
    main()
