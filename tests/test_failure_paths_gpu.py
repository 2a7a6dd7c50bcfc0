"""Failure paths on the device that fault, trap or hang nothing.

A sharded attention launch waits, at its tail, for every rank to publish a completion flag.  Here one
GPU plays rank 0 of a world of two whose second "rank" is a pair of local buffers nobody else touches:
its flag is never published, so the wait runs out after its (short) poll limit, the kernel records
status 1 and returns, and the context stays usable.  The reference's behaviour for a failed launch is
a return code only (src/atb/operation/operation_base.cpp:933-935); the status word is this library's
addition for failures that happen after the call has returned.
"""
import ctypes

import numpy as np
import pytest

from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, tol_for, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _sharded_launch(case, h, d, poll_limit):
    """Launches `case` as rank 0 of 2 (its heads are the first half of a model with twice as many);
    returns (return code, device status, this rank's gathered buffer as a tensor)."""
    tdt = wl.torch_dtype(case.q_dtype)
    total_heads = 2 * case.heads
    gathered = [torch.zeros((case.batch, total_heads, case.dv), dtype=tdt, device="cuda") for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    desc = capi.make_desc(case.batch, case.heads, case.kv_heads, case.dk, case.dv, case.block_size, h["num_blocks"],
                          h["block_tables"].shape[1], case.q_dtype, case.kvd, case.qk_scale)
    plan = capi.PaPlan(desc, h["context_lens"])
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], None, d["k_descale"], d["v_descale"],
                           d["k_offset"], d["v_offset"])
    peers = capi.PaPeers()
    peers.world, peers.rank, peers.total_heads, peers.head_offset = 2, 0, total_heads, 0
    for r in range(2):
        peers.peer_out[r] = gathered[r].data_ptr()
        peers.peer_flags[r] = flags[r].data_ptr()
    peers.epoch, peers.poll_limit = 1, poll_limit
    rc = capi.lib().atb_b200_pa_launch_gathered(plan.handle, ctypes.byref(tens), ctypes.byref(peers),
                                                ctypes.c_void_p(ws.data_ptr()), ws.numel(), capi.torch_stream_ptr())
    torch.cuda.synchronize()
    status = plan.device_status(ws.data_ptr(), capi.torch_stream_ptr())
    return rc, status, gathered, flags


@pytest.mark.parametrize("case", [
    wl.Case("timeout_gqa4_bf16", batch=5, heads=16, kv_heads=4, q_dtype="bf16", ctx=("uniform", 60, 3000), seed=81),
    wl.Case("timeout_int8_fp16", batch=3, heads=8, kv_heads=1, q_dtype="fp16", kv_dtype="int8", ctx=("uniform", 100, 900),
            seed=82),
], ids=lambda c: c.name)
def test_wait_for_a_peer_that_never_arrives_times_out(case):
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    rc, status, gathered, flags = _sharded_launch(case, h, d, poll_limit=2000)
    assert rc == 0                       # the call only enqueues
    assert status == 1                   # kStatusWaitTimeout: the second rank never published its flag
    # this rank published its own step number into both flag arrays, slot 0; nobody wrote slot 1
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1 and int(flags[0][1]) == 0
    # its own heads are whole in both gathered buffers, the other rank's columns are untouched
    ref = oracle_out(case, h)
    for g in gathered:
        mine = wl.torch_to_host(g[:, :case.heads].contiguous(), case.q_dtype)
        assert max_abs_err(mine, ref, case.q_dtype) <= tol_for(case)
        assert float(g[:, case.heads:].float().abs().max()) == 0.0
    # the context is intact: an ordinary launch right after is clean and correct
    out, plan, ws = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], h["context_lens"],
                                         case.qk_scale, k_descale=d["k_descale"], v_descale=d["v_descale"],
                                         return_plan=True)
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
    assert max_abs_err(wl.torch_to_host(out, case.q_dtype), ref, case.q_dtype) <= tol_for(case)


def test_wait_succeeds_when_the_flag_is_already_there():
    """The same set-up with the second rank's flag published beforehand: no time-out."""
    case = wl.Case("flag_present", batch=4, heads=8, kv_heads=2, q_dtype="fp16", ctx=("uniform", 200, 1500), seed=83)
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    tdt = wl.torch_dtype(case.q_dtype)
    gathered = torch.zeros((case.batch, 2 * case.heads, case.dv), dtype=tdt, device="cuda")
    other = torch.zeros_like(gathered)
    flags0 = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags1 = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags0[1] = 7                         # "rank 1 has finished step 7" in this rank's flag array
    desc = capi.make_desc(case.batch, case.heads, case.kv_heads, 128, 128, 128, h["num_blocks"], h["block_tables"].shape[1],
                          case.q_dtype, case.kvd, case.qk_scale)
    plan = capi.PaPlan(desc, h["context_lens"])
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], None)
    peers = capi.PaPeers()
    peers.world, peers.rank, peers.total_heads, peers.head_offset = 2, 0, 2 * case.heads, 0
    peers.peer_out[0], peers.peer_out[1] = gathered.data_ptr(), other.data_ptr()
    peers.peer_flags[0], peers.peer_flags[1] = flags0.data_ptr(), flags1.data_ptr()
    peers.epoch, peers.poll_limit = 7, 2000
    plan.launch_gathered(tens, peers, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
    ref = oracle_out(case, h)
    assert max_abs_err(wl.torch_to_host(gathered[:, :case.heads].contiguous(), case.q_dtype), ref, case.q_dtype) <= tol_for(case)


def test_status_survives_a_plan_that_grows_after_the_launch():
    """The status word of a launch that used a prefetched plan lives in plan-owned device memory.  When the
    next, larger plan makes that memory grow, the old copy is freed: the status of the finished launch must
    still be readable (here: 2, a block id outside the cache) and nothing may read freed memory."""
    case = wl.Case("status_regrow", batch=3, heads=8, kv_heads=2, q_dtype="bf16", ctx=("list", [38400, 200, 150]), seed=84)
    h = wl.make_host_inputs(case)
    h["block_tables"] = h["block_tables"].copy()
    h["block_tables"][0, 1] = h["num_blocks"] + 3
    d = host_inputs_to_device(case, h)
    short = np.array([300, 200, 150], dtype=np.int32)       # a prefix of every sequence: few work items
    desc = capi.make_desc(case.batch, case.heads, case.kv_heads, 128, 128, 128, h["num_blocks"], h["block_tables"].shape[1],
                          case.q_dtype, case.kvd, case.qk_scale)
    plan = capi.PaPlan(desc, short)
    small_bytes = plan.info.plan_bytes
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.bfloat16, device="cuda")
    tens = capi.pa_tensors(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], out)
    ws = torch.empty(16 << 20, dtype=torch.uint8, device="cuda")
    sp = capi.torch_stream_ptr()
    plan.prefetch(sp)
    plan.launch(tens, ws.data_ptr(), ws.numel(), sp)
    torch.cuda.synchronize()
    plan.update(h["context_lens"])                          # one long sequence: the work list grows several times over
    assert plan.info.plan_bytes > 2 * small_bytes and plan.info.workspace_bytes <= ws.numel()
    plan.prefetch(sp)                                       # the device copy is re-allocated here
    assert plan.device_status(ws.data_ptr(), sp) == 2       # the finished launch's status, not freed memory
    h["block_tables"][0, 1] = h["block_tables"][0, 0]       # repair the table (any valid block) and run the long plan
    d["block_tables"].copy_(torch.from_numpy(h["block_tables"]))
    plan.launch(tens, ws.data_ptr(), ws.numel(), sp)
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), sp) == 0
    assert torch.isfinite(out.float()).all()
