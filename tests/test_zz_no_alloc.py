"""The allocation-free entry point against the regular one.

Some callers of this library cannot allocate: a server that gave all device memory to its own pool
and bans cudaMalloc, or a host thread with a latency bound.  For them the library has
`atb_b200_pa_decode_static_scratch`, which keeps its workspace in a scratch array built into the
library.  This test calls it twice in a row through the C ABI (the second call finds the first
call's leftovers in the shared scratch) and compares with `atb_b200_pa_launch`, which uses a
caller-provided workspace, on the same inputs; both plan the same split (only the order in which the
split-KV partials are summed differs), so the outputs must agree to within the parity tolerance, and
each is also held against the CPU oracle.  It also checks that a call beyond the built-in capacity is
refused.  The file name sorts last so that a run stopping at the first
failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, tol_for, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _static_scratch_call(case, h, d, out):
    desc = capi.make_desc(case.batch, case.heads, case.kv_heads, case.dk, case.dv, case.block_size, h["num_blocks"],
                          h["block_tables"].shape[1], case.q_dtype, case.kvd, case.qk_scale,
                          v_row_dim=case.dk if case.mla else case.dv)
    t = capi.pa_tensors(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], out, d["k_descale"], d["v_descale"],
                        d["k_offset"], d["v_offset"])
    lens = np.ascontiguousarray(h["context_lens"], dtype=np.int32)
    return capi.lib().atb_b200_pa_decode_static_scratch(ctypes.byref(desc), lens.ctypes.data, ctypes.byref(t),
                                                        capi.torch_stream_ptr())


def _scratch_status():
    st = ctypes.c_int32(-1)
    assert capi.lib().atb_b200_pa_static_scratch_status(capi.torch_stream_ptr(), ctypes.byref(st)) == 0
    return st.value


@pytest.mark.parametrize("case", [
    wl.Case("noalloc_gqa4_bf16", batch=12, heads=32, kv_heads=8, q_dtype="bf16", ctx=("uniform", 500, 6000), seed=41),
    wl.Case("noalloc_gqa15_fp16", batch=6, heads=30, kv_heads=2, q_dtype="fp16", ctx=("uniform", 88, 4000), seed=42),
    wl.Case("noalloc_int8_fp16", batch=7, heads=16, kv_heads=2, q_dtype="fp16", kv_dtype="int8", offsets=True,
            ctx=("uniform", 100, 5000), seed=43),
], ids=lambda c: c.name)
def test_static_scratch_matches_workspace_entry_point(case):
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    quant = dict(k_descale=d["k_descale"], v_descale=d["v_descale"], k_offset=d["k_offset"], v_offset=d["v_offset"])
    ref = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], h["context_lens"],
                               case.qk_scale, dv=case.dv, **quant)
    torch.cuda.synchronize()
    ref_f = ref.float().cpu().numpy()
    golden = oracle_out(case, h)
    for call in range(2):                      # two calls in a row share the scratch
        out = torch.zeros_like(ref)
        rc = _static_scratch_call(case, h, d, out)
        assert rc == 0, rc
        assert _scratch_status() == 0
        torch.cuda.synchronize()
        err = np.abs(out.float().cpu().numpy() - ref_f).max()
        assert err <= tol_for(case), (call, err)
        assert max_abs_err(wl.torch_to_host(out, case.q_dtype), golden, case.q_dtype) <= tol_for(case), call
    # a different, shorter workload right after: nothing stale may leak from the previous call
    h2 = dict(h, context_lens=np.maximum(h["context_lens"] // 3, 1).astype(np.int32))
    ref2 = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], h2["context_lens"],
                                case.qk_scale, dv=case.dv, **quant)
    out2 = torch.zeros_like(ref2)
    assert _static_scratch_call(case, h2, d, out2) == 0
    torch.cuda.synchronize()
    assert np.abs(out2.float().cpu().numpy() - ref2.float().cpu().numpy()).max() <= tol_for(case)
    assert max_abs_err(wl.torch_to_host(out2, case.q_dtype), oracle_out(case, h2), case.q_dtype) <= tol_for(case)


def test_static_scratch_reports_a_block_id_outside_the_cache():
    """The status word of the scratch: 2 after a call whose block table points outside the cache (the tile is replaced
    by zeros, nothing faults), 0 again after the next clean call."""
    case = wl.Case("noalloc_bad_block", batch=4, heads=16, kv_heads=4, q_dtype="bf16", ctx=("list", [300, 1000, 64, 129]), seed=44)
    h = wl.make_host_inputs(case)
    bad = dict(h, block_tables=h["block_tables"].copy())
    bad["block_tables"][1, 3] = h["num_blocks"] + 5
    d_bad = host_inputs_to_device(case, bad)
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.bfloat16, device="cuda")
    assert _static_scratch_call(case, bad, d_bad, out) == 0
    assert _scratch_status() == 2
    assert torch.isfinite(out.float()).all()
    d = host_inputs_to_device(case, h)
    assert _static_scratch_call(case, h, d, out) == 0
    assert _scratch_status() == 0
    assert max_abs_err(wl.torch_to_host(out, "bf16"), oracle_out(case, h), "bf16") <= tol_for(case)
    assert capi.lib().atb_b200_pa_static_scratch_status(capi.torch_stream_ptr(), None) == capi.ERROR_INVALID_PARAM


def test_static_scratch_refuses_a_stream_under_capture():
    """The plan is uploaded from the caller's stack, so a call may not become part of a captured graph:
    it is refused with ERROR_INVALID_PARAM while the stream is capturing, and nothing is enqueued."""
    case = wl.Case("noalloc_capture", batch=2, heads=8, kv_heads=2, q_dtype="bf16", ctx=("list", [200, 300]), seed=44)
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.bfloat16, device="cuda")
    assert _static_scratch_call(case, h, d, out) == 0      # the first call on the device: outside any capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        graph.capture_begin()
        try:
            rc = _static_scratch_call(case, h, d, out)
        finally:
            graph.capture_end()
    assert rc == capi.ERROR_INVALID_PARAM
    torch.cuda.synchronize()


def test_static_scratch_refuses_oversized_calls():
    # 1025 sequences: above the built-in batch limit; must be refused before anything is launched
    desc = capi.make_desc(1025, 8, 8, 128, 128, 128, 16, 1, "fp16", qk_scale=0.1)
    lens = np.ones(1025, dtype=np.int32)
    q = torch.zeros(1, device="cuda")
    t = capi.pa_tensors(q, q, q, q, q)
    rc = capi.lib().atb_b200_pa_decode_static_scratch(ctypes.byref(desc), lens.ctypes.data, ctypes.byref(t),
                                                      capi.torch_stream_ptr())
    assert rc == capi.ERROR_INVALID_PARAM
    torch.cuda.synchronize()
