"""Shared helpers of the tests: package loading, host<->device movement, running a case on the GPU."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
wl, capi = pkg.workloads, pkg.capi

# tolerances of the parity contract: max-abs error against the reference golden
TOL = {"fp16": 2e-3, "bf16": 8e-3, "int8": 1e-2}


def tol_for(case):
    return TOL["int8"] if case.kvd == "int8" else TOL[case.q_dtype]


def to_dev(a, dtype, device="cuda"):
    import torch
    if a is None:
        return None
    if dtype == "bf16":
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(a).to(device)


def host_inputs_to_device(case, h, device="cuda"):
    import torch
    d = {"q": to_dev(h["q"], case.q_dtype, device), "k_cache": to_dev(h["k_cache"], case.kvd, device),
         "v_cache": to_dev(h["v_cache"], case.kvd, device),
         "block_tables": torch.from_numpy(h["block_tables"]).to(device)}
    for k in ("k_descale", "v_descale", "k_offset", "v_offset"):
        d[k] = torch.from_numpy(h[k]).to(device) if h.get(k) is not None else None
    return d


def run_gpu_case(case, h, kernel=0, out_fill=None):
    """Runs one decode step through the kernel-level C ABI; returns (out numpy, plan info)."""
    import torch
    d = host_inputs_to_device(case, h)
    out = None
    if out_fill is not None:
        tdt = wl.torch_dtype(case.q_dtype)
        out = torch.full((case.batch, case.heads, case.dv), out_fill, dtype=tdt, device="cuda")
    out, plan, ws = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], h["context_lens"],
                                         case.qk_scale, dv=case.dv, k_descale=d["k_descale"],
                                         v_descale=d["v_descale"], k_offset=d["k_offset"], v_offset=d["v_offset"],
                                         out=out, kernel=kernel, return_plan=True)
    torch.cuda.synchronize()
    status = plan.device_status(ws.data_ptr(), capi.torch_stream_ptr())
    assert status == 0, f"device status {status}"
    info = plan.info
    return wl.torch_to_host(out, case.q_dtype), info


def oracle_out(case, h, out=None, want_high=False):
    import oracle
    return oracle.paged_attention(h["q"], h["k_cache"], h["v_cache"], h["block_tables"], h["context_lens"],
                                  case.qk_scale, case.q_dtype, kv_dtype=case.kvd, dv=case.dv,
                                  k_descale=h.get("k_descale"), v_descale=h.get("v_descale"),
                                  k_offset=h.get("k_offset"), v_offset=h.get("v_offset"), out=out, want_high=want_high)


def max_abs_err(a, b, dtype):
    """Largest |a - b|, not counting differences of one unit in the last place where that unit is
    already coarser than the parity tolerance (bf16 spacing is 2^-6 for |x| in [2,4): a short context
    returns near-copies of V rows of that size, and one differently rounded product flips one ulp)."""
    if not a.size:
        return 0.0
    fa, fb = wl.to_f32(a, dtype), wl.to_f32(b, dtype)
    diff = np.abs(fa - fb)
    mant = 10 if dtype == "fp16" else 7
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(fb), 2.0 ** -14))) - mant)
    one_ulp_coarse = (diff <= ulp * 1.001) & (ulp > TOL[dtype])
    return float(np.max(np.where(one_ulp_coarse, 0.0, diff)))
