"""The opt-in MLA kernel that runs a token range on a pair of CTAs (ATB_B200_MLA_PAIR=1): parity with the oracle.

The variable is read when a plan is made, so each test sets it for its own plans only.  The default MLA kernel is
covered by test_parity_gpu.py; the cases here are the ones that exercise what differs in the pair kernel: a single tile,
ragged tails (rows of V past the end of a range), more than one token range per pair, fewer heads than the 128 rows of a
pair, 128 and 160 heads (one and two head columns), split sequences merged by the combine kernel, a block size of one
TMA box, the split latent / rope cache, and a block table that points outside the cache.  Golden: multi-latent attention of the reference's Python test
(tests/apitest/kernelstest/mix/test_paged_attention_common.py:229-366 of the reference) through the oracle.
"""
import numpy as np
import pytest

from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, tol_for, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

KERNEL_MLA = 3

_CASES = [
    wl.Case("pair_8h_1seq_128", batch=1, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True, ctx=("list", [128]), seed=1),
    wl.Case("pair_8h_ragged", batch=4, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True, ctx=("list", [1, 64, 65, 300]),
            seed=2),
    wl.Case("pair_64h", batch=3, heads=64, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True, ctx=("list", [129, 700, 128]), seed=3),
    wl.Case("pair_128h_split", batch=2, heads=128, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True, ctx=("list", [9000, 5000]),
            seed=4),
    wl.Case("pair_16h_bs64", batch=3, heads=16, kv_heads=1, dk=576, dv=512, block_size=64, q_dtype="bf16", mla=True,
            ctx=("list", [500, 63, 2000]), seed=5),
    wl.Case("pair_160h_two_columns", batch=2, heads=160, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True, ctx=("list", [1500, 333]),
            seed=7),
    wl.Case("pair_40h_empty_seq", batch=4, heads=40, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True, ctx=("list", [0, 257, 0, 31]),
            seed=6),
]


@pytest.fixture
def pair_kernel(monkeypatch):
    monkeypatch.setenv("ATB_B200_MLA_PAIR", "1")


def _run(case, h, d):
    out, plan, ws = capi.paged_attention(d["q"], d["k_cache"], None, d["block_tables"], h["context_lens"], case.qk_scale, dv=case.dv,
                                         return_plan=True)
    torch.cuda.synchronize()
    return out, plan, plan.device_status(ws.data_ptr(), capi.torch_stream_ptr())


@pytest.mark.parametrize("case", _CASES, ids=lambda c: c.name)
def test_pair_kernel_matches_oracle(case, pair_kernel):
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    out, plan, status = _run(case, h, d)
    assert plan.info.kernel == KERNEL_MLA
    assert plan.info.num_ctas % 2 == 0, "the pair kernel launches whole pairs"
    assert status == 0
    got = wl.torch_to_host(out, "bf16")
    ref = oracle_out(case, h)
    live = np.asarray(h["context_lens"]) > 0
    assert max_abs_err(got[live], ref[live], "bf16") <= tol_for(case)


def test_pair_kernel_is_deterministic_and_matches_default_kernel(monkeypatch):
    """Same inputs through the default MLA kernel and the pair kernel: both within tolerance of each other, and the pair
    kernel bit-identical from launch to launch."""
    case = _CASES[3]
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    monkeypatch.delenv("ATB_B200_MLA_PAIR", raising=False)
    base, plan0, st0 = _run(case, h, d)
    monkeypatch.setenv("ATB_B200_MLA_PAIR", "1")
    a, plan1, st1 = _run(case, h, d)
    b, _, st2 = _run(case, h, d)
    assert st0 == 0 and st1 == 0 and st2 == 0
    assert plan1.info.num_ctas != plan0.info.num_ctas or plan1.info.num_ctas % 2 == 0
    assert torch.equal(a, b)
    assert max_abs_err(wl.torch_to_host(a, "bf16"), wl.torch_to_host(base, "bf16"), "bf16") <= 2 * tol_for(case)


def test_pair_kernel_reports_a_block_id_outside_the_cache(pair_kernel):
    case = _CASES[2]
    h = wl.make_host_inputs(case)
    h["block_tables"] = h["block_tables"].copy()
    h["block_tables"][1, 2] = h["num_blocks"] + 7
    d = host_inputs_to_device(case, h)
    out, plan, status = _run(case, h, d)
    assert status == 2
    # the other sequences are untouched by the bad entry
    got = wl.torch_to_host(out, "bf16")
    ref = oracle_out(case, wl.make_host_inputs(case))
    assert max_abs_err(got[[0, 2]], ref[[0, 2]], "bf16") <= tol_for(case)
    assert np.isfinite(wl.to_f32(got, "bf16")).all()


def test_pair_kernel_with_the_split_latent_and_rope_cache(pair_kernel):
    """rope_dim = 64: query and cache given as latent [.., 512] and rope [.., 64] tensors; the rope halves of the two CTAs
    come from the second tensor map.  Same arithmetic as the combined cache: identical bits."""
    case = _CASES[4]
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    combined, _, st = _run(case, h, d)
    assert st == 0
    q, kc = d["q"], d["k_cache"]
    q_nope, q_rope = q[..., :512].contiguous(), q[..., 512:].contiguous()
    ct_kv, k_rope = kc[..., :512].contiguous(), kc[..., 512:].contiguous()
    out = torch.zeros((case.batch, case.heads, 512), dtype=q.dtype, device="cuda")
    desc = capi.make_desc(case.batch, case.heads, 1, 576, 512, case.block_size, kc.shape[0], d["block_tables"].shape[1], "bf16",
                          qk_scale=case.qk_scale, v_row_dim=512, rope_dim=64)
    plan = capi.PaPlan(desc, h["context_lens"])
    assert plan.info.kernel == KERNEL_MLA and plan.info.num_ctas % 2 == 0
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(q_nope, ct_kv, ct_kv, d["block_tables"], out, q_rope=q_rope, k_rope_cache=k_rope)
    plan.launch(tens, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
    assert torch.equal(out, combined)
    assert max_abs_err(wl.torch_to_host(out, "bf16"), oracle_out(case, h), "bf16") <= tol_for(case)
