"""Pins the C oracle against outputs of the reference's own Python golden (tests/golden/*.npz)."""
import hashlib
import os

import numpy as np
import pytest

import oracle
from golden_cases import GOLDEN_PA_CASES, GOLDEN_RAC_CASES, HERE, load_workloads, rac_inputs

wl = load_workloads()


def _digest(d):
    h = hashlib.sha256()
    for k in sorted(d):
        v = d[k]
        if isinstance(v, np.ndarray):
            h.update(k.encode())
            h.update(np.ascontiguousarray(v).tobytes())
    return h.hexdigest()


def ulp(dtype):
    return 2.0 ** -10 if dtype == "fp16" else 2.0 ** -7


@pytest.mark.parametrize("case", GOLDEN_PA_CASES, ids=lambda c: c.name)
def test_oracle_matches_reference_golden(case):
    fx = np.load(os.path.join(HERE, f"pa_{case.name}.npz"))
    d = wl.make_host_inputs(case)
    assert _digest(d) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    out, high = oracle.paged_attention(
        d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"], case.qk_scale, case.q_dtype,
        kv_dtype=case.kvd, dv=case.dv, k_descale=d.get("k_descale"), v_descale=d.get("v_descale"),
        k_offset=d.get("k_offset"), v_offset=d.get("v_offset"), want_high=True)
    ref_high = fx["out_high"]
    # fp32 path: only summation order differs between torch.matmul and the C loops
    np.testing.assert_allclose(high, ref_high, rtol=2e-4, atol=2e-5)
    got = wl.to_f32(out, case.q_dtype)
    ref = wl.to_f32(fx["out"], case.q_dtype)
    # rounded output: a couple of units in the last place (a 1-ulp fp32 difference in exp() can flip the
    # rounding of one probability, which moves the output by ulp(P) * |v|)
    tol = 2 * ulp(case.q_dtype) * np.maximum(np.abs(ref), 2.0 ** -6)
    assert np.all(np.abs(got - ref) <= tol), float(np.max(np.abs(got - ref)))
    # and nearly all elements bit-identical
    same = np.mean(out.view(np.uint16) == fx["out"].view(np.uint16))
    assert same > 0.95, same


@pytest.mark.parametrize("spec", GOLDEN_RAC_CASES, ids=lambda s: s["name"])
def test_oracle_reshape_and_cache_bit_exact(spec):
    fx = np.load(os.path.join(HERE, f"rac_{spec['name']}.npz"))
    inp = rac_inputs(spec)
    assert _digest(inp) == bytes(fx["input_sha256"]).decode()
    kdt = fx["key_cache"].dtype
    kc = np.zeros((spec["num_blocks"], spec["block_size"], spec["heads"], spec["dk"]), dtype=kdt)
    vc = np.zeros((spec["num_blocks"], spec["block_size"], spec["heads"], spec["dv"]), dtype=kdt)
    oracle.reshape_and_cache(inp["key"].view(kdt), inp["value"].view(kdt), kc, vc, inp["slot_mapping"])
    assert np.array_equal(kc.view(np.uint8), fx["key_cache"].view(np.uint8))
    assert np.array_equal(vc.view(np.uint8), fx["value_cache"].view(np.uint8))


def test_oracle_skips_empty_sequences():
    case = wl.Case("z", batch=3, heads=4, kv_heads=2, q_dtype="fp16", ctx=("list", [0, 5, 0]), seed=5)
    d = wl.make_host_inputs(case)
    out = np.full((3, 4, 128), 7.0, dtype=np.float16)
    oracle.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                           case.qk_scale, "fp16", out=out)
    assert np.all(out[0] == 7.0) and np.all(out[2] == 7.0) and not np.all(out[1] == 7.0)


# ------------------------------------------------------------------ cache-management siblings (bit-exact)

from golden_cases import GOLDEN_BLOCKCOPY_CASES, GOLDEN_PCL_CASES, blockcopy_inputs, pcl_inputs  # noqa: E402


def _bits(a):
    return a.view(np.uint16) if a.dtype == np.float16 else a


@pytest.mark.parametrize("spec", GOLDEN_BLOCKCOPY_CASES, ids=lambda s: s["name"])
def test_block_copy_oracle_matches_reference_golden(spec):
    fx = np.load(os.path.join(HERE, f"blockcopy_{spec['name']}.npz"))
    inp = blockcopy_inputs(spec)
    assert _digest(inp) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    k, v = oracle.cache_ops.block_copy(inp["k_cache"].copy(), inp["v_cache"].copy(), inp["src"], inp["dst"], inp["cum"])
    assert np.array_equal(_bits(k), _bits(fx["k_cache"])) and np.array_equal(_bits(v), _bits(fx["v_cache"]))
    assert not np.array_equal(_bits(k), _bits(inp["k_cache"]))          # the case does move data


@pytest.mark.parametrize("spec", GOLDEN_PCL_CASES, ids=lambda s: s["name"])
def test_paged_cache_load_oracle_matches_reference_golden(spec):
    fx = np.load(os.path.join(HERE, f"pcl_{spec['name']}.npz"))
    inp = pcl_inputs(spec)
    assert _digest(inp) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    total = int(inp["cu_lens"][-1])
    key = np.zeros((total,) + inp["k_cache"].shape[2:], dtype=inp["k_cache"].dtype)
    value = np.zeros((total,) + inp["v_cache"].shape[2:], dtype=inp["v_cache"].dtype)
    oracle.cache_ops.paged_cache_load(inp["k_cache"], inp["v_cache"], inp["block_tables"], inp["cu_lens"], key, value,
                                      seq_starts=inp["seq_starts"], cumulative=True)
    assert np.array_equal(_bits(key), _bits(fx["key"])) and np.array_equal(_bits(value), _bits(fx["value"]))
    # lengths instead of running totals give the same rows
    key2, value2 = np.zeros_like(key), np.zeros_like(value)
    oracle.cache_ops.paged_cache_load(inp["k_cache"], inp["v_cache"], inp["block_tables"], inp["lens"], key2, value2,
                                      seq_starts=inp["seq_starts"], cumulative=False)
    assert np.array_equal(_bits(key2), _bits(key)) and np.array_equal(_bits(value2), _bits(value))


# ------------------------------------------------------------------ PagedAttention with a mask / logN scale

from golden_cases import GOLDEN_PA_FEATURE_CASES, pa_mask  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_PA_FEATURE_CASES, ids=lambda s: s["case"].name)
def test_oracle_mask_and_logn_match_reference_golden(spec):
    case = spec["case"]
    fx = np.load(os.path.join(HERE, f"pa_{case.name}.npz"))
    d = wl.make_host_inputs(case)
    assert _digest(d) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    mask = pa_mask(spec)
    mask_f32 = None if mask is None else wl.to_f32(mask, case.q_dtype)
    logn = fx["logn"] if spec["logn"] else None
    out, high = oracle.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                                       case.qk_scale, case.q_dtype, want_high=True, mask=mask_f32, logn=logn)
    np.testing.assert_allclose(high, fx["out_high"], rtol=2e-4, atol=2e-5)
    got, ref = wl.to_f32(out, case.q_dtype), wl.to_f32(fx["out"], case.q_dtype)
    assert np.abs(got - ref).max() <= 2 * ulp(case.q_dtype) * max(1.0, float(np.abs(ref).max()))
    # the feature is not a no-op on this case
    plain = oracle.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                                   case.qk_scale, case.q_dtype)
    assert np.abs(wl.to_f32(plain, case.q_dtype) - ref).max() > 8 * ulp(case.q_dtype)


@pytest.mark.parametrize("case", [c for c in GOLDEN_PA_CASES if c.mla], ids=lambda c: c.name)
def test_split_cache_mla_oracle_matches_reference_golden(case):
    """MultiLatentAttention with the split cache: the reference's golden is the combined-cache one with
    query and cache split [512, 64] afterwards, so the same fixtures pin it."""
    fx = np.load(os.path.join(HERE, f"pa_{case.name}.npz"))
    d = wl.make_host_inputs(case)
    q, kc = d["q"], d["k_cache"]
    out = oracle.multi_latent_attention(np.ascontiguousarray(q[..., :512]), np.ascontiguousarray(q[..., 512:]),
                                        np.ascontiguousarray(kc[..., :512]), np.ascontiguousarray(kc[..., 512:]),
                                        d["block_tables"], d["context_lens"], case.qk_scale, case.q_dtype)
    combined = oracle.paged_attention(q, kc, None, d["block_tables"], d["context_lens"], case.qk_scale, case.q_dtype,
                                      dv=case.dv)
    assert np.array_equal(out.view(np.uint16), combined.view(np.uint16))
    got, ref = wl.to_f32(out, case.q_dtype), wl.to_f32(fx["out"], case.q_dtype)
    assert np.all(np.abs(got - ref) <= 2 * ulp(case.q_dtype) * np.maximum(np.abs(ref), 2.0 ** -6))


# ------------------------------------------------------------------ fused RMSNorm + RoPE + cache write

from golden_cases import GOLDEN_NRR_CASES, nrr_inputs  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_NRR_CASES, ids=lambda s: s["name"])
def test_norm_rope_reshape_oracle_matches_reference_golden(spec):
    fx = np.load(os.path.join(HERE, f"nrr_{spec['name']}.npz"))
    inp = nrr_inputs(spec)
    assert _digest(inp) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    store = np.float16 if spec["dtype"] == "fp16" else np.uint16
    cache = np.zeros((spec["blocks"], spec["block_size"], 1, spec["dx"] + spec["dr"]), dtype=store)
    oracle.cache_ops.norm_rope_reshape(inp["x"], inp["gamma"], inp["key_rope"], inp["cos"], inp["sin"],
                                       inp["slot_mapping"], cache, spec["eps"], spec["dtype"])
    if spec["dtype"] == "fp16":
        # the reference rounds to float16 itself: bit-exact
        assert np.array_equal(cache.view(np.uint16), fx["key_cache"].view(np.uint16))
    else:
        # the reference keeps float32 rows for bf16 inputs: ours are those rows rounded to bf16 (half an ulp)
        got, ref = wl.to_f32(cache, "bf16"), fx["key_cache"]
        assert np.all(np.abs(got - ref) <= 2.0 ** -8 * np.maximum(np.abs(ref), 2.0 ** -20))
    assert np.count_nonzero(cache) > 0


# ------------------------------------------------------------------ PagedAttention, parallel decoding

from golden_cases import GOLDEN_PA_SPEC_CASES, spec_inputs  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_PA_SPEC_CASES, ids=lambda s: s["case"].name)
def test_oracle_parallel_decoding_matches_reference_golden(spec):
    """The reference's lookahead golden rounds the scores and the output to fp16 between its steps, so it is matched
    at that test's own threshold, 2^-8 * max(1, |golden|)
    (tests/apitest/kernelstest/mix/test_paged_attention_lookahead.py:49-55)."""
    case = spec["case"]
    fx = np.load(os.path.join(HERE, f"pa_{case.name}.npz"))
    d = spec_inputs(spec)
    assert _digest(d) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    out = oracle.paged_attention_spec(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["q_lens"],
                                      d["context_lens"], case.qk_scale, case.q_dtype, wl.to_f32(d["mask"], case.q_dtype),
                                      mask_rows_are_tokens=spec["mask"] == "spec")
    got, ref = wl.to_f32(out, case.q_dtype), wl.to_f32(fx["out"], case.q_dtype)
    assert np.all(np.abs(got - ref) <= 2.0 ** -8 * np.maximum(1.0, np.abs(ref)))
    # the mask matters: without it the later tokens of a sequence would see their successors
    owner = np.repeat(np.arange(case.batch), d["q_lens"])
    unmasked = oracle.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"][owner],
                                      d["context_lens"][owner], case.qk_scale, case.q_dtype)
    assert np.abs(wl.to_f32(unmasked, case.q_dtype) - ref).max() > 2.0 ** -5


@pytest.mark.parametrize("case", [c for c in GOLDEN_PA_CASES if c.mla], ids=lambda c: c.name)
def test_oracle_lse_matches_reference_golden(case):
    """The log-sum-exp output of MultiLatentAttention (CALC_TYPE_RING) against ref_masked_attention of the reference's
    split-cache kernel test: same fp32 arithmetic up to summation order, so at most one unit in the last place."""
    fx = np.load(os.path.join(HERE, f"mla_lse_{case.name}.npz"))
    d = wl.make_host_inputs(case)
    assert _digest(d) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    lse = oracle.attention_lse(d["q"], d["k_cache"], d["block_tables"], d["context_lens"], case.qk_scale, case.q_dtype)
    got, ref = wl.to_f32(lse, case.q_dtype), wl.to_f32(fx["lse"], case.q_dtype)
    assert got.shape == (case.batch, case.heads, 1)
    assert np.all(np.abs(got - ref) <= ulp(case.q_dtype) * np.maximum(np.abs(ref), 1.0))
    assert np.mean(got == ref) > 0.9


from golden_cases import GOLDEN_MLA_MTP_CASES, mla_mtp_inputs  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_MLA_MTP_CASES, ids=lambda s: s["case"].name)
def test_oracle_mla_parallel_decoding_matches_reference_golden(spec):
    """MultiLatentAttention with CALC_TYPE_SPEC(_AND_RING): output and log-sum-exp of every query token against the
    golden of the reference's MTP split-cache kernel test (fp32 arithmetic like the oracle's)."""
    case = spec["case"]
    fx = np.load(os.path.join(HERE, f"pa_{case.name}.npz"))
    d = mla_mtp_inputs(spec)
    assert _digest(d) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    mask = wl.to_f32(d["mask"], case.q_dtype) if spec["mask"] else None
    out, lse = oracle.paged_attention_spec(d["q"], d["k_cache"], None, d["block_tables"], d["q_lens"], d["context_lens"],
                                           case.qk_scale, case.q_dtype, mask, mask_rows_are_tokens=True, dv=case.dv,
                                           want_lse=True)
    got, ref = wl.to_f32(out, case.q_dtype), wl.to_f32(fx["out"], case.q_dtype)
    assert np.all(np.abs(got - ref) <= 2 * ulp(case.q_dtype) * np.maximum(np.abs(ref), 2.0 ** -6))
    gl, rl = wl.to_f32(lse, case.q_dtype), wl.to_f32(fx["lse"], case.q_dtype)
    assert np.all(np.abs(gl - rl) <= ulp(case.q_dtype) * np.maximum(np.abs(rl), 1.0))


# ------------------------------------------------------------------ int8 Q, K and V (QUANT_QKV online / offline)

from golden_cases import GOLDEN_PA_QUANT_CASES, quant_inputs  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_PA_QUANT_CASES, ids=lambda s: s["name"])
def test_oracle_qkv_quant_matches_reference_golden(spec):
    """The restated int32 matmuls, per-tile quantisation of P and split merge against the reference's own golden
    (test_paged_attention_common.py:104-110, 142-227), run with the same tile and split sizes."""
    fx = np.load(os.path.join(HERE, f"pa_{spec['name']}.npz"))
    d = quant_inputs(spec)
    dig = {k: v for k, v in d.items() if isinstance(v, np.ndarray)}
    assert _digest(dig) == bytes(fx["input_sha256"]).decode(), "seeded inputs changed; regenerate the fixtures"
    dt = spec["out_dtype"]
    out = oracle.paged_attention_qkv_quant(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                                           d["k_descale"], d["v_descale"], 1.0 / np.sqrt(128.0), dt, p_scale=d["p_scale"],
                                           tile_tokens=spec["tile"], split_tokens=spec["split"])
    got, ref = wl.to_f32(out, dt), wl.to_f32(fx["out"], dt)
    scale = max(float(np.abs(ref).max()), 1e-6)
    assert np.abs(got - ref).max() <= 2 * ulp(dt) * scale
    assert (got == ref).mean() >= 0.95
    # the quantisation of P is not a no-op: another tile size moves the result (a little)
    other = oracle.paged_attention_qkv_quant(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                                             d["k_descale"], d["v_descale"], 1.0 / np.sqrt(128.0), dt, p_scale=d["p_scale"],
                                             tile_tokens=16, split_tokens=spec["split"])
    diff = np.abs(wl.to_f32(other, dt) - ref).max()
    assert 0 < diff <= 1e-2 * scale
