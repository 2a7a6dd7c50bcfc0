"""Parity of the CUDA path against the CPU oracle and the reference-golden fixtures, through the C ABI.

Tolerances (max-abs error against the reference golden): fp16 2e-3, bf16 8e-3, int8 cache 1e-2;
ReshapeAndCache must be bit-exact.
"""
import ctypes
import os

import numpy as np
import pytest

import oracle
from golden_cases import GOLDEN_PA_CASES, GOLDEN_RAC_CASES, HERE as GOLDEN_DIR, rac_inputs
from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, run_gpu_case, to_dev, tol_for, wl

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _kernels_for(case):
    ks = [capi.KERNEL_AUTO]
    if case.dk == case.dv and case.dk in (64, 128, 256) and case.block_size in (16, 32, 64, 128, 256) and not case.mla:
        ks.append(capi.KERNEL_GENERIC)                 # the tiled kernel runs these: check the CUDA-core one too
    if case.mla and case.batch * case.heads <= 4096:
        ks.append(capi.KERNEL_GENERIC)
    return ks


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("case", GOLDEN_PA_CASES, ids=lambda c: c.name)
def test_attention_matches_reference_golden(case):
    fx = np.load(os.path.join(GOLDEN_DIR, f"pa_{case.name}.npz"))
    h = wl.make_host_inputs(case)
    for kernel in _kernels_for(case):
        out, info = run_gpu_case(case, h, kernel=kernel)
        err = max_abs_err(out, fx["out"], case.q_dtype)
        assert err <= tol_for(case), (kernel, info.kernel, err)


@pytest.mark.parametrize("spec", GOLDEN_RAC_CASES, ids=lambda s: s["name"])
def test_reshape_and_cache_matches_reference_golden(spec):
    fx = np.load(os.path.join(GOLDEN_DIR, f"rac_{spec['name']}.npz"))
    inp = rac_inputs(spec)
    dt = spec["dtype"]
    key, value = to_dev(inp["key"], dt), to_dev(inp["value"], dt)
    tdt = wl.torch_dtype(dt)
    kc = torch.zeros((spec["num_blocks"], spec["block_size"], spec["heads"], spec["dk"]), dtype=tdt, device="cuda")
    vc = torch.zeros((spec["num_blocks"], spec["block_size"], spec["heads"], spec["dv"]), dtype=tdt, device="cuda")
    capi.reshape_and_cache(key, value, kc, vc, torch.from_numpy(inp["slot_mapping"]).cuda())
    torch.cuda.synchronize()
    assert np.array_equal(wl.torch_to_host(kc, dt).view(np.uint8), fx["key_cache"].view(np.uint8))
    assert np.array_equal(wl.torch_to_host(vc, dt).view(np.uint8), fx["value_cache"].view(np.uint8))


# ------------------------------------------------------------------ seeded cases vs the oracle
@pytest.mark.parametrize("case", wl.SMALL_CASES, ids=lambda c: c.name)
def test_attention_matches_oracle_small(case):
    h = wl.make_host_inputs(case)
    ref = oracle_out(case, h, out=np.full((case.batch, case.heads, case.dv), 0, dtype=h["q"].dtype))
    for kernel in _kernels_for(case):
        out, info = run_gpu_case(case, h, kernel=kernel, out_fill=0.0)
        err = max_abs_err(out, ref, case.q_dtype)
        assert err <= tol_for(case), (kernel, info.kernel, err)


def test_empty_sequences_leave_output_untouched():
    case = [c for c in wl.SMALL_CASES if c.name == "zero_and_one_ctx"][0]
    h = wl.make_host_inputs(case)
    out, _ = run_gpu_case(case, h, out_fill=3.0)
    f = wl.to_f32(out, case.q_dtype)
    lens = h["context_lens"]
    for b in range(case.batch):
        if lens[b] == 0:
            assert np.all(f[b] == 3.0)
        else:
            assert not np.all(f[b] == 3.0)
    # ctx == 1: the output is exactly the single V row
    b = int(np.where(lens == 1)[0][0])
    blk = h["block_tables"][b, 0]
    v = wl.to_f32(h["v_cache"][blk, 0], case.q_dtype)      # [kv_heads, D]
    group = case.heads // case.kv_heads
    assert np.array_equal(f[b], np.repeat(v, group, axis=0))


@pytest.mark.parametrize("idx", [0, 1, 2, 3, 4], ids=lambda i: wl.CONFIGS[i].name)
def test_benchmark_config_full_size_matches_oracle(idx):
    case = wl.CONFIGS[idx]
    d = wl.make_device_inputs(case, "cuda")
    lens = d["context_lens_host"]
    # ReshapeAndCache of the step's new tokens first, as a serving step does
    capi.reshape_and_cache(d["new_k"], d["new_v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    out = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], lens, case.qk_scale,
                               dv=case.dv, k_descale=d.get("k_descale"), v_descale=d.get("v_descale"))
    torch.cuda.synchronize()
    hk = wl.torch_to_host(d["k_cache"], case.kvd)
    hv = None if case.mla else wl.torch_to_host(d["v_cache"], case.kvd)
    # the scatter is checked bit-exactly through its effect: the new rows sit at their slots
    nk = wl.torch_to_host(d["new_k"], case.kvd)
    slots = d["slot_mapping_host"]
    flat = hk.reshape(-1, case.kv_heads, case.dk)
    assert np.array_equal(flat[slots[slots >= 0]], nk[slots >= 0])
    ref = oracle.paged_attention(wl.torch_to_host(d["q"], case.q_dtype), hk, hv, d["block_tables_host"], lens,
                                 case.qk_scale, case.q_dtype, kv_dtype=case.kvd, dv=case.dv,
                                 k_descale=None if "k_descale" not in d else d["k_descale"].cpu().numpy(),
                                 v_descale=None if "v_descale" not in d else d["v_descale"].cpu().numpy())
    err = max_abs_err(wl.torch_to_host(out, case.q_dtype), ref, case.q_dtype)
    assert err <= tol_for(case), err


# ------------------------------------------------------------------ size-independent properties
def test_block_permutation_invariance_is_bit_exact():
    """Moving the pages in memory and permuting block_tables accordingly must not change a bit."""
    case = wl.CONFIGS[1]
    d = wl.make_device_inputs(case, "cuda")
    lens = d["context_lens_host"]
    out1 = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], lens, case.qk_scale)
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    nb = d["k_cache"].shape[0]
    perm = torch.randperm(nb, generator=g, device="cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nb, device="cuda")
    k2, v2 = d["k_cache"][perm].contiguous(), d["v_cache"][perm].contiguous()   # new[i] = old[perm[i]]
    bt = d["block_tables"].long()
    bt2 = torch.where(bt >= 0, inv[bt.clamp(min=0)], bt).int().contiguous()
    out2 = capi.paged_attention(d["q"], k2, v2, bt2, lens, case.qk_scale)
    torch.cuda.synchronize()
    assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))


def test_constant_value_rows_give_that_constant():
    """softmax weights sum to 1: with V[t, :] = c for every token the output is c (up to rounding)."""
    case = wl.CONFIGS[3]
    case = wl.Case("c4_small", batch=32, heads=64, kv_heads=8, q_dtype="bf16",
                   ctx=("lognormal", 7.6, 1.0, 16, 32768), seed=1004)
    d = wl.make_device_inputs(case, "cuda")
    c = torch.linspace(-2, 2, 128, device="cuda").to(torch.bfloat16)
    d["v_cache"][:] = c
    out = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens_host"],
                               case.qk_scale)
    torch.cuda.synchronize()
    err = (out.float() - c.float()).abs().max().item()
    assert err <= 8e-3 * 2, err


def test_split_and_unsplit_agree():
    """The same long sequences planned for 148 SMs (split-KV + combine) and for 1 SM (few cuts)."""
    case = wl.Case("long", batch=3, heads=32, kv_heads=8, q_dtype="fp16", ctx=("list", [9000, 130, 20000]), seed=31)
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    outs = []
    for sm in (148, 1):
        desc = capi.make_desc(case.batch, case.heads, case.kv_heads, 128, 128, 128, h["num_blocks"],
                              h["block_tables"].shape[1], "fp16", qk_scale=case.qk_scale, sm_count=sm)
        plan = capi.PaPlan(desc, h["context_lens"])
        out = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], h["context_lens"],
                                   case.qk_scale, plan=plan)
        torch.cuda.synchronize()
        outs.append(out.float().cpu().numpy())
    assert np.abs(outs[0] - outs[1]).max() <= 1e-3
    ref = wl.to_f32(oracle_out(case, h), "fp16")
    assert np.abs(outs[0] - ref).max() <= 2e-3


def test_plan_reuse_over_decode_steps():
    """A plan updated in place for growing context_lens keeps giving oracle results."""
    case = wl.Case("steps", batch=5, heads=16, kv_heads=4, q_dtype="bf16", ctx=("list", [126, 127, 128, 255, 600]),
                   seed=33, pool_blocks=40)
    h = wl.make_host_inputs(case)
    # give every sequence room for three more tokens
    h["block_tables"] = np.concatenate([h["block_tables"], np.full((5, 1), -1, np.int32)], axis=1)
    used = set(h["block_tables"][h["block_tables"] >= 0].tolist())
    free = [b for b in range(h["num_blocks"]) if b not in used]
    for b in range(5):
        n = (h["context_lens"][b] + 127) // 128
        h["block_tables"][b, n] = free.pop()
    d = host_inputs_to_device(case, h)
    lens = h["context_lens"].copy()
    plan, ws = None, None
    for step in range(3):
        out, plan, ws = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], lens,
                                             case.qk_scale, plan=plan, workspace=ws, return_plan=True)
        torch.cuda.synchronize()
        hh = dict(h, context_lens=lens)
        ref = oracle_out(case, hh)
        assert max_abs_err(wl.torch_to_host(out, "bf16"), ref, "bf16") <= 8e-3
        lens = lens + 1
        plan.update(lens)


def test_bad_block_id_is_reported_not_faulted():
    """A block id outside the cache (a caller bug) must not fault the GPU: the generic kernel skips the
    token, the TMA kernels load a zero tile in its place, and all of them set the status word to 2."""
    case = wl.Case("badblk", batch=2, heads=8, kv_heads=2, dk=96, dv=96, block_size=16, q_dtype="fp16",
                   ctx=("list", [40, 33]), seed=71)
    h = wl.make_host_inputs(case)
    h["block_tables"] = h["block_tables"].copy()
    h["block_tables"][1, 1] = h["num_blocks"] + 5
    d = host_inputs_to_device(case, h)
    out, plan, ws = capi.paged_attention(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], h["context_lens"],
                                         case.qk_scale, return_plan=True)
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 2
    assert torch.isfinite(out.float()).all()
    case2 = wl.Case("badblk128", batch=2, heads=8, kv_heads=2, q_dtype="bf16", ctx=("list", [300, 200]), seed=72)
    h2 = wl.make_host_inputs(case2)
    h2["block_tables"] = h2["block_tables"].copy()
    h2["block_tables"][0, 1] = -1
    d2 = host_inputs_to_device(case2, h2)
    out2, plan2, ws2 = capi.paged_attention(d2["q"], d2["k_cache"], d2["v_cache"], d2["block_tables"], h2["context_lens"],
                                            case2.qk_scale, return_plan=True)
    torch.cuda.synchronize()
    assert plan2.info.kernel == capi.KERNEL_TMA_MMA
    assert plan2.device_status(ws2.data_ptr(), capi.torch_stream_ptr()) == 2
    assert torch.isfinite(out2.float()).all()
    # the int8 and the MLA kernels report the same caller error
    for case3 in (wl.Case("badblk_i8", batch=2, heads=8, kv_heads=2, q_dtype="fp16", kv_dtype="int8",
                          ctx=("list", [300, 200]), seed=73),
                  wl.Case("badblk_mla", batch=2, heads=16, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                          ctx=("list", [300, 200]), seed=74)):
        h3 = wl.make_host_inputs(case3)
        h3["block_tables"] = h3["block_tables"].copy()
        h3["block_tables"][1, 0] = h3["num_blocks"]
        d3 = host_inputs_to_device(case3, h3)
        out3, plan3, ws3 = capi.paged_attention(d3["q"], d3["k_cache"], d3["v_cache"], d3["block_tables"],
                                                h3["context_lens"], case3.qk_scale, dv=case3.dv,
                                                k_descale=d3["k_descale"], v_descale=d3["v_descale"], return_plan=True)
        torch.cuda.synchronize()
        assert plan3.info.kernel != capi.KERNEL_GENERIC, case3.name
        assert plan3.device_status(ws3.data_ptr(), capi.torch_stream_ptr()) == 2, case3.name
        assert torch.isfinite(out3.float()).all(), case3.name


def _random_cases(n, seed, block_sizes=(128,)):
    """Seeded random shapes around the tile / block / split boundaries of the tiled kernels."""
    rng = np.random.default_rng(seed)
    bs_rng = np.random.default_rng(seed + 7)
    cases = []
    boundary = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257, 511, 512, 513, 1000, 2047, 2048,
                2049, 4097]
    for i in range(n):
        kind = i % 3
        kv_heads = int(rng.choice([1, 2, 4, 8]))
        group = int(rng.choice([1, 2, 3, 4, 5, 8]))
        batch = int(rng.integers(1, 24))
        lens = [int(rng.choice(boundary)) if rng.random() < 0.6 else int(rng.integers(1, 6000)) for _ in range(batch)]
        if rng.random() < 0.3:
            lens[int(rng.integers(0, batch))] = 0
        kw = dict(batch=batch, heads=kv_heads * group, kv_heads=kv_heads, ctx=("list", lens), seed=1000 + i,
                  block_size=int(bs_rng.choice(block_sizes)))
        if kind == 0:
            cases.append(wl.Case(f"rand{i}_bs{kw['block_size']}_bf16", q_dtype="bf16", **kw))
        elif kind == 1:
            cases.append(wl.Case(f"rand{i}_bs{kw['block_size']}_fp16", q_dtype="fp16", **kw))
        else:
            cases.append(wl.Case(f"rand{i}_bs{kw['block_size']}_int8", q_dtype=str(rng.choice(["fp16", "bf16"])), kv_dtype="int8",
                                 offsets=bool(rng.random() < 0.5), **kw))
    return cases


@pytest.mark.parametrize("case", _random_cases(24, 2024) + _random_cases(24, 4242, (16, 32, 64, 256)),
                         ids=lambda c: c.name)
def test_randomized_shapes_match_oracle(case):
    h = wl.make_host_inputs(case)
    ref = oracle_out(case, h, out=np.zeros((case.batch, case.heads, case.dv), dtype=h["q"].dtype))
    out, info = run_gpu_case(case, h, out_fill=0.0)
    assert info.kernel == capi.KERNEL_TMA_MMA
    err = max_abs_err(out, ref, case.q_dtype)
    assert err <= tol_for(case), err


@pytest.mark.parametrize("heads,lens", [(8, [1, 64, 65, 4000]), (128, [300, 6000, 63]), (64, [129, 128, 127]),
                                         (16, [5000]), (192, [100, 2500])])
def test_randomized_mla_shapes_match_oracle(heads, lens):
    case = wl.Case(f"mla_rand_h{heads}", batch=len(lens), heads=heads, kv_heads=1, dk=576, dv=512, q_dtype="bf16",
                   mla=True, ctx=("list", lens), seed=500 + heads)
    h = wl.make_host_inputs(case)
    ref = oracle_out(case, h)
    out, info = run_gpu_case(case, h)
    assert info.kernel == capi.KERNEL_MLA_TC5
    assert max_abs_err(out, ref, "bf16") <= 8e-3


# Shapes the tiled kernel took over from the CUDA-core one: head sizes 64 and 256 (one, two or four 64-element TMA
# boxes per row) and more than 8 query heads per kv head (one CTA column per 8 heads), down to the reference's own
# regression shapes (tests/apitest/kernelstest/mix/test_paged_attention_common.py:1928 gqa_2 127 / 1, :1977 gqa_3
# 30 / 2 of the reference), with split sequences, small blocks and empty sequences.
_WIDE_CASES = [
    wl.Case("d64_mha_fp16", batch=5, heads=8, kv_heads=8, dk=64, dv=64, q_dtype="fp16", ctx=("list", [1, 63, 64, 700, 3000]), seed=301),
    wl.Case("d64_gqa4_bf16_bs16", batch=4, heads=16, kv_heads=4, dk=64, dv=64, block_size=16, q_dtype="bf16",
            ctx=("list", [17, 0, 5000, 129]), seed=302),
    wl.Case("d256_mha_bf16_bs64", batch=4, heads=4, kv_heads=4, dk=256, dv=256, block_size=64, q_dtype="bf16",
            ctx=("list", [1, 65, 2500, 640]), seed=303),
    wl.Case("d256_gqa8_fp16_bs32_split", batch=2, heads=16, kv_heads=2, dk=256, dv=256, block_size=32, q_dtype="fp16",
            ctx=("list", [9000, 31]), seed=304),
    wl.Case("gqa16_bf16_split", batch=3, heads=32, kv_heads=2, q_dtype="bf16", ctx=("list", [12000, 64, 300]), seed=305),
    wl.Case("gqa15_fp16_long", batch=4, heads=30, kv_heads=2, q_dtype="fp16", ctx=("list", [88, 4000, 0, 1025]), seed=306),
    wl.Case("gqa127_fp16_long", batch=3, heads=127, kv_heads=1, q_dtype="fp16", ctx=("list", [88, 2000, 130]), seed=307),
    wl.Case("gqa12_int8_fp16", batch=3, heads=24, kv_heads=2, q_dtype="fp16", kv_dtype="int8", offsets=True,
            ctx=("list", [300, 5000, 64]), seed=308),
    wl.Case("gqa9_d64_bf16", batch=2, heads=18, kv_heads=2, dk=64, dv=64, q_dtype="bf16", ctx=("list", [513, 77]), seed=309),
    # head sizes between the geometries: multiples of 16 run padded (TMA zero-fills the part of a box past the row)
    wl.Case("d96_gqa4_bf16_split", batch=3, heads=16, kv_heads=4, dk=96, dv=96, q_dtype="bf16", ctx=("list", [9000, 1, 700]), seed=310),
    wl.Case("d96_mha_fp16_bs16", batch=4, heads=6, kv_heads=6, dk=96, dv=96, block_size=16, q_dtype="fp16",
            ctx=("list", [15, 16, 17, 1200]), seed=311),
    wl.Case("d80_gqa2_fp16", batch=3, heads=8, kv_heads=4, dk=80, dv=80, q_dtype="fp16", ctx=("list", [333, 64, 2049]), seed=312),
    wl.Case("d112_gqa8_bf16_bs32", batch=2, heads=16, kv_heads=2, dk=112, dv=112, block_size=32, q_dtype="bf16",
            ctx=("list", [5000, 90]), seed=313),
    wl.Case("d32_mha_fp16", batch=3, heads=4, kv_heads=4, dk=32, dv=32, q_dtype="fp16", ctx=("list", [70, 1, 900]), seed=314),
    wl.Case("d48_gqa3_bf16_bs64", batch=2, heads=6, kv_heads=2, dk=48, dv=48, block_size=64, q_dtype="bf16", ctx=("list", [640, 65]),
            seed=315),
    wl.Case("d160_mha_bf16", batch=3, heads=4, kv_heads=4, dk=160, dv=160, q_dtype="bf16", ctx=("list", [2, 1500, 129]), seed=316),
    wl.Case("d192_gqa4_fp16_bs64_split", batch=2, heads=8, kv_heads=2, dk=192, dv=192, block_size=64, q_dtype="fp16",
            ctx=("list", [7000, 300]), seed=317),
    wl.Case("d240_mha_fp16_bs16", batch=2, heads=3, kv_heads=3, dk=240, dv=240, block_size=16, q_dtype="fp16", ctx=("list", [47, 800]),
            seed=318),
]


@pytest.mark.parametrize("case", _WIDE_CASES, ids=lambda c: c.name)
def test_head_sizes_and_large_groups_run_on_the_tiled_kernel(case):
    h = wl.make_host_inputs(case)
    out, info = run_gpu_case(case, h, out_fill=3.0)
    assert info.kernel == capi.KERNEL_TMA_MMA
    ref = oracle_out(case, h, out=wl.encode(np.full((case.batch, case.heads, case.dv), 3.0, dtype=np.float32), case.q_dtype))
    assert max_abs_err(out, ref, case.q_dtype) <= tol_for(case)
    # and the CUDA-core kernel agrees on the same inputs
    out_g, info_g = run_gpu_case(case, h, kernel=capi.KERNEL_GENERIC, out_fill=3.0)
    assert info_g.kernel == capi.KERNEL_GENERIC
    assert max_abs_err(out_g, ref, case.q_dtype) <= tol_for(case)
