"""GPU tests of what was added to the operator layer after the hot path (dynamic batch, ...).  They sit
in a file of their own, collected after the hot-path tests: a failure here stops nothing that the
parity contract of the hot path depends on."""
import numpy as np
import pytest

from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, tol_for, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _run_dynamic_batch(case, h, status, extra_rows=0):
    """PagedAttention with batchRunStatusEnable through the atb operator API; the control tensors may
    carry `extra_rows` more sequences than there are query tokens."""
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    out = torch.full((case.batch, case.heads, case.dv), 7.0, dtype=wl.torch_dtype(case.q_dtype), device="cuda")
    lens_h = np.concatenate([h["context_lens"], np.full(extra_rows, 33, dtype=np.int32)])
    bt = d["block_tables"]
    if extra_rows:
        bt = torch.cat([bt, torch.zeros((extra_rows, bt.shape[1]), dtype=bt.dtype, device="cuda")])
    lens_dev = torch.from_numpy(lens_h).cuda()
    status_h = np.concatenate([np.asarray(status, dtype=np.int32), np.ones(extra_rows, dtype=np.int32)])
    status_dev = torch.from_numpy(status_h).cuda()
    ins = [T(d["q"]), T(d["k_cache"]), T(d["v_cache"]), T(bt), T(lens_dev, host=lens_h), T(status_dev, host=status_h)]
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale,
                                                 batchRunStatusEnable=True))
    assert op.input_num == len(ins)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    return wl.torch_to_host(out, case.q_dtype)


@pytest.mark.parametrize("extra_rows", [0, 2])
def test_dynamic_batch_skips_switched_off_sequences(extra_rows):
    # lengths and status pattern of the reference's test_pa_fp16_case_dynamic_batch_1
    # (tests/apitest/kernelstest/mix/test_paged_attention_common.py:1723-1741)
    lens = [2028, 0, 707, 0, 15, 1] * 2
    status = [1, 0, 1, 0, 1, 1] * 2
    status[4] = 0                                # a switched-off sequence that still has a length
    case = wl.Case("dyn_batch", batch=len(lens), heads=32, kv_heads=32, q_dtype="fp16", ctx=("list", lens), seed=81)
    h = wl.make_host_inputs(case)
    out = _run_dynamic_batch(case, h, status, extra_rows)
    eff = dict(h, context_lens=np.where(np.asarray(status) == 0, 0, h["context_lens"]).astype(np.int32))
    ref = oracle_out(case, eff, out=np.full((case.batch, case.heads, case.dv), 7.0, dtype=np.float16))
    assert max_abs_err(out, ref, case.q_dtype) <= tol_for(case)
    off = [b for b, s in enumerate(status) if s == 0]
    assert np.all(out[off] == np.float16(7.0))   # rows of skipped sequences are left untouched


# ------------------------------------------------------------------ BlockCopy / PagedCacheLoad

import os  # noqa: E402

import oracle  # noqa: E402
from golden_cases import (GOLDEN_BLOCKCOPY_CASES, GOLDEN_PCL_CASES, HERE as GOLDEN_DIR,  # noqa: E402
                          blockcopy_inputs, pcl_inputs)
from helpers import to_dev  # noqa: E402


def _bits(a):
    return a.view(np.uint16) if a.dtype == np.float16 else a


def _i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


@pytest.mark.parametrize("spec", GOLDEN_BLOCKCOPY_CASES, ids=lambda s: s["name"])
def test_block_copy_matches_reference_golden(spec):
    fx = np.load(os.path.join(GOLDEN_DIR, f"blockcopy_{spec['name']}.npz"))
    inp = blockcopy_inputs(spec)
    k, v = to_dev(inp["k_cache"], spec["dtype"]), to_dev(inp["v_cache"], spec["dtype"])
    capi.block_copy(k, v, _i32(inp["src"]), _i32(inp["dst"]), _i32(inp["cum"]))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(wl.torch_to_host(k, spec["dtype"])), _bits(fx["k_cache"]))
    assert np.array_equal(_bits(wl.torch_to_host(v, spec["dtype"])), _bits(fx["v_cache"]))


def test_block_copy_operation_large_blocks():
    """Blocks of 256 KB (several chunks per block) through the atb operator API, against the oracle."""
    rng = np.random.default_rng(91)
    shape = (24, 128, 8, 128)
    kc = rng.integers(-30000, 30000, size=shape, dtype=np.int16)
    vc = rng.integers(-30000, 30000, size=shape, dtype=np.int16)
    src = np.array([3, 7, 11], dtype=np.int32)
    dst = np.array([0, 1, 2, 4, 5, 20, 23], dtype=np.int32)
    cum = np.array([2, 3, 7], dtype=np.int32)
    ref_k, ref_v = oracle.cache_ops.block_copy(kc.copy(), vc.copy(), src, dst, cum)
    k = torch.from_numpy(kc).cuda().view(torch.bfloat16)
    v = torch.from_numpy(vc).cuda().view(torch.bfloat16)
    s, d, c = _i32(src), _i32(dst), _i32(cum)
    T = capi.atb_tensor
    op = capi.Operation(capi.BlockCopyParam())
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ins = [T(k), T(v), T(s), T(d), T(c)]
    assert op.setup(ins, [], ctx) == 0
    op.execute(ins, [], None, 0, ctx)
    torch.cuda.synchronize()
    assert np.array_equal(k.view(torch.int16).cpu().numpy(), ref_k)
    assert np.array_equal(v.view(torch.int16).cpu().numpy(), ref_v)


@pytest.mark.parametrize("cumulative", [True, False])
@pytest.mark.parametrize("spec", GOLDEN_PCL_CASES, ids=lambda s: s["name"])
def test_paged_cache_load_matches_reference_golden(spec, cumulative):
    fx = np.load(os.path.join(GOLDEN_DIR, f"pcl_{spec['name']}.npz"))
    inp = pcl_inputs(spec)
    kc, vc = to_dev(inp["k_cache"], spec["dtype"]), to_dev(inp["v_cache"], spec["dtype"])
    total = int(inp["cu_lens"][-1])
    key = torch.zeros((total,) + tuple(kc.shape[2:]), dtype=kc.dtype, device="cuda")
    value = torch.zeros((total,) + tuple(vc.shape[2:]), dtype=vc.dtype, device="cuda")
    lens = _i32(inp["cu_lens"] if cumulative else inp["lens"])
    capi.paged_cache_load(kc, vc, _i32(inp["block_tables"]), lens, key, value, seq_starts=_i32(inp["seq_starts"]),
                          cumulative=cumulative)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(wl.torch_to_host(key, spec["dtype"])), _bits(fx["key"]))
    assert np.array_equal(_bits(wl.torch_to_host(value, spec["dtype"])), _bits(fx["value"]))


def test_paged_cache_load_operation_reference_shape():
    """The shape of the reference's kernel test (16 sequences, 16 heads, 144 / 128 wide, block 128:
    tests/apitest/kernelstest/mix/test_paged_cache_load_nd.py:151-178) through the operator API."""
    rng = np.random.default_rng(92)
    nb, bs, heads, dk, dv, batch = 32, 128, 16, 144, 128, 16
    kc = rng.integers(-30000, 30000, size=(nb, bs, heads, dk), dtype=np.int16)
    vc = rng.integers(-30000, 30000, size=(nb, bs, heads, dv), dtype=np.int16)
    lens = rng.integers(1, 400, size=batch).astype(np.int32)
    lens[3] = 300                                           # long enough to reach the hole below
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cols = (int(lens.max()) + bs - 1) // bs + 4
    tables = rng.integers(0, nb, size=(batch, cols)).astype(np.int32)
    tables[3, 1] = -1                                       # a hole: those rows stay as they are
    starts = (rng.integers(0, 5, size=batch) * bs).astype(np.int32)
    starts[3] = 0
    total = int(cu[-1])
    ref_k = np.full((total, heads, dk), 5, np.int16)
    ref_v = np.full((total, heads, dv), 5, np.int16)
    oracle.cache_ops.paged_cache_load(kc, vc, tables, cu, ref_k, ref_v, seq_starts=starts, cumulative=True)
    T = capi.atb_tensor
    d_kc, d_vc = torch.from_numpy(kc).cuda().view(torch.float16), torch.from_numpy(vc).cuda().view(torch.float16)
    key = torch.full((total, heads, dk), 5, dtype=torch.int16, device="cuda").view(torch.float16)
    value = torch.full((total, heads, dv), 5, dtype=torch.int16, device="cuda").view(torch.float16)
    d_t, d_cu, d_st = _i32(tables), _i32(cu), _i32(starts)
    p = capi.PagedCacheLoadParam()
    p.kvCacheCfg, p.isSeqLensCumsumMode, p.hasSeqStarts = 1, True, True
    op = capi.Operation(p)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ins = [T(d_kc), T(d_vc), T(d_t), T(d_cu), T(key), T(value), T(d_st)]
    outs = [T(key), T(value)]
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    assert np.array_equal(key.view(torch.int16).cpu().numpy(), ref_k)
    assert np.array_equal(value.view(torch.int16).cpu().numpy(), ref_v)
    assert (ref_k == 5).all(axis=(1, 2)).any()              # the hole left rows untouched


def test_reshape_and_cache_with_stride_from_fused_qkv():
    """K and V as column slices of one fused [tokens, q | k | v] tensor, through the operator API, bit-exact
    against the oracle (which gathers the rows and applies the pinned ReshapeAndCache oracle)."""
    rng = np.random.default_rng(93)
    tokens, heads, q_heads, d, bs, nb = 37, 8, 32, 128, 128, 6
    width = (q_heads + 2 * heads) * d
    fused_h = rng.integers(-30000, 30000, size=(tokens, width), dtype=np.int16)
    k_off, v_off = q_heads * d, (q_heads + heads) * d
    kc_h = rng.integers(-30000, 30000, size=(nb, bs, heads, d), dtype=np.int16)
    vc_h = rng.integers(-30000, 30000, size=(nb, bs, heads, d), dtype=np.int16)
    slots_h = rng.choice(np.arange(0, nb * bs), size=tokens, replace=False).astype(np.int32)
    slots_h[5] = -2                                        # "do not store"
    ref_k, ref_v = oracle.cache_ops.reshape_and_cache_with_stride(fused_h, fused_h, kc_h.copy(), vc_h.copy(), slots_h,
                                                                  heads, d, d, width, k_off, v_off)
    fused = torch.from_numpy(fused_h).cuda().view(torch.bfloat16)
    kc = torch.from_numpy(kc_h).cuda().view(torch.bfloat16)
    vc = torch.from_numpy(vc_h).cuda().view(torch.bfloat16)
    slots = _i32(slots_h)
    strides = np.array([width, d, 1], dtype=np.int64)
    koff, voff = np.array([k_off], dtype=np.int64), np.array([v_off], dtype=np.int64)
    T = capi.atb_tensor
    # key and value: the fused tensor's address with the logical [tokens, heads, d] shape
    key_t = T(dtype=capi.ACL_BF16, shape=(tokens, heads, d), device_ptr=fused.data_ptr())
    val_t = T(dtype=capi.ACL_BF16, shape=(tokens, heads, d), device_ptr=fused.data_ptr())
    i64 = capi.ACL_INT64
    ins = [key_t, val_t, T(kc), T(vc), T(slots), T(dtype=i64, shape=(3,), host=strides),
           T(dtype=i64, shape=(3,), host=strides), T(dtype=i64, shape=(1,), host=koff), T(dtype=i64, shape=(1,), host=voff)]
    outs = [T(kc), T(vc)]
    op = capi.Operation(capi.ReshapeAndCacheWithStrideParam())
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    assert op.setup(ins, outs, ctx) == 0
    op.execute(ins, outs, None, 0, ctx)
    torch.cuda.synchronize()
    assert np.array_equal(kc.view(torch.int16).cpu().numpy(), ref_k)
    assert np.array_equal(vc.view(torch.int16).cpu().numpy(), ref_v)


# ------------------------------------------------------------------ fused RMSNorm + RoPE + cache write

from golden_cases import GOLDEN_NRR_CASES, nrr_inputs  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_NRR_CASES, ids=lambda s: s["name"])
def test_norm_rope_reshape_matches_oracle(spec):
    """Through the operator API against the oracle (itself pinned on the reference golden).  The tolerance is
    the reference test's own for this operation (test_rms_norm_and_rope_and_reshape_and_cache.py:74-86:
    |diff| <= 2^-8 * max(1, |golden|)); the kernel's summation order, emulated on the CPU, reproduces the
    oracle bit for bit on these cases, so nearly all elements must also be identical."""
    inp = nrr_inputs(spec)
    dt = spec["dtype"]
    shape = (spec["blocks"], spec["block_size"], 1, spec["dx"] + spec["dr"])
    rng = np.random.default_rng(spec["seed"] + 1)
    cache_h = wl.encode(rng.standard_normal(shape).astype(np.float32), dt)        # other slots must survive
    ref = cache_h.copy()
    oracle.cache_ops.norm_rope_reshape(inp["x"], inp["gamma"], inp["key_rope"], inp["cos"], inp["sin"],
                                       inp["slot_mapping"], ref, spec["eps"], dt)
    d = {k: to_dev(inp[k], dt) for k in ("x", "gamma", "key_rope", "cos", "sin")}
    slots = _i32(inp["slot_mapping"])
    cache = to_dev(cache_h, dt)
    T = capi.atb_tensor
    op = capi.Operation(capi.NormRopeReshapeParam(epsilon=spec["eps"]))
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ins = [T(d["x"]), T(d["gamma"]), T(d["key_rope"]), T(d["cos"]), T(d["sin"]), T(slots), T(cache)]
    outs = [T(cache)]
    assert op.setup(ins, outs, ctx) == 0
    op.execute(ins, outs, None, 0, ctx)
    torch.cuda.synchronize()
    got_bits = wl.torch_to_host(cache, dt)
    got, want = wl.to_f32(got_bits, dt), wl.to_f32(ref, dt)
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.maximum(1.0, np.abs(want)))
    assert np.mean(got_bits.view(np.uint16) == ref.view(np.uint16)) > 0.99


# ------------------------------------------------------------------ MLA with the split latent / rope cache

def _run_split_mla(case, h):
    """The kernel-level C ABI with rope_dim = 64: query and cache given as latent [.., 512] and rope [.., 64] tensors."""
    dt = case.q_dtype
    q, kc = to_dev(h["q"], dt), to_dev(h["k_cache"], dt)
    q_nope, q_rope = q[..., :512].contiguous(), q[..., 512:].contiguous()
    ct_kv, k_rope = kc[..., :512].contiguous(), kc[..., 512:].contiguous()
    bt = torch.from_numpy(h["block_tables"]).cuda()
    out = torch.zeros((case.batch, case.heads, 512), dtype=q.dtype, device="cuda")
    desc = capi.make_desc(case.batch, case.heads, 1, 576, 512, case.block_size, kc.shape[0], bt.shape[1], dt,
                          qk_scale=case.qk_scale, v_row_dim=512, rope_dim=64)
    plan = capi.PaPlan(desc, h["context_lens"])
    assert plan.info.kernel == capi.KERNEL_MLA_TC5
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(q_nope, ct_kv, ct_kv, bt, out, q_rope=q_rope, k_rope_cache=k_rope)
    plan.launch(tens, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
    return wl.torch_to_host(out, dt)


@pytest.mark.parametrize("name", ["mla_8h_fp16", "mla_8h_bf16", "mla_128h_bf16"])
def test_split_cache_mla_kernel_matches_oracle_and_combined_cache(name):
    case = [c for c in wl.SMALL_CASES if c.name == name][0]
    h = wl.make_host_inputs(case)
    got = _run_split_mla(case, h)
    ref = oracle.multi_latent_attention(np.ascontiguousarray(h["q"][..., :512]), np.ascontiguousarray(h["q"][..., 512:]),
                                        np.ascontiguousarray(h["k_cache"][..., :512]),
                                        np.ascontiguousarray(h["k_cache"][..., 512:]), h["block_tables"], h["context_lens"],
                                        case.qk_scale, case.q_dtype)
    assert max_abs_err(got, ref, case.q_dtype) <= tol_for(case)
    from helpers import run_gpu_case
    combined, info = run_gpu_case(case, h)
    assert info.kernel == capi.KERNEL_MLA_TC5
    assert np.array_equal(got.view(np.uint16), combined.view(np.uint16))      # same kernel, same arithmetic


def test_split_cache_needs_both_rope_tensors():
    case = [c for c in wl.SMALL_CASES if c.name == "mla_8h_bf16"][0]
    h = wl.make_host_inputs(case)
    desc = capi.make_desc(case.batch, case.heads, 1, 576, 512, case.block_size, h["k_cache"].shape[0],
                          h["block_tables"].shape[1], "bf16", qk_scale=case.qk_scale, v_row_dim=512, rope_dim=64)
    plan = capi.PaPlan(desc, h["context_lens"])
    fake = torch.zeros(16, dtype=torch.uint8, device="cuda")
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(fake, fake, fake, fake, fake)                      # no rope tensors
    with pytest.raises(capi.AtbError):
        plan.launch(tens, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
    with pytest.raises(capi.AtbError):                                       # other shapes have no split form
        capi.PaPlan(capi.make_desc(2, 8, 2, 128, 128, 128, 8, 4, "bf16", rope_dim=64), h["context_lens"][:2])


# ------------------------------------------------------------------ MultiLatentAttentionOperation (atb operator API)

@pytest.mark.parametrize("name", ["mla_8h_fp16", "mla_8h_bf16", "mla_128h_bf16"])
def test_multi_latent_attention_operation_matches_oracle(name):
    case = [c for c in wl.SMALL_CASES if c.name == name][0]
    h = wl.make_host_inputs(case)
    dt = case.q_dtype
    q, kc = to_dev(h["q"], dt), to_dev(h["k_cache"], dt)
    q_nope, q_rope = q[..., :512].contiguous(), q[..., 512:].contiguous()
    ct_kv, k_rope = kc[..., :512].contiguous(), kc[..., 512:].contiguous()
    bt = torch.from_numpy(h["block_tables"]).cuda()
    lens_dev = torch.from_numpy(h["context_lens"]).cuda()
    out = torch.full((case.batch, case.heads, 512), 7.0, dtype=q.dtype, device="cuda")
    T = capi.atb_tensor
    ins = [T(q_nope), T(q_rope), T(ct_kv), T(k_rope), T(bt), T(lens_dev, host=h["context_lens"])]
    outs = [T(out)]
    lse = torch.full((case.batch, case.heads, 1), 7.0, dtype=q.dtype, device="cuda")
    outs.append(T(lse))                                                   # CALC_TYPE_RING: log-sum-exp as second output
    op = capi.Operation(capi.MultiLatentAttentionParam(headNum=case.heads, kvHeadNum=1, qkScale=case.qk_scale, cacheMode=1,
                                                       calcType=2))
    assert op.infer_shape(ins, 2) == [tuple(out.shape), tuple(lse.shape)]
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    for lens in (h["context_lens"], np.maximum(h["context_lens"] // 2, 1).astype(np.int32)):   # second Setup re-plans
        ins[5] = T(lens_dev, host=lens)
        ws_bytes = op.setup(ins, outs, ctx)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
        op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
        torch.cuda.synchronize()
        got = wl.torch_to_host(out, dt)
        ref = oracle.multi_latent_attention(np.ascontiguousarray(h["q"][..., :512]), np.ascontiguousarray(h["q"][..., 512:]),
                                            np.ascontiguousarray(h["k_cache"][..., :512]),
                                            np.ascontiguousarray(h["k_cache"][..., 512:]), h["block_tables"], lens,
                                            case.qk_scale, dt)
        assert max_abs_err(got, ref, dt) <= tol_for(case)
        want_lse = wl.to_f32(oracle.attention_lse(h["q"], h["k_cache"], h["block_tables"], lens, case.qk_scale, dt), dt)
        got_lse = wl.to_f32(wl.torch_to_host(lse, dt), dt)
        unit = 2.0 ** (-10 if dt == "fp16" else -7)
        assert np.all(np.abs(got_lse - want_lse) <= 2 * unit * np.maximum(np.abs(want_lse), 1.0))


# ------------------------------------------------------------------ masks (NORM, ALIBI) and logN scaling

from golden_cases import GOLDEN_PA_FEATURE_CASES, pa_mask  # noqa: E402


def _run_pa_op(case, h, param_kw, mask=None, logn=None, lens=None):
    """PagedAttention through the atb operator API with the optional mask (after contextLens) and logN (last) inputs."""
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    lens = h["context_lens"] if lens is None else lens
    out = torch.full((case.batch, case.heads, case.dv), 7.0, dtype=wl.torch_dtype(case.q_dtype), device="cuda")
    lens_dev = torch.from_numpy(lens).cuda()
    ins = [T(d["q"]), T(d["k_cache"]), T(d["v_cache"]), T(d["block_tables"]), T(lens_dev, host=lens)]
    keep = [lens_dev]
    if mask is not None:
        keep.append(to_dev(mask, case.q_dtype))
        ins.append(T(keep[-1]))
    if logn is not None:
        keep.append(torch.from_numpy(np.ascontiguousarray(logn, dtype=np.float32)).cuda())
        ins.append(T(keep[-1]))
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale,
                                                 **param_kw))
    assert op.input_num == len(ins)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    return wl.torch_to_host(out, case.q_dtype)


def _feature_param(spec):
    kw = {}
    if spec["mask"] is not None:
        kw["maskType"] = 2 if spec["mask"] == "alibi" else 1
    if spec["logn"]:
        kw["scaleType"] = 1
    return kw


@pytest.mark.parametrize("kernel", [capi.KERNEL_TMA_MMA, capi.KERNEL_GENERIC], ids=["tma_mma", "generic"])
@pytest.mark.parametrize("spec", GOLDEN_PA_FEATURE_CASES, ids=lambda s: s["case"].name)
def test_mask_and_logn_match_reference_golden(spec, kernel, monkeypatch):
    case = spec["case"]
    fx = np.load(os.path.join(GOLDEN_DIR, f"pa_{case.name}.npz"))
    h = wl.make_host_inputs(case)
    monkeypatch.setenv("ATB_B200_FORCE_KERNEL", str(kernel))
    got = _run_pa_op(case, h, _feature_param(spec), mask=pa_mask(spec), logn=fx["logn"] if spec["logn"] else None)
    assert max_abs_err(got, fx["out"], case.q_dtype) <= tol_for(case)


@pytest.mark.parametrize("dim", [128, 96], ids=["d128", "d96_padded"])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_shared_alibi_rows_split_sequences_and_masked_out_prefix(dtype, dim):
    """Long sequences (split over several CTAs and merged), the alibi mask given once for all sequences
    ([heads, 1, tokens]), logN factors, and - in a second run - a norm mask that removes a whole prefix with -inf,
    longer than one CTA's first tile, which must neither produce NaN nor let the removed tokens through."""
    case = wl.Case(f"feat_long_{dtype}_{dim}", batch=5, heads=16, kv_heads=4, dk=dim, dv=dim, q_dtype=dtype,
                   ctx=("list", [4000, 37, 2100, 640, 1]), seed=77)
    h = wl.make_host_inputs(case)
    lens = h["context_lens"]
    tmax = int(lens.max())
    rng = np.random.default_rng(5)
    slopes = np.exp2(-8.0 * (np.arange(case.heads, dtype=np.float32) + 1) / case.heads)
    alibi = (slopes[:, None, None] * (np.arange(tmax, dtype=np.float32) - tmax + 1)[None, None, :]).astype(np.float32)
    alibi_enc = wl.encode(alibi, dtype)
    logn = rng.uniform(0.8, 1.6, size=case.batch).astype(np.float32)
    got = _run_pa_op(case, h, dict(maskType=2, scaleType=1), mask=alibi_enc, logn=logn)
    mask_f32 = np.broadcast_to(wl.to_f32(alibi_enc, dtype)[None], (case.batch, case.heads, 1, tmax))
    ref = oracle.paged_attention(h["q"], h["k_cache"], h["v_cache"], h["block_tables"], lens, case.qk_scale, dtype,
                                 mask=np.ascontiguousarray(mask_f32), logn=logn)
    assert max_abs_err(got, ref, dtype) <= tol_for(case)

    norm = np.zeros((case.batch, 1, tmax), dtype=np.float32)
    cut = [300, 5, 0, 639, 0]                                  # tokens removed at the start of each sequence
    for b, n in enumerate(cut):
        norm[b, 0, :n] = -np.inf
    got = _run_pa_op(case, h, dict(maskType=1), mask=wl.encode(norm, dtype))
    assert np.isfinite(wl.to_f32(got, dtype)).all()
    ref = oracle.paged_attention(h["q"], h["k_cache"], h["v_cache"], h["block_tables"], lens, case.qk_scale, dtype,
                                 mask=np.maximum(norm, -60000.0))
    assert max_abs_err(got, ref, dtype) <= tol_for(case)


def test_mask_shorter_than_a_context_is_refused():
    spec = GOLDEN_PA_FEATURE_CASES[1]
    case = spec["case"]
    h = wl.make_host_inputs(case)
    short = pa_mask(spec)[..., : int(h["context_lens"].max()) - 1]
    with pytest.raises(capi.AtbError) as e:
        _run_pa_op(case, h, dict(maskType=1), mask=np.ascontiguousarray(short))
    assert e.value.code == capi.ERROR_INVALID_TENSOR_DIM


# ------------------------------------------------------------------ heads-major cache blocks (inputLayout TYPE_BNSD)

@pytest.mark.parametrize("kernel", [capi.KERNEL_TMA_MMA, capi.KERNEL_GENERIC], ids=["tma_mma", "generic"])
@pytest.mark.parametrize("name,block_size", [("zero_and_one_ctx", 128), ("mha_fp16_no_mask", 16), ("gqa4_bf16_mid", 32)])
def test_bnsd_cache_layout_matches_token_major_result(name, block_size, kernel, monkeypatch):
    """The same cache contents with blocks stored [kv_heads, block_size, head_size] give the same output bits as the
    token-major layout (same kernel, same arithmetic), which the hot-path tests pin to the oracle."""
    import dataclasses
    base = [c for c in wl.SMALL_CASES if c.name == name][0]
    case = dataclasses.replace(base, block_size=block_size)
    h = wl.make_host_inputs(case)
    from helpers import run_gpu_case
    want, info = run_gpu_case(case, h, kernel=kernel, out_fill=7.0)     # empty sequences keep the fill value
    assert info.kernel == kernel
    assert max_abs_err(want, oracle_out(case, h, out=np.full_like(want, wl.encode(np.float32(7.0), case.q_dtype))), case.q_dtype) <= tol_for(case)
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    kc = d["k_cache"].permute(0, 2, 1, 3).contiguous()
    vc = d["v_cache"].permute(0, 2, 1, 3).contiguous()
    out = torch.full((case.batch, case.heads, case.dv), 7.0, dtype=kc.dtype, device="cuda")
    lens_dev = torch.from_numpy(h["context_lens"]).cuda()
    ins = [T(d["q"]), T(kc), T(vc), T(d["block_tables"]), T(lens_dev, host=h["context_lens"])]
    outs = [T(out)]
    monkeypatch.setenv("ATB_B200_FORCE_KERNEL", str(kernel))
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale,
                                                 inputLayout=1))
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    got = wl.torch_to_host(out, case.q_dtype)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


# ------------------------------------------------------------------ parallel decoding (CALC_TYPE_SPEC)

from golden_cases import GOLDEN_PA_SPEC_CASES, spec_inputs  # noqa: E402


def _run_spec_op(case, d, mask_kind, q_lens, lens):
    dt = case.q_dtype
    T = capi.atb_tensor
    q, kc, vc = to_dev(d["q"], dt), to_dev(d["k_cache"], dt), to_dev(d["v_cache"], dt)
    bt = torch.from_numpy(d["block_tables"]).cuda()
    mask = to_dev(d["mask"], dt)
    lens_dev, ql_dev = torch.from_numpy(lens).cuda(), torch.from_numpy(q_lens).cuda()
    out = torch.full((q.shape[0], case.heads, case.dv), 7.0, dtype=q.dtype, device="cuda")
    ins = [T(q), T(kc), T(vc), T(bt), T(lens_dev, host=lens), T(mask), T(ql_dev, host=q_lens)]
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale,
                                                 calcType=1, maskType=3 if mask_kind == "spec" else 1))
    assert op.infer_shape(ins, 1) == [tuple(out.shape)]
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    return wl.torch_to_host(out, dt)


@pytest.mark.parametrize("kernel", [capi.KERNEL_TMA_MMA, capi.KERNEL_GENERIC], ids=["tma_mma", "generic"])
@pytest.mark.parametrize("spec", GOLDEN_PA_SPEC_CASES, ids=lambda s: s["case"].name)
def test_parallel_decoding_matches_reference_golden(spec, kernel, monkeypatch):
    case = spec["case"]
    fx = np.load(os.path.join(GOLDEN_DIR, f"pa_{case.name}.npz"))
    d = spec_inputs(spec)
    monkeypatch.setenv("ATB_B200_FORCE_KERNEL", str(kernel))
    got = _run_spec_op(case, d, spec["mask"], d["q_lens"], d["context_lens"])
    ref = oracle.paged_attention_spec(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["q_lens"], d["context_lens"],
                                      case.qk_scale, case.q_dtype, wl.to_f32(d["mask"], case.q_dtype),
                                      mask_rows_are_tokens=spec["mask"] == "spec")
    assert max_abs_err(got, ref, case.q_dtype) <= tol_for(case)
    # and the reference's own golden at that test's threshold (it rounds scores and output to fp16 on the way)
    g, r = wl.to_f32(got, case.q_dtype), wl.to_f32(fx["out"], case.q_dtype)
    assert np.all(np.abs(g - r) <= 2.0 ** -8 * np.maximum(1.0, np.abs(r)))


def test_parallel_decoding_long_sequences_bf16():
    """Multi-token queries over sequences long enough to be split over CTAs, a sequence with no query token, bf16."""
    case = wl.Case("spec_long_bf16", batch=4, heads=16, kv_heads=4, q_dtype="bf16", ctx=("list", [5000, 700, 64, 2300]), seed=91)
    spec = dict(case=case, q_lens=[4, 0, 3, 2], mask="norm")
    d = spec_inputs(spec)
    got = _run_spec_op(case, d, "norm", d["q_lens"], d["context_lens"])
    ref = oracle.paged_attention_spec(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["q_lens"], d["context_lens"],
                                      case.qk_scale, "bf16", wl.to_f32(d["mask"], "bf16"), mask_rows_are_tokens=False)
    assert max_abs_err(got, ref, "bf16") <= tol_for(case)


# ------------------------------------------------------------------ KvCache (contiguous per-layer cache)

from golden_cases import GOLDEN_KVCACHE_CASES, kvcache_inputs  # noqa: E402


@pytest.mark.parametrize("spec", GOLDEN_KVCACHE_CASES, ids=lambda s: s["name"])
def test_kv_cache_matches_reference_golden(spec):
    fx = np.load(os.path.join(GOLDEN_DIR, f"kvcache_{spec['name']}.npz"))
    inp = kvcache_inputs(spec)
    dt = spec["dtype"]
    T = capi.atb_tensor
    dev = {k: (to_dev(v, dt) if k in ("new_kv", "past") else torch.from_numpy(v).cuda()) for k, v in inp.items()}
    ins = [T(dev["new_kv"]), T(dev["layer_id"]), T(dev["past"]), T(dev["token_offset"]), T(dev["seq_len"])]
    op = capi.Operation(capi.KvCacheParam())
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    assert op.setup(ins, [], ctx) == 0
    op.execute(ins, [], None, 0, ctx)
    torch.cuda.synchronize()
    got = wl.torch_to_host(dev["past"], dt)
    bits = lambda a: a.view(np.uint16) if a.dtype == np.float16 else a
    assert np.array_equal(bits(got), bits(fx["past"]))


def test_kv_cache_large_rows_keep_the_rest_of_the_cache():
    rng = np.random.default_rng(17)
    layers, batch, max_seqlen, hidden = 3, 9, 300, 1024                  # 2 KB rows, runs of up to 600 KB (many chunks)
    seq_len = rng.integers(0, 290, size=batch).astype(np.int32)
    seq_len[3] = 0
    token_offset = (seq_len + rng.integers(0, 10, size=batch)).astype(np.int32)
    new_kv = rng.integers(0, 2 ** 15, size=(int(seq_len.sum()), hidden)).astype(np.uint16)
    before = rng.integers(0, 2 ** 15, size=(layers, batch, max_seqlen, hidden)).astype(np.uint16)
    want = oracle.cache_ops.kv_cache(new_kv, 2, before.copy(), token_offset, seq_len)
    past = torch.from_numpy(before.view(np.int16)).cuda().view(torch.bfloat16)
    kv = torch.from_numpy(new_kv.view(np.int16)).cuda().view(torch.bfloat16)
    capi.kv_cache(kv, torch.tensor([2], dtype=torch.int32, device="cuda"), past, torch.from_numpy(token_offset).cuda(),
                  torch.from_numpy(seq_len).cuda())
    torch.cuda.synchronize()
    got = past.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, want)


# ------------------------------------------------------------------ MultiLatentAttention, parallel decoding (MTP)

from golden_cases import GOLDEN_MLA_MTP_CASES, mla_mtp_inputs  # noqa: E402


def _run_mla_mtp(case, d, mask_type, ring, mask=None):
    dt = case.q_dtype
    T = capi.atb_tensor
    q, kc = to_dev(d["q"], dt), to_dev(d["k_cache"], dt)
    q_nope, q_rope = q[..., :512].contiguous(), q[..., 512:].contiguous()
    ct_kv, k_rope = kc[..., :512].contiguous(), kc[..., 512:].contiguous()
    bt = torch.from_numpy(d["block_tables"]).cuda()
    lens_dev, ql_dev = torch.from_numpy(d["context_lens"]).cuda(), torch.from_numpy(d["q_lens"]).cuda()
    out = torch.full((q.shape[0], case.heads, 512), 7.0, dtype=q.dtype, device="cuda")
    lse = torch.full((q.shape[0], case.heads, 1), 7.0, dtype=q.dtype, device="cuda")
    ins = [T(q_nope), T(q_rope), T(ct_kv), T(k_rope), T(bt), T(lens_dev, host=d["context_lens"])]
    keep = []
    if mask_type:
        keep.append(to_dev(mask, dt))
        ins.append(T(keep[-1]))
    ins.append(T(ql_dev, host=d["q_lens"]))
    outs = [T(out)] + ([T(lse)] if ring else [])
    op = capi.Operation(capi.MultiLatentAttentionParam(headNum=case.heads, kvHeadNum=1, qkScale=case.qk_scale, cacheMode=1,
                                                       calcType=3 if ring else 1, maskType=mask_type))
    assert op.input_num == len(ins) and op.output_num == len(outs)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    return wl.torch_to_host(out, dt), wl.torch_to_host(lse, dt)


@pytest.mark.parametrize("spec", GOLDEN_MLA_MTP_CASES, ids=lambda s: s["case"].name)
def test_mla_parallel_decoding_matches_reference_golden(spec):
    case = spec["case"]
    dt = case.q_dtype
    fx = np.load(os.path.join(GOLDEN_DIR, f"pa_{case.name}.npz"))
    d = mla_mtp_inputs(spec)
    got, lse = _run_mla_mtp(case, d, 1 if spec["mask"] else 0, ring=True, mask=d.get("mask"))
    assert max_abs_err(got, fx["out"], dt) <= tol_for(case)
    unit = 2.0 ** (-10 if dt == "fp16" else -7)
    gl, rl = wl.to_f32(lse, dt), wl.to_f32(fx["lse"], dt)
    assert np.all(np.abs(gl - rl) <= 2 * unit * np.maximum(np.abs(rl), 1.0))
    if spec["mask"]:
        # MASK_FREE is the same causal rule without reading a mask: same result up to the masked terms' exp(-10000) = 0
        free, _ = _run_mla_mtp(case, d, 2, ring=False, mask=np.zeros((8, 128), dtype=d["mask"].dtype))
        assert max_abs_err(free, fx["out"], dt) <= tol_for(case)


def test_mla_parallel_decoding_long_sequences():
    """128 heads (two CTAs per range), sequences long enough to be split and merged, three tokens per sequence."""
    case = wl.Case("mla_mtp_long", batch=3, heads=128, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                   ctx=("list", [3000, 77, 1500]), seed=93)
    spec = dict(case=case, q_lens=[3, 1, 2], mask="spec")
    d = mla_mtp_inputs(spec)
    got, lse = _run_mla_mtp(case, d, 1, ring=True, mask=d["mask"])
    ref, ref_lse = oracle.paged_attention_spec(d["q"], d["k_cache"], None, d["block_tables"], d["q_lens"], d["context_lens"],
                                               case.qk_scale, "bf16", wl.to_f32(d["mask"], "bf16"), mask_rows_are_tokens=True,
                                               dv=512, want_lse=True)
    assert max_abs_err(got, ref, "bf16") <= tol_for(case)
    gl, rl = wl.to_f32(lse, "bf16"), wl.to_f32(ref_lse, "bf16")
    assert np.all(np.abs(gl - rl) <= 2 * 2.0 ** -7 * np.maximum(np.abs(rl), 1.0))


def test_mla_combined_cache_with_norm_mask():
    """PagedAttention over the MLA combined cache (mlaVHeadSize) with a plain mask [batch, 1, tokens]: the mask variant
    of the MLA kernel without per-token rows."""
    case = [c for c in wl.SMALL_CASES if c.name == "mla_8h_bf16"][0]
    h = wl.make_host_inputs(case)
    dt, lens = case.q_dtype, h["context_lens"]
    tmax = int(lens.max())
    rng = np.random.default_rng(3)
    mask = np.where(rng.random((case.batch, 1, tmax)) < 0.3, -10000.0, 0.0).astype(np.float32)
    mask[:, 0, 0] = 0.0                                                   # every sequence keeps a visible token
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    out = torch.full((case.batch, case.heads, case.dv), 7.0, dtype=d["q"].dtype, device="cuda")
    lens_dev, mask_dev = torch.from_numpy(lens).cuda(), to_dev(wl.encode(mask, dt), dt)
    ins = [T(d["q"]), T(d["k_cache"]), T(d["block_tables"]), T(lens_dev, host=lens), T(mask_dev)]
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=1, qkScale=case.qk_scale, mlaVHeadSize=case.dv,
                                                 maskType=1))
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    ref = oracle.paged_attention(h["q"], h["k_cache"], None, h["block_tables"], lens, case.qk_scale, dt, dv=case.dv, mask=mask)
    assert max_abs_err(wl.torch_to_host(out, dt), ref, dt) <= tol_for(case)


# ------------------------------------------------------------------ parallel decoding planned per sequence (uniform q_len)

@pytest.mark.parametrize("mask_kind", ["spec", "norm"])
@pytest.mark.parametrize("heads,kv_heads,q_len,dtype,dim", [(8, 2, 2, "bf16", 128), (8, 4, 4, "fp16", 128), (4, 4, 3, "fp16", 128),
                                                            (16, 2, 1, "bf16", 128), (8, 2, 2, "bf16", 80), (4, 4, 3, "fp16", 192)])
def test_parallel_decoding_same_token_count_per_sequence(heads, kv_heads, q_len, dtype, dim, mask_kind, monkeypatch):
    """Every sequence has q_len query tokens: the operator plans one row per sequence whose CTA columns are the (token,
    head) pairs (the cache is read once) when q_len x heads-per-kv-head <= 8, else one row per token.  Both must give
    the oracle's result, and the per-sequence form the same as the per-token form (forced through the environment)."""
    case = wl.Case(f"mtp_{heads}_{kv_heads}_{q_len}_{dtype}_{dim}", batch=5, heads=heads, kv_heads=kv_heads, dk=dim, dv=dim,
                   q_dtype=dtype, ctx=("list", [3000, 37, 640, 1, 129 if q_len < 4 else 200]), seed=97)
    spec = dict(case=case, q_lens=[q_len] * 5, mask=mask_kind)
    d = spec_inputs(spec)
    lens = d["context_lens"].copy()
    if mask_kind == "norm":
        lens = np.maximum(lens, q_len).astype(np.int32)                   # the square mask needs ctx >= q_len
        d["context_lens"] = lens
    ref = oracle.paged_attention_spec(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["q_lens"], lens, case.qk_scale,
                                      dtype, wl.to_f32(d["mask"], dtype), mask_rows_are_tokens=mask_kind == "spec")
    got = _run_spec_op(case, d, mask_kind, d["q_lens"], lens)
    assert max_abs_err(got, ref, dtype) <= tol_for(case)
    monkeypatch.setenv("ATB_B200_SPEC_EXPAND", "1")
    per_token = _run_spec_op(case, d, mask_kind, d["q_lens"], lens)
    assert max_abs_err(per_token, ref, dtype) <= tol_for(case)
    assert max_abs_err(got, per_token, dtype) <= tol_for(case)


@pytest.mark.parametrize("mask_type", [0, 1, 2], ids=["no_mask", "spec_mask", "mask_free"])
@pytest.mark.parametrize("heads,q_len,dtype", [(16, 2, "bf16"), (8, 3, "fp16"), (128, 2, "bf16")])
def test_mla_parallel_decoding_same_token_count_per_sequence(heads, q_len, dtype, mask_type, monkeypatch):
    """MTP with q_len tokens for every sequence: planned per sequence (the MLA kernel's rows are the (token, head) pairs,
    64 per CTA) and, forced through the environment, per token; both against the oracle, with the log-sum-exp."""
    case = wl.Case(f"mla_mtp_{heads}_{q_len}_{dtype}", batch=4, heads=heads, kv_heads=1, dk=576, dv=512, q_dtype=dtype, mla=True,
                   ctx=("list", [1500, 64, 130, q_len]), seed=99)
    spec = dict(case=case, q_lens=[q_len] * 4, mask="spec")
    d = mla_mtp_inputs(spec)
    lens = d["context_lens"]
    mask_f32 = wl.to_f32(d["mask"], dtype)                                # the causal triangle in columns [ctx - q_len, ctx)
    ref, ref_lse = oracle.paged_attention_spec(d["q"], d["k_cache"], None, d["block_tables"], d["q_lens"], lens, case.qk_scale,
                                               dtype, None if mask_type == 0 else mask_f32, mask_rows_are_tokens=True, dv=512,
                                               want_lse=True)
    given = {0: None, 1: d["mask"], 2: np.zeros((8, 128), dtype=d["mask"].dtype)}[mask_type]
    unit = 2.0 ** (-10 if dtype == "fp16" else -7)
    for form in ("ATB_B200_SPEC_FUSE", "ATB_B200_SPEC_EXPAND", None):    # per sequence, per token, the operator's choice
        monkeypatch.delenv("ATB_B200_SPEC_FUSE", raising=False)
        monkeypatch.delenv("ATB_B200_SPEC_EXPAND", raising=False)
        if form:
            monkeypatch.setenv(form, "1")
        got, lse = _run_mla_mtp(case, d, mask_type, ring=True, mask=given)
        assert max_abs_err(got, ref, dtype) <= tol_for(case)
        gl, rl = wl.to_f32(lse, dtype), wl.to_f32(ref_lse, dtype)
        assert np.all(np.abs(gl - rl) <= 2 * unit * np.maximum(np.abs(rl), 1.0))


def test_mla_plan_balances_ranges_and_every_cta_reports_its_time():
    """The MLA plan weighs every token range it starts like six tiles, so CTAs that hold two ranges get fewer tiles; the
    all-CTA form of the probe (CTA selector 255) shows the result: every CTA's end is after its start and the CTAs that
    work end close together."""
    case = wl.Case("mla_plan_balance", batch=6, heads=128, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                   ctx=("list", [9000, 7000, 8000, 6000, 9500, 5000]), seed=95)
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=d["q"].dtype, device="cuda")
    desc = capi.make_desc(case.batch, case.heads, 1, 576, 512, case.block_size, d["k_cache"].shape[0], d["block_tables"].shape[1],
                          "bf16", qk_scale=case.qk_scale, v_row_dim=576)
    plan = capi.PaPlan(desc, h["context_lens"])
    info = plan.info
    items, groups = plan.dump()
    n_groups = info.num_ctas // 2
    cost = np.array([sum((e - b + 63) // 64 for _, b, e, _ in items[groups[g]:groups[g + 1]]) + 6 * (groups[g + 1] - groups[g])
                     for g in range(n_groups)])
    assert cost.max() <= np.sort(cost)[n_groups // 2] + 7                  # greedy packing: full groups differ by < one range
    ws = torch.empty(max(int(info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(d["q"], d["k_cache"], None, d["block_tables"], out)
    trace = torch.zeros(4096, dtype=torch.int64, device="cuda")
    plan.set_trace(trace.data_ptr(), 4096 | (255 << 24))
    plan.launch(tens, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
    torch.cuda.synchronize()
    plan.set_trace(0, 0)
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
    t = trace.cpu().numpy()
    start, end = t[1:1 + 2 * info.num_ctas:2], t[2:2 + 2 * info.num_ctas:2]
    assert np.all(end > start) and np.all(start > 0)
    ref = oracle.paged_attention(h["q"], h["k_cache"], None, h["block_tables"], h["context_lens"], case.qk_scale, "bf16", dv=512)
    assert max_abs_err(wl.torch_to_host(out, "bf16"), ref, "bf16") <= tol_for(case)
