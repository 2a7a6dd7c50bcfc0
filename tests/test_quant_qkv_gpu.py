"""int8 query, int8 K/V cache (quantType TYPE_QUANT_QKV_ONLINE / OFFLINE) on the GPU: both contractions on the
integer tensor cores, one dequantisation scale per query head, P quantised to int8.

The reference golden quantises P per tile of its own kernel (128 tokens or more,
tests/apitest/kernelstest/mix/test_paged_attention_common.py:142-227); the CUDA kernel's tiles are the 16 tokens a
warp owns in a stage.  Where the tiles fall decides which small probabilities round to zero, so the result moves by
the quantisation noise of P:
  * ONLINE: a tile's int8 probabilities depend on the tile alone (127 * p / tile maximum), so the kernel must agree
    closely (2e-3 of the output scale) with the oracle run with 16-token tiles, and within 2 % of the output scale
    with the golden's 128-token tiles (the fixtures made by the reference golden, and the oracle pinned on them);
  * OFFLINE: they also depend on the running maximum when the tile is reached (p * pScale), which a warp of the
    kernel keeps over its own tiles only; compared at 2.5 % of the output scale.
"""
import ctypes

import numpy as np
import pytest

import oracle
from golden_cases import GOLDEN_PA_QUANT_CASES, quant_inputs
from helpers import capi, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
HERE = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)), "golden")


def _run(d, heads, kv_heads, out_dtype, offline, scale):
    dev = {k: torch.from_numpy(v).cuda() for k, v in d.items() if isinstance(v, np.ndarray)}
    B = d["q"].shape[0]
    tdt = wl.torch_dtype(out_dtype)
    out = torch.full((B, heads, 128), 3.0, dtype=tdt, device="cuda")
    desc = capi.make_desc(B, heads, kv_heads, 128, 128, d["k_cache"].shape[1], d["k_cache"].shape[0],
                          d["block_tables"].shape[1], "int8", "int8", scale,
                          qkv_quant=capi.QUANT_OFFLINE if offline else capi.QUANT_ONLINE, out_dtype=out_dtype)
    plan = capi.PaPlan(desc, d["context_lens"])
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    t = capi.pa_tensors(dev["q"], dev["k_cache"], dev["v_cache"], dev["block_tables"], out, dev["k_descale"],
                        dev["v_descale"], p_scale=dev.get("p_scale") if offline else None)
    plan.launch(t, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
    torch.cuda.synchronize()
    assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
    assert plan.info.kernel == capi.KERNEL_TMA_MMA
    return wl.torch_to_host(out, out_dtype), plan.info


def _close(got, ref, dt, rel):
    """max |got - ref| within `rel` of the output scale (plus one unit in the last place of the output type)."""
    g, r = wl.to_f32(got, dt), wl.to_f32(ref, dt)
    scale = max(float(np.abs(r).max()), 1e-6)
    err = float(np.abs(g - r).max())
    ulp = 2.0 ** -10 if dt == "fp16" else 2.0 ** -7
    assert err <= (rel + ulp) * scale, (err, scale)


@pytest.mark.parametrize("spec", GOLDEN_PA_QUANT_CASES, ids=lambda s: s["name"])
def test_quant_qkv_matches_reference_golden_fixtures(spec):
    fx = np.load(__import__("os").path.join(HERE, f"pa_{spec['name']}.npz"))
    d = quant_inputs(spec)
    got, _ = _run(d, spec["heads"], spec["kv_heads"], spec["out_dtype"], spec["offline"], 1.0 / np.sqrt(128.0))
    _close(got, fx["out"], spec["out_dtype"], 2.5e-2 if spec["offline"] else 2e-2)


def _big_inputs(batch, heads, kv_heads, lens, offline, seed, block_size=128):
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, dtype=np.int32)
    need = (lens + block_size - 1) // block_size
    pool = int(max(2 * need.sum(), 2))
    perm = rng.permutation(pool).astype(np.int32)
    bt = np.full((batch, max(int(need.max()), 1)), -1, dtype=np.int32)
    pos = 0
    for b in range(batch):
        bt[b, :need[b]] = perm[pos:pos + need[b]]
        pos += need[b]
    d = {"context_lens": lens, "block_tables": bt}
    d["q"] = rng.integers(-127, 128, size=(batch, heads, 128), dtype=np.int8)
    d["k_cache"] = rng.integers(-127, 128, size=(pool, block_size, kv_heads, 128), dtype=np.int8)
    d["v_cache"] = rng.integers(-127, 128, size=(pool, block_size, kv_heads, 128), dtype=np.int8)
    # scores of a few units: q and k of ~73 rms over 128 dims give dot products of ~6e4
    d["k_descale"] = rng.uniform(0.5e-4, 2e-4, heads).astype(np.float32)
    d["v_descale"] = rng.uniform(0.005, 0.02, heads).astype(np.float32)
    if offline:
        d["p_scale"] = rng.uniform(60.0, 127.0, heads).astype(np.float32)
    return d


@pytest.mark.parametrize("name,batch,heads,kv_heads,lens,offline,out_dtype,block_size", [
    ("gqa8_online_split", 3, 64, 8, [5000, 130, 9000], False, "fp16", 128),
    ("gqa16_online_chunks", 4, 32, 2, [700, 0, 64, 2500], False, "bf16", 128),
    ("mha_offline_ragged", 7, 8, 8, [1, 15, 16, 17, 63, 300, 1025], True, "fp16", 128),
    ("gqa4_offline_bs32", 3, 16, 4, [333, 47, 1200], True, "bf16", 32),
    ("gqa4_online_bs32", 3, 16, 4, [333, 47, 1200], False, "fp16", 32),
    ("gqa2_online_bs16", 2, 4, 2, [100, 700], False, "bf16", 16),
])
def test_quant_qkv_matches_oracle(name, batch, heads, kv_heads, lens, offline, out_dtype, block_size):
    d = _big_inputs(batch, heads, kv_heads, lens, offline, seed=__import__("zlib").crc32(name.encode()) % 1000, block_size=block_size)
    scale = 1.0 / np.sqrt(128.0)
    got, info = _run(d, heads, kv_heads, out_dtype, offline, scale)
    ref = oracle.paged_attention_qkv_quant(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                                           d["k_descale"], d["v_descale"], scale, out_dtype, p_scale=d.get("p_scale"))
    live = np.asarray(lens) > 0
    _close(got[live], ref[live], out_dtype, 2.5e-2 if offline else 2e-2)
    if not offline:
        same_tiles = oracle.paged_attention_qkv_quant(d["q"], d["k_cache"], d["v_cache"], d["block_tables"],
                                                      d["context_lens"], d["k_descale"], d["v_descale"], scale, out_dtype,
                                                      tile_tokens=16)
        _close(got[live], same_tiles[live], out_dtype, 2e-3)
    # rows of empty sequences are left as they were
    assert np.all(wl.to_f32(got[~live], out_dtype) == 3.0)


def test_quant_qkv_operator():
    """TYPE_QUANT_QKV_ONLINE / OFFLINE through atb::Operation: int8 query and caches, kDescale, vDescale (and pScale)
    after contextLens, output of the type outDataType names
    (src/ops/ops_infer/paged_attention/paged_attention_operation.cpp:249-276, 436-443 of the reference)."""
    T = capi.atb_tensor
    for offline in (False, True):
        d = _big_inputs(4, 16, 2, [200, 1500, 77, 640], offline, seed=7 + offline)
        dev = {k: torch.from_numpy(v).cuda() for k, v in d.items() if isinstance(v, np.ndarray)}
        out = torch.zeros((4, 16, 128), dtype=torch.bfloat16, device="cuda")
        ins = [T(dev["q"]), T(dev["k_cache"]), T(dev["v_cache"]), T(dev["block_tables"]),
               T(dev["context_lens"], host=d["context_lens"]), T(dev["k_descale"]), T(dev["v_descale"])]
        if offline:
            ins.append(T(dev["p_scale"]))
        scale = 1.0 / np.sqrt(128.0)
        op = capi.Operation(capi.PagedAttentionParam(headNum=16, kvHeadNum=2, qkScale=scale, quantType=2 if offline else 3,
                                                     outDataType=capi.ACL_BF16))
        assert op.input_num == len(ins)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        ctx = capi.Context(stream.cuda_stream)
        ws_bytes = op.setup(ins, [T(out)], ctx)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
        op.execute(ins, [T(out)], ws.data_ptr(), ws_bytes, ctx)
        torch.cuda.synchronize()
        ref = oracle.paged_attention_qkv_quant(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], d["context_lens"],
                                               d["k_descale"], d["v_descale"], scale, "bf16", p_scale=d.get("p_scale"))
        _close(wl.torch_to_host(out, "bf16"), ref, "bf16", 2.5e-2 if offline else 2e-2)
    # parameter rules of the reference
    for bad in (dict(quantType=3, outDataType=capi.ACL_FLOAT), dict(quantType=2, outDataType=capi.ACL_BF16, hasQuantOffset=True),
                dict(quantType=3, outDataType=capi.ACL_BF16, calcType=1)):
        with pytest.raises(capi.AtbError) as e:
            capi.Operation(capi.PagedAttentionParam(headNum=8, kvHeadNum=8, qkScale=0.1, **bad))
        assert e.value.code == capi.ERROR_INVALID_PARAM
