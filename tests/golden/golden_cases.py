"""The small seeded cases whose reference-golden outputs are stored in this directory."""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG_DIR = os.path.join(ROOT, "ascend-transformer-boost_b200")


def load_workloads():
    """The package directory name is not a Python identifier, so load the module by path."""
    name = "atb_b200_workloads"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_wl = load_workloads()
Case = _wl.Case

GOLDEN_PA_CASES = [
    Case("mha_fp16", batch=3, heads=4, kv_heads=4, q_dtype="fp16", ctx=("list", [1, 130, 300]), seed=101),
    Case("gqa4_bf16", batch=2, heads=8, kv_heads=2, q_dtype="bf16", ctx=("list", [200, 257]), seed=102),
    Case("gqa8_fp16", batch=2, heads=8, kv_heads=1, q_dtype="fp16", ctx=("list", [88, 129]), seed=103),
    Case("d96_bs16_fp16", batch=3, heads=5, kv_heads=5, dk=96, dv=96, block_size=16, q_dtype="fp16",
         ctx=("list", [33, 1, 65]), seed=104),
    Case("int8_fp16", batch=2, heads=8, kv_heads=8, q_dtype="fp16", kv_dtype="int8", ctx=("list", [150, 64]),
         seed=105),
    Case("int8_bf16_gqa_offsets", batch=2, heads=8, kv_heads=1, q_dtype="bf16", kv_dtype="int8", offsets=True,
         ctx=("list", [140, 256]), seed=106),
    Case("int8_fp16_gqa_offsets", batch=2, heads=8, kv_heads=2, q_dtype="fp16", kv_dtype="int8", offsets=True,
         ctx=("list", [77, 131]), seed=107),
    Case("mla_bf16", batch=2, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
         ctx=("list", [140, 90]), seed=108),
    Case("mla_fp16", batch=2, heads=16, kv_heads=1, dk=576, dv=512, q_dtype="fp16", mla=True,
         ctx=("list", [129, 60]), seed=109),
    Case("dk_ne_dv_fp16", batch=2, heads=4, kv_heads=2, dk=192, dv=128, q_dtype="fp16", ctx=("list", [70, 140]),
         seed=110),
]

GOLDEN_RAC_CASES = [
    dict(name="fp16_eq", tokens=20, heads=4, dk=32, dv=32, block_size=16, num_blocks=6, dtype="fp16", seed=201),
    dict(name="bf16_dk_ne_dv", tokens=17, heads=3, dk=48, dv=24, block_size=8, num_blocks=9, dtype="bf16", seed=202),
    dict(name="int8_mla_like", tokens=30, heads=2, dk=576, dv=512, block_size=16, num_blocks=5, dtype="int8",
         seed=203),
    dict(name="fp16_odd", tokens=11, heads=5, dk=7, dv=13, block_size=4, num_blocks=10, dtype="fp16", seed=204),
]


def rac_inputs(spec):
    """Seeded ReshapeAndCache inputs: distinct slots drawn from [-num_slots, num_slots) as the
    reference test does (negative slots must be skipped)."""
    rng = np.random.default_rng(spec["seed"])
    n, h = spec["tokens"], spec["heads"]
    num_slots = spec["block_size"] * spec["num_blocks"]
    slots = rng.choice(np.arange(-num_slots, num_slots), size=n, replace=False).astype(np.int32)

    def gen(d):
        if spec["dtype"] == "int8":
            return rng.integers(-127, 128, size=(n, h, d), dtype=np.int8)
        return _wl.encode(rng.standard_normal((n, h, d), dtype=np.float32), spec["dtype"])

    return {"key": gen(spec["dk"]), "value": gen(spec["dv"]), "slot_mapping": slots}


# ------------------------------------------------------------------ cache-management siblings

GOLDEN_BLOCKCOPY_CASES = [
    dict(name="fp16_small", blocks=15, block_size=2, heads=2, d=2, n_src=3, n_dst=10, dtype="fp16", seed=301),
    dict(name="bf16_mid", blocks=40, block_size=16, heads=3, d=24, n_src=7, n_dst=19, dtype="bf16", seed=302),
    dict(name="int8_one_to_one", blocks=24, block_size=8, heads=2, d=20, n_src=6, n_dst=6, dtype="int8", seed=303),
]


def blockcopy_inputs(spec):
    """Seeded BlockCopy inputs as the reference test draws them (tests/apitest/kernelstest/mix/
    test_blockcopy.py:17-55): destinations are distinct blocks that are not sources, cumSum is a
    sorted running total ending at the number of destinations."""
    rng = np.random.default_rng(spec["seed"])
    shape = (spec["blocks"], spec["block_size"], spec["heads"], spec["d"])

    def gen():
        if spec["dtype"] == "int8":
            return rng.integers(-127, 128, size=shape, dtype=np.int8)
        return _wl.encode(rng.standard_normal(shape, dtype=np.float32), spec["dtype"])

    src = rng.integers(0, spec["blocks"], size=spec["n_src"]).astype(np.int32)
    free = np.setdiff1d(np.arange(spec["blocks"]), src)
    dst = rng.choice(free, size=spec["n_dst"], replace=False).astype(np.int32)
    inner = np.sort(rng.choice(np.arange(1, spec["n_dst"]), size=spec["n_src"] - 1, replace=False))
    cum = np.append(inner, spec["n_dst"]).astype(np.int32)
    return {"k_cache": gen(), "v_cache": gen(), "src": src, "dst": dst, "cum": cum}


GOLDEN_PCL_CASES = [
    dict(name="fp16_cumsum_starts", batch=5, heads=3, dk=40, dv=24, block_size=16, blocks=20, max_len=70,
         dtype="fp16", cumulative=True, starts=True, seed=311),
    dict(name="bf16_cumsum_starts", batch=3, heads=1, dk=144, dv=128, block_size=128, blocks=6, max_len=200,
         dtype="bf16", cumulative=True, starts=True, seed=312),
    dict(name="int8_cumsum_starts", batch=6, heads=4, dk=32, dv=32, block_size=8, blocks=30, max_len=50,
         dtype="int8", cumulative=True, starts=True, seed=313),
]


def pcl_inputs(spec):
    """Seeded PagedCacheLoad inputs shaped like the reference test's (tests/apitest/kernelstest/mix/
    test_paged_cache_load_nd.py:25-63): random block tables with four spare columns, cumulative
    lengths, sequence starts of 0..4 whole blocks."""
    rng = np.random.default_rng(spec["seed"])
    bs = spec["block_size"]

    def gen(d):
        shape = (spec["blocks"], bs, spec["heads"], d)
        if spec["dtype"] == "int8":
            return rng.integers(-127, 128, size=shape, dtype=np.int8)
        return _wl.encode(rng.standard_normal(shape, dtype=np.float32), spec["dtype"])

    lens = rng.integers(1, spec["max_len"] + 1, size=spec["batch"])
    cols = (int(lens.max()) + bs - 1) // bs + 4
    tables = rng.integers(0, spec["blocks"], size=(spec["batch"], cols)).astype(np.int32)
    starts = (rng.integers(0, 5, size=spec["batch"]) * bs).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    return {"k_cache": gen(spec["dk"]), "v_cache": gen(spec["dv"]), "block_tables": tables, "cu_lens": cu,
            "lens": lens.astype(np.int32), "seq_starts": starts}


GOLDEN_KVCACHE_CASES = [
    dict(name="fp16_prefill", layers=3, layer_id=1, batch=4, max_seqlen=24, hidden=32, dtype="fp16", decode=False, seed=501),
    dict(name="bf16_decode", layers=2, layer_id=0, batch=5, max_seqlen=16, hidden=48, dtype="bf16", decode=True, seed=502),
    dict(name="int8_mixed", layers=2, layer_id=1, batch=3, max_seqlen=20, hidden=64, dtype="int8", decode=False, seed=503),
]


def kvcache_inputs(spec):
    """Seeded KvCache inputs in the manner of the reference test (tests/apitest/kernelstest/mix/test_kvcache.py:
    95-108): prefill has token_offset = seq_len, decode one new row per sequence at a random position.  `past`
    starts as zeros, as the reference golden assumes."""
    rng = np.random.default_rng(spec["seed"])
    b, s = spec["batch"], spec["max_seqlen"]
    if spec["decode"]:
        seq_len = np.ones(b, dtype=np.int32)
        token_offset = rng.integers(1, s + 1, size=b).astype(np.int32)
    else:
        seq_len = rng.integers(1, s // 2, size=b).astype(np.int32)
        token_offset = seq_len.copy()
        token_offset[-1] += 3                      # one sequence appends behind three cached tokens
    n = int(seq_len.sum())
    if spec["dtype"] == "int8":
        new_kv = rng.integers(-127, 128, size=(n, spec["hidden"]), dtype=np.int8)
    else:
        new_kv = _wl.encode(rng.uniform(-5, 5, size=(n, spec["hidden"])).astype(np.float32), spec["dtype"])
    past = np.zeros((spec["layers"], b, s, spec["hidden"]), dtype=new_kv.dtype)
    return {"new_kv": new_kv, "layer_id": np.array([spec["layer_id"]], dtype=np.int32), "past": past,
            "token_offset": token_offset, "seq_len": seq_len}


# ------------------------------------------------------------------ PagedAttention with a mask / logN scale

GOLDEN_PA_FEATURE_CASES = [
    dict(case=Case("alibi_fp16", batch=3, heads=8, kv_heads=8, q_dtype="fp16", ctx=("list", [70, 130, 257]), seed=121),
         mask="alibi", logn=False),
    dict(case=Case("norm_mask_bf16_gqa", batch=4, heads=8, kv_heads=2, q_dtype="bf16", ctx=("list", [33, 129, 200, 64]),
                   seed=122), mask="norm", logn=False),
    dict(case=Case("logn_fp16", batch=3, heads=4, kv_heads=4, q_dtype="fp16", ctx=("list", [150, 31, 300]), seed=123),
         mask=None, logn=True),
    dict(case=Case("alibi_logn_bf16", batch=2, heads=8, kv_heads=4, q_dtype="bf16", ctx=("list", [140, 90]), seed=124),
         mask="alibi", logn=True),
]


def pa_mask(spec):
    """The additive mask of a feature case in the query dtype's encoding, built like the reference test
    builds it (tests/apitest/kernelstest/mix/test_paged_attention_common.py:488-506): alibi
    [batch, heads, 1, max_ctx] = slope_h * (position - context_len + 1); plain [batch, 1, max_ctx] with
    -10000 on the first i positions of sequence i."""
    case = spec["case"]
    lens = _wl.context_lens(case)
    T = int(lens.max())
    if spec["mask"] == "alibi":
        h = case.heads
        slopes = np.exp2(-8.0 * (np.arange(h, dtype=np.float32) + 1) / h).astype(np.float32)
        m = np.zeros((case.batch, h, 1, T), dtype=np.float32)
        for i, n in enumerate(lens):
            m[i, :, 0, :n] = slopes[:, None] * (np.arange(n, dtype=np.float32) - n + 1)[None, :]
    elif spec["mask"] == "norm":
        m = np.zeros((case.batch, 1, T), dtype=np.float32)
        for i in range(case.batch):
            m[i, :, :i] = -10000.0
    else:
        return None
    return _wl.encode(m, case.q_dtype)


# ------------------------------------------------------------------ PagedAttention with int8 Q, K and V (QUANT_QKV)

GOLDEN_PA_QUANT_CASES = [
    dict(name="quant_online_fp16", batch=3, heads=8, kv_heads=8, out_dtype="fp16", lens=[70, 300, 129], offline=False,
         tile=128, split=1 << 30, seed=131),
    dict(name="quant_online_bf16_gqa_split", batch=2, heads=8, kv_heads=2, out_dtype="bf16", lens=[700, 257], offline=False,
         tile=128, split=256, seed=132),
    dict(name="quant_offline_fp16_gqa", batch=3, heads=8, kv_heads=1, out_dtype="fp16", lens=[33, 260, 128], offline=True,
         tile=128, split=1 << 30, seed=133),
]


def quant_inputs(spec):
    """Seeded inputs of a QUANT_QKV case with the value ranges of the reference test
    (tests/apitest/kernelstest/mix/test_paged_attention_common.py:444-450, 540-543): int8 query and caches
    in [-5, 5]; one dequantisation scale per query head for Q.K^T and one for P.V (the reference draws them from
    (-5/127, 5/127); here (0.2/127, 1/127), positive, so that no head's scores flip sign as a whole); for the
    offline form one P scale per head (the reference: (0, 127); here (20, 127), away from the degenerate 0)."""
    rng = np.random.default_rng(spec["seed"])
    bs, d = 128, 128
    lens = np.asarray(spec["lens"], dtype=np.int32)
    need = (lens + bs - 1) // bs
    pool = int(2 * need.sum())
    perm = rng.permutation(pool).astype(np.int32)
    bt = np.full((spec["batch"], int(need.max())), -1, dtype=np.int32)
    pos = 0
    for b in range(spec["batch"]):
        bt[b, :need[b]] = perm[pos:pos + need[b]]
        pos += need[b]
    out = {"context_lens": lens, "block_tables": bt, "num_blocks": pool}
    out["q"] = rng.integers(-5, 6, size=(spec["batch"], spec["heads"], d), dtype=np.int8)
    out["k_cache"] = rng.integers(-5, 6, size=(pool, bs, spec["kv_heads"], d), dtype=np.int8)
    out["v_cache"] = rng.integers(-5, 6, size=(pool, bs, spec["kv_heads"], d), dtype=np.int8)
    out["k_descale"] = rng.uniform(0.2 / 127, 1.0 / 127, spec["heads"]).astype(np.float32)
    out["v_descale"] = rng.uniform(0.2 / 127, 1.0 / 127, spec["heads"]).astype(np.float32)
    out["p_scale"] = rng.uniform(20.0, 127.0, spec["heads"]).astype(np.float32) if spec["offline"] else None
    return out


# ------------------------------------------------------------------ PagedAttention, parallel decoding (CALC_TYPE_SPEC)

GOLDEN_PA_SPEC_CASES = [
    dict(case=Case("spec_mask_fp16", batch=4, heads=8, kv_heads=8, q_dtype="fp16", ctx=("list", [10, 64, 64, 64]),
                   seed=131), q_lens=[1, 15, 30, 6], mask="spec"),
    dict(case=Case("spec_norm_mask_gqa_fp16", batch=3, heads=8, kv_heads=2, q_dtype="fp16", ctx=("list", [140, 33, 257]),
                   seed=132), q_lens=[4, 2, 5], mask="norm"),
]


GOLDEN_MLA_MTP_CASES = [
    dict(case=Case("mla_mtp_spec_mask_bf16", batch=3, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                   ctx=("list", [140, 90, 257]), seed=141), q_lens=[2, 2, 3], mask="spec"),
    dict(case=Case("mla_mtp_no_mask_fp16", batch=2, heads=16, kv_heads=1, dk=576, dv=512, q_dtype="fp16", mla=True,
                   ctx=("list", [129, 60]), seed=142), q_lens=[2, 1], mask=None),
]


def mla_mtp_inputs(spec):
    """Inputs of an MLA parallel-decoding case (combined 576-wide rows; the tests split them [512, 64]): cache, block
    tables and context lengths of `case`, a query with sum(q_lens) tokens, and for MASK_TYPE_SPEC the mask
    [tokens, max_ctx] with every sequence's causal triangle in columns [ctx - q_len, ctx), as the reference test
    builds it (tests/apitest/kernelstest/mix/test_paged_attention_mla_mtp_split.py:246-257)."""
    case = spec["case"]
    d = _wl.make_host_inputs(case)
    q_lens = np.asarray(spec["q_lens"], dtype=np.int32)
    tokens, T = int(q_lens.sum()), int(d["context_lens"].max())
    rng = np.random.default_rng(case.seed + 31)
    d["q"] = _wl.encode(rng.standard_normal((tokens, case.heads, case.dk)).astype(np.float32), case.q_dtype)
    d["q_lens"] = q_lens
    if spec["mask"] == "spec":
        m = np.zeros((tokens, T), dtype=np.float32)
        pre = 0
        for n, k in zip(q_lens, d["context_lens"]):
            m[pre:pre + n, k - n:k] = np.triu(np.ones((n, n), dtype=np.float32), 1) * -10000.0
            pre += n
        d["mask"] = _wl.encode(m, case.q_dtype)
    for k in ("v_cache", "new_v"):
        d.pop(k, None)
    return d


def spec_inputs(spec):
    """Inputs of a parallel-decoding case: the caches, block tables and context lengths of `case` (one row per
    sequence), a query with sum(q_lens) tokens, and the mask built like the reference test builds it
    (tests/apitest/kernelstest/mix/test_paged_attention_lookahead.py:176-191): MASK_TYPE_SPEC
    [tokens, max_ctx] with the causal triangle of every sequence in its last q_len columns; MASK_TYPE_NORM the
    square causal mask [max_ctx, max_ctx] (a token reads row ctx - q_len + j)."""
    case = spec["case"]
    d = _wl.make_host_inputs(case)
    q_lens = np.asarray(spec["q_lens"], dtype=np.int32)
    tokens, T = int(q_lens.sum()), int(d["context_lens"].max())
    rng = np.random.default_rng(case.seed + 29)
    d["q"] = _wl.encode(rng.standard_normal((tokens, case.heads, case.dk)).astype(np.float32), case.q_dtype)
    if spec["mask"] == "spec":
        m = np.zeros((tokens, T), dtype=np.float32)
        pre = 0
        for n in q_lens:
            m[pre:pre + n, T - n:] = np.triu(np.ones((n, n), dtype=np.float32), 1) * -10000.0
            pre += n
    else:
        m = np.triu(np.ones((T, T), dtype=np.float32), 1) * -10000.0
    d["mask"] = _wl.encode(m, case.q_dtype)
    d["q_lens"] = q_lens
    return d


# ------------------------------------------------------------------ fused RMSNorm + RoPE + cache write

GOLDEN_NRR_CASES = [
    dict(name="fp16_mla", tokens=40, dx=512, dr=64, block_size=16, blocks=4, dtype="fp16", eps=1e-5, seed=401),
    dict(name="bf16_mla", tokens=33, dx=512, dr=64, block_size=8, blocks=6, dtype="bf16", eps=1e-6, seed=402),
    dict(name="fp16_small", tokens=9, dx=32, dr=16, block_size=4, blocks=5, dtype="fp16", eps=1e-5, seed=403),
]


def nrr_inputs(spec):
    """Seeded inputs of the fused op, value ranges of a real layer (x ~ N(0,1) * 3, gamma ~ U(0.5, 1.5), cos /
    sin of random angles) rather than the reference test's U(-100, 100); distinct slots, some negative."""
    rng = np.random.default_rng(spec["seed"])
    t, dx, dr = spec["tokens"], spec["dx"], spec["dr"]
    enc = lambda a: _wl.encode(a.astype(np.float32), spec["dtype"])
    angle = rng.uniform(0, 2 * np.pi, size=(t, dr // 2)).astype(np.float32)
    cos = np.concatenate([np.cos(angle), np.cos(angle)], axis=1)
    sin = np.concatenate([np.sin(angle), np.sin(angle)], axis=1)
    slots = rng.choice(np.arange(spec["blocks"] * spec["block_size"]), size=t, replace=False).astype(np.int32)
    slots[2] = -1
    return {"x": enc(3.0 * rng.standard_normal((t, 1, dx))), "gamma": enc(rng.uniform(0.5, 1.5, size=dx)),
            "key_rope": enc(rng.standard_normal((t, dr))), "cos": enc(cos), "sin": enc(sin), "slot_mapping": slots}
