"""Generates the golden fixtures in this directory from the REFERENCE's own CPU golden code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/ascend-transformer-boost

It imports, unmodified, the golden functions of the reference test-suite
  tests/apitest/kernelstest/mix/test_paged_attention_common.py   (TestPagedAttention:
      ref_single_query_cached_kv_attention / ref_masked_attention / group_mm_torch)
  tests/apitest/opstest/python/operations/paged_attention/test_paged_attention_operation_mla.py
      (TestPagedAttentionMLA: same functions for the combined K/V cache)
  tests/apitest/kernelstest/mix/test_reshape_and_cache.py        (generate_test_data)
  tests/apitest/kernelstest/mix/test_blockcopy.py                (TestBlockCopy.golden_calc)
  tests/apitest/kernelstest/mix/test_paged_cache_load_nd.py      (TestPagedCacheLoad.generate_test_data)
  tests/apitest/kernelstest/mix/test_rms_norm_and_rope_and_reshape_and_cache{,_bf16}.py
                                                                 (rmsnorm_golden, rope_golden, rac_golden)
with the NPU-only imports (`torch_npu`, `op_test`, `operation_test`) replaced by empty stubs, feeds
them this repository's seeded inputs, and stores the outputs as small .npz files.  The inputs are
not stored: they are regenerated from the seed and checked against the stored SHA-256.
"""
import hashlib
import importlib.util
import os
import sys
import types
import unittest

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)

from golden_cases import GOLDEN_PA_QUANT_CASES, quant_inputs  # noqa: E402
from golden_cases import (GOLDEN_BLOCKCOPY_CASES, GOLDEN_PA_CASES, GOLDEN_KVCACHE_CASES, GOLDEN_MLA_MTP_CASES, GOLDEN_PA_FEATURE_CASES, GOLDEN_PA_SPEC_CASES, GOLDEN_PCL_CASES,  # noqa: E402
                          GOLDEN_NRR_CASES, GOLDEN_RAC_CASES, blockcopy_inputs, load_workloads, nrr_inputs, kvcache_inputs, mla_mtp_inputs, pa_mask, spec_inputs,
                          pcl_inputs, rac_inputs)

wl = load_workloads()


def _stub_modules():
    class _Any(unittest.TestCase):
        def runTest(self):
            pass

    def _decorator_factory(*a, **k):
        if len(a) == 1 and callable(a[0]) and not k:
            return a[0]
        return lambda f: f

    for name, cls in (("op_test", "OpTest"), ("operation_test", "OperationTest")):
        m = types.ModuleType(name)
        setattr(m, cls, _Any)
        m.__getattr__ = lambda attr: _decorator_factory
        sys.modules[name] = m
    sys.modules["torch_npu"] = types.ModuleType("torch_npu")


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def to_torch(a, dtype):
    if dtype == "bf16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(a))


def from_torch(t, dtype):
    if dtype == "bf16":
        return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)
    if dtype == "fp16":
        return t.to(torch.float16).contiguous().numpy()
    return t.contiguous().numpy()


def digest(d):
    h = hashlib.sha256()
    for k in sorted(d):
        v = d[k]
        if isinstance(v, np.ndarray):
            h.update(k.encode())
            h.update(np.ascontiguousarray(v).tobytes())
    return h.hexdigest()


def run_pa_case(ref_root, case, cls_common, cls_mla):
    d = wl.make_host_inputs(case)
    tdt = {"fp16": torch.float16, "bf16": torch.bfloat16}[case.q_dtype]
    q = to_torch(d["q"], case.q_dtype)
    kc = to_torch(d["k_cache"], case.kvd)
    if case.mla or case.dk != case.dv:
        # the MLA golden class reads K and V widths separately, so it also serves Dk != Dv
        t = cls_mla()
        t.compressHead = False
        t.is_int8_flag = False
        t.num_heads, t.kv_heads, t.num_tokens = case.heads, case.kv_heads, case.batch
        t.head_size_qk, t.head_size_vo = case.dk, case.dv
        vc = kc[:, :, :, :case.dv] if case.mla else to_torch(d["v_cache"], case.kvd)
        out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.float32)
        high = torch.zeros_like(out)
        # the reference packs outputs of non-empty sequences; golden cases for MLA have none empty
        t.ref_single_query_cached_kv_attention(out, high, q, kc, vc, d["block_tables"].tolist(),
                                               d["context_lens"].tolist(), None, mask_dim=0,
                                               mask_data_type=tdt)
    else:
        t = cls_common()
        t.compressHead = False
        t.is_int8_flag = case.kvd == "int8"
        t.is_quant_flag = 0
        t.has_bias = case.offsets
        t.scaleType = 0
        t.num_heads, t.kv_heads, t.num_tokens, t.head_size = case.heads, case.kv_heads, case.batch, case.dk
        if t.is_int8_flag:
            t.de_scale1_fp32 = torch.from_numpy(d["k_descale"])
            t.de_scale2_fp32 = torch.from_numpy(d["v_descale"])
            if case.offsets:
                t.offset1 = torch.from_numpy(d["k_offset"])
                t.offset2 = torch.from_numpy(d["v_offset"])
        vc = to_torch(d["v_cache"], case.kvd)
        out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.float32)
        high = torch.zeros_like(out)
        assert (d["context_lens"] > 0).all(), "the reference golden packs rows when a length is 0"
        t.ref_single_query_cached_kv_attention(out, high, q, kc, vc, d["block_tables"].tolist(),
                                               d["context_lens"].tolist(), None, None, False, mask_dim=0,
                                               mask_data_type=tdt)
    return {"out": from_torch(out, case.q_dtype), "out_high": high.numpy(),
            "input_sha256": np.frombuffer(digest(d).encode(), dtype=np.uint8)}


def run_rac_case(rac_mod, spec):
    inp = rac_inputs(spec)
    # generate_test_data of the reference reads these attributes of the test object
    t = rac_mod.TestReshapeAndCache() if hasattr(rac_mod, "TestReshapeAndCache") else None
    if t is None:
        cls = [v for v in vars(rac_mod).values() if isinstance(v, type) and hasattr(v, "generate_test_data")][0]
        t = cls()
    t.num_tokens, t.num_heads = spec["tokens"], spec["heads"]
    t.head_size_k, t.head_size_v = spec["dk"], spec["dv"]
    t.block_size, t.num_blocks = spec["block_size"], spec["num_blocks"]
    t.dtype = {"fp16": "float16", "bf16": "bfloat16", "int8": "int8"}[spec["dtype"]]
    # the reference holds bf16 test data as float32 values; decode ours the same way
    t.key = wl.to_f32(inp["key"], spec["dtype"]) if spec["dtype"] == "bf16" else inp["key"]
    t.value = wl.to_f32(inp["value"], spec["dtype"]) if spec["dtype"] == "bf16" else inp["value"]
    t.slot_mapping = inp["slot_mapping"]
    kexp, vexp = t.generate_test_data()   # caches start from zeros in the reference golden
    if spec["dtype"] == "bf16":
        kexp, vexp = wl.f32_to_bf16_bits(kexp), wl.f32_to_bf16_bits(vexp)
    return {"key_cache": kexp, "value_cache": vexp,
            "input_sha256": np.frombuffer(digest(inp).encode(), dtype=np.uint8)}


def run_pa_feature_case(common, spec):
    """PagedAttention with the additive mask (alibi: mask_dim 4, plain: mask_dim 3) and / or the logN scale,
    through the same golden function as the plain cases."""
    case = spec["case"]
    d = wl.make_host_inputs(case)
    tdt = {"fp16": torch.float16, "bf16": torch.bfloat16}[case.q_dtype]
    t = common.TestPagedAttention()
    t.compressHead = False
    t.is_int8_flag = False
    t.is_quant_flag = 0
    t.has_bias = False
    t.scaleType = common.ScaleType.SCALE_LOGN_FP32.value if spec["logn"] else 0
    t.num_heads, t.kv_heads, t.num_tokens, t.head_size = case.heads, case.kv_heads, case.batch, case.dk
    mask_np = pa_mask(spec)
    mask = None if mask_np is None else to_torch(mask_np, case.q_dtype)
    mask_dim = {None: 0, "alibi": 4, "norm": 3}[spec["mask"]]
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.float32)
    high = torch.zeros_like(out)
    torch.manual_seed(case.seed)                       # the golden draws logN from torch's generator
    t.ref_single_query_cached_kv_attention(out, high, to_torch(d["q"], case.q_dtype), to_torch(d["k_cache"], case.kvd),
                                           to_torch(d["v_cache"], case.kvd), d["block_tables"].tolist(),
                                           d["context_lens"].tolist(), mask, None, False, mask_dim=mask_dim,
                                           mask_data_type=tdt)
    res = {"out": from_torch(out, case.q_dtype), "out_high": high.numpy(),
           "input_sha256": np.frombuffer(digest(d).encode(), dtype=np.uint8)}
    if spec["logn"]:
        res["logn"] = t.logN.numpy().astype(np.float32)
    return res


def run_pa_quant_case(common, spec):
    """int8 Q, K and V (QUANT_QKV online / offline) through the reference golden: the int32 matmuls, the per-tile
    quantisation of P and the log-sum-exp merge of the splits are all the reference's code; only the tile size
    (its block_size_calc) and the split length (its kv_split_per_core) are set here instead of derived from the
    core count of an Ascend SoC."""
    d = quant_inputs(spec)
    t = common.TestPagedAttention()
    t.compressHead = False
    t.is_int8_flag = False
    t.is_quant_flag = 1
    t.is_quant_offiline = 1 if spec["offline"] else 0
    t.has_bias = False
    t.scaleType = 0
    t.num_heads, t.kv_heads, t.num_tokens, t.head_size = spec["heads"], spec["kv_heads"], spec["batch"], 128
    t.block_size = 128
    t.block_size_calc = spec["tile"]
    max_len = int(d["context_lens"].max())
    t.kv_split_per_core = min(spec["split"], max_len)
    t.kvsplit = (max_len + t.kv_split_per_core - 1) // t.kv_split_per_core
    t.de_scale1_fp32 = torch.from_numpy(d["k_descale"])
    t.de_scale2_fp32 = torch.from_numpy(d["v_descale"])
    if spec["offline"]:
        t.scale = torch.from_numpy(d["p_scale"])
    tdt = {"fp16": torch.float16, "bf16": torch.bfloat16}[spec["out_dtype"]]
    out = torch.zeros((spec["batch"], spec["heads"], 128), dtype=torch.float32)
    high = torch.zeros_like(out)
    t.ref_single_query_cached_kv_attention(out, high, torch.from_numpy(d["q"]), torch.from_numpy(d["k_cache"]),
                                           torch.from_numpy(d["v_cache"]), d["block_tables"].tolist(),
                                           d["context_lens"].tolist(), None, None, False, mask_dim=0, mask_data_type=tdt)
    dig = {k: v for k, v in d.items() if isinstance(v, np.ndarray)}
    return {"out": from_torch(out, spec["out_dtype"]), "out_f32": out.numpy(),
            "input_sha256": np.frombuffer(digest(dig).encode(), dtype=np.uint8)}


def run_pa_spec_case(lookahead, spec):
    """Parallel decoding through the golden function of the reference's lookahead test (numpy, fp16; mask_type 3 =
    MASK_TYPE_SPEC rows per token, 0 = rows of the square causal mask)."""
    case = spec["case"]
    assert case.q_dtype == "fp16"
    d = spec_inputs(spec)
    t = lookahead.TestUnpadPagedAttention()
    out = np.zeros((d["q"].shape[0], case.heads, case.dv), dtype=np.float16)
    t.ref_single_query_cached_kv_attention(out, d["q"], d["k_cache"], d["v_cache"], d["block_tables"].tolist(),
                                           d["q_lens"].tolist(), d["context_lens"].tolist(), d["mask"],
                                           3 if spec["mask"] == "spec" else 0)
    dig = {k: v for k, v in d.items() if isinstance(v, np.ndarray)}
    return {"out": out, "input_sha256": np.frombuffer(digest(dig).encode(), dtype=np.uint8)}


def run_nrr_case(mod_fp16, mod_bf16, spec):
    """The fused RMSNorm + RoPE + cache write: the reference's three golden functions in golden_calc's order.
    fp16: rounded float16 rows; bf16: the reference keeps float32 rows (stored as such)."""
    inp = nrr_inputs(spec)
    mod = mod_fp16 if spec["dtype"] == "fp16" else mod_bf16
    t = mod.TestRmsNormAndRopeAndReshapeAndCacheOperation()
    val = lambda a: (a if spec["dtype"] == "fp16" else wl.to_f32(a, "bf16"))
    x, gamma, kr, cos, sin = (val(inp[k]) for k in ("x", "gamma", "key_rope", "cos", "sin"))
    cache = np.zeros((spec["blocks"], spec["block_size"], 1, spec["dx"] + spec["dr"]),
                     dtype=np.float16 if spec["dtype"] == "fp16" else np.float32)
    norm = t.rmsnorm_golden(x, gamma, spec["eps"])
    rope = t.rope_golden(kr, sin, cos).reshape(sin.shape[0], -1, sin.shape[-1])
    rows = np.concatenate((norm, rope), axis=-1)
    out = t.rac_golden(spec["block_size"], rows, inp["slot_mapping"], cache)
    return {"key_cache": out, "input_sha256": np.frombuffer(digest(inp).encode(), dtype=np.uint8)}


def _as_ref_values(a, dtype):
    """The reference tests hold bf16 data as float32 values; fp16 / int8 as they are."""
    return wl.to_f32(a, dtype) if dtype == "bf16" else a


def run_blockcopy_case(mod, spec):
    inp = blockcopy_inputs(spec)
    t = mod.TestBlockCopy()
    t.kCache = _as_ref_values(inp["k_cache"], spec["dtype"]).copy()
    t.vCache = _as_ref_values(inp["v_cache"], spec["dtype"]).copy()
    idx = [torch.from_numpy(inp[k]) for k in ("src", "dst", "cum")]
    kexp, vexp = t.golden_calc([None, None] + idx)
    if spec["dtype"] == "bf16":
        kexp, vexp = wl.f32_to_bf16_bits(kexp), wl.f32_to_bf16_bits(vexp)
    return {"k_cache": kexp, "v_cache": vexp, "input_sha256": np.frombuffer(digest(inp).encode(), dtype=np.uint8)}


def run_mla_lse_case(mla_split, case):
    """The log-sum-exp output of MultiLatentAttention (ring form) for an MLA case, through ref_masked_attention of the
    reference's split-cache kernel test, sequence by sequence as its gather loop calls it (mask None)."""
    d = wl.make_host_inputs(case)
    tdt = {"fp16": torch.float16, "bf16": torch.bfloat16}[case.q_dtype]
    t = mla_split.TestPagedAttentionMLA()
    t.is_int8_flag = False
    q, kc = to_torch(d["q"], case.q_dtype), to_torch(d["k_cache"], case.q_dtype)
    lse = torch.zeros((case.batch, case.heads, 1), dtype=tdt)
    for b in range(case.batch):
        n = int(d["context_lens"][b])
        if n == 0:
            continue
        keys = torch.stack([kc[int(d["block_tables"][b, j // case.block_size]), j % case.block_size] for j in range(n)], 0)
        values = keys[..., :case.dv]
        _, _, _, lse_b = t.ref_masked_attention(q[b].view(1, case.heads, case.dk), keys, values, np.float32(case.qk_scale),
                                                None, tdt)
        lse[b] = lse_b.reshape(case.heads, 1).to(tdt)
    return {"lse": from_torch(lse, case.q_dtype), "input_sha256": np.frombuffer(digest(d).encode(), dtype=np.uint8)}


def run_mla_mtp_case(mtp, spec):
    """MLA parallel decoding (output and log-sum-exp) through the golden of the reference's MTP split-cache kernel test;
    mask_type 3 = MASK_TYPE_SPEC rows per token, 0 = no mask."""
    case = spec["case"]
    d = mla_mtp_inputs(spec)
    tdt = {"fp16": torch.float16, "bf16": torch.bfloat16}[case.q_dtype]
    t = mtp.TestUnpadPagedAttention()
    t.post_mask_factor = 1.0
    q, kc = to_torch(d["q"], case.q_dtype), to_torch(d["k_cache"], case.q_dtype)
    tokens = q.shape[0]
    out, out_high = torch.zeros((tokens, case.heads, case.dv), dtype=tdt), torch.zeros((tokens, case.heads, case.dv))
    lse, lse_high = torch.zeros((tokens, case.heads, 1), dtype=tdt), torch.zeros((tokens, case.heads, 1))
    mask = to_torch(d["mask"], case.q_dtype) if spec["mask"] else None
    t.ref_single_query_cached_kv_attention(out, out_high, lse, lse_high, q, kc, kc[..., :case.dv], d["block_tables"].tolist(),
                                           d["q_lens"].tolist(), d["context_lens"].tolist(), mask, 3 if spec["mask"] else 0)
    return {"out": from_torch(out, case.q_dtype), "lse": from_torch(lse, case.q_dtype),
            "input_sha256": np.frombuffer(digest(d).encode(), dtype=np.uint8)}


def run_kvcache_case(mod, spec):
    """KvCache through golden_calc of the reference's kernel test (values as that test holds them: fp16 / int8 numpy;
    bf16 as float32 numpy, exact)."""
    inp = kvcache_inputs(spec)
    t = mod.TestKvcache()
    t.format_nd, t.format_nz = 2, 29                   # ACL_FORMAT_ND / FRACTAL_NZ, attributes of the stubbed base class
    t.case_param_gen({"format": t.format_nd, "layer": spec["layers"], "layer_id": spec["layer_id"], "batch": spec["batch"],
                      "max_seqlen": spec["max_seqlen"], "hidden_size": spec["hidden"]})
    t.newkv = _as_ref_values(inp["new_kv"], spec["dtype"])
    t.token_offset, t.seqlen = inp["token_offset"], inp["seq_len"]
    (out,) = t.golden_calc(None)
    out = out.numpy()
    if spec["dtype"] == "bf16":
        out = wl.f32_to_bf16_bits(out)
    return {"past": out.astype(inp["new_kv"].dtype) if spec["dtype"] != "bf16" else out,
            "input_sha256": np.frombuffer(digest(inp).encode(), dtype=np.uint8)}


def run_pcl_case(mod, spec):
    inp = pcl_inputs(spec)
    t = mod.TestPagedCacheLoad()
    t.num_tokens, t.num_heads = spec["batch"], spec["heads"]
    t.head_size_k, t.head_size_v = spec["dk"], spec["dv"]
    t.block_size, t.num_blocks = spec["block_size"], spec["blocks"]
    t.dtype = {"fp16": "float16", "bf16": "bfloat16", "int8": "int8"}[spec["dtype"]]
    t.key_cache = _as_ref_values(inp["k_cache"], spec["dtype"])
    t.value_cache = _as_ref_values(inp["v_cache"], spec["dtype"])
    t.block_tables, t.context_lens, t.seq_starts = inp["block_tables"], inp["cu_lens"], inp["seq_starts"]
    kexp, vexp = t.generate_test_data()
    if spec["dtype"] == "bf16":
        kexp, vexp = wl.f32_to_bf16_bits(kexp), wl.f32_to_bf16_bits(vexp)
    return {"key": kexp, "value": vexp, "input_sha256": np.frombuffer(digest(inp).encode(), dtype=np.uint8)}


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/ascend-transformer-boost")
    ref_root = sys.argv[1]
    _stub_modules()
    kt = os.path.join(ref_root, "tests/apitest/kernelstest")
    sys.path.insert(0, kt)
    sys.path.insert(0, os.path.join(kt, "mix"))
    cwd = os.getcwd()
    os.chdir(os.path.join(kt, "mix"))
    common = _load(os.path.join(kt, "mix/test_paged_attention_common.py"), "ref_pa_common")
    rac = _load(os.path.join(kt, "mix/test_reshape_and_cache.py"), "ref_rac")
    mla = _load(os.path.join(ref_root, "tests/apitest/opstest/python/operations/paged_attention/"
                                       "test_paged_attention_operation_mla.py"), "ref_pa_mla")
    blockcopy = _load(os.path.join(kt, "mix/test_blockcopy.py"), "ref_blockcopy")
    pcl = _load(os.path.join(kt, "mix/test_paged_cache_load_nd.py"), "ref_pcl")
    nrr16 = _load(os.path.join(kt, "mix/test_rms_norm_and_rope_and_reshape_and_cache.py"), "ref_nrr_fp16")
    nrrbf = _load(os.path.join(kt, "mix/test_rms_norm_and_rope_and_reshape_and_cache_bf16.py"), "ref_nrr_bf16")
    kvcache = _load(os.path.join(kt, "mix/test_kvcache.py"), "ref_kvcache")
    mla_split = _load(os.path.join(kt, "mix/test_paged_attention_mla_split.py"), "ref_pa_mla_split")
    mtp = _load(os.path.join(kt, "mix/test_paged_attention_mla_mtp_split.py"), "ref_pa_mla_mtp")
    lookahead = _load(os.path.join(kt, "mix/test_paged_attention_lookahead.py"), "ref_pa_lookahead")
    os.chdir(cwd)
    for spec in GOLDEN_PA_QUANT_CASES:
        res = run_pa_quant_case(common, spec)
        np.savez_compressed(os.path.join(HERE, f"pa_{spec['name']}.npz"), **res)
        print("wrote", spec["name"], res["out"].shape)
    if "--quant-only" in sys.argv:
        return
    for spec in GOLDEN_PA_SPEC_CASES:
        res = run_pa_spec_case(lookahead, spec)
        np.savez_compressed(os.path.join(HERE, f"pa_{spec['case'].name}.npz"), **res)
        print("wrote", spec["case"].name, res["out"].shape)
    for case in GOLDEN_PA_CASES:
        if case.mla:
            np.savez_compressed(os.path.join(HERE, f"mla_lse_{case.name}.npz"), **run_mla_lse_case(mla_split, case))
            print("wrote mla_lse", case.name)
    for spec in GOLDEN_MLA_MTP_CASES:
        np.savez_compressed(os.path.join(HERE, f"pa_{spec['case'].name}.npz"), **run_mla_mtp_case(mtp, spec))
        print("wrote", spec["case"].name)
    for spec in GOLDEN_KVCACHE_CASES:
        np.savez_compressed(os.path.join(HERE, f"kvcache_{spec['name']}.npz"), **run_kvcache_case(kvcache, spec))
        print("wrote kvcache", spec["name"])
    if "--spec-only" in sys.argv:
        return
    for spec in GOLDEN_NRR_CASES:
        np.savez_compressed(os.path.join(HERE, f"nrr_{spec['name']}.npz"), **run_nrr_case(nrr16, nrrbf, spec))
        print("wrote nrr", spec["name"])
    for spec in GOLDEN_BLOCKCOPY_CASES:
        np.savez_compressed(os.path.join(HERE, f"blockcopy_{spec['name']}.npz"), **run_blockcopy_case(blockcopy, spec))
        print("wrote blockcopy", spec["name"])
    for spec in GOLDEN_PCL_CASES:
        np.savez_compressed(os.path.join(HERE, f"pcl_{spec['name']}.npz"), **run_pcl_case(pcl, spec))
        print("wrote pcl", spec["name"])
    for spec in GOLDEN_PA_FEATURE_CASES:
        res = run_pa_feature_case(common, spec)
        np.savez_compressed(os.path.join(HERE, f"pa_{spec['case'].name}.npz"), **res)
        print("wrote", spec["case"].name, res["out"].shape)
    if "--siblings-only" in sys.argv:
        return
    for case in GOLDEN_PA_CASES:
        res = run_pa_case(ref_root, case, common.TestPagedAttention, mla.TestPagedAttentionMLA)
        np.savez_compressed(os.path.join(HERE, f"pa_{case.name}.npz"), **res)
        print("wrote", case.name, res["out"].shape)
    for spec in GOLDEN_RAC_CASES:
        res = run_rac_case(rac, spec)
        np.savez_compressed(os.path.join(HERE, f"rac_{spec['name']}.npz"), **res)
        print("wrote", spec["name"])


if __name__ == "__main__":
    main()
