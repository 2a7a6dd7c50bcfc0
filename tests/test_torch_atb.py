"""The Python operator API (`torch_atb`-shaped): parameter classes and Operation on CPU, forward() on
the GPU against the oracle.  Usage follows the reference's
tests/apitest/torch_atb_test/op_test/paged_attention/paged_attention_BSND_910B_test.py:451-468
(param object -> torch_atb.Operation(param) -> forward([...]) with context_lens as a CPU tensor)."""
import ctypes
import json

import numpy as np
import pytest

import oracle
from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, pkg, to_dev, tol_for, wl

torch_atb = pkg.torch_atb
torch = pytest.importorskip("torch")


def test_param_defaults_match_the_c_structs():
    p = torch_atb.PagedAttentionParam()
    c = p._c_param()
    assert ctypes.sizeof(c) == 120
    assert (c.headNum, c.kvHeadNum, c.maskType, c.quantType, c.outDataType, c.compressType, c.calcType, c.scaleType,
            c.inputLayout, c.mlaVHeadSize) == (0, 0, 0, 0, -1, 0, 0, 0, 0, 0)
    assert c.qkScale == 1.0 and c.qScale == 0.0 and not c.batchRunStatusEnable and not c.hasQuantOffset
    r = torch_atb.ReshapeAndCacheParam()._c_param()
    assert ctypes.sizeof(r) == 24 and (r.compressType, r.kvCacheCfg) == (0, 0)


def test_param_keywords_fields_and_repr():
    p = torch_atb.PagedAttentionParam(head_num=40, kv_head_num=10, qk_scale=0.0625,
                                      mask_type=torch_atb.PagedAttentionParam.MaskType.MASK_TYPE_NORM)
    p.input_layout = torch_atb.InputLayout.TYPE_BSND
    c = p._c_param()
    assert (c.headNum, c.kvHeadNum, c.maskType, c.inputLayout) == (40, 10, 1, 0) and abs(c.qkScale - 0.0625) < 1e-9
    name, _, body = repr(p).partition(": ")
    assert name == "PagedAttentionParam" and json.loads(body)["headNum"] == 40
    with pytest.raises(TypeError):
        torch_atb.PagedAttentionParam(headNum=1)
    r = torch_atb.ReshapeAndCacheParam(kv_cache_cfg=torch_atb.ReshapeAndCacheParam.KvCacheCfg.K_CACHE_V_BYPASS)
    assert r._c_param().kvCacheCfg == 1 and repr(r).startswith("ReshapeAndCacheParam: ")


def test_enum_values_are_the_reference_ones():
    P = torch_atb.PagedAttentionParam
    assert [int(x) for x in P.MaskType] == [0, 1, 2, 3, 4, 5]
    assert int(P.QuantType.TYPE_DEQUANT_FUSION) == 1 and int(P.QuantType.TYPE_QUANT_QKV_ONLINE) == 3
    assert int(P.CalcType.CALC_TYPE_SPEC) == 1 and int(P.ScaleType.SCALE_TYPE_LOGN) == 1
    assert int(torch_atb.AclDataType.ACL_BF16) == 27 and int(torch_atb.AclDataType.ACL_FLOAT16) == 1
    assert int(torch_atb.InputLayout.TYPE_BNSD) == 1


def test_operation_properties_without_a_gpu():
    op = torch_atb.Operation(torch_atb.PagedAttentionParam(head_num=32, kv_head_num=8, qk_scale=0.088))
    assert (op.name, op.input_num, op.output_num) == ("PagedAttentionOperation", 5, 1)
    assert repr(op) == "op name: PagedAttentionOperation, input_num: 5, output_num: 1"
    mla = torch_atb.Operation(torch_atb.PagedAttentionParam(head_num=128, kv_head_num=1, mla_v_head_size=512))
    assert mla.input_num == 4
    quant = torch_atb.Operation(torch_atb.PagedAttentionParam(
        head_num=8, kv_head_num=8, quant_type=torch_atb.PagedAttentionParam.QuantType.TYPE_DEQUANT_FUSION,
        has_quant_offset=True))
    assert quant.input_num == 9
    rac = torch_atb.Operation(torch_atb.ReshapeAndCacheParam())
    assert (rac.name, rac.input_num, rac.output_num) == ("ReshapeAndCacheOperation", 5, 2)
    siso = torch_atb.Operation(torch_atb.ReshapeAndCacheParam(
        kv_cache_cfg=torch_atb.ReshapeAndCacheParam.KvCacheCfg.K_CACHE_V_BYPASS))
    assert (siso.input_num, siso.output_num) == (3, 1)


def test_operation_rejects_bad_params():
    with pytest.raises(RuntimeError, match="Failed to create operation"):
        torch_atb.Operation(torch_atb.PagedAttentionParam(head_num=0))
    with pytest.raises(TypeError):
        torch_atb.Operation(object())
    with pytest.raises(ValueError):
        torch_atb.set_buffer_size(-1)


def test_operation_name_buffer_is_always_terminated():
    op = capi.Operation(capi.PagedAttentionParam(headNum=8, kvHeadNum=8))
    buf = ctypes.create_string_buffer(b"\xff" * 8, 8)
    assert capi.lib().atb_b200_operation_name(op.handle, buf, 8) == 0
    assert buf.raw[:7] == b"PagedAt" and buf.raw[7:8] == b"\0"
    assert capi.lib().atb_b200_operation_name(op.handle, None, 8) != 0
    assert capi.lib().atb_b200_operation_name(op.handle, buf, 0) != 0


# ------------------------------------------------------------------ forward() on the GPU

def _pa_inputs(case, h):
    d = host_inputs_to_device(case, h)
    ins = [d["q"], d["k_cache"]]
    if not case.mla:
        ins.append(d["v_cache"])
    ins += [d["block_tables"], torch.from_numpy(h["context_lens"])]      # context_lens stays on the host
    return ins


@pytest.mark.gpu
@pytest.mark.parametrize("use_side_stream", [False, True], ids=["own_stream", "default_stream"])
def test_forward_paged_attention_matches_oracle(use_side_stream):
    case = wl.Case("tatb_gqa", batch=7, heads=32, kv_heads=8, q_dtype="bf16", ctx=("uniform", 100, 1500), seed=71)
    h = wl.make_host_inputs(case)
    ref = oracle_out(case, h)
    op = torch_atb.Operation(torch_atb.PagedAttentionParam(head_num=case.heads, kv_head_num=case.kv_heads,
                                                           qk_scale=case.qk_scale))
    ins = _pa_inputs(case, h)
    torch.cuda.synchronize()
    if use_side_stream:
        (out,) = op.forward(ins)                       # caller on the legacy default stream
    else:
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            (out,) = op.forward(ins)
    torch.cuda.synchronize()
    assert tuple(out.shape) == (case.batch, case.heads, case.dv) and out.dtype == torch.bfloat16
    assert max_abs_err(wl.torch_to_host(out, case.q_dtype), ref, case.q_dtype) <= tol_for(case)
    stats = torch_atb.Prof.get_prof_stats().get_run_time_stats()
    assert len(stats["PagedAttentionOperation"]) >= 1


@pytest.mark.gpu
def test_forward_mla_matches_oracle():
    case = wl.Case("tatb_mla", batch=3, heads=16, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                   ctx=("list", [300, 64, 1000]), seed=72)
    h = wl.make_host_inputs(case)
    ref = oracle_out(case, h)
    op = torch_atb.Operation(torch_atb.PagedAttentionParam(head_num=case.heads, kv_head_num=1, qk_scale=case.qk_scale,
                                                           mla_v_head_size=case.dv))
    (out,) = op.forward(_pa_inputs(case, h))
    assert tuple(out.shape) == (case.batch, case.heads, case.dv)
    assert max_abs_err(wl.torch_to_host(out, case.q_dtype), ref, case.q_dtype) <= tol_for(case)


@pytest.mark.gpu
def test_forward_reshape_and_cache_writes_in_place():
    case = wl.Case("tatb_rac", batch=9, heads=8, kv_heads=2, q_dtype="fp16", ctx=("uniform", 5, 300), seed=73)
    h = wl.make_host_inputs(case)
    kc, vc = h["k_cache"].copy(), h["v_cache"].copy()
    oracle.reshape_and_cache(h["new_k"], h["new_v"], kc, vc, h["slot_mapping"])
    d = host_inputs_to_device(case, h)
    key, value = to_dev(h["new_k"], case.kvd), to_dev(h["new_v"], case.kvd)
    slots = torch.from_numpy(h["slot_mapping"]).cuda()
    op = torch_atb.Operation(torch_atb.ReshapeAndCacheParam())
    outs = op.forward([key, value, d["k_cache"], d["v_cache"], slots])
    assert outs[0].data_ptr() == d["k_cache"].data_ptr() and outs[1].data_ptr() == d["v_cache"].data_ptr()
    assert np.array_equal(wl.torch_to_host(d["k_cache"], case.kvd), kc)
    assert np.array_equal(wl.torch_to_host(d["v_cache"], case.kvd), vc)
    with pytest.raises(RuntimeError):
        op.forward([key, value, d["k_cache"].transpose(0, 1), d["v_cache"], slots])


@pytest.mark.gpu
def test_forward_reports_setup_failures():
    case = wl.Case("tatb_err", batch=2, heads=8, kv_heads=2, q_dtype="fp16", ctx=("uniform", 5, 300), seed=74)
    h = wl.make_host_inputs(case)
    op = torch_atb.Operation(torch_atb.PagedAttentionParam(head_num=case.heads, kv_head_num=case.kv_heads,
                                                           qk_scale=case.qk_scale))
    ins = _pa_inputs(case, h)
    ins[-1] = ins[-1].cuda()                           # context_lens without host data
    with pytest.raises(RuntimeError, match="Setup fail"):
        op.forward(ins)
    with pytest.raises(RuntimeError):
        op.forward(ins[:3])
