"""CPU-only checks: the library loads and exports its C ABI, the host planner's invariants, and the
error behaviour of the operator layer (no kernel is launched here)."""
import ctypes
import os
import re

import numpy as np
import pytest

from helpers import ROOT, capi, wl


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "atb_b200.h")).read()
    declared = set(re.findall(r"\b(atb_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(capi.EXPORTS)
    lib = ctypes.CDLL(capi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert b"atb-b200" in capi.lib().atb_b200_version()


def test_param_struct_sizes_match_reference_abi():
    # tests/unittest/ops/test_op_param_size.cpp:47,51 of the reference
    assert ctypes.sizeof(capi.PagedAttentionParam) == 120
    assert ctypes.sizeof(capi.ReshapeAndCacheParam) == 24


def _plan(case, lens=None, kernel=0, sm=148):
    lens = wl.context_lens(case) if lens is None else np.asarray(lens, dtype=np.int32)
    need = int(((lens.astype(np.int64) + case.block_size - 1) // case.block_size).max()) if len(lens) else 1
    d = capi.make_desc(case.batch, case.heads, case.kv_heads, case.dk, case.dv, case.block_size, 1 << 20,
                       max(need, 1), case.q_dtype, case.kvd, case.qk_scale,
                       v_row_dim=case.dk if case.mla else case.dv, kernel=kernel, sm_count=sm)
    return capi.PaPlan(d, lens), lens


@pytest.mark.parametrize("case", wl.CONFIGS + wl.SMALL_CASES, ids=lambda c: c.name)
def test_plan_covers_every_token_exactly_once(case):
    plan, lens = _plan(case)
    info = plan.info
    items, groups = plan.dump()
    cols = info.num_ctas // max(1, (info.num_ctas // max(1, _cols(case, info))))
    covered = {}
    for seq, b, e, slot in items:
        assert 0 <= b < e <= lens[seq]
        assert b % 64 == 0
        covered.setdefault(seq, []).append((b, e, slot))
    n_partials = 0
    for seq in range(case.batch):
        parts = sorted(covered.get(seq, []))
        if lens[seq] == 0:
            assert not parts
            continue
        assert parts[0][0] == 0 and parts[-1][1] == lens[seq]
        for (b0, e0, _), (b1, e1, _) in zip(parts, parts[1:]):
            assert e0 == b1
        if len(parts) == 1:
            assert parts[0][2] == -1
        else:
            slots = [p[2] for p in parts]
            assert slots == list(range(slots[0], slots[0] + len(parts)))
            n_partials += len(parts)
    assert n_partials == info.num_partials
    n_groups = len([g for g in groups if True]) and (info.num_ctas // _cols(case, info))
    assert groups[0] == 0 and groups[n_groups] == info.num_items
    assert np.all(np.diff(groups[:n_groups + 1]) >= 0)


def _cols(case, info):
    if info.kernel == capi.KERNEL_TMA_MMA:
        return case.kv_heads * ((case.heads // case.kv_heads + 7) // 8)   # a column per 8 query heads of a kv head
    if info.kernel == capi.KERNEL_MLA_TC5:
        return (case.heads + 63) // 64
    dmax = max(case.dk, case.dv)
    gh = 8 if dmax <= 128 else (4 if dmax <= 256 else 2)
    group = case.heads // case.kv_heads
    return case.kv_heads * ((group + gh - 1) // gh)


@pytest.mark.parametrize("idx", [1, 2, 3])
def test_plan_is_balanced_on_benchmark_configs(idx):
    case = wl.CONFIGS[idx]
    plan, lens = _plan(case)
    info = plan.info
    items, groups = plan.dump()
    n_groups = info.num_ctas // _cols(case, info)
    per_sm = {capi.KERNEL_TMA_MMA: 2, capi.KERNEL_MLA_TC5: 1}.get(info.kernel, 4)
    assert info.num_ctas <= 148 * per_sm, "the grid must fit one wave of resident CTAs"
    tiles = [sum((e - b + 63) // 64 for _, b, e, _ in items[groups[g]:groups[g + 1]]) for g in range(n_groups)]
    assert max(tiles) <= np.mean(tiles) * 1.03 + 1


def test_plan_update_replans_in_place():
    case = wl.CONFIGS[1]
    plan, lens = _plan(case)
    before = plan.dump()[0].copy()
    plan.update(lens + 1)
    after = plan.dump()[0]
    assert after[:, 2].max() == (lens + 1).max()
    assert before.shape[0] > 0


def test_plan_rejects_bad_arguments():
    case = wl.CONFIGS[1]
    lens = wl.context_lens(case)
    d = capi.make_desc(case.batch, 32, 5, 128, 128, 128, 1000, 32, "bf16", sm_count=148)  # 32 % 5 != 0
    with pytest.raises(capi.AtbError) as e:
        capi.PaPlan(d, lens)
    assert e.value.code == capi.ERROR_INVALID_PARAM
    d = capi.make_desc(case.batch, 32, 8, 128, 128, 128, 1000, 4, "bf16", sm_count=148)  # lens exceed 4 blocks
    with pytest.raises(capi.AtbError) as e:
        capi.PaPlan(d, lens)
    assert e.value.code == capi.ERROR_INVALID_PARAM
    d = capi.make_desc(case.batch, 32, 8, 128, 128, 128, 1000, 32, "bf16", sm_count=148)
    d.q_per_seq = -1
    with pytest.raises(capi.AtbError):
        capi.PaPlan(d, lens)
    # a kernel that does not support the shape
    d = capi.make_desc(4, 8, 8, 72, 72, 16, 1000, 64, "fp16", kernel=capi.KERNEL_TMA_MMA, sm_count=148)
    with pytest.raises(capi.AtbError) as e:
        capi.PaPlan(d, np.array([5, 6, 7, 8], dtype=np.int32))
    assert e.value.code == capi.ERROR_INVALID_TENSOR_DIM


def test_kernel_selection():
    assert _plan(wl.CONFIGS[1])[0].info.kernel == capi.KERNEL_TMA_MMA
    assert _plan(wl.CONFIGS[0])[0].info.kernel == capi.KERNEL_TMA_MMA
    small = {c.name: c for c in wl.SMALL_CASES}
    assert _plan(small["ragged_d96_bs16_fp16"])[0].info.kernel == capi.KERNEL_TMA_MMA     # 96 runs padded on the 128 geometry
    # more than 8 query heads per kv head: the tiled kernel, a CTA column per chunk of 8 heads
    p127 = _plan(small["gqa127_fp16"])[0].info
    assert p127.kernel == capi.KERNEL_TMA_MMA and p127.num_ctas % 16 == 0
    assert _plan(small["gqa15_fp16"])[0].info.kernel == capi.KERNEL_TMA_MMA
    assert _plan(small["mla_128h_bf16"])[0].info.kernel == capi.KERNEL_MLA_TC5
    assert _plan(wl.CONFIGS[2])[0].info.kernel == capi.KERNEL_TMA_MMA      # int8 cache
    assert _plan(wl.CONFIGS[4])[0].info.kernel == capi.KERNEL_MLA_TC5


# ---------------------------------------------------------------- operator layer, error behaviour

def _pa_param(**kw):
    base = dict(headNum=8, kvHeadNum=2, qkScale=0.1)
    base.update(kw)
    return capi.PagedAttentionParam(**base)


def _expect(code, fn, *a, **k):
    with pytest.raises(capi.AtbError) as e:
        fn(*a, **k)
    assert e.value.code == code, e.value.code


def test_create_operation_param_checks():
    capi.Operation(_pa_param())
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(headNum=0))
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(kvHeadNum=-1))
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(headNum=8, kvHeadNum=3))
    p = _pa_param()
    p.rsv[5] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, p)
    # MLA rules: one kv head, no dequant fusion, width <= 576
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(mlaVHeadSize=512, kvHeadNum=2))
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(mlaVHeadSize=512, kvHeadNum=1, quantType=1))
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(mlaVHeadSize=600, kvHeadNum=1))
    capi.Operation(_pa_param(mlaVHeadSize=512, kvHeadNum=1))
    # dequant needs calcType UNDEFINED
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(quantType=1, calcType=1))
    rp = capi.ReshapeAndCacheParam()
    capi.Operation(rp)
    rp2 = capi.ReshapeAndCacheParam()
    rp2.kvCacheCfg = 7
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, rp2)
    rp3 = capi.ReshapeAndCacheParam()
    rp3.rsv[0] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, rp3)


def test_input_output_counts():
    assert capi.Operation(_pa_param()).input_num == 5
    assert capi.Operation(_pa_param(quantType=1)).input_num == 7
    assert capi.Operation(_pa_param(quantType=1, hasQuantOffset=True)).input_num == 9
    assert capi.Operation(_pa_param(mlaVHeadSize=512, kvHeadNum=1)).input_num == 4
    assert capi.Operation(capi.ReshapeAndCacheParam()).input_num == 5
    siso = capi.ReshapeAndCacheParam()
    siso.kvCacheCfg = 1
    op = capi.Operation(siso)
    assert (op.input_num, op.output_num) == (3, 1)


def _pa_tensors(batch=3, heads=8, kvh=2, d=128, bs=128, nb=16, maxb=4, dtype=capi.ACL_FLOAT16, lens=None):
    T = capi.atb_tensor
    lens = np.array([5, 130, 400], dtype=np.int32) if lens is None else lens
    fake = 0x1000
    ins = [T(dtype=dtype, shape=(batch, heads, d), device_ptr=fake), T(dtype=dtype, shape=(nb, bs, kvh, d), device_ptr=fake),
           T(dtype=dtype, shape=(nb, bs, kvh, d), device_ptr=fake), T(dtype=capi.ACL_INT32, shape=(batch, maxb), device_ptr=fake),
           T(dtype=capi.ACL_INT32, shape=(batch,), device_ptr=fake, host=lens)]
    outs = [T(dtype=dtype, shape=(batch, heads, d), device_ptr=fake)]
    return ins, outs, lens


def test_setup_checks_and_plan_without_gpu(monkeypatch):
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    op = capi.Operation(_pa_param())
    ctx = capi.Context()
    ins, outs, lens = _pa_tensors()
    assert op.infer_shape(ins, 1) == [(3, 8, 128)]
    ws = op.setup(ins, outs, ctx)
    assert ws >= 256
    # wrong tensor count
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, op.setup, ins[:4], outs, ctx)
    # dtype combination not allowed (int8 cache without dequant fusion)
    bad = list(ins)
    bad[1] = capi.atb_tensor(dtype=capi.ACL_INT8, shape=(16, 128, 2, 128), device_ptr=0x1000)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, bad, outs, ctx)
    # key cache must be 4-D
    bad = list(ins)
    bad[1] = capi.atb_tensor(dtype=capi.ACL_FLOAT16, shape=(16, 128, 256), device_ptr=0x1000)
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.setup, bad, outs, ctx)
    # head size mismatch between query and key cache
    bad = list(ins)
    bad[0] = capi.atb_tensor(dtype=capi.ACL_FLOAT16, shape=(3, 8, 64), device_ptr=0x1000)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, bad, outs, ctx)
    # output head size must equal the value head size
    bad_out = [capi.atb_tensor(dtype=capi.ACL_FLOAT16, shape=(3, 8, 64), device_ptr=0x1000)]
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, ins, bad_out, ctx)
    # contextLens without hostData
    bad = list(ins)
    bad[4] = capi.atb_tensor(dtype=capi.ACL_INT32, shape=(3,), device_ptr=0x1000)
    _expect(capi.ERROR_INVALID_PARAM, op.setup, bad, outs, ctx)
    # null context
    _expect(capi.ERROR_INVALID_PARAM, op.setup, ins, outs, None)
    # zero-sized dim
    bad = list(ins)
    bad[3] = capi.atb_tensor(dtype=capi.ACL_INT32, shape=(3, 0), device_ptr=0x1000)
    _expect(capi.ERROR_INVALID_TENSOR_SIZE, op.setup, bad, outs, ctx)


def test_batch_run_status_switches_sequences_off(monkeypatch):
    """Dynamic batch (batchRunStatusEnable): one more host tensor after contextLens; a sequence whose status is
    0 is planned as empty.  The plan is observed through the workspace size (split-KV partials need room)."""
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    T = capi.atb_tensor
    ctx = capi.Context()
    long_lens = np.array([5, 40000, 40000], dtype=np.int32)
    ins, outs, _ = _pa_tensors(maxb=320, nb=1024, lens=long_lens)
    plain = capi.Operation(_pa_param())
    ws_all = plain.setup(ins, outs, ctx)
    ins0, _, _ = _pa_tensors(maxb=320, nb=1024, lens=np.array([5, 0, 0], dtype=np.int32))
    ws_first_only = capi.Operation(_pa_param()).setup(ins0, outs, ctx)
    assert ws_first_only < ws_all

    op = capi.Operation(_pa_param(batchRunStatusEnable=True))
    assert op.input_num == 6
    status = np.array([1, 0, 0], dtype=np.int32)
    with_status = ins + [T(dtype=capi.ACL_INT32, shape=(3,), device_ptr=0x1000, host=status)]
    assert op.infer_shape(with_status, 1) == [(3, 8, 128)]
    assert op.setup(with_status, outs, ctx) == ws_first_only
    status[:] = 1
    assert op.setup(with_status, outs, ctx) == ws_all
    # the status tensor must carry host data, one value per query token
    bad = ins + [T(dtype=capi.ACL_INT32, shape=(3,), device_ptr=0x1000)]
    _expect(capi.ERROR_INVALID_PARAM, op.setup, bad, outs, ctx)
    bad = ins + [T(dtype=capi.ACL_INT32, shape=(2,), device_ptr=0x1000, host=status[:2].copy())]
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, bad, outs, ctx)
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, op.setup, ins, outs, ctx)
    # the control tensors may describe more sequences than there are query tokens, never fewer
    lens5 = np.array([5, 40000, 40000, 7, 9], dtype=np.int32)
    more = list(with_status)
    more[3] = T(dtype=capi.ACL_INT32, shape=(5, 320), device_ptr=0x1000)
    more[4] = T(dtype=capi.ACL_INT32, shape=(5,), device_ptr=0x1000, host=lens5)
    assert op.setup(more, outs, ctx) == ws_all
    fewer = list(with_status)
    fewer[4] = T(dtype=capi.ACL_INT32, shape=(2,), device_ptr=0x1000, host=lens5[:2].copy())
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, fewer, outs, ctx)
    # with the int8 cache the scales follow the status tensor
    q8 = capi.Operation(_pa_param(batchRunStatusEnable=True, quantType=1))
    assert q8.input_num == 8


def test_execute_contract_without_gpu(monkeypatch):
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    op = capi.Operation(_pa_param())
    ctx = capi.Context()
    ins, outs, _ = _pa_tensors()
    # Execute before Setup
    _expect(capi.ERROR_INVALID_PARAM, op.execute, ins, outs, None, 0, ctx)
    ws = op.setup(ins, outs, ctx)
    # the context has no stream yet
    _expect(capi.ERROR_INVALID_PARAM, op.execute, ins, outs, 0x2000, ws, ctx)
    ctx.set_stream(0x3000)
    # another context than the one given to Setup
    other = capi.Context(0x3000)
    _expect(capi.ERROR_INVALID_PARAM, op.execute, ins, outs, 0x2000, ws, other)
    # workspace smaller than Setup asked for / null workspace
    _expect(capi.ERROR_INVALID_PARAM, op.execute, ins, outs, 0x2000, ws - 1, ctx)
    _expect(capi.ERROR_INVALID_PARAM, op.execute, ins, outs, None, ws, ctx)
    # dataSize differs from Setup's
    bad = list(ins)
    bad[0] = capi.atb_tensor(dtype=capi.ACL_FLOAT16, shape=(3, 8, 128), device_ptr=0x1000)
    bad[0].data_size -= 2
    _expect(capi.ERROR_INVALID_PARAM, op.execute, bad, outs, 0x2000, ws, ctx)
    # a tensor with neither device nor host data
    bad = list(ins)
    bad[0] = capi.atb_tensor(dtype=capi.ACL_FLOAT16, shape=(3, 8, 128), device_ptr=None)
    _expect(capi.ERROR_INVALID_PARAM, op.execute, bad, outs, 0x2000, ws, ctx)


def test_reshape_and_cache_setup_checks():
    T = capi.atb_tensor
    op = capi.Operation(capi.ReshapeAndCacheParam())
    ctx = capi.Context()
    f = 0x1000
    ins = [T(dtype=capi.ACL_BF16, shape=(4, 8, 128), device_ptr=f), T(dtype=capi.ACL_BF16, shape=(4, 8, 64), device_ptr=f),
           T(dtype=capi.ACL_BF16, shape=(10, 128, 8, 128), device_ptr=f), T(dtype=capi.ACL_BF16, shape=(10, 128, 8, 64), device_ptr=f),
           T(dtype=capi.ACL_INT32, shape=(4,), device_ptr=f)]
    outs = [ins[2], ins[3]]
    assert op.setup(ins, outs, ctx) == 0
    assert op.infer_shape(ins, 2) == [(10, 128, 8, 128), (10, 128, 8, 64)]
    bad = list(ins)
    bad[1] = T(dtype=capi.ACL_BF16, shape=(5, 8, 64), device_ptr=f)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, bad, outs, ctx)
    bad = list(ins)
    bad[2] = T(dtype=capi.ACL_BF16, shape=(10, 128, 8 * 128), device_ptr=f)
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.setup, bad, [bad[2], ins[3]], ctx)
    # outputs must describe the caches
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, ins, [ins[3], ins[3]], ctx)
    # mixed dtypes
    bad = list(ins)
    bad[0] = T(dtype=capi.ACL_FLOAT16, shape=(4, 8, 128), device_ptr=f)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, bad, outs, ctx)


# ------------------------------------------------------------------ MultiLatentAttentionOperation

def _mla_param(**kw):
    base = dict(headNum=128, kvHeadNum=1, qkScale=0.0417, cacheMode=1)
    base.update(kw)
    return capi.MultiLatentAttentionParam(**base)


def _mla_tensors(batch=3, heads=128, nb=16, maxb=4, dtype=capi.ACL_BF16, lens=None):
    T = capi.atb_tensor
    lens = np.array([5, 130, 400], dtype=np.int32) if lens is None else lens
    fake = 0x1000
    ins = [T(dtype=dtype, shape=(batch, heads, 512), device_ptr=fake), T(dtype=dtype, shape=(batch, heads, 64), device_ptr=fake),
           T(dtype=dtype, shape=(nb, 128, 1, 512), device_ptr=fake), T(dtype=dtype, shape=(nb, 128, 1, 64), device_ptr=fake),
           T(dtype=capi.ACL_INT32, shape=(batch, maxb), device_ptr=fake),
           T(dtype=capi.ACL_INT32, shape=(batch,), device_ptr=fake, host=lens)]
    outs = [T(dtype=dtype, shape=(batch, heads, 512), device_ptr=fake)]
    return ins, outs


def test_multi_latent_attention_param_checks():
    # tests/unittest/ops/test_op_param_size.cpp:68 of the reference
    assert ctypes.sizeof(capi.MultiLatentAttentionParam) == 64
    op = capi.Operation(_mla_param())
    assert (op.name, op.input_num, op.output_num) == ("MultiLatentAttentionOperation", 6, 1)
    for bad in (dict(qkScale=0.0), dict(qkScale=1.5), dict(headNum=24), dict(kvHeadNum=2), dict(cacheMode=0),
                dict(cacheMode=9), dict(maskType=7), dict(calcType=9),
                dict(maskType=1), dict(maskType=2, calcType=2),            # only mtp (CALC_TYPE_SPEC) supports masks
                # forms of the reference this build does not carry
                dict(calcType=4), dict(maskType=3, calcType=1), dict(maskType=4, calcType=1, windowSize=8),
                dict(cacheMode=2), dict(cacheMode=3), dict(maskUseStatusType=1, calcType=3)):
        _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _mla_param(**bad))
    p = _mla_param()
    p.rsv[31] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, p)


def test_multi_latent_attention_setup_checks(monkeypatch):
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    op = capi.Operation(_mla_param())
    ctx = capi.Context()
    ins, outs = _mla_tensors()
    assert op.infer_shape(ins, 1) == [(3, 128, 512)]
    assert op.setup(ins, outs, ctx) >= 256
    T = capi.atb_tensor

    def swapped(i, **kw):
        bad = list(ins)
        bad[i] = T(device_ptr=0x1000, **kw)
        return bad
    bf = capi.ACL_BF16
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, op.setup, ins[:5], outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, swapped(1, dtype=capi.ACL_FLOAT16, shape=(3, 128, 64)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.setup, swapped(2, dtype=bf, shape=(16, 128, 512)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(2, dtype=bf, shape=(16, 64, 1, 512)), outs, ctx)   # block size
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(3, dtype=bf, shape=(15, 128, 1, 64)), outs, ctx)   # block count
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(0, dtype=bf, shape=(3, 64, 512)), outs, ctx)       # heads
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(1, dtype=bf, shape=(3, 128, 32)), outs, ctx)       # rope width
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(0, dtype=bf, shape=(4, 128, 512)), outs, ctx)      # tokens != batch
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, ins, [T(dtype=bf, shape=(3, 128, 576), device_ptr=0x1000)], ctx)
    _expect(capi.ERROR_INVALID_PARAM, op.setup, swapped(5, dtype=capi.ACL_INT32, shape=(3,)), outs, ctx)        # no host lens
    # CALC_TYPE_RING: the log-sum-exp [tokens, heads, 1] is a second output
    ring = capi.Operation(_mla_param(calcType=2))
    assert (ring.input_num, ring.output_num) == (6, 2)
    assert ring.infer_shape(ins, 2) == [(3, 128, 512), (3, 128, 1)]
    lse = T(dtype=bf, shape=(3, 128, 1), device_ptr=0x1000)
    assert ring.setup(ins, outs + [lse], ctx) >= 256
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, ring.setup, ins, outs, ctx)            # wrong tensor count
    _expect(capi.ERROR_INVALID_TENSOR_DIM, ring.setup, ins, outs + [T(dtype=bf, shape=(3, 128, 512), device_ptr=0x1000)], ctx)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, ring.setup, ins,
            outs + [T(dtype=capi.ACL_FLOAT, shape=(3, 128, 1), device_ptr=0x1000)], ctx)
    # CALC_TYPE_SPEC (MTP): qSeqLens as host data after the optional mask; one planned row per query token
    qlens = np.array([2, 1, 2], dtype=np.int32)
    spec_ins = [T(dtype=bf, shape=(5, 128, 512), device_ptr=0x1000), T(dtype=bf, shape=(5, 128, 64), device_ptr=0x1000)] + ins[2:]
    spec_outs = [T(dtype=bf, shape=(5, 128, 512), device_ptr=0x1000)]
    ql = T(dtype=capi.ACL_INT32, shape=(3,), device_ptr=0x1000, host=qlens)
    nomask = capi.Operation(_mla_param(calcType=1))
    assert nomask.input_num == 7
    assert nomask.setup(spec_ins + [ql], spec_outs, ctx) >= 256
    _expect(capi.ERROR_INVALID_PARAM, nomask.setup, spec_ins + [T(dtype=capi.ACL_INT32, shape=(3,), device_ptr=0x1000)],
            spec_outs, ctx)                                                                              # no host qSeqLens
    _expect(capi.ERROR_INVALID_PARAM, nomask.setup,
            spec_ins + [T(dtype=capi.ACL_INT32, shape=(3,), device_ptr=0x1000, host=np.array([2, 2, 2], dtype=np.int32))],
            spec_outs, ctx)                                                                              # sum != tokens
    _expect(capi.ERROR_INVALID_TENSOR_DIM, nomask.setup, spec_ins + [T(dtype=capi.ACL_INT32, shape=(2,), device_ptr=0x1000,
                                                                      host=qlens)], spec_outs, ctx)
    masked = capi.Operation(_mla_param(calcType=3, maskType=1))                                          # SPEC_AND_RING + spec mask
    assert (masked.input_num, masked.output_num) == (8, 2)
    m_ok = T(dtype=bf, shape=(5, 400), device_ptr=0x1000)
    lse5 = T(dtype=bf, shape=(5, 128, 1), device_ptr=0x1000)
    assert masked.setup(spec_ins + [m_ok, ql], spec_outs + [lse5], ctx) >= 256
    _expect(capi.ERROR_INVALID_TENSOR_DIM, masked.setup, spec_ins + [T(dtype=bf, shape=(4, 400), device_ptr=0x1000), ql],
            spec_outs + [lse5], ctx)                                                                     # a row per token
    _expect(capi.ERROR_INVALID_TENSOR_DIM, masked.setup, spec_ins + [T(dtype=bf, shape=(5, 399), device_ptr=0x1000), ql],
            spec_outs + [lse5], ctx)                                                                     # shorter than a context
    free = capi.Operation(_mla_param(calcType=1, maskType=2))                                            # MASK_FREE: causal
    assert free.setup(spec_ins + [T(dtype=bf, shape=(129, 128), device_ptr=0x1000), ql], spec_outs, ctx) >= 256
    # execute before a successful setup of these tensors is refused without touching the device
    op2 = capi.Operation(_mla_param())
    _expect(capi.ERROR_INVALID_PARAM, op2.execute, ins, outs, 0x1000, 1 << 20, ctx)


# ------------------------------------------------------------------ masks and logN scaling

def test_mask_and_logn_param_rules():
    assert capi.Operation(_pa_param(maskType=1)).input_num == 6            # NORM
    assert capi.Operation(_pa_param(maskType=2)).input_num == 6            # ALIBI
    assert capi.Operation(_pa_param(scaleType=1)).input_num == 6           # logN
    assert capi.Operation(_pa_param(maskType=2, scaleType=1, batchRunStatusEnable=True)).input_num == 8
    assert capi.Operation(_pa_param(maskType=1, quantType=1, hasQuantOffset=True)).input_num == 10
    for bad in (dict(maskType=3), dict(maskType=4), dict(maskType=5),      # SPEC, MASK_FREE, NORM_COMPRESS
                dict(scaleType=1, quantType=1), dict(scaleType=2),
                dict(mlaVHeadSize=512, kvHeadNum=1, maskType=2), dict(mlaVHeadSize=512, kvHeadNum=1, scaleType=1)):
        _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(**bad))


def test_mask_and_logn_setup_checks(monkeypatch):
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    T = capi.atb_tensor
    ctx = capi.Context()
    f16, fake = capi.ACL_FLOAT16, 0x1000
    ins, outs, lens = _pa_tensors()                                        # batch 3, 8 heads, longest context 400

    def with_extra(*extra):
        return list(ins) + list(extra)
    norm = capi.Operation(_pa_param(maskType=1))
    assert norm.setup(with_extra(T(dtype=f16, shape=(3, 1, 512), device_ptr=fake)), outs, ctx) >= 256
    assert norm.setup(with_extra(T(dtype=f16, shape=(1, 400), device_ptr=fake)), outs, ctx) >= 256
    _expect(capi.ERROR_INVALID_TENSOR_DIM, norm.setup, with_extra(T(dtype=f16, shape=(3, 1, 399), device_ptr=fake)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, norm.setup, with_extra(T(dtype=f16, shape=(2, 1, 512), device_ptr=fake)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, norm.setup, with_extra(T(dtype=f16, shape=(512, 512), device_ptr=fake)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, norm.setup, with_extra(T(dtype=f16, shape=(3, 8, 1, 512), device_ptr=fake)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, norm.setup,
            with_extra(T(dtype=capi.ACL_BF16, shape=(3, 1, 512), device_ptr=fake)), outs, ctx)   # mask dtype = query dtype
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, norm.setup, ins, outs, ctx)
    alibi = capi.Operation(_pa_param(maskType=2))
    assert alibi.setup(with_extra(T(dtype=f16, shape=(3, 8, 1, 400), device_ptr=fake)), outs, ctx) >= 256
    assert alibi.setup(with_extra(T(dtype=f16, shape=(8, 1, 400), device_ptr=fake)), outs, ctx) >= 256
    _expect(capi.ERROR_INVALID_TENSOR_DIM, alibi.setup, with_extra(T(dtype=f16, shape=(3, 4, 1, 400), device_ptr=fake)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, alibi.setup, with_extra(T(dtype=f16, shape=(1, 400), device_ptr=fake)), outs, ctx)
    logn = capi.Operation(_pa_param(scaleType=1))
    assert logn.setup(with_extra(T(dtype=capi.ACL_FLOAT, shape=(3,), device_ptr=fake)), outs, ctx) >= 256
    _expect(capi.ERROR_INVALID_TENSOR_DIM, logn.setup, with_extra(T(dtype=capi.ACL_FLOAT, shape=(4,), device_ptr=fake)), outs, ctx)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, logn.setup, with_extra(T(dtype=f16, shape=(3,), device_ptr=fake)), outs, ctx)
    both = capi.Operation(_pa_param(maskType=2, scaleType=1))
    assert both.setup(with_extra(T(dtype=f16, shape=(8, 1, 400), device_ptr=fake),
                                 T(dtype=capi.ACL_FLOAT, shape=(3,), device_ptr=fake)), outs, ctx) >= 256


def test_planner_routes_score_modifiers():
    lens = np.array([100, 900], dtype=np.int32)

    def plan(dk=128, kv="bf16", mods=capi.SCORE_MASK, kernel=0, **kw):
        d = capi.make_desc(2, 8, 2, dk, dk, 128, 64, 8, "bf16", kv, sm_count=148, score_mods=mods, kernel=kernel, **kw)
        return capi.PaPlan(d, lens).info.kernel
    assert plan() == capi.KERNEL_TMA_MMA
    assert plan(mods=capi.SCORE_LOGN | capi.SCORE_MASK) == capi.KERNEL_TMA_MMA
    assert plan(dk=64) == capi.KERNEL_TMA_MMA and plan(dk=256) == capi.KERNEL_TMA_MMA
    assert plan(dk=96) == capi.KERNEL_TMA_MMA and plan(dk=192) == capi.KERNEL_TMA_MMA   # multiples of 16: padded geometry
    assert plan(dk=72) == capi.KERNEL_GENERIC
    assert plan(kv="int8") == capi.KERNEL_GENERIC                          # the int8 TMA kernel carries no mask code
    assert plan(kernel=capi.KERNEL_GENERIC) == capi.KERNEL_GENERIC
    _expect(capi.ERROR_INVALID_TENSOR_DIM, plan, kv="int8", kernel=capi.KERNEL_TMA_MMA)
    _expect(capi.ERROR_INVALID_PARAM, plan, mods=8)
    mla = lambda mods: capi.PaPlan(capi.make_desc(2, 8, 1, 576, 512, 128, 64, 8, "bf16", sm_count=148, v_row_dim=512,
                                                  rope_dim=64, score_mods=mods), lens).info.kernel
    assert mla(capi.SCORE_MASK | capi.SCORE_ROWS) == capi.KERNEL_MLA_TC5    # per-token mask rows on the split MLA cache
    with pytest.raises(capi.AtbError):                                     # no logN scaling in the MLA kernel
        mla(capi.SCORE_LOGN)


def test_launch_refuses_missing_or_short_mask_before_touching_the_device():
    lens = np.array([100, 900], dtype=np.int32)
    d = capi.make_desc(2, 8, 2, 128, 128, 128, 64, 8, "bf16", sm_count=148, score_mods=capi.SCORE_MASK | capi.SCORE_LOGN)
    plan = capi.PaPlan(d, lens)
    t = capi.PaTensors()
    for f in ("q", "k_cache", "v_cache", "block_tables", "out"):
        setattr(t, f, 0x1000)
    _expect(capi.ERROR_INVALID_PARAM, plan.launch, t, 0x1000, 1 << 30, None)          # no mask
    t.mask, t.mask_tokens = 0x1000, 899
    _expect(capi.ERROR_INVALID_PARAM, plan.launch, t, 0x1000, 1 << 30, None)          # shorter than the longest context
    t.mask_tokens = 900
    _expect(capi.ERROR_INVALID_PARAM, plan.launch, t, 0x1000, 1 << 30, None)          # no logN factors


def test_bnsd_layout_rules(monkeypatch):
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    T = capi.atb_tensor
    ctx = capi.Context()
    f16, fake = capi.ACL_FLOAT16, 0x1000
    op = capi.Operation(_pa_param(inputLayout=1))
    for bad in (dict(inputLayout=1, quantType=1), dict(inputLayout=1, scaleType=1), dict(inputLayout=1, calcType=1),
                dict(inputLayout=2), dict(inputLayout=1, mlaVHeadSize=512, kvHeadNum=1)):
        _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(**bad))
    lens = np.array([5, 130, 400], dtype=np.int32)
    ins = [T(dtype=f16, shape=(3, 8, 128), device_ptr=fake), T(dtype=f16, shape=(16, 2, 64, 128), device_ptr=fake),
           T(dtype=f16, shape=(16, 2, 64, 128), device_ptr=fake), T(dtype=capi.ACL_INT32, shape=(3, 8), device_ptr=fake),
           T(dtype=capi.ACL_INT32, shape=(3,), device_ptr=fake, host=lens)]
    outs = [T(dtype=f16, shape=(3, 8, 128), device_ptr=fake)]
    assert op.setup(ins, outs, ctx) >= 256
    bad = list(ins)                                                        # token-major blocks given to a BNSD operation
    bad[1] = bad[2] = T(dtype=f16, shape=(16, 64, 2, 128), device_ptr=fake)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, bad, outs, ctx)
    # kernel level: heads-major blocks exist for fp16 / bf16 caches without the split MLA cache
    d = capi.make_desc(3, 8, 2, 128, 128, 64, 16, 8, "fp16", sm_count=148, kv_layout=1)
    assert capi.PaPlan(d, lens).info.kernel == capi.KERNEL_TMA_MMA
    assert capi.PaPlan(capi.make_desc(3, 8, 2, 72, 72, 64, 16, 8, "fp16", sm_count=148, kv_layout=1),
                       lens).info.kernel == capi.KERNEL_GENERIC
    _expect(capi.ERROR_INVALID_PARAM, capi.PaPlan, capi.make_desc(3, 8, 2, 128, 128, 64, 16, 8, "fp16", "int8", sm_count=148,
                                                                   kv_layout=1), lens)
    _expect(capi.ERROR_INVALID_PARAM, capi.PaPlan, capi.make_desc(3, 8, 2, 128, 128, 64, 16, 8, "fp16", sm_count=148,
                                                                   kv_layout=2), lens)


# ------------------------------------------------------------------ parallel decoding (CALC_TYPE_SPEC)

def test_parallel_decoding_param_and_setup_rules(monkeypatch):
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    T = capi.atb_tensor
    ctx = capi.Context()
    f16, i32, fake = capi.ACL_FLOAT16, capi.ACL_INT32, 0x1000
    assert capi.Operation(_pa_param(calcType=1, maskType=3)).input_num == 7
    assert capi.Operation(_pa_param(calcType=1, maskType=1)).input_num == 7
    for bad in (dict(calcType=1), dict(calcType=1, maskType=2), dict(calcType=1, maskType=3, batchRunStatusEnable=True),
                dict(maskType=3), dict(calcType=2, maskType=3), dict(calcType=1, maskType=3, scaleType=1),
                dict(calcType=1, maskType=3, inputLayout=1), dict(calcType=1, maskType=3, quantType=1)):
        _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pa_param(**bad))
    lens = np.array([40, 300], dtype=np.int32)
    qlens = np.array([3, 2], dtype=np.int32)

    def tensors(tokens=5, mask_shape=(5, 300), qlens=qlens, bs=128):
        ins = [T(dtype=f16, shape=(tokens, 8, 128), device_ptr=fake), T(dtype=f16, shape=(16, bs, 2, 128), device_ptr=fake),
               T(dtype=f16, shape=(16, bs, 2, 128), device_ptr=fake), T(dtype=i32, shape=(2, 4), device_ptr=fake),
               T(dtype=i32, shape=(2,), device_ptr=fake, host=lens), T(dtype=f16, shape=mask_shape, device_ptr=fake),
               T(dtype=i32, shape=(2,), device_ptr=fake, host=qlens)]
        return ins, [T(dtype=f16, shape=(tokens, 8, 128), device_ptr=fake)]
    spec = capi.Operation(_pa_param(calcType=1, maskType=3))
    assert spec.setup(*tensors(), ctx) >= 256
    _expect(capi.ERROR_INVALID_PARAM, spec.setup, *tensors(tokens=6, mask_shape=(6, 300)), ctx)       # sum(qSeqLens) != tokens
    _expect(capi.ERROR_INVALID_TENSOR_DIM, spec.setup, *tensors(mask_shape=(4, 300)), ctx)            # a mask row per token
    _expect(capi.ERROR_INVALID_TENSOR_DIM, spec.setup, *tensors(mask_shape=(5, 299)), ctx)            # shorter than a context
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, spec.setup, *tensors(mask_shape=(5, 1, 300)), ctx)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, spec.setup, *tensors(bs=256), ctx)
    ins, outs = tensors()
    ins[6] = T(dtype=i32, shape=(2,), device_ptr=fake)                                                # qSeqLens without host data
    _expect(capi.ERROR_INVALID_PARAM, spec.setup, ins, outs, ctx)
    norm = capi.Operation(_pa_param(calcType=1, maskType=1))
    assert norm.setup(*tensors(mask_shape=(512, 512)), ctx) >= 256
    _expect(capi.ERROR_INVALID_TENSOR_DIM, norm.setup, *tensors(mask_shape=(5, 512)), ctx)            # must be square
    _expect(capi.ERROR_INVALID_PARAM, norm.setup, *tensors(tokens=43, mask_shape=(512, 512),
                                                            qlens=np.array([41, 2], dtype=np.int32)), ctx)  # q_len > ctx


def test_plan_rows_contract():
    lens = np.array([40, 40, 40, 300, 300], dtype=np.int32)
    d = capi.make_desc(5, 8, 2, 128, 128, 128, 16, 4, "fp16", sm_count=148, score_mods=capi.SCORE_ROWS | capi.SCORE_MASK)
    plan = capi.PaPlan(d, lens)
    plan.set_rows([0, 0, 0, 1, 1], 2, [0, 1, 2, 3, 4], 5)
    _expect(capi.ERROR_INVALID_PARAM, plan.set_rows, [0, 0, 0, 1, 2], 2, [0, 1, 2, 3, 4], 5)       # block-table row out of range
    _expect(capi.ERROR_INVALID_PARAM, plan.set_rows, [0, 0, 0, 1, 1], 2, [0, 1, 2, 3, 5], 5)       # mask row out of range
    _expect(capi.ERROR_INVALID_PARAM, plan.set_rows, [0, 0, 0, 1, 1], 2, None, 0)                  # masked plan needs mask rows
    plain = capi.PaPlan(capi.make_desc(5, 8, 2, 128, 128, 128, 16, 4, "fp16", sm_count=148), lens)
    _expect(capi.ERROR_INVALID_PARAM, plain.set_rows, [0, 0, 0, 1, 1], 2)                          # not a SCORE_ROWS plan
    plan.update(lens + 1)                                                                          # rows survive a re-plan
    assert plan.info.plan_bytes > plain.info.plan_bytes - 256


def test_fused_parallel_decoding_plan_rules(monkeypatch):
    """q_per_seq > 1: one planned row per sequence whose CTA columns are (token, head) pairs - the D = 128 fp16 / bf16
    kernel only, at most 8 pairs per kv head."""
    lens = np.array([100, 900], dtype=np.int32)

    def plan(heads=16, kvh=4, n=2, dk=128, kv="bf16", kernel=0):
        d = capi.make_desc(2, heads, kvh, dk, dk, 128, 64, 8, "bf16", kv, sm_count=148, score_mods=capi.SCORE_MASK,
                           q_per_seq=n, kernel=kernel)
        return capi.PaPlan(d, lens).info.kernel
    assert plan() == capi.KERNEL_TMA_MMA                                   # 2 tokens x 2 heads per kv head
    assert plan(heads=32, kvh=4, n=2) == capi.KERNEL_TMA_MMA               # 8 pairs
    _expect(capi.ERROR_INVALID_TENSOR_DIM, plan, heads=48, kvh=4, n=3)     # 12 pairs
    assert plan(dk=64) == capi.KERNEL_TMA_MMA                              # head sizes 64 / 128 / 256
    assert plan(dk=96) == capi.KERNEL_TMA_MMA                              # padded on the 128 geometry
    _expect(capi.ERROR_INVALID_TENSOR_DIM, plan, dk=72)
    _expect(capi.ERROR_INVALID_TENSOR_DIM, plan, kv="int8")
    _expect(capi.ERROR_INVALID_TENSOR_DIM, plan, kernel=capi.KERNEL_GENERIC)
    _expect(capi.ERROR_INVALID_PARAM, plan, heads=18, kvh=2, n=4)          # heads not a multiple of the token count
    # the causal rule needs several query tokens per sequence; the MLA kernel takes any number of (token, head) rows
    _expect(capi.ERROR_INVALID_PARAM, capi.PaPlan,
            capi.make_desc(2, 8, 2, 128, 128, 128, 64, 8, "bf16", sm_count=148, score_mods=capi.SCORE_CAUSAL), lens)
    mla = capi.make_desc(2, 3 * 128, 1, 576, 512, 128, 64, 8, "bf16", sm_count=148, v_row_dim=512, rope_dim=64,
                         score_mods=capi.SCORE_CAUSAL, q_per_seq=3)
    info = capi.PaPlan(mla, lens).info
    assert info.kernel == capi.KERNEL_MLA_TC5 and info.num_ctas % 6 == 0       # 384 rows = 6 CTAs per token range
    # the operator plans uniform qSeqLens this way and falls back to one row per token where it cannot
    monkeypatch.setenv("ATB_B200_SM_COUNT", "148")
    T = capi.atb_tensor
    f16, i32, fake = capi.ACL_FLOAT16, capi.ACL_INT32, 0x1000
    ctx = capi.Context()
    qlens = np.array([2, 2], dtype=np.int32)
    for d, expect_ws in ((128, None), (96, None)):
        ins = [T(dtype=f16, shape=(4, 8, d), device_ptr=fake), T(dtype=f16, shape=(16, 128, 2, d), device_ptr=fake),
               T(dtype=f16, shape=(16, 128, 2, d), device_ptr=fake), T(dtype=i32, shape=(2, 8), device_ptr=fake),
               T(dtype=i32, shape=(2,), device_ptr=fake, host=lens), T(dtype=f16, shape=(4, 900), device_ptr=fake),
               T(dtype=i32, shape=(2,), device_ptr=fake, host=qlens)]
        outs = [T(dtype=f16, shape=(4, 8, d), device_ptr=fake)]
        op = capi.Operation(_pa_param(calcType=1, maskType=3))
        assert op.setup(ins, outs, ctx) >= 256
        assert op.setup(ins, outs, ctx) >= 256                              # second Setup re-plans in place


def test_ctypes_mirror_matches_the_c_header(tmp_path):
    """The header is plain C: compile a probe against it and compare sizes and field offsets with the ctypes mirror."""
    import subprocess
    fields = {"atb_b200_pa_desc": (capi.PaDesc, ["qk_scale", "rope_dim", "score_mods", "kv_layout", "q_per_seq"]),
              "atb_b200_pa_tensors": (capi.PaTensors, ["out", "q_rope", "mask", "mask_tokens", "mask_q_stride", "logn", "lse_out"]),
              "atb_b200_pa_plan_info": (capi.PaPlanInfo, ["workspace_bytes", "kernels_per_launch"]),
              "atb_b200_pa_peers": (capi.PaPeers, ["peer_out", "peer_flags", "epoch"])}
    lines = []
    for name, (_, names) in fields.items():
        lines.append(f'printf("%zu", sizeof({name}));')
        lines += [f'printf(" %zu", offsetof({name}, {f}));' for f in names]
        lines.append('printf("\\n");')
    src = tmp_path / "probe.c"
    src.write_text('#include <stddef.h>\n#include <stdio.h>\n#include "atb_b200.h"\nint main(void) {\n' + "\n".join(lines) +
                   "\nreturn 0;\n}\n")
    exe = tmp_path / "probe"
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = subprocess.check_output([str(exe)], text=True).strip().splitlines()
    for line, (name, (cls, names)) in zip(out, fields.items()):
        want = [ctypes.sizeof(cls)] + [getattr(cls, f).offset for f in names]
        assert [int(x) for x in line.split()] == want, name


def test_mla_plan_weighs_token_ranges():
    """The MLA kernel pays for every token range it starts about as much as for six tiles; its plan packs
    cost = tiles + 6 x ranges evenly, so groups that straddle a sequence boundary get fewer tiles."""
    case = wl.CONFIGS[4]
    plan, lens = _plan(case)
    info = plan.info
    assert info.kernel == capi.KERNEL_MLA_TC5
    items, groups = plan.dump()
    n_groups = info.num_ctas // 2
    tiles = np.array([sum((e - b + 63) // 64 for _, b, e, _ in items[groups[g]:groups[g + 1]]) for g in range(n_groups)])
    ranges = np.array([groups[g + 1] - groups[g] for g in range(n_groups)])
    cost = tiles + 6 * ranges
    total = int(((lens.astype(np.int64) + 63) // 64).sum())
    assert tiles.sum() == total
    assert cost.max() <= (total + 6 * len(items)) / n_groups + 7           # within one range of the mean cost
    assert tiles[ranges == 2].max() < tiles[ranges == 1].max()            # two ranges -> fewer tiles
