"""BlockCopy and PagedCacheLoad without a GPU: the CUDA kernels' per-thread bodies (csrc/cache_ops_body.h)
run on the CPU over an emulated grid and must reproduce the reference goldens bit for bit; an
AddressSanitizer build of the same bodies takes randomized and hostile inputs; the C ABI rejects bad
arguments before any launch."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import oracle
from golden_cases import (GOLDEN_BLOCKCOPY_CASES, GOLDEN_KVCACHE_CASES, GOLDEN_PCL_CASES, HERE as GOLDEN_DIR, blockcopy_inputs,
                          kvcache_inputs, pcl_inputs)
from helpers import capi, pkg

_emu = None


def emu():
    global _emu
    if _emu is None:
        L = ctypes.CDLL(pkg._build.build_host_emulation())
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        L.emu_block_copy.argtypes = [vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, i32, i32]
        L.emu_paged_cache_load.argtypes = [vp] * 7 + [i32, i32, i32, i64, i64, i64, i64, i32, vp, i32, i32]
        L.emu_rac_strided.argtypes = [vp] * 5 + [i32, i64, i64, i64, i64, i64, i32, i32]
        L.emu_kv_cache.argtypes = [vp] * 5 + [i64, i32, i32, i32, i64, i32, i32]
        _emu = L
    return _emu


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _bits(a):
    return a.view(np.uint16) if a.dtype == np.float16 else a


def test_kernel_bodies_survive_address_sanitizer():
    exe = pkg._build.build_body_selftest()
    r = subprocess.run([exe, "300"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failures" in r.stdout


@pytest.mark.parametrize("chunks,threads", [(0, 4), (1, 1), (3, 5)])
@pytest.mark.parametrize("spec", GOLDEN_BLOCKCOPY_CASES, ids=lambda s: s["name"])
def test_block_copy_body_matches_reference_golden(spec, chunks, threads):
    fx = np.load(os.path.join(GOLDEN_DIR, f"blockcopy_{spec['name']}.npz"))
    inp = blockcopy_inputs(spec)
    k, v = inp["k_cache"].copy(), inp["v_cache"].copy()
    emu().emu_block_copy(_p(k), _p(v), _p(inp["src"]), _p(inp["dst"]), _p(inp["cum"]), len(inp["src"]), len(inp["dst"]),
                         k[0].nbytes, v[0].nbytes, k.shape[0], chunks, threads)
    assert np.array_equal(_bits(k), _bits(fx["k_cache"])) and np.array_equal(_bits(v), _bits(fx["v_cache"]))


@pytest.mark.parametrize("cumulative", [True, False])
@pytest.mark.parametrize("chunks,threads", [(0, 3), (2, 1)])
@pytest.mark.parametrize("spec", GOLDEN_PCL_CASES, ids=lambda s: s["name"])
def test_paged_cache_load_body_matches_reference_golden(spec, chunks, threads, cumulative):
    fx = np.load(os.path.join(GOLDEN_DIR, f"pcl_{spec['name']}.npz"))
    inp = pcl_inputs(spec)
    kc, vc = inp["k_cache"], inp["v_cache"]
    total = int(inp["cu_lens"][-1])
    key = np.zeros((total,) + kc.shape[2:], dtype=kc.dtype)
    value = np.zeros((total,) + vc.shape[2:], dtype=vc.dtype)
    lens = inp["cu_lens"] if cumulative else inp["lens"]
    ws = np.zeros(spec["batch"] + 1, dtype=np.int32)
    emu().emu_paged_cache_load(_p(kc), _p(vc), _p(inp["block_tables"]), _p(lens), _p(inp["seq_starts"]), _p(key),
                               _p(value), spec["batch"], inp["block_tables"].shape[1], spec["block_size"],
                               kc[0, 0].nbytes, vc[0, 0].nbytes, kc.shape[0], total, int(cumulative), _p(ws), chunks,
                               threads)
    assert np.array_equal(_bits(key), _bits(fx["key"])) and np.array_equal(_bits(value), _bits(fx["value"]))


def test_paged_cache_load_body_against_oracle_with_holes():
    """Negative block ids and a missing seq_starts: rows of such tokens stay untouched, as in the oracle."""
    rng = np.random.default_rng(5)
    kc = rng.integers(-100, 100, size=(9, 4, 2, 24), dtype=np.int8)
    vc = rng.integers(-100, 100, size=(9, 4, 2, 8), dtype=np.int8)
    tables = rng.integers(-2, 9, size=(5, 6)).astype(np.int32)
    lens = np.array([3, 0, 17, 24, 9], dtype=np.int32)
    total = int(lens.sum())
    key, value = np.full((total, 2, 24), 7, np.int8), np.full((total, 2, 8), 7, np.int8)
    ref_k, ref_v = key.copy(), value.copy()
    oracle.cache_ops.paged_cache_load(kc, vc, tables, lens, ref_k, ref_v)
    ws = np.zeros(6, dtype=np.int32)
    emu().emu_paged_cache_load(_p(kc), _p(vc), _p(tables), _p(lens), None, _p(key), _p(value), 5, 6, 4, 48, 16, 9, total,
                               0, _p(ws), 0, 4)
    assert np.array_equal(key, ref_k) and np.array_equal(value, ref_v)
    assert (ref_k == 7).any()                                  # the case does have holes


def test_c_abi_rejects_bad_arguments_before_launching():
    L = capi.lib()
    fake = ctypes.c_void_p(0x1000)
    assert L.atb_b200_block_copy(None, fake, fake, fake, fake, 1, 1, 64, 64, 4, None) == capi.ERROR_INVALID_PARAM
    assert L.atb_b200_block_copy(fake, fake, None, fake, fake, 1, 1, 64, 64, 4, None) == capi.ERROR_INVALID_PARAM
    assert L.atb_b200_block_copy(fake, fake, fake, fake, fake, 1, 1, 0, 64, 4, None) == capi.ERROR_INVALID_PARAM
    assert L.atb_b200_block_copy(fake, fake, fake, fake, fake, 0, 0, 64, 64, 4, None) == 0      # nothing to do
    assert L.atb_b200_paged_cache_load_workspace_bytes(100, 1) == 0
    assert L.atb_b200_paged_cache_load_workspace_bytes(100, 0) >= 101 * 4
    args = [fake, fake, fake, fake, None, fake, fake, 4, 8, 16, 64, 64, 10, 100, 0, None, 0, None]
    assert L.atb_b200_paged_cache_load(*args) == capi.ERROR_INVALID_PARAM                       # no workspace
    args = [fake, None, fake, fake, None, fake, fake, 4, 8, 16, 64, 64, 10, 100, 1, None, 0, None]
    assert L.atb_b200_paged_cache_load(*args) == capi.ERROR_INVALID_PARAM                       # value without v_cache
    args = [fake, fake, fake, fake, None, fake, fake, 0, 8, 16, 64, 64, 10, 100, 1, None, 0, None]
    assert L.atb_b200_paged_cache_load(*args) == 0                                              # empty batch


# ------------------------------------------------------------------ the operations' host side (no GPU)

def _expect(code, fn, *a):
    with pytest.raises(capi.AtbError) as e:
        fn(*a)
    assert e.value.code == code, (e.value.code, code)


def _T(dtype, shape, host=None):
    return capi.atb_tensor(dtype=dtype, shape=shape, device_ptr=0x1000, host=host)


def test_block_copy_operation_checks():
    assert ctypes.sizeof(capi.BlockCopyParam) == 16
    op = capi.Operation(capi.BlockCopyParam())
    assert (op.name, op.input_num, op.output_num) == ("BlockCopyOperation", 5, 0)
    bad = capi.BlockCopyParam()
    bad.rsv[3] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, bad)
    ctx = capi.Context()
    f16, i32 = capi.ACL_FLOAT16, capi.ACL_INT32
    cache = (20, 16, 2, 64)
    ins = [_T(f16, cache), _T(f16, cache), _T(i32, (3,)), _T(i32, (10,)), _T(i32, (3,))]
    assert op.setup(ins, [], ctx) == 0
    wrong = list(ins)
    wrong[1] = _T(f16, (20, 16, 2, 32))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, [], ctx)                 # caches differ
    wrong = list(ins)
    wrong[4] = _T(i32, (4,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, [], ctx)                 # cumSum vs sources
    wrong = list(ins)
    wrong[3] = _T(i32, (21,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, [], ctx)                 # more destinations than blocks
    wrong = list(ins)
    wrong[2] = _T(i32, (3, 1))
    wrong[4] = _T(i32, (3, 1))
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.setup, wrong, [], ctx)
    wrong = list(ins)
    wrong[2] = _T(capi.ACL_INT64, (3,))
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, wrong, [], ctx)
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, op.setup, ins[:4], [], ctx)


def _pcl_param(**kw):
    p = capi.PagedCacheLoadParam()
    p.kvCacheCfg = 1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_paged_cache_load_operation_checks():
    assert ctypes.sizeof(capi.PagedCacheLoadParam) == 64
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, capi.PagedCacheLoadParam())    # the NZ layout (reference default)
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, _pcl_param(kvCacheCfg=2))
    bad = _pcl_param()
    bad.rsv[60] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, bad)
    op = capi.Operation(_pcl_param(isSeqLensCumsumMode=True, hasSeqStarts=True))
    assert (op.name, op.input_num, op.output_num) == ("PagedCacheLoadOperation", 7, 2)
    ctx = capi.Context()
    bf16, i32 = capi.ACL_BF16, capi.ACL_INT32
    ins = [_T(bf16, (128, 128, 16, 144)), _T(bf16, (128, 128, 16, 128)), _T(i32, (16, 12)), _T(i32, (17,)),
           _T(bf16, (900, 16, 144)), _T(bf16, (900, 16, 128)), _T(i32, (16,))]
    outs = [_T(bf16, (900, 16, 144)), _T(bf16, (900, 16, 128))]
    assert op.infer_shape(ins, 2) == [(900, 16, 144), (900, 16, 128)]
    assert op.setup(ins, outs, ctx) == 0                                              # running totals: no workspace
    plain = capi.Operation(_pcl_param())
    lens_ins = list(ins)
    lens_ins[3] = _T(i32, (16,))
    assert plain.setup(lens_ins, outs, ctx) >= 17 * 4                                 # room for the running totals
    _expect(capi.ERROR_INVALID_TENSOR_DIM, plain.setup, ins, outs, ctx)              # 17 lengths for 16 sequences
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, lens_ins, outs, ctx)
    wrong = list(ins)
    wrong[6] = _T(i32, (15,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)               # seqStarts per sequence
    wrong = list(ins)
    wrong[1] = _T(bf16, (128, 64, 16, 128))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)               # block sizes differ
    wrong = list(ins)
    wrong[0] = _T(bf16, (128, 128, 3, 5))
    wrong[1] = _T(bf16, (128, 128, 3, 5))
    wrong[4] = _T(bf16, (900, 3, 5))
    wrong[5] = _T(bf16, (900, 3, 5))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, [wrong[4], wrong[5]], ctx)   # heads*headSize % 16
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, ins, [outs[0], _T(bf16, (900, 16, 64))], ctx)
    wrong = list(ins)
    wrong[5] = _T(bf16, (901, 16, 128))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, [outs[0], wrong[5]], ctx)    # rows of key and value
    wrong = list(ins)
    wrong[2] = _T(i32, (16,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.setup, wrong, outs, ctx)


# ------------------------------------------------------------------ ReshapeAndCache over strided inputs

def _qkv_case(seed, tokens, heads, dk, dv, dtype, block_size=4, blocks=7):
    """K and V as slices of one fused [tokens, q | k | v] projection output (the case the operation is for)."""
    rng = np.random.default_rng(seed)
    width = 3 * dk + heads * dk + heads * dv + 5          # some query columns first, padding at the end
    fused = rng.integers(-120, 120, size=(tokens, width)).astype(dtype)
    k_off, v_off = 3 * dk, 3 * dk + heads * dk
    kc = rng.integers(-120, 120, size=(blocks, block_size, heads, dk)).astype(dtype)
    vc = rng.integers(-120, 120, size=(blocks, block_size, heads, dv)).astype(dtype)
    slots = rng.choice(np.arange(0, blocks * block_size), size=tokens, replace=False).astype(np.int32)
    slots[1] = -3                                          # "do not store"
    return fused, width, k_off, v_off, kc, vc, slots


@pytest.mark.parametrize("dtype,dk,dv", [(np.int16, 16, 8), (np.int8, 32, 48), (np.int16, 5, 3)])
@pytest.mark.parametrize("chunks,threads", [(0, 4), (3, 2)])
def test_rac_strided_body_matches_oracle(dtype, dk, dv, chunks, threads):
    heads, tokens = 3, 9
    fused, width, k_off, v_off, kc, vc, slots = _qkv_case(7, tokens, heads, dk, dv, dtype)
    ref_k, ref_v = oracle.cache_ops.reshape_and_cache_with_stride(fused, fused, kc.copy(), vc.copy(), slots, heads, dk, dv,
                                                                  width, k_off, v_off)
    es = fused.itemsize
    flat = fused.reshape(-1)
    k_view, v_view = flat[k_off:], flat[v_off:]
    emu().emu_rac_strided(_p(k_view), _p(v_view), _p(kc), _p(vc), _p(slots), tokens, heads * dk * es, heads * dv * es,
                          width * es, width * es, kc.shape[0] * kc.shape[1], chunks, threads)
    assert np.array_equal(kc, ref_k) and np.array_equal(vc, ref_v)
    assert (slots < 0).any()                                # skipped tokens are part of the case


def test_reshape_and_cache_with_stride_operation_checks():
    assert ctypes.sizeof(capi.ReshapeAndCacheWithStrideParam) == 24
    op = capi.Operation(capi.ReshapeAndCacheWithStrideParam())
    assert (op.name, op.input_num, op.output_num) == ("ReshapeAndCacheWithStrideOperation", 9, 2)
    siso_p = capi.ReshapeAndCacheWithStrideParam()
    siso_p.kvCacheCfg = 1
    siso = capi.Operation(siso_p)
    assert (siso.input_num, siso.output_num) == (5, 1)
    bad = capi.ReshapeAndCacheWithStrideParam()
    bad.compressType = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, bad)
    bad = capi.ReshapeAndCacheWithStrideParam()
    bad.kvCacheCfg = 2
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, bad)
    ctx = capi.Context()
    f16, i32, i64 = capi.ACL_FLOAT16, capi.ACL_INT32, capi.ACL_INT64
    strides = np.array([3 * 8 * 128, 128, 1], dtype=np.int64)
    koff, voff = np.array([8 * 128], dtype=np.int64), np.array([2 * 8 * 128], dtype=np.int64)
    ins = [_T(f16, (6, 8, 128)), _T(f16, (6, 8, 128)), _T(f16, (10, 16, 8, 128)), _T(f16, (10, 16, 8, 128)),
           _T(i32, (6,)), _T(i64, (3,), host=strides), _T(i64, (3,), host=strides), _T(i64, (1,), host=koff),
           _T(i64, (1,), host=voff)]
    outs = [ins[2], ins[3]]
    assert op.infer_shape(ins, 2) == [(10, 16, 8, 128), (10, 16, 8, 128)]
    assert op.setup(ins, outs, ctx) == 0
    wrong = list(ins)
    wrong[5] = _T(i64, (3,))
    _expect(capi.ERROR_INVALID_PARAM, op.setup, wrong, outs, ctx)                     # strides without host data
    neg = np.array([-1], dtype=np.int64)
    wrong = list(ins)
    wrong[7] = _T(i64, (1,), host=neg)
    _expect(capi.ERROR_INVALID_PARAM, op.setup, wrong, outs, ctx)                     # negative offset
    wrong = list(ins)
    wrong[1] = _T(f16, (5, 8, 128))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)                # tokens of key and value
    wrong = list(ins)
    wrong[4] = _T(i32, (7,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)                # slots per token
    wrong = list(ins)
    wrong[5] = _T(i32, (3,), host=strides)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, wrong, outs, ctx)          # strides must be int64
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, ins, [ins[2], _T(f16, (10, 16, 8, 64))], ctx)
    _expect(capi.ERROR_INVALID_IN_TENSOR_NUM, op.setup, ins[:5], outs, ctx)
    s_ins = [ins[0], ins[2], ins[4], ins[5], ins[7]]
    assert siso.setup(s_ins, [ins[2]], ctx) == 0
    L = capi.lib()
    fake = ctypes.c_void_p(0x1000)
    assert L.atb_b200_reshape_and_cache_strided(None, None, fake, None, fake, 4, 64, 0, 128, 0, 10, None) == \
        capi.ERROR_INVALID_PARAM
    assert L.atb_b200_reshape_and_cache_strided(fake, fake, fake, None, fake, 4, 64, 64, 128, 128, 10, None) == \
        capi.ERROR_INVALID_PARAM                                                      # value without its cache
    assert L.atb_b200_reshape_and_cache_strided(fake, None, fake, None, fake, 4, 64, 0, -16, 0, 10, None) == \
        capi.ERROR_INVALID_PARAM
    assert L.atb_b200_reshape_and_cache_strided(fake, None, fake, None, fake, 0, 64, 0, 128, 0, 10, None) == 0


# ------------------------------------------------------------------ fused RMSNorm + RoPE + cache write

def test_norm_rope_reshape_operation_checks():
    assert ctypes.sizeof(capi.NormRopeReshapeParam) == 28
    op = capi.Operation(capi.NormRopeReshapeParam())
    assert (op.name, op.input_num, op.output_num) == ("NormRopeReshapeOperation", 7, 1)
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, capi.NormRopeReshapeParam(epsilon=0.0))
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, capi.NormRopeReshapeParam(rotaryCoeff=4))
    bad = capi.NormRopeReshapeParam()
    bad.rsv[15] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, bad)
    ctx = capi.Context()
    bf, i32 = capi.ACL_BF16, capi.ACL_INT32
    ins = [_T(bf, (32, 1, 512)), _T(bf, (512,)), _T(bf, (32, 64)), _T(bf, (32, 64)), _T(bf, (32, 64)), _T(i32, (32,)),
           _T(bf, (10, 128, 1, 576))]
    outs = [ins[6]]
    assert op.infer_shape(ins, 1) == [(10, 128, 1, 576)]
    assert op.setup(ins, outs, ctx) == 0
    wrong = list(ins)
    wrong[1] = _T(bf, (256,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)                # gamma vs x
    wrong = list(ins)
    wrong[3] = _T(bf, (32, 32))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)                # cos vs keyRope
    wrong = list(ins)
    wrong[6] = _T(bf, (10, 128, 1, 512))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, [wrong[6]], ctx)          # cache row width
    wrong = list(ins)
    wrong[5] = _T(i32, (31,))
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, wrong, outs, ctx)                # one slot per token
    wrong = list(ins)
    wrong[0] = _T(bf, (32, 512))
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.setup, wrong, outs, ctx)
    wrong = list(ins)
    wrong[1] = _T(capi.ACL_FLOAT16, (512,))
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, wrong, outs, ctx)          # mixed dtypes
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, ins, [_T(bf, (10, 64, 1, 576))], ctx)
    L = capi.lib()
    fake = ctypes.c_void_p(0x1000)
    ok = [fake] * 7 + [4, 512, 64, 1, 1e-5, 1280, None]
    assert L.atb_b200_norm_rope_reshape(*([fake] * 7 + [0, 512, 64, 1, 1e-5, 1280, None])) == 0     # no tokens
    for pos, val in [(0, None), (9, 63), (10, 2), (11, 0.0), (12, 0)]:
        args = list(ok)
        args[pos] = val
        assert L.atb_b200_norm_rope_reshape(*args) == capi.ERROR_INVALID_PARAM, pos


# ------------------------------------------------------------------ KvCache

def _run_emu_kv_cache(inp, past, chunks, threads):
    return emu().emu_kv_cache(_p(inp["new_kv"]), _p(inp["layer_id"]), _p(past), _p(inp["token_offset"]), _p(inp["seq_len"]),
                              inp["new_kv"].shape[0], past.shape[0], past.shape[1], past.shape[2], past[0, 0, 0].nbytes,
                              chunks, threads)


@pytest.mark.parametrize("chunks,threads", [(0, 4), (1, 1), (3, 5)])
@pytest.mark.parametrize("spec", GOLDEN_KVCACHE_CASES, ids=lambda s: s["name"])
def test_kv_cache_oracle_and_body_match_reference_golden(spec, chunks, threads):
    fx = np.load(os.path.join(GOLDEN_DIR, f"kvcache_{spec['name']}.npz"))
    inp = kvcache_inputs(spec)
    want = oracle.cache_ops.kv_cache(inp["new_kv"], inp["layer_id"][0], inp["past"].copy(), inp["token_offset"], inp["seq_len"])
    assert np.array_equal(_bits(want), _bits(fx["past"]))
    assert np.any(_bits(want) != 0)
    past = inp["past"].copy()
    _run_emu_kv_cache(inp, past, chunks, threads)
    assert np.array_equal(_bits(past), _bits(fx["past"]))


def test_kv_cache_body_keeps_other_rows_and_skips_runs_that_do_not_fit():
    rng = np.random.default_rng(9)
    spec = GOLDEN_KVCACHE_CASES[0]
    inp = kvcache_inputs(spec)
    before = rng.integers(1, 2 ** 15, size=inp["past"].shape).astype(np.uint16).view(np.float16)
    want = oracle.cache_ops.kv_cache(inp["new_kv"], inp["layer_id"][0], before.copy(), inp["token_offset"], inp["seq_len"])
    past = before.copy()
    _run_emu_kv_cache(inp, past, 0, 7)
    assert np.array_equal(_bits(past), _bits(want))                       # everything not written is untouched
    for field, b, value in (("token_offset", 1, 0), ("token_offset", 2, spec["max_seqlen"] + 1), ("seq_len", 0, -3),
                            ("layer_id", 0, spec["layers"]), ("layer_id", 0, -1)):
        hostile = {k: v.copy() for k, v in inp.items()}
        hostile[field][b] = value
        past = before.copy()
        _run_emu_kv_cache(hostile, past, 2, 3)                            # must not write outside `past` (ASan build checks too)
        if field == "layer_id":
            assert np.array_equal(_bits(past), _bits(before))
        else:
            assert np.array_equal(_bits(past[:, b]), _bits(before[:, b]))  # the offending sequence is skipped


def test_kv_cache_operation_checks():
    assert ctypes.sizeof(capi.KvCacheParam) == 8                          # tests/unittest/ops/test_op_param_size.cpp:36
    op = capi.Operation(capi.KvCacheParam())
    assert (op.name, op.input_num, op.output_num) == ("KvCacheOperation", 5, 0)
    bad = capi.KvCacheParam()
    bad.rsv[7] = 1
    _expect(capi.ERROR_INVALID_PARAM, capi.Operation, bad)
    ctx = capi.Context()
    f16, i32, i8 = capi.ACL_FLOAT16, capi.ACL_INT32, capi.ACL_INT8
    ins = [_T(f16, (37, 1024)), _T(i32, (1,)), _T(f16, (28, 16, 384, 1024)), _T(i32, (16,)), _T(i32, (16,))]
    assert op.infer_shape(ins, 0) == []
    assert op.setup(ins, [], ctx) == 0
    four_d = list(ins)
    four_d[0] = _T(f16, (16, 2, 8, 128))                                   # [batch, seq, heads, headSize]
    assert op.setup(four_d, [], ctx) == 0

    def swapped(i, t):
        w = list(ins)
        w[i] = t
        return w
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(0, _T(f16, (37, 512))), [], ctx)          # hidden sizes differ
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(3, _T(i32, (15,))), [], ctx)              # batches differ
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, swapped(0, _T(f16, (37, 8, 128))), [], ctx)       # 3-D newKv
    _expect(capi.ERROR_INVALID_TENSOR_DIM_NUM, op.infer_shape, swapped(0, _T(f16, (37, 8, 128))), 0)
    _expect(capi.ERROR_INVALID_TENSOR_INI_MATCH, op.setup, swapped(0, _T(capi.ACL_BF16, (37, 1024))), [], ctx)
    odd = [_T(f16, (37, 1000)), ins[1], _T(f16, (28, 16, 384, 1000)), ins[3], ins[4]]
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, odd, [], ctx)                                     # hidden % 16
    int8 = [_T(i8, (37, 48)), ins[1], _T(i8, (28, 16, 384, 48)), ins[3], ins[4]]
    _expect(capi.ERROR_INVALID_TENSOR_DIM, op.setup, int8, [], ctx)                                    # int8: hidden % 32
    lib = capi.lib()
    assert lib.atb_b200_kv_cache(None, 0x1000, 0x1000, 0x1000, 0x1000, 4, 1, 1, 8, 64, None) == capi.ERROR_INVALID_PARAM
    assert lib.atb_b200_kv_cache(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 4, 0, 1, 8, 64, None) == capi.ERROR_INVALID_PARAM
    assert lib.atb_b200_kv_cache(0x1000, 0x1000, 0x1000, 0x1000, 0x1000, 0, 1, 1, 8, 64, None) == 0    # nothing to copy
