"""ctypes front end of liboracle.so (see pa_oracle.c).  Arrays are numpy; bf16 travels as uint16 bits."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

FP16, BF16, INT8 = 0, 1, 2
_DT = {"fp16": FP16, "bf16": BF16, "int8": INT8}


def build(force=False):
    """Compile pa_oracle.c with gcc (OpenMP) into oracle/liboracle.so."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "pa_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def load():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        lib = ctypes.CDLL(so)
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float
        lib.oracle_paged_attention.restype = ctypes.c_int
        lib.oracle_paged_attention.argtypes = [vp] * 11 + [i32] * 10 + [f32, i32]
        lib.oracle_paged_attention_ex.restype = ctypes.c_int
        lib.oracle_paged_attention_ex.argtypes = [vp] * 11 + [i32] * 10 + [f32, i32, vp, i64, i64, vp]
        lib.oracle_reshape_and_cache.restype = ctypes.c_int
        lib.oracle_reshape_and_cache.argtypes = [vp] * 5 + [i32, i64, i64, i64]
        lib.oracle_num_threads.restype = ctypes.c_int
        lib.oracle_paged_attention_qkv_quant.restype = ctypes.c_int
        lib.oracle_paged_attention_qkv_quant.argtypes = [vp] * 9 + [i32] * 7 + [f32] + [i32] * 3
        _LIB = lib
    return _LIB


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


def num_threads():
    return int(load().oracle_num_threads())


def paged_attention(q, k_cache, v_cache, block_tables, context_lens, scale, q_dtype, kv_dtype=None, dv=None,
                    k_descale=None, v_descale=None, k_offset=None, v_offset=None, out=None, want_high=False,
                    nthreads=0, mask=None, logn=None):
    """Decode attention golden.  `v_cache=None` means the MLA combined cache (V = K[..., :dv]).

    mask: additive fp32 bias of shape [B, H, 1, T] (alibi), [B, 1, T] or [B, T] (plain mask per
    sequence) or [1, T] / [T] (one row for all), T >= the longest context; logn: [B] fp32 factors of
    the scale (SCALE_TYPE_LOGN).

    q: [B,H,Dk] (float16, or uint16 holding bf16 bits); caches [NB,BS,Hkv,D] in the same encoding or
    int8.  Returns out [B,H,Dv] in q's encoding (rows of zero-length sequences keep `out`'s
    previous contents, zeros if `out` is None) and optionally the fp32 high-precision output.
    """
    lib = load()
    kv_dtype = kv_dtype or q_dtype
    B, H, Dk = q.shape
    NB, BS, Hkv, Dk2 = k_cache.shape
    assert Dk == Dk2
    if v_cache is None:
        v_cache, dv_row = k_cache, Dk
        assert dv is not None
    else:
        dv_row = v_cache.shape[3]
        dv = dv or dv_row
    block_tables = np.ascontiguousarray(block_tables, dtype=np.int32)
    context_lens = np.ascontiguousarray(context_lens, dtype=np.int32)
    if out is None:
        out = np.zeros((B, H, dv), dtype=q.dtype)
    high = np.zeros((B, H, dv), dtype=np.float32) if want_high else None
    f32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
    i32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.int32)
    kd, vd, ko, vo = f32(k_descale), f32(v_descale), i32(k_offset), i32(v_offset)
    mb = mh = 0
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.float32)
        T = mask.shape[-1]
        assert T >= int(context_lens.max(initial=0)), "the mask is shorter than the longest context"
        if mask.ndim == 4:
            assert mask.shape[:3] == (B, H, 1)
            mb, mh = H * T, T
        elif mask.size == T:
            mb = mh = 0
        else:
            assert mask.size == B * T
            mb, mh = T, 0
    logn = f32(logn)
    rc = lib.oracle_paged_attention_ex(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(context_lens),
                                       _ptr(kd), _ptr(vd), _ptr(ko), _ptr(vo), _ptr(out), _ptr(high), B, H, Hkv, Dk,
                                       dv, dv_row, BS, block_tables.shape[1], _DT[q_dtype], _DT[kv_dtype],
                                       float(scale), int(nthreads), _ptr(mask), mb, mh, _ptr(logn))
    if rc != 0:
        raise ValueError("oracle_paged_attention rejected its arguments")
    return (out, high) if want_high else out


def paged_attention_qkv_quant(q, k_cache, v_cache, block_tables, context_lens, k_descale, v_descale, scale, out_dtype,
                              p_scale=None, tile_tokens=128, split_tokens=1 << 30, nthreads=0):
    """Decode attention golden for int8 Q, K and V (TYPE_QUANT_QKV_ONLINE; with `p_scale` OFFLINE).

    q [B,H,D] int8, caches [NB,BS,Hkv,D] int8, k_descale / v_descale / p_scale [H] fp32.  P is quantised to int8 per
    tile of `tile_tokens` inside splits of `split_tokens` (the golden's block_size_calc and kv_split_per_core).
    Returns out [B,H,D] in `out_dtype` ('fp16' as float16, 'bf16' as uint16 bits); rows of empty sequences are zero."""
    lib = load()
    B, H, D = q.shape
    NB, BS, Hkv, _ = k_cache.shape
    assert q.dtype == np.int8 and k_cache.dtype == np.int8 and v_cache.dtype == np.int8
    block_tables = np.ascontiguousarray(block_tables, dtype=np.int32)
    context_lens = np.ascontiguousarray(context_lens, dtype=np.int32)
    out = np.zeros((B, H, D), dtype=np.float16 if out_dtype == "fp16" else np.uint16)
    f32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
    kd, vd, ps = f32(k_descale), f32(v_descale), f32(p_scale)
    rc = lib.oracle_paged_attention_qkv_quant(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(context_lens),
                                              _ptr(kd), _ptr(vd), _ptr(ps), _ptr(out), B, H, Hkv, D, BS,
                                              block_tables.shape[1], _DT[out_dtype], float(scale), int(tile_tokens),
                                              int(min(split_tokens, 1 << 30)), int(nthreads))
    if rc != 0:
        raise ValueError("oracle_paged_attention_qkv_quant rejected its arguments")
    return out


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping):
    """In-place scatter golden; `value`/`value_cache` may be None (K-only variant)."""
    lib = load()
    slot_mapping = np.ascontiguousarray(slot_mapping, dtype=np.int32)
    n = slot_mapping.shape[0]
    krow = key[0].nbytes if key is not None and n else 0
    vrow = value[0].nbytes if value is not None and n else 0
    nslots = key_cache.shape[0] * key_cache.shape[1]
    rc = lib.oracle_reshape_and_cache(_ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache), _ptr(slot_mapping),
                                      n, krow, vrow, nslots)
    if rc != 0:
        raise ValueError("oracle_reshape_and_cache rejected its arguments")


def _to_f32(a, dtype):
    """This module's encodings (float16 arrays; bf16 as uint16 bits) to float32."""
    a = np.asarray(a)
    if dtype == "bf16":
        return (a.astype(np.uint32) << 16).view(np.float32)
    return a.astype(np.float32)


def _from_f32(a, dtype):
    """float32 to this module's encodings, round to nearest even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == "bf16":
        u = a.view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return a.astype(np.float16)


def attention_lse(q, k_cache, block_tables, context_lens, scale, q_dtype, mask=None):
    """Natural-log log-sum-exp of the scaled scores of every (token, head), rounded to the query dtype: the second
    output of MultiLatentAttention with CALC_TYPE_RING.  Follows softmax_numpy (row_max + log(row_sum), fp32) and the
    cast in ref_masked_attention of tests/apitest/kernelstest/mix/test_paged_attention_mla_split.py:124-132, 171-175
    of the reference.  q [B, H, Dk] and k_cache [blocks, block_size, kv_heads, Dk] in this module's encodings;
    sequences of length 0 keep 0.  mask: optional fp32 [B, 1, T], added to the scaled scores of every head."""
    qf, kf = _to_f32(q, q_dtype), _to_f32(k_cache, q_dtype)
    B, H, _ = qf.shape
    kvh, bs = kf.shape[2], kf.shape[1]
    out = np.zeros((B, H, 1), dtype=np.float32)
    for b in range(B):
        n = int(context_lens[b])
        if n == 0:
            continue
        rows = [kf[int(block_tables[b, t // bs]), t % bs] for t in range(n)]
        keys = np.stack(rows, axis=0)                                       # [n, kv_heads, Dk]
        for h in range(H):
            s = (keys[:, h // (H // kvh), :] @ qf[b, h]).astype(np.float32) * np.float32(scale)
            if mask is not None:
                s = s + mask[b, 0, :n]
            mx = s.max()
            out[b, h, 0] = mx + np.log(np.exp(s - mx).sum(dtype=np.float32))
    return _from_f32(out, q_dtype)


def paged_attention_spec(q, k_cache, v_cache, block_tables, q_lens, context_lens, scale, q_dtype, mask, mask_rows_are_tokens,
                         nthreads=0, dv=None, want_lse=False):
    """Parallel decoding (PagedAttentionParam::CALC_TYPE_SPEC): sequence b owns q_lens[b] consecutive query tokens,
    each of which attends to all context_lens[b] cached tokens of that sequence plus a row of `mask` (fp32):
    row = the token's index for MASK_TYPE_SPEC ([tokens, T]; `mask_rows_are_tokens`), row = ctx - q_len + j of the
    square causal mask [T, T] for MASK_TYPE_NORM.  Restates ref_single_query_cached_kv_attention of
    tests/apitest/kernelstest/mix/test_paged_attention_lookahead.py:97-140 by expanding every query token into a
    sequence of its own (its sequence's block-table row and length, its mask row) for `paged_attention`.
    mask=None: every token sees its sequence's whole context.  v_cache=None with dv: the MLA combined cache
    (V = K[..., :dv]); want_lse also returns the log-sum-exp [tokens, heads, 1] as
    tests/apitest/kernelstest/mix/test_paged_attention_mla_mtp_split.py:85-122 does (fp32, rounded to the query dtype)."""
    q_lens = np.asarray(q_lens, dtype=np.int64)
    context_lens = np.asarray(context_lens, dtype=np.int32)
    tokens = int(q_lens.sum())
    assert q.shape[0] == tokens and len(q_lens) == len(context_lens) == block_tables.shape[0]
    owner = np.repeat(np.arange(len(q_lens)), q_lens)
    within = np.arange(tokens) - np.repeat(np.cumsum(q_lens) - q_lens, q_lens)
    lens = context_lens[owner]
    per_token = None
    if mask is not None:
        mask = np.asarray(mask, dtype=np.float32)
        rows = np.arange(tokens) if mask_rows_are_tokens else lens.astype(np.int64) - q_lens[owner] + within
        assert rows.min(initial=0) >= 0 and rows.max(initial=0) < mask.shape[0]
        per_token = np.ascontiguousarray(mask[rows][:, None, :])                 # [tokens, 1, T]
    tables = np.ascontiguousarray(block_tables[owner])
    out = paged_attention(q, k_cache, v_cache, tables, lens, scale, q_dtype, nthreads=nthreads, mask=per_token, dv=dv)
    if not want_lse:
        return out
    return out, attention_lse(q, k_cache, tables, lens, scale, q_dtype, mask=per_token)


def multi_latent_attention(q_nope, q_rope, ct_kv, k_rope, block_tables, context_lens, scale, q_dtype, **kw):
    """MultiLatentAttention decode golden with the split cache (cacheMode 1 of the reference): the
    latent part [.., 512] and the rope part [.., 64] of the query and of the cache are separate
    tensors; V is the latent part.  The reference's golden computes on the joined tensors and splits
    them afterwards (tests/apitest/opstest/python/operations/multi_latent_attention/
    test_multi_latent_attention.py:330-347), so this joins them and runs the combined-cache golden."""
    q = np.ascontiguousarray(np.concatenate([q_nope, q_rope], axis=-1))
    cache = np.ascontiguousarray(np.concatenate([ct_kv, k_rope], axis=-1))
    return paged_attention(q, cache, None, block_tables, context_lens, scale, q_dtype, dv=ct_kv.shape[-1], **kw)
