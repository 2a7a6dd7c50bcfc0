"""CPU oracle of the cache-management siblings of ReshapeAndCache (test infrastructure only).

Pure byte movement, restated in numpy from the reference's CPU goldens:
  block_copy         tests/apitest/kernelstest/mix/test_blockcopy.py:65-81  (TestBlockCopy.golden_calc)
  paged_cache_load   tests/apitest/kernelstest/mix/test_paged_cache_load_nd.py:67-110
                     (generate_test_data), with the device kernel's row placement
                     (src/kernels/mixkernels/paged_cache_load/op_kernel/paged_cache_load_nd.cpp:139-160):
                     token j of sequence i always lands in row start_i + j.
  reshape_and_cache_with_stride   the same scatter as ReshapeAndCache
                     (tests/apitest/kernelstest/mix/test_reshape_and_cache.py:45-68) over strided views
  norm_rope_reshape  tests/apitest/kernelstest/mix/test_rms_norm_and_rope_and_reshape_and_cache.py:24-72
                     (rmsnorm_golden, rope_golden, rac_golden, golden_calc) and its _bf16 twin
Pinned against outputs of those reference functions stored under tests/golden/.
"""
import numpy as np


def block_copy(k_cache, v_cache, src_blocks, dst_blocks, cum_sum):
    """In place: source block i is copied to the destination blocks dst[cum[i-1]:cum[i]] (cum is the
    running total of destinations per source), in source order, as the golden does."""
    start = 0
    for i, src in enumerate(np.asarray(src_blocks)):
        end = int(cum_sum[i])
        for j in range(start, end):
            dst = int(dst_blocks[j])
            k_cache[dst] = k_cache[int(src)].copy()
            if v_cache is not None:
                v_cache[dst] = v_cache[int(src)].copy()
        start = end
    return k_cache, v_cache


def paged_cache_load(k_cache, v_cache, block_tables, context_lens, key_out, value_out, seq_starts=None,
                     cumulative=False):
    """Gathers the cached tokens of every sequence back into contiguous rows (the reverse of
    ReshapeAndCache).  context_lens holds lengths [B], or with `cumulative` the running totals [B+1];
    seq_starts (tokens, used in whole blocks) offsets each sequence's walk through its block table.
    Rows whose block id is negative are left untouched."""
    block_size = k_cache.shape[1]
    lens = np.asarray(context_lens).astype(np.int64)
    if cumulative:
        starts, ends = lens[:-1], lens[1:]
    else:
        ends = np.cumsum(lens)
        starts = ends - lens
    for i in range(len(starts)):
        table_off = 0 if seq_starts is None else int(seq_starts[i]) // block_size
        for j in range(int(ends[i] - starts[i])):
            blk = int(block_tables[i, table_off + j // block_size])
            if blk < 0:
                continue
            key_out[starts[i] + j] = k_cache[blk, j % block_size]
            if v_cache is not None:
                value_out[starts[i] + j] = v_cache[blk, j % block_size]
    return key_out, value_out


def reshape_and_cache_with_stride(key_storage, value_storage, key_cache, value_cache, slot_mapping, num_heads, dk, dv,
                                  token_stride, k_offset, v_offset=0):
    """ReshapeAndCache reading strided rows: token t's key row is the num_heads*dk elements of the flat
    array key_storage starting at k_offset + t*token_stride (value: v_offset + t*token_stride, the KEY's
    token stride, as the reference kernel applies it).  The gathered rows go through the pinned
    ReshapeAndCache oracle."""
    from .oracle import reshape_and_cache
    n = len(slot_mapping)
    kflat = np.ascontiguousarray(key_storage).reshape(-1)
    key = np.stack([kflat[k_offset + t * token_stride: k_offset + t * token_stride + num_heads * dk]
                    for t in range(n)]).reshape(n, num_heads, dk)
    value = None
    if value_storage is not None:
        vflat = np.ascontiguousarray(value_storage).reshape(-1)
        value = np.stack([vflat[v_offset + t * token_stride: v_offset + t * token_stride + num_heads * dv]
                          for t in range(n)]).reshape(n, num_heads, dv)
        value = np.ascontiguousarray(value)
    reshape_and_cache(np.ascontiguousarray(key), value, key_cache, value_cache, slot_mapping)
    return key_cache, value_cache


def _round_to(a32, dtype):
    """fp32 -> the storage encoding: float16, or bf16 bits (round to nearest even) as uint16."""
    if dtype == "fp16":
        return a32.astype(np.float16)
    bits = np.ascontiguousarray(a32, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def _to_f32(a, dtype):
    if dtype == "fp16":
        return a.astype(np.float32)
    return (a.astype(np.uint32) << 16).view(np.float32)


def norm_rope_reshape(x, gamma, key_rope, cos, sin, slot_mapping, key_cache, epsilon, dtype):
    """Fused RMSNorm(x) * gamma | RoPE(key_rope) -> cache row (the MLA latent cache update), in place.

    x [T, 1, Dx], gamma [Dx], key_rope / cos / sin [T, Dr], key_cache [blocks, block_size, 1, Dx + Dr], all in
    `dtype` encoding (float16, or uint16 holding bf16 bits).  fp32 arithmetic in the golden's order:
    rms = 1 / sqrt(sum(x^2) / Dx + eps); norm = (rms * x) * gamma; rope = k * cos + rotate_half(k) * sin with
    rotate_half(k) = (-k[Dr/2:], k[:Dr/2]); each rounded once to the storage type.  Negative slots are skipped."""
    xf = _to_f32(np.asarray(x), dtype).reshape(x.shape[0], -1)
    gf = _to_f32(np.asarray(gamma), dtype)
    square_sum = np.sum(np.square(xf), axis=-1, keepdims=True)
    rms = (1.0 / np.sqrt(square_sum / np.float32(xf.shape[-1]) + np.float32(epsilon))).astype(np.float32)
    norm = rms * xf * gf
    kf, cf, sf = (_to_f32(np.asarray(t), dtype) for t in (key_rope, cos, sin))
    first, second = np.split(kf, 2, axis=1)
    rope = kf * cf + np.concatenate((-second, first), axis=1) * sf
    rows = np.concatenate((_round_to(norm.astype(np.float32), dtype), _round_to(rope.astype(np.float32), dtype)), axis=-1)
    block_size = key_cache.shape[1]
    for i, slot in enumerate(np.asarray(slot_mapping)):
        if slot < 0:
            continue
        key_cache[slot // block_size, slot % block_size, 0] = rows[i]
    return key_cache


def kv_cache(new_kv, layer_id, past, token_offset, seq_len):
    """KvCache on numpy arrays, in place on `past` [layers, batch, max_seqlen, hidden]: sequence i's seq_len[i] rows of
    new_kv [tokens, hidden] (sequences back to back) go to positions [token_offset[i] - seq_len[i], token_offset[i]) of
    past[layer_id].  Follows golden_calc of tests/apitest/kernelstest/mix/test_kvcache.py:65-78 of the reference."""
    prefix = 0
    for i in range(past.shape[1]):
        n, off = int(seq_len[i]), int(token_offset[i])
        for j in range(n):
            past[int(layer_id), i, off - n + j, :] = new_kv[prefix + j, :]
        prefix += n
    return past
