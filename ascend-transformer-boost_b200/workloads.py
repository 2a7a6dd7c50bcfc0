"""Seeded synthetic decode workloads: the five benchmark configurations and small parity cases.

Real serving traces are not available offline, so every tensor is synthetic with the shapes, dtypes
and value distributions of the benchmark configurations (Q/K/V ~ N(0,1); int8 caches uniform in
[-127,127] with per-channel scales ~ U(0.005,0.02) rounded to fp16; block tables = slices of one
random permutation of the block pool, padded with -1).  Layouts follow the reference operator
(src/ops/ops_infer/paged_attention/paged_attention_operation.cpp:408-470 of the reference):
query [tokens, heads, Dk], caches [blocks, block_size, kv_heads, D], int32 block_tables
[tokens, max_blocks] and context_lens [tokens].

bf16 tensors are carried in numpy as uint16 bit patterns.
"""
from dataclasses import dataclass, field, replace
import math

import numpy as np


def f32_to_bf16_bits(x):
    """Round-to-nearest-even float32 -> bf16 bit pattern (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_f32(a, dtype):
    """Decode a host array of the given logical dtype ('fp16' | 'bf16' | 'int8') to float32."""
    if dtype == "bf16":
        return bf16_bits_to_f32(a)
    return np.asarray(a).astype(np.float32)


def encode(x, dtype):
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    if dtype == "fp16":
        return np.asarray(x, dtype=np.float32).astype(np.float16)
    raise ValueError(dtype)


@dataclass(frozen=True)
class Case:
    name: str
    batch: int
    heads: int
    kv_heads: int
    dk: int = 128
    dv: int = 128                 # V width read by attention (MLA: 512)
    block_size: int = 128
    q_dtype: str = "bf16"         # 'fp16' | 'bf16'
    kv_dtype: str = ""            # '' = same as q_dtype, or 'int8'
    ctx: tuple = ("uniform", 1, 1024)   # ("uniform", lo, hi) | ("lognormal", mu, sigma, lo, hi) | ("list", [...])
    mla: bool = False             # combined cache: one K tensor, V = K[..., :dv]
    offsets: bool = False         # int8 cache: also int32 k/v offsets
    pool_blocks: int = 0          # 0 = 2x the blocks the sequences need
    seed: int = 0
    scale: float = 0.0            # 0 = 1/sqrt(dk)

    @property
    def kvd(self):
        return self.kv_dtype or self.q_dtype

    @property
    def qk_scale(self):
        return self.scale or 1.0 / math.sqrt(self.dk)

    @property
    def kv_elem_bytes(self):
        return 1 if self.kvd == "int8" else 2

    def shard_heads(self, rank, world):
        """The slice of this case one rank owns when kv heads are sharded over `world` GPUs."""
        assert self.kv_heads % world == 0
        return replace(self, name=f"{self.name}/r{rank}of{world}", heads=self.heads // world,
                       kv_heads=self.kv_heads // world)

    def shard_sequences(self, rank, world):
        """The slice of this case one rank owns when the sequences are sharded over `world` GPUs
        (the MLA cache has one kv head, so it is split by sequence): same lengths as the unsharded
        case, taken in contiguous chunks."""
        assert self.batch % world == 0
        per = self.batch // world
        lens = context_lens(self)[rank * per:(rank + 1) * per]
        return replace(self, name=f"{self.name}/seq{rank}of{world}", batch=per, ctx=("list", [int(x) for x in lens]))


# The benchmark configurations, in order (index 0 is the CPU-runnable golden case).
CONFIGS = [
    Case("c1_mha_fp16", batch=4, heads=32, kv_heads=32, q_dtype="fp16", ctx=("uniform", 1, 1024),
         pool_blocks=64, seed=1001),
    Case("c2_gqa_bf16_llama3_8b", batch=64, heads=32, kv_heads=8, q_dtype="bf16", ctx=("uniform", 2048, 4096),
         seed=1002),
    Case("c3_int8kv_70b", batch=128, heads=64, kv_heads=8, q_dtype="fp16", kv_dtype="int8",
         ctx=("uniform", 2048, 8192), seed=1003),
    Case("c4_gqa_bf16_skewed", batch=256, heads=64, kv_heads=8, q_dtype="bf16",
         ctx=("lognormal", 7.6, 1.0, 16, 32768), seed=1004),
    Case("c5_mla_bf16_dsv3", batch=32, heads=128, kv_heads=1, dk=576, dv=512, q_dtype="bf16",
         ctx=("uniform", 4096, 8192), mla=True, seed=1005),
]


def context_lens(case):
    rng = np.random.default_rng(case.seed)
    kind = case.ctx[0]
    if kind == "uniform":
        return rng.integers(case.ctx[1], case.ctx[2] + 1, size=case.batch).astype(np.int32)
    if kind == "lognormal":
        _, mu, sigma, lo, hi = case.ctx
        return np.clip(rng.lognormal(mu, sigma, size=case.batch), lo, hi).astype(np.int32)
    if kind == "list":
        lens = np.asarray(case.ctx[1], dtype=np.int32)
        assert lens.shape[0] == case.batch
        return lens
    raise ValueError(kind)


def block_tables(case, lens):
    """Slices of one random permutation of the pool (no block shared), -1 padded."""
    rng = np.random.default_rng(case.seed + 7)
    need = (lens.astype(np.int64) + case.block_size - 1) // case.block_size
    total = int(need.sum())
    pool = case.pool_blocks or max(2 * total, 1)
    assert pool >= total, "block pool smaller than the blocks the sequences need"
    perm = rng.permutation(pool).astype(np.int32)
    width = max(int(need.max()) if len(need) else 1, 1)
    bt = np.full((case.batch, width), -1, dtype=np.int32)
    pos = 0
    for b in range(case.batch):
        n = int(need[b])
        bt[b, :n] = perm[pos:pos + n]
        pos += n
    return bt, pool


def kv_bytes(case, lens):
    """Algorithmic KV bytes one decode step must read: sum ctx * kv_heads * (Dk+Dv) * sizeof
    (the combined MLA cache row is read once: ctx * Dk * sizeof)."""
    per_tok = case.kv_heads * (case.dk if case.mla else case.dk + case.dv) * case.kv_elem_bytes
    return int(np.asarray(lens, dtype=np.int64).sum()) * per_tok


def attn_flops(case, lens):
    return int(np.asarray(lens, dtype=np.int64).sum()) * case.heads * 2 * (case.dk + case.dv)


def _normal(rng, shape, dtype):
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.uint16 if dtype == "bf16" else np.float16)
    step = 1 << 24
    for i in range(0, n, step):
        chunk = rng.standard_normal(min(step, n - i), dtype=np.float32)
        out[i:i + step] = encode(chunk, dtype)
    return out.reshape(shape)


def make_host_inputs(case):
    """All tensors of one decode step as numpy arrays (use for cases that fit comfortably in RAM)."""
    lens = context_lens(case)
    bt, pool = block_tables(case, lens)
    rng = np.random.default_rng(case.seed + 13)
    d = {"context_lens": lens, "block_tables": bt, "num_blocks": pool}
    d["q"] = _normal(rng, (case.batch, case.heads, case.dk), case.q_dtype)
    kshape = (pool, case.block_size, case.kv_heads, case.dk)
    vshape = (pool, case.block_size, case.kv_heads, case.dv)
    if case.kvd == "int8":
        d["k_cache"] = rng.integers(-127, 128, size=kshape, dtype=np.int8)
        d["v_cache"] = rng.integers(-127, 128, size=vshape, dtype=np.int8)
        d["k_descale"] = rng.uniform(0.005, 0.02, case.kv_heads * case.dk).astype(np.float16).astype(np.float32)
        d["v_descale"] = rng.uniform(0.005, 0.02, case.kv_heads * case.dv).astype(np.float16).astype(np.float32)
        if case.offsets:
            d["k_offset"] = rng.integers(-20, 20, case.kv_heads * case.dk).astype(np.int32)
            d["v_offset"] = rng.integers(-20, 20, case.kv_heads * case.dv).astype(np.int32)
    else:
        d["k_cache"] = _normal(rng, kshape, case.kvd)
        d["v_cache"] = None if case.mla else _normal(rng, vshape, case.kvd)
    # the new token of every sequence (what ReshapeAndCache writes before attention reads it)
    d["new_k"] = (rng.integers(-127, 128, size=(case.batch, case.kv_heads, case.dk), dtype=np.int8)
                  if case.kvd == "int8" else _normal(rng, (case.batch, case.kv_heads, case.dk), case.kvd))
    if not case.mla:
        d["new_v"] = (rng.integers(-127, 128, size=(case.batch, case.kv_heads, case.dv), dtype=np.int8)
                      if case.kvd == "int8" else _normal(rng, (case.batch, case.kv_heads, case.dv), case.kvd))
    else:
        d["new_v"] = None
    d["slot_mapping"] = last_token_slots(case, lens, bt)
    return d


def last_token_slots(case, lens, bt):
    """Physical slot of each sequence's newest token (position ctx-1); -1 for empty sequences."""
    slots = np.full(case.batch, -1, dtype=np.int32)
    for b in range(case.batch):
        n = int(lens[b])
        if n > 0:
            slots[b] = int(bt[b, (n - 1) // case.block_size]) * case.block_size + (n - 1) % case.block_size
    return slots


def torch_dtype(name):
    import torch
    return {"fp16": torch.float16, "bf16": torch.bfloat16, "int8": torch.int8}[name]


def make_device_inputs(case, device):
    """Same step, with the big tensors generated directly on `device` by a seeded torch generator.

    Control tensors (context_lens, block_tables, slot_mapping) are the numpy ones of
    make_host_inputs, so the host planner sees identical lengths.  Returns torch tensors plus the
    numpy control arrays under the keys '*_host'.
    """
    import torch
    lens = context_lens(case)
    bt, pool = block_tables(case, lens)
    g = torch.Generator(device=device)
    g.manual_seed(case.seed + 13)
    qd, kd = torch_dtype(case.q_dtype), torch_dtype(case.kvd)
    d = {"context_lens_host": lens, "block_tables_host": bt, "num_blocks": pool}
    d["q"] = torch.randn((case.batch, case.heads, case.dk), generator=g, device=device, dtype=torch.float32).to(qd)
    kshape = (pool, case.block_size, case.kv_heads, case.dk)
    vshape = (pool, case.block_size, case.kv_heads, case.dv)

    def normal(shape, dt):
        out = torch.empty(shape, device=device, dtype=dt)
        flat = out.view(-1)
        step = 1 << 26
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randn(n, generator=g, device=device, dtype=torch.float32).to(dt)
        return out

    def int8(shape):
        out = torch.empty(shape, device=device, dtype=torch.int8)
        flat = out.view(-1)
        step = 1 << 26
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randint(-127, 128, (n,), generator=g, device=device, dtype=torch.int8)
        return out

    if case.kvd == "int8":
        d["k_cache"], d["v_cache"] = int8(kshape), int8(vshape)
        rng = np.random.default_rng(case.seed + 17)
        ks = rng.uniform(0.005, 0.02, case.kv_heads * case.dk).astype(np.float16).astype(np.float32)
        vs = rng.uniform(0.005, 0.02, case.kv_heads * case.dv).astype(np.float16).astype(np.float32)
        d["k_descale"] = torch.from_numpy(ks).to(device)
        d["v_descale"] = torch.from_numpy(vs).to(device)
        d["new_k"] = int8((case.batch, case.kv_heads, case.dk))
        d["new_v"] = int8((case.batch, case.kv_heads, case.dv))
    else:
        d["k_cache"] = normal(kshape, kd)
        d["v_cache"] = None if case.mla else normal(vshape, kd)
        d["new_k"] = normal((case.batch, case.kv_heads, case.dk), kd)
        d["new_v"] = None if case.mla else normal((case.batch, case.kv_heads, case.dv), kd)
    d["block_tables"] = torch.from_numpy(bt).to(device)
    d["context_lens"] = torch.from_numpy(lens).to(device)
    slots = last_token_slots(case, lens, bt)
    d["slot_mapping_host"] = slots
    d["slot_mapping"] = torch.from_numpy(slots).to(device)
    return d


def torch_to_host(t, dtype):
    """torch tensor -> numpy in this module's host encoding (bf16 as uint16 bits)."""
    import torch
    t = t.detach().cpu().contiguous()
    if dtype == "bf16":
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


# Small cases mirroring the shapes of the reference's own regression tests
# (tests/apitest/kernelstest/mix/test_paged_attention_common.py:1574-2961 and
# tests/apitest/kernelstest/mix/test_paged_attention_mla.py:713-721 of the reference); data is seeded.
SMALL_CASES = [
    Case("mha_fp16_no_mask", batch=6, heads=32, kv_heads=32, q_dtype="fp16", ctx=("uniform", 819, 819), seed=11),
    Case("gqa8_fp16_short", batch=13, heads=8, kv_heads=1, q_dtype="fp16", ctx=("uniform", 88, 88), seed=12),
    Case("gqa127_fp16", batch=5, heads=127, kv_heads=1, q_dtype="fp16", ctx=("uniform", 88, 88), seed=13),
    Case("gqa15_fp16", batch=6, heads=30, kv_heads=2, q_dtype="fp16", ctx=("uniform", 88, 88), seed=14),
    Case("odd_heads_fp16", batch=5, heads=33, kv_heads=33, q_dtype="fp16", ctx=("uniform", 88, 88), seed=15),
    Case("gqa12_splitkv_fp16", batch=1, heads=12, kv_heads=1, q_dtype="fp16", ctx=("uniform", 16390, 16390), seed=16),
    Case("gqa12_splitkv_bf16", batch=3, heads=12, kv_heads=1, q_dtype="bf16", ctx=("uniform", 32768, 32768), seed=17),
    Case("cross_group_bf16", batch=5, heads=8, kv_heads=4, q_dtype="bf16", ctx=("uniform", 13164, 13164), seed=18),
    Case("ragged_d96_bs16_fp16", batch=9, heads=40, kv_heads=40, dk=96, dv=96, block_size=16, q_dtype="fp16",
         ctx=("list", [3000, 300, 14000, 33, 65, 1, 16, 14000, 300]), seed=19),
    Case("int8_fp16_norm", batch=24, heads=8, kv_heads=8, q_dtype="fp16", kv_dtype="int8",
         ctx=("uniform", 256, 256), seed=20),
    Case("int8_bf16_gqa", batch=16, heads=8, kv_heads=1, q_dtype="bf16", kv_dtype="int8",
         ctx=("uniform", 256, 256), seed=21),
    Case("int8_fp16_gqa_offsets", batch=16, heads=8, kv_heads=1, q_dtype="fp16", kv_dtype="int8", offsets=True,
         ctx=("uniform", 256, 256), seed=22),
    Case("int8_splitkv_offsets", batch=1, heads=8, kv_heads=8, q_dtype="fp16", kv_dtype="int8", offsets=True,
         ctx=("uniform", 1780, 1780), seed=23),
    Case("mla_8h_fp16", batch=8, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="fp16", mla=True,
         ctx=("uniform", 819, 819), seed=24),
    Case("mla_8h_bf16", batch=8, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
         ctx=("uniform", 819, 819), seed=25),
    Case("mla_128h_bf16", batch=20, heads=128, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
         ctx=("uniform", 256, 256), seed=26),
    Case("zero_and_one_ctx", batch=6, heads=8, kv_heads=2, q_dtype="bf16",
         ctx=("list", [0, 1, 127, 128, 129, 0]), seed=27),
    Case("gqa4_bf16_mid", batch=7, heads=32, kv_heads=8, q_dtype="bf16", ctx=("uniform", 100, 1500), seed=28),
]
