"""KV-head sharding of one decode step over the GPUs of a node.

Rank r of R owns kv heads [r*Hkv/R, (r+1)*Hkv/R) with their query heads, i.e. a cache shard
[num_blocks, block_size, Hkv/R, D]; block tables, context lengths and slot mapping are replicated.
Attention is independent per kv head, so the only exchange is an all-gather of the per-rank outputs
[tokens, heads/R, Dv]; the gathered tensor is rank-major [R, tokens, heads/R, Dv] (the convention of
ATB's AllGatherOperation, src/ops/ops_infer/all_gather/all_gather_operation.cpp:79-89 of the
reference) and `gathered_to_full` views it as [tokens, heads, Dv].
The MLA combined cache has a single kv head (kvHeadNum == 1 is enforced,
src/ops/ops_infer/paged_attention/paged_attention_operation.cpp:355-358) and cannot be sharded this
way; it is sharded by sequence instead: rank r owns the contiguous sequences
[r*B/R, (r+1)*B/R) with their cache blocks (data-parallel attention), and the all-gather of the
per-rank outputs [B/R, heads, Dv] along the first dimension is already the final [B, heads, Dv].
"""
import numpy as np


def head_slices(case, rank, world):
    if case.kv_heads % world != 0:
        raise ValueError(f"{case.kv_heads} kv heads cannot be split over {world} ranks")
    hkv = case.kv_heads // world
    group = case.heads // case.kv_heads
    return slice(rank * hkv, (rank + 1) * hkv), slice(rank * hkv * group, (rank + 1) * hkv * group)


def shard_host_inputs(case, h, rank, world):
    """Slices the numpy inputs of workloads.make_host_inputs down to one rank's heads."""
    kvs, qs = head_slices(case, rank, world)
    d = dict(h)
    d["q"] = np.ascontiguousarray(h["q"][:, qs])
    d["k_cache"] = np.ascontiguousarray(h["k_cache"][:, :, kvs])
    d["v_cache"] = None if h["v_cache"] is None else np.ascontiguousarray(h["v_cache"][:, :, kvs])
    d["new_k"] = np.ascontiguousarray(h["new_k"][:, kvs])
    d["new_v"] = None if h["new_v"] is None else np.ascontiguousarray(h["new_v"][:, kvs])
    for name, width in (("k_descale", case.dk), ("v_descale", case.dv), ("k_offset", case.dk), ("v_offset", case.dv)):
        if h.get(name) is not None:
            d[name] = np.ascontiguousarray(h[name].reshape(case.kv_heads, width)[kvs].reshape(-1))
    return d


def sequence_slice(batch, rank, world):
    """Contiguous sequences of one rank when a step is sharded by sequence (MLA)."""
    if batch % world != 0:
        raise ValueError(f"{batch} sequences cannot be split evenly over {world} ranks")
    per = batch // world
    return slice(rank * per, (rank + 1) * per)


def shard_host_inputs_by_sequence(case, h, rank, world):
    """Slices the numpy inputs of workloads.make_host_inputs down to one rank's sequences.  The block
    pool stays whole (a real deployment gives each rank only its sequences' blocks; the ids in the
    block tables are unchanged here, so the result is identical)."""
    sl = sequence_slice(case.batch, rank, world)
    d = dict(h)
    for name in ("q", "block_tables", "context_lens", "slot_mapping", "new_k", "new_v"):
        if h.get(name) is not None:
            d[name] = np.ascontiguousarray(h[name][sl])
    return d


def gathered_sequences_to_full(gathered):
    """[R, B/R, heads, Dv] (rank-major all-gather of sequence shards) -> [B, heads, Dv], a pure view."""
    r, b, hh, dv = gathered.shape
    return gathered.reshape(r * b, hh, dv)


def gathered_to_full(gathered):
    """[R, tokens, heads/R, Dv] (rank-major all-gather result) -> [tokens, heads, Dv]."""
    r, b, hl, dv = gathered.shape
    if hasattr(gathered, "permute"):
        return gathered.permute(1, 0, 2, 3).reshape(b, r * hl, dv)
    return np.transpose(gathered, (1, 0, 2, 3)).reshape(b, r * hl, dv)


def all_gather_outputs(out_local, gathered=None):
    """NCCL / gloo all-gather of the per-rank outputs into a rank-major buffer."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size()
    if gathered is None:
        gathered = torch.empty((world,) + tuple(out_local.shape), dtype=out_local.dtype, device=out_local.device)
    # gathered as raw bytes: every backend (NCCL, gloo) moves uint8, whatever the element type
    dist.all_gather_into_tensor(gathered.view(torch.uint8).view(-1), out_local.contiguous().view(torch.uint8).view(-1))
    return gathered
