"""KV-head sharding of one decode step over the GPUs of a node.

Rank r of R owns kv heads [r*Hkv/R, (r+1)*Hkv/R) with their query heads, i.e. a cache shard
[num_blocks, block_size, Hkv/R, D]; block tables, context lengths and slot mapping are replicated.
Attention is independent per kv head, so the only exchange is an all-gather of the per-rank outputs
[tokens, heads/R, Dv]; the gathered tensor is rank-major [R, tokens, heads/R, Dv] (the convention of
ATB's AllGatherOperation, src/ops/ops_infer/all_gather/all_gather_operation.cpp:79-89 of the
reference) and `gathered_to_full` views it as [tokens, heads, Dv].
The MLA combined cache has a single kv head and cannot be sharded this way.
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
