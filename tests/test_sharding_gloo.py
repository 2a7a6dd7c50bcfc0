"""The multi-GPU host logic on CPU: two gloo ranks shard a decode step by kv head, compute their
shards (with the CPU oracle standing in for the kernels), all-gather the outputs and must reproduce
the unsharded result exactly."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, case_kw, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import __graft_entry__ as entry
    import oracle
    pkg = entry.load_package()
    wl, sh = pkg.workloads, pkg.sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    mine = sh.shard_host_inputs(case, h, rank, world)
    shard = case.shard_heads(rank, world)
    # this rank's slice of the step: cache update, then attention over its kv heads
    oracle.reshape_and_cache(mine["new_k"], mine["new_v"], mine["k_cache"], mine["v_cache"], mine["slot_mapping"])
    out = oracle.paged_attention(mine["q"], mine["k_cache"], mine["v_cache"], mine["block_tables"],
                                 mine["context_lens"], shard.qk_scale, shard.q_dtype, kv_dtype=shard.kvd, dv=shard.dv,
                                 k_descale=mine.get("k_descale"), v_descale=mine.get("v_descale"),
                                 k_offset=mine.get("k_offset"), v_offset=mine.get("v_offset"), nthreads=2)
    out_t = torch.from_numpy(out.view(np.int16) if out.dtype == np.uint16 else out)
    gathered = sh.all_gather_outputs(out_t)
    full = sh.gathered_to_full(gathered).contiguous().numpy()
    if rank == 0:
        np.save(os.path.join(result_dir, "full.npy"), full)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case_kw", [
    dict(name="shard_gqa", batch=5, heads=16, kv_heads=4, q_dtype="bf16", ctx=("list", [1, 100, 129, 300, 64]), seed=51),
    dict(name="shard_int8", batch=3, heads=8, kv_heads=2, q_dtype="fp16", kv_dtype="int8", offsets=True,
         ctx=("list", [70, 200, 131]), seed=52),
], ids=lambda k: k["name"])
def test_two_rank_head_sharding_reproduces_unsharded_result(case_kw, tmp_path):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    import oracle
    oracle.build()
    pkg = entry.load_package()
    wl = pkg.workloads
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), case_kw, str(tmp_path)), nprocs=world, join=True)
    full = np.load(os.path.join(str(tmp_path), "full.npy"))
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    oracle.reshape_and_cache(h["new_k"], h["new_v"], h["k_cache"], h["v_cache"], h["slot_mapping"])
    ref = oracle.paged_attention(h["q"], h["k_cache"], h["v_cache"], h["block_tables"], h["context_lens"],
                                 case.qk_scale, case.q_dtype, kv_dtype=case.kvd, dv=case.dv,
                                 k_descale=h.get("k_descale"), v_descale=h.get("v_descale"),
                                 k_offset=h.get("k_offset"), v_offset=h.get("v_offset"))
    ref_bits = ref.view(np.int16) if ref.dtype == np.uint16 else ref
    assert full.shape == ref_bits.shape
    assert np.array_equal(full, ref_bits)


def _rank_main_sequences(rank, world, port, case_kw, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import __graft_entry__ as entry
    import oracle
    pkg = entry.load_package()
    wl, sh = pkg.workloads, pkg.sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    mine = sh.shard_host_inputs_by_sequence(case, h, rank, world)
    # this rank's sequences: cache update (its own new tokens only), then attention
    oracle.reshape_and_cache(mine["new_k"], None, mine["k_cache"], None, mine["slot_mapping"])
    out = oracle.paged_attention(mine["q"], mine["k_cache"], None, mine["block_tables"], mine["context_lens"],
                                 case.qk_scale, case.q_dtype, dv=case.dv, nthreads=2)
    out_t = torch.from_numpy(out.view(np.int16) if out.dtype == np.uint16 else out)
    gathered = sh.all_gather_outputs(out_t)
    full = sh.gathered_sequences_to_full(gathered).contiguous().numpy()
    if rank == 0:
        np.save(os.path.join(result_dir, "full.npy"), full)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sequence_sharding_of_the_mla_cache_reproduces_unsharded_result(tmp_path):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    import oracle
    oracle.build()
    pkg = entry.load_package()
    wl = pkg.workloads
    case_kw = dict(name="shard_mla", batch=4, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                   ctx=("list", [70, 200, 131, 1]), seed=53)
    world = 2
    mp.spawn(_rank_main_sequences, args=(world, _free_port(), case_kw, str(tmp_path)), nprocs=world, join=True)
    full = np.load(os.path.join(str(tmp_path), "full.npy"))
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    oracle.reshape_and_cache(h["new_k"], None, h["k_cache"], None, h["slot_mapping"])
    ref = oracle.paged_attention(h["q"], h["k_cache"], None, h["block_tables"], h["context_lens"], case.qk_scale,
                                 case.q_dtype, dv=case.dv)
    ref_bits = ref.view(np.int16) if ref.dtype == np.uint16 else ref
    assert full.shape == ref_bits.shape
    assert np.array_equal(full, ref_bits)


def test_sequence_shards_of_a_case_keep_its_lengths():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    wl = entry.load_package().workloads
    case = wl.CONFIGS[4]
    lens = wl.context_lens(case)
    parts = [wl.context_lens(case.shard_sequences(r, 4)) for r in range(4)]
    assert np.array_equal(np.concatenate(parts), lens)
    assert all(case.shard_sequences(r, 4).batch == case.batch // 4 for r in range(4))


def test_mla_cannot_be_head_sharded():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    pkg = entry.load_package()
    case = pkg.workloads.CONFIGS[4]
    with pytest.raises(ValueError):
        pkg.sharding.head_slices(case, 0, 2)
