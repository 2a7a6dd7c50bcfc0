"""Decode on 2 GPUs, as child processes (one per GPU); skipped when fewer than 2 GPUs are visible.

Head-sharded: each rank's attention kernel stores its heads into every rank's gathered output through peer
memory; both ranks must end up with the unsharded oracle result.  Sequence-sharded (the MLA cache has one kv
head): each rank runs its contiguous share of the batch and the outputs are all-gathered along the first
dimension (NCCL); the result must equal the unsharded oracle result too."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

pytestmark = pytest.mark.gpu
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
    pkg = entry.load_package()
    wl, sh, capi = pkg.workloads, pkg.sharding, pkg.capi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from helpers import host_inputs_to_device, to_dev
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    mine = sh.shard_host_inputs(case, h, rank, world)
    shard = case.shard_heads(rank, world)
    d = host_inputs_to_device(shard, mine)
    nk, nv = to_dev(mine["new_k"], shard.kvd), to_dev(mine["new_v"], shard.kvd)
    slots = torch.from_numpy(mine["slot_mapping"]).cuda()
    tdt = wl.torch_dtype(case.q_dtype)
    ex = capi.PeerExchange(case.batch * case.heads * case.dv * 2, case.heads, rank * shard.heads)
    desc = capi.make_desc(shard.batch, shard.heads, shard.kv_heads, 128, 128, 128, h["num_blocks"],
                          h["block_tables"].shape[1], shard.q_dtype, shard.kvd, shard.qk_scale)
    plan = capi.PaPlan(desc, h["context_lens"])
    ws = torch.empty(max(int(plan.info.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
    tens = capi.pa_tensors(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], None, d["k_descale"],
                           d["v_descale"], d["k_offset"], d["v_offset"])
    results = []
    for step in range(3):                  # alternates the two gathered buffers
        capi.reshape_and_cache(nk, nv, d["k_cache"], d["v_cache"], slots)
        peers, local_ptr = ex.peers()
        plan.launch_gathered(tens, peers, ws.data_ptr(), ws.numel(), capi.torch_stream_ptr())
        torch.cuda.synchronize()
        assert plan.device_status(ws.data_ptr(), capi.torch_stream_ptr()) == 0
        full = ex.local_tensor(local_ptr, (case.batch, case.heads, case.dv), tdt)
        results.append(wl.torch_to_host(full.clone(), case.q_dtype))
    np.save(os.path.join(result_dir, f"full_{rank}.npy"), np.stack(results))
    ex.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("case_kw", [
    dict(name="p2p_gqa", batch=9, heads=32, kv_heads=8, q_dtype="bf16", ctx=("uniform", 60, 3000), seed=61),
    dict(name="p2p_int8", batch=5, heads=16, kv_heads=2, q_dtype="fp16", kv_dtype="int8", offsets=True,
         ctx=("uniform", 100, 2000), seed=62),
], ids=lambda k: k["name"])
def test_peer_store_gather_matches_oracle(case_kw, tmp_path):
    sys.path.insert(0, ROOT)
    import oracle
    from helpers import max_abs_err, tol_for, wl
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), case_kw, str(tmp_path)), nprocs=world, join=True)
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    oracle.reshape_and_cache(h["new_k"], h["new_v"], h["k_cache"], h["v_cache"], h["slot_mapping"])
    ref = oracle.paged_attention(h["q"], h["k_cache"], h["v_cache"], h["block_tables"], h["context_lens"],
                                 case.qk_scale, case.q_dtype, kv_dtype=case.kvd, dv=case.dv,
                                 k_descale=h.get("k_descale"), v_descale=h.get("v_descale"),
                                 k_offset=h.get("k_offset"), v_offset=h.get("v_offset"))
    for rank in range(world):
        got = np.load(os.path.join(str(tmp_path), f"full_{rank}.npy"))
        for step in range(got.shape[0]):
            g = got[step].view(ref.dtype) if got.dtype != ref.dtype else got[step]
            assert max_abs_err(g, ref, case.q_dtype) <= tol_for(case), (rank, step)


def _mla_rank_main(rank, world, port, case_kw, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    wl, sh, capi = pkg.workloads, pkg.sharding, pkg.capi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from helpers import to_dev
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    mine = sh.shard_host_inputs_by_sequence(case, h, rank, world)
    q = to_dev(mine["q"], case.q_dtype)
    kc = to_dev(mine["k_cache"], case.kvd)
    bt = torch.from_numpy(mine["block_tables"]).cuda()
    nk = to_dev(mine["new_k"], case.kvd)
    slots = torch.from_numpy(mine["slot_mapping"]).cuda()
    capi.reshape_and_cache(nk, None, kc, None, slots)
    out = capi.paged_attention(q, kc, None, bt, mine["context_lens"], case.qk_scale, dv=case.dv)
    gathered = sh.all_gather_outputs(out)
    torch.cuda.synchronize()
    full = sh.gathered_sequences_to_full(gathered)
    np.save(os.path.join(result_dir, f"mla_full_{rank}.npy"), wl.torch_to_host(full, case.q_dtype))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_sharded_mla_matches_oracle(tmp_path):
    sys.path.insert(0, ROOT)
    import oracle
    from helpers import max_abs_err, tol_for, wl
    case_kw = dict(name="seqshard_mla", batch=6, heads=128, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
                   ctx=("list", [700, 64, 1500, 129, 3000, 257]), seed=63)
    world = 2
    mp.spawn(_mla_rank_main, args=(world, _free_port(), case_kw, str(tmp_path)), nprocs=world, join=True)
    case = wl.Case(**case_kw)
    h = wl.make_host_inputs(case)
    oracle.reshape_and_cache(h["new_k"], None, h["k_cache"], None, h["slot_mapping"])
    ref = oracle.paged_attention(h["q"], h["k_cache"], None, h["block_tables"], h["context_lens"], case.qk_scale,
                                 case.q_dtype, dv=case.dv)
    for rank in range(world):
        got = np.load(os.path.join(str(tmp_path), f"mla_full_{rank}.npy"))
        g = got.view(ref.dtype) if got.dtype != ref.dtype else got
        assert max_abs_err(g, ref, case.q_dtype) <= tol_for(case), rank
