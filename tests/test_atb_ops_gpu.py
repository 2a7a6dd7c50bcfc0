"""The atb::Operation layer on the GPU: CreateOperation -> Setup -> Execute on a VariantPack, as the
reference's demos and OperationTorch harness drive it (example/op_demo/paged_attention/paged_attention_demo.cpp:94-134
of the reference), checked against the oracle."""
import ctypes

import numpy as np
import pytest

import oracle
from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, to_dev, tol_for, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

_STREAMS = []


def _new_ctx():
    """A context with its own (non-null) stream, as the reference requires; inputs made on torch's
    default stream are synchronised first."""
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    _STREAMS.append(s)
    return capi.Context(s.cuda_stream)


def _run_pa_op(case, h, param, scale_encoding="fp32"):
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=wl.torch_dtype(case.q_dtype), device="cuda")
    lens_dev = torch.from_numpy(h["context_lens"]).cuda()
    ins = [T(d["q"]), T(d["k_cache"])]
    if not case.mla:
        ins.append(T(d["v_cache"]))
    ins += [T(d["block_tables"]), T(lens_dev, host=h["context_lens"])]
    keep = []
    if case.kvd == "int8":
        def enc(a):
            if scale_encoding == "fp32":
                t = torch.from_numpy(a).cuda()
            elif scale_encoding == "int64":
                t = torch.from_numpy(a.view(np.uint32).astype(np.int64)).cuda()
            else:
                t = torch.from_numpy(a.astype(np.float16)).cuda()
            keep.append(t)
            return T(t)
        ins.append(enc(h["k_descale"]))
        if case.offsets:
            ins.append(T(d["k_offset"]))
        ins.append(enc(h["v_descale"]))
        if case.offsets:
            ins.append(T(d["v_offset"]))
    outs = [T(out)]
    op = capi.Operation(param)
    assert op.input_num == len(ins)
    ctx = _new_ctx()
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    # a second Setup/Execute pair on the same operation (next decode step re-plans)
    ws_bytes2 = op.setup(ins, outs, ctx)
    ws2 = torch.empty(max(ws_bytes2, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws2.data_ptr(), ws_bytes2, ctx)
    torch.cuda.synchronize()
    return wl.torch_to_host(out, case.q_dtype)


def test_c1_reshape_and_cache_then_paged_attention():
    case = wl.CONFIGS[0]
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    nk, nv = to_dev(h["new_k"], case.kvd), to_dev(h["new_v"], case.kvd)
    slots = torch.from_numpy(h["slot_mapping"]).cuda()
    rac = capi.Operation(capi.ReshapeAndCacheParam())
    ctx = _new_ctx()
    ins = [T(nk), T(nv), T(d["k_cache"]), T(d["v_cache"]), T(slots)]
    outs = [T(d["k_cache"]), T(d["v_cache"])]          # outputs alias the caches
    assert rac.setup(ins, outs, ctx) == 0
    rac.execute(ins, outs, None, 0, ctx)
    torch.cuda.synchronize()
    kc, vc = h["k_cache"].copy(), h["v_cache"].copy()
    oracle.reshape_and_cache(h["new_k"], h["new_v"], kc, vc, h["slot_mapping"])
    assert np.array_equal(wl.torch_to_host(d["k_cache"], case.kvd), kc)
    assert np.array_equal(wl.torch_to_host(d["v_cache"], case.kvd), vc)
    h2 = dict(h, k_cache=kc, v_cache=vc)
    param = capi.PagedAttentionParam(headNum=32, kvHeadNum=32, qkScale=case.qk_scale)
    out = _run_pa_op(case, h2, param)
    assert max_abs_err(out, oracle_out(case, h2), "fp16") <= 2e-3


def test_reshape_and_cache_outputs_must_alias():
    T = capi.atb_tensor
    k = torch.zeros((2, 2, 8), dtype=torch.float16, device="cuda")
    kc = torch.zeros((2, 4, 2, 8), dtype=torch.float16, device="cuda")
    other = torch.zeros_like(kc)
    slots = torch.zeros(2, dtype=torch.int32, device="cuda")
    p = capi.ReshapeAndCacheParam()
    p.kvCacheCfg = 1
    op = capi.Operation(p)
    ctx = _new_ctx()
    op.setup([T(k), T(kc), T(slots)], [T(other)], ctx)
    with pytest.raises(capi.AtbError) as e:
        op.execute([T(k), T(kc), T(slots)], [T(other)], None, 0, ctx)
    assert e.value.code == capi.ERROR_INVALID_TENSOR_ADDR


def test_siso_reshape_and_cache_mla_row():
    T = capi.atb_tensor
    rng = np.random.default_rng(3)
    key = torch.from_numpy(rng.standard_normal((32, 1, 576), dtype=np.float32)).cuda().to(torch.bfloat16)
    kc = torch.zeros((10, 128, 1, 576), dtype=torch.bfloat16, device="cuda")
    slots_h = rng.choice(1280, 32, replace=False).astype(np.int32)
    slots_h[3] = -1
    slots = torch.from_numpy(slots_h).cuda()
    p = capi.ReshapeAndCacheParam()
    p.kvCacheCfg = 1
    op = capi.Operation(p)
    ctx = _new_ctx()
    op.setup([T(key), T(kc), T(slots)], [T(kc)], ctx)
    op.execute([T(key), T(kc), T(slots)], [T(kc)], None, 0, ctx)
    torch.cuda.synchronize()
    ref = torch.zeros_like(kc).view(-1, 1, 576)
    for i, s in enumerate(slots_h):
        if s >= 0:
            ref[s] = key[i]
    assert torch.equal(ref.view_as(kc), kc)


@pytest.mark.parametrize("name", ["gqa4_bf16_mid", "gqa15_fp16", "ragged_d96_bs16_fp16"])
def test_paged_attention_op_plain(name):
    case = [c for c in wl.SMALL_CASES if c.name == name][0]
    h = wl.make_host_inputs(case)
    param = capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale)
    out = _run_pa_op(case, h, param)
    assert max_abs_err(out, oracle_out(case, h), case.q_dtype) <= tol_for(case)


@pytest.mark.parametrize("enc", ["fp32", "int64", "fp16"])
def test_paged_attention_op_dequant_fusion(enc):
    case = [c for c in wl.SMALL_CASES if c.name == "int8_fp16_gqa_offsets"][0]
    h = wl.make_host_inputs(case)
    param = capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale,
                                     quantType=1, hasQuantOffset=True)
    out = _run_pa_op(case, h, param, scale_encoding=enc)
    assert max_abs_err(out, oracle_out(case, h), case.q_dtype) <= 1e-2


def test_paged_attention_op_mla_and_qscale():
    case = [c for c in wl.SMALL_CASES if c.name == "mla_8h_bf16"][0]
    h = wl.make_host_inputs(case)
    # qScale folds into the score scale: qkScale * qScale must equal the case's scale
    param = capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=1, qkScale=case.qk_scale * 2.0, qScale=0.5,
                                     mlaVHeadSize=512)
    out = _run_pa_op(case, h, param)
    assert max_abs_err(out, oracle_out(case, h), case.q_dtype) <= tol_for(case)


def test_paged_attention_operation_stores_into_the_gathered_buffer():
    """Heads sharded over the GPUs of a node, driven through the operator: with gather peers set on the context the
    Execute stores this rank's heads into the gathered [tokens, all heads, Dv] buffer and leaves attnOut alone.
    One GPU stands for a world of one here (the 2-GPU form is in test_multi_gpu.py)."""
    case = wl.Case("op_gather", batch=5, heads=16, kv_heads=4, q_dtype="bf16", ctx=("uniform", 100, 2500), seed=91)
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    total_heads, offset = 48, 16                         # this rank owns heads 16..31 of a 48-head model
    out = torch.full((case.batch, case.heads, case.dv), 7.0, dtype=torch.bfloat16, device="cuda")
    gathered = torch.zeros((case.batch, total_heads, case.dv), dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    lens_dev = torch.from_numpy(h["context_lens"]).cuda()
    ins = [T(d["q"]), T(d["k_cache"]), T(d["v_cache"]), T(d["block_tables"]), T(lens_dev, host=h["context_lens"])]
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale))
    ctx = _new_ctx()
    peers = capi.PaPeers()
    peers.world, peers.rank, peers.total_heads, peers.head_offset = 1, 0, total_heads, offset
    peers.peer_out[0], peers.peer_flags[0] = gathered.data_ptr(), flags.data_ptr()
    ref = oracle_out(case, h)
    for step in (1, 2):
        peers.epoch = step
        ctx.set_gather(peers)
        ws_bytes = op.setup(ins, outs, ctx)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
        op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
        torch.cuda.synchronize()
        got = wl.torch_to_host(gathered[:, offset:offset + case.heads].contiguous(), case.q_dtype)
        assert max_abs_err(got, ref, case.q_dtype) <= tol_for(case)
        assert float(gathered[:, :offset].float().abs().max()) == 0.0
        assert float(out.float().min()) == 7.0 and float(out.float().max()) == 7.0
        assert int(flags[0]) == step
        gathered.zero_()
    # switched off again: the ordinary output
    ctx.set_gather(None)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    assert max_abs_err(wl.torch_to_host(out, case.q_dtype), ref, case.q_dtype) <= tol_for(case)


def test_stream_sync_every_operation(monkeypatch):
    """ATB_STREAM_SYNC_EVERY_OPERATION_ENABLE=1 (src/atb/utils/config.cpp:36 and
    src/atb/operation/operation_base.cpp:1059-1062 of the reference): Execute returns with its stream drained."""
    case = wl.CONFIGS[1]                                   # ~130 us of kernel time: not done by the time a launch returns
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    out = torch.zeros((case.batch, case.heads, case.dv), dtype=wl.torch_dtype(case.q_dtype), device="cuda")
    lens_dev = torch.from_numpy(h["context_lens"]).cuda()
    ins = [T(d["q"]), T(d["k_cache"]), T(d["v_cache"]), T(d["block_tables"]), T(lens_dev, host=h["context_lens"])]
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale))
    ctx = _new_ctx()
    stream = _STREAMS[-1]
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    monkeypatch.setenv("ATB_STREAM_SYNC_EVERY_OPERATION_ENABLE", "1")
    for _ in range(3):
        op.setup(ins, outs, ctx)
        op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
        assert stream.query()                              # nothing left in flight
    monkeypatch.setenv("ATB_STREAM_SYNC_EVERY_OPERATION_ENABLE", "0")
    op.setup(ins, outs, ctx)
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    assert max_abs_err(wl.torch_to_host(out, case.q_dtype), oracle_out(case, h), case.q_dtype) <= tol_for(case)


def test_tensor_dump_before_and_after_execute(monkeypatch, tmp_path):
    """ATB_SAVE_TENSOR_DIR: every Execute writes its tensors before and after the launch (the reference's Probe hooks,
    src/atb/runner/runner.cpp:102-135): intensor<i>.bin / outtensor<i>.bin, one text header line and the raw bytes."""
    case = wl.CONFIGS[0]
    h = wl.make_host_inputs(case)
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    nk, nv = to_dev(h["new_k"], case.kvd), to_dev(h["new_v"], case.kvd)
    slots = torch.from_numpy(h["slot_mapping"]).cuda()
    rac = capi.Operation(capi.ReshapeAndCacheParam())
    ctx = _new_ctx()
    ins = [T(nk), T(nv), T(d["k_cache"]), T(d["v_cache"]), T(slots)]
    outs = [T(d["k_cache"]), T(d["v_cache"])]
    k_before = wl.torch_to_host(d["k_cache"], case.kvd).copy()
    monkeypatch.setenv("ATB_SAVE_TENSOR_DIR", str(tmp_path))
    assert rac.setup(ins, outs, ctx) == 0
    rac.execute(ins, outs, None, 0, ctx)
    monkeypatch.delenv("ATB_SAVE_TENSOR_DIR")
    torch.cuda.synchronize()
    dirs = sorted(p.name for p in tmp_path.iterdir())
    assert len(dirs) == 1 and dirs[0].startswith("0_") and "ReshapeAndCache" in dirs[0]

    def load(path):
        raw = path.read_bytes()
        head, body = raw.split(b"\n", 1)
        f = dict(kv.split("=") for kv in head.decode().split())
        assert int(f["bytes"]) == len(body)
        return f, body

    base = tmp_path / dirs[0]
    assert sorted(p.name for p in (base / "before").iterdir()) == ["intensor0.bin", "intensor1.bin", "intensor2.bin", "intensor3.bin",
                                                                    "intensor4.bin", "outtensor0.bin", "outtensor1.bin"]
    f, body = load(base / "before" / "intensor0.bin")
    assert f["dims"] == ",".join(str(x) for x in h["new_k"].shape) and int(f["dtype"]) == capi.ACL_FLOAT16
    assert body == h["new_k"].tobytes()
    _, cache_before = load(base / "before" / "outtensor0.bin")
    _, cache_after = load(base / "after" / "outtensor0.bin")
    assert cache_before == k_before.tobytes()
    kc, vc = h["k_cache"].copy(), h["v_cache"].copy()
    oracle.reshape_and_cache(h["new_k"], h["new_v"], kc, vc, h["slot_mapping"])
    assert cache_after == kc.tobytes() and cache_after != cache_before
    _, slots_bytes = load(base / "after" / "intensor4.bin")
    assert slots_bytes == h["slot_mapping"].tobytes()
