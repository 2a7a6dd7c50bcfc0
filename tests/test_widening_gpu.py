"""GPU tests of what was added to the operator layer after the hot path (dynamic batch, ...).  They sit
in a file of their own, collected after the hot-path tests: a failure here stops nothing that the
parity contract of the hot path depends on."""
import numpy as np
import pytest

from helpers import capi, host_inputs_to_device, max_abs_err, oracle_out, tol_for, wl

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _run_dynamic_batch(case, h, status, extra_rows=0):
    """PagedAttention with batchRunStatusEnable through the atb operator API; the control tensors may
    carry `extra_rows` more sequences than there are query tokens."""
    d = host_inputs_to_device(case, h)
    T = capi.atb_tensor
    out = torch.full((case.batch, case.heads, case.dv), 7.0, dtype=wl.torch_dtype(case.q_dtype), device="cuda")
    lens_h = np.concatenate([h["context_lens"], np.full(extra_rows, 33, dtype=np.int32)])
    bt = d["block_tables"]
    if extra_rows:
        bt = torch.cat([bt, torch.zeros((extra_rows, bt.shape[1]), dtype=bt.dtype, device="cuda")])
    lens_dev = torch.from_numpy(lens_h).cuda()
    status_h = np.concatenate([np.asarray(status, dtype=np.int32), np.ones(extra_rows, dtype=np.int32)])
    status_dev = torch.from_numpy(status_h).cuda()
    ins = [T(d["q"]), T(d["k_cache"]), T(d["v_cache"]), T(bt), T(lens_dev, host=lens_h), T(status_dev, host=status_h)]
    outs = [T(out)]
    op = capi.Operation(capi.PagedAttentionParam(headNum=case.heads, kvHeadNum=case.kv_heads, qkScale=case.qk_scale,
                                                 batchRunStatusEnable=True))
    assert op.input_num == len(ins)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    ctx = capi.Context(stream.cuda_stream)
    ws_bytes = op.setup(ins, outs, ctx)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    op.execute(ins, outs, ws.data_ptr(), ws_bytes, ctx)
    torch.cuda.synchronize()
    return wl.torch_to_host(out, case.q_dtype)


@pytest.mark.parametrize("extra_rows", [0, 2])
def test_dynamic_batch_skips_switched_off_sequences(extra_rows):
    # lengths and status pattern of the reference's test_pa_fp16_case_dynamic_batch_1
    # (tests/apitest/kernelstest/mix/test_paged_attention_common.py:1723-1741)
    lens = [2028, 0, 707, 0, 15, 1] * 2
    status = [1, 0, 1, 0, 1, 1] * 2
    status[4] = 0                                # a switched-off sequence that still has a length
    case = wl.Case("dyn_batch", batch=len(lens), heads=32, kv_heads=32, q_dtype="fp16", ctx=("list", lens), seed=81)
    h = wl.make_host_inputs(case)
    out = _run_dynamic_batch(case, h, status, extra_rows)
    eff = dict(h, context_lens=np.where(np.asarray(status) == 0, 0, h["context_lens"]).astype(np.int32))
    ref = oracle_out(case, eff, out=np.full((case.batch, case.heads, case.dv), 7.0, dtype=np.float16))
    assert max_abs_err(out, ref, case.q_dtype) <= tol_for(case)
    off = [b for b, s in enumerate(status) if s == 0]
    assert np.all(out[off] == np.float16(7.0))   # rows of skipped sequences are left untouched
