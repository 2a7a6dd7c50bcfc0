"""Host-side logic of bench.py that needs no GPU: the sub-batches of the pipelined end-to-end step."""
import importlib.util
import os

import numpy as np

from helpers import wl

_spec = importlib.util.spec_from_file_location("bench_module", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
bench = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bench)


def _check_cover(chunks, batch):
    assert chunks[0][0] == 0 and chunks[-1][1] == batch
    for (a0, a1), (b0, b1) in zip(chunks, chunks[1:]):
        assert a1 == b0 and a0 < a1
    assert chunks[-1][0] < chunks[-1][1]


def test_sub_batches_cover_the_batch_and_balance_tokens():
    for idx, step_ms in ((3, 0.509), (2, 0.231), (4, 0.130), (1, 0.130), (0, 0.024)):
        case = wl.CONFIGS[idx]
        lens = wl.context_lens(case)
        chunks = bench.e2e_chunks(case, lens, 1, step_ms)
        _check_cover(chunks, case.batch)
        tokens = [int(np.sum(lens[a:b])) for a, b in chunks]
        if len(chunks) > 1:
            assert max(tokens) - min(tokens) <= 2 * int(np.max(lens)), (case.name, tokens)
    # copies that are small next to the kernel: no pipelining; large: two or four sub-batches
    assert len(bench.e2e_chunks(wl.CONFIGS[1], wl.context_lens(wl.CONFIGS[1]), 1, 0.130)) == 1
    assert len(bench.e2e_chunks(wl.CONFIGS[3], wl.context_lens(wl.CONFIGS[3]), 1, 0.509)) == 4
    assert len(bench.e2e_chunks(wl.CONFIGS[4], wl.context_lens(wl.CONFIGS[4]), 1, 0.130)) == 2
    # never at N > 1, never more sub-batches than half the batch, a forced count is honoured
    assert len(bench.e2e_chunks(wl.CONFIGS[3], wl.context_lens(wl.CONFIGS[3]), 8, 0.509)) == 1
    small = wl.Case("tiny", batch=3, heads=8, kv_heads=8, q_dtype="fp16", ctx=("list", [5, 6, 7]), seed=1)
    assert len(bench.e2e_chunks(small, np.array([5, 6, 7]), 1, 1e-6, forced=4)) == 1
    forced = bench.e2e_chunks(wl.CONFIGS[1], wl.context_lens(wl.CONFIGS[1]), 1, 0.130, forced=3)
    assert len(forced) == 3
    _check_cover(forced, wl.CONFIGS[1].batch)
