"""Times the REFERENCE's own Python golden of paged attention, as it is, on benchmark configuration 1.

    python tests/golden/time_reference_golden.py /path/to/ascend-transformer-boost

The golden (tests/apitest/kernelstest/mix/test_paged_attention_common.py:229-366 of the reference) gathers the
cache token by token in Python and runs torch matmuls per sequence; it exists to check results, not to be fast.
It can only run where the reference checkout is, so this figure is taken on the authoring machine and quoted in
BASELINE.md / DESIGN.md; bench.py times the C restatement of the same arithmetic instead (`cpu_baseline`, kind
"port"), which is what travels to the GPU box.  Prints one JSON line.
"""
import json
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import make_golden as mg  # noqa: E402


def main():
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    ref_root = sys.argv[1]
    mg._stub_modules()
    kt = os.path.join(ref_root, "tests/apitest/kernelstest")
    sys.path.insert(0, kt)
    sys.path.insert(0, os.path.join(kt, "mix"))
    cwd = os.getcwd()
    os.chdir(os.path.join(kt, "mix"))
    common = mg._load(os.path.join(kt, "mix/test_paged_attention_common.py"), "ref_pa_common")
    os.chdir(cwd)
    wl = mg.wl
    case = wl.CONFIGS[0]
    torch.set_num_threads(os.cpu_count() or 1)
    d = wl.make_host_inputs(case)
    t = common.TestPagedAttention()
    t.compressHead = False
    t.is_int8_flag = False
    t.is_quant_flag = 0
    t.has_bias = False
    t.scaleType = 0
    t.num_heads, t.kv_heads, t.num_tokens, t.head_size = case.heads, case.kv_heads, case.batch, case.dk
    q, kc, vc = (mg.to_torch(d[k], case.q_dtype) for k in ("q", "k_cache", "v_cache"))
    times = []
    for _ in range(3):
        out = torch.zeros((case.batch, case.heads, case.dv), dtype=torch.float32)
        high = torch.zeros_like(out)
        t0 = time.perf_counter()
        t.ref_single_query_cached_kv_attention(out, high, q, kc, vc, d["block_tables"].tolist(), d["context_lens"].tolist(),
                                               None, None, False, mask_dim=0, mask_data_type=torch.float16)
        times.append(time.perf_counter() - t0)
    dt = min(times)
    kvb = wl.kv_bytes(case, d["context_lens"])
    print(json.dumps({"workload": case.name, "impl": "reference Python golden, unmodified", "seconds": dt,
                      "kv_gb_per_s": kvb / dt / 1e9, "tokens": int(d["context_lens"].sum()),
                      "cores": os.cpu_count(), "torch_threads": torch.get_num_threads()}))


if __name__ == "__main__":
    main()
