"""The small seeded cases whose reference-golden outputs are stored in this directory."""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG_DIR = os.path.join(ROOT, "ascend-transformer-boost_b200")


def load_workloads():
    """The package directory name is not a Python identifier, so load the module by path."""
    name = "atb_b200_workloads"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_wl = load_workloads()
Case = _wl.Case

GOLDEN_PA_CASES = [
    Case("mha_fp16", batch=3, heads=4, kv_heads=4, q_dtype="fp16", ctx=("list", [1, 130, 300]), seed=101),
    Case("gqa4_bf16", batch=2, heads=8, kv_heads=2, q_dtype="bf16", ctx=("list", [200, 257]), seed=102),
    Case("gqa8_fp16", batch=2, heads=8, kv_heads=1, q_dtype="fp16", ctx=("list", [88, 129]), seed=103),
    Case("d96_bs16_fp16", batch=3, heads=5, kv_heads=5, dk=96, dv=96, block_size=16, q_dtype="fp16",
         ctx=("list", [33, 1, 65]), seed=104),
    Case("int8_fp16", batch=2, heads=8, kv_heads=8, q_dtype="fp16", kv_dtype="int8", ctx=("list", [150, 64]),
         seed=105),
    Case("int8_bf16_gqa_offsets", batch=2, heads=8, kv_heads=1, q_dtype="bf16", kv_dtype="int8", offsets=True,
         ctx=("list", [140, 256]), seed=106),
    Case("int8_fp16_gqa_offsets", batch=2, heads=8, kv_heads=2, q_dtype="fp16", kv_dtype="int8", offsets=True,
         ctx=("list", [77, 131]), seed=107),
    Case("mla_bf16", batch=2, heads=8, kv_heads=1, dk=576, dv=512, q_dtype="bf16", mla=True,
         ctx=("list", [140, 90]), seed=108),
    Case("mla_fp16", batch=2, heads=16, kv_heads=1, dk=576, dv=512, q_dtype="fp16", mla=True,
         ctx=("list", [129, 60]), seed=109),
    Case("dk_ne_dv_fp16", batch=2, heads=4, kv_heads=2, dk=192, dv=128, q_dtype="fp16", ctx=("list", [70, 140]),
         seed=110),
]

GOLDEN_RAC_CASES = [
    dict(name="fp16_eq", tokens=20, heads=4, dk=32, dv=32, block_size=16, num_blocks=6, dtype="fp16", seed=201),
    dict(name="bf16_dk_ne_dv", tokens=17, heads=3, dk=48, dv=24, block_size=8, num_blocks=9, dtype="bf16", seed=202),
    dict(name="int8_mla_like", tokens=30, heads=2, dk=576, dv=512, block_size=16, num_blocks=5, dtype="int8",
         seed=203),
    dict(name="fp16_odd", tokens=11, heads=5, dk=7, dv=13, block_size=4, num_blocks=10, dtype="fp16", seed=204),
]


def rac_inputs(spec):
    """Seeded ReshapeAndCache inputs: distinct slots drawn from [-num_slots, num_slots) as the
    reference test does (negative slots must be skipped)."""
    rng = np.random.default_rng(spec["seed"])
    n, h = spec["tokens"], spec["heads"]
    num_slots = spec["block_size"] * spec["num_blocks"]
    slots = rng.choice(np.arange(-num_slots, num_slots), size=n, replace=False).astype(np.int32)

    def gen(d):
        if spec["dtype"] == "int8":
            return rng.integers(-127, 128, size=(n, h, d), dtype=np.int8)
        return _wl.encode(rng.standard_normal((n, h, d), dtype=np.float32), spec["dtype"])

    return {"key": gen(spec["dk"]), "value": gen(spec["dv"]), "slot_mapping": slots}
