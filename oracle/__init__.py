"""CPU oracle for the paged-decode hot path (test infrastructure only).

Only tests, the smoke check and the CPU-baseline leg of the bench may import this package; the
product library never does.  `pa_oracle.c` restates the reference's CPU golden
(tests/apitest/kernelstest/mix/test_paged_attention_common.py:229-366 and
tests/apitest/kernelstest/mix/test_reshape_and_cache.py:45-68 of the reference) and is pinned
against outputs of those Python functions stored under tests/golden/.
"""
from .oracle import (attention_lse, build, load, multi_latent_attention, num_threads, paged_attention,  # noqa: F401
                     paged_attention_qkv_quant,
                     paged_attention_spec, reshape_and_cache)
from . import cache_ops  # noqa: F401
