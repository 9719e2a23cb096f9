"""CPU restatement of the reference's torch goldens for the quantized DeepSeek-V3.2 decode path.

TEST INFRASTRUCTURE ONLY. Nothing under this directory is imported by the `pypto_b200` package;
only the test-suite, the repository smoke check and the benchmark's CPU-baseline leg use it, and
there only as the checker / the timed CPU baseline, never as the product path.

Parity is pinned: the restatement is checked (tests/test_oracle_golden.py) against outputs of the
reference's own golden functions, produced by importing the reference's example drivers with
tests/golden/make_golden.py and committed under tests/golden/.
"""
from .li_oracle import (li_scores, li_scores_fp16_chain, li_scores_nonquant, li_topk, lightning_indexer,  # noqa: F401
                        lightning_indexer_nonquant)
from .sfa_oracle import (dequantised_cache, sparse_attention, sparse_attention_online,  # noqa: F401
                         sparse_attention_packed)
from .compare import attention_errors, topk_set_diff  # noqa: F401
