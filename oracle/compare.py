"""Comparison rules for the decode path.

Top-k: set comparison per row, as the reference's `topk_idx_compare`
(deepseekv32_lightning_indexer_quant.py:272-314) does, but exact: a differing index is accepted
only when its score is tied with the k-th score (torch.topk's tie order is unspecified).
Attention: max-abs and relative L2 error, plus the reference's element-count rule
(utils/compare.py:83-128: |a-b| > atol + rtol*|b| on at most 0.5 % of the elements).
"""
from __future__ import annotations

import torch


def topk_set_diff(got_row, want_row, score_row=None, rel_tie=1e-6):
    """Returns (n_missing_untied, n_missing_tied) for one row of indices."""
    got = set(int(x) for x in got_row.reshape(-1).tolist() if x >= 0)
    want = set(int(x) for x in want_row.reshape(-1).tolist() if x >= 0)
    if got == want:
        return 0, 0
    diff = (got - want) | (want - got)
    if score_row is None or len(want) == 0:
        return len(diff), 0
    kth = min(float(score_row[i]) for i in want)
    tied = sum(1 for i in diff if 0 <= i < len(score_row) and abs(float(score_row[i]) - kth) <= rel_tie * abs(kth))
    return len(diff) - tied, tied


def attention_errors(got, want):
    g = got.to(torch.float32).reshape(-1)
    w = want.to(torch.float32).reshape(-1)
    diff = (g - w).abs()
    max_abs = float(diff.max()) if diff.numel() else 0.0
    denom = float(w.norm())
    rel_l2 = float((g - w).norm()) / denom if denom > 0 else float((g - w).norm())
    bad = int((diff > 1e-4 + 5e-3 * w.abs()).sum())
    return dict(max_abs=max_abs, rel_l2=rel_l2, bad_frac=bad / max(g.numel(), 1))
