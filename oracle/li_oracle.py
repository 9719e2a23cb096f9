"""Lightning-indexer oracle (CPU, torch, vectorised per sequence).

Follows the reference golden `lightning_indexer_compute`
(examples/models/deepseek_v32_exp/deepseekv32_lightning_indexer_quant.py:184-269):

  d     = int32(q . k)                      per (head, key)          (:223-224)
  h     = fp16( relu(fp32(d)) * 2^-11 )                              (:224-226)
  ws    = q_scale * weight    in the scales' own dtype               (:212)
  score = ( sum_h fp32(ws_h) * fp32(h) ) * fp32(k_scale)             (:235-238)
  top-k over score[:eff_seq], eff_seq = S - (s1 - 1 - i), padded with -1 (:244-262)

The integer dot is evaluated as an fp32 matmul: |d| <= 128*127*127 < 2^24 and every partial sum is
an integer below 2^24, so fp32 accumulation is exact in any order and equals the int32 result.
"""
from __future__ import annotations

import torch

BLOCK = 128


def _gather_pages(cache2d: torch.Tensor, table_row: torch.Tensor, seq: int, block_size: int):
    n_pages = (seq + block_size - 1) // block_size
    pages = table_row[:n_pages].long()
    rows = (pages[:, None] * block_size + torch.arange(block_size)[None, :]).reshape(-1)[:seq]
    return cache2d[rows], rows


def li_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq, block_table, s1,
              return_first_mm=False):
    """Per query token the fp32 score row over its sequence's keys.

    Returns a list (length t) of 1-D fp32 tensors of length S_b (all keys of the sequence, the
    causal cut is applied by `li_topk`). With `return_first_mm` also the fp16 [64, S_b] tiles
    (the reference ST's `first_mm` hook).
    """
    t, n_heads, dim = idx_query.shape
    block_num, block_size = idx_key_cache.shape[0], idx_key_cache.shape[1]
    keys2d = idx_key_cache.reshape(block_num * block_size, dim)
    kscale1d = idx_key_scale.reshape(block_num * block_size)
    b = len(act_seq)
    assert t == b * s1
    rows_out, fm_out = [], []
    for bi in range(b):
        seq = int(act_seq[bi])
        k, rows = _gather_pages(keys2d, block_table[bi], seq, block_size)
        kf = k.to(torch.float32)  # [S, 128]
        ks = kscale1d[rows].to(torch.float32)  # [S]
        for i in range(s1):
            ti = bi * s1 + i
            q = idx_query[ti].to(torch.float32)  # [64, 128]
            d = q @ kf.T  # exact integers in fp32
            h = (torch.relu(d) * (1.0 / 2048)).to(torch.float16)
            ws = (idx_query_scale[ti] * idx_weight[ti]).to(torch.float32)  # product in own dtype
            score = (ws[None, :] @ h.to(torch.float32)).reshape(-1) * ks
            rows_out.append(score)
            if return_first_mm:
                fm_out.append(h)
    return (rows_out, fm_out) if return_first_mm else rows_out


def li_scores_fp16_chain(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq, block_table, s1):
    """The older quantised formulation, `LightningIndexerTopkImpl`
    (framework/src/operator/models/deepseek_v3.2_exp/lightning_indexer.cpp:150-196; golden
    `indexer_topk_compute(is_quant=True)`, framework/tests/st/operator/src/test_deepseek_v3.2_exp/
    gen_lightning_indexer.py:243-257): everything between the int32 dot and the head sum stays in fp16,

      h     = fp16( fp32(d) * 2^-11 )          (no relu yet)
      a     = fp16( fp16(h * q_scale_h) * k_scale_key )
      m     = fp16( relu(a) * weight_h )
      score = sum_h fp32(m)

    with fp16 scales and weights. Same return value as `li_scores`."""
    t, n_heads, dim = idx_query.shape
    block_num, block_size = idx_key_cache.shape[0], idx_key_cache.shape[1]
    assert idx_query_scale.dtype == torch.float16 and idx_key_scale.dtype == torch.float16
    assert idx_weight.dtype == torch.float16
    keys2d = idx_key_cache.reshape(block_num * block_size, dim)
    kscale1d = idx_key_scale.reshape(block_num * block_size)
    b = len(act_seq)
    rows_out = []
    for bi in range(b):
        seq = int(act_seq[bi])
        k, rows = _gather_pages(keys2d, block_table[bi], seq, block_size)
        kf = k.to(torch.float32)
        ks = kscale1d[rows]  # fp16 [S]
        for i in range(s1):
            ti = bi * s1 + i
            d = idx_query[ti].to(torch.float32) @ kf.T  # [64, S], exact integers
            h = (d * (1.0 / 2048)).to(torch.float16)
            a = (h * idx_query_scale[ti].reshape(-1, 1)) * ks.reshape(1, -1)  # two fp16 products, left to right
            m = torch.relu(a) * idx_weight[ti].reshape(-1, 1)
            rows_out.append(m.to(torch.float32).sum(dim=0))
    return rows_out


def li_scores_nonquant(idx_query, idx_key_cache, idx_weight, act_seq, block_table, s1):
    """The non-quantised formulation, `LightningIndexerTopkImpl` with isQuant = false
    (framework/src/operator/models/deepseek_v3.2_exp/lightning_indexer.cpp:113-147; golden
    `indexer_topk_compute(is_quant=False)`, framework/tests/st/operator/src/test_deepseek_v3.2_exp/
    gen_lightning_indexer.py:258-266):

      mm    = fp32(q) @ fp32(k)^T            bf16 inputs, fp32 product        (:258)
      score = sum_h relu(mm_h) * fp32(w_h)   fp32                             (:260-263)

    Same return value as `li_scores`."""
    t, n_heads, dim = idx_query.shape
    block_num, block_size = idx_key_cache.shape[0], idx_key_cache.shape[1]
    keys2d = idx_key_cache.reshape(block_num * block_size, dim)
    b = len(act_seq)
    rows_out = []
    for bi in range(b):
        seq = int(act_seq[bi])
        k, _ = _gather_pages(keys2d, block_table[bi], seq, block_size)
        kf = k.to(torch.float32)
        for i in range(s1):
            ti = bi * s1 + i
            mm = idx_query[ti].to(torch.float32) @ kf.T  # [64, S]
            w = idx_weight[ti].to(torch.float32).reshape(-1, 1)
            rows_out.append((torch.relu(mm) * w).sum(dim=0))
    return rows_out


def lightning_indexer_nonquant(idx_query, idx_key_cache, idx_weight, act_seq, block_table, s1, selected_count=2048):
    rows = li_scores_nonquant(idx_query, idx_key_cache, idx_weight, act_seq, block_table, s1)
    idx, vals = li_topk(rows, act_seq, s1, selected_count)
    return idx, vals, rows


def li_topk(score_rows, act_seq, s1, selected_count=2048):
    """Exact top-k per row over the causal prefix; value-descending; -1 padding."""
    t = len(score_rows)
    out = torch.full((t, 1, selected_count), -1, dtype=torch.int32)
    vals = torch.full((t, selected_count), float("-inf"), dtype=torch.float32)
    for ti in range(t):
        bi, i = divmod(ti, s1)
        eff = int(act_seq[bi]) - (s1 - 1 - i)
        if eff <= 0:
            continue
        k = min(eff, selected_count)
        v, idx = torch.topk(score_rows[ti][:eff], k)
        out[ti, 0, :k] = idx.to(torch.int32)
        vals[ti, :k] = v
    return out, vals


def lightning_indexer(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq, block_table,
                      s1, selected_count=2048, fp16_chain=False):
    fn = li_scores_fp16_chain if fp16_chain else li_scores
    rows = fn(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq, block_table, s1)
    idx, vals = li_topk(rows, act_seq, s1, selected_count)
    return idx, vals, rows
