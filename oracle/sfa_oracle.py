"""Sparse MLA attention oracle (CPU, torch, one matmul pair per query token).

Follows the reference golden `compute_attention_no_flash`
(examples/models/deepseek_v32_exp/deepseekv32_sparse_flash_attention_quant.py:169-254), the one the
example asserts against (:375):

  n   = clamp(S_b - s1 + 1 + i, 0, topk)                                   (:197)
  r_j = block_table[b, idx_j // bs] * bs + idx_j % bs   for the first n indices  (:213-217)
  kn  = bf16( fp32(int8 row) * scale[r, c // 128] )                         (:226-230)
        (a bf16 `key_nope_2d` is the golden's is_kn_quant = 0 branch, :231-232: kn = the row itself)
  s   = ( fp32(q) @ fp32([kn | kr]).T ) * softmax_scale                     (:238-240)
  P   = bf16( exp(s - max) / sum )                                          (:241-245)
  O   = bf16( fp32(P) @ fp32(kn) )                                          (:246, :248)

`sparse_attention_online` is the un-normalised-P online formulation of `compute_attention`
(:49-166) evaluated in tiles, the model for a split-K GPU kernel; `sparse_attention_packed` reads
the 656-byte packed rows of `compute_attention_aq`
(deepseekv32_sparse_attention_antiquant.py:49-136).
"""
from __future__ import annotations

import torch


def _physical_rows(idx_row, table_row, n, block_size):
    idx = idx_row[:n].long()
    return table_row[idx // block_size].long() * block_size + idx % block_size


def _latent_rows(key_nope_2d, k_nope_scales, rows):
    if key_nope_2d.dtype == torch.bfloat16:  # non-quantised cache: rows are used as they are (:231-232)
        return key_nope_2d[rows]
    return _dequant(key_nope_2d[rows], k_nope_scales[rows])


def _dequant(kn_rows_i8, scales):
    n = kn_rows_i8.shape[0]
    kf = kn_rows_i8.to(torch.float32).reshape(n, 4, 128) * scales.reshape(n, 4, 1)
    return kf.reshape(n, 512).to(torch.bfloat16)


def _valid_count(seq, s1, i, topk):
    return min(max(int(seq) - s1 + 1 + i, 0), topk)


def sparse_attention(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices, block_table,
                     act_seq, s1, nq=128, softmax_scale=576 ** -0.5, topk=2048, block_size=128):
    t = topk_indices.shape[0]
    b = len(act_seq)
    assert t == b * s1
    qn = query_nope.reshape(t, nq, -1)
    qr = query_rope.reshape(t, nq, -1)
    out = torch.zeros((b, s1, nq, qn.shape[-1]), dtype=torch.bfloat16)
    for ti in range(t):
        bi, i = divmod(ti, s1)
        n = _valid_count(act_seq[bi], s1, i, topk)
        if n == 0:
            continue
        rows = _physical_rows(topk_indices[ti], block_table[bi], n, block_size)
        kn = _latent_rows(key_nope_2d, k_nope_scales, rows)
        k = torch.cat([kn, key_rope_2d[rows]], dim=-1).to(torch.float32)
        q = torch.cat([qn[ti], qr[ti]], dim=-1).to(torch.float32)
        s = (q @ k.T) * softmax_scale
        p = torch.exp(s - s.amax(dim=-1, keepdim=True))
        p = (p / p.sum(dim=-1, keepdim=True)).to(torch.bfloat16)
        out[bi, i] = (p.to(torch.float32) @ kn.to(torch.float32)).to(torch.bfloat16)
    return out


def sparse_attention_online(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                            block_table, act_seq, s1, nq=128, softmax_scale=576 ** -0.5, topk=2048, block_size=128,
                            tile=64):
    """Online-softmax evaluation: P = bf16(exp(s - running max)) un-normalised, fp32 (m, l, O)."""
    t = topk_indices.shape[0]
    b = len(act_seq)
    qn = query_nope.reshape(t, nq, -1)
    qr = query_rope.reshape(t, nq, -1)
    out = torch.zeros((b, s1, nq, qn.shape[-1]), dtype=torch.bfloat16)
    for ti in range(t):
        bi, i = divmod(ti, s1)
        n = _valid_count(act_seq[bi], s1, i, topk)
        if n == 0:
            continue
        rows = _physical_rows(topk_indices[ti], block_table[bi], n, block_size)
        kn = _latent_rows(key_nope_2d, k_nope_scales, rows)
        k = torch.cat([kn, key_rope_2d[rows]], dim=-1).to(torch.float32)
        q = torch.cat([qn[ti], qr[ti]], dim=-1).to(torch.float32)
        m = torch.full((nq, 1), float("-inf"))
        l = torch.zeros((nq, 1))
        o = torch.zeros((nq, 512))
        for j0 in range(0, n, tile):
            s = (q @ k[j0:j0 + tile].T) * softmax_scale
            m_new = torch.maximum(m, s.amax(dim=-1, keepdim=True))
            alpha = torch.exp(m - m_new)
            p = torch.exp(s - m_new)
            l = l * alpha + p.sum(dim=-1, keepdim=True)
            o = o * alpha + p.to(torch.bfloat16).to(torch.float32) @ kn[j0:j0 + tile].to(torch.float32)
            m = m_new
        out[bi, i] = (o / l).to(torch.bfloat16)
    return out


def dequantised_cache(key_nope_2d, k_nope_scales):
    """The bf16 latent cache that holds exactly the values the int8 cache dequantises to."""
    return _dequant(key_nope_2d, k_nope_scales)


def unpack_kv_rows(nope_cache):
    """Split [N, 656] int8 rows into (int8 latent [N,512], bf16 rope [N,64], fp32 scales [N,4])."""
    kn = nope_cache[:, :512].contiguous()
    kr = nope_cache[:, 512:640].contiguous().view(torch.bfloat16)
    sc = nope_cache[:, 640:656].contiguous().view(torch.float32)
    return kn, kr, sc


def sparse_attention_packed(query_nope, query_rope, nope_cache, topk_indices, block_table, act_seq, s1, nq=128,
                            softmax_scale=576 ** -0.5, topk=2048, block_size=128):
    kn, kr, sc = unpack_kv_rows(nope_cache)
    return sparse_attention(query_nope, query_rope, kn, kr, sc, topk_indices, block_table, act_seq, s1, nq,
                            softmax_scale, topk, block_size)
