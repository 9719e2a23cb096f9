"""The operators as `torch.library` custom ops, so that `torch.compile` traces a model that calls them
without a graph break and a compiled model can be recorded into a CUDA graph.

The reference reaches the same end by wrapping a jitted kernel in `torch._dynamo.allow_in_graph` with a
FakeTensor branch that returns an empty result (examples/03_advanced/aclgraph/aclgraph.py:96-106,
docs/tutorials/network_integration/PyTorch集成和接入.md:10-45). Here every operator writes into buffers the
caller passes, so each op is registered with those buffers in `mutates_args`, returns nothing, and its fake
implementation does nothing: tracing needs no shapes from it and the functionalisation pass knows which
arguments change. Importing this module registers the namespace `torch.ops.pypto_b200`:

    import pypto_b200.torch_ops
    torch.ops.pypto_b200.decode_indexer_attention_quant(idx_query, ..., topk_res, attention_out, 128, scale, 2048,
                                                        False, False)

Arguments are plain tensors and scalars (the tiling objects of the reference's signatures carry nothing
this implementation reads, so they are not part of the op schemas).
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import ops

_NS = "pypto_b200"


@torch.library.custom_op(f"{_NS}::lightning_indexer_decode", mutates_args=("topk_res",))
def lightning_indexer_decode(idx_query: Tensor, idx_query_scale: Tensor, idx_key_cache: Tensor, idx_key_scale: Tensor,
                             idx_weight: Tensor, act_seq_key: Tensor, block_table: Tensor, topk_res: Tensor,
                             selected_count: int = 2048, sort: bool = True, fp16_chain: bool = False) -> None:
    ops.lightning_indexer_decode(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                                 block_table, topk_res, None, None, selected_count, sort=sort, fp16_chain=fp16_chain)


@torch.library.custom_op(f"{_NS}::sparse_flash_attention_quant", mutates_args=("attention_out",))
def sparse_flash_attention_quant(query_nope: Tensor, query_rope: Tensor, key_nope_2d: Tensor, key_rope_2d: Tensor,
                                 k_nope_scales: Tensor, topk_indices: Tensor, block_table: Tensor, kv_act_seqs: Tensor,
                                 attention_out: Tensor, nq: int, n_kv: int, softmax_scale: float, topk: int,
                                 block_size: int, max_blocknum_perbatch: int, head_begin: int = 0,
                                 nq_total: int = -1) -> None:
    ops.sparse_flash_attention_quant_d(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                       block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk,
                                       block_size, max_blocknum_perbatch, None, head_begin=head_begin,
                                       nq_total=None if nq_total < 0 else nq_total)


@torch.library.custom_op(f"{_NS}::sparse_attention_antiquant", mutates_args=("attention_out",))
def sparse_attention_antiquant(query_nope: Tensor, query_rope: Tensor, nope_cache: Tensor, topk_indices: Tensor,
                               block_table: Tensor, kv_act_seqs: Tensor, attention_out: Tensor, nq: int, n_kv: int,
                               softmax_scale: float, topk: int, block_size: int, max_blocknum_perbatch: int) -> None:
    ops.sparse_attention_antiquant_d(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                     attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                     None)


@torch.library.custom_op(f"{_NS}::decode_indexer_attention_quant", mutates_args=("topk_res", "attention_out"))
def decode_indexer_attention_quant(idx_query: Tensor, idx_query_scale: Tensor, idx_key_cache: Tensor,
                                   idx_key_scale: Tensor, idx_weight: Tensor, query_nope: Tensor, query_rope: Tensor,
                                   key_nope_2d: Tensor, key_rope_2d: Tensor, k_nope_scales: Tensor, act_seq: Tensor,
                                   block_table: Tensor, topk_res: Tensor, attention_out: Tensor, nq: int = 128,
                                   softmax_scale: float = 576 ** -0.5, selected_count: int = 2048, sort: bool = False,
                                   fp16_chain: bool = False) -> None:
    ops.decode_indexer_attention_quant(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight,
                                       query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, act_seq,
                                       block_table, topk_res, attention_out, nq, softmax_scale, selected_count,
                                       sort=sort, fp16_chain=fp16_chain)


@torch.library.custom_op(f"{_NS}::lightning_indexer_topk_nonquant", mutates_args=("topk_res",))
def lightning_indexer_topk_nonquant(idx_query: Tensor, idx_key_cache: Tensor, idx_weight: Tensor, act_seq_key: Tensor,
                                    block_table: Tensor, topk_res: Tensor, selected_count: int = 2048,
                                    sort: bool = True) -> None:
    ops.lightning_indexer_topk_nonquant(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table, topk_res,
                                        selected_count, sort=sort)


@torch.library.custom_op(f"{_NS}::decode_indexer_attention", mutates_args=("topk_res", "attention_out"))
def decode_indexer_attention(idx_query: Tensor, idx_key_cache: Tensor, idx_weight: Tensor, query_nope: Tensor,
                             query_rope: Tensor, key_nope_2d: Tensor, key_rope_2d: Tensor, act_seq: Tensor,
                             block_table: Tensor, topk_res: Tensor, attention_out: Tensor, nq: int = 128,
                             softmax_scale: float = 576 ** -0.5, selected_count: int = 2048,
                             sort: bool = False) -> None:
    ops.decode_indexer_attention(idx_query, idx_key_cache, idx_weight, query_nope, query_rope, key_nope_2d, key_rope_2d,
                                 act_seq, block_table, topk_res, attention_out, nq, softmax_scale, selected_count,
                                 sort=sort)


_PROLOG_OUT = ("mla_kv_cache", "mla_kr_cache", "mla_k_scale_cache", "ip_k_cache", "ip_k_cache_scale",
               "mla_query_nope_out", "mla_query_rope_out", "ip_q_int8_out", "ip_q_scale_out", "ip_weights_out")


@torch.library.custom_op(f"{_NS}::mla_indexer_prolog_quant", mutates_args=_PROLOG_OUT)
def mla_indexer_prolog_quant(token_x: Tensor, mla_w_dq: Tensor, mla_w_uq_qr: Tensor, mla_dequant_scale: Tensor,
                             mla_w_uk: Tensor, mla_w_dkv_kr: Tensor, mla_gamma_cq: Tensor, mla_gamma_ckv: Tensor,
                             cos: Tensor, sin: Tensor, cache_index: Tensor, mla_kv_cache: Tensor, mla_kr_cache: Tensor,
                             mla_k_scale_cache: Tensor, ip_w_qb_in: Tensor, ip_w_qb_scale_in: Tensor, ip_wk_in: Tensor,
                             ip_w_proj_in: Tensor, ip_ln_gamma_k_in: Tensor, ip_ln_beta_k_in: Tensor,
                             ip_hadamard_q_in: Tensor, ip_hadamard_k_in: Tensor, ip_k_cache: Tensor,
                             ip_k_cache_scale: Tensor, mla_query_nope_out: Tensor, mla_query_rope_out: Tensor,
                             ip_q_int8_out: Tensor, ip_q_scale_out: Tensor, ip_weights_out: Tensor,
                             mla_epsilon_cq: float, mla_epsilon_ckv: float) -> None:
    """The five caches are updated in place (the reference's separate `*_out` cache arguments alias them)."""
    ops.mla_indexer_prolog_quant_d(token_x, mla_w_dq, mla_w_uq_qr, mla_dequant_scale, mla_w_uk, mla_w_dkv_kr,
                                   mla_gamma_cq, mla_gamma_ckv, cos, sin, cache_index, mla_kv_cache, mla_kr_cache,
                                   mla_k_scale_cache, ip_w_qb_in, ip_w_qb_scale_in, ip_wk_in, ip_w_proj_in,
                                   ip_ln_gamma_k_in, ip_ln_beta_k_in, ip_hadamard_q_in, ip_hadamard_k_in, ip_k_cache,
                                   ip_k_cache_scale, mla_query_nope_out, mla_query_rope_out, mla_kv_cache,
                                   mla_kr_cache, mla_k_scale_cache, ip_q_int8_out, ip_q_scale_out, ip_k_cache,
                                   ip_k_cache_scale, ip_weights_out, mla_epsilon_cq, mla_epsilon_ckv)


@torch.library.custom_op(f"{_NS}::mla_indexer_prolog",
                         mutates_args=("kv_cache", "kr_cache", "idx_k_cache", "query_nope_out", "query_rope_out",
                                       "idx_query_out", "idx_weights_out"))
def mla_indexer_prolog(token_x: Tensor, w_dq: Tensor, w_uq_qr: Tensor, w_uk: Tensor, w_dkv_kr: Tensor, gamma_cq: Tensor,
                       gamma_ckv: Tensor, cos: Tensor, sin: Tensor, cache_index: Tensor, kv_cache: Tensor,
                       kr_cache: Tensor, idx_w_qb: Tensor, idx_wk: Tensor, idx_w_proj: Tensor, idx_ln_gamma: Tensor,
                       idx_ln_beta: Tensor, idx_k_cache: Tensor, query_nope_out: Tensor, query_rope_out: Tensor,
                       idx_query_out: Tensor, idx_weights_out: Tensor, epsilon_cq: float = 1e-5,
                       epsilon_ckv: float = 1e-5) -> None:
    """The two prologs of the non-quantised chain; the three bf16 caches are updated in place."""
    ops.mla_indexer_prolog(token_x, w_dq, w_uq_qr, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index, kv_cache,
                           kr_cache, idx_w_qb, idx_wk, idx_w_proj, idx_ln_gamma, idx_ln_beta, idx_k_cache,
                           query_nope_out, query_rope_out, idx_query_out, idx_weights_out, epsilon_cq, epsilon_ckv)


def _no_result(*args, **kwargs) -> None:
    return None


OPS = (lightning_indexer_decode, sparse_flash_attention_quant, sparse_attention_antiquant,
       decode_indexer_attention_quant, lightning_indexer_topk_nonquant, decode_indexer_attention,
       mla_indexer_prolog_quant, mla_indexer_prolog)
for _op in OPS:
    _op.register_fake(_no_result)
