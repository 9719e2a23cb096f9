"""Operators of the quantized DeepSeek-V3.2 sparse-attention decode path, with the reference's
names and positional signatures (examples/models/deepseek_v32_exp):

  lightning_indexer_decode          lightning_indexer_quant_impl.py:315-346
  sparse_flash_attention_quant_d/_p sparse_flash_attention_quant_impl.py:420-476 / :479-538
  sparse_attention_antiquant_d/_p   sparse_attention_antiquant_impl.py:246-358
  decode_indexer_attention_quant    the fused order of
                                    framework/src/operator/models/deepseek_v3.2_exp/deepseek_indexer_attention_quant.cpp:170-250

Like the reference's `pypto.jit` callables (python/pypto/runtime.py:218-253) they take device
tensors (raw torch CUDA tensors or `from_torch` handles), write the output tensor in place, return
None and run asynchronously on the current stream; the caller synchronises. Host-side validation
raises ValueError / RuntimeError / TypeError before anything is launched. The scratch workspace is
a cached torch allocation per (device, stream), so a call inside CUDA-graph capture allocates
nothing once warmed up.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import torch

from . import _lib
from .compat import unwrap

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def workspace_status(device=None):
    """Status words of the current stream's workspace (synchronises the stream).
    Word 0 is an OR of PTO_ST_BAD_PAGE / PTO_ST_WAIT_EXPIRED."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(device, 256)
    out = (C.c_int32 * _lib.PTO_STATUS_WORDS)()
    _lib.check(_lib.load().pto_workspace_status(ws.data_ptr(), out, torch.cuda.current_stream(device).cuda_stream))
    return list(out)


def launch_count() -> int:
    """Kernels of the CUDA library enqueued so far by this process (a launch recorded during stream capture
    counts once, at capture time)."""
    return int(_lib.load().pto_launch_count())


def reset_workspace_status(device=None):
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(device, 256)
    _lib.check(_lib.load().pto_workspace_reset(ws.data_ptr(), torch.cuda.current_stream(device).cuda_stream))


def _need(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


def _same_device(tensors):
    if not tensors:
        raise RuntimeError("at least one tensor is required")
    dev = tensors[0].device
    for t in tensors:
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    if dev.type != "cuda":
        raise RuntimeError(f"tensors are on {dev}; this operator runs on a CUDA device only (no CPU path)")
    return dev


def _scale_dtype(*ts):
    dt = ts[0].dtype
    _need(all(t.dtype == dt for t in ts), "idx_query_scale, idx_key_scale and idx_weight must share one dtype")
    if dt == torch.float16:
        return _lib.PTO_DT_F16
    if dt == torch.float32:
        return _lib.PTO_DT_F32
    raise ValueError(f"scale dtype {dt}: float16 or float32 expected")


def _li_args(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key, block_table):
    q = unwrap(idx_query, "idx_query")
    qs = unwrap(idx_query_scale, "idx_query_scale")
    kc = unwrap(idx_key_cache, "idx_key_cache")
    ks = unwrap(idx_key_scale, "idx_key_scale")
    w = unwrap(idx_weight, "idx_weight")
    act = unwrap(act_seq_key, "act_seq_key")
    bt = unwrap(block_table, "block_table")
    _need(q.dtype == torch.int8 and q.dim() == 3, "idx_query: int8 [t, n_heads, head_dim]")
    t, n_heads, head_dim = q.shape
    _need(kc.dtype == torch.int8 and kc.dim() == 4 and kc.shape[2] == 1 and kc.shape[3] == head_dim,
          "idx_key_cache: int8 [block_num, block_size, 1, head_dim]")
    block_num, block_size = kc.shape[0], kc.shape[1]
    _need(tuple(qs.shape) == (t, n_heads), "idx_query_scale: [t, n_heads]")
    _need(tuple(w.shape) == (t, n_heads), "idx_weight: [t, n_heads]")
    _need(ks.numel() == block_num * block_size, "idx_key_scale: [block_num, block_size, 1]")
    _need(act.dtype == torch.int32 and act.dim() == 1, "act_seq_key: int32 [b]")
    b = act.shape[0]
    _need(b >= 1 and t % b == 0, "t must be a multiple of the batch size")
    _need(bt.dtype == torch.int32 and bt.dim() == 2 and bt.shape[0] == b, "block_table: int32 [b, max_blocks]")
    sd = _scale_dtype(qs, ks, w)
    _need(n_heads == 64 and head_dim == 128 and block_size == 128,
          "indexer geometry: 64 heads x 128 dims, 128-token blocks")
    return None, (q, qs, kc, ks, w, act, bt), dict(t=t, b=b, s1=t // b, n_heads=n_heads, head_dim=head_dim,
                                                   block_size=block_size, block_num=block_num,
                                                   max_blocks=bt.shape[1], scale_dtype=sd)


def _li_args_bf16(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table):
    """Argument check of the non-quantised indexer: bf16 queries, keys and weights, no scales."""
    q = unwrap(idx_query, "idx_query")
    kc = unwrap(idx_key_cache, "idx_key_cache")
    w = unwrap(idx_weight, "idx_weight")
    act = unwrap(act_seq_key, "act_seq_key")
    bt = unwrap(block_table, "block_table")
    bf = torch.bfloat16
    _need(q.dtype == bf and q.numel() % (64 * 128) == 0, "idx_query: bfloat16 [t, 64, 128] (or [b, s1, 64, 128])")
    t = q.numel() // (64 * 128)
    _need(kc.dtype == bf and kc.dim() == 4 and tuple(kc.shape[1:]) == (128, 1, 128),
          "idx_key_cache: bfloat16 [block_num, 128, 1, 128]")
    _need(w.dtype == bf and w.numel() == t * 64, "idx_weight: bfloat16 [t, 64]")
    _need(act.dtype == torch.int32 and act.dim() == 1, "act_seq_key: int32 [b]")
    b = act.shape[0]
    _need(b >= 1 and t % b == 0, "t must be a multiple of the batch size")
    _need(bt.dtype == torch.int32 and bt.dim() == 2 and bt.shape[0] == b, "block_table: int32 [b, max_blocks]")
    return (q, kc, w, act, bt), dict(t=t, b=b, s1=t // b, block_num=kc.shape[0], max_blocks=bt.shape[1])


def lightning_indexer_topk_nonquant(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table, topk_res,
                                    selected_count=2048, tile_config=None, unroll_list=None, *, sort=True,
                                    scores_out=None):
    """The non-quantised indexer, `LightningIndexerTopk(query, key, weights, actSeqKey, blockTable, topkRes,
    selectedCount, tileConfig, unrollList)` (framework/src/operator/models/deepseek_v3.2_exp/lightning_indexer.cpp:
    198-203, body :23-147 with isQuant = false): score = sum_h w_h * relu(q_h . k) over bf16 tensors in fp32, top-
    `selected_count` per query token. `scores_out` (float32 [t, max_blocks*128], optional) receives the score rows
    instead of the top-k running (the reference's `tmpOut` hook)."""
    (q, kc, w, act, bt), m = _li_args_bf16(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table)
    lib = _lib.load()
    common = (m["b"], m["s1"], 64, 128, 128, m["block_num"], m["max_blocks"])
    if scores_out is not None:
        sc = unwrap(scores_out, "scores_out")
        _need(sc.dtype == torch.float32 and sc.numel() == m["t"] * m["max_blocks"] * 128,
              "scores_out: float32 [t, max_blocks*128]")
        dev = _same_device([q, kc, w, act, bt, sc])
        with torch.cuda.device(dev):
            ws = _workspace(dev, lib.pto_li_workspace_bytes(1, 1, 128))
            _lib.check(lib.pto_li_scores_bf16(q.data_ptr(), kc.data_ptr(), w.data_ptr(), act.data_ptr(), bt.data_ptr(),
                                              sc.data_ptr(), *common, 0, ws.data_ptr(), ws.numel(),
                                              torch.cuda.current_stream(dev).cuda_stream))
        return None
    out = unwrap(topk_res, "topk_res")
    _need(out.dtype == torch.int32 and out.numel() == m["t"] * selected_count,
          "topk_res: int32 [t, 1, selected_count]")
    _need(1 <= selected_count <= 2048, "selected_count must be in [1, 2048]")
    dev = _same_device([q, kc, w, act, bt, out])
    nbytes = lib.pto_li_workspace_bytes(m["t"], m["max_blocks"], 128)
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        _lib.check(lib.pto_li_decode_bf16(q.data_ptr(), kc.data_ptr(), w.data_ptr(), act.data_ptr(), bt.data_ptr(),
                                          out.data_ptr(), *common, int(selected_count),
                                          0 if sort else _lib.PTO_LI_UNSORTED, ws.data_ptr(), ws.numel(),
                                          torch.cuda.current_stream(dev).cuda_stream))
    return None


def lightning_indexer_decode(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                             block_table, topk_res, unroll_list=None, configs=None, selected_count=2048, *,
                             sort=True, _simt_scores=False, fp16_chain=False, histogram=False):
    """Top-`selected_count` key positions per query token (value-descending, -1 padded).
    `fp16_chain=True` (not in the reference's Python signature) scores with the older formulation of
    LightningIndexerTopkImpl, lightning_indexer.cpp:150-196 (fp16 scales and weights only).
    A bfloat16 `idx_query` selects the non-quantised formulation (`lightning_indexer_topk_nonquant`; the two scale
    arguments must then be None). `histogram=True` (s1 <= 2): the score kernel leaves a histogram of every row for
    the selection to start from (same results; measured slightly slower, hence off by default)."""
    if unwrap(idx_query, "idx_query").dtype == torch.bfloat16:
        _need(idx_query_scale is None and idx_key_scale is None, "bfloat16 idx_query: the scale tensors must be None")
        _need(not (_simt_scores or fp16_chain), "bfloat16 idx_query: one formulation, tensor cores only")
        return lightning_indexer_topk_nonquant(idx_query, idx_key_cache, idx_weight, act_seq_key, block_table,
                                               topk_res, selected_count, sort=sort)
    dev, (q, qs, kc, ks, w, act, bt), m = _li_args(idx_query, idx_query_scale, idx_key_cache, idx_key_scale,
                                                    idx_weight, act_seq_key, block_table)
    out = unwrap(topk_res, "topk_res")
    _need(out.dtype == torch.int32 and out.numel() == m["t"] * selected_count,
          "topk_res: int32 [t, 1, selected_count]")
    _need(1 <= selected_count <= 2048, "selected_count must be in [1, 2048]")
    dev = _same_device([q, qs, kc, ks, w, act, bt, out])
    lib = _lib.load()
    nbytes = lib.pto_li_workspace_bytes(m["t"], m["max_blocks"], m["block_size"])
    flags = (0 if sort else _lib.PTO_LI_UNSORTED) | (_lib.PTO_LI_SCORE_SIMT if _simt_scores else 0)
    flags |= _lib.PTO_LI_FP16_CHAIN if fp16_chain else 0
    flags |= _lib.PTO_LI_EPILOGUE_HIST if histogram else 0
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        _lib.check(lib.pto_li_decode(q.data_ptr(), qs.data_ptr(), kc.data_ptr(), ks.data_ptr(), w.data_ptr(),
                                     m["scale_dtype"], act.data_ptr(), bt.data_ptr(), out.data_ptr(), m["b"], m["s1"],
                                     m["n_heads"], m["head_dim"], m["block_size"], m["block_num"], m["max_blocks"],
                                     int(selected_count), flags, ws.data_ptr(), ws.numel(),
                                     torch.cuda.current_stream(dev).cuda_stream))
    return None


def lightning_indexer_scores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                             block_table, scores, first_mm=None, *, simt=False, fp16_chain=False):
    """Score stage alone: fp32 [t, max_blocks*block_size] (the reference ST's `mm_out` hook);
    positions at or beyond a sequence's length are left untouched. `first_mm` (fp16
    [t*64, max_blocks*block_size]) is available with simt=True only."""
    dev, (q, qs, kc, ks, w, act, bt), m = _li_args(idx_query, idx_query_scale, idx_key_cache, idx_key_scale,
                                                    idx_weight, act_seq_key, block_table)
    sc = unwrap(scores, "scores")
    stride = m["max_blocks"] * m["block_size"]
    _need(sc.dtype == torch.float32 and tuple(sc.shape) == (m["t"], stride),
          "scores: float32 [t, max_blocks*block_size]")
    fm_ptr = None
    devs = [q, qs, kc, ks, w, act, bt, sc]
    if first_mm is not None:
        fm = unwrap(first_mm, "first_mm")
        _need(simt, "first_mm needs simt=True")
        _need(fm.dtype == torch.float16 and tuple(fm.shape) == (m["t"] * m["n_heads"], stride),
              "first_mm: float16 [t*n_heads, max_blocks*block_size]")
        fm_ptr = fm.data_ptr()
        devs.append(fm)
    dev = _same_device(devs)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(dev, 256)
        _lib.check(lib.pto_li_scores(q.data_ptr(), qs.data_ptr(), kc.data_ptr(), ks.data_ptr(), w.data_ptr(),
                                     m["scale_dtype"], act.data_ptr(), bt.data_ptr(), sc.data_ptr(), fm_ptr, m["b"],
                                     m["s1"], m["n_heads"], m["head_dim"], m["block_size"], m["block_num"],
                                     m["max_blocks"],
                                     (_lib.PTO_LI_SCORE_SIMT if simt else 0) | (_lib.PTO_LI_FP16_CHAIN if fp16_chain else 0),
                                     ws.data_ptr(), ws.numel(),
                                     torch.cuda.current_stream(dev).cuda_stream))
    return None


def lightning_indexer_topk(scores, act_seq_key, topk_res, s1=1, selected_count=2048, *, sort=True):
    """Top-k stage alone over fp32 score rows [t, row_stride]."""
    sc = unwrap(scores, "scores")
    act = unwrap(act_seq_key, "act_seq_key")
    out = unwrap(topk_res, "topk_res")
    _need(sc.dtype == torch.float32 and sc.dim() == 2, "scores: float32 [t, row_stride]")
    _need(act.dtype == torch.int32 and act.dim() == 1 and act.shape[0] * s1 == sc.shape[0], "act_seq_key: int32 [t/s1]")
    _need(out.dtype == torch.int32 and out.numel() == sc.shape[0] * selected_count, "topk_res: int32 [t, 1, k]")
    _need(1 <= selected_count <= 2048, "selected_count must be in [1, 2048]")
    dev = _same_device([sc, act, out])
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(dev, 256)
        _lib.check(lib.pto_li_topk(sc.data_ptr(), sc.shape[1], act.data_ptr(), out.data_ptr(), act.shape[0], int(s1),
                                   int(selected_count), 0 if sort else _lib.PTO_LI_UNSORTED, ws.data_ptr(), ws.numel(),
                                   torch.cuda.current_stream(dev).cuda_stream))
    return None


def _sfa_common(query_nope, query_rope, topk_indices, block_table, kv_act_seqs, attention_out, nq, n_kv, topk,
                nq_total=None, head_begin=0):
    nq_slice, nq = int(nq), int(nq if nq_total is None else nq_total)  # rows per token in the query / output arrays
    _need(0 <= int(head_begin) and int(head_begin) + nq_slice <= nq, "head slice [head_begin, head_begin + nq) outside nq_total")
    qn = unwrap(query_nope, "query_nope")
    qr = unwrap(query_rope, "query_rope")
    ti = unwrap(topk_indices, "topk_indices")
    bt = unwrap(block_table, "block_table")
    act = unwrap(kv_act_seqs, "kv_act_seqs")
    out = unwrap(attention_out, "attention_out")
    _need(qn.dtype == torch.bfloat16 and qn.dim() == 2 and qn.shape[1] == 512, "query_nope: bfloat16 [t*nq, 512]")
    _need(qr.dtype == torch.bfloat16 and tuple(qr.shape) == (qn.shape[0], 64), "query_rope: bfloat16 [t*nq, 64]")
    _need(int(n_kv) == 1, "n_kv must be 1")
    _need(qn.shape[0] % nq == 0, "query rows must be a multiple of nq")
    t = qn.shape[0] // nq
    _need(ti.dtype == torch.int32 and ti.numel() == t * topk, "topk_indices: int32 [t, n_kv*topk]")
    _need(act.dtype == torch.int32 and act.dim() == 1 and t % act.shape[0] == 0, "kv_act_seqs: int32 [b]")
    b = act.shape[0]
    _need(bt.dtype == torch.int32 and bt.dim() == 2 and bt.shape[0] == b, "block_table: int32 [b, max_blocks]")
    _need(out.dtype == torch.bfloat16 and out.numel() == t * nq * 512, "attention_out: bfloat16 [b, s1, nq, 512]")
    return qn, qr, ti, bt, act, out, t, b


def _sparse_flash_attention_quant(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                  block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk, block_size,
                                  max_blocknum_perbatch, tile_config=None, head_begin=0, nq_total=None):
    qn, qr, ti, bt, act, out, t, b = _sfa_common(query_nope, query_rope, topk_indices, block_table, kv_act_seqs,
                                                 attention_out, nq, n_kv, topk, nq_total, head_begin)
    kn = unwrap(key_nope_2d, "key_nope_2d")
    kr = unwrap(key_rope_2d, "key_rope_2d")
    _need(kn.dtype in (torch.int8, torch.bfloat16) and kn.dim() == 2 and kn.shape[1] == 512,
          "key_nope_2d: int8 (quantized cache) or bfloat16 [block_num*block_size, 512]")
    n_rows = kn.shape[0]
    _need(kr.dtype == torch.bfloat16 and tuple(kr.shape) == (n_rows, 64), "key_rope_2d: bfloat16 [rows, 64]")
    _need(bt.shape[1] >= int(max_blocknum_perbatch), "block_table narrower than max_blocknum_perbatch")
    _need(int(nq) % 16 == 0, "nq must be a multiple of 16")
    lib = _lib.load()
    nbytes = lib.pto_sfa_workspace_bytes(t, int(nq))
    tail = (b, t // b, int(nq), int(n_kv), float(softmax_scale), int(topk), int(block_size), n_rows, bt.shape[1],
            int(nq if nq_total is None else nq_total), int(head_begin))
    if kn.dtype == torch.bfloat16:
        # the reference takes the latent rows as they are when the cache is not int8
        # (sparse_flash_attention_quant_impl.py:149-153, :199-202); the scales are not read
        dev = _same_device([qn, qr, kn, kr, ti, bt, act, out])
        with torch.cuda.device(dev):
            ws = _workspace(dev, nbytes)
            _lib.check(lib.pto_sfa_bf16(qn.data_ptr(), qr.data_ptr(), kn.data_ptr(), kr.data_ptr(), ti.data_ptr(),
                                        bt.data_ptr(), act.data_ptr(), out.data_ptr(), *tail, ws.data_ptr(),
                                        ws.numel(), torch.cuda.current_stream(dev).cuda_stream))
        return None
    sc = unwrap(k_nope_scales, "k_nope_scales")
    _need(sc.dtype == torch.float32 and tuple(sc.shape) == (n_rows, 4), "k_nope_scales: float32 [rows, 4]")
    dev = _same_device([qn, qr, kn, kr, sc, ti, bt, act, out])
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        _lib.check(lib.pto_sfa_quant(qn.data_ptr(), qr.data_ptr(), kn.data_ptr(), kr.data_ptr(), sc.data_ptr(),
                                     ti.data_ptr(), bt.data_ptr(), act.data_ptr(), out.data_ptr(), *tail,
                                     ws.data_ptr(), ws.numel(), torch.cuda.current_stream(dev).cuda_stream))
    return None


def sparse_flash_attention_quant_d(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                   block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk, block_size,
                                   max_blocknum_perbatch, tile_config=None, *, head_begin=0, nq_total=None):
    """Decode entry: attention_out[b, s1, nq, 512] over the selected int8 latent + bf16 rope rows
    (or bf16 latent rows: a bfloat16 `key_nope_2d` selects the non-quantised branch, nq = 128 only).
    Not in the reference's signature: `nq_total`, `head_begin` process heads [head_begin, head_begin + nq) of
    query / output arrays that hold nq_total heads per token (a device's share of a head-sharded prefill chunk
    without slicing copies); the other heads' output rows are not touched."""
    return _sparse_flash_attention_quant(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales,
                                         topk_indices, block_table, kv_act_seqs, attention_out, nq, n_kv,
                                         softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config,
                                         head_begin, nq_total)


def sparse_flash_attention_quant_p(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                   block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk, block_size,
                                   max_blocknum_perbatch, tile_config=None, *, head_begin=0, nq_total=None):
    """Prefill entry: same arithmetic and kernel as the decode entry (the reference differs only
    in compiler options between the two)."""
    return _sparse_flash_attention_quant(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales,
                                         topk_indices, block_table, kv_act_seqs, attention_out, nq, n_kv,
                                         softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config,
                                         head_begin, nq_total)


def _sparse_attention_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                tile_config=None):
    qn, qr, ti, bt, act, out, t, b = _sfa_common(query_nope, query_rope, topk_indices, block_table, kv_act_seqs,
                                                 attention_out, nq, n_kv, topk)
    cache = unwrap(nope_cache, "nope_cache")
    _need(cache.dtype == torch.int8 and cache.dim() == 2 and cache.shape[1] == 656,
          "nope_cache: int8 [rows, 656] = 512 int8 | 64 bf16 | 4 fp32")
    dev = _same_device([qn, qr, cache, ti, bt, act, out])
    lib = _lib.load()
    nbytes = lib.pto_sfa_workspace_bytes(t, int(nq))
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        _lib.check(lib.pto_sfa_packed(qn.data_ptr(), qr.data_ptr(), cache.data_ptr(), ti.data_ptr(), bt.data_ptr(),
                                      act.data_ptr(), out.data_ptr(), b, t // b, int(nq), int(n_kv),
                                      float(softmax_scale), int(topk), int(block_size), cache.shape[0], bt.shape[1],
                                      int(nq), 0, ws.data_ptr(), ws.numel(),
                                      torch.cuda.current_stream(dev).cuda_stream))
    return None


def sparse_attention_antiquant_d(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                 attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                 tile_config=None):
    """Decode entry over the packed 656-byte cache rows."""
    return _sparse_attention_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                       attention_out, nq, n_kv, softmax_scale, topk, block_size,
                                       max_blocknum_perbatch, tile_config)


def sparse_attention_antiquant_p(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                 attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                 tile_config=None):
    """Prefill entry over the packed 656-byte cache rows."""
    return _sparse_attention_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                       attention_out, nq, n_kv, softmax_scale, topk, block_size,
                                       max_blocknum_perbatch, tile_config)


def _cache_out(cache_in, cache_out, name):
    """The reference binds the same tensor as cache input and output (the update is in place); when a caller
    passes two tensors the untouched rows are carried over first."""
    a, o = unwrap(cache_in, name), unwrap(cache_out, name + "_out")
    _need(a.shape == o.shape and a.dtype == o.dtype, f"{name} and {name}_out differ in shape or dtype")
    if a.data_ptr() != o.data_ptr():
        o.copy_(a)
    return o


_PACKED_X_WEIGHTS = {}


def _packed_x_weights(lib, dev, w_dq, w_dkvkr, w_idx_k, w_idx_proj, h, q_lora):
    """The four weights that multiply the token, packed side by side once per set of weight tensors (keyed by
    address and in-place version, so a weight that is overwritten is packed again; an entry keeps its weight
    tensors alive, so an address cannot come back with other contents while the entry exists)."""
    ws = (w_dq, w_dkvkr, w_idx_k, w_idx_proj)
    key = tuple((w.data_ptr(), w._version) for w in ws) + (dev.index,)
    hit = _PACKED_X_WEIGHTS.get(key)
    if hit is None:
        if torch.cuda.is_current_stream_capturing():
            return None  # no allocation inside a capture: the warm-up call before it has filled the cache
        hit = torch.empty((h, q_lora + 768), dtype=torch.bfloat16, device=dev)
        _lib.check(lib.pto_prolog_pack_weights(*[w.data_ptr() for w in ws], h, q_lora, hit.data_ptr(),
                                               torch.cuda.current_stream(dev).cuda_stream))
        if len(_PACKED_X_WEIGHTS) >= 8:
            _PACKED_X_WEIGHTS.pop(next(iter(_PACKED_X_WEIGHTS)))
        _PACKED_X_WEIGHTS[key] = (hit, ws)
        return hit
    return hit[0]


def _mla_indexer_prolog_quant(token_x, mla_w_dq, mla_w_uq_qr, mla_dequant_scale, mla_w_uk, mla_w_dkv_kr, mla_gamma_cq,
                              mla_gamma_ckv, cos, sin, cache_index, mla_kv_cache, mla_kr_cache, mla_k_scale_cache,
                              ip_w_qb_in, ip_w_qb_scale_in, ip_wk_in, ip_w_proj_in, ip_ln_gamma_k_in, ip_ln_beta_k_in,
                              ip_hadamard_q_in, ip_hadamard_k_in, ip_k_cache, ip_k_cache_scale, mla_query_nope_out,
                              mla_query_rope_out, mla_kv_cache_out, mla_kr_cache_out, mla_k_scale_cache_out,
                              ip_q_int8_out, ip_q_scale_out, ip_k_int8_out, ip_k_scale_out, ip_weights_out,
                              mla_epsilon_cq, mla_epsilon_ckv, mla_cache_mode="PA_BSND", mla_tile_config=None,
                              ip_attrs=None, ip_configs=None, rope_cfg=None, *, packed_kv_cache=None):
    bf, i8, f32, f16 = torch.bfloat16, torch.int8, torch.float32, torch.float16
    x = unwrap(token_x, "token_x")
    _need(x.dtype == bf and x.dim() == 2, "token_x: bfloat16 [t, h]")
    t, h = x.shape
    w_dq = unwrap(mla_w_dq, "mla_w_dq")
    _need(w_dq.dtype == bf and w_dq.dim() == 2 and w_dq.shape[0] == h, "mla_w_dq: bfloat16 [h, q_lora_rank]")
    q_lora = w_dq.shape[1]

    def want(x_, name, dtype, numel, what):
        v = unwrap(x_, name)
        _need(v.dtype == dtype and v.numel() == numel, f"{name}: {what}")
        return v

    w_uqqr = want(mla_w_uq_qr, "mla_w_uq_qr", i8, q_lora * 128 * 192, "int8 [q_lora_rank, 128*192]")
    w_qb_scale = want(mla_dequant_scale, "mla_dequant_scale", f32, 128 * 192, "float32 [128*192, 1]")
    w_uk = want(mla_w_uk, "mla_w_uk", bf, 128 * 128 * 512, "bfloat16 [128, 128, 512]")
    w_dkvkr = want(mla_w_dkv_kr, "mla_w_dkv_kr", bf, h * 576, "bfloat16 [h, 576]")
    g_cq = want(mla_gamma_cq, "mla_gamma_cq", bf, q_lora, "bfloat16 [q_lora_rank]")
    g_ckv = want(mla_gamma_ckv, "mla_gamma_ckv", bf, 512, "bfloat16 [512]")
    cos_t = want(cos, "cos", bf, t * 64, "bfloat16 [t, 64]")
    sin_t = want(sin, "sin", bf, t * 64, "bfloat16 [t, 64]")
    ci = want(cache_index, "cache_index", torch.int64, t, "int64 [t]")
    w_idx_qb = want(ip_w_qb_in, "ip_w_qb_in", i8, q_lora * 64 * 128, "int8 [q_lora_rank, 64*128]")
    w_idx_qb_scale = want(ip_w_qb_scale_in, "ip_w_qb_scale_in", f32, 64 * 128, "float32 [64*128, 1]")
    w_idx_k = want(ip_wk_in, "ip_wk_in", bf, h * 128, "bfloat16 [h, 128]")
    w_idx_proj = want(ip_w_proj_in, "ip_w_proj_in", bf, h * 64, "bfloat16 [h, 64]")
    ln_g = want(ip_ln_gamma_k_in, "ip_ln_gamma_k_in", bf, 128, "bfloat16 [128]")
    ln_b = want(ip_ln_beta_k_in, "ip_ln_beta_k_in", bf, 128, "bfloat16 [128]")
    had_q = want(ip_hadamard_q_in, "ip_hadamard_q_in", bf, 128 * 128, "bfloat16 [128, 128]")
    had_k = want(ip_hadamard_k_in, "ip_hadamard_k_in", bf, 128 * 128, "bfloat16 [128, 128]")
    _need(str(mla_cache_mode) == "PA_BSND", "mla_cache_mode: only the paged layout 'PA_BSND'")
    kv = _cache_out(mla_kv_cache, mla_kv_cache_out, "mla_kv_cache")
    kr = _cache_out(mla_kr_cache, mla_kr_cache_out, "mla_kr_cache")
    ks = _cache_out(mla_k_scale_cache, mla_k_scale_cache_out, "mla_k_scale_cache")
    ik = _cache_out(ip_k_cache, ip_k_int8_out, "ip_k_cache")
    iks = _cache_out(ip_k_cache_scale, ip_k_scale_out, "ip_k_cache_scale")
    _need(kv.dtype == i8 and kv.numel() % 512 == 0, "mla_kv_cache: int8 [block_num, block_size, 1, 512]")
    rows = kv.numel() // 512
    _need(kr.dtype == bf and kr.numel() == rows * 64, "mla_kr_cache: bfloat16 [block_num, block_size, 1, 64]")
    _need(ks.dtype == f32 and ks.numel() == rows * 4, "mla_k_scale_cache: float32 [block_num, block_size, 1, 4]")
    _need(ik.dtype == i8 and ik.numel() == rows * 128, "ip_k_cache: int8 [block_num, block_size, 1, 128]")
    _need(iks.dtype == f16 and iks.numel() == rows, "ip_k_cache_scale: float16 [block_num, block_size, 1, 1]")
    q_nope = want(mla_query_nope_out, "mla_query_nope_out", bf, t * 128 * 512, "bfloat16 [t, 128, 512]")
    q_rope = want(mla_query_rope_out, "mla_query_rope_out", bf, t * 128 * 64, "bfloat16 [t, 128, 64]")
    q_i8 = want(ip_q_int8_out, "ip_q_int8_out", i8, t * 64 * 128, "int8 [t, 64, 128]")
    q_sc = want(ip_q_scale_out, "ip_q_scale_out", f16, t * 64, "float16 [t, 64, 1]")
    w_out = want(ip_weights_out, "ip_weights_out", f16, t * 64, "float16 [t, 64]")
    ln_eps = float(getattr(ip_attrs, "eps", 1e-6)) if ip_attrs is not None else 1e-6
    tensors = [x, w_dq, w_uqqr, w_qb_scale, w_uk, w_dkvkr, g_cq, g_ckv, cos_t, sin_t, ci, kv, kr, ks, w_idx_qb,
               w_idx_qb_scale, w_idx_k, w_idx_proj, ln_g, ln_b, had_q, had_k, ik, iks, q_nope, q_rope, q_i8, q_sc,
               w_out]
    pk = None
    if packed_kv_cache is not None:
        pk = unwrap(packed_kv_cache, "packed_kv_cache")
        _need(pk.dtype == i8 and pk.numel() == rows * 656, "packed_kv_cache: int8 [block_num*block_size, 656]")
    dev = _same_device(tensors + ([pk] if pk is not None else []))
    lib = _lib.load()
    nbytes = lib.pto_prolog_workspace_bytes(t, h, q_lora)
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        packed = _packed_x_weights(lib, dev, w_dq, w_dkvkr, w_idx_k, w_idx_proj, h, q_lora)
        _lib.check(lib.pto_mla_indexer_prolog_quant(*[v.data_ptr() for v in tensors],
                                                    packed.data_ptr() if packed is not None else None,
                                                    pk.data_ptr() if pk is not None else None, t, h, q_lora, rows,
                                                    float(mla_epsilon_cq), float(mla_epsilon_ckv), ln_eps,
                                                    ws.data_ptr(), ws.numel(),
                                                    torch.cuda.current_stream(dev).cuda_stream))
    return None


def mla_indexer_prolog_quant_d(*args, **kwargs):
    """Decode entry of the fused MLA + indexer prolog; positional signature of the reference
    (mla_indexer_prolog_quant_impl.py:142-256): 24 inputs, 10 outputs (the five caches are updated in
    place), then mla_epsilon_cq, mla_epsilon_ckv, mla_cache_mode, mla_tile_config, ip_attrs, ip_configs,
    rope_cfg. The tiling objects are accepted and not read; `ip_attrs.eps` is the LayerNorm epsilon.
    Not in the reference: keyword `packed_kv_cache` (int8 [rows, 656]) also receives the token's row in the
    packed layout `sparse_attention_antiquant_d/_p` read."""
    return _mla_indexer_prolog_quant(*args, **kwargs)


def mla_indexer_prolog_quant_p(*args, **kwargs):
    """Prefill entry: the same arithmetic and kernels (the reference differs in scheduling options only,
    mla_indexer_prolog_quant_impl.py:37-139)."""
    return _mla_indexer_prolog_quant(*args, **kwargs)


def pack_kv_cache(key_nope_2d, key_rope_2d, k_nope_scales, nope_cache):
    """Split latent cache -> packed 656-byte rows (int8 latent | bf16 rope | 4 fp32 scales), on the device."""
    kn, kr, sc, out = (unwrap(x, n) for x, n in ((key_nope_2d, "key_nope_2d"), (key_rope_2d, "key_rope_2d"),
                                                 (k_nope_scales, "k_nope_scales"), (nope_cache, "nope_cache")))
    _need(kn.dtype == torch.int8 and kn.numel() % 512 == 0, "key_nope_2d: int8 [rows, 512]")
    rows = kn.numel() // 512
    _need(kr.dtype == torch.bfloat16 and kr.numel() == rows * 64, "key_rope_2d: bfloat16 [rows, 64]")
    _need(sc.dtype == torch.float32 and sc.numel() == rows * 4, "k_nope_scales: float32 [rows, 4]")
    _need(out.dtype == torch.int8 and out.numel() == rows * 656, "nope_cache: int8 [rows, 656]")
    dev = _same_device([kn, kr, sc, out])
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_kv_pack_rows(kn.data_ptr(), kr.data_ptr(), sc.data_ptr(), rows, out.data_ptr(),
                                                torch.cuda.current_stream(dev).cuda_stream))
    return None


def decode_indexer_attention_quant(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, query_nope,
                                   query_rope, key_nope_2d, key_rope_2d, k_nope_scales, act_seq, block_table,
                                   topk_res, attention_out, nq=128, softmax_scale=576 ** -0.5, selected_count=2048, *,
                                   sort=False, fp16_chain=False, histogram=False):
    """Fused chain: indexer score -> top-k -> sparse attention with the kernel's own indices.
    Both caches share `block_table` / `act_seq`. Writes `topk_res` and `attention_out`."""
    dev, (q, qs, kc, ks, w, act, bt), m = _li_args(idx_query, idx_query_scale, idx_key_cache, idx_key_scale,
                                                    idx_weight, act_seq, block_table)
    out_idx = unwrap(topk_res, "topk_res")
    qn, qr, ti, bt2, act2, out, t, b = _sfa_common(query_nope, query_rope, out_idx, bt, act, attention_out, nq, 1,
                                                   selected_count)
    kn = unwrap(key_nope_2d, "key_nope_2d")
    kr = unwrap(key_rope_2d, "key_rope_2d")
    sc = unwrap(k_nope_scales, "k_nope_scales")
    _need(t == m["t"], "indexer and attention query token counts differ")
    _need(m["block_size"] == 128, "block_size must be 128")
    n_rows = m["block_num"] * 128
    _need(kn.dtype == torch.int8 and tuple(kn.shape) == (n_rows, 512), "key_nope_2d: int8 [block_num*128, 512]")
    _need(kr.dtype == torch.bfloat16 and tuple(kr.shape) == (n_rows, 64), "key_rope_2d: bfloat16 [block_num*128, 64]")
    _need(sc.dtype == torch.float32 and tuple(sc.shape) == (n_rows, 4), "k_nope_scales: float32 [block_num*128, 4]")
    dev = _same_device([q, qs, kc, ks, w, act, bt, qn, qr, kn, kr, sc, out_idx, out])
    lib = _lib.load()
    nbytes = lib.pto_decode_workspace_bytes(t, m["max_blocks"], 128, int(nq))
    flags = (0 if sort else _lib.PTO_LI_UNSORTED) | (_lib.PTO_LI_FP16_CHAIN if fp16_chain else 0)
    flags |= _lib.PTO_LI_EPILOGUE_HIST if histogram else 0
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        _lib.check(lib.pto_decode_fused(q.data_ptr(), qs.data_ptr(), kc.data_ptr(), ks.data_ptr(), w.data_ptr(),
                                        m["scale_dtype"], qn.data_ptr(), qr.data_ptr(), kn.data_ptr(), kr.data_ptr(),
                                        sc.data_ptr(), act.data_ptr(), bt.data_ptr(), out_idx.data_ptr(),
                                        out.data_ptr(), b, m["s1"], m["block_num"], m["max_blocks"],
                                        int(selected_count), int(nq), float(softmax_scale), flags, ws.data_ptr(),
                                        ws.numel(), torch.cuda.current_stream(dev).cuda_stream))
    return None


def decode_indexer_attention(idx_query, idx_key_cache, idx_weight, query_nope, query_rope, key_nope_2d, key_rope_2d,
                             act_seq, block_table, topk_res, attention_out, nq=128, softmax_scale=576 ** -0.5,
                             selected_count=2048, *, sort=False):
    """The non-quantised chain behind the two prologs of `DecodeIndexerAttention`
    (framework/src/operator/models/deepseek_v3.2_exp/decode_indexer_attention.cpp:108-129): bf16 indexer -> top-k
    -> sparse attention over the bf16 latent cache with the kernel's own indices. Writes `topk_res` and
    `attention_out`."""
    (q, kc, w, act, bt), m = _li_args_bf16(idx_query, idx_key_cache, idx_weight, act_seq, block_table)
    out_idx = unwrap(topk_res, "topk_res")
    qn, qr, ti, bt2, act2, out, t, b = _sfa_common(query_nope, query_rope, out_idx, bt, act, attention_out, nq, 1,
                                                   selected_count)
    kn = unwrap(key_nope_2d, "key_nope_2d")
    kr = unwrap(key_rope_2d, "key_rope_2d")
    _need(t == m["t"], "indexer and attention query token counts differ")
    _need(int(nq) == 128, "bfloat16 latent cache: all 128 heads of a token")
    n_rows = m["block_num"] * 128
    _need(kn.dtype == torch.bfloat16 and tuple(kn.shape) == (n_rows, 512), "key_nope_2d: bfloat16 [block_num*128, 512]")
    _need(kr.dtype == torch.bfloat16 and tuple(kr.shape) == (n_rows, 64), "key_rope_2d: bfloat16 [block_num*128, 64]")
    dev = _same_device([q, kc, w, act, bt, qn, qr, kn, kr, out_idx, out])
    lib = _lib.load()
    nbytes = lib.pto_decode_workspace_bytes(t, m["max_blocks"], 128, int(nq))
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        _lib.check(lib.pto_decode_fused_bf16(q.data_ptr(), kc.data_ptr(), w.data_ptr(), qn.data_ptr(), qr.data_ptr(),
                                             kn.data_ptr(), kr.data_ptr(), act.data_ptr(), bt.data_ptr(),
                                             out_idx.data_ptr(), out.data_ptr(), b, m["s1"], m["block_num"],
                                             m["max_blocks"], int(selected_count), int(nq), float(softmax_scale),
                                             0 if sort else _lib.PTO_LI_UNSORTED, ws.data_ptr(), ws.numel(),
                                             torch.cuda.current_stream(dev).cuda_stream))
    return None


def mla_indexer_prolog(token_x, w_dq, w_uq_qr, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index, kv_cache,
                       kr_cache, idx_w_qb, idx_wk, idx_w_proj, idx_ln_gamma, idx_ln_beta, idx_k_cache, query_nope_out,
                       query_rope_out, idx_query_out, idx_weights_out, epsilon_cq=1e-5, epsilon_ckv=1e-5,
                       cache_mode="PA_BSND", *, ln_eps=1e-6, q_norm_out=None):
    """The two prologs in front of the non-quantised chain, in one call: `MlaPrologComputeV32` without quantisation
    (framework/src/operator/models/deepseek_v3.2_exp/dynamic_mla_v32.cpp:187-345) and
    `LightningIndexerPrologCompute` on its normalised query (.../lightning_indexer_prolog.cpp:129-227), as
    `DecodeIndexerAttention` runs them (.../decode_indexer_attention.cpp:85-106).

    token_x bf16 [t, h]; w_dq [h, q_lora]; w_uq_qr [q_lora, 128*192]; w_uk [128, 128, 512]; w_dkv_kr [h, 576];
    cos, sin [t, 64]; cache_index int64 [t]; idx_w_qb [q_lora, 64*128]; idx_wk [h, 128]; idx_w_proj [h, 64];
    LayerNorm gamma / beta [128]. Updated in place at row cache_index[i]: kv_cache bf16 [.., 512], kr_cache bf16
    [.., 64], idx_k_cache bf16 [.., 128]. Written: query_nope_out [t, 128, 512], query_rope_out [t, 128, 64],
    idx_query_out [t, 64, 128], idx_weights_out [t, 64] (all bf16), and `q_norm_out` [t, q_lora] (the reference's
    `rmsRes`) when given."""
    bf = torch.bfloat16
    x = unwrap(token_x, "token_x")
    _need(x.dtype == bf and x.dim() == 2, "token_x: bfloat16 [t, h]")
    t, h = x.shape
    wdq = unwrap(w_dq, "w_dq")
    _need(wdq.dtype == bf and wdq.dim() == 2 and wdq.shape[0] == h, "w_dq: bfloat16 [h, q_lora_rank]")
    q_lora = wdq.shape[1]

    def want(x_, name, numel, what, dtype=bf):
        v = unwrap(x_, name)
        _need(v.dtype == dtype and v.numel() == numel and v.is_contiguous(), f"{name}: {what}")
        return v

    w_uqqr = want(w_uq_qr, "w_uq_qr", q_lora * 128 * 192, "bfloat16 [q_lora_rank, 128*192]")
    wuk = want(w_uk, "w_uk", 128 * 128 * 512, "bfloat16 [128, 128, 512]")
    w_dkvkr = want(w_dkv_kr, "w_dkv_kr", h * 576, "bfloat16 [h, 576]")
    g_cq = want(gamma_cq, "gamma_cq", q_lora, "bfloat16 [q_lora_rank]")
    g_ckv = want(gamma_ckv, "gamma_ckv", 512, "bfloat16 [512]")
    cos_t = want(cos, "cos", t * 64, "bfloat16 [t, 64]")
    sin_t = want(sin, "sin", t * 64, "bfloat16 [t, 64]")
    ci = want(cache_index, "cache_index", t, "int64 [t]", torch.int64)
    w_qb = want(idx_w_qb, "idx_w_qb", q_lora * 64 * 128, "bfloat16 [q_lora_rank, 64*128]")
    w_k = want(idx_wk, "idx_wk", h * 128, "bfloat16 [h, 128]")
    w_proj = want(idx_w_proj, "idx_w_proj", h * 64, "bfloat16 [h, 64]")
    ln_g = want(idx_ln_gamma, "idx_ln_gamma", 128, "bfloat16 [128]")
    ln_b = want(idx_ln_beta, "idx_ln_beta", 128, "bfloat16 [128]")
    _need(str(cache_mode) == "PA_BSND", "cache_mode: only the paged layout 'PA_BSND'")
    kv = unwrap(kv_cache, "kv_cache")
    _need(kv.dtype == bf and kv.numel() % 512 == 0 and kv.is_contiguous(), "kv_cache: bfloat16 [block_num, block_size, 1, 512]")
    rows = kv.numel() // 512
    kr = want(kr_cache, "kr_cache", rows * 64, "bfloat16 [block_num, block_size, 1, 64]")
    ik = want(idx_k_cache, "idx_k_cache", rows * 128, "bfloat16 [block_num, block_size, 1, 128]")
    q_nope = want(query_nope_out, "query_nope_out", t * 128 * 512, "bfloat16 [t, 128, 512]")
    q_rope = want(query_rope_out, "query_rope_out", t * 128 * 64, "bfloat16 [t, 128, 64]")
    iq = want(idx_query_out, "idx_query_out", t * 64 * 128, "bfloat16 [t, 64, 128]")
    w_out = want(idx_weights_out, "idx_weights_out", t * 64, "bfloat16 [t, 64]")
    tensors = [x, wdq, w_uqqr, wuk, w_dkvkr, g_cq, g_ckv, cos_t, sin_t, ci, kv, kr, w_qb, w_k, w_proj, ln_g, ln_b, ik,
               q_nope, q_rope, iq, w_out]
    qn = None
    if q_norm_out is not None:
        qn = want(q_norm_out, "q_norm_out", t * q_lora, "bfloat16 [t, q_lora_rank]")
    dev = _same_device(tensors + ([qn] if qn is not None else []))
    lib = _lib.load()
    nbytes = lib.pto_prolog_nonquant_workspace_bytes(t, h, q_lora)
    with torch.cuda.device(dev):
        ws = _workspace(dev, nbytes)
        packed = _packed_x_weights(lib, dev, wdq, w_dkvkr, w_k, w_proj, h, q_lora)
        _lib.check(lib.pto_mla_indexer_prolog(*[v.data_ptr() for v in tensors],
                                              qn.data_ptr() if qn is not None else None,
                                              packed.data_ptr() if packed is not None else None, t, h, q_lora, rows,
                                              float(epsilon_cq), float(epsilon_ckv), float(ln_eps), ws.data_ptr(),
                                              ws.numel(), torch.cuda.current_stream(dev).cuda_stream))
    return None


def decode_indexer_attention_layer(x, w_dq, w_uq_qr, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, sin, cos, cache_index,
                                   kv_cache, kr_cache, block_table, act_seqs, q_w, k_w, proj_w, ln_w, ln_bias,
                                   index_k_cache, attention_out, *, topk_res=None, scratch=None, eps=1e-5,
                                   softmax_scale=576 ** -0.5, selected_count=2048, sort=False):
    """`DecodeIndexerAttention` whole, inputs in the reference's order
    (framework/src/operator/models/deepseek_v3.2_exp/decode_indexer_attention.cpp:22-131; note sin before cos):
    the two prologs (`mla_indexer_prolog`), then indexer -> top-k -> sparse attention over the caches they have just
    updated (`decode_indexer_attention`). x is [b, s1, h] or [t, h]; `act_seqs` int32 [b].

    `scratch`: dict with bf16 tensors query_nope [t,128,512], query_rope [t,128,64], idx_query [t,64,128],
    idx_weights [t,64] and int32 topk_res [t,1,selected_count]; allocated when absent (pass it to record the call
    into a CUDA graph). Returns the scratch dict (the selected positions are in scratch["topk_res"])."""
    xt = unwrap(x, "x")
    x2 = xt.reshape(-1, xt.shape[-1])
    t = x2.shape[0]
    dev = x2.device
    if scratch is None:
        bf = torch.bfloat16
        scratch = dict(query_nope=torch.empty((t, 128, 512), dtype=bf, device=dev),
                       query_rope=torch.empty((t, 128, 64), dtype=bf, device=dev),
                       idx_query=torch.empty((t, 64, 128), dtype=bf, device=dev),
                       idx_weights=torch.empty((t, 64), dtype=bf, device=dev),
                       topk_res=torch.empty((t, 1, int(selected_count)), dtype=torch.int32, device=dev))
    if topk_res is not None:
        scratch["topk_res"] = unwrap(topk_res, "topk_res")
    kv = unwrap(kv_cache, "kv_cache")
    kr = unwrap(kr_cache, "kr_cache")
    ik = unwrap(index_k_cache, "index_k_cache")
    mla_indexer_prolog(x2, w_dq, w_uq_qr, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, unwrap(cos, "cos").reshape(t, -1),
                       unwrap(sin, "sin").reshape(t, -1), unwrap(cache_index, "cache_index").reshape(-1), kv, kr, q_w,
                       k_w, proj_w, ln_w, ln_bias, ik, scratch["query_nope"], scratch["query_rope"],
                       scratch["idx_query"], scratch["idx_weights"], eps, eps)
    decode_indexer_attention(scratch["idx_query"], ik.reshape(-1, 128, 1, 128), scratch["idx_weights"],
                             scratch["query_nope"].reshape(t * 128, 512), scratch["query_rope"].reshape(t * 128, 64),
                             kv.reshape(-1, 512), kr.reshape(-1, 64), act_seqs, block_table, scratch["topk_res"],
                             attention_out, 128, softmax_scale, selected_count, sort=sort)
    return scratch
