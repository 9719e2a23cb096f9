"""MLA + lightning-indexer prolog oracle (CPU, torch). TEST INFRASTRUCTURE ONLY.

Restates the reference's torch goldens of the fused prolog operator
(examples/models/deepseek_v32_exp/deepseekv32_mla_indexer_prolog_quant.py):

  mla_prolog        `mla_prolog_quant_v32_compute`  :409-541, with is_quant_a = False, is_quant_b = True,
                    no smoothing (the configuration the example runs, :645)
  indexer_prolog    `indexer_prolog`                :544-614
  helpers           `quant` :35-53, `rms_norm` :56-73, `apply_rotary_pos_emb_v2` :106-131,
                    `single_rope` :140-152, `layer_norm` :155-162, scatter :76-103

Every intermediate rounding of the goldens is kept: projections are rounded to bf16 where the golden
casts, the int8 quantisation is round-half-even of x*127/max followed by the fp16 -> trunc chain, and
the dequantisation scale is 1/(127/max) in fp32. `eps` arguments default to 0, which is the golden's
arithmetic (its RMSNorm has no epsilon); the operator passes the caller's value.

The two prologs in front of the non-quantised chain (`DecodeIndexerAttention`,
framework/src/operator/models/deepseek_v3.2_exp/decode_indexer_attention.cpp:85-106) follow the system
tests' goldens:

  mla_prolog_nonquant      `mla_prolog_compute` with is_quant_a = is_quant_b = False
                           (framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_mla_prolog_golden_v32.py:176-303)
  indexer_prolog_nonquant  `indexer_prolog` (.../gen_lightning_indexer_prolog.py:253-293)
  chained as `mla_prolog_golden` + `gen_deepseek_dsa_golden` chain them (.../gen_decode_indexer_attention.py:195-262):
  the normalised query (`q_a_layernorm`) is the indexer prolog's `qr`.
"""
from __future__ import annotations

import torch


def quant_rows(x: torch.Tensor):
    """Per-row symmetric int8 quantisation over the last axis (:35-53): (int8, fp32 dequant scale)."""
    xf = x.to(torch.float32)
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale_q = 127.0 / amax
    q = torch.round(xf * scale_q).to(torch.int32).to(torch.float16)
    return torch.trunc(q).to(torch.int8), 1.0 / scale_q


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 0.0):
    """x / sqrt(sum(x*x / n) + eps) * gamma in fp32, back to x's dtype (:56-73)."""
    xf = x.to(torch.float32)
    ms = (xf * xf * (1.0 / x.shape[-1])).sum(dim=-1, keepdim=True)
    if eps:
        ms = ms + eps
    return (xf / torch.sqrt(ms) * gamma).to(x.dtype)


def _rotate_half(x):
    a, b = x.chunk(2, dim=-1)
    return torch.cat((-b, a), dim=-1)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """MLA rope (:106-131): even dims first, odd dims second, then x*cos + rotate_half(x)*sin.
    x [t, n, d] bf16, cos/sin [t, d]."""
    t, n, d = x.shape
    xf = x.to(torch.float32).reshape(t, n, d // 2, 2).permute(0, 1, 3, 2).reshape(t, n, d)
    c = cos.to(torch.float32).unsqueeze(1)
    s = sin.to(torch.float32).unsqueeze(1)
    return (xf * c + _rotate_half(xf) * s).to(x.dtype)


def rope_halves(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Indexer rope (:140-152): no de-interleave. x [t, n, d], cos/sin [t, d]."""
    xf = x.to(torch.float32)
    c = cos.to(torch.float32).unsqueeze(1)
    s = sin.to(torch.float32).unsqueeze(1)
    return (xf * c + _rotate_half(xf) * s).to(x.dtype)


def layer_norm(x: torch.Tensor, gamma, beta, eps: float = 1e-6):
    """(:155-162) fp32 statistics, biased variance."""
    xf = x.to(torch.float32)
    mean = xf.mean(dim=-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(dim=-1, keepdim=True)
    y = (xf - mean) / torch.sqrt(var + eps)
    return (y * gamma.to(torch.float32) + beta.to(torch.float32)).to(x.dtype)


def mla_prolog(x, w_dq, w_uqqr, w_qb_scale, w_uk, w_dkvkr, gamma_cq, gamma_ckv, cos, sin, cache_index, kv_cache,
               kr_cache, kv_scale_cache, eps_cq: float = 0.0, eps_ckv: float = 0.0):
    """x [t, h] bf16 ... -> dict of outputs; caches are returned as updated copies.

    w_dq [h, q_lora] bf16, w_uqqr [q_lora, n*(128+64)] int8 with per-column scale w_qb_scale [n*192],
    w_uk [n, 128, 512] bf16, w_dkvkr [h, 512+64] bf16, cos/sin [t, 64] bf16, cache_index [t] int64,
    kv_cache int8 [rows, 512], kr_cache bf16 [rows, 64], kv_scale_cache fp32 [rows, 4]."""
    t = x.shape[0]
    n, d_nope, lora = w_uk.shape
    d_rope = cos.shape[-1]
    xf = x.to(torch.float32)
    # query: down-projection, RMSNorm, per-token int8, up-projection in int32, two-step dequantisation (:432-479)
    q_a = (xf @ w_dq.to(torch.float32)).to(x.dtype)
    q_norm = rms_norm(q_a, gamma_cq, eps_cq)
    q_norm_i8, q_norm_scale = quant_rows(q_norm)  # [t, q_lora], [t, 1]
    q_b = (q_norm_i8.to(torch.int32) @ w_uqqr.to(torch.int32)).to(torch.float32)
    q_b = (q_b * q_norm_scale * w_qb_scale.reshape(1, -1)).to(x.dtype).reshape(t, n, d_nope + d_rope)
    # absorbed nope part: per head [t, 128] @ [128, 512] (:487-494)
    q_nope = torch.matmul(q_b[:, :, :d_nope].permute(1, 0, 2).to(torch.float32), w_uk.to(torch.float32))
    q_nope = q_nope.to(x.dtype).permute(1, 0, 2).contiguous()  # [t, n, 512]
    # key/value: down-projection, RMSNorm of the latent part, int8 per 128-wide tile (:496-520)
    kv_a = (xf @ w_dkvkr.to(torch.float32)).to(x.dtype)
    latent = rms_norm(kv_a[:, :lora], gamma_ckv, eps_ckv)
    latent_i8, latent_scale = quant_rows(latent.reshape(t, 4, lora // 4))
    latent_i8 = latent_i8.reshape(t, lora)
    latent_scale = latent_scale.reshape(t, 4)
    # rope on the query's and the key's rope parts (:522-530)
    q_rope = rope_interleaved(q_b[:, :, d_nope:], cos, sin)
    k_rope = rope_interleaved(kv_a[:, lora:].reshape(t, 1, d_rope), cos, sin).reshape(t, d_rope)
    # scatter into the paged caches (:532-548)
    kv_out, kr_out, sc_out = kv_cache.clone(), kr_cache.clone(), kv_scale_cache.clone()
    idx = cache_index.reshape(-1).long()
    for i in range(t):  # in order: a repeated index keeps the last token, as the golden's loop does
        kv_out[idx[i]] = latent_i8[i]
        kr_out[idx[i]] = k_rope[i]
        sc_out[idx[i]] = latent_scale[i]
    return dict(q_nope=q_nope, q_rope=q_rope, q_norm=q_norm_i8, q_norm_scale=q_norm_scale, kv_cache=kv_out,
                kr_cache=kr_out, kv_scale_cache=sc_out)


def indexer_prolog(x, q_norm, q_norm_scale, w_idx_qb, w_idx_qb_scale, w_idx_k, w_idx_proj, ln_gamma, ln_beta, cos,
                   sin, hadamard_q, hadamard_k, idx_k_cache, idx_k_scale_cache, cache_index, ln_eps: float = 1e-6):
    """(:544-614) x [t, h] bf16, q_norm int8 [t, q_lora] + fp32 scale [t, 1], w_idx_qb int8 [q_lora, 64*128]
    with per-column scale, w_idx_k bf16 [h, 128], w_idx_proj bf16 [h, 64], hadamard bf16 [128, 128],
    idx_k_cache int8 [rows, 128], idx_k_scale_cache fp16 [rows, 1]."""
    t = x.shape[0]
    d = hadamard_q.shape[0]
    n = w_idx_qb.shape[1] // d
    rope = cos.shape[-1]
    xf = x.to(torch.float32)
    q = (q_norm.to(torch.int32) @ w_idx_qb.to(torch.int32)).to(torch.float32)
    q = (q * q_norm_scale * w_idx_qb_scale.reshape(1, -1)).reshape(t, n, d).to(torch.bfloat16)
    q = torch.cat([rope_halves(q[..., :rope], cos, sin), q[..., rope:]], dim=-1)
    q = (q.to(torch.float32) @ hadamard_q.to(torch.float32)).to(x.dtype)
    q_i8, q_scale = quant_rows(q)
    k = layer_norm(xf @ w_idx_k.to(torch.float32), ln_gamma, ln_beta, ln_eps).to(x.dtype)
    k = torch.cat([rope_halves(k[:, None, :rope], cos, sin)[:, 0], k[:, rope:]], dim=-1)
    k = (k.to(torch.float32) @ hadamard_k.to(torch.float32)).to(x.dtype)
    k_i8, k_scale = quant_rows(k)
    kc, ks = idx_k_cache.clone(), idx_k_scale_cache.clone()
    idx = cache_index.reshape(-1).long()
    for i in range(t):
        kc[idx[i]] = k_i8[i]
        ks[idx[i]] = k_scale[i].to(torch.float16)
    w = (xf @ w_idx_proj.to(torch.float32)).to(x.dtype).to(torch.float32)
    w = (w * (n ** -0.5) * (d ** -0.5)).to(torch.float16)
    return dict(q_int8=q_i8, q_scale=q_scale.to(torch.float16), idx_k_cache=kc, idx_k_scale_cache=ks, weights=w)


def mla_indexer_prolog(p: dict, eps_cq: float = 0.0, eps_ckv: float = 0.0, ln_eps: float = 1e-6) -> dict:
    """The fused operator's arithmetic (mla_indexer_prolog_quant_impl.py:37-256: the MLA prolog, then the
    indexer prolog on its q_norm / q_norm_scale) over a dict of inputs named as `make_prolog_inputs` names them."""
    m = mla_prolog(p["token_x"], p["w_dq"], p["w_uqqr"], p["w_qb_scale"], p["w_uk"], p["w_dkvkr"], p["gamma_cq"],
                   p["gamma_ckv"], p["cos"], p["sin"], p["cache_index"], p["kv_cache"], p["kr_cache"],
                   p["kv_scale_cache"], eps_cq, eps_ckv)
    i = indexer_prolog(p["token_x"], m["q_norm"], m["q_norm_scale"], p["w_idx_qb"], p["w_idx_qb_scale"], p["w_idx_k"],
                       p["w_idx_proj"], p["ln_gamma"], p["ln_beta"], p["cos"], p["sin"], p["hadamard_q"],
                       p["hadamard_k"], p["idx_k_cache"], p["idx_k_scale_cache"], p["cache_index"], ln_eps)
    m.update(i)
    return m


def mla_prolog_nonquant(x, w_dq, w_uqqr, w_uk, w_dkvkr, gamma_cq, gamma_ckv, cos, sin, cache_index, kv_cache, kr_cache,
                        eps_cq: float = 0.0, eps_ckv: float = 0.0):
    """`mla_prolog_compute` without quantisation (gen_mla_prolog_golden_v32.py:176-303): every product is an fp32
    matmul rounded to bf16, both caches are bf16. w_uqqr bf16 [q_lora, n*192], kv_cache bf16 [rows, 512],
    kr_cache bf16 [rows, 64]; the rest as `mla_prolog`."""
    t = x.shape[0]
    n, d_nope, lora = w_uk.shape
    d_rope = cos.shape[-1]
    xf = x.to(torch.float32)
    q_a = (xf @ w_dq.to(torch.float32)).to(x.dtype)
    q_norm = rms_norm(q_a, gamma_cq, eps_cq)  # bf16 [t, q_lora]: also the indexer prolog's `qr`
    q_b = (q_norm.to(torch.float32) @ w_uqqr.to(torch.float32)).to(x.dtype).reshape(t, n, d_nope + d_rope)
    q_nope = torch.matmul(q_b[:, :, :d_nope].permute(1, 0, 2).to(torch.float32), w_uk.to(torch.float32))
    q_nope = q_nope.to(x.dtype).permute(1, 0, 2).contiguous()
    kv_a = (xf @ w_dkvkr.to(torch.float32)).to(x.dtype)
    latent = rms_norm(kv_a[:, :lora], gamma_ckv, eps_ckv)
    q_rope = rope_interleaved(q_b[:, :, d_nope:], cos, sin)
    k_rope = rope_interleaved(kv_a[:, lora:].reshape(t, 1, d_rope), cos, sin).reshape(t, d_rope)
    kv_out, kr_out = kv_cache.clone(), kr_cache.clone()
    idx = cache_index.reshape(-1).long()
    for i in range(t):
        kv_out[idx[i]] = latent[i]
        kr_out[idx[i]] = k_rope[i]
    return dict(q_nope=q_nope, q_rope=q_rope, q_norm=q_norm, kv_cache=kv_out, kr_cache=kr_out)


def indexer_prolog_nonquant(x, qr, w_idx_qb, w_idx_k, w_idx_proj, ln_gamma, ln_beta, cos, sin, idx_k_cache, cache_index,
                            ln_eps: float = 1e-6):
    """`indexer_prolog` of the non-quantised indexer (gen_lightning_indexer_prolog.py:253-293): query = bf16(qr @ wq_b)
    with the de-interleaving rope on the first 64 dims of every head; key = bf16(LayerNorm(fp32(x @ wk))) with the
    same rope, scattered into the bf16 key cache; weights = bf16(x @ weights_proj), unscaled. w_idx_qb bf16
    [q_lora, 64*128], idx_k_cache bf16 [rows, 128]."""
    t = x.shape[0]
    d = w_idx_k.shape[1]
    n = w_idx_qb.shape[1] // d
    rope = cos.shape[-1]
    xf = x.to(torch.float32)
    q = (qr.to(torch.float32) @ w_idx_qb.to(torch.float32)).to(qr.dtype).reshape(t, n, d)
    q = torch.cat([rope_interleaved(q[..., :rope], cos, sin), q[..., rope:]], dim=-1)
    k = layer_norm(xf @ w_idx_k.to(torch.float32), ln_gamma, ln_beta, ln_eps).to(x.dtype)
    k = torch.cat([rope_interleaved(k[:, None, :rope], cos, sin)[:, 0], k[:, rope:]], dim=-1)
    kc = idx_k_cache.clone()
    idx = cache_index.reshape(-1).long()
    for i in range(t):
        kc[idx[i]] = k[i]
    w = (xf @ w_idx_proj.to(torch.float32)).to(x.dtype)
    return dict(idx_query=q, idx_k_cache=kc, weights=w)


def mla_indexer_prolog_nonquant(p: dict, eps_cq: float = 0.0, eps_ckv: float = 0.0, ln_eps: float = 1e-6) -> dict:
    """Both prologs of the non-quantised chain over a dict named as `make_prolog_nonquant_inputs` names it."""
    m = mla_prolog_nonquant(p["token_x"], p["w_dq"], p["w_uqqr"], p["w_uk"], p["w_dkvkr"], p["gamma_cq"], p["gamma_ckv"],
                            p["cos"], p["sin"], p["cache_index"], p["kv_cache"], p["kr_cache"], eps_cq, eps_ckv)
    i = indexer_prolog_nonquant(p["token_x"], m["q_norm"], p["w_idx_qb"], p["w_idx_k"], p["w_idx_proj"], p["ln_gamma"],
                                p["ln_beta"], p["cos"], p["sin"], p["idx_k_cache"], p["cache_index"], ln_eps)
    m.update(i)
    return m
