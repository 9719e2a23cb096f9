"""The fused decode step recorded into a CUDA graph and replayed: same results as eager calls, new results
after the static inputs are refreshed in place, no device allocation inside the capture."""
import pytest
import torch

import pypto_b200 as pto
from pypto_b200 import inputs as gen

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args(g, idx, out):
    return (g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight, g.query_nope, g.query_rope,
            g.key_nope_2d, g.key_rope_2d, g.k_nope_scales, g.act_seq_key, g.block_table, idx, out)


def test_captured_step_replays_and_tracks_input_updates():
    d = gen.make_inputs([5000, 3000, 9000, 2048, 70], s1=1, seed=21)
    g = d.to(DEV)
    idx_e = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    out_e = torch.zeros((d.b, d.s1, 128, 512), dtype=torch.bfloat16, device=DEV)
    pto.decode_indexer_attention_quant(*_args(g, idx_e, out_e), sort=True)
    torch.cuda.synchronize()

    idx_g = torch.zeros_like(idx_e)
    out_g = torch.zeros_like(out_e)
    before = torch.cuda.memory_allocated()
    step = pto.CapturedCall(pto.decode_indexer_attention_quant, *_args(g, idx_g, out_g), sort=True)
    idx_g.fill_(-7)
    out_g.fill_(3.0)
    step.replay()
    torch.cuda.synchronize()
    assert step.workspace_status()[0] == 0
    assert torch.equal(idx_g, idx_e) and torch.equal(out_g, out_e)
    # the capture added one workspace for its stream at most, nothing per replay
    after_first = torch.cuda.memory_allocated()
    for _ in range(3):
        step.replay()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == after_first
    assert after_first - before <= 64 << 20

    # refresh the static inputs in place: another batch of queries and shorter sequences
    d2 = gen.make_inputs([5000, 3000, 9000, 2048, 70], s1=1, seed=22)
    g.idx_query.copy_(d2.idx_query.to(DEV))
    g.query_nope.copy_(d2.query_nope.to(DEV))
    g.query_rope.copy_(d2.query_rope.to(DEV))
    g.act_seq_key.copy_(torch.tensor([4000, 3000, 1, 2047, 0], dtype=torch.int32))
    step.replay()
    pto.decode_indexer_attention_quant(*_args(g, idx_e, out_e), sort=True)
    torch.cuda.synchronize()
    assert torch.equal(idx_g, idx_e) and torch.equal(out_g, out_e)
    assert torch.all(out_g[4] == 0) and torch.all(idx_g[4] == -1)


def test_captured_prolog_then_decode_layer():
    """The prolog (eight kernels on two streams) and the decode chain behind it in ONE
    graph: a replay reproduces the eager sequence bit for bit, tracks a new token batch written into the static
    input, and allocates nothing."""
    act = [3000, 700, 4500, 129]
    p = gen.make_prolog_inputs(act, s1=1, seed=55, device=DEV)
    t, rows = len(act), p["kv_cache"].shape[0]
    caches0 = {k: p[k].clone() for k in ("kv_cache", "kr_cache", "kv_scale_cache", "idx_k_cache", "idx_k_scale_cache")}
    names = ["token_x", "w_dq", "w_uqqr", "w_qb_scale", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin",
             "cache_index", "kv_cache", "kr_cache", "kv_scale_cache", "w_idx_qb", "w_idx_qb_scale", "w_idx_k",
             "w_idx_proj", "ln_gamma", "ln_beta", "hadamard_q", "hadamard_k", "idx_k_cache", "idx_k_scale_cache"]
    q_nope = torch.zeros(t, 128, 512, dtype=torch.bfloat16, device=DEV)
    q_rope = torch.zeros(t, 128, 64, dtype=torch.bfloat16, device=DEV)
    q_i8 = torch.zeros(t, 64, 128, dtype=torch.int8, device=DEV)
    q_sc = torch.zeros(t, 64, 1, dtype=torch.float16, device=DEV)
    w = torch.zeros(t, 64, dtype=torch.float16, device=DEV)
    topk = torch.zeros(t, 1, 2048, dtype=torch.int32, device=DEV)
    out = torch.zeros(t, 1, 128, 512, dtype=torch.bfloat16, device=DEV)
    act_t = torch.tensor(act, dtype=torch.int32, device=DEV)

    def layer(_anchor):
        pto.mla_indexer_prolog_quant_d(*[p[n] for n in names], q_nope, q_rope, p["kv_cache"], p["kr_cache"],
                                       p["kv_scale_cache"], q_i8, q_sc, p["idx_k_cache"], p["idx_k_scale_cache"], w,
                                       1e-5, 1e-5, "PA_BSND", None, None, None, None)
        pto.decode_indexer_attention_quant(q_i8, q_sc.reshape(t, 64), p["idx_k_cache"].reshape(rows // 128, 128, 1, 128),
                                           p["idx_k_scale_cache"].reshape(rows // 128, 128, 1), w,
                                           q_nope.reshape(t * 128, 512), q_rope.reshape(t * 128, 64), p["kv_cache"],
                                           p["kr_cache"], p["kv_scale_cache"], act_t, p["block_table"], topk, out,
                                           sort=True)

    def reset_caches():
        for k, v in caches0.items():
            p[k].copy_(v)

    layer(out)
    torch.cuda.synchronize()
    want = [x.clone() for x in (q_nope, q_rope, q_i8, q_sc, w, topk, out, p["kv_cache"], p["idx_k_cache"])]
    reset_caches()
    step = pto.CapturedCall(layer, out)  # (its warm-up call and the capture leave the same cache contents)
    for x in (q_nope, q_rope, q_i8, q_sc, w, topk, out):
        x.fill_(1)
    reset_caches()
    base = torch.cuda.memory_allocated()
    step.replay()
    torch.cuda.synchronize()
    assert step.workspace_status()[0] == 0
    got = (q_nope, q_rope, q_i8, q_sc, w, topk, out, p["kv_cache"], p["idx_k_cache"])
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    # a new batch of hidden states in the static input: the replay follows it
    p["token_x"].copy_(torch.roll(p["token_x"], 1, dims=0))
    reset_caches()
    step.replay()
    torch.cuda.synchronize()
    assert not torch.equal(q_nope, want[0])
    assert torch.cuda.memory_allocated() == base
