"""The two prologs in front of the non-quantised chain on the GPU, against the reference-made fixtures
(`mla_prolog_compute` without quantisation and the non-quantised `indexer_prolog` of the reference's system tests)
and the CPU oracle; then the whole `DecodeIndexerAttention` layer: prologs -> bf16 indexer -> top-k -> attention over
the caches the prologs have just updated.

Tolerances. Every output is a bf16 rounding of an fp32 sum of bf16 products that the tensor core adds in an order of
its own, so an element equals the golden's or lies one bf16 step from it (2^-8 relative) when the sum falls near a
rounding boundary; errors of one stage are carried through the next product. The reference's own system tests accept
0.003 relative per element (test_lightning_indexer_prolog.cpp:174-179, test_decode_indexer_attention.cpp:223-227); the
bound here is the quantised prolog's (an element fails when |got - want| > atol + rtol*|want| with atol 0.005 and
rtol 1/128, at most 0.5 % may fail), and in addition rel-L2 <= 3e-3 per tensor."""
import pytest
import torch

import oracle
import pypto_b200 as pto
from oracle import prolog_oracle as po
from pypto_b200 import inputs as gen
from golden_util import PROLOG_HEADS, PROLOG_NONQUANT_CASES, from_np_bf16, load_prolog_nonquant_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(got, want, name, atol=0.005, rtol=0.0078125, ratio=0.005, rel_l2=3e-3):
    got, want = got.detach().cpu().to(torch.float64), want.detach().cpu().to(torch.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert torch.isfinite(got).all(), name
    bad = int(((got - want).abs() > atol + rtol * want.abs()).sum())
    assert bad <= round(ratio * want.numel()), (name, bad, want.numel(), float((got - want).abs().max()))
    err = float((got - want).norm() / want.norm().clamp_min(1e-30))
    assert err <= rel_l2, (name, err)


def run_prolog(p, eps_cq=1e-5, eps_ckv=1e-5, with_q_norm=True):
    g = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
    t = g["token_x"].shape[0]
    bf = torch.bfloat16
    out = dict(q_nope=torch.zeros(t, 128, 512, dtype=bf, device=DEV), q_rope=torch.zeros(t, 128, 64, dtype=bf, device=DEV),
               idx_query=torch.zeros(t, 64, 128, dtype=bf, device=DEV), weights=torch.zeros(t, 64, dtype=bf, device=DEV))
    if with_q_norm:
        out["q_norm"] = torch.zeros(t, 1536, dtype=bf, device=DEV)
    pto.mla_indexer_prolog(g["token_x"], g["w_dq"], g["w_uqqr"], g["w_uk"], g["w_dkvkr"], g["gamma_cq"], g["gamma_ckv"],
                           g["cos"], g["sin"], g["cache_index"], g["kv_cache"], g["kr_cache"], g["w_idx_qb"],
                           g["w_idx_k"], g["w_idx_proj"], g["ln_gamma"], g["ln_beta"], g["idx_k_cache"], out["q_nope"],
                           out["q_rope"], out["idx_query"], out["weights"], eps_cq, eps_ckv,
                           q_norm_out=out.get("q_norm"))
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    for k in ("kv_cache", "kr_cache", "idx_k_cache"):
        out[k] = g[k]
    return {k: v.cpu() for k, v in out.items()}, g


def check_untouched(o, p):
    idx = p["cache_index"]
    keep = torch.ones(p["kv_cache"].shape[0], dtype=torch.bool)
    keep[idx] = False
    for key in ("kv_cache", "kr_cache", "idx_k_cache"):
        assert torch.equal(o[key][keep], p[key][keep]), key


@pytest.mark.parametrize("name", PROLOG_NONQUANT_CASES)
def test_matches_reference_fixture(name):
    p, z = load_prolog_nonquant_case(name)
    o, _ = run_prolog(p, eps_cq=0.0, eps_ckv=0.0)  # the goldens' RMSNorm is called with epsilon 0 by the fixture maker
    idx = p["cache_index"]
    close(o["q_norm"], from_np_bf16(z["q_norm"]), "q_norm")
    close(o["q_nope"][:, list(PROLOG_HEADS)], from_np_bf16(z["q_nope_heads"]), "q_nope")
    close(o["q_rope"], from_np_bf16(z["q_rope"]), "q_rope")
    close(o["kv_cache"][idx], from_np_bf16(z["kv_rows"]), "kv rows")
    close(o["kr_cache"][idx], from_np_bf16(z["kr_rows"]), "kr rows")
    close(o["idx_query"], from_np_bf16(z["idx_query"]), "idx_query")
    close(o["idx_k_cache"][idx], from_np_bf16(z["idx_k_rows"]), "idx k rows")
    close(o["weights"], from_np_bf16(z["weights"]), "weights")
    check_untouched(o, p)


@pytest.mark.parametrize("act_seq,s1", [([4096] * 64, 1), ([700, 129, 5000], 4), ([300] * 100, 3)])
def test_against_oracle(act_seq, s1):
    """The decode batch, a ragged multi-token case and more than 256 tokens (several token blocks per product)."""
    p = gen.make_prolog_nonquant_inputs(act_seq, s1=s1, seed=31 + s1)
    o, _ = run_prolog(p, with_q_norm=(s1 != 4))
    want = po.mla_indexer_prolog_nonquant(p, 1e-5, 1e-5)
    idx = p["cache_index"]
    for key in ("q_nope", "q_rope", "idx_query", "weights"):
        close(o[key], want[key], key)
    if "q_norm" in o:
        close(o["q_norm"], want["q_norm"], "q_norm")
    for key in ("kv_cache", "kr_cache", "idx_k_cache"):
        close(o[key][idx], want[key][idx], key)
    check_untouched(o, p)


def test_whole_layer_against_oracle_chain():
    """`decode_indexer_attention_layer` (arguments in the reference's order, sin before cos): its selection against
    the oracle indexer run on the oracle prolog's outputs, its attention against the oracle attention on the kernel's
    own selection and the oracle prolog's queries and caches."""
    act = [5000, 3000, 2048, 70]
    s1 = 2
    p = gen.make_prolog_nonquant_inputs(act, s1=s1, seed=77)
    g = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
    b, t = len(act), len(act) * s1
    act_t = torch.tensor(act, dtype=torch.int32, device=DEV)
    out = torch.full((b, s1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    nb = p["kv_cache"].shape[0] // 128
    sc = pto.decode_indexer_attention_layer(
        g["token_x"].reshape(b, s1, -1), g["w_dq"], g["w_uqqr"], g["w_uk"], g["w_dkvkr"], g["gamma_cq"], g["gamma_ckv"],
        g["sin"].reshape(b, s1, -1), g["cos"].reshape(b, s1, -1), g["cache_index"].reshape(b, s1),
        g["kv_cache"].reshape(nb, 128, 1, 512), g["kr_cache"].reshape(nb, 128, 1, 64), g["block_table"], act_t,
        g["w_idx_qb"], g["w_idx_k"], g["w_idx_proj"], g["ln_gamma"], g["ln_beta"],
        g["idx_k_cache"].reshape(nb, 128, 1, 128), out, sort=True)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    want = po.mla_indexer_prolog_nonquant(p, 1e-5, 1e-5)
    idx = sc["topk_res"].cpu()
    # selection: the oracle indexer on the kernel's own prolog outputs (a score moves with every bf16 step of the
    # query, so the oracle prolog's query would tie-break differently)
    want_idx, _, rows = oracle.lightning_indexer_nonquant(sc["idx_query"].cpu(), g["idx_k_cache"].cpu().reshape(nb, 128, 1, 128),
                                                          sc["idx_weights"].cpu(), act, p["block_table"], s1)
    for ti in range(t):
        untied, _ = oracle.topk_set_diff(idx[ti], want_idx[ti], rows[ti], rel_tie=1e-4)
        assert untied == 0, (ti, untied)
    close(sc["idx_query"], want["idx_query"], "idx_query")
    close(sc["query_nope"], want["q_nope"], "q_nope")
    ref = oracle.sparse_attention(want["q_nope"].reshape(t * 128, 512), want["q_rope"].reshape(t * 128, 64),
                                  want["kv_cache"], want["kr_cache"], None, idx.reshape(t, 2048), p["block_table"], act, s1)
    got = out.cpu()
    for bi in range(b):
        for i in range(s1):
            e = oracle.attention_errors(got[bi, i], ref[bi, i])
            assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 1e-2, (bi, i, e)


def test_arguments_are_checked():
    p = gen.make_prolog_nonquant_inputs([300], s1=1, seed=3)
    g = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
    bf = torch.bfloat16
    outs = [torch.zeros(1, 128, 512, dtype=bf, device=DEV), torch.zeros(1, 128, 64, dtype=bf, device=DEV),
            torch.zeros(1, 64, 128, dtype=bf, device=DEV), torch.zeros(1, 64, dtype=bf, device=DEV)]
    args = [g["token_x"], g["w_dq"], g["w_uqqr"], g["w_uk"], g["w_dkvkr"], g["gamma_cq"], g["gamma_ckv"], g["cos"],
            g["sin"], g["cache_index"], g["kv_cache"], g["kr_cache"], g["w_idx_qb"], g["w_idx_k"], g["w_idx_proj"],
            g["ln_gamma"], g["ln_beta"], g["idx_k_cache"]] + outs
    bad = list(args)
    bad[2] = g["w_uqqr"].to(torch.int8)  # the quantised prolog's weight
    with pytest.raises(ValueError):
        pto.mla_indexer_prolog(*bad)
    bad = list(args)
    bad[10] = g["kv_cache"].to(torch.int8)
    with pytest.raises(ValueError):
        pto.mla_indexer_prolog(*bad)
    bad = list(args)
    bad[21] = torch.zeros(1, 64, dtype=torch.float16, device=DEV)  # the quantised prolog's weights dtype
    with pytest.raises(ValueError):
        pto.mla_indexer_prolog(*bad)
    # a cache row outside the cache is skipped and reported
    ci = g["cache_index"].clone()
    ci[0] = p["kv_cache"].shape[0] + 5
    args[9] = ci
    pto.reset_workspace_status()
    pto.mla_indexer_prolog(*args)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] != 0
    pto.reset_workspace_status()


def test_layer_recorded_into_a_cuda_graph_and_prolog_through_the_registration():
    """The whole layer (prologs + chain, scratch passed in) captured once and replayed after the token's hidden
    states are refreshed in place gives the eager result of the new input; the prolog alone through
    `torch.ops.pypto_b200.mla_indexer_prolog` equals the direct call."""
    import pypto_b200.torch_ops  # noqa: F401  (registers the namespace)

    act, s1 = [3000, 700, 129], 1
    p = gen.make_prolog_nonquant_inputs(act, s1=s1, seed=91)
    p2 = gen.make_prolog_nonquant_inputs(act, s1=s1, seed=92)
    g = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
    b = t = len(act)
    bf = torch.bfloat16
    act_t = torch.tensor(act, dtype=torch.int32, device=DEV)

    def fresh_scratch():
        return dict(query_nope=torch.zeros(t, 128, 512, dtype=bf, device=DEV), query_rope=torch.zeros(t, 128, 64, dtype=bf, device=DEV),
                    idx_query=torch.zeros(t, 64, 128, dtype=bf, device=DEV), idx_weights=torch.zeros(t, 64, dtype=bf, device=DEV),
                    topk_res=torch.zeros(t, 1, 2048, dtype=torch.int32, device=DEV))

    def layer_args(x, caches, out):
        return [x, g["w_dq"], g["w_uqqr"], g["w_uk"], g["w_dkvkr"], g["gamma_cq"], g["gamma_ckv"], g["sin"], g["cos"],
                g["cache_index"], caches["kv_cache"], caches["kr_cache"], g["block_table"], act_t, g["w_idx_qb"],
                g["w_idx_k"], g["w_idx_proj"], g["ln_gamma"], g["ln_beta"], caches["idx_k_cache"], out]

    # captured: static input buffer x, own copies of the caches
    x = g["token_x"].clone()
    caches_c = {k: g[k].clone() for k in ("kv_cache", "kr_cache", "idx_k_cache")}
    out_c = torch.zeros((b, s1, 128, 512), dtype=bf, device=DEV)
    sc_c = fresh_scratch()
    step = pto.CapturedCall(pto.decode_indexer_attention_layer, *layer_args(x, caches_c, out_c), scratch=sc_c, sort=True)
    x.copy_(p2["token_x"].to(DEV))
    step.replay()
    torch.cuda.synchronize()
    assert step.workspace_status()[0] == 0
    # eager on the same new input
    caches_e = {k: g[k].clone() for k in ("kv_cache", "kr_cache", "idx_k_cache")}
    out_e = torch.zeros_like(out_c)
    sc_e = pto.decode_indexer_attention_layer(*layer_args(p2["token_x"].to(DEV), caches_e, out_e), scratch=fresh_scratch(),
                                              sort=True)
    torch.cuda.synchronize()
    assert torch.equal(out_c, out_e) and torch.equal(sc_c["topk_res"], sc_e["topk_res"])
    for k in caches_c:
        assert torch.equal(caches_c[k], caches_e[k]), k

    # the prolog through the registered op
    o1 = fresh_scratch()
    o2 = fresh_scratch()
    c1 = {k: g[k].clone() for k in ("kv_cache", "kr_cache", "idx_k_cache")}
    c2 = {k: g[k].clone() for k in ("kv_cache", "kr_cache", "idx_k_cache")}
    common = [g["token_x"], g["w_dq"], g["w_uqqr"], g["w_uk"], g["w_dkvkr"], g["gamma_cq"], g["gamma_ckv"], g["cos"], g["sin"],
              g["cache_index"]]
    tail = [g["w_idx_qb"], g["w_idx_k"], g["w_idx_proj"], g["ln_gamma"], g["ln_beta"]]
    pto.mla_indexer_prolog(*common, c1["kv_cache"], c1["kr_cache"], *tail, c1["idx_k_cache"], o1["query_nope"],
                           o1["query_rope"], o1["idx_query"], o1["idx_weights"], 1e-5, 1e-5)
    torch.ops.pypto_b200.mla_indexer_prolog(*common, c2["kv_cache"], c2["kr_cache"], *tail, c2["idx_k_cache"],
                                            o2["query_nope"], o2["query_rope"], o2["idx_query"], o2["idx_weights"], 1e-5,
                                            1e-5)
    torch.cuda.synchronize()
    for k in ("query_nope", "query_rope", "idx_query", "idx_weights"):
        assert torch.equal(o1[k], o2[k]), k
    for k in c1:
        assert torch.equal(c1[k], c2[k]), k
