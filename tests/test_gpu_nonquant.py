"""The non-quantised formulation on the GPU: bf16 indexer (tcgen05 kind::f16 in the score kernel's ring) and the
chain indexer -> top-k -> attention over the bf16 latent cache, against the reference-made fixtures and the oracle.

Tolerances. Scores: a dot of 128 bf16 products is accumulated in fp32 by the tensor core in an order of its own, so
a score (a signed 64-term sum of such dots, |score| up to ~100) is compared with rtol 2e-5 and atol 1e-3. Selected
sets: exact except where a differing position's score lies within 1e-4 (relative) of the k-th score. Attention:
max-abs 2e-2, rel-L2 5e-3, the benchmark's statement for the quantised path."""
import pytest
import torch

import oracle
import pypto_b200 as pto
from pypto_b200 import inputs as gen
from golden_util import NONQUANT_CASES, load_case

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_TIE = 1e-4


def _scores(g, d):
    sc = torch.full((d.t, d.max_blocks * 128), float("nan"), dtype=torch.float32, device=DEV)
    pto.lightning_indexer_topk_nonquant(g.idx_query, g.idx_key_cache, g.idx_weight, g.act_seq_key, g.block_table, None,
                                        scores_out=sc)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    return sc.cpu()


def _topk(g, d, **kw):
    idx = torch.full((d.t, 1, 2048), -7, dtype=torch.int32, device=DEV)
    pto.lightning_indexer_topk_nonquant(g.idx_query, g.idx_key_cache, g.idx_weight, g.act_seq_key, g.block_table, idx,
                                        **kw)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    return idx.cpu()


def _check_sets(idx, want_idx, rows, d):
    for ti in range(d.t):
        bi, i = divmod(ti, d.s1)
        eff = d.act_seq[bi] - (d.s1 - 1 - i)
        untied, _ = oracle.topk_set_diff(idx[ti], want_idx[ti], rows[ti], rel_tie=REL_TIE)
        assert untied == 0, (ti, untied)
        nvalid = max(0, min(eff, 2048))
        assert int((idx[ti] >= 0).sum()) == nvalid
        assert torch.all(idx[ti, 0, nvalid:] == -1)


@pytest.mark.parametrize("name", NONQUANT_CASES)
def test_scores_and_sets_match_reference_fixture(name):
    d, z = load_case(name)
    g = d.to(DEV)
    sc = _scores(g, d)
    want_rows = torch.from_numpy(z["rows"])
    for ti in range(d.t):
        bi, i = divmod(ti, d.s1)
        eff = d.act_seq[bi] - (d.s1 - 1 - i)
        if eff > 0:
            torch.testing.assert_close(sc[ti, :eff], want_rows[ti, :eff], rtol=2e-5, atol=1e-3)
        # positions past the sequence are not written
        assert torch.isnan(sc[ti, d.act_seq[bi]:]).all()
    idx = _topk(g, d)
    _check_sets(idx, torch.from_numpy(z["topk_res"]), want_rows, d)
    # value-descending on the kernel's own scores
    for ti in range(d.t):
        n = int((idx[ti] >= 0).sum())
        v = sc[ti][idx[ti, 0, :n].long()]
        assert torch.all(v[:-1] >= v[1:])
    # the quantised operator's name dispatches on the query dtype
    idx2 = torch.zeros_like(idx, device=DEV)
    pto.lightning_indexer_decode(g.idx_query, None, g.idx_key_cache, None, g.idx_weight, g.act_seq_key, g.block_table,
                                 idx2)
    torch.cuda.synchronize()
    assert torch.equal(idx2.cpu(), idx)


@pytest.mark.parametrize("s1", [1, 2, 3, 5])
def test_many_pages_and_token_groups_against_oracle(s1):
    """Long ragged sequences (CTA ranges cross sequence boundaries) and more query tokens per sequence than one
    launch takes (groups of two)."""
    g0 = torch.Generator().manual_seed(40 + s1)
    act = torch.randint(1, 20000, (7,), generator=g0).tolist() + [s1, 1, 4096]
    d = gen.make_nonquant_inputs(act, s1=s1, seed=77 + s1, with_attention=False)
    g = d.to(DEV)
    sc = _scores(g, d)
    want_idx, _, rows = oracle.lightning_indexer_nonquant(d.idx_query, d.idx_key_cache, d.idx_weight, d.act_seq,
                                                          d.block_table, d.s1)
    for ti in range(d.t):
        n = d.act_seq[ti // s1]
        torch.testing.assert_close(sc[ti, :n], rows[ti], rtol=2e-5, atol=1e-3)
    _check_sets(_topk(g, d, sort=False), want_idx, rows, d)


def test_nonquant_chain_against_oracle():
    """bf16 indexer -> top-k -> attention over the bf16 latent cache in one call, against the oracle chain run on
    the kernel's own selection (the sets are checked separately)."""
    d = gen.make_nonquant_inputs([5000, 3000, 9000, 2048, 70, 1], s1=2, seed=5)
    g = d.to(DEV)
    idx = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    out = torch.full((d.b, d.s1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    pto.decode_indexer_attention(g.idx_query, g.idx_key_cache, g.idx_weight, g.query_nope, g.query_rope, g.key_nope_2d,
                                 g.key_rope_2d, g.act_seq_key, g.block_table, idx, out)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    want_idx, _, rows = oracle.lightning_indexer_nonquant(d.idx_query, d.idx_key_cache, d.idx_weight, d.act_seq,
                                                          d.block_table, d.s1)
    _check_sets(idx.cpu(), want_idx, rows, d)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, None,
                                   idx.cpu().reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    got = out.cpu()
    for bi in range(d.b):
        for i in range(d.s1):
            if d.act_seq[bi] - d.s1 + 1 + i > 0:
                e = oracle.attention_errors(got[bi, i], want[bi, i])
                assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, (bi, i, e)
            else:
                assert torch.all(got[bi, i] == 0) and torch.all(idx[bi * d.s1 + i] == -1)
    # the chain equals its stages run one by one (ordered output: the unordered one depends on the order in which
    # the selecting threads append)
    pto.decode_indexer_attention(g.idx_query, g.idx_key_cache, g.idx_weight, g.query_nope, g.query_rope, g.key_nope_2d,
                                 g.key_rope_2d, g.act_seq_key, g.block_table, idx, out, sort=True)
    idx2 = torch.zeros_like(idx)
    pto.lightning_indexer_topk_nonquant(g.idx_query, g.idx_key_cache, g.idx_weight, g.act_seq_key, g.block_table, idx2)
    out2 = torch.zeros_like(out)
    pto.sparse_flash_attention_quant_d(g.query_nope, g.query_rope, g.key_nope_2d, g.key_rope_2d, None, idx2,
                                       g.block_table, g.act_seq_key, out2, 128, 1, 576 ** -0.5, 2048, 128, d.max_blocks)
    torch.cuda.synchronize()
    assert torch.equal(idx2, idx) and torch.equal(out2, out)


def test_nonquant_arguments_are_checked():
    d = gen.make_nonquant_inputs([300], s1=1, seed=3, with_attention=False)
    g = d.to(DEV)
    idx = torch.zeros((1, 1, 2048), dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError):
        pto.lightning_indexer_topk_nonquant(g.idx_query.to(torch.float16), g.idx_key_cache, g.idx_weight,
                                            g.act_seq_key, g.block_table, idx)
    with pytest.raises(ValueError):
        pto.lightning_indexer_decode(g.idx_query, g.idx_weight, g.idx_key_cache, None, g.idx_weight, g.act_seq_key,
                                     g.block_table, idx)
