"""The fused chain (indexer -> top-k -> sparse attention) on the GPU against the oracle chain."""
import pytest
import torch

import oracle
import pypto_b200 as pto
from pypto_b200 import inputs as gen

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fused(d, sort=False, fill=0, **kw):
    g = d.to(DEV)
    idx = torch.full((d.t, 1, 2048), fill, dtype=torch.int32, device=DEV)
    out = torch.full((d.b, d.s1, 128, 512), float(fill), dtype=torch.bfloat16, device=DEV)
    pto.decode_indexer_attention_quant(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                       g.query_nope, g.query_rope, g.key_nope_2d, g.key_rope_2d, g.k_nope_scales,
                                       g.act_seq_key, g.block_table, idx, out, sort=sort, **kw)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    return idx.cpu(), out.cpu()


def test_fused_chain_with_the_score_kernels_histogram_gives_the_same_result():
    """`histogram=True`: the selection starts from the histogram the score kernel leaves (behind the attention
    partials in the workspace); ordered indices and outputs are those of the default call, bit for bit."""
    d = gen.make_inputs([4096, 9000, 300, 2047, 2048, 2049, 15, 30000], s1=2, seed=77)
    idx, out = _fused(d, sort=True)
    idx_h, out_h = _fused(d, sort=True, histogram=True)
    assert torch.equal(idx_h, idx) and torch.equal(out_h, out)


@pytest.mark.parametrize("s1,act", [(1, [4096, 9000, 300, 2047, 2048, 2049, 15]), (2, [6000, 1, 2500, 130])])
def test_fused_chain_matches_oracle_chain(s1, act):
    d = gen.make_inputs(act, s1=s1, seed=50 + s1)
    idx, out = _fused(d)
    want_idx, _, rows = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                 d.idx_weight, d.act_seq, d.block_table, d.s1)
    for ti in range(d.t):
        untied, _ = oracle.topk_set_diff(idx[ti], want_idx[ti], rows[ti])
        assert untied == 0
    # attention against the oracle fed with the oracle's own indices (order differs, sets equal)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   want_idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    e = oracle.attention_errors(out, want)
    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, e
    # sorted variant gives the same sets and an attention output within rounding
    idx2, out2 = _fused(d, sort=True)
    for ti in range(d.t):
        assert set(idx2[ti].reshape(-1).tolist()) == set(idx[ti].reshape(-1).tolist())
    e = oracle.attention_errors(out2, want)
    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, e


def test_fused_is_deterministic_and_idempotent():
    d = gen.make_inputs([7000, 3000, 12000], s1=1, seed=77)
    i1, o1 = _fused(d, sort=True)
    i2, o2 = _fused(d, sort=True)
    assert torch.equal(i1, i2)
    assert torch.equal(o1, o2)


def test_prefill_chunk_many_query_tokens_per_sequence():
    """A prefill chunk: one sequence, 12 new query tokens at the end of a 5000-token context
    (query i sees the first S - 11 + i positions). The indexer runs the tokens in groups of four
    per launch; the attention entry is the prefill one."""
    s1, S = 12, 5000
    d = gen.make_inputs([S], s1=s1, seed=91)
    g = d.to(DEV)
    idx = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_decode(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, idx, None, None, 2048)
    out = torch.zeros((d.b, s1, 128, 512), dtype=torch.bfloat16, device=DEV)
    pto.sparse_flash_attention_quant_p(g.query_nope, g.query_rope, g.key_nope_2d, g.key_rope_2d, g.k_nope_scales,
                                       idx.reshape(d.t, 2048), g.block_table, g.act_seq_key, out, 128, 1, 576 ** -0.5,
                                       2048, 128, d.max_blocks, pto.SaTileShapeConfig())
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    want_idx, _, rows = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                 d.idx_weight, d.act_seq, d.block_table, s1)
    idx = idx.cpu()
    for ti in range(d.t):
        untied, _ = oracle.topk_set_diff(idx[ti], want_idx[ti], rows[ti])
        assert untied == 0, f"token {ti}"
        assert int(idx[ti].max()) < S - (s1 - 1 - ti)  # causal cut
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   want_idx.reshape(d.t, 2048), d.block_table, d.act_seq, s1)
    e = oracle.attention_errors(out.cpu(), want)
    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, e


def test_mtp_long_context_properties():
    """Configuration-3-like shape at reduced batch: 4 sequences of 131072 keys, two query tokens
    each. Size-independent checks: every index inside the causal range, indices distinct, the
    selected scores dominate a sample of unselected ones, attention rows finite and normalised
    (each output element within the min/max of the dequantised values of its column is too weak;
    instead the output equals the oracle attention evaluated on the kernel's own indices)."""
    d = gen.make_inputs([131072] * 4, s1=2, seed=333)
    g = d.to(DEV)
    idx = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    out = torch.zeros((d.b, 2, 128, 512), dtype=torch.bfloat16, device=DEV)
    pto.decode_indexer_attention_quant(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                       g.query_nope, g.query_rope, g.key_nope_2d, g.key_rope_2d, g.k_nope_scales,
                                       g.act_seq_key, g.block_table, idx, out)
    sc = torch.zeros((d.t, d.max_blocks * 128), dtype=torch.float32, device=DEV)
    pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, sc)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    idx_c, sc_c = idx.cpu().reshape(d.t, 2048), sc.cpu()
    for ti in range(d.t):
        eff = 131072 - (1 - ti % 2)
        row = idx_c[ti]
        assert int(row.min()) >= 0 and int(row.max()) < eff
        assert len(set(row.tolist())) == 2048
        kth = sc_c[ti][row.long()].min()
        mask = torch.ones(eff, dtype=torch.bool)
        mask[row.long()] = False
        assert float(sc_c[ti][:eff][mask].max()) <= float(kth)  # exact top-k of the kernel's own scores
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   idx_c, d.block_table, d.act_seq, 2)
    e = oracle.attention_errors(out.cpu(), want)
    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, e


def test_empty_and_tiny_sequences():
    """A sequence of length 0 selects nothing (all -1) and its attention row stays zero; lengths
    1 and 5 select every position."""
    d = gen.make_inputs([0, 1, 5, 300], s1=1, seed=8)
    idx, out = _fused(d, sort=True, fill=7)   # outputs pre-filled: every element must be overwritten
    assert torch.all(idx[0] == -1) and torch.all(out[0] == 0)
    assert idx[1, 0, 0] == 0 and torch.all(idx[1, 0, 1:] == -1)
    assert sorted(idx[2, 0, :5].tolist()) == [0, 1, 2, 3, 4] and torch.all(idx[2, 0, 5:] == -1)
    want_idx, _, _ = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                              d.idx_weight, d.act_seq, d.block_table, d.s1)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   want_idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    e = oracle.attention_errors(out, want)
    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, e


@pytest.mark.parametrize("b,s1", [(3, 2), (64, 1), (70, 1)])
def test_back_to_back_fused_calls_equal_the_stages_run_one_by_one(b, s1):
    """Inside the fused call the top-k and attention kernels are launched with programmatic serialization (they
    may start while their predecessor drains). Six calls without any synchronisation in between, a fill kernel
    before each, must give the index sets of the stand-alone indexer and, for those indices, bit for bit the
    output of the stand-alone attention operator."""
    g0 = torch.Generator().manual_seed(b * 10 + s1)
    choices = [1, 100, 2047, 2049, 5000, 9000, 20000, 40000]
    act = [choices[int(torch.randint(0, len(choices), (1,), generator=g0))] for _ in range(b)]
    d = gen.make_inputs(act, s1=s1, seed=900 + b, device=DEV)
    li = (d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale, d.idx_weight)
    reps = 6
    idxs = [torch.full((d.t, 1, 2048), -7, dtype=torch.int32, device=DEV) for _ in range(reps)]
    outs = [torch.full((d.b, d.s1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(reps)]
    junk = torch.empty(32 << 20, dtype=torch.uint8, device=DEV)
    for r in range(reps):
        junk.fill_(r)
        pto.decode_indexer_attention_quant(*li, d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d,
                                           d.k_nope_scales, d.act_seq_key, d.block_table, idxs[r], outs[r])
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    idx_ref = torch.zeros_like(idxs[0])
    pto.lightning_indexer_decode(*li, d.act_seq_key, d.block_table, idx_ref, None, None, 2048)
    torch.cuda.synchronize()
    want_sets = idx_ref.sort(dim=-1).values
    for r in range(reps):
        assert torch.equal(idxs[r].sort(dim=-1).values, want_sets)
        out2 = torch.zeros_like(outs[r])
        pto.sparse_flash_attention_quant_d(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                           idxs[r].reshape(d.t, 2048), d.block_table, d.act_seq_key, out2, 128, 1,
                                           576 ** -0.5, 2048, 128, d.max_blocks)
        torch.cuda.synchronize()
        assert torch.equal(out2, outs[r])


def test_random_shapes_against_oracle_chain():
    """Forty seeded random cases: batch 1-8, one to four query tokens per sequence, lengths drawn around the page and
    selection boundaries (1, 127-129, 2047-2050, 4095-4097) and up to 40000 keys, both scale dtypes, ordered and
    unordered output. Selected sets against the oracle indexer (exact on untied scores, -1 padding, no duplicates,
    positions inside the causal prefix), attention against the oracle on the kernel's own selection."""
    import random

    rng = random.Random(2024)
    special = [1, 2, 3, 127, 128, 129, 2047, 2048, 2049, 2050, 4095, 4096, 4097, 2048 + 127, 2048 + 128]
    for case in range(40):
        b = rng.choice([1, 1, 2, 3, 5, 8])
        s1 = rng.choice([1, 1, 2, 3, 4])
        act = []
        for _ in range(b):
            r = rng.random()
            act.append(rng.choice(special) if r < 0.4 else rng.randint(1, 9000) if r < 0.8 else rng.randint(9000, 40000))
        dt = rng.choice([torch.float32, torch.float16])
        sort = rng.random() < 0.5
        d = gen.make_inputs(act, s1=s1, seed=1000 + case, scale_dtype=dt)
        idx, out = _fused(d, sort=sort, fill=5)
        want_idx, _, rows = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                     d.idx_weight, d.act_seq, d.block_table, d.s1)
        for ti in range(d.t):
            bi, i = divmod(ti, s1)
            eff = act[bi] - (s1 - 1 - i)
            nvalid = max(0, min(eff, 2048))
            untied, _ = oracle.topk_set_diff(idx[ti], want_idx[ti], rows[ti])
            assert untied == 0, (case, act, s1, ti, untied)
            assert int((idx[ti] >= 0).sum()) == nvalid and torch.all(idx[ti, 0, nvalid:] == -1), (case, ti)
            v = idx[ti, 0, :nvalid]
            assert nvalid == 0 or (int(v.max()) < eff and len(set(v.tolist())) == nvalid), (case, ti)
        want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                       idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
        for bi in range(d.b):
            for i in range(s1):
                if act[bi] - s1 + 1 + i > 0:
                    e = oracle.attention_errors(out[bi, i], want[bi, i])
                    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, (case, act, s1, bi, i, e)
                else:
                    assert torch.all(out[bi, i] == 0), (case, bi, i)
