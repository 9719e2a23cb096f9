"""Lightning indexer on the GPU against the CPU oracle and the reference-made fixtures.
Everything goes through the operator wrappers, i.e. through the C ABI."""
import pytest
import torch

import oracle
import pypto_b200 as pto
from pypto_b200 import inputs as gen
from golden_util import LI_CASES, load_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _scores(d, simt, first_mm=False):
    g = d.to(DEV)
    stride = d.max_blocks * 128
    sc = torch.full((d.t, stride), float("nan"), dtype=torch.float32, device=DEV)
    fm = torch.zeros((d.t * 64, stride), dtype=torch.float16, device=DEV) if first_mm else None
    pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, sc, fm, simt=simt)
    torch.cuda.synchronize()
    return sc.cpu(), (fm.cpu() if fm is not None else None)


def _decode(d, **kw):
    g = d.to(DEV)
    out = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_decode(pto.from_torch(g.idx_query, name="idx_query", dynamic_axis=[0]), g.idx_query_scale,
                                 g.idx_key_cache, g.idx_key_scale, g.idx_weight, g.act_seq_key, g.block_table,
                                 pto.from_torch(out), [128, 64, 32, 16, 8, 4, 1], pto.LightningIndexerConfigs(), 2048,
                                 **kw)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    return out.cpu()


def _check_rows(sc, rows, d, rtol):
    for ti, row in enumerate(rows):
        n = row.numel()
        torch.testing.assert_close(sc[ti, :n], row, rtol=rtol, atol=1e-9)
        # positions past the sequence are left untouched
        assert torch.isnan(sc[ti, n:]).all()


@pytest.mark.parametrize("name", LI_CASES)
@pytest.mark.parametrize("simt", [True, False], ids=["simt", "tcgen05"])
def test_scores_match_oracle_on_fixtures(name, simt):
    d, z = load_case(name)
    rows, first_mm = oracle.li_oracle.li_scores(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                d.idx_weight, d.act_seq, d.block_table, d.s1, return_first_mm=True)
    sc, fm = _scores(d, simt, first_mm=simt)
    # same formula; the 64-term fp32 head sum is taken in a different order
    _check_rows(sc, rows, d, rtol=3e-6)
    mm_out = torch.from_numpy(z["mm_out"])
    for ti, row in enumerate(rows):
        torch.testing.assert_close(sc[ti, :row.numel()], mm_out[ti, :row.numel()], rtol=3e-6, atol=1e-9)
    if simt:
        for ti, row in enumerate(rows):  # fp16 relu(dot)/2048 tiles: bit-exact
            assert torch.equal(fm[ti * 64:(ti + 1) * 64, :row.numel()], first_mm[ti])


@pytest.mark.parametrize("s1", [1, 2, 3, 4])
def test_integer_dots_bit_exact(s1):
    """One-hot head weight with unit scales turns the score into fp16(relu(q_h.k)/2048) itself,
    which exposes every int32 dot product of the tensor-core path exactly."""
    act = [1000, 77, 513][: max(1, 4 - s1)] + [300]
    d = gen.make_inputs(act, s1=s1, seed=11 + s1, with_attention=False)
    d.idx_query_scale.fill_(1.0)
    d.idx_key_scale.fill_(1.0)
    for head in (0, 21, 63):
        d.idx_weight.zero_()
        d.idx_weight[:, head] = 1.0
        rows, first_mm = oracle.li_oracle.li_scores(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                    d.idx_weight, d.act_seq, d.block_table, d.s1, return_first_mm=True)
        sc, _ = _scores(d, simt=False)
        for ti, row in enumerate(rows):
            want = first_mm[ti][head].to(torch.float32)
            assert torch.equal(sc[ti, :row.numel()], want), f"token {ti} head {head}"
            assert torch.equal(row, want)


def test_tensor_core_scores_equal_simt_scores_on_large_ragged_batch():
    g = torch.Generator().manual_seed(5)
    act = torch.randint(1, 9000, (37,), generator=g).tolist() + [16384, 128, 127, 129]
    d = gen.make_inputs(act, s1=2, seed=99, scale_dtype=torch.float16, with_attention=False)
    a, _ = _scores(d, simt=True)
    b, _ = _scores(d, simt=False)
    for bi, s in enumerate(act):
        for i in range(2):
            torch.testing.assert_close(b[bi * 2 + i, :s], a[bi * 2 + i, :s], rtol=3e-6, atol=1e-9)
    assert pto.workspace_status()[0] == 0


@pytest.mark.parametrize("name", LI_CASES)
@pytest.mark.parametrize("simt", [True, False], ids=["simt", "tcgen05"])
def test_topk_matches_reference_fixture(name, simt):
    d, z = load_case(name)
    got = _decode(d, _simt_scores=simt)
    want = torch.from_numpy(z["topk_res"])
    mm_out = torch.from_numpy(z["mm_out"])
    for ti in range(d.t):
        untied, tied = oracle.topk_set_diff(got[ti], want[ti], mm_out[ti])
        assert untied == 0, f"row {ti}: {untied} untied differences ({tied} tied)"
        bi, i = divmod(ti, d.s1)
        eff = max(0, min(2048, d.act_seq[bi] - (d.s1 - 1 - i)))
        assert torch.all(got[ti, 0, :eff] >= 0) and torch.all(got[ti, 0, eff:] == -1)
        assert len(set(got[ti, 0, :eff].tolist())) == eff
        # value-descending order
        vals = mm_out[ti][got[ti, 0, :eff].long()]
        assert torch.all(vals[:-1] >= vals[1:] - 1e-6 * vals[:-1].abs())


def test_topk_stage_exact_on_kernel_scores():
    """Selection alone: over the kernel's own score rows the selected set must equal torch.topk's
    exactly (ties broken toward the smaller position)."""
    g = torch.Generator().manual_seed(3)
    rows = [5000, 2049, 2048, 131072, 40000, 1, 70000]
    stride = 131072
    sc = torch.randn((len(rows), stride), generator=g)
    sc[4, :40000] = torch.randint(0, 50, (40000,), generator=g).float()  # heavy ties
    sc[6, :70000] = 1.25  # all equal: the radix path must pick the 2048 smallest positions
    act = torch.tensor(rows, dtype=torch.int32)
    out = torch.zeros((len(rows), 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_topk(sc.to(DEV), act.to(DEV), out, s1=1, selected_count=2048)
    torch.cuda.synchronize()
    out = out.cpu()
    for r, n in enumerate(rows):
        k = min(n, 2048)
        key = sc[r, :n].double() * 1e6 - torch.arange(n).double() * 1e-3 if r in (4, 6) else sc[r, :n].double()
        want = torch.topk(key, k).indices
        assert set(out[r, 0, :k].tolist()) == set(want.tolist()), f"row {r}"
        assert torch.all(out[r, 0, k:] == -1)
        # value-descending, ties toward the smaller position (rows this long are scanned by a cluster of CTAs)
        got_keys = key[out[r, 0, :k].long()]
        assert torch.all(got_keys[:-1] >= got_keys[1:]), f"row {r} not ordered"
    # unsorted variant selects the same sets
    out2 = torch.zeros_like(out, device=DEV)
    pto.lightning_indexer_topk(sc.to(DEV), act.to(DEV), out2, s1=1, selected_count=2048, sort=False)
    torch.cuda.synchronize()
    for r, n in enumerate(rows):
        assert set(out2[r, 0].cpu().tolist()) == set(out[r, 0].tolist())


def test_config1_shape_against_oracle():
    """Benchmark configuration 1 (batch 8, context 32768) end to end."""
    d = gen.make_config(1)
    idx, vals, rows = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                               d.idx_weight, d.act_seq, d.block_table, d.s1)
    got = _decode(d)
    for ti in range(d.t):
        untied, _ = oracle.topk_set_diff(got[ti], idx[ti], rows[ti])
        assert untied == 0


@pytest.mark.parametrize("simt", [False, True], ids=["tcgen05", "simt"])
def test_rejected_page_sets_status_without_fault(simt):
    d = gen.make_inputs([700, 300], s1=1, seed=4, with_attention=False)
    d.block_table[0, 2] = d.block_num + 5  # outside the cache: the page is skipped and reads as zeros
    pto.reset_workspace_status()
    g = d.to(DEV)
    out = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_decode(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, out, None, None, 2048, _simt_scores=simt)
    st = pto.workspace_status()
    assert st[0] & 0x1 and st[1] == d.block_num + 5
    pto.reset_workspace_status()
    assert pto.workspace_status()[0] == 0
    # both score kernels give the rejected page's 128 positions the score 0, whatever the buffer held before
    sc = torch.full((d.t, d.max_blocks * 128), float("nan"), dtype=torch.float32, device=DEV)
    pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, sc, simt=simt)
    torch.cuda.synchronize()
    assert torch.all(sc[0, 256:384] == 0) and not torch.isnan(sc[0, :700]).any()
    pto.reset_workspace_status()


@pytest.mark.parametrize("name", [n for n in LI_CASES if n.endswith("f16")])
@pytest.mark.parametrize("simt", [True, False], ids=["simt", "tcgen05"])
def test_fp16_chain_formulation_matches_st_golden(name, simt):
    """The older formulation (LightningIndexerTopkImpl, flag PTO_LI_FP16_CHAIN): scores against the ST golden's
    quantised branch (every fp16 step reproduces exactly; the fp32 head sum is taken in another order), selected
    sets exact on untied scores."""
    d, z = load_case(name)
    g = d.to(DEV)
    stride = d.max_blocks * 128
    sc = torch.full((d.t, stride), float("nan"), dtype=torch.float32, device=DEV)
    pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, sc, None, simt=simt, fp16_chain=True)
    torch.cuda.synchronize()
    sc = sc.cpu()
    want_rows = torch.from_numpy(z["chain_rows"])
    rows = oracle.li_scores_fp16_chain(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale, d.idx_weight,
                                       d.act_seq, d.block_table, d.s1)
    for bi in range(d.b):
        for i in range(d.s1):
            ti = bi * d.s1 + i
            eff = d.act_seq[bi] - (d.s1 - 1 - i)
            torch.testing.assert_close(sc[ti, :d.act_seq[bi]], rows[ti], rtol=3e-6, atol=1e-9)
            if eff > 0:
                torch.testing.assert_close(sc[ti, :eff], want_rows[ti, :eff], rtol=3e-6, atol=1e-9)
    got = _decode(d, _simt_scores=simt, fp16_chain=True)
    want = torch.from_numpy(z["chain_topk_res"])
    for ti in range(d.t):
        untied, _ = oracle.topk_set_diff(got[ti], want[ti], want_rows[ti])
        assert untied == 0, f"row {ti}: {untied} untied differences"


def test_fp16_chain_needs_fp16_scales():
    d = gen.make_inputs([300], s1=1, seed=5, scale_dtype=torch.float32, with_attention=False)
    g = d.to(DEV)
    sc = torch.zeros((d.t, d.max_blocks * 128), dtype=torch.float32, device=DEV)
    with pytest.raises(RuntimeError, match="fp16"):
        pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                     g.act_seq_key, g.block_table, sc, None, fp16_chain=True)


@pytest.mark.parametrize("s1", [3, 4])
def test_three_and_four_query_tokens_with_many_pages_per_cta(s1):
    """s1 = 3, 4 leave room for two accumulator slots only; with more than four pages per CTA every slot is
    reused many times by the epilogue warps (one sequence of 131072 keys: about seven pages per CTA). The
    tensor-core scores must equal the CUDA-core kernel's."""
    d = gen.make_inputs([131072], s1=s1, seed=60 + s1, with_attention=False)
    a, _ = _scores(d, simt=True)
    b, _ = _scores(d, simt=False)
    assert pto.workspace_status()[0] == 0
    for i in range(s1):
        torch.testing.assert_close(b[i, :131072], a[i, :131072], rtol=3e-6, atol=1e-9)


def test_prefill_chunk_groups_share_a_launch():
    """22 query tokens per sequence: five full groups of four go into one launch (grid y), the last two tokens
    into a second one. Scores equal the CUDA-core kernel's for every token."""
    d = gen.make_inputs([9000, 300], s1=22, seed=77, with_attention=False)
    a, _ = _scores(d, simt=True)
    b, _ = _scores(d, simt=False)
    assert pto.workspace_status()[0] == 0
    for bi, s in enumerate(d.act_seq):
        for i in range(22):
            torch.testing.assert_close(b[bi * 22 + i, :s], a[bi * 22 + i, :s], rtol=3e-6, atol=1e-9)


@pytest.mark.parametrize("s1", [1, 2, 3])
def test_chained_selection_from_the_score_kernels_histogram_equals_the_two_stages(s1):
    """Asked to (`histogram=True`), with at most two query tokens per sequence, the score kernel leaves a 4096-bin
    histogram per row and the selection starts from it (one scan of the row, a radix step over the candidates in
    shared memory); with three tokens it scans the row for min/max and its own histogram as it does by default.
    Either way the ordered result must equal the selection run alone over the same score rows. Cases: ragged
    lengths, sequences whose causal end cuts a page, a row shorter than k, and rows whose scores all tie (zero
    weights: one bin holds the whole row, which sends the selection back to its own passes and the radix path)."""
    g0 = torch.Generator().manual_seed(50 + s1)
    act = torch.randint(2049, 30000, (6,), generator=g0).tolist() + [2048 + s1, 300, 9000, 4097]
    d = gen.make_inputs(act, s1=s1, seed=91 + s1, with_attention=False)
    d.idx_weight[8 * s1:9 * s1] = 0  # sequence 8: every score is +0
    got = _decode(d, histogram=True)
    assert torch.equal(got, _decode(d))
    g = d.to(DEV)
    sc = torch.zeros((d.t, d.max_blocks * 128), dtype=torch.float32, device=DEV)
    pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, sc)
    want = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_topk(sc, g.act_seq_key, want, s1=s1, selected_count=2048)
    torch.cuda.synchronize()
    assert torch.equal(got, want.cpu())
    # the tied rows select the smallest positions
    for i in range(s1):
        assert got[8 * s1 + i, 0].tolist() == list(range(2048))
    # unordered output: the same sets
    got_u = _decode(d, sort=False, histogram=True)
    for ti in range(d.t):
        assert set(got_u[ti, 0].tolist()) == set(got[ti, 0].tolist())


def test_two_ctas_per_row_with_thousands_of_tied_candidates():
    """24 rows: two CTAs per row. Unordered output with a single exchange between them: rank 1 writes its selected
    positions from the end of the row and pushes its candidates to the end of rank 0's buffer. Rows of eight
    distinct values put ~3700 keys into the threshold bucket, half in each rank, so that the two candidate segments
    overlap when rank 0 joins them; rows of 300 distinct values are the ordinary case."""
    g = torch.Generator().manual_seed(11)
    n, rows = 30000, 24
    sc = torch.empty((rows, 32768))
    sc[:12, :n] = torch.randint(0, 8, (12, n), generator=g).float()
    sc[12:, :n] = torch.randint(0, 300, (12, n), generator=g).float()
    act = torch.full((rows,), n, dtype=torch.int32)
    out = torch.zeros((rows, 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_topk(sc.to(DEV), act.to(DEV), out, s1=1, selected_count=2048, sort=False)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    out = out.cpu()
    for r in range(rows):
        key = sc[r, :n].double() * 1e6 - torch.arange(n).double() * 1e-3  # ties toward the smaller position
        want = set(torch.topk(key, 2048).indices.tolist())
        got = out[r, 0].tolist()
        assert len(set(got)) == 2048 and set(got) == want, f"row {r}"
