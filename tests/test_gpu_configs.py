"""The benchmark's own configurations and the reference's own test-case lists on the GPU against the
CPU oracle, at their real sizes where the oracle finishes in seconds.

  * configuration 2 exactly as bench.py builds it (64 sequences, lengths U[4096, 65536], data drawn on the
    device from the benchmark's seed), the fused operator against the oracle chain;
  * configuration 3 at a reduced batch (131072 keys, two query tokens per sequence): scores and top-k sets
    against the oracle;
  * configuration 4's shape in small: one sequence, 64 new query tokens, a 16-head slice with head_begin > 0;
  * the case lists of the reference's system tests:
      attention  framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_gather_selected_attention.py:334-454
                 and examples/models/deepseek_v32_exp/deepseekv32_sparse_flash_attention_quant.py:462-472,
      fused      framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_decode_indexer_attention_quant.py:468-479,
      indexer    framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_lightning_indexer.py:374-376, :428-430;
  * the paged-gather known answer of python/pypto/experimental.py:62-87 through the attention kernel's gather.

Tolerances are the benchmark's: top-k sets exact on untied scores, attention max-abs 2e-2 and rel-L2 5e-3,
per query token.
"""
import numpy as np
import pytest
import torch

import oracle
import pypto_b200 as pto
from pypto_b200 import inputs as gen
from golden_util import GOLDEN

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCALE = 576 ** -0.5
MAX_ABS, REL_L2 = 2e-2, 5e-3


def _check_attention(got, want, d):
    """Whole output and every query token on its own (a short row cannot hide behind a long one)."""
    got, want = got.reshape(d.t, -1, 512), want.reshape(d.t, -1, 512)
    e = oracle.attention_errors(got, want)
    assert e["max_abs"] <= MAX_ABS and e["rel_l2"] <= REL_L2, e
    worst = 0.0
    for ti in range(d.t):
        bi, i = divmod(ti, d.s1)
        if d.act_seq[bi] - d.s1 + 1 + i <= 0:
            assert torch.all(got[ti] == 0)
            continue
        et = oracle.attention_errors(got[ti], want[ti])
        assert et["max_abs"] <= MAX_ABS and et["rel_l2"] <= REL_L2, (ti, et)
        worst = max(worst, et["rel_l2"])
    return e, worst


def _check_topk(idx, d_cpu):
    want_idx, _, rows = oracle.lightning_indexer(d_cpu.idx_query, d_cpu.idx_query_scale, d_cpu.idx_key_cache,
                                                 d_cpu.idx_key_scale, d_cpu.idx_weight, d_cpu.act_seq,
                                                 d_cpu.block_table, d_cpu.s1)
    tied = 0
    for ti in range(d_cpu.t):
        untied, t_ = oracle.topk_set_diff(idx[ti], want_idx[ti], rows[ti])
        assert untied == 0, f"token {ti}: {untied} selected positions differ on untied scores"
        tied += t_
    return want_idx, rows, tied


def _fused(g, sort=False):
    idx = torch.full((g.t, 1, 2048), -7, dtype=torch.int32, device=DEV)
    out = torch.full((g.b, g.s1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    pto.decode_indexer_attention_quant(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                       g.query_nope, g.query_rope, g.key_nope_2d, g.key_rope_2d, g.k_nope_scales,
                                       g.act_seq_key, g.block_table, idx, out, sort=sort)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    return idx.cpu(), out.cpu()


def _fused_against_oracle(g):
    d = g.to("cpu")
    idx, out = _fused(g)
    want_idx, _, _ = _check_topk(idx, d)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   want_idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    return _check_attention(out, want, d)


def test_config2_full_size_against_oracle_chain():
    """Benchmark configuration 2 as bench.py builds it for rank 0 of 1: same lengths, same seed, data drawn on
    the device. 64 sequences, 2.2 M keys."""
    c = gen.config_act_seq(2)
    g = gen.make_inputs(c["act_seq"], s1=c["s1"], seed=c["seed"], device=DEV)
    assert g.b == 64 and min(g.act_seq) >= 4096 and max(g.act_seq) <= 65536
    e, worst = _fused_against_oracle(g)
    print("config 2:", e, "worst token rel-L2", worst)


def test_config2_rank_shard_is_a_slice_of_the_full_batch():
    """The shard a rank of 8 runs (bench.py --gpus 8: 8 of the 64 sequences, page ids renumbered) gives,
    sequence by sequence, the ordered indices of the full batch on one GPU bit for bit, and its attention
    output up to the rounding of another split of the selected rows over CTAs."""
    c = gen.config_act_seq(2)
    g = gen.make_inputs(c["act_seq"], s1=c["s1"], seed=c["seed"], device=DEV)
    idx_full, out_full = _fused(g, sort=True)
    for rank in (0, 5):
        mine = gen.shard_act_seq(c["act_seq"], rank, 8)
        assert len(mine) == 8
        idx, out = _fused(gen.take_sequences(g, mine), sort=True)
        assert torch.equal(idx, idx_full[mine])
        e = oracle.attention_errors(out, out_full[mine])
        assert e["max_abs"] <= MAX_ABS and e["rel_l2"] <= REL_L2, e


def test_config3_reduced_batch_scores_and_sets_against_oracle():
    """Configuration 3 (131072 keys per sequence, two query tokens with the causal cut between them) at 4
    sequences: fp32 scores of the tensor-core kernel against the oracle's rows, top-k sets exact on untied
    scores, attention of the fused call against the oracle chain."""
    d = gen.make_inputs([131072] * 4, s1=2, seed=1237)
    g = d.to(DEV)
    sc = torch.full((d.t, d.max_blocks * 128), float("nan"), dtype=torch.float32, device=DEV)
    pto.lightning_indexer_scores(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, sc)
    idx, out = _fused(g)
    want_idx, rows, tied = _check_topk(idx, d)
    sc = sc.cpu()
    for ti, row in enumerate(rows):
        torch.testing.assert_close(sc[ti, :row.numel()], row, rtol=3e-6, atol=1e-9)
        assert row.numel() == 131072  # scores cover the whole sequence; the causal cut is applied by the top-k
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   want_idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    _check_attention(out, want, d)


def test_config4_shape_in_small_head_slice_with_many_query_tokens():
    """Configuration 4's real shape, scaled down: one sequence, 64 new query tokens at the end of a 6000-key
    context (query i sees the first S - 63 + i keys), the indexer over all of them, and the attention on a
    device's share of the heads: 16 heads starting at head 32 of arrays that hold all 128. The other heads'
    output rows keep what they held."""
    s1, S, hb = 64, 6000, 32
    d = gen.make_inputs([S], s1=s1, seed=1238)
    g = d.to(DEV)
    idx = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    pto.lightning_indexer_decode(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight,
                                 g.act_seq_key, g.block_table, idx, None, None, 2048)
    out = torch.full((1, s1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    pto.sparse_flash_attention_quant_p(g.query_nope, g.query_rope, g.key_nope_2d, g.key_rope_2d, g.k_nope_scales,
                                       idx.reshape(d.t, 2048), g.block_table, g.act_seq_key, out, 16, 1, SCALE, 2048,
                                       128, d.max_blocks, None, head_begin=hb, nq_total=128)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    want_idx, _, _ = _check_topk(idx.cpu(), d)
    qn = d.query_nope.reshape(d.t, 128, 512)[:, hb:hb + 16].reshape(-1, 512)
    qr = d.query_rope.reshape(d.t, 128, 64)[:, hb:hb + 16].reshape(-1, 64)
    want = oracle.sparse_attention(qn, qr, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales, want_idx.reshape(d.t, 2048),
                                   d.block_table, d.act_seq, s1, nq=16)
    out = out.cpu()
    _check_attention(out[:, :, hb:hb + 16].contiguous(), want, d)
    assert torch.all(out[:, :, :hb] == 7.0) and torch.all(out[:, :, hb + 16:] == 7.0)


# (b, s1, lengths) of the reference's attention system tests and of its example driver; every shape is run
# with the int8 cache and (where the reference does) with the bf16 cache of the same values
TEST1 = [666, 532, 768, 900]
TEST2 = [666, 532, 768, 900, 5698, 2358, 324, 2048]
ATTENTION_CASES = {
    "b4_s2_seq64K": (2, [65536] * 4, ("int8",)),
    "b4_s2_seqTest1": (2, TEST1, ("int8",)),
    "b32_s1_seq511": (1, [511] * 32, ("bf16", "int8")),
    "b1_s1_seq2049": (1, [2049], ("bf16", "int8")),
    "b1_s3_seq2047": (3, [2047], ("bf16", "int8")),
    "b128_s1_seq8k": (1, [8096] * 128, ("bf16", "int8")),
    "b8_s1_seq128k": (1, [131072] * 8, ("bf16", "int8")),
    "b4_s1_seqTest1": (1, TEST1, ("bf16", "int8")),
    "b8_s1_seqTest2": (1, TEST2, ("bf16", "int8")),
    "b8_s4_seqTest2": (4, TEST2, ("bf16", "int8")),
    "example_b4_s2_ragged": (2, [65536, 16381, 666, 15], ("int8",)),
}


@pytest.mark.parametrize("name", list(ATTENTION_CASES))
def test_reference_attention_case_list(name):
    s1, act, kinds = ATTENTION_CASES[name]
    d = gen.make_inputs(act, s1=s1, seed=7000 + len(act) * 10 + s1, with_indexer=False, with_topk=True)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   d.topk_indices, d.block_table, d.act_seq, d.s1)
    g = d.to(DEV)
    outs = {}
    for kind in kinds:
        kn = g.key_nope_2d if kind == "int8" else oracle.dequantised_cache(d.key_nope_2d, d.k_nope_scales).to(DEV)
        out = torch.full((d.b, d.s1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV)
        pto.sparse_flash_attention_quant_d(g.query_nope, g.query_rope, kn, g.key_rope_2d, g.k_nope_scales,
                                           g.topk_indices, g.block_table, g.act_seq_key, out, 128, 1, SCALE, 2048, 128,
                                           d.max_blocks, pto.SaTileShapeConfig())
        torch.cuda.synchronize()
        assert pto.workspace_status()[0] == 0
        outs[kind] = out.cpu()
        _check_attention(outs[kind], want, d)
    if len(outs) == 2:  # same values in the key tiles; two kernels, so equal up to the summation order
        e = oracle.attention_errors(outs["bf16"], outs["int8"])
        assert e["max_abs"] <= MAX_ABS and e["rel_l2"] <= REL_L2, e


FUSED_CASES = {
    "4B_mtp": (2, [768, 4097, 8192, 131071]),
    "4B_mtp_perf": (2, [65536, 65537, 65538, 65539]),
    "32B": (1, [8192] * 32),
}


@pytest.mark.parametrize("name", list(FUSED_CASES))
def test_reference_fused_case_list(name):
    s1, act = FUSED_CASES[name]
    d = gen.make_inputs(act, s1=s1, seed=7100 + len(act))
    _fused_against_oracle(d.to(DEV))


@pytest.mark.parametrize("name,s1,act,dt", [("b4_s2_64k", 2, [65536] * 4, torch.float16),
                                            ("b4_s2_ragged", 2, [768, 4097, 8192, 131071], torch.float16)])
def test_reference_indexer_case_list(name, s1, act, dt):
    """The two indexer system-test shapes, with fp16 scales and weights as the reference generates them; the
    second also in the older formulation its generator belongs to (PTO_LI_FP16_CHAIN)."""
    d = gen.make_inputs(act, s1=s1, seed=7200 + len(name), scale_dtype=dt, with_attention=False)
    g = d.to(DEV)
    idx = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    li = (g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight, g.act_seq_key, g.block_table)
    pto.lightning_indexer_decode(*li, idx, None, None, 2048)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    _check_topk(idx.cpu(), d)
    if name == "b4_s2_ragged":
        pto.lightning_indexer_decode(*li, idx, None, None, 2048, fp16_chain=True)
        torch.cuda.synchronize()
        want_idx, _, rows = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                     d.idx_weight, d.act_seq, d.block_table, d.s1, fp16_chain=True)
        idx_c = idx.cpu()
        for ti in range(d.t):
            untied, _ = oracle.topk_set_diff(idx_c[ti], want_idx[ti], rows[ti])
            assert untied == 0, f"token {ti}"


def test_paged_gather_known_answer_through_the_attention_kernel():
    """The reference's docstring example of the paged gather (6 token rows of 4 values in 3 blocks of 2, block
    table [0, 2, 1], indices [0, 4, 3] -> rows 0, 2, 5) run through the CUDA gather: three sequences share the
    block table, each selects one of the indices, and with a single selected row the softmax weight is 1, so the
    attention output IS the gathered, dequantised row."""
    z = np.load(GOLDEN / "gather_kat.npz")
    param, indices, table = z["param"], z["indices"], z["block_table"]
    bs, n_rows, b = int(z["block_size"]), param.shape[0], len(indices)
    kn = torch.zeros((n_rows, 512), dtype=torch.int8)
    kn[:, :param.shape[1]] = torch.from_numpy(param).to(torch.int8)
    kr = torch.zeros((n_rows, 64), dtype=torch.bfloat16)
    sc = torch.ones((n_rows, 4), dtype=torch.float32)
    gq = torch.Generator().manual_seed(5)
    qn = torch.randn((b * 128, 512), generator=gq).to(torch.bfloat16)
    qr = torch.randn((b * 128, 64), generator=gq).to(torch.bfloat16)
    topk = torch.from_numpy(indices).reshape(b, 1).to(torch.int32)
    bt = torch.from_numpy(table).reshape(1, -1).repeat(b, 1).to(torch.int32).contiguous()
    act = torch.full((b,), n_rows, dtype=torch.int32)
    out = torch.full((b, 1, 128, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    for packed in (False, True):
        if packed:
            cache = gen.pack_kv_rows(kn, kr, sc).to(DEV)
            pto.sparse_attention_antiquant_d(qn.to(DEV), qr.to(DEV), cache, topk.to(DEV), bt.to(DEV), act.to(DEV),
                                             out.reshape(-1, 512), 128, 1, SCALE, 1, bs, bt.shape[1])
        else:
            pto.sparse_flash_attention_quant_d(qn.to(DEV), qr.to(DEV), kn.to(DEV), kr.to(DEV), sc.to(DEV), topk.to(DEV),
                                               bt.to(DEV), act.to(DEV), out, 128, 1, SCALE, 1, bs, bt.shape[1])
        torch.cuda.synchronize()
        assert pto.workspace_status()[0] == 0
        got = out.cpu().float()
        for j in range(b):
            assert np.array_equal(got[j, 0, :, :param.shape[1]].numpy(), np.tile(z["out"][j], (128, 1))), (packed, j)
            assert torch.all(got[j, 0, :, param.shape[1]:] == 0)
        out.fill_(7.0)
