"""Synthetic input generators, the byte model used by the benchmark, and the batch partition."""
import torch

import oracle
from pypto_b200 import inputs as gen


def test_configs_have_the_benchmark_shapes():
    c0 = gen.config_act_seq(0)
    assert c0["act_seq"] == [8192, 8192] and c0["s1"] == 1
    c1 = gen.config_act_seq(1)
    assert c1["act_seq"] == [32768] * 8
    c2 = gen.config_act_seq(2)
    assert len(c2["act_seq"]) == 64 and min(c2["act_seq"]) >= 4096 and max(c2["act_seq"]) <= 65536
    assert gen.config_act_seq(2)["act_seq"] == c2["act_seq"]  # seeded
    c3 = gen.config_act_seq(3)
    assert c3["act_seq"] == [131072] * 128 and c3["s1"] == 2
    c4 = gen.config_act_seq(4)
    assert c4["act_seq"] == [131072] and c4["s1"] == 4096


def test_block_table_is_a_permutation_with_minus_one_padding():
    d = gen.make_inputs([300, 129, 1], seed=3, with_attention=False)
    used = d.block_table[d.block_table >= 0]
    assert sorted(used.tolist()) == list(range(d.block_num))
    assert d.block_table.shape == (3, 3) and (d.block_table[2, 1:] == -1).all()


def test_value_ranges():
    d = gen.make_inputs([512], seed=9)
    assert int(d.idx_key_cache.min()) >= -127 and int(d.idx_key_cache.max()) <= 127
    assert float(d.k_nope_scales.min()) >= 1e-3 and float(d.k_nope_scales.max()) <= 1e-2
    assert d.query_nope.dtype == torch.bfloat16 and d.idx_weight.dtype == torch.float32


def test_shards_cover_the_batch_once_and_balance_keys():
    act = gen.config_act_seq(2)["act_seq"]
    for world in (2, 4, 8):
        parts = [gen.shard_act_seq(act, r, world) for r in range(world)]
        flat = sorted(i for p in parts for i in p)
        assert flat == list(range(64))
        assert all(len(p) == 64 // world for p in parts)
        loads = [sum(act[i] for i in p) for p in parts]
        assert max(loads) / min(loads) < 1.25


def test_take_sequences_preserves_results():
    d = gen.make_inputs([300, 700, 129, 2500], s1=2, seed=1, with_topk=True)
    sub = gen.take_sequences(d, [3, 1])
    a, _, _ = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale, d.idx_weight,
                                       d.act_seq, d.block_table, 2)
    b, _, _ = oracle.lightning_indexer(sub.idx_query, sub.idx_query_scale, sub.idx_key_cache, sub.idx_key_scale,
                                       sub.idx_weight, sub.act_seq, sub.block_table, 2)
    assert torch.equal(a[6:8], b[0:2]) and torch.equal(a[2:4], b[2:4])
    fa = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                 d.topk_indices, d.block_table, d.act_seq, 2)
    fb = oracle.sparse_attention(sub.query_nope, sub.query_rope, sub.key_nope_2d, sub.key_rope_2d, sub.k_nope_scales,
                                 sub.topk_indices, sub.block_table, sub.act_seq, 2)
    assert torch.equal(fa[3], fb[0]) and torch.equal(fa[1], fb[1])


def test_byte_model():
    d = gen.make_inputs([65536], seed=2, with_attention=True)
    by = gen.algorithmic_bytes(d)
    # per query token at 64K context, fp32 scales: 8.67 MB indexer, 1.63 MB attention
    assert abs(by["indexer"] - 8.67e6) < 0.05e6
    assert abs(by["attention"] - 1.63e6) < 0.02e6
    assert gen.score_stage_bytes(d) == 65536 * 132 + 8192 + 64 * 8 + 4 * 512


def test_take_sequences_with_a_permuted_page_order_holds_the_same_data():
    """`permute_seed` renumbers the copied pages in a random order (the block table stays a permutation, as
    the benchmark configurations ask); what the table points at is unchanged."""
    d = gen.make_inputs([300, 700, 129, 1000], s1=1, seed=12)
    a = gen.take_sequences(d, [3, 1])
    b = gen.take_sequences(d, [3, 1], permute_seed=99)
    assert a.act_seq == b.act_seq == [1000, 700]
    assert not torch.equal(a.block_table, b.block_table)
    used = b.block_table[b.block_table >= 0]
    assert sorted(used.tolist()) == list(range(b.block_num))
    for j in range(2):
        n = (a.act_seq[j] + 127) // 128
        pa, pb = a.block_table[j, :n].long(), b.block_table[j, :n].long()
        assert torch.equal(a.idx_key_cache[pa], b.idx_key_cache[pb])
        assert torch.equal(a.idx_key_scale[pa], b.idx_key_scale[pb])
        ra = (pa[:, None] * 128 + torch.arange(128)[None, :]).reshape(-1)
        rb = (pb[:, None] * 128 + torch.arange(128)[None, :]).reshape(-1)
        assert torch.equal(a.key_nope_2d[ra], b.key_nope_2d[rb])
        assert torch.equal(a.k_nope_scales[ra], b.k_nope_scales[rb])
    assert torch.equal(a.idx_query, b.idx_query)
