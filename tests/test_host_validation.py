"""Host-side validation of the operator wrappers: every bad call is refused with a Python exception
before anything is launched (failures are injected on the host only)."""
import pytest
import torch

import pypto_b200 as pto
from pypto_b200 import inputs as gen


@pytest.fixture(scope="module")
def d():
    return gen.make_inputs([300, 129], s1=1, seed=1, with_topk=True)


def li_args(d, **over):
    a = dict(idx_query=d.idx_query, idx_query_scale=d.idx_query_scale, idx_key_cache=d.idx_key_cache,
             idx_key_scale=d.idx_key_scale, idx_weight=d.idx_weight, act_seq_key=d.act_seq_key,
             block_table=d.block_table, topk_res=torch.zeros((d.t, 1, 2048), dtype=torch.int32))
    a.update(over)
    return list(a.values()) + [None, None, 2048]


def sfa_args(d, **over):
    a = dict(query_nope=d.query_nope, query_rope=d.query_rope, key_nope_2d=d.key_nope_2d, key_rope_2d=d.key_rope_2d,
             k_nope_scales=d.k_nope_scales, topk_indices=d.topk_indices, block_table=d.block_table,
             kv_act_seqs=d.act_seq_key, attention_out=torch.zeros((d.b, 1, 128, 512), dtype=torch.bfloat16))
    a.update(over)
    return list(a.values()) + [128, 1, 576 ** -0.5, 2048, 128, d.max_blocks, None]


def test_from_torch_mirrors_the_reference_rules():
    t = torch.zeros(4, 6)
    h = pto.from_torch(t, name="x", dynamic_axis=[0])
    assert h.shape == [-1, 6] and h.ori_shape == [4, 6] and h.data_ptr == t.data_ptr() and h.dtype == torch.float32
    with pytest.raises(TypeError):
        pto.from_torch([1, 2, 3])
    with pytest.raises(RuntimeError, match="not all tensors are contiguous"):
        pto.from_torch(t.t())
    assert pto.from_torch(torch.tensor(3.0)).shape == [1]


def test_cpu_tensors_are_refused_there_is_no_cpu_path(d):
    with pytest.raises(RuntimeError, match="no CPU path"):
        pto.lightning_indexer_decode(*li_args(d))
    with pytest.raises(RuntimeError, match="no CPU path"):
        pto.sparse_flash_attention_quant_d(*sfa_args(d))


@pytest.mark.parametrize("field,bad,exc", [
    ("idx_query", lambda d: d.idx_query.to(torch.int32), ValueError),
    ("idx_query", lambda d: d.idx_query[:, :32].contiguous(), ValueError),
    ("idx_query_scale", lambda d: d.idx_query_scale.to(torch.float16), ValueError),  # mixed scale dtypes
    ("idx_key_cache", lambda d: d.idx_key_cache.reshape(-1, 128), ValueError),
    ("idx_weight", lambda d: d.idx_weight[:, :10].contiguous(), ValueError),
    ("act_seq_key", lambda d: d.act_seq_key.to(torch.int64), ValueError),
    ("block_table", lambda d: d.block_table[:1].contiguous(), ValueError),
    ("topk_res", lambda d: torch.zeros((d.t, 1, 100), dtype=torch.int32), ValueError),
    ("idx_query", lambda d: d.idx_query.transpose(1, 2), RuntimeError),  # non-contiguous
    ("idx_query", lambda d: "not a tensor", TypeError),
])
def test_indexer_rejects_bad_arguments(d, field, bad, exc):
    with pytest.raises(exc):
        pto.lightning_indexer_decode(*li_args(d, **{field: bad(d)}))


@pytest.mark.parametrize("field,bad,exc", [
    ("query_nope", lambda d: d.query_nope.to(torch.float16), ValueError),
    ("query_rope", lambda d: d.query_rope[:, :32].contiguous(), ValueError),
    ("key_nope_2d", lambda d: d.key_nope_2d.to(torch.float16), ValueError),  # int8 or bfloat16 only
    ("k_nope_scales", lambda d: d.k_nope_scales[:, :2].contiguous(), ValueError),
    ("topk_indices", lambda d: d.topk_indices.to(torch.int64), ValueError),
    ("kv_act_seqs", lambda d: d.act_seq_key.float(), ValueError),
    ("attention_out", lambda d: torch.zeros((d.b, 1, 128, 256), dtype=torch.bfloat16), ValueError),
    ("block_table", lambda d: d.block_table.t(), RuntimeError),
])
def test_attention_rejects_bad_arguments(d, field, bad, exc):
    with pytest.raises(exc):
        pto.sparse_flash_attention_quant_d(*sfa_args(d, **{field: bad(d)}))


def test_scalar_arguments(d):
    a = sfa_args(d)
    a[10] = 2  # n_kv
    with pytest.raises(ValueError):
        pto.sparse_flash_attention_quant_p(*a)
    a = li_args(d)
    a[-1] = 4096  # selected_count
    a[7] = torch.zeros((d.t, 1, 4096), dtype=torch.int32)
    with pytest.raises(ValueError):
        pto.lightning_indexer_decode(*a)


def test_packed_cache_shape(d):
    cache = gen.pack_kv_rows(d.key_nope_2d, d.key_rope_2d, d.k_nope_scales)
    assert cache.shape == (d.block_num * 128, 656)
    with pytest.raises(ValueError):
        pto.sparse_attention_antiquant_d(d.query_nope, d.query_rope, cache[:, :640].contiguous(), d.topk_indices,
                                         d.block_table, d.act_seq_key,
                                         torch.zeros((d.t * 128, 512), dtype=torch.bfloat16), 128, 1, 0.04, 2048, 128,
                                         d.max_blocks, None)


def test_tiling_dataclasses_are_accepted_and_inert():
    c = pto.LightningIndexerConfigs()
    assert c.extend_param["scale"] == 1 / 2048.0
    s = pto.SaTileShapeConfig(g_tile=128, s_kv_tile=2048, c1_tile_shape=[128] * 6, v1_tile_shape=[8, 2048],
                              c2_tile_shape=[128] * 6, v2_tile_shape=[64, 128])
    assert s.s_kv_tile == 2048


def test_prolog_rejects_bad_arguments_before_any_launch():
    p = gen.make_prolog_inputs([200], s1=1, seed=1)
    t = 1
    outs = [torch.zeros(t, 128, 512, dtype=torch.bfloat16), torch.zeros(t, 128, 64, dtype=torch.bfloat16),
            p["kv_cache"], p["kr_cache"], p["kv_scale_cache"], torch.zeros(t, 64, 128, dtype=torch.int8),
            torch.zeros(t, 64, 1, dtype=torch.float16), p["idx_k_cache"], p["idx_k_scale_cache"],
            torch.zeros(t, 64, dtype=torch.float16)]
    names = ["token_x", "w_dq", "w_uqqr", "w_qb_scale", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin",
             "cache_index", "kv_cache", "kr_cache", "kv_scale_cache", "w_idx_qb", "w_idx_qb_scale", "w_idx_k",
             "w_idx_proj", "ln_gamma", "ln_beta", "hadamard_q", "hadamard_k", "idx_k_cache", "idx_k_scale_cache"]
    tail = [1e-5, 1e-5, "PA_BSND", None, None, None, None]

    def call(**over):
        ins = [over.get(n, p[n]) for n in names]
        return pto.mla_indexer_prolog_quant_d(*ins, *outs, *tail)

    with pytest.raises(RuntimeError, match="no CPU path"):
        call()  # CPU tensors: there is no CPU path
    with pytest.raises(ValueError, match="token_x"):
        call(token_x=p["token_x"].float())
    with pytest.raises(ValueError, match="mla_w_uq_qr"):
        call(w_uqqr=p["w_uqqr"][:, :100].contiguous())
    with pytest.raises(ValueError, match="cache_index"):
        call(cache_index=p["cache_index"].to(torch.int32))
    with pytest.raises(ValueError, match="PA_BSND"):
        pto.mla_indexer_prolog_quant_d(*[p[n] for n in names], *outs, 1e-5, 1e-5, "BSND", None, None, None, None)


def test_nonquant_prolog_rejects_bad_arguments_before_any_launch():
    p = gen.make_prolog_nonquant_inputs([200], s1=1, seed=1)
    bf = torch.bfloat16
    outs = [torch.zeros(1, 128, 512, dtype=bf), torch.zeros(1, 128, 64, dtype=bf), torch.zeros(1, 64, 128, dtype=bf),
            torch.zeros(1, 64, dtype=bf)]
    names = ["token_x", "w_dq", "w_uqqr", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin", "cache_index",
             "kv_cache", "kr_cache", "w_idx_qb", "w_idx_k", "w_idx_proj", "ln_gamma", "ln_beta", "idx_k_cache"]

    def call(*tail, **over):
        return pto.mla_indexer_prolog(*[over.get(n, p[n]) for n in names], *outs, *tail)

    with pytest.raises(RuntimeError, match="no CPU path"):
        call()
    with pytest.raises(ValueError, match="w_uq_qr"):
        call(w_uqqr=p["w_uqqr"].to(torch.int8))
    with pytest.raises(ValueError, match="kv_cache"):
        call(kv_cache=p["kv_cache"].to(torch.int8))
    with pytest.raises(ValueError, match="idx_k_cache"):
        call(idx_k_cache=p["idx_k_cache"][:-1].contiguous())
    with pytest.raises(ValueError, match="cache_index"):
        call(cache_index=p["cache_index"].to(torch.int32))
    with pytest.raises(ValueError, match="PA_BSND"):
        call(1e-5, 1e-5, "BSND")
