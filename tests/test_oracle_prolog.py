"""The prolog oracle against the outputs of the reference's torch goldens (fixtures made by
tests/golden/make_golden.py from `mla_prolog_quant_v32_compute` and `indexer_prolog`)."""
import numpy as np
import pytest
import torch

from oracle import prolog_oracle as po
from golden_util import (PROLOG_CASES, PROLOG_HEADS, PROLOG_NONQUANT_CASES, from_np_bf16, load_prolog_case,
                         load_prolog_nonquant_case, sha)


def _same_or_close(got, want, name, rel=1e-3):
    """Bit-identical where the host's BLAS sums in the order the fixture's did; otherwise within a rounding."""
    if torch.equal(got, want):
        return
    g, w = got.to(torch.float32), want.to(torch.float32)
    err = float((g - w).norm() / w.norm().clamp_min(1e-30))
    assert err < rel, (name, err)


@pytest.mark.parametrize("name", PROLOG_CASES)
def test_prolog_oracle_matches_reference_goldens(name):
    p, z = load_prolog_case(name)
    o = po.mla_indexer_prolog(p)  # eps 0 = the goldens' RMSNorm
    idx = p["cache_index"]
    t = idx.numel()
    _same_or_close(o["q_nope"][:, list(PROLOG_HEADS), :], from_np_bf16(z["q_nope_heads"]), "q_nope")
    _same_or_close(o["q_rope"], from_np_bf16(z["q_rope"]), "q_rope")
    _same_or_close(o["q_norm_scale"].reshape(t), torch.from_numpy(z["q_norm_scale"]), "q_norm_scale", 1e-6)
    _same_or_close(o["kr_cache"][idx], from_np_bf16(z["kr_rows"]), "kr rows")
    _same_or_close(o["kv_scale_cache"][idx], torch.from_numpy(z["kv_scale_rows"]), "kv scales", 1e-6)
    _same_or_close(o["q_scale"].reshape(t, 64), torch.from_numpy(z["q_scale"]), "q_scale")
    _same_or_close(o["idx_k_scale_cache"].reshape(-1)[idx], torch.from_numpy(z["idx_k_scale_rows"]), "k_scale")
    _same_or_close(o["weights"], torch.from_numpy(z["weights"]), "weights")
    # int8 outputs: a different summation order may move a value across a rounding boundary, by one step
    for key, want in (("q_norm", z["q_norm"]), ("q_int8", z["q_int8"])):
        d = (o[key].to(torch.int32) - torch.from_numpy(want).to(torch.int32)).abs()
        assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 1e-3, key
    for key, rows in (("kv_cache", z["kv_rows"]), ("idx_k_cache", z["idx_k_rows"])):
        d = (o[key][idx].to(torch.int32) - torch.from_numpy(rows).to(torch.int32)).abs()
        assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 1e-3, key
    # rows the operator did not write are untouched
    keep = torch.ones(p["kv_cache"].shape[0], dtype=torch.bool)
    keep[idx] = False
    for key in ("kv_cache", "kr_cache", "kv_scale_cache", "idx_k_cache", "idx_k_scale_cache"):
        assert torch.equal(o[key][keep], p[key][keep]), key
    # on this host the restatement is expected to be bit-identical; report when it is
    same = {k: sha(o[k]) == str(z[f"{k}_sha"]) for k in ("q_nope", "kv_cache", "kr_cache", "kv_scale_cache",
                                                          "idx_k_cache", "idx_k_scale_cache")}
    print(name, "digests equal:", same)


@pytest.mark.parametrize("name", PROLOG_NONQUANT_CASES)
def test_nonquant_prolog_oracle_matches_reference_goldens(name):
    """`mla_prolog_compute` without quantisation (numpy, ml_dtypes) and the non-quantised `indexer_prolog` (torch) of
    the reference's system tests, chained; the fixture keeps their outputs."""
    p, z = load_prolog_nonquant_case(name)
    o = po.mla_indexer_prolog_nonquant(p)
    idx = p["cache_index"]
    _same_or_close(o["q_norm"], from_np_bf16(z["q_norm"]), "q_norm")
    _same_or_close(o["q_nope"][:, list(PROLOG_HEADS), :], from_np_bf16(z["q_nope_heads"]), "q_nope")
    _same_or_close(o["q_rope"], from_np_bf16(z["q_rope"]), "q_rope")
    _same_or_close(o["kv_cache"][idx], from_np_bf16(z["kv_rows"]), "kv rows")
    _same_or_close(o["kr_cache"][idx], from_np_bf16(z["kr_rows"]), "kr rows")
    _same_or_close(o["idx_query"], from_np_bf16(z["idx_query"]), "idx_query")
    _same_or_close(o["idx_k_cache"][idx], from_np_bf16(z["idx_k_rows"]), "idx k rows")
    _same_or_close(o["weights"], from_np_bf16(z["weights"]), "weights")
    keep = torch.ones(p["kv_cache"].shape[0], dtype=torch.bool)
    keep[idx] = False
    for key in ("kv_cache", "kr_cache", "idx_k_cache"):
        assert torch.equal(o[key][keep], p[key][keep]), key
    same = {k: sha(o[k]) == str(z[f"{k}_sha"]) for k in ("q_nope", "kv_cache", "kr_cache", "idx_k_cache")}
    print(name, "digests equal:", same)


def test_quant_rows_rounding_chain():
    """round-half-even, then fp16, then truncation (deepseekv32_mla_indexer_prolog_quant.py:35-53)."""
    x = torch.tensor([[127.0, 63.5, -63.5, 0.5, 1.5, -2.5, 126.49, -127.0]])
    q, s = po.quant_rows(x)
    assert q.tolist() == [[127, 64, -64, 0, 2, -2, 126, -127]]
    assert float(s) == pytest.approx(1.0)
    q, s = po.quant_rows(torch.tensor([[0.02, -0.01]]))
    assert q.tolist() == [[127, -64]] and float(s) == pytest.approx(0.02 / 127, rel=1e-6)


def test_rope_layouts():
    """The MLA rope de-interleaves (even dims first), the indexer rope does not."""
    x = torch.arange(8, dtype=torch.float32).reshape(1, 1, 8).to(torch.bfloat16)
    one, zero = torch.ones(1, 8, dtype=torch.bfloat16), torch.zeros(1, 8, dtype=torch.bfloat16)
    assert po.rope_interleaved(x, one, zero).flatten().tolist() == [0, 2, 4, 6, 1, 3, 5, 7]
    assert po.rope_interleaved(x, zero, one).flatten().tolist() == [-1, -3, -5, -7, 0, 2, 4, 6]
    assert po.rope_halves(x, zero, one).flatten().tolist() == [-4, -5, -6, -7, 0, 1, 2, 3]
