"""Sparse MLA attention on the GPU against the CPU oracle and the reference-made fixtures.
Tolerance (stated by the benchmark): max-abs 2e-2 and relative L2 5e-3 on the bf16 output."""
import pytest
import torch

import oracle
import pypto_b200 as pto
from pypto_b200 import inputs as gen
from golden_util import SFA_CASES, from_np_bf16, load_case, mask_empty_rows

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, REL_L2 = 2e-2, 5e-3
SCALE = 576 ** -0.5


def _run(d, packed=False, prefill=False, nq=128, bf16_cache=False):
    g = d.to(DEV)
    if bf16_cache:  # the non-quantised branch: the cache holds the values the int8 rows dequantise to
        g.key_nope_2d = oracle.dequantised_cache(d.key_nope_2d, d.k_nope_scales).to(DEV)
        g.k_nope_scales = torch.zeros(1, 4, device=DEV)  # not read
    out = torch.full((d.b, d.s1, nq, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    cfg = pto.SaTileShapeConfig()
    if packed:
        cache = gen.pack_kv_rows(g.key_nope_2d, g.key_rope_2d, g.k_nope_scales)
        fn = pto.sparse_attention_antiquant_p if prefill else pto.sparse_attention_antiquant_d
        fn(g.query_nope, g.query_rope, cache, g.topk_indices, g.block_table, g.act_seq_key, out.reshape(-1, 512), nq,
           1, SCALE, 2048, 128, d.max_blocks, cfg)
    else:
        fn = pto.sparse_flash_attention_quant_p if prefill else pto.sparse_flash_attention_quant_d
        fn(pto.from_torch(g.query_nope, dynamic_axis=[0], name="q_nope"), g.query_rope, g.key_nope_2d, g.key_rope_2d,
           g.k_nope_scales, g.topk_indices, g.block_table, g.act_seq_key, out, nq, 1, SCALE, 2048, 128, d.max_blocks,
           cfg)
    torch.cuda.synchronize()
    assert pto.workspace_status()[0] == 0
    return out.cpu()


def _check(got, want):
    e = oracle.attention_errors(got, want)
    assert e["max_abs"] <= MAX_ABS and e["rel_l2"] <= REL_L2, e
    return e


@pytest.mark.parametrize("name", SFA_CASES)
@pytest.mark.parametrize("packed", [False, True], ids=["split_arrays", "packed_rows"])
def test_matches_reference_fixture(name, packed):
    d, z = load_case(name)
    want = mask_empty_rows(from_np_bf16(z["out_no_flash"]).reshape(d.b, d.s1, 128, 512), d)
    got = _run(d, packed=packed)
    _check(got, want)
    # per token too, so that a short row cannot hide behind a long one
    for bi in range(d.b):
        for i in range(d.s1):
            if d.act_seq[bi] - d.s1 + 1 + i > 0:
                _check(got[bi, i], want[bi, i])
            else:
                assert torch.all(got[bi, i] == 0)


def test_config0_against_oracle():
    """Benchmark configuration 0: batch 2, context 8192, 2048 selected rows, split over many CTAs."""
    d = gen.make_config(0)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   d.topk_indices, d.block_table, d.act_seq, d.s1)
    e = _check(_run(d), want)
    print("config0 errors", e)


def test_many_tokens_unsplit_and_prefill_entry():
    """More than 148 (token, head-block) CTAs: the unsplit path that writes bf16 directly."""
    g = torch.Generator().manual_seed(8)
    act = torch.randint(1, 700, (40,), generator=g).tolist()
    d = gen.make_inputs(act, s1=2, seed=21, with_indexer=False, with_topk=True)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   d.topk_indices, d.block_table, d.act_seq, d.s1)
    got = _run(d, prefill=True)
    _check(got, want)
    for bi in range(d.b):
        for i in range(d.s1):
            if act[bi] - 2 + 1 + i > 0:
                _check(got[bi, i], want[bi, i])
            else:
                assert torch.all(got[bi, i] == 0)


def test_head_slice_of_16():
    """16 heads per device, the head-sharded prefill layout."""
    d = gen.make_inputs([3000, 150], s1=1, seed=33, with_indexer=False, with_topk=True, attn_heads=16)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   d.topk_indices, d.block_table, d.act_seq, d.s1, nq=16)
    _check(_run(d, nq=16), want)


def test_order_of_indices_does_not_matter_beyond_rounding():
    d = gen.make_inputs([5000], s1=1, seed=2, with_indexer=False, with_topk=True)
    a = _run(d)
    d.topk_indices = d.topk_indices.flip(-1).contiguous()
    b = _run(d)
    _check(a, b)


@pytest.mark.parametrize("name", SFA_CASES)
def test_bf16_cache_matches_reference_fixture(name):
    """Non-quantised `key_nope_2d` (the golden's is_kn_quant = 0): the reference's output over the bf16
    cache of dequantised values is the fixture's `out_no_flash` itself."""
    d, z = load_case(name)
    assert bool(z["out_bf16_equals_no_flash"])
    want = mask_empty_rows(from_np_bf16(z["out_no_flash"]).reshape(d.b, d.s1, 128, 512), d)
    got = _run(d, bf16_cache=True)
    _check(got, want)
    for bi in range(d.b):
        for i in range(d.s1):
            if d.act_seq[bi] - d.s1 + 1 + i > 0:
                _check(got[bi, i], want[bi, i])
            else:
                assert torch.all(got[bi, i] == 0)
    # the key tiles hold the values the int8 path dequantises to and both caches run the same kernel (only the
    # producers differ): the outputs are equal bit for bit
    assert torch.equal(got, _run(d))


def test_bf16_cache_many_tokens_and_split():
    """Both launch shapes of the bf16 branch: config 0 (2 tokens, split over CTAs) and 80 ragged tokens."""
    d = gen.make_config(0)
    assert torch.equal(_run(d, bf16_cache=True), _run(d))
    g = torch.Generator().manual_seed(18)
    act = torch.randint(1, 900, (40,), generator=g).tolist()
    d = gen.make_inputs(act, s1=2, seed=23, with_indexer=False, with_topk=True)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, oracle.dequantised_cache(d.key_nope_2d, d.k_nope_scales),
                                   d.key_rope_2d, None, d.topk_indices, d.block_table, d.act_seq, d.s1)
    got = _run(d, bf16_cache=True, prefill=True)
    _check(got, want)
    assert torch.equal(got, _run(d))


def test_bf16_cache_head_slice_is_refused():
    d = gen.make_inputs([300], s1=1, seed=3, with_indexer=False, with_topk=True, attn_heads=16)
    with pytest.raises(RuntimeError, match="128 heads"):
        _run(d, nq=16, bf16_cache=True)


@pytest.mark.parametrize("name", SFA_CASES)
def test_packed_rows_equal_split_arrays_bit_for_bit(name):
    """The packed 656-byte rows and the three split arrays hold the same bytes and go through the same kernel."""
    d, _ = load_case(name)
    assert torch.equal(_run(d, packed=True), _run(d, packed=False))
