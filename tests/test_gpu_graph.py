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
