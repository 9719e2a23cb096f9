"""The `torch.library` registration of the operators: schemas, traceability without a device, and on the GPU a
compiled module (no graph break) that gives the eager operator's result, also when recorded into a CUDA graph."""
import pytest
import torch

import pypto_b200.torch_ops as top
from pypto_b200 import inputs as gen


def test_schemas_name_the_buffers_each_op_writes():
    ns = torch.ops.pypto_b200
    want = {
        "lightning_indexer_decode": {"topk_res"},
        "sparse_flash_attention_quant": {"attention_out"},
        "sparse_attention_antiquant": {"attention_out"},
        "decode_indexer_attention_quant": {"topk_res", "attention_out"},
        "lightning_indexer_topk_nonquant": {"topk_res"},
        "decode_indexer_attention": {"topk_res", "attention_out"},
        "mla_indexer_prolog_quant": set(top._PROLOG_OUT),
        "mla_indexer_prolog": {"kv_cache", "kr_cache", "idx_k_cache", "query_nope_out", "query_rope_out",
                               "idx_query_out", "idx_weights_out"},
    }
    for name, written in want.items():
        schema = getattr(ns, name).default._schema
        got = {a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write}
        assert got == written, (name, got)
        assert len(schema.returns) == 0


def test_traces_under_fake_tensors_without_a_device():
    """What `torch.compile` does first: run the model on fake tensors. No kernel may be reached."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        t, blocks = 4, 9
        i8, bf, f16, i32 = torch.int8, torch.bfloat16, torch.float16, torch.int32
        q = torch.empty(t, 64, 128, dtype=i8)
        qs = torch.empty(t, 64, dtype=f16)
        kc = torch.empty(blocks, 128, 1, 128, dtype=i8)
        ks = torch.empty(blocks, 128, 1, dtype=f16)
        w = torch.empty(t, 64, dtype=f16)
        act = torch.empty(t, dtype=i32)
        bt = torch.empty(t, 3, dtype=i32)
        idx = torch.empty(t, 1, 2048, dtype=i32)
        assert torch.ops.pypto_b200.lightning_indexer_decode(q, qs, kc, ks, w, act, bt, idx) is None
        qn = torch.empty(t * 128, 512, dtype=bf)
        qr = torch.empty(t * 128, 64, dtype=bf)
        kn = torch.empty(blocks * 128, 512, dtype=i8)
        kr = torch.empty(blocks * 128, 64, dtype=bf)
        sc = torch.empty(blocks * 128, 4)
        out = torch.empty(t, 1, 128, 512, dtype=bf)
        assert torch.ops.pypto_b200.decode_indexer_attention_quant(q, qs, kc, ks, w, qn, qr, kn, kr, sc, act, bt, idx,
                                                                   out) is None


def test_real_cpu_tensors_are_refused_loudly():
    """No CPU fallback behind the registration: host tensors reach the operator's own device check."""
    d = gen.make_inputs([300], s1=1, seed=5)
    idx = torch.zeros((1, 1, 2048), dtype=torch.int32)
    with pytest.raises(RuntimeError):
        torch.ops.pypto_b200.lightning_indexer_decode(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                                      d.idx_weight, d.act_seq_key, d.block_table, idx)


class _Layer(torch.nn.Module):
    """A model step that calls the fused operator between two ordinary torch ops."""

    def forward(self, g_args, idx, out, bias):
        torch.ops.pypto_b200.decode_indexer_attention_quant(*g_args, idx, out, 128, 576 ** -0.5, 2048, True, False)
        return out.float() + bias, idx


@pytest.mark.gpu
def test_compiled_module_matches_eager_and_captures_into_a_cuda_graph():
    import pypto_b200 as pto

    dev = "cuda"
    d = gen.make_inputs([5000, 3000, 700, 64], s1=1, seed=31)
    g = d.to(dev)
    args = (g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale, g.idx_weight, g.query_nope, g.query_rope,
            g.key_nope_2d, g.key_rope_2d, g.k_nope_scales, g.act_seq_key, g.block_table)
    idx_e = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=dev)
    out_e = torch.zeros((d.b, d.s1, 128, 512), dtype=torch.bfloat16, device=dev)
    pto.decode_indexer_attention_quant(*args, idx_e, out_e, sort=True)
    bias = torch.full((1,), 0.5, device=dev)

    model = torch.compile(_Layer(), backend="eager", fullgraph=True)  # fullgraph: a graph break would raise
    idx_c = torch.zeros_like(idx_e)
    out_c = torch.zeros_like(out_e)
    y, idx_r = model(args, idx_c, out_c, bias)
    torch.cuda.synchronize()
    assert torch.equal(idx_c, idx_e) and torch.equal(out_c, out_e)
    assert torch.equal(y, out_e.float() + 0.5) and idx_r.data_ptr() == idx_c.data_ptr()

    # the compiled model inside a CUDA graph (the reference's capture-and-replay mode around torch.compile)
    idx_c.fill_(-3)
    out_c.fill_(1.0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model(args, idx_c, out_c, bias)  # warm-up on the capture stream: its workspace exists before the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        y_g, _ = model(args, idx_c, out_c, bias)
    idx_c.fill_(-3)
    out_c.fill_(1.0)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(idx_c, idx_e) and torch.equal(out_c, out_e) and torch.equal(y_g, out_e.float() + 0.5)


@pytest.mark.gpu
def test_stage_ops_through_the_registration():
    import oracle

    dev = "cuda"
    d = gen.make_inputs([3000, 150], s1=1, seed=33)
    g = d.to(dev)
    idx = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=dev)
    torch.ops.pypto_b200.lightning_indexer_decode(g.idx_query, g.idx_query_scale, g.idx_key_cache, g.idx_key_scale,
                                                  g.idx_weight, g.act_seq_key, g.block_table, idx)
    out = torch.zeros((d.b, d.s1, 128, 512), dtype=torch.bfloat16, device=dev)
    torch.ops.pypto_b200.sparse_flash_attention_quant(g.query_nope.reshape(-1, 512), g.query_rope.reshape(-1, 64),
                                                      g.key_nope_2d, g.key_rope_2d, g.k_nope_scales, idx, g.block_table,
                                                      g.act_seq_key, out, 128, 1, 576 ** -0.5, 2048, 128, d.max_blocks)
    out_p = torch.zeros_like(out)
    cache = gen.pack_kv_rows(g.key_nope_2d, g.key_rope_2d, g.k_nope_scales)
    torch.ops.pypto_b200.sparse_attention_antiquant(g.query_nope.reshape(-1, 512), g.query_rope.reshape(-1, 64), cache,
                                                    idx, g.block_table, g.act_seq_key, out_p, 128, 1, 576 ** -0.5, 2048,
                                                    128, d.max_blocks)
    torch.cuda.synchronize()
    assert torch.equal(out, out_p)
    want = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   idx.cpu().reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    e = oracle.attention_errors(out.cpu(), want)
    assert e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3, e
