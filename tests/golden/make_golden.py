#!/usr/bin/env python3
"""Generate the committed golden vectors by running the REFERENCE's own torch goldens.

Run once, where the reference checkout is available ($PYPTO_REFERENCE, default: a directory
`reference` next to this repository):

    python tests/golden/make_golden.py

The reference's example drivers import `torch_npu` and `pypto` at module level; neither exists
off an Ascend host, so permissive stub modules are installed in `sys.modules` first. Only the
drivers' pure-torch golden functions are called:

  * lightning_indexer_compute  (examples/models/deepseek_v32_exp/deepseekv32_lightning_indexer_quant.py:184-269)
  * its ST twin that also returns first_mm / mm_out
    (framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_lightning_indexer.py:282-360)
  * indexer_topk_compute(is_quant=False), the non-quantised indexer   (same ST file, :189-279)
  * compute_attention_no_flash / compute_attention
    (examples/models/deepseek_v32_exp/deepseekv32_sparse_flash_attention_quant.py:169-254, :49-166)
  * compute_attention_aq       (examples/models/deepseek_v32_exp/deepseekv32_sparse_attention_antiquant.py:49-136)
  * mla_prolog_compute without quantisation (numpy + ml_dtypes;
    framework/tests/st/operator/src/test_deepseek_v3.2_exp/gen_mla_prolog_golden_v32.py:176-303) and the
    non-quantised indexer_prolog (.../gen_lightning_indexer_prolog.py:253-293), chained as
    .../gen_decode_indexer_attention.py:195-262 chains them

Inputs come from `pypto_b200.inputs.make_inputs` (seeded); each fixture stores the seed, a sha256
of every input tensor and the reference's outputs, so the tests regenerate identical inputs
without the reference being present.
"""
from __future__ import annotations

import hashlib
import importlib
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from pypto_b200 import inputs as gen  # noqa: E402

REF = Path(os.environ.get("PYPTO_REFERENCE", str(ROOT.parent / "reference")))


class _Anything(types.ModuleType):
    """Module stub: any attribute is another stub; calling it works as a pass-through decorator."""

    def __getattr__(self, name):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        child = _Anything(f"{self.__name__}.{name}")
        setattr(self, name, child)
        return child

    def __call__(self, *args, **kwargs):
        if len(args) == 1 and callable(args[0]) and not kwargs:
            return args[0]
        return self

    def __mro_entries__(self, bases):
        return (object,)


def load_reference():
    for name in ("torch_npu", "pypto", "pypto.experimental", "pypto.operation", "pypto.pypto_impl",
                 "common_func", "golden_register", "ml_dtypes"):
        if name == "ml_dtypes":
            try:
                importlib.import_module(name)
                continue
            except ImportError:
                pass
        sys.modules[name] = _Anything(name)
    sys.path.insert(0, str(REF / "examples/models/deepseek_v32_exp"))
    sys.path.insert(0, str(REF / "framework/tests/st/operator/src/test_deepseek_v3.2_exp"))
    li = importlib.import_module("deepseekv32_lightning_indexer_quant")
    sfa = importlib.import_module("deepseekv32_sparse_flash_attention_quant")
    aq = importlib.import_module("deepseekv32_sparse_attention_antiquant")
    st_li = importlib.import_module("gen_lightning_indexer")
    return li, sfa, aq, st_li


def sha(t: torch.Tensor) -> str:
    raw = t.contiguous().view(torch.uint8).numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()


def input_hashes(d: gen.DecodeInputs):
    return {k: sha(v) for k, v in sorted(d.tensors().items())}


def as_np(t: torch.Tensor):
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.numpy()


LI_CASES = {
    # name: (act_seq, s1, scale dtype)
    "li_ragged_f32": ([15, 666, 2049, 4100], 1, "float32"),
    "li_mtp_f16": ([129, 2500, 3000], 2, "float16"),
    "li_short_f16": ([1, 2048, 2047], 2, "float16"),
}
SFA_CASES = {
    "sfa_ragged_mtp": ([2500, 700, 1], 2),
    "sfa_single": ([2300], 1),
}


def make_li(li_mod, st_mod, name, act_seq, s1, dt):
    dtype = getattr(torch, dt)
    seed = 7000 + sum(act_seq) + s1
    d = gen.make_inputs(act_seq, s1=s1, seed=seed, scale_dtype=dtype, with_attention=False)
    params = dict(block_size=128, selected_count=2048, b=d.b, s1=s1, n1=64, d=128, block_num=d.block_num,
                  max_block_num=d.max_blocks)
    data = dict(query=d.idx_query.reshape(d.b, s1, 64, 128), key=d.idx_key_cache, q_scale=d.idx_query_scale,
                k_scale=d.idx_key_scale, weights=d.idx_weight, act_seq=d.act_seq_key, block_table=d.block_table)
    topk = li_mod.lightning_indexer_compute(dict(data), params).reshape(d.t, 1, 2048)
    first_mm, mm_out, topk_value, topk2 = st_mod.lightning_indexer_compute(dict(data), params)
    assert torch.equal(topk.reshape(-1), topk2.reshape(-1).to(torch.int32)), "example and ST goldens disagree"
    extra = {}
    if dtype == torch.float16:
        # the older formulation (fp16 chain between the dot and the head sum) on the same inputs: the ST golden
        # of LightningIndexerTopkImpl, quantised branch
        _, chain_topk, chain_rows = st_mod.indexer_topk_compute(dict(data), dict(params, n2=1), True)
        extra = dict(chain_topk_res=chain_topk.reshape(d.t, 1, 2048).numpy().astype(np.int32),
                     chain_rows=chain_rows.numpy().astype(np.float32))
    np.savez_compressed(
        HERE / f"{name}.npz",
        act_seq=np.array(act_seq, dtype=np.int32), s1=np.int32(s1), seed=np.int64(seed), scale_dtype=dt,
        hashes=np.array([f"{k}={v}" for k, v in input_hashes(d).items()]),
        topk_res=topk.numpy().astype(np.int32),
        mm_out=mm_out.numpy().astype(np.float32),
        first_mm_sha=sha(first_mm),
        first_mm_head0=first_mm.reshape(d.t, 64, -1)[:, 0, :].numpy(),
        **extra,
    )
    print(name, "t", d.t, "blocks", d.block_num)


NONQUANT_CASES = {
    # name: (act_seq, s1)
    "li_nonquant_mtp": ([129, 2500, 3000], 2),
    "li_nonquant_ragged": ([15, 666, 2049, 4100], 1),
}


def make_li_nonquant(st_mod, name, act_seq, s1):
    """The ST golden of LightningIndexerTopkImpl with isQuant = false on bf16 inputs of
    `pypto_b200.inputs.make_nonquant_inputs`."""
    seed = 13000 + sum(act_seq) + s1
    d = gen.make_nonquant_inputs(act_seq, s1=s1, seed=seed, with_attention=False)
    params = dict(block_size=128, selected_count=2048, b=d.b, s1=s1, n1=64, d=128, n2=1, block_num=d.block_num,
                  max_block_num=d.max_blocks)
    data = dict(query=d.idx_query.reshape(d.b, s1, 64, 128), key=d.idx_key_cache, weights=d.idx_weight,
                act_seq=d.act_seq_key, block_table=d.block_table)
    _, topk, rows = st_mod.indexer_topk_compute(dict(data), params, False)
    np.savez_compressed(
        HERE / f"{name}.npz",
        act_seq=np.array(act_seq, dtype=np.int32), s1=np.int32(s1), seed=np.int64(seed),
        hashes=np.array([f"{k}={v}" for k, v in input_hashes(d).items()]),
        topk_res=topk.reshape(d.t, 1, 2048).numpy().astype(np.int32),
        rows=rows.numpy().astype(np.float32),
    )
    print(name, "t", d.t, "blocks", d.block_num)


def make_sfa(sfa_mod, aq_mod, name, act_seq, s1):
    seed = 9000 + sum(act_seq) + s1
    d = gen.make_inputs(act_seq, s1=s1, seed=seed, with_indexer=False, with_topk=True)
    q = torch.cat([d.query_nope.reshape(d.b, s1, 128, 512), d.query_rope.reshape(d.b, s1, 128, 64)], dim=-1)
    scale = 576 ** -0.5
    data = [q, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales, d.topk_indices, d.block_table, list(act_seq)]
    params = [128, scale, 2048, 512, 1]
    out_nf, _ = sfa_mod.compute_attention_no_flash(data, params, 2048)
    out_fl, _ = sfa_mod.compute_attention(data, params, 2048)
    # non-quantised branch (is_kn_quant = 0) over the bf16 cache holding the dequantised values
    kn_bf16 = (d.key_nope_2d.to(torch.float32).reshape(-1, 4, 128) * d.k_nope_scales.reshape(-1, 4, 1)
               ).reshape(-1, 512).to(torch.bfloat16)
    out_bf, _ = sfa_mod.compute_attention_no_flash(
        [q, kn_bf16, d.key_rope_2d, d.k_nope_scales, d.topk_indices, d.block_table, list(act_seq)],
        [128, scale, 2048, 512, 0], 2048)
    packed = gen.pack_kv_rows(d.key_nope_2d, d.key_rope_2d, d.k_nope_scales)
    out_aq, _ = aq_mod.compute_attention_aq(
        [d.query_nope, d.query_rope, packed, d.topk_indices, d.block_table, list(act_seq)],
        [128, 128, scale, 2048, 512, 64], 2048)
    np.savez_compressed(
        HERE / f"{name}.npz",
        act_seq=np.array(act_seq, dtype=np.int32), s1=np.int32(s1), seed=np.int64(seed),
        hashes=np.array([f"{k}={v}" for k, v in input_hashes(d).items()]),
        out_no_flash=as_np(out_nf),
        # the packed-row golden and the single-tile online golden are stored as digests plus one head
        out_packed_sha=sha(out_aq), out_packed_equals_no_flash=bool(torch.equal(out_aq, out_nf)),
        out_flash_sha=sha(out_fl), out_flash_head0=as_np(out_fl[:, :, 0, :]),
        out_bf16_sha=sha(out_bf), out_bf16_equals_no_flash=bool(torch.equal(out_bf, out_nf)),
    )
    print(name, "t", d.t, "rows", d.block_num * 128)


PROLOG_CASES = {
    # name: (act_seq, s1)
    "prolog_mtp": ([300, 131], 2),
    "prolog_single": ([129, 1, 640], 1),
}
PROLOG_HEADS = (0, 37, 127)  # heads of q_nope kept in full; the whole tensor is kept as a digest


def make_prolog(pro_mod, name, act_seq, s1):
    """Runs the reference's two torch goldens (`mla_prolog_quant_v32_compute`, then `indexer_prolog` on its
    q_norm outputs, as gen_test_data does, deepseekv32_mla_indexer_prolog_quant.py:617-712) on inputs of
    `pypto_b200.inputs.make_prolog_inputs`, reshaped to the [b, s, ...] layouts the goldens take."""
    seed = 11000 + sum(act_seq) + s1
    p = gen.make_prolog_inputs(act_seq, s1=s1, seed=seed)
    b, t = len(act_seq), len(act_seq) * s1
    rows = p["kv_cache"].shape[0]
    nb = rows // 128
    mla_in = dict(dtype=torch.bfloat16, is_quant_a=False, is_quant_b=True, has_smooth=False,
                  gamma_cq=p["gamma_cq"], gamma_ckv=p["gamma_ckv"], x=p["token_x"].reshape(b, s1, -1),
                  w_dq=p["w_dq"], w_uqqr=p["w_uqqr"], w_uk=p["w_uk"], w_dkvkr=p["w_dkvkr"],
                  cos=p["cos"].reshape(b, s1, -1), sin=p["sin"].reshape(b, s1, -1),
                  kv_cache=p["kv_cache"].reshape(nb, 128, 1, 512), kr_cache=p["kr_cache"].reshape(nb, 128, 1, 64),
                  kv_quant_scale_cache=p["kv_scale_cache"].reshape(nb, 128, 1, 4),
                  cache_index=p["cache_index"].reshape(b, s1), w_qb_scale=p["w_qb_scale"].reshape(1, -1))
    q_nope, q_rope, q_norm, q_norm_scale, kv_out, kr_out, sc_out = pro_mod.mla_prolog_quant_v32_compute(mla_in)
    ip_in = dict(token_x=mla_in["x"], q_norm=q_norm.reshape(b, s1, -1), q_norm_scale=q_norm_scale.reshape(b, s1, 1),
                 w_idx_qb=p["w_idx_qb"], w_idx_qb_scale=p["w_idx_qb_scale"].reshape(1, -1), w_idx_k=p["w_idx_k"],
                 w_idx_proj=p["w_idx_proj"], layer_norm_gamma=p["ln_gamma"], layer_norm_beta=p["ln_beta"],
                 cos_idx_rope=mla_in["cos"], sin_idx_rope=mla_in["sin"], hadamard_q=p["hadamard_q"],
                 hadamard_k=p["hadamard_k"], idx_k_cache=p["idx_k_cache"].reshape(nb, 128, 1, 128),
                 idx_k_scale_cache=p["idx_k_scale_cache"].reshape(nb, 128, 1, 1),
                 idx_k_cache_index=mla_in["cache_index"], idx_block_table=p["block_table"])
    ip = pro_mod.indexer_prolog(ip_in, dict(b=b, t=t, idx_n_heads=64, idx_head_dim=128, rope_head_dim=64))
    idx = p["cache_index"]
    q_nope = q_nope.reshape(t, 128, 512)
    tensors = {k: v for k, v in p.items() if isinstance(v, torch.Tensor)}
    np.savez_compressed(
        HERE / f"{name}.npz",
        act_seq=np.array(act_seq, dtype=np.int32), s1=np.int32(s1), seed=np.int64(seed),
        hashes=np.array([f"{k}={sha(v)}" for k, v in sorted(tensors.items())]),
        q_nope_sha=sha(q_nope), q_nope_heads=as_np(q_nope[:, list(PROLOG_HEADS), :]),
        q_rope=as_np(q_rope.reshape(t, 128, 64)),
        q_norm=q_norm.reshape(t, -1).numpy(), q_norm_scale=q_norm_scale.reshape(t).numpy(),
        # caches: the rows the operator wrote, plus a digest of the whole updated cache
        kv_rows=kv_out.reshape(rows, 512)[idx].numpy(), kv_cache_sha=sha(kv_out),
        kr_rows=as_np(kr_out.reshape(rows, 64)[idx]), kr_cache_sha=sha(kr_out),
        kv_scale_rows=sc_out.reshape(rows, 4)[idx].numpy(), kv_scale_cache_sha=sha(sc_out),
        q_int8=ip["q_int8"].reshape(t, 64, 128).numpy(),
        q_scale=ip["q_scale"].reshape(t, 64).numpy(),
        idx_k_rows=ip["idx_k_cache_out"].reshape(rows, 128)[idx].numpy(), idx_k_cache_sha=sha(ip["idx_k_cache_out"]),
        idx_k_scale_rows=ip["idx_k_scale_cache_out"].reshape(rows)[idx].numpy(),
        idx_k_scale_cache_sha=sha(ip["idx_k_scale_cache_out"]),
        weights=ip["weights"].reshape(t, 64).numpy(),
    )
    print(name, "t", t, "rows", rows)


PROLOG_NONQUANT_CASES = {
    # name: (act_seq, s1)
    "prolog_nonquant_single": ([300, 129, 1000], 1),
    "prolog_nonquant_mtp": ([257, 2048], 2),
}


def make_prolog_nonquant(name, act_seq, s1):
    """Runs the system tests' goldens of the two non-quantised prologs on inputs of
    `pypto_b200.inputs.make_prolog_nonquant_inputs`: `mla_prolog_compute` (numpy, ml_dtypes bfloat16; is_quant_a =
    is_quant_b = False, cache mode PA_BSND), then `indexer_prolog` (torch) with the first one's normalised query as
    `qr`."""
    import ml_dtypes
    mla_mod = importlib.import_module("gen_mla_prolog_golden_v32")
    ip_mod = importlib.import_module("gen_lightning_indexer_prolog")
    seed = 15000 + sum(act_seq) + s1
    p = gen.make_prolog_nonquant_inputs(act_seq, s1=s1, seed=seed)
    b, t = len(act_seq), len(act_seq) * s1
    rows = p["kv_cache"].shape[0]
    nb = rows // 128
    bf = ml_dtypes.bfloat16

    def nbf(x):
        return x.contiguous().view(torch.int16).numpy().view(bf).copy()

    def tbf(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(torch.bfloat16)

    mla_in = dict(dtype=bf, is_quant_a=False, is_quant_b=False, has_smooth=False, cache_mode="PA_BSND", epsilon=0.0,
                  gamma_cq=nbf(p["gamma_cq"]).astype(np.float32), gamma_ckv=nbf(p["gamma_ckv"]).astype(np.float32),
                  x=nbf(p["token_x"]).reshape(b, s1, -1), w_dq=nbf(p["w_dq"]), w_uqqr=nbf(p["w_uqqr"]),
                  w_uk=nbf(p["w_uk"]), w_dkvkr=nbf(p["w_dkvkr"]), cos=nbf(p["cos"]).reshape(b, s1, -1),
                  sin=nbf(p["sin"]).reshape(b, s1, -1), kv_cache=nbf(p["kv_cache"]).reshape(nb, 128, 1, 512),
                  kr_cache=nbf(p["kr_cache"]).reshape(nb, 128, 1, 64),
                  cache_index=p["cache_index"].reshape(b, s1).numpy())
    q_out, q_rope, kv_out, kr_out, q_norm = mla_mod.mla_prolog_compute(mla_in)
    q_nope, q_rope, q_norm = tbf(q_out).reshape(t, 128, 512), tbf(q_rope).reshape(t, 128, 64), tbf(q_norm).reshape(t, -1)
    kv_out, kr_out = tbf(kv_out).reshape(rows, 512), tbf(kr_out).reshape(rows, 64)
    ip_in = dict(token_x=p["token_x"].reshape(b, s1, -1), qr=q_norm.reshape(b, s1, -1), wq_b=p["w_idx_qb"],
                 wk=p["w_idx_k"], cos_idx_rope=p["cos"].reshape(b, s1, -1), sin_idx_rope=p["sin"].reshape(b, s1, -1),
                 weight_layer_norm=p["ln_gamma"], bias_layer_norm=p["ln_beta"],
                 idx_k_cache=p["idx_k_cache"].reshape(nb, 128, 1, 128),
                 idx_k_cache_index=p["cache_index"].reshape(b, s1), weights_proj=p["w_idx_proj"])
    ip = ip_mod.indexer_prolog(ip_in, dict(b=b, seq=s1, idx_n_heads=64, idx_head_dim=128, rope_head_dim=64))
    idx = p["cache_index"]
    tensors = {k: v for k, v in p.items() if isinstance(v, torch.Tensor)}
    np.savez_compressed(
        HERE / f"{name}.npz",
        act_seq=np.array(act_seq, dtype=np.int32), s1=np.int32(s1), seed=np.int64(seed),
        hashes=np.array([f"{k}={sha(v)}" for k, v in sorted(tensors.items())]),
        q_nope_sha=sha(q_nope), q_nope_heads=as_np(q_nope[:, list(PROLOG_HEADS), :]),
        q_rope=as_np(q_rope), q_norm=as_np(q_norm),
        kv_rows=as_np(kv_out[idx]), kv_cache_sha=sha(kv_out),
        kr_rows=as_np(kr_out[idx]), kr_cache_sha=sha(kr_out),
        idx_query=as_np(ip["query"].reshape(t, 64, 128)),
        idx_k_rows=as_np(ip["idx_k_cache_out"].reshape(rows, 128)[idx]), idx_k_cache_sha=sha(ip["idx_k_cache_out"]),
        weights=as_np(ip["weights"].reshape(t, 64)),
    )
    print(name, "t", t, "rows", rows)


def make_gather_kat():
    """The paged-gather known answer printed in the reference docstring
    (python/pypto/experimental.py:62-87) and the `10*token + h` buffer pattern of
    python/tests/st/test_gatherinub.py:83-94, written down as data."""
    param = np.array([[10 * r + c for c in range(4)] for r in range(6)], dtype=np.float32)
    np.savez_compressed(HERE / "gather_kat.npz", param=param, indices=np.array([0, 4, 3], dtype=np.int32),
                        block_table=np.array([0, 2, 1], dtype=np.int32), block_size=np.int32(2),
                        out=np.array([[0, 1, 2, 3], [20, 21, 22, 23], [50, 51, 52, 53]], dtype=np.float32))


def main():
    torch.set_num_threads(os.cpu_count() or 1)
    li_mod, sfa_mod, aq_mod, st_mod = load_reference()
    for name, (act, s1, dt) in LI_CASES.items():
        make_li(li_mod, st_mod, name, act, s1, dt)
    for name, (act, s1) in NONQUANT_CASES.items():
        make_li_nonquant(st_mod, name, act, s1)
    for name, (act, s1) in SFA_CASES.items():
        make_sfa(sfa_mod, aq_mod, name, act, s1)
    make_gather_kat()
    pro_mod = importlib.import_module("deepseekv32_mla_indexer_prolog_quant")
    for name, (act, s1) in PROLOG_CASES.items():
        make_prolog(pro_mod, name, act, s1)
    for name, (act, s1) in PROLOG_NONQUANT_CASES.items():
        make_prolog_nonquant(name, act, s1)


if __name__ == "__main__":
    main()
