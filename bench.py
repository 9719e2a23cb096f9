#!/usr/bin/env python3
"""Benchmark of the fused decode step: lightning indexer -> top-2048 -> sparse MLA attention.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload: benchmark configuration 2 - batch 64, one query token per sequence, context lengths uniform
in [4096, 65536], int8 indexer keys and int8 latent KV with fp32 scales, bf16 q and rope, paged cache
with 128-token blocks and a permuted block table; seeded synthetic data. With N > 1 the 64 sequences
are dealt out to the ranks (batch-partitioned, 64/N sequences each, no collective on the data path):
the total work is fixed, the scaling is strong. One step = one pass of the fused chain over the rank's
sequences: the public fused operator recorded once into a CUDA graph (`pypto_b200.CapturedCall`) and
replayed; `eager` gives the same operator called from the host every step, `weak` the step with a full
batch of 64 on every rank.

Before anything is timed the step's results are checked: rank 0 runs the whole batch on its GPU and
compares it with the CPU oracle chain (`parity_checked`), and with N > 1 the ranks' outputs are
gathered with an NCCL all_gather and compared with that single-GPU result (`multi_gpu_validation`).

Prints ONE JSON line on rank 0. `value` = query tokens/s over all ranks with inputs resident in
HBM, device-timed (CUDA events, max over ranks). `e2e` = the same step through the public Python
operator with the step's inputs (queries, scales, weights, lengths, block table) copied from pinned
host memory and the attention output copied back every step; the KV caches are resident state.
`e2e_layer` = what a serving loop moves: the new tokens' hidden states in, prolog -> fused decode on
the device, the attention output back. `--impl reference` times the CPU restatement of the reference's
torch goldens (oracle/) on the host cores on a bounded sample of the same workload.

`--config 3` (MTP: 128 sequences x 131072 keys, two query tokens) and `--config 4` (prefill chunk:
4096 query tokens over 131072 keys; `--partition heads` = 16 heads per rank with the whole indexer on
every rank, `--partition tokens` = 4096/N query tokens per rank, all heads) run the same way.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from pypto_b200 import inputs as gen  # noqa: E402

METRIC = "decode_queries_per_s"
UNIT = "queries/s"
SCALE = 576 ** -0.5


def load_peaks(which="hbm_gbs"):
    """Measured roofline denominators (driver-written file), else the pool's earlier measurement."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            j = json.loads(p.read_text())
            return float(j[which]), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}[which], "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def oracle_chain(d):
    import oracle
    idx, _, _ = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                         d.idx_weight, d.act_seq, d.block_table, d.s1)
    return oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                   idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)


def cpu_sample(n_seq: int, seed_rank: int = 0):
    """The first `n_seq` sequences of configuration 2 (lengths as in the GPU workload), on the host."""
    c = gen.config_act_seq(2)
    act = c["act_seq"][:n_seq]
    return gen.make_inputs(act, s1=1, seed=c["seed"] + 1000 * seed_rank, device="cpu")


def time_cpu(d, repeats=1):
    torch.set_num_threads(os.cpu_count() or 1)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle_chain(d)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def run_reference(args, rank, world):
    """CPU arm: the oracle port of the reference goldens, all host threads, bounded sample per step."""
    if rank != 0:
        return
    n_seq = args.cpu_seqs
    d = cpu_sample(n_seq)
    for _ in range(min(args.warmup, 1)):
        oracle_chain(gen.take_sequences(d, [0]))
    times = []
    for _ in range(args.steps):
        times.append(time_cpu(d))
    tot = sum(times)
    value = n_seq * len(times) / tot
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * tot / len(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8+bf16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "config2: fused indexer -> top-2048 -> sparse MLA decode, batch 64, ctx U[4096,65536]",
                   "sample": f"first {n_seq} sequences of the batch per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"oracle chain (torch CPU restatement of the reference goldens) on the first "
                                   f"{n_seq} sequences of config 2, {len(times)} step(s)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def measure_prolog(dev, batch, ctx, s1, steps, warmup):
    """The fused MLA + indexer prolog for `batch` sequences x `s1` tokens, eager and replayed from a CUDA graph,
    timed with CUDA events. Algorithmic bytes = every weight once + the token's rows."""
    import pypto_b200 as pto

    p = gen.make_prolog_inputs([ctx] * batch, s1=s1, seed=4321, device=dev)
    t = batch * s1
    out = [torch.zeros(t, 128, 512, dtype=torch.bfloat16, device=dev), torch.zeros(t, 128, 64, dtype=torch.bfloat16, device=dev),
           p["kv_cache"], p["kr_cache"], p["kv_scale_cache"], torch.zeros(t, 64, 128, dtype=torch.int8, device=dev),
           torch.zeros(t, 64, 1, dtype=torch.float16, device=dev), p["idx_k_cache"], p["idx_k_scale_cache"],
           torch.zeros(t, 64, dtype=torch.float16, device=dev)]
    names = ["token_x", "w_dq", "w_uqqr", "w_qb_scale", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin",
             "cache_index", "kv_cache", "kr_cache", "kv_scale_cache", "w_idx_qb", "w_idx_qb_scale", "w_idx_k",
             "w_idx_proj", "ln_gamma", "ln_beta", "hadamard_q", "hadamard_k", "idx_k_cache", "idx_k_scale_cache"]
    call_args = [p[n] for n in names] + out + [1e-5, 1e-5, "PA_BSND", None, None, None, None]
    weights = ["w_dq", "w_uqqr", "w_qb_scale", "w_uk", "w_dkvkr", "w_idx_qb", "w_idx_qb_scale", "w_idx_k", "w_idx_proj",
               "hadamard_q", "hadamard_k"]
    by = sum(p[n].numel() * p[n].element_size() for n in weights)
    by += t * (7168 * 2 + 128 * 576 * 2 + 64 * 128 + 64 * 4 + 656 + 130)
    captured = pto.CapturedCall(pto.mla_indexer_prolog_quant_d, *call_args)
    res = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # the weights (100 MB) would stay in the 126 MB L2
    for tag, fn in (("eager", lambda: pto.mla_indexer_prolog_quant_d(*call_args)), ("graph", captured.replay)):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for e0, e1 in ev:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        res[tag + "_ms"] = statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)
    peak, src = load_peaks()
    return {"stage": "prolog", "tokens": t, **res, "algorithmic_bytes": by,
            "achieved_gbs": by / res["graph_ms"] / 1e6, "peak_gbs": peak, "peak_source": src,
            "frac": by / res["graph_ms"] / 1e6 / peak, "gpu_launches_per_call": 7,
            "l2": "256 MB written between timed calls", "status": pto.workspace_status(dev)[0]}


def measure_prolog_nonquant(dev, batch, ctx, s1, steps, warmup):
    """The two prologs of the non-quantised chain (`pto.mla_indexer_prolog`) for `batch` x `s1` tokens, eager and
    replayed from a CUDA graph. Algorithmic bytes = every (bf16) weight once + the token's rows."""
    import pypto_b200 as pto

    p = gen.make_prolog_nonquant_inputs([ctx] * batch, s1=s1, seed=4321, device=dev)
    t = batch * s1
    bf = torch.bfloat16
    out = [torch.zeros(t, 128, 512, dtype=bf, device=dev), torch.zeros(t, 128, 64, dtype=bf, device=dev),
           torch.zeros(t, 64, 128, dtype=bf, device=dev), torch.zeros(t, 64, dtype=bf, device=dev)]
    names = ["token_x", "w_dq", "w_uqqr", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin", "cache_index",
             "kv_cache", "kr_cache", "w_idx_qb", "w_idx_k", "w_idx_proj", "ln_gamma", "ln_beta", "idx_k_cache"]
    call_args = [p[n] for n in names] + out + [1e-5, 1e-5]
    weights = ["w_dq", "w_uqqr", "w_uk", "w_dkvkr", "w_idx_qb", "w_idx_k", "w_idx_proj"]
    by = sum(p[n].numel() * p[n].element_size() for n in weights)
    by += t * (7168 * 2 + 128 * 576 * 2 + 64 * 128 * 2 + 64 * 2 + (512 + 64 + 128) * 2)
    captured = pto.CapturedCall(pto.mla_indexer_prolog, *call_args)
    res = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for tag, fn in (("eager", lambda: pto.mla_indexer_prolog(*call_args)), ("graph", captured.replay)):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for e0, e1 in ev:
            flush.zero_()
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        res[tag + "_ms"] = statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)
    peak, src = load_peaks()
    return {"stage": "prolog_nonquant", "tokens": t, **res, "algorithmic_bytes": by,
            "achieved_gbs": by / res["graph_ms"] / 1e6, "peak_gbs": peak, "peak_source": src,
            "frac": by / res["graph_ms"] / 1e6 / peak, "gpu_launches_per_call": 7,
            "l2": "256 MB written between timed calls", "status": pto.workspace_status(dev)[0]}


def run_prolog_stage(args, dev):
    fn = measure_prolog_nonquant if args.stage == "prolog_nonquant" else measure_prolog
    print(json.dumps(fn(dev, args.batch, args.ctx, args.s1, args.steps, args.warmup)), flush=True)


def run_layer_stage(args, dev):
    """Profiling aid: what one decoder layer runs of this path per step - the prolog on the new tokens' hidden
    states, then indexer -> top-2048 -> sparse attention on the prolog's outputs and the caches it has just
    updated - recorded into one CUDA graph and replayed. Caches hold random rows; --ctx keys per sequence."""
    import pypto_b200 as pto

    act = [args.ctx] * args.batch
    p = gen.make_prolog_inputs(act, s1=args.s1, seed=4321, device=dev)
    t, rows = args.batch * args.s1, p["kv_cache"].shape[0]
    q_nope = torch.zeros(t, 128, 512, dtype=torch.bfloat16, device=dev)
    q_rope = torch.zeros(t, 128, 64, dtype=torch.bfloat16, device=dev)
    q_i8 = torch.zeros(t, 64, 128, dtype=torch.int8, device=dev)
    q_sc = torch.zeros(t, 64, 1, dtype=torch.float16, device=dev)
    w = torch.zeros(t, 64, dtype=torch.float16, device=dev)
    names = ["token_x", "w_dq", "w_uqqr", "w_qb_scale", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin",
             "cache_index", "kv_cache", "kr_cache", "kv_scale_cache", "w_idx_qb", "w_idx_qb_scale", "w_idx_k",
             "w_idx_proj", "ln_gamma", "ln_beta", "hadamard_q", "hadamard_k", "idx_k_cache", "idx_k_scale_cache"]
    pro_args = [p[n] for n in names] + [q_nope, q_rope, p["kv_cache"], p["kr_cache"], p["kv_scale_cache"], q_i8, q_sc,
                                        p["idx_k_cache"], p["idx_k_scale_cache"], w, 1e-5, 1e-5, "PA_BSND", None, None,
                                        None, None]
    act_t = torch.tensor(act, dtype=torch.int32, device=dev)
    topk = torch.zeros(t, 1, 2048, dtype=torch.int32, device=dev)
    out = torch.zeros(args.batch, args.s1, 128, 512, dtype=torch.bfloat16, device=dev)
    # the indexer reads its key scales in the dtype of the query scales: fp16 here, as the prolog writes them
    dec_args = [q_i8, q_sc.reshape(t, 64), p["idx_k_cache"].reshape(rows // 128, 128, 1, 128),
                p["idx_k_scale_cache"].reshape(rows // 128, 128, 1), w, q_nope.reshape(t * 128, 512),
                q_rope.reshape(t * 128, 64), p["kv_cache"], p["kr_cache"], p["kv_scale_cache"], act_t, p["block_table"],
                topk, out]

    def layer(_out):
        pto.mla_indexer_prolog_quant_d(*pro_args)
        pto.decode_indexer_attention_quant(*dec_args)

    captured = pto.CapturedCall(layer, out)
    for _ in range(args.warmup):
        captured.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        captured.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / max(args.steps, 1)
    print(json.dumps({"stage": "layer", "batch": args.batch, "ctx": args.ctx, "s1": args.s1, "ms": ms,
                      "tokens_per_s": t / ms * 1e3, "gpu_launches_per_step": 12,
                      "l2": "caches larger than L2; the 100 MB of weights may stay in L2 between replays",
                      "status": pto.workspace_status(dev)[0], "finite": bool(torch.isfinite(out.float()).all())}),
          flush=True)


def run_stage(args, dev):
    """Profiling aid: one stage alone on a uniform synthetic case, timed with CUDA events."""
    import pypto_b200 as pto

    if args.stage in ("prolog", "prolog_nonquant"):
        return run_prolog_stage(args, dev)
    if args.stage == "layer":
        return run_layer_stage(args, dev)
    d = gen.make_inputs([args.ctx] * args.batch, s1=args.s1, seed=4321, device=dev,
                        scale_dtype=getattr(torch, args.scale_dtype), with_topk=True, attn_heads=args.nq)
    t = d.t
    idx = torch.zeros((t, 1, 2048), dtype=torch.int32, device=dev)
    out = torch.zeros((d.b, d.s1, args.nq, 512), dtype=torch.bfloat16, device=dev)
    sc = torch.randn((t, d.max_blocks * 128), dtype=torch.float32, device=dev)
    li = (d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale, d.idx_weight, d.act_seq_key, d.block_table)
    kn_bf16 = None
    if args.stage == "sfa_bf16":  # the non-quantised latent cache holding the values the int8 one dequantises to
        kn_bf16 = (d.key_nope_2d.to(torch.float32).reshape(-1, 4, 128) * d.k_nope_scales.reshape(-1, 4, 1)
                   ).reshape(-1, 512).to(torch.bfloat16)
    packed = torch.empty((d.key_nope_2d.shape[0], 656), dtype=torch.int8, device=dev) if args.stage == "kv_pack" else None
    nq_d = gen.make_nonquant_inputs([args.ctx] * args.batch, s1=args.s1, seed=4321, device=dev,
                                    with_attention=False) if args.stage == "li_score_nonquant" else None
    fns = {
        "kv_pack": lambda: pto.pack_kv_cache(d.key_nope_2d, d.key_rope_2d, d.k_nope_scales, packed),
        "li_score_nonquant": lambda: pto.lightning_indexer_topk_nonquant(
            nq_d.idx_query, nq_d.idx_key_cache, nq_d.idx_weight, nq_d.act_seq_key, nq_d.block_table, None, scores_out=sc),
        "li_score": lambda: pto.lightning_indexer_scores(*li, sc),
        "li_score_chain": lambda: pto.lightning_indexer_scores(*li, sc, fp16_chain=True),  # needs --scale-dtype float16
        "li_decode": lambda: pto.lightning_indexer_decode(*li, idx, None, None, 2048),
        "topk": lambda: pto.lightning_indexer_topk(sc, d.act_seq_key, idx, s1=d.s1),
        "topk_unsorted": lambda: pto.lightning_indexer_topk(sc, d.act_seq_key, idx, s1=d.s1, sort=False),
        "sfa": lambda: pto.sparse_flash_attention_quant_d(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d,
                                                          d.k_nope_scales, d.topk_indices, d.block_table,
                                                          d.act_seq_key, out, args.nq, 1, SCALE, 2048, 128, d.max_blocks),
        "sfa_bf16": lambda: pto.sparse_flash_attention_quant_d(d.query_nope, d.query_rope, kn_bf16, d.key_rope_2d,
                                                               d.k_nope_scales, d.topk_indices, d.block_table,
                                                               d.act_seq_key, out, 128, 1, SCALE, 2048, 128,
                                                               d.max_blocks),
        "fused": lambda: pto.decode_indexer_attention_quant(*li[:5], d.query_nope, d.query_rope, d.key_nope_2d,
                                                            d.key_rope_2d, d.k_nope_scales, d.act_seq_key,
                                                            d.block_table, idx, out),
    }
    fn = fns[args.stage]
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / max(args.steps, 1)
    by = gen.algorithmic_bytes(d)
    print(json.dumps({"stage": args.stage, "batch": args.batch, "ctx": args.ctx, "s1": args.s1, "ms": ms,
                      "score_stage_bytes": gen.score_stage_bytes(d), "algorithmic_bytes": by,
                      "status": pto.workspace_status(dev)[0]}), flush=True)


def li_ops(d) -> int:
    """int8 multiply-adds x 2 of the score stage: 64 heads x 128 dims per (query token, key of its sequence)."""
    return sum(2 * 64 * 128 * max(s, 0) * d.s1 for s in d.act_seq)


def sfa_flops(d) -> int:
    """2 * 128 heads * n selected rows * (576 + 512) per query token."""
    f = 0
    for s in d.act_seq:
        for i in range(d.s1):
            f += 2 * 128 * min(max(s - d.s1 + 1 + i, 0), 2048) * (576 + 512)
    return f


def build_workload(args, rank, world, dev):
    """The rank's share of the configuration. Returns (shard, full, mine, describe): `full` is the whole batch on
    this device where the configuration is small enough to hold and to validate against (configuration 2)."""
    c = gen.config_act_seq(args.config)
    sdt = getattr(torch, args.scale_dtype)
    if args.config == 2:
        full = gen.make_inputs(c["act_seq"], s1=c["s1"], seed=c["seed"], device=dev, scale_dtype=sdt)
        if world == 1:
            return full, full, list(range(full.b)), "whole batch"
        mine = gen.shard_act_seq(c["act_seq"], rank, world)
        shard = gen.take_sequences(full, mine, permute_seed=c["seed"] + 1000 * rank)
        return shard, full, mine, f"{len(mine)} of {full.b} sequences per rank, longest-first by keys"
    if args.config == 3:
        assert 128 % world == 0
        per = 128 // world
        d = gen.make_inputs(c["act_seq"][:per], s1=c["s1"], seed=c["seed"] + 1000 * rank, device=dev, scale_dtype=sdt)
        return d, None, list(range(rank * per, rank * per + per)), f"{per} of 128 sequences per rank"
    if args.config == 4:
        S, chunk = 131072, 4096
        if args.partition == "heads" and world > 1:
            # every rank runs the whole indexer and the attention of its 128/N heads (query rows of those heads only)
            nq = 128 // world
            d = gen.make_inputs([S], s1=chunk, seed=c["seed"], device=dev, scale_dtype=sdt, attn_heads=nq)
            d.extras["nq"] = nq
            return d, None, [0], f"{nq} heads per rank, the indexer whole on every rank"
        per = chunk // world
        # rank r takes query tokens [r*per, (r+1)*per) of the chunk: positions S - chunk + r*per .. ; its causal
        # range ends at its own last token
        d = gen.make_inputs([S], s1=per, seed=c["seed"] + 1000 * rank, device=dev, scale_dtype=sdt)
        end = S - chunk + (rank + 1) * per
        d.act_seq = [end]
        d.act_seq_key = torch.tensor([end], dtype=torch.int32, device=dev)
        return d, None, [0], f"{per} of {chunk} query tokens per rank, all heads"
    raise SystemExit("bench.py times configurations 2, 3 and 4 (0 and 1 are parity-test cases)")


def fused_call(d, idx, out, **kw):
    import pypto_b200 as pto
    pto.decode_indexer_attention_quant(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale, d.idx_weight,
                                       d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                       d.act_seq_key, d.block_table, idx, out, nq=d.extras.get("nq", 128), **kw)


def check_against_oracle(d_dev, idx, out, seq_ids=None, last_tokens=None):
    """Operator results against the CPU oracle chain for the listed sequences (default: all) or, for a prefill
    chunk, its last `last_tokens` query tokens. Sets must be equal on untied scores; attention errors returned."""
    import oracle
    nq = d_dev.extras.get("nq", 128)
    if last_tokens is not None:
        s1 = last_tokens
        sub = gen.DecodeInputs(1, s1, list(d_dev.act_seq), d_dev.block_num, d_dev.max_blocks)
        for k, v in d_dev.tensors().items():
            setattr(sub, k, v.cpu() if k not in ("idx_query", "idx_query_scale", "idx_weight", "query_nope", "query_rope") else None)
        t0 = d_dev.t - s1
        sub.idx_query, sub.idx_query_scale, sub.idx_weight = (x[t0:].cpu() for x in (d_dev.idx_query, d_dev.idx_query_scale, d_dev.idx_weight))
        sub.query_nope, sub.query_rope = d_dev.query_nope[t0 * nq:].cpu(), d_dev.query_rope[t0 * nq:].cpu()
        got_idx, got_out = idx[t0:].cpu(), out.reshape(d_dev.t, nq, 512)[t0:].cpu()
    else:
        seq_ids = list(range(d_dev.b)) if seq_ids is None else list(seq_ids)
        sub = gen.take_sequences(d_dev, seq_ids, device="cpu") if len(seq_ids) < d_dev.b else d_dev.to("cpu")
        tok = [i * d_dev.s1 + k for i in seq_ids for k in range(d_dev.s1)]
        got_idx, got_out = idx.cpu()[tok], out.reshape(d_dev.t, nq, 512).cpu()[tok]
    want_idx, _, rows = oracle.lightning_indexer(sub.idx_query, sub.idx_query_scale, sub.idx_key_cache, sub.idx_key_scale,
                                                 sub.idx_weight, sub.act_seq, sub.block_table, sub.s1)
    untied = tied = 0
    for ti in range(sub.t):
        u, t_ = oracle.topk_set_diff(got_idx[ti], want_idx[ti], rows[ti])
        untied += u
        tied += t_
    want = oracle.sparse_attention(sub.query_nope, sub.query_rope, sub.key_nope_2d, sub.key_rope_2d, sub.k_nope_scales,
                                   want_idx.reshape(sub.t, 2048), sub.block_table, sub.act_seq, sub.s1, nq=nq)
    e = oracle.attention_errors(got_out, want.reshape(sub.t, nq, 512))
    worst = max((oracle.attention_errors(got_out[ti], want.reshape(sub.t, nq, 512)[ti])["rel_l2"] for ti in range(sub.t)
                 if float(want.reshape(sub.t, nq, 512)[ti].float().abs().max()) > 0), default=0.0)
    ok = untied == 0 and e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3 and worst <= 5e-3
    return {"ok": bool(ok), "tokens_checked": sub.t, "topk_untied_mismatches": untied, "topk_tied_swaps": tied,
            "attention_max_abs": e["max_abs"], "attention_rel_l2": e["rel_l2"], "worst_token_rel_l2": worst,
            "tolerance": "sets exact on untied scores; max-abs 2e-2, rel-L2 5e-3 per token"}


def time_each(fn, steps, stream, before=None):
    """Mean CUDA-event time of `fn` over `steps` launches, each bracketed by its own pair of events; `before`
    runs untimed ahead of every launch (an L2 flush)."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in ev:
        if before is not None:
            before()
        e0.record(stream)
        fn()
        e1.record(stream)
    torch.cuda.synchronize()
    return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)


def measure_e2e_layer(d, dev, steps, barrier):
    """Serving-shaped end to end: per step the new tokens' hidden states (and rope tables, cache rows, lengths,
    block table) cross from pinned host memory, the prolog produces the queries and updates the caches, the fused
    decode runs on them, the attention output goes back to the host - all recorded into one CUDA graph per buffer
    set, two sets alternating on two streams. The caches are the step workload's (fp16 indexer key scales, as the
    prolog writes them); weights are random."""
    import pypto_b200 as pto

    t, b = d.t, d.b
    p = gen.make_prolog_inputs([128] * b, s1=d.s1, seed=4321, device=dev)  # weights, token states, rope tables
    rows = d.block_num * 128
    ks16 = d.idx_key_scale.to(torch.float16).reshape(rows, 1).contiguous()
    kcache = d.idx_key_cache.reshape(rows, 128)
    ci = torch.empty(t, dtype=torch.int64)
    table_cpu = d.block_table.cpu()
    for bi, s in enumerate(d.act_seq):
        for j in range(d.s1):
            pos = max(s - d.s1 + j, 0)
            ci[bi * d.s1 + j] = int(table_cpu[bi, pos // 128]) * 128 + pos % 128
    step_in = {"token_x": p["token_x"], "cos": p["cos"], "sin": p["sin"], "cache_index": ci.to(dev),
               "act_seq_key": d.act_seq_key, "block_table": d.block_table}
    layout, total = {}, 0
    for n, v in step_in.items():
        layout[n] = (total, v.numel() * v.element_size(), v.dtype, tuple(v.shape))
        total += (v.numel() * v.element_size() + 255) // 256 * 256

    def views(arena):
        return {n: arena[off:off + nb].view(dt).reshape(shape) for n, (off, nb, dt, shape) in layout.items()}

    host_arena = gen.pinned_staging(total)  # write-combined: the host writes it, the GPU reads it
    hv = views(host_arena)
    for n, v in step_in.items():
        hv[n].copy_(v.cpu())
    names = ["token_x", "w_dq", "w_uqqr", "w_qb_scale", "w_uk", "w_dkvkr", "gamma_cq", "gamma_ckv", "cos", "sin",
             "cache_index", "kv_cache", "kr_cache", "kv_scale_cache", "w_idx_qb", "w_idx_qb_scale", "w_idx_k",
             "w_idx_proj", "ln_gamma", "ln_beta", "hadamard_q", "hadamard_k", "idx_k_cache", "idx_k_scale_cache"]
    caches = {"kv_cache": d.key_nope_2d, "kr_cache": d.key_rope_2d, "kv_scale_cache": d.k_nope_scales,
              "idx_k_cache": kcache, "idx_k_scale_cache": ks16}
    sets = []
    for i in range(2):
        arena = torch.empty(total, dtype=torch.uint8, device=dev)
        arena.copy_(host_arena)
        x = views(arena)
        q_nope = torch.zeros(t, 128, 512, dtype=torch.bfloat16, device=dev)
        q_rope = torch.zeros(t, 128, 64, dtype=torch.bfloat16, device=dev)
        q_i8 = torch.zeros(t, 64, 128, dtype=torch.int8, device=dev)
        q_sc = torch.zeros(t, 64, 1, dtype=torch.float16, device=dev)
        w = torch.zeros(t, 64, dtype=torch.float16, device=dev)
        topk = torch.zeros(t, 1, 2048, dtype=torch.int32, device=dev)
        out = torch.zeros(b, d.s1, 128, 512, dtype=torch.bfloat16, device=dev)
        out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        src = {**p, **caches, **x}
        pro_args = [src[n] for n in names] + [q_nope, q_rope, caches["kv_cache"], caches["kr_cache"],
                                              caches["kv_scale_cache"], q_i8, q_sc, caches["idx_k_cache"],
                                              caches["idx_k_scale_cache"], w, 1e-5, 1e-5, "PA_BSND", None, None, None,
                                              None]
        dec_args = [q_i8, q_sc.reshape(t, 64), d.idx_key_cache, ks16.reshape(d.block_num, 128, 1), w,
                    q_nope.reshape(t * 128, 512), q_rope.reshape(t * 128, 64), d.key_nope_2d, d.key_rope_2d,
                    d.k_nope_scales, x["act_seq_key"], x["block_table"], topk, out]

        def layer(_out, arena=arena, pro_args=pro_args, dec_args=dec_args, out=out, out_host=out_host):
            arena.copy_(host_arena, non_blocking=True)
            pto.mla_indexer_prolog_quant_d(*pro_args)
            pto.decode_indexer_attention_quant(*dec_args)
            out_host.copy_(out, non_blocking=True)

        n0 = pto.launch_count()
        g = pto.CapturedCall(layer, out)
        sets.append((g, torch.cuda.Stream(dev), out, out_host, (pto.launch_count() - n0) // 2))

    def run(n):
        for k in range(n):
            g, s, _, _, _ = sets[k & 1]
            with torch.cuda.stream(s):
                g.replay()
        torch.cuda.synchronize()

    run(4)
    barrier()
    t0 = time.perf_counter()
    run(steps)
    barrier()
    dt = time.perf_counter() - t0
    status = [g.workspace_status()[0] for g, *_ in sets]
    finite = all(bool(torch.isfinite(oh.float()).all()) for _, _, _, oh, _ in sets)
    d2h = sets[0][3].numel() * sets[0][3].element_size()
    return dt, {"h2d_bytes_per_step": total, "d2h_bytes_per_step": d2h, "status": status, "finite": finite,
                "own_kernel_launches_per_step": sets[0][4],
                "note": "hidden states, rope tables, cache rows, lengths and block table from one pinned arena -> prolog -> "
                        "fused decode -> output to pinned host memory, one CUDA graph per buffer set, two sets on two "
                        "streams; caches and weights are resident device state"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--partition", default="heads", choices=["heads", "tokens"], help="configuration 4 on N > 1 GPUs")
    ap.add_argument("--cpu-seqs", type=int, default=64, help="sequences in the CPU-baseline sample")
    ap.add_argument("--stage", default=None, choices=["li_score", "li_decode", "topk", "sfa", "sfa_bf16", "fused", "prolog", "layer", "li_score_chain",
                             "kv_pack", "li_score_nonquant", "topk_unsorted", "prolog_nonquant"],
                    help="profiling aid: run only this stage --steps times on a uniform case (--batch x --ctx) and exit")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=65536)
    ap.add_argument("--s1", type=int, default=1)
    ap.add_argument("--nq", type=int, default=128, help="--stage sfa: heads per token (a head slice below 128)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sustained loop, the weak-scaling figure, e2e_layer and the prolog")
    ap.add_argument("--scale-dtype", default="float32", choices=["float32", "float16"])
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist

    import pypto_b200 as pto

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.stage is not None:
        run_stage(args, dev)
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    d, full, mine, partition = build_workload(args, rank, world, dev)
    t, nq = d.t, d.extras.get("nq", 128)
    stream = torch.cuda.current_stream(dev)
    idx = torch.zeros((t, 1, 2048), dtype=torch.int32, device=dev)
    out = torch.zeros((d.b, d.s1, nq, 512), dtype=torch.bfloat16, device=dev)

    # ---- results first: the step that is about to be timed is checked against the CPU oracle, and the ranks'
    # outputs against the whole batch on one GPU (NCCL is used for this gather and for the barriers only) ----
    fused_call(d, idx, out)
    torch.cuda.synchronize()
    assert pto.workspace_status(dev)[0] == 0, "device status flagged an error"
    parity, multi = None, None
    if args.config == 2:
        idx_f, out_f = idx, out
        if world > 1:
            idx_f, out_f = torch.zeros((full.t, 1, 2048), dtype=torch.int32, device=dev), torch.zeros((full.b, 1, 128, 512), dtype=torch.bfloat16, device=dev)
            if rank == 0:
                fused_call(full, idx_f, out_f)
            per = len(mine)
            g_idx = [torch.zeros_like(idx) for _ in range(world)]
            g_out = [torch.zeros_like(out) for _ in range(world)]
            g_ids = [torch.zeros(per, dtype=torch.int64, device=dev) for _ in range(world)]
            dist.all_gather(g_idx, idx)
            dist.all_gather(g_out, out)
            dist.all_gather(g_ids, torch.tensor(mine, dtype=torch.int64, device=dev))
            if rank == 0:
                got_idx, got_out = torch.zeros_like(idx_f), torch.zeros_like(out_f)
                for r in range(world):
                    got_idx[g_ids[r]] = g_idx[r]
                    got_out[g_ids[r]] = g_out[r]
                sets_equal = bool(torch.equal(got_idx.sort(dim=-1).values, idx_f.sort(dim=-1).values))
                rel = float((got_out.float() - out_f.float()).norm() / out_f.float().norm())
                mx = float((got_out.float() - out_f.float()).abs().max())
                multi = {"gathered_with": "nccl all_gather of topk_res and attention_out", "ranks": world,
                         "index_sets_equal_single_gpu": sets_equal, "attention_rel_l2_vs_single_gpu": rel,
                         "attention_max_abs_vs_single_gpu": mx, "ok": bool(sets_equal and rel <= 5e-3 and mx <= 2e-2)}
                assert multi["ok"], f"gathered multi-GPU outputs differ from the single-GPU run: {multi}"
        if rank == 0:
            parity = check_against_oracle(full, idx_f, out_f)
    elif rank == 0:
        parity = (check_against_oracle(d, idx, out, seq_ids=[0, d.b - 1]) if args.config == 3
                  else check_against_oracle(d, idx, out, last_tokens=8))
    if rank == 0:
        assert parity["ok"], f"the step's results differ from the CPU oracle: {parity}"
    if world > 1 and full is not None and rank != 0 and args.no_extras:
        full = None
    barrier()

    # ---- the timed step: the public fused operator recorded once into a CUDA graph and replayed ---------------
    n0 = pto.launch_count()
    captured = pto.CapturedCall(fused_call, d, idx, out)
    launches_per_step = (pto.launch_count() - n0) // 2  # one warm-up call + the recorded call
    step = captured.replay
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert captured.workspace_status()[0] == 0, "device status flagged an error during warm-up"

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record(stream)
    for k in range(args.steps):
        step()
        ev[k + 1].record(stream)
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = [ev[k].elapsed_time(ev[k + 1]) for k in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None

    # ---- the same operator called from the host every step -------------------------------------------------------
    idx_e, out_e = torch.zeros_like(idx), torch.zeros_like(out)
    for _ in range(3):
        fused_call(d, idx_e, out_e)
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for _ in range(args.steps):
        fused_call(d, idx_e, out_e)
    g1.record(stream)
    torch.cuda.synchronize()
    eager_ms = g0.elapsed_time(g1) / args.steps
    rel_g = float((out_e.float() - out.float()).norm() / out.float().norm())
    assert rel_g < 5e-3, f"graph replay output differs from the eager run (rel-L2 {rel_g})"

    # ---- each kernel of the step alone, CUDA events around every launch -----------------------------------------
    # score kernel: streams more than L2 holds every launch; top-k: reads the score rows the score kernel has just
    # written (L2-resident in the step too); attention: 256 MB written before every launch, as the score kernel's
    # stream evicts the cache rows between two steps
    li = (d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale, d.idx_weight, d.act_seq_key, d.block_table)
    sc = torch.empty((t, d.max_blocks * 128), dtype=torch.float32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    idx_k = torch.zeros_like(idx)
    out_k = torch.zeros_like(out)
    sfa_idx = idx.reshape(t, 2048)
    kfn = {
        "li_score": (lambda: pto.lightning_indexer_scores(*li, sc), None),
        "topk": (lambda: pto.lightning_indexer_topk(sc, d.act_seq_key, idx_k, s1=d.s1, sort=False), None),
        "sfa": (lambda: pto.sparse_flash_attention_quant_d(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d,
                                                            d.k_nope_scales, sfa_idx, d.block_table, d.act_seq_key, out_k,
                                                            nq, 1, SCALE, 2048, 128, d.max_blocks), flush.zero_),
    }
    kernel_ms = {}
    for name, (fn, before) in kfn.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        kernel_ms[name] = time_each(fn, args.steps, stream, before)
    assert pto.workspace_status(dev)[0] == 0, "device status flagged an error"
    # the whole step with 256 MB written before every replay: the timed loop above replays the same inputs, so the
    # rows the attention gathered in one step (about 100 MB on one GPU) are partly still in L2 in the next
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    cold_ms = time_each(step, args.steps, stream, flush.zero_)

    # ---- sustained: the same replay looped for at least two seconds, clocks sampled (nothing is set) -------------
    sustained = None
    if not args.no_extras:
        n_loop = max(int(2.2e3 / max(total_ms / args.steps, 1e-3)), args.steps)
        s2 = ClockSampler(local_rank)
        if rank == 0:
            s2.start()
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record(stream)
        for _ in range(n_loop):
            step()
        h1.record(stream)
        barrier()
        sus_ms = h0.elapsed_time(h1)
        sustained = {"steps": n_loop, "seconds": sus_ms * 1e-3, "ms_per_step": sus_ms / n_loop,
                     "clocks": s2.stop() if rank == 0 else None}

    # ---- weak scaling beside it: a full batch of 64 on every rank (configuration 2, N > 1) -----------------------
    weak_ms = None
    if world > 1 and full is not None and not args.no_extras:
        idx_w = torch.zeros((full.t, 1, 2048), dtype=torch.int32, device=dev)
        out_w = torch.zeros((full.b, 1, 128, 512), dtype=torch.bfloat16, device=dev)
        cap_w = pto.CapturedCall(fused_call, full, idx_w, out_w)
        for _ in range(3):
            cap_w.replay()
        barrier()
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0.record(stream)
        for _ in range(args.steps):
            cap_w.replay()
        w1.record(stream)
        barrier()
        weak_ms = w0.elapsed_time(w1) / args.steps
        del cap_w, idx_w, out_w
    if world > 1:
        full = None

    # ---- end to end through the public operator with host buffers --------------------------
    # Every step copies its inputs (queries, scales, weights, lengths, block table) from pinned host
    # memory, runs the fused operator (replayed from a captured graph per buffer set) and copies the attention
    # output back. Steps are double buffered over three streams (H2D / compute / D2H), as a serving loop would
    # run them: the copies of neighbouring steps overlap the compute, every byte is still moved every step.
    host_names = ["idx_query", "idx_query_scale", "idx_weight", "query_nope", "query_rope", "act_seq_key",
                  "block_table"]
    # one pinned staging arena on the host and one arena per buffer set on the device, the operator's tensors
    # being views into them: a step's inputs cross the bus as ONE copy (seven separate copies of 0.1-8 MB were
    # measured at 266 us against 188 us for the same bytes in one)
    layout, total = {}, 0
    for n in host_names:
        v = getattr(d, n)
        layout[n] = (total, v.numel() * v.element_size(), v.dtype, tuple(v.shape))
        total += (v.numel() * v.element_size() + 255) // 256 * 256

    def views(arena):
        return {n: arena[off:off + nb].view(dt).reshape(shape) for n, (off, nb, dt, shape) in layout.items()}

    host_arena = gen.pinned_staging(total)  # write-combined: the host writes it, the GPU reads it
    host = views(host_arena)
    for n in host_names:
        host[n].copy_(getattr(d, n).cpu())
    dev_arena = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(2)]
    dev_in = [views(a) for a in dev_arena]
    dev_idx = [torch.zeros_like(idx) for _ in range(2)]
    dev_out = [torch.zeros_like(out) for _ in range(2)]
    out_host = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
    h2d = total
    d2h = out_host[0].numel() * out_host[0].element_size()
    s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_ready = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    for i in range(2):  # (valid contents for the warm-up call inside the capture helper)
        dev_arena[i].copy_(host_arena, non_blocking=True)
    torch.cuda.synchronize()
    e2e_steps = [pto.CapturedCall(pto.decode_indexer_attention_quant, x["idx_query"], x["idx_query_scale"],
                                  d.idx_key_cache, d.idx_key_scale, x["idx_weight"], x["query_nope"], x["query_rope"],
                                  d.key_nope_2d, d.key_rope_2d, d.k_nope_scales, x["act_seq_key"], x["block_table"],
                                  dev_idx[i], dev_out[i], nq=nq) for i, x in enumerate(dev_in)]

    def e2e_run(n_steps):
        for k in range(n_steps):
            i = k & 1
            with torch.cuda.stream(s_in):
                if k >= 2:
                    s_in.wait_event(comp_done[i])  # step k-2 no longer reads this input set
                dev_arena[i].copy_(host_arena, non_blocking=True)
                in_ready[i].record(s_in)
            with torch.cuda.stream(s_comp):
                s_comp.wait_event(in_ready[i])
                if k >= 2:
                    s_comp.wait_event(out_done[i])  # step k-2's output has been copied out
                e2e_steps[i].replay()
                comp_done[i].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[i])
                out_host[i].copy_(dev_out[i], non_blocking=True)
                out_done[i].record(s_out)
        torch.cuda.synchronize()

    e2e_run(4)
    barrier()
    t0 = time.perf_counter()
    e2e_run(args.steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    # same result as the resident-input run, up to the rounding of a different summation order (the fused
    # call leaves the selected indices unordered)
    e2e_out = out_host[(args.steps - 1) & 1].to(dev).float()
    rel = float((e2e_out - out.float()).norm() / out.float().norm())
    assert rel < 5e-3, f"end-to-end output differs from the resident-input run (rel-L2 {rel})"
    # the host -> device copy of one step's inputs alone, on its stream
    with torch.cuda.stream(s_in):
        h2d_ms = time_each(lambda: dev_arena[0].copy_(host_arena, non_blocking=True), 10, s_in)
    del e2e_steps, dev_arena, dev_in, dev_out, dev_idx

    layer_s, layer_info = None, None
    if not args.no_extras and args.config in (2, 3):
        try:
            layer_s, layer_info = measure_e2e_layer(d, dev, args.steps, barrier)
        except Exception as e:  # the headline line must not depend on it
            if world > 1:
                raise
            layer_info = {"error": str(e)[:300]}

    # max over ranks
    v = torch.tensor([total_ms, e2e_s, kernel_ms["li_score"], kernel_ms["topk"], kernel_ms["sfa"], eager_ms,
                      sustained["ms_per_step"] if sustained else 0.0, weak_ms or 0.0, layer_s or 0.0, h2d_ms, cold_ms],
                     dtype=torch.float64, device=dev)
    # algorithmic bytes and flops summed over the ranks' shards
    by = gen.algorithmic_bytes(d)
    # a head-sharded chunk: every rank holds all query tokens for its 128/N heads, so a token counts once over the ranks
    t_share = t * d.extras.get("nq", 128) / 128.0
    w = torch.tensor([by["indexer"], by["attention"], gen.score_stage_bytes(d), sfa_flops(d), t_share, li_ops(d)],
                     dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        dist.all_reduce(w, op=dist.ReduceOp.SUM)
    (total_ms, e2e_s, li_ms, topk_ms, sfa_ms, eager_ms, sus_ms_step, weak_ms, layer_s, h2d_ms, cold_ms) = (float(x) for x in v.tolist())
    by_li, by_sfa, by_score, fl_sfa, t_all, ops_li = (float(x) for x in w.tolist())

    if rank == 0:
        peak, peak_src = load_peaks("hbm_gbs")
        tf_peak, tf_src = load_peaks("bf16_tflops")
        tf_sus, _ = load_peaks("bf16_tflops_sustained")
        ms_per_step = total_ms / args.steps
        value = t_all * args.steps / (total_ms * 1e-3)
        e2e_value = t_all * args.steps / e2e_s
        # per-GPU rates of the slowest rank's launch: the whole job's work / N over the max-over-ranks time
        per_gpu = 1.0 / world
        li_gbs = by_score * per_gpu / (li_ms * 1e-3) / 1e9
        sfa_tfs = fl_sfa * per_gpu / (sfa_ms * 1e-3) / 1e12
        sfa_gbs = by_sfa * per_gpu / (sfa_ms * 1e-3) / 1e9
        step_gbs = (by_li + by_sfa) * per_gpu / (ms_per_step * 1e-3) / 1e9
        roof_li = {"bound": "hbm", "kernel": "li_score_tc_kernel", "achieved": li_gbs, "peak": peak, "unit": "GB/s",
                   "frac": li_gbs / peak,
                   # dram read+write of one launch: ncu measured 143.93 MB for 138.58 MB algorithmic on batch 16 x
                   # 65536 (profiles/); the extra is the 4 B/key score write, which scales with the keys
                   "traffic": int(by_score * per_gpu * 143.93 / 138.58), "peak_source": peak_src,
                   "algorithmic_bytes_per_launch": int(by_score * per_gpu), "ms_per_launch": li_ms}
        # the score stage is bound by the tensor pipe, not by HBM, once a key page serves many query tokens (prefill
        # chunks): int8 ops / time against twice the measured bf16 peak (int8 dense is nominally 2 x bf16; no int8
        # peak was measured on this pool)
        li_tops = ops_li * per_gpu / (li_ms * 1e-3) / 1e12
        roof_li["frac_hbm"] = roof_li["frac"]
        roof_li["frac_tensor_int8"] = li_tops / (2 * tf_peak)
        roof_li["achieved_tops_int8"] = li_tops
        if ops_li / (2 * tf_peak * 1e12) > by_score / (peak * 1e9):
            roof_li.update({"bound": "tensor", "achieved": li_tops, "peak": 2 * tf_peak, "unit": "TOP/s (int8)",
                            "frac": li_tops / (2 * tf_peak),
                            "peak_source": "2 x " + tf_src + " bf16 burst peak (stated, not measured for int8)"})
        sfa_kernel = "sfa_pair_kernel" if nq == 128 else "sfa_mma_kernel"
        tensor_bound = fl_sfa / (tf_peak * 1e12) >= by_sfa / (peak * 1e9)
        roof_sfa = {"bound": "tensor" if tensor_bound else "hbm", "kernel": sfa_kernel,
                    "achieved": sfa_tfs if tensor_bound else sfa_gbs, "peak": tf_peak if tensor_bound else peak,
                    "unit": "TFLOP/s" if tensor_bound else "GB/s",
                    "frac": sfa_tfs / tf_peak if tensor_bound else sfa_gbs / peak,
                    "frac_tensor": sfa_tfs / tf_peak, "frac_hbm": sfa_gbs / peak, "achieved_tflops": sfa_tfs,
                    "achieved_gbs": sfa_gbs, "peak_source": tf_src + " (bf16 burst: the kernel is timed alone)",
                    # ncu: 104.4 MB of DRAM traffic for 104.3 MB algorithmic on 64 tokens x 2048 rows (profiles/)
                    "traffic": int(by_sfa * per_gpu * 104.4 / 104.3), "flops_per_launch": int(fl_sfa * per_gpu),
                    "algorithmic_bytes_per_launch": int(by_sfa * per_gpu), "ms_per_launch": sfa_ms,
                    "l2": "256 MB written before every timed launch"}
        dominant = "sfa" if sfa_ms >= li_ms else "li_score"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if args.config in (2, 3, 4) else "weak",
            "vs_baseline": None, "dtype": "int8+bf16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"config{args.config}: fused indexer -> top-2048 -> sparse MLA decode",
                       "step": "the public fused operator, recorded once into a CUDA graph and replayed",
                       "global_batch": int(round(t_all)) // d.s1 if args.config != 4 else 1, "query_tokens_per_step": int(round(t_all)),
                       "per_gpu_sequences": d.b, "s1": d.s1, "heads_per_gpu": nq,
                       "context": f"{min(d.act_seq)}..{max(d.act_seq)} keys per sequence on rank 0, mean {sum(d.act_seq) / d.b:.0f}",
                       "scale_dtype": args.scale_dtype,
                       "partition": f"{partition}; no collective on the data path",
                       "l2": f"inputs ({d.block_num * 128 * (132 + 656) / 1e9:.2f} GB of cache on rank 0) larger than L2, "
                             "no flush between the timed steps; `step_cold_l2` is the same step with 256 MB written "
                             "before every replay"},
            "parity_checked": bool(parity and parity["ok"]), "parity": parity,
            "multi_gpu_validation": multi,
            "roofline": roof_sfa if dominant == "sfa" else roof_li,
            "roofline_li_score": roof_li, "roofline_sfa": roof_sfa,
            "roofline_step": {"bound": "hbm", "achieved": step_gbs, "peak": peak, "unit": "GB/s",
                              "frac": step_gbs / peak, "algorithmic_bytes_per_step_all_ranks":
                                  {"indexer": int(by_li), "attention": int(by_sfa), "total": int(by_li + by_sfa)},
                              "note": "per GPU: all ranks' algorithmic bytes / N over the max-over-ranks step time"},
            "step_cold_l2": {"ms_per_step": cold_ms, "value": t_all / (cold_ms * 1e-3),
                             "note": "every replay timed alone with CUDA events, 256 MB written before it: the replayed "
                                     "inputs are the same every step, so without the flush part of the rows the "
                                     "attention gathered (and the queries) are still in L2 from the step before"},
            "kernel_ms": {"li_score": li_ms, "topk": topk_ms, "sfa": sfa_ms, "sum": li_ms + topk_ms + sfa_ms,
                          "note": "each kernel alone, CUDA events around every launch, max over ranks; the attention "
                                  "launch includes its combine kernel when the rows are split over CTAs"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "h2d_copy_ms": h2d_ms, "ms_per_step": 1e3 * e2e_s / args.steps,
                    "note": "per-step inputs (queries, scales, weights, lengths, block table) from one pinned (write-combined) "
                            "host arena in one copy, output copied back, steps double-buffered over H2D/compute/D2H streams; "
                            "KV caches are resident device state; h2d_copy_ms = that copy alone (per rank, max over ranks)"},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "eager": {"ms_per_step": eager_ms, "value": t_all * 1e3 / eager_ms,
                      "note": "the same operator called from the host every step instead of replayed"},
            "clocks": clocks,
            "step_ms_min_max": [min(step_ms), max(step_ms)],
        }
        if sustained:
            line["sustained"] = {"ms_per_step": sus_ms_step, "value": t_all * 1e3 / sus_ms_step, "steps": sustained["steps"],
                                 "seconds": sustained["seconds"], "clocks": sustained["clocks"],
                                 "bf16_peak_sustained_tflops": tf_sus}
        if weak_ms:
            line["weak"] = {"ms_per_step": weak_ms, "value": 64 * world * 1e3 / weak_ms, "global_batch": 64 * world,
                            "note": "a full batch of 64 sequences on every rank"}
        if layer_info is not None:
            line["e2e_layer"] = dict(layer_info)
            if layer_s:
                line["e2e_layer"].update({"value": t_all * args.steps / layer_s, "unit": UNIT,
                                          "ms_per_step": 1e3 * layer_s / args.steps})
        if world == 1 and not args.no_extras:
            # the producer of the step's inputs, measured beside it (not part of `value`): the fused MLA + indexer
            # prolog for this batch's new tokens, 100 MB of weights streamed from HBM every call
            try:
                pr = measure_prolog(dev, d.b, 8192, d.s1, 10, 3)
                line["prolog"] = {"ms_per_call": pr["graph_ms"], "eager_ms_per_call": pr["eager_ms"],
                                  "tokens": pr["tokens"], "algorithmic_bytes": pr["algorithmic_bytes"],
                                  "achieved_gbs": pr["achieved_gbs"], "frac_of_hbm_peak": pr["frac"],
                                  "gpu_launches_per_call": pr["gpu_launches_per_call"], "l2": pr["l2"]}
            except Exception as e:  # the headline line must not depend on it
                line["prolog"] = {"error": str(e)[:200]}
        if not args.no_cpu_baseline and world == 1:
            n_seq = args.cpu_seqs
            dcpu = cpu_sample(n_seq)
            passes, spent = 0, 0.0
            while spent < 10.0 and passes < 50:
                spent += time_cpu(dcpu)
                passes += 1
            line["cpu_baseline"] = {"value": n_seq * passes / spent, "unit": UNIT, "cores": os.cpu_count() or 1,
                                    "kind": "port",
                                    "sample": f"oracle chain (torch CPU) on the first {n_seq} sequences of config 2, "
                                              f"{passes} passes, {spent:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
