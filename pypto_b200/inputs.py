"""Seeded synthetic inputs for the quantized DeepSeek-V3.2 sparse-attention decode path.

The tensors follow the layouts the reference's example drivers hand to the operators
(examples/models/deepseek_v32_exp/deepseekv32_lightning_indexer_quant.py:358-388 for the
indexer, deepseekv32_sparse_flash_attention_quant.py:417-441 for the attention): a paged
cache with 128-token blocks, one block table shared by the indexer cache and the latent cache,
per-sequence lengths, and one query token (or s1 tokens) per sequence.

Value distributions are the benchmark's (uniform int8 in [-127,127], scales uniform in
[1e-3,1e-2], bf16 N(0,1) for q and rope, weights N(0,1)/8); the reference's goldens are
distribution-agnostic.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

BLOCK_SIZE = 128
IDX_HEADS = 64
IDX_DIM = 128
ATT_HEADS = 128
KV_LORA = 512
ROPE_DIM = 64
TOPK = 2048
PACKED_ROW_BYTES = KV_LORA + 2 * ROPE_DIM + 16  # 656


@dataclass
class DecodeInputs:
    """All tensors of one decode step. Attribute names are the reference's argument names."""

    b: int
    s1: int
    act_seq: List[int]
    block_num: int
    max_blocks: int
    # shared paging state
    act_seq_key: torch.Tensor = None  # int32 [b]
    block_table: torch.Tensor = None  # int32 [b, max_blocks], -1 in unused slots
    # lightning indexer
    idx_query: Optional[torch.Tensor] = None  # int8 [t, 64, 128]
    idx_query_scale: Optional[torch.Tensor] = None  # f16|f32 [t, 64]
    idx_key_cache: Optional[torch.Tensor] = None  # int8 [block_num, 128, 1, 128]
    idx_key_scale: Optional[torch.Tensor] = None  # f16|f32 [block_num, 128, 1]
    idx_weight: Optional[torch.Tensor] = None  # f16|f32 [t, 64]
    # sparse attention
    query_nope: Optional[torch.Tensor] = None  # bf16 [t*128, 512]
    query_rope: Optional[torch.Tensor] = None  # bf16 [t*128, 64]
    key_nope_2d: Optional[torch.Tensor] = None  # int8 [block_num*128, 512]
    key_rope_2d: Optional[torch.Tensor] = None  # bf16 [block_num*128, 64]
    k_nope_scales: Optional[torch.Tensor] = None  # f32 [block_num*128, 4]
    topk_indices: Optional[torch.Tensor] = None  # int32 [t, 2048] (attention-only cases)
    extras: dict = field(default_factory=dict)

    @property
    def t(self) -> int:
        return self.b * self.s1

    def to(self, device) -> "DecodeInputs":
        out = DecodeInputs(self.b, self.s1, list(self.act_seq), self.block_num, self.max_blocks)
        for k, v in self.__dict__.items():
            if isinstance(v, torch.Tensor):
                setattr(out, k, v.to(device))
        out.extras = dict(self.extras)
        return out

    def tensors(self):
        return {k: v for k, v in self.__dict__.items() if isinstance(v, torch.Tensor)}


def make_block_table(act_seq: Sequence[int], gen: torch.Generator, device="cpu", max_blocks: Optional[int] = None):
    """Random permutation of the physical blocks, handed out to the sequences in order; unused
    slots hold -1 (same convention as gen_block_table,
    deepseekv32_sparse_flash_attention_quant.py:257-279)."""
    per = [math.ceil(s / BLOCK_SIZE) for s in act_seq]
    block_num = max(sum(per), 1)
    if max_blocks is None:
        max_blocks = max(max(per), 1)
    perm = torch.randperm(block_num, generator=gen, device=device).to(torch.int32)
    table = torch.full((len(act_seq), max_blocks), -1, dtype=torch.int32, device=device)
    off = 0
    for i, n in enumerate(per):
        table[i, :n] = perm[off:off + n]
        off += n
    return block_num, max_blocks, table


def _uniform(shape, lo, hi, gen, device, dtype=torch.float32):
    return (torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo).to(dtype)


def _int8(shape, gen, device):
    return torch.randint(-127, 128, shape, generator=gen, device=device, dtype=torch.int8)


def random_topk_indices(act_seq, s1, gen, device="cpu", topk=TOPK):
    """Distinct positions per query token, uniform over the causal range; rows shorter than
    topk list every position and are padded with -1 (the indexer's own padding value)."""
    b = len(act_seq)
    out = torch.full((b * s1, topk), -1, dtype=torch.int32, device=device)
    for bi, s in enumerate(act_seq):
        for i in range(s1):
            eff = s - (s1 - 1 - i)
            if eff <= 0:
                continue
            perm = torch.randperm(eff, generator=gen, device=device)[:topk].to(torch.int32)
            out[bi * s1 + i, : perm.numel()] = perm
    return out


def make_inputs(
    act_seq: Sequence[int],
    s1: int = 1,
    seed: int = 1234,
    device="cpu",
    scale_dtype: torch.dtype = torch.float32,
    with_indexer: bool = True,
    with_attention: bool = True,
    with_topk: bool = False,
    max_blocks: Optional[int] = None,
    attn_heads: int = ATT_HEADS,
) -> DecodeInputs:
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    act_seq = [int(s) for s in act_seq]
    b = len(act_seq)
    t = b * s1
    block_num, max_blocks, table = make_block_table(act_seq, gen, device, max_blocks)
    d = DecodeInputs(b, s1, act_seq, block_num, max_blocks)
    d.block_table = table
    d.act_seq_key = torch.tensor(act_seq, dtype=torch.int32, device=device)
    n_rows = block_num * BLOCK_SIZE
    if with_indexer:
        d.idx_query = _int8((t, IDX_HEADS, IDX_DIM), gen, device)
        d.idx_query_scale = _uniform((t, IDX_HEADS), 1e-3, 1e-2, gen, device, scale_dtype)
        d.idx_key_cache = _int8((block_num, BLOCK_SIZE, 1, IDX_DIM), gen, device)
        d.idx_key_scale = _uniform((block_num, BLOCK_SIZE, 1), 1e-3, 1e-2, gen, device, scale_dtype)
        d.idx_weight = (torch.randn((t, IDX_HEADS), generator=gen, device=device) / 8).to(scale_dtype)
    if with_attention:
        d.query_nope = torch.randn((t * attn_heads, KV_LORA), generator=gen, device=device).to(torch.bfloat16)
        d.query_rope = torch.randn((t * attn_heads, ROPE_DIM), generator=gen, device=device).to(torch.bfloat16)
        d.key_nope_2d = _int8((n_rows, KV_LORA), gen, device)
        d.key_rope_2d = torch.randn((n_rows, ROPE_DIM), generator=gen, device=device).to(torch.bfloat16)
        d.k_nope_scales = _uniform((n_rows, 4), 1e-3, 1e-2, gen, device)
    if with_topk:
        d.topk_indices = random_topk_indices(act_seq, s1, gen, device)
    return d


def make_nonquant_inputs(act_seq: Sequence[int], s1: int = 1, seed: int = 4321, device="cpu",
                         with_attention: bool = True, max_blocks: Optional[int] = None) -> DecodeInputs:
    """Inputs of the non-quantised formulation: bf16 indexer queries, keys and weights drawn as the reference's
    ST does (standard normal, gen_lightning_indexer.py:123-133), no scale tensors, and a bf16 latent cache."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    act_seq = [int(s) for s in act_seq]
    b = len(act_seq)
    t = b * s1
    block_num, max_blocks, table = make_block_table(act_seq, gen, device, max_blocks)
    d = DecodeInputs(b, s1, act_seq, block_num, max_blocks)
    d.block_table = table
    d.act_seq_key = torch.tensor(act_seq, dtype=torch.int32, device=device)
    n_rows = block_num * BLOCK_SIZE
    bf = torch.bfloat16
    d.idx_query = torch.randn((t, IDX_HEADS, IDX_DIM), generator=gen, device=device).to(bf)
    d.idx_key_cache = torch.randn((block_num, BLOCK_SIZE, 1, IDX_DIM), generator=gen, device=device).to(bf)
    d.idx_weight = torch.randn((t, IDX_HEADS), generator=gen, device=device).to(bf)
    if with_attention:
        d.query_nope = torch.randn((t * ATT_HEADS, KV_LORA), generator=gen, device=device).to(bf)
        d.query_rope = torch.randn((t * ATT_HEADS, ROPE_DIM), generator=gen, device=device).to(bf)
        d.key_nope_2d = (torch.randn((n_rows, KV_LORA), generator=gen, device=device) * 0.35).to(bf)
        d.key_rope_2d = torch.randn((n_rows, ROPE_DIM), generator=gen, device=device).to(bf)
    return d


def pack_kv_rows(key_nope_2d, key_rope_2d, k_nope_scales):
    """One 656-byte int8 row per token: 512 int8 latent | 64 bf16 rope | 4 fp32 scales
    (deepseekv32_sparse_attention_antiquant.py:258-268)."""
    n = key_nope_2d.shape[0]
    out = torch.empty((n, PACKED_ROW_BYTES), dtype=torch.int8, device=key_nope_2d.device)
    out[:, :KV_LORA] = key_nope_2d
    out[:, KV_LORA:KV_LORA + 2 * ROPE_DIM] = key_rope_2d.contiguous().view(torch.int8)
    out[:, KV_LORA + 2 * ROPE_DIM:] = k_nope_scales.contiguous().view(torch.int8)
    return out


# --- the five benchmark configurations ------------------------------------------------------

def config_act_seq(config_id: int, seed: Optional[int] = None) -> dict:
    """Sequence lengths and shapes of benchmark configuration `config_id` (0..4)."""
    seed = 1234 + config_id if seed is None else seed
    if config_id == 0:
        return dict(act_seq=[8192] * 2, s1=1, indexer=False, attention=True, topk=True, seed=seed)
    if config_id == 1:
        return dict(act_seq=[32768] * 8, s1=1, indexer=True, attention=False, topk=False, seed=seed)
    if config_id == 2:
        g = torch.Generator().manual_seed(seed)
        act = torch.randint(4096, 65536 + 1, (64,), generator=g).tolist()
        return dict(act_seq=act, s1=1, indexer=True, attention=True, topk=False, seed=seed)
    if config_id == 3:
        return dict(act_seq=[131072] * 128, s1=2, indexer=True, attention=True, topk=False, seed=seed)
    if config_id == 4:
        return dict(act_seq=[131072], s1=4096, indexer=True, attention=True, topk=False, seed=seed)
    raise ValueError(f"unknown config {config_id}")


def shard_act_seq(act_seq: Sequence[int], rank: int, world: int) -> List[int]:
    """Batch partition used for multi-GPU decode: sequences are dealt out longest-first to the
    rank with the least keys so far (indexer cost is proportional to the keys scanned)."""
    order = sorted(range(len(act_seq)), key=lambda i: -act_seq[i])
    loads = [0] * world
    owner = [0] * len(act_seq)
    counts = [0] * world
    cap = math.ceil(len(act_seq) / world)
    for i in order:
        cands = [r for r in range(world) if counts[r] < cap]
        r = min(cands, key=lambda r_: loads[r_])
        owner[i] = r
        loads[r] += act_seq[i]
        counts[r] += 1
    return [i for i in range(len(act_seq)) if owner[i] == rank]


def make_config(config_id: int, device="cpu", rank: int = 0, world: int = 1,
                scale_dtype=torch.float32, seed: Optional[int] = None) -> DecodeInputs:
    c = config_act_seq(config_id, seed)
    act = c["act_seq"]
    if world > 1:
        mine = shard_act_seq(act, rank, world)
        act = [act[i] for i in mine]
    return make_inputs(act, s1=c["s1"], seed=c["seed"] + 1000 * rank, device=device, scale_dtype=scale_dtype,
                       with_indexer=c["indexer"], with_attention=c["attention"], with_topk=c["topk"])


def take_sequences(d: DecodeInputs, seq_ids: Sequence[int], device=None, permute_seed: Optional[int] = None) -> DecodeInputs:
    """Compact copy holding only the listed sequences: their cache pages are renumbered 0..n-1 (in
    block-table order, or in a random order drawn from `permute_seed`, which keeps the block table a
    permutation), query rows are sliced. Used to cut a bounded CPU sample out of a large configuration and
    to hand each rank its batch shard."""
    device = torch.device(device) if device is not None else d.block_table.device
    src = d.block_table.device
    seq_ids = list(seq_ids)
    act = [d.act_seq[i] for i in seq_ids]
    per = [math.ceil(s / BLOCK_SIZE) for s in act]
    max_blocks = max(max(per), 1)
    block_num = max(sum(per), 1)
    out = DecodeInputs(len(seq_ids), d.s1, act, block_num, max_blocks)
    if permute_seed is None:
        new_ids = torch.arange(block_num, dtype=torch.long)
    else:
        new_ids = torch.randperm(block_num, generator=torch.Generator().manual_seed(permute_seed))
    table = torch.full((len(seq_ids), max_blocks), -1, dtype=torch.int32)
    old_pages = []
    off = 0
    for j, (i, n) in enumerate(zip(seq_ids, per)):
        old_pages.append(d.block_table[i, :n].to("cpu", torch.long))
        table[j, :n] = new_ids[off:off + n].to(torch.int32)
        off += n
    pages = torch.cat(old_pages) if old_pages else torch.zeros(0, dtype=torch.long)
    if pages.numel() == 0:
        pages = torch.zeros(1, dtype=torch.long)
    # page new_ids[k] of the copy holds old page pages[k]: gather with the inverse map
    inv = torch.empty(block_num, dtype=torch.long)
    inv[new_ids[:pages.numel()]] = torch.arange(pages.numel())
    pages_dev = pages[inv].to(src)
    rows_dev = (pages_dev[:, None] * BLOCK_SIZE + torch.arange(BLOCK_SIZE, device=src)[None, :]).reshape(-1)
    tok = torch.tensor([i * d.s1 + k for i in seq_ids for k in range(d.s1)], dtype=torch.long, device=src)
    out.block_table = table.to(device)
    out.act_seq_key = torch.tensor(act, dtype=torch.int32, device=device)
    if d.idx_query is not None:
        out.idx_query = d.idx_query[tok].to(device)
        out.idx_query_scale = d.idx_query_scale[tok].to(device)
        out.idx_weight = d.idx_weight[tok].to(device)
        out.idx_key_cache = d.idx_key_cache[pages_dev].to(device)
        out.idx_key_scale = d.idx_key_scale[pages_dev].to(device)
    if d.query_nope is not None:
        nq = d.query_nope.shape[0] // d.t
        out.query_nope = d.query_nope.reshape(d.t, nq, -1)[tok].reshape(-1, KV_LORA).to(device)
        out.query_rope = d.query_rope.reshape(d.t, nq, -1)[tok].reshape(-1, ROPE_DIM).to(device)
        out.key_nope_2d = d.key_nope_2d[rows_dev].to(device)
        out.key_rope_2d = d.key_rope_2d[rows_dev].to(device)
        out.k_nope_scales = d.k_nope_scales[rows_dev].to(device)
    if d.topk_indices is not None:
        out.topk_indices = d.topk_indices[tok].to(device)
    return out


def algorithmic_bytes(d: DecodeInputs, indexer=True, attention=True, topk=TOPK) -> dict:
    """Bytes one pass must move at minimum (no scratch): the indexer reads every key and scale of
    each sequence once, its queries, scales and weights and the used block-table entries, and
    writes the indices; the attention reads the selected rows (656 B each), q, the indices and
    writes the output."""
    s_el = d.idx_key_scale.element_size() if d.idx_key_scale is not None else 4
    li = 0
    sfa = 0
    for s in d.act_seq:
        if indexer:
            li += s * (IDX_DIM + s_el) + d.s1 * (IDX_HEADS * IDX_DIM + IDX_HEADS * 2 * s_el) \
                + 4 * math.ceil(s / BLOCK_SIZE) + d.s1 * topk * 4
        if attention:
            for i in range(d.s1):
                n = min(max(s - d.s1 + 1 + i, 0), topk)
                sfa += n * PACKED_ROW_BYTES + ATT_HEADS * (KV_LORA + ROPE_DIM) * 2 + 4 * n + ATT_HEADS * KV_LORA * 2
    return dict(indexer=li, attention=sfa, total=li + sfa)


def score_stage_bytes(d: DecodeInputs) -> int:
    """Algorithmic bytes of the score kernel alone: keys + key scales + queries + q scales/weights
    + block-table entries (the fp32 score scratch it writes is not algorithmic)."""
    s_el = d.idx_key_scale.element_size()
    return sum(s * (IDX_DIM + s_el) + d.s1 * (IDX_HEADS * IDX_DIM + IDX_HEADS * 2 * s_el) + 4 * math.ceil(s / BLOCK_SIZE)
               for s in d.act_seq)


# ---------------------------------------------------------------------------------------------
# MLA + indexer prolog (the producer of every tensor above)
# ---------------------------------------------------------------------------------------------
HIDDEN = 7168
Q_LORA = 1536
NOPE_DIM = 128  # per-head query width before absorption


def make_prolog_inputs(act_seq: Sequence[int], s1: int = 1, seed: int = 0, device="cpu") -> dict:
    """Inputs of the fused prolog operator, named after the reference driver's dictionaries and drawn from
    its distributions (examples/models/deepseek_v32_exp/deepseekv32_mla_indexer_prolog_quant.py:229-406):
    activations U(-1,1), bf16 weights U(-0.1,0.1), the query up-projection quantised per output column,
    cos/sin U(-0.1,0.1), random cache contents, `cache_index` = the paged row of each new token
    (positions S-s1 .. S-1 of its sequence). Tokens are flattened: t = b*s1 rows."""
    g = torch.Generator().manual_seed(seed)
    b = len(act_seq)
    t = b * s1
    block_num, _, table = make_block_table(act_seq, g)
    rows = block_num * BLOCK_SIZE
    bf = torch.bfloat16

    def uni(shape, lo, hi, dtype=bf):
        return _uniform(shape, lo, hi, g, "cpu", torch.float32).to(dtype)

    cache_index = torch.empty(t, dtype=torch.int64)
    for bi, s in enumerate(act_seq):
        for j in range(s1):
            pos = s - s1 + j
            cache_index[bi * s1 + j] = int(table[bi, pos // BLOCK_SIZE]) * BLOCK_SIZE + pos % BLOCK_SIZE
    w_uqqr_f = _uniform((Q_LORA, ATT_HEADS * (NOPE_DIM + ROPE_DIM)), -0.1, 0.1, g, "cpu")
    col_max = w_uqqr_f.abs().amax(dim=0, keepdim=True)
    w_uqqr = torch.round(w_uqqr_f * (127.0 / col_max)).to(torch.int8)
    p = dict(
        token_x=uni((t, HIDDEN), -1, 1),
        w_dq=uni((HIDDEN, Q_LORA), -0.1, 0.1),
        w_uqqr=w_uqqr,
        w_qb_scale=(col_max / 127.0).reshape(-1, 1).contiguous(),
        w_uk=uni((ATT_HEADS, NOPE_DIM, KV_LORA), -0.1, 0.1),
        w_dkvkr=uni((HIDDEN, KV_LORA + ROPE_DIM), -0.1, 0.1),
        gamma_cq=uni((Q_LORA,), -1, 1),
        gamma_ckv=uni((KV_LORA,), -1, 1),
        cos=uni((t, ROPE_DIM), -0.1, 0.1),
        sin=uni((t, ROPE_DIM), -0.1, 0.1),
        cache_index=cache_index,
        kv_cache=_int8((rows, KV_LORA), g, "cpu"),
        kr_cache=uni((rows, ROPE_DIM), -1, 1),
        kv_scale_cache=_uniform((rows, 4), 1e-3, 1e-2, g, "cpu"),
        w_idx_qb=torch.randint(-128, 128, (Q_LORA, IDX_HEADS * IDX_DIM), generator=g, dtype=torch.int8),
        w_idx_qb_scale=_uniform((IDX_HEADS * IDX_DIM, 1), -1, 1, g, "cpu"),
        w_idx_k=uni((HIDDEN, IDX_DIM), -1, 1),
        w_idx_proj=uni((HIDDEN, IDX_HEADS), -1, 1),
        ln_gamma=uni((IDX_DIM,), 0.5, 1.5),
        ln_beta=uni((IDX_DIM,), -0.5, 0.5),
        hadamard_q=uni((IDX_DIM, IDX_DIM), -1, 1),
        hadamard_k=uni((IDX_DIM, IDX_DIM), -1, 1),
        idx_k_cache=_int8((rows, IDX_DIM), g, "cpu"),
        idx_k_scale_cache=_uniform((rows, 1), 1e-3, 1e-2, g, "cpu").to(torch.float16),
        block_table=table,
    )
    if str(device) != "cpu":
        p = {k: v.to(device) for k, v in p.items()}
    p["act_seq"] = list(act_seq)
    p["s1"] = s1
    return p


def make_prolog_nonquant_inputs(act_seq: Sequence[int], s1: int = 1, seed: int = 0, device="cpu") -> dict:
    """Inputs of the two prologs in front of the non-quantised chain (`DecodeIndexerAttention`,
    framework/src/operator/models/deepseek_v3.2_exp/decode_indexer_attention.cpp:64-106): as `make_prolog_inputs`,
    with bf16 up-projection weights, bf16 latent / rope / indexer-key caches and no Hadamard matrices or scales."""
    g = torch.Generator().manual_seed(seed)
    b = len(act_seq)
    t = b * s1
    block_num, _, table = make_block_table(act_seq, g)
    rows = block_num * BLOCK_SIZE
    bf = torch.bfloat16

    def uni(shape, lo, hi, dtype=bf):
        return _uniform(shape, lo, hi, g, "cpu", torch.float32).to(dtype)

    cache_index = torch.empty(t, dtype=torch.int64)
    for bi, s in enumerate(act_seq):
        for j in range(s1):
            pos = s - s1 + j
            cache_index[bi * s1 + j] = int(table[bi, pos // BLOCK_SIZE]) * BLOCK_SIZE + pos % BLOCK_SIZE
    p = dict(
        token_x=uni((t, HIDDEN), -1, 1),
        w_dq=uni((HIDDEN, Q_LORA), -0.1, 0.1),
        w_uqqr=uni((Q_LORA, ATT_HEADS * (NOPE_DIM + ROPE_DIM)), -0.1, 0.1),
        w_uk=uni((ATT_HEADS, NOPE_DIM, KV_LORA), -0.1, 0.1),
        w_dkvkr=uni((HIDDEN, KV_LORA + ROPE_DIM), -0.1, 0.1),
        gamma_cq=uni((Q_LORA,), -1, 1),
        gamma_ckv=uni((KV_LORA,), -1, 1),
        cos=uni((t, ROPE_DIM), -1, 1),
        sin=uni((t, ROPE_DIM), -1, 1),
        cache_index=cache_index,
        kv_cache=uni((rows, KV_LORA), -1, 1),
        kr_cache=uni((rows, ROPE_DIM), -1, 1),
        w_idx_qb=uni((Q_LORA, IDX_HEADS * IDX_DIM), -0.1, 0.1),
        w_idx_k=uni((HIDDEN, IDX_DIM), -0.1, 0.1),
        w_idx_proj=uni((HIDDEN, IDX_HEADS), -0.1, 0.1),
        ln_gamma=uni((IDX_DIM,), 0.5, 1.5),
        ln_beta=uni((IDX_DIM,), -0.5, 0.5),
        idx_k_cache=uni((rows, IDX_DIM), -1, 1),
        block_table=table,
    )
    if str(device) != "cpu":
        p = {k: v.to(device) for k, v in p.items()}
    p["act_seq"] = list(act_seq)
    p["s1"] = s1
    return p


# --- host staging ----------------------------------------------------------------------------

_HOST_ARENAS = []  # keeps the cudaHostAlloc'd regions alive for the life of the process


def pinned_staging(nbytes: int, write_combined: bool = True) -> torch.Tensor:
    """A uint8 host tensor over page-locked memory for staging a step's inputs. With `write_combined` the
    region is allocated `cudaHostAllocWriteCombined`: the host only writes it and the GPU reads it across the bus,
    which is what that memory type is for (measured on this path: a 10 MB host-to-device copy 186 us instead of
    202 us alone, 226 us instead of 292 us beside a device-to-host copy). Falls back to `pin_memory()` when the
    CUDA runtime library cannot be reached through ctypes. Never read such a region from the host in a hot loop."""
    import ctypes

    if write_combined:
        try:
            rt = ctypes.CDLL("libcudart.so.12")
            ptr = ctypes.c_void_p()
            if rt.cudaHostAlloc(ctypes.byref(ptr), ctypes.c_size_t(nbytes), ctypes.c_uint(4)) == 0 and ptr.value:
                buf = (ctypes.c_uint8 * nbytes).from_address(ptr.value)
                t = torch.frombuffer(buf, dtype=torch.uint8)
                _HOST_ARENAS.append((buf, t))
                return t
        except (OSError, AttributeError):
            pass
    return torch.empty(nbytes, dtype=torch.uint8).pin_memory()
