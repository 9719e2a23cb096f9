"""Batch-partitioned multi-rank path on CPU: two gloo ranks each take their shard of the batch,
run the (oracle) chain on it with rank-local page ids, and the gathered outputs equal the
single-rank result. Exercises exactly the host logic bench.py and a multi-GPU caller use:
`shard_act_seq`, `take_sequences`, gather by sequence id. No collective sits on the data path."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from pypto_b200 import inputs as gen

ACT = [900, 300, 2100, 129, 513, 40]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _chain(d):
    idx, _, _ = oracle.lightning_indexer(d.idx_query, d.idx_query_scale, d.idx_key_cache, d.idx_key_scale,
                                         d.idx_weight, d.act_seq, d.block_table, d.s1)
    out = oracle.sparse_attention(d.query_nope, d.query_rope, d.key_nope_2d, d.key_rope_2d, d.k_nope_scales,
                                  idx.reshape(d.t, 2048), d.block_table, d.act_seq, d.s1)
    return idx, out


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    full = gen.make_inputs(ACT, s1=1, seed=31)
    mine = gen.shard_act_seq(ACT, rank, world)
    shard = gen.take_sequences(full, mine)
    idx, out = _chain(shard)
    # validation-only exchange: gather every rank's rows and put them back in batch order
    ids = [None] * world
    dist.all_gather_object(ids, mine)
    outs = [torch.zeros_like(out) for _ in range(world)]
    idxs = [torch.zeros_like(idx) for _ in range(world)]
    dist.all_gather(outs, out)
    dist.all_gather(idxs, idx)
    if rank == 0:
        got_out = torch.zeros((len(ACT), 1, 128, 512), dtype=torch.bfloat16)
        got_idx = torch.zeros((len(ACT), 1, 2048), dtype=torch.int32)
        for r in range(world):
            for j, seq in enumerate(ids[r]):
                got_out[seq] = outs[r][j]
                got_idx[seq] = idxs[r][j]
        want_idx, want_out = _chain(full)
        ret["idx_equal"] = bool(torch.equal(got_idx, want_idx))
        # the same per-token arithmetic in another process: the host BLAS may sum in another order there
        # (its kernels depend on buffer alignment and thread state), so allow a rounding, not more
        e = oracle.attention_errors(got_out, want_out)
        ret["out_rel_l2"], ret["out_max_abs"] = e["rel_l2"], e["max_abs"]
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_batch_partition_matches_single_rank():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert ret.get("idx_equal")
    assert ret.get("out_rel_l2") < 1e-3 and ret.get("out_max_abs") < 2e-3, dict(ret)
