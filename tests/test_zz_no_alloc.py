"""`pto_li_decode_static`: the indexer entry point for callers that cannot allocate device memory
(a serving engine whose pool owns all of HBM, a process that must stay off the allocator). Its
scratch is a fixed array inside the library, so it takes no workspace. The test drives it through
the C ABI exactly as such a caller would and checks it against `pto_li_decode` (caller-allocated
workspace): same inputs, bit-identical indices, on two calls in a row - the second call sees
the first call's leftovers in the shared array and must not be disturbed by them.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import pytest
import torch

from pypto_b200 import _lib
from pypto_b200 import inputs as gen

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, fn_name, d, out, tail):
    g = d
    fn = getattr(lib, fn_name)
    return fn(g.idx_query.data_ptr(), g.idx_query_scale.data_ptr(), g.idx_key_cache.data_ptr(),
              g.idx_key_scale.data_ptr(), g.idx_weight.data_ptr(),
              _lib.PTO_DT_F16 if g.idx_query_scale.dtype == torch.float16 else _lib.PTO_DT_F32,
              g.act_seq_key.data_ptr(), g.block_table.data_ptr(), out.data_ptr(), d.b, d.s1, 64, 128, 128, d.block_num,
              d.max_blocks, 2048, 0, *tail)


def _reference_entry(lib, d):
    out = torch.zeros((d.t, 1, 2048), dtype=torch.int32, device=DEV)
    nbytes = lib.pto_li_workspace_bytes(d.t, d.max_blocks, 128)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_call(lib, "pto_li_decode", d, out, (ws.data_ptr(), ws.numel(), stream)))
    torch.cuda.synchronize()
    return out.cpu()


def _static_entry(lib, d):
    out = torch.full((d.t, 1, 2048), -7, dtype=torch.int32, device=DEV)
    status = (C.c_int32 * _lib.PTO_STATUS_WORDS)()
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_call(lib, "pto_li_decode_static", d, out, (status, stream)))
    assert status[0] == 0
    return out.cpu()


def test_static_scratch_entry_matches_workspace_entry_twice():
    lib = _lib.load()
    # first call: rows of up to 30000 scores (about 0.5 MB of the array); second call: a different, shorter,
    # ragged batch with two query tokens per sequence, so stale scores of the first call lie beyond its rows
    first = gen.make_inputs([30000, 17000, 2049, 9000], s1=1, seed=101, with_attention=False).to(DEV)
    second = gen.make_inputs([5000, 130, 2500], s1=2, seed=202, scale_dtype=torch.float16, with_attention=False).to(DEV)
    for d in (first, second):
        want = _reference_entry(lib, d)
        got = _static_entry(lib, d)
        assert torch.equal(got, want)
    # and once more in the opposite order
    assert torch.equal(_static_entry(lib, first), _reference_entry(lib, first))


def test_static_scratch_entry_rejects_oversized_problem():
    lib = _lib.load()
    d = gen.make_inputs([4096] * 2, s1=1, seed=5, with_attention=False).to(DEV)
    out = torch.zeros((64, 1, 2048), dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    # claim 64 tokens x 1024 blocks: 32 MiB of scores, beyond the 8 MiB array -> refused before any launch
    rc = lib.pto_li_decode_static(d.idx_query.data_ptr(), d.idx_query_scale.data_ptr(), d.idx_key_cache.data_ptr(),
                                  d.idx_key_scale.data_ptr(), d.idx_weight.data_ptr(), _lib.PTO_DT_F32,
                                  d.act_seq_key.data_ptr(), d.block_table.data_ptr(), out.data_ptr(), 64, 1, 64, 128,
                                  128, d.block_num, 1024, 2048, 0, None, stream)
    assert rc == -2
    assert b"static array" in lib.pto_last_error()


def test_static_scratch_capacity_edge():
    """The array holds exactly 8 MiB of score rows: 16 tokens x 1024 blocks x 128 keys x 4 bytes are accepted
    (and run: the block table is that wide, the sequences themselves are short), one more block is refused on
    the host with nothing launched. The status words of an accepted call can be read back afterwards."""
    lib = _lib.load()
    d = gen.make_inputs([700, 129, 3000, 64] * 4, s1=1, seed=303, with_attention=False, max_blocks=1025).to(DEV)
    assert d.b * 1024 * 128 * 4 == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream

    def call(max_blocks, table, out):
        return lib.pto_li_decode_static(d.idx_query.data_ptr(), d.idx_query_scale.data_ptr(), d.idx_key_cache.data_ptr(),
                                        d.idx_key_scale.data_ptr(), d.idx_weight.data_ptr(), _lib.PTO_DT_F32,
                                        d.act_seq_key.data_ptr(), table.data_ptr(), out.data_ptr(), d.b, 1, 64, 128, 128,
                                        d.block_num, max_blocks, 2048, 0, None, stream)

    out = torch.full((d.t, 1, 2048), -7, dtype=torch.int32, device=DEV)
    assert call(1025, d.block_table, out) == -2 and b"static array" in lib.pto_last_error()
    torch.cuda.synchronize()
    assert torch.all(out == -7)  # refused before any launch
    narrow = d.block_table[:, :1024].contiguous()
    _lib.check(call(1024, narrow, out))
    status = (C.c_int32 * _lib.PTO_STATUS_WORDS)()
    _lib.check(lib.pto_li_static_status(status, stream))
    assert status[0] == 0
    d.max_blocks, d.block_table = 1024, narrow
    assert torch.equal(out.cpu(), _reference_entry(lib, d))
