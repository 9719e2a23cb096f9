"""The shared library loads without a GPU driver and exports every function the public header
declares; the ctypes table covers the same set."""
import ctypes
import re
from pathlib import Path

import pytest

from pypto_b200 import _lib, build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_functions():
    text = (ROOT / "include" / "pypto_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pto_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("pto_li_decode", "pto_li_scores", "pto_li_topk", "pto_sfa_quant", "pto_sfa_bf16", "pto_sfa_packed",
                 "pto_decode_fused", "pto_li_decode_static", "pto_workspace_status"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    raw = ctypes.CDLL(str(_lib.lib_path()))
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} is declared in include/pypto_b200.h but not exported"


def test_ctypes_table_matches_header(lib):
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_host_only_calls(lib):
    assert lib.pto_abi_version() == 1
    assert lib.pto_strerror(0) == b"ok"
    assert lib.pto_strerror(-2).startswith(b"workspace")
    # status words, fp32 score rows, one 4096-bin histogram row per query token
    assert lib.pto_li_workspace_bytes(8, 256, 128) == 256 + 8 * 256 * 128 * 4 + 8 * 4096 * 4
    assert lib.pto_li_workspace_bytes(0, 256, 128) == 0
    # 64 tokens x 2 head blocks fill the device: unsplit, status words only
    assert lib.pto_sfa_workspace_bytes(80, 128) == 256
    assert lib.pto_sfa_workspace_bytes(2, 128) > 2 * 16 * 128 * 512 * 4
    assert lib.pto_decode_workspace_bytes(64, 512, 128, 128) == (256 + 64 * 512 * 128 * 4 + lib.pto_sfa_workspace_bytes(64, 128)
                                                                 - 256 + 64 * 4096 * 4)


def test_argument_errors_are_reported_before_any_cuda_call(lib):
    # null pointers: rejected on the host, no launch, no GPU needed
    rc = lib.pto_li_decode(None, None, None, None, None, 1, None, None, None, 1, 1, 64, 128, 128, 1, 1, 2048, 0,
                           None, 0, None)
    assert rc == -1 and b"null" in lib.pto_last_error()
    rc = lib.pto_li_topk(None, 128, None, None, 1, 1, 2048, 0, None, 0, None)
    assert rc == -1
    rc = lib.pto_workspace_status(None, None, None)
    assert rc == -1
