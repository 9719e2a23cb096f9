"""ctypes binding of libpypto_b200.so (the C ABI declared in include/pypto_b200.h).

There is no fallback: if the shared object is missing or does not load, importing the operators
raises. Build it with `python -m pypto_b200.build`.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libpypto_b200.so"

PTO_DT_F16, PTO_DT_F32 = 0, 1
PTO_LI_SCORE_SIMT, PTO_LI_UNSORTED, PTO_LI_FP16_CHAIN, PTO_LI_EPILOGUE_HIST = 0x1, 0x2, 0x4, 0x8
PTO_STATUS_WORDS = 8
PTO_LI_STATIC_SCRATCH_BYTES = (8 << 20) + 256
PTO_ST_BAD_PAGE, PTO_ST_WAIT_EXPIRED = 0x1, 0x2

_vp, _i, _sz, _i64, _f = C.c_void_p, C.c_int, C.c_size_t, C.c_int64, C.c_float

# name -> (restype, argtypes); mirrors include/pypto_b200.h one to one
SIGNATURES = {
    "pto_abi_version": (_i, []),
    "pto_strerror": (C.c_char_p, [_i]),
    "pto_last_error": (C.c_char_p, []),
    "pto_launch_count": (C.c_longlong, []),
    "pto_workspace_status": (_i, [_vp, _vp, _vp]),
    "pto_workspace_reset": (_i, [_vp, _vp]),
    "pto_li_workspace_bytes": (_sz, [_i, _i, _i]),
    "pto_li_decode": (_i, [_vp] * 5 + [_i] + [_vp] * 3 + [_i] * 9 + [_vp, _sz, _vp]),
    "pto_li_decode_static": (_i, [_vp] * 5 + [_i] + [_vp] * 3 + [_i] * 9 + [_vp, _vp]),
    "pto_li_static_status": (_i, [_vp, _vp]),
    "pto_li_scores": (_i, [_vp] * 5 + [_i] + [_vp] * 4 + [_i] * 8 + [_vp, _sz, _vp]),
    "pto_li_decode_bf16": (_i, [_vp] * 6 + [_i] * 9 + [_vp, _sz, _vp]),
    "pto_li_scores_bf16": (_i, [_vp] * 6 + [_i] * 8 + [_vp, _sz, _vp]),
    "pto_li_topk": (_i, [_vp, _i64, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "pto_sfa_workspace_bytes": (_sz, [_i, _i]),
    "pto_sfa_quant": (_i, [_vp] * 9 + [_i, _i, _i, _i, _f, _i, _i, _i64, _i, _i, _i, _vp, _sz, _vp]),
    "pto_sfa_bf16": (_i, [_vp] * 8 + [_i, _i, _i, _i, _f, _i, _i, _i64, _i, _i, _i, _vp, _sz, _vp]),
    "pto_sfa_packed": (_i, [_vp] * 7 + [_i, _i, _i, _i, _f, _i, _i, _i64, _i, _i, _i, _vp, _sz, _vp]),
    "pto_prolog_workspace_bytes": (_sz, [_i, _i, _i]),
    "pto_prolog_pack_weights": (_i, [_vp] * 4 + [_i, _i, _vp, _vp]),
    "pto_kv_pack_rows": (_i, [_vp] * 3 + [_i64, _vp, _vp]),
    "pto_mla_indexer_prolog_quant": (_i, [_vp] * 31 + [_i, _i, _i, _i64, _f, _f, _f, _vp, _sz, _vp]),
    "pto_prolog_nonquant_workspace_bytes": (_sz, [_i, _i, _i]),
    "pto_mla_indexer_prolog": (_i, [_vp] * 24 + [_i, _i, _i, _i64, _f, _f, _f, _vp, _sz, _vp]),
    "pto_decode_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "pto_decode_fused": (_i, [_vp] * 5 + [_i] + [_vp] * 9 + [_i] * 6 + [_f, _i, _vp, _sz, _vp]),
    "pto_decode_fused_bf16": (_i, [_vp] * 11 + [_i] * 6 + [_f, _i, _vp, _sz, _vp]),
}

_lib = None


class PtoError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build the CUDA library with `python -m pypto_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    if lib.pto_abi_version() != 1:
        raise ImportError(f"libpypto_b200.so has ABI version {lib.pto_abi_version()}, expected 1")
    _lib = lib
    return lib


def check(rc: int):
    if rc != 0:
        lib = load()
        raise PtoError(f"{lib.pto_strerror(rc).decode()} ({rc}): {lib.pto_last_error().decode()}")
