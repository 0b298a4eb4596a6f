"""ctypes binding of ``libtokenselect_b200.so`` (declarations: ``include/tokenselect_b200.h``).

There is no CPU fallback: if the library is missing or does not load, importing callers get a
``RuntimeError`` that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TOKENSELECT_B200_LIB points at another build of the same sources (e.g. one compiled with diagnostic macros)
LIB_PATH = os.environ.get("TOKENSELECT_B200_LIB") or os.path.join(HERE, "libtokenselect_b200.so")

TS_OK = 0
TS_DTYPE_BF16, TS_DTYPE_F32 = 0, 1
TS_GQA_MOD, TS_GQA_DIV = 0, 1
TS_FLAG_DENSE, TS_FLAG_RECOMPUTE, TS_FLAG_REUSE = 0, 1, 2
TS_CFG_PLAIN_SCORE = 1
TS_CFG_PHASE_STAMPS = 32
TS_ABI_VERSION = 3

# every symbol include/tokenselect_b200.h declares
EXPORTS = [
    "ts_abi_version", "ts_status_string", "ts_query_workspace", "ts_vote_buffer_elems", "ts_create",
    "ts_destroy", "ts_reset_request", "ts_decode_layer", "ts_tp_prepare", "ts_tp_score_vote",
    "ts_tp_select_attend", "ts_get_counters", "ts_last_error", "ts_last_cuda_error", "ts_debug_read",
    "ts_launch_count", "ts_timing_begin", "ts_timing_end", "ts_attend_rows_static", "ts_tp_symmetric_bytes", "ts_tp_attach_peers",
    "ts_extend_chunk",
]


class TsConfig(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32), ("n_layers", C.c_int32), ("hq", C.c_int32),
        ("hkv", C.c_int32), ("head_dim", C.c_int32), ("dtype", C.c_int32), ("n_init", C.c_int32),
        ("n_local", C.c_int32), ("top_k", C.c_int32), ("kernel_size", C.c_int32), ("query_cache", C.c_int32),
        ("similarity_threshold", C.c_float), ("gqa_map", C.c_int32), ("rope_base", C.c_double),
        ("rope_scale", C.c_double), ("sm_scale", C.c_float), ("logit_cap", C.c_float), ("max_reqs", C.c_int32),
        ("max_batch", C.c_int32), ("max_ctx", C.c_int32), ("max_total_tokens", C.c_int64),
        ("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("flags", C.c_uint32), ("prefill_chunk", C.c_int32),
        ("wait_limit_us", C.c_uint32), ("reserved0", C.c_uint32),
        ("score_cos_sin", C.c_void_p), ("attn_cos_sin", C.c_void_p),
    ]


class TsDecodeArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("layer", C.c_int32), ("batch", C.c_int32), ("reserved", C.c_int32),
        ("q", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("out_cache_loc", C.c_void_p),
        ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("pool_rows", C.c_int64),
        ("req_to_token", C.c_void_p), ("req_to_token_stride", C.c_int64), ("req_pool_indices", C.c_void_p),
        ("seq_lens", C.c_void_p), ("out", C.c_void_p), ("tp_votes", C.c_void_p), ("tp_cos", C.c_void_p),
        ("dbg_sel_slots", C.c_void_p), ("dbg_sel_pos", C.c_void_p), ("dbg_sel_count", C.c_void_p),
        ("dbg_flags", C.c_void_p), ("stream", C.c_void_p),
    ]


class TsExtendArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("layer", C.c_int32), ("chunk_len", C.c_int32), ("req_pool_index", C.c_int32),
        ("seq_len", C.c_int32), ("reserved", C.c_int32),
        ("q", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("out_cache_loc", C.c_void_p),
        ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("pool_rows", C.c_int64),
        ("req_to_token", C.c_void_p), ("req_to_token_stride", C.c_int64), ("chunk_cos_sin", C.c_void_p),
        ("out", C.c_void_p), ("dbg_sel_slots", C.c_void_p), ("dbg_sel_pos", C.c_void_p),
        ("dbg_sel_count", C.c_void_p), ("dbg_flags", C.c_void_p), ("dbg_fingerprint", C.c_void_p),
        ("stream", C.c_void_p),
    ]


class TsAttendStaticArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("hq", C.c_int32), ("hkv", C.c_int32),
        ("head_dim", C.c_int32), ("count", C.c_int32), ("q", C.c_void_p), ("k_pool", C.c_void_p),
        ("v_pool", C.c_void_p), ("pool_rows", C.c_int64), ("rows", C.c_void_p), ("out", C.c_void_p),
        ("sm_scale", C.c_float), ("logit_cap", C.c_float), ("rope_base", C.c_double), ("rope_scale", C.c_double),
        ("status", C.c_void_p), ("stream", C.c_void_p),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and declare the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tokenselect_b200.build` "
            "(nvcc, sm_100a). tokenselect_b200 has no CPU or library fallback.")
    lib = C.CDLL(LIB_PATH)
    H = C.c_void_p
    for name in EXPORTS:
        getattr(lib, name).restype = C.c_int     # raises AttributeError if a symbol is missing
    lib.ts_status_string.restype = C.c_char_p
    lib.ts_status_string.argtypes = [C.c_int]
    lib.ts_query_workspace.argtypes = [C.POINTER(TsConfig), C.POINTER(C.c_size_t)]
    lib.ts_vote_buffer_elems.argtypes = [C.POINTER(TsConfig), C.POINTER(C.c_int64)]
    lib.ts_create.argtypes = [C.POINTER(TsConfig), C.POINTER(H)]
    lib.ts_destroy.argtypes = [H]
    lib.ts_reset_request.argtypes = [H, C.c_int32, C.c_void_p]
    for name in ("ts_decode_layer", "ts_tp_prepare", "ts_tp_score_vote", "ts_tp_select_attend"):
        getattr(lib, name).argtypes = [H, C.POINTER(TsDecodeArgs)]
    lib.ts_get_counters.argtypes = [H, C.c_int32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_void_p]
    lib.ts_last_error.argtypes = [H, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.ts_last_cuda_error.argtypes = [H]
    lib.ts_last_cuda_error.restype = C.c_char_p
    lib.ts_debug_read.argtypes = [H, C.c_int32, C.c_void_p, C.c_size_t]
    lib.ts_launch_count.argtypes = [H, C.POINTER(C.c_uint64)]
    lib.ts_timing_begin.argtypes = [H, C.c_int32]
    lib.ts_timing_end.argtypes = [H, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]
    lib.ts_attend_rows_static.argtypes = [C.POINTER(TsAttendStaticArgs)]
    lib.ts_tp_symmetric_bytes.argtypes = [C.POINTER(TsConfig), C.POINTER(C.c_size_t)]
    lib.ts_tp_attach_peers.argtypes = [H, C.POINTER(C.c_uint64), C.c_int32]
    lib.ts_extend_chunk.argtypes = [H, C.POINTER(TsExtendArgs)]
    if lib.ts_abi_version() != TS_ABI_VERSION:
        raise RuntimeError("libtokenselect_b200.so was built from a different header; rebuild it")
    _lib = lib
    return lib


class TokenSelectError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        msg = load().ts_status_string(status).decode()
        super().__init__(f"{what}: {msg} (status {status}){(' -- ' + detail) if detail else ''}")


def check(status: int, what: str, handle=None) -> None:
    if status != TS_OK:
        detail = ""
        if handle is not None and status == 3:
            detail = load().ts_last_cuda_error(handle).decode()
        raise TokenSelectError(status, what, detail)
