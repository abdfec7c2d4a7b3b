"""ctypes binding of liblf_sm100.so (declarations mirror include/lf_sm100.h).

Loading fails loudly: there is no Python or CPU substitute for the kernels.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "liblf_sm100.so"

LF_MAX_MODS = 8

# Every symbol include/lf_sm100.h declares.
EXPORTS = [
    "lf_query", "lf_strerror", "lf_last_cuda_error", "lf_prefill_bf16", "lf_skip_range",
    "lf_decode_bf16", "lf_decode_paged_bf16", "lf_decode_auto_splits",
    "lf_decode_workspace_bytes", "lf_combine_f32", "lf_paged_gather_bf16",
    "lf_decode_bf16_static", "lf_prefill_kv_tile", "lf_prefill_q_tile", "lf_tile_map_cache_stats",
    "lf_kv_append_bf16", "lf_selftest_wait_timeout", "lf_add_bf16", "lf_debug_bounds",
]

LF_STATIC_SCRATCH_BYTES = 8 << 20


class LfPrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32),
        ("Skv", C.c_int32), ("D", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("scale", C.c_float), ("n_mod", C.c_int32),
        ("mod_op", C.c_int32 * LF_MAX_MODS), ("mod_arg", C.c_float * LF_MAX_MODS),
        ("mask_kind", C.c_int32), ("window", C.c_int32), ("causal_offset", C.c_int32),
        ("status", C.c_void_p), ("dbg_ranges", C.c_void_p), ("kv_tile", C.c_int32),
        ("k_block_table", C.c_void_p), ("v_block_table", C.c_void_p), ("bt_stride", C.c_int64),
        ("page_size", C.c_int32), ("n_pages", C.c_int32),
        ("sm_margin", C.c_int32),
        ("score_bias", C.c_void_p), ("bias_stride", C.c_int64 * 3), ("bias_pos", C.c_int32),
        ("q_pe", C.c_void_p), ("k_pe", C.c_void_p), ("qpe_stride", C.c_int64 * 3),
        ("kpe_stride", C.c_int64 * 3), ("D_pe", C.c_int32),
    ]


class LfDecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("B", C.c_int32), ("Hkv", C.c_int32), ("G", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("scale", C.c_float), ("n_mod", C.c_int32),
        ("mod_op", C.c_int32 * LF_MAX_MODS), ("mod_arg", C.c_float * LF_MAX_MODS),
        ("block_table", C.c_void_p), ("block_table_v", C.c_void_p), ("bt_stride", C.c_int64),
        ("page_size", C.c_int32), ("n_pages", C.c_int32),
        ("splits", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
    ]


class LfKvAppendArgs(C.Structure):
    _fields_ = [
        ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("k_pool", C.c_void_p),
        ("v_pool", C.c_void_p), ("block_table", C.c_void_p), ("block_table_v", C.c_void_p),
        ("seq_pos", C.c_void_p), ("start_pos", C.c_int32),
        ("B", C.c_int32), ("Hkv", C.c_int32), ("T", C.c_int32), ("D", C.c_int32),
        ("kn_stride", C.c_int64 * 3), ("vn_stride", C.c_int64 * 3),
        ("kp_stride", C.c_int64 * 3), ("vp_stride", C.c_int64 * 3),
        ("bt_stride", C.c_int64), ("bt_blocks", C.c_int32), ("page_size", C.c_int32),
        ("n_pages", C.c_int32), ("status", C.c_void_p),
    ]


class LfDeviceInfo(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("device", C.c_int32), ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32), ("sm_count", C.c_int32), ("max_smem_optin", C.c_int32),
        ("total_mem", C.c_int64),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the kernel library (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = LIB_PATH
    if os.environ.get("LF_DEBUG_BOUNDS", "0") not in ("", "0"):
        # the range-checking build of the same sources (python -m loopfuse_b200.build
        # --debug-bounds); results are the same, violations show up in the status word
        path = LIB_PATH.with_name("liblf_sm100_dbg.so")
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m loopfuse_b200.build` "
            "(needs nvcc). There is no fallback implementation.")
    lib = C.CDLL(str(path))
    lib.lf_debug_bounds.argtypes = []
    lib.lf_debug_bounds.restype = C.c_int
    lib.lf_query.argtypes = [C.POINTER(LfDeviceInfo)]
    lib.lf_query.restype = C.c_int
    lib.lf_strerror.argtypes = [C.c_int]
    lib.lf_strerror.restype = C.c_char_p
    lib.lf_last_cuda_error.argtypes = []
    lib.lf_last_cuda_error.restype = C.c_char_p
    lib.lf_prefill_bf16.argtypes = [C.POINTER(LfPrefillArgs), C.c_void_p]
    lib.lf_prefill_bf16.restype = C.c_int
    lib.lf_prefill_q_tile.argtypes = [C.POINTER(LfPrefillArgs)]
    lib.lf_prefill_q_tile.restype = C.c_int
    lib.lf_prefill_kv_tile.argtypes = [C.POINTER(LfPrefillArgs)]
    lib.lf_prefill_kv_tile.restype = C.c_int
    lib.lf_tile_map_cache_stats.argtypes = [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    lib.lf_tile_map_cache_stats.restype = None
    lib.lf_kv_append_bf16.argtypes = [C.POINTER(LfKvAppendArgs), C.c_void_p]
    lib.lf_kv_append_bf16.restype = C.c_int
    lib.lf_add_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                C.c_int32, C.c_int32, C.POINTER(C.c_int64),
                                C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_void_p]
    lib.lf_add_bf16.restype = C.c_int
    lib.lf_selftest_wait_timeout.argtypes = [C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.lf_selftest_wait_timeout.restype = C.c_int
    lib.lf_skip_range.argtypes = [C.c_int32] * 8 + [C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.lf_skip_range.restype = None
    for name in ("lf_decode_bf16", "lf_decode_paged_bf16", "lf_decode_bf16_static"):
        fn = getattr(lib, name)
        fn.argtypes = [C.POINTER(LfDecodeArgs), C.c_void_p]
        fn.restype = C.c_int
    lib.lf_decode_auto_splits.argtypes = [C.c_int32] * 6
    lib.lf_decode_auto_splits.restype = C.c_int
    lib.lf_decode_workspace_bytes.argtypes = [C.c_int32] * 5
    lib.lf_decode_workspace_bytes.restype = C.c_size_t
    lib.lf_combine_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                   C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64),
                                   C.c_void_p]
    lib.lf_combine_f32.restype = C.c_int
    lib.lf_paged_gather_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.POINTER(C.c_int64), C.c_int64, C.c_void_p,
                                         C.c_void_p]
    lib.lf_paged_gather_bf16.restype = C.c_int
    _lib = lib
    return lib


class LfError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = load()
        msg = lib.lf_strerror(rc).decode()
        cuda = lib.lf_last_cuda_error().decode()
        raise LfError(f"{what} failed: {msg} [{rc}]" + (f" - {cuda}" if rc == -5 and cuda else ""))


def c_skip_range(mask_kind: int, window: int, causal_offset: int, s_q: int, s_kv: int,
                 tile_q: int, tile_k: int, iq: int) -> tuple[int, int]:
    lo, hi = C.c_int32(), C.c_int32()
    load().lf_skip_range(mask_kind, window, causal_offset, s_q, s_kv, tile_q, tile_k, iq,
                         C.byref(lo), C.byref(hi))
    return lo.value, hi.value
