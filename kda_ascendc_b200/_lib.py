"""ctypes binding of libkda_b200.so (declarations: include/kda_b200.h).

There is no fallback: if the shared library is missing, importing the kernels
raises, and every entry point refuses tensors that are not on a CUDA device.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libkda_b200.so"

KDA_G_FP32, KDA_G_BF16 = 0, 1
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024   # KDA_STATIC_SCRATCH_BYTES of include/kda_b200.h
FLAG_GATE, FLAG_L2NORM, FLAG_BETA_SIGMOID, FLAG_STATE_K_FIRST = 1, 2, 4, 8

EXPORTS = (
    "kda_fwd_workspace_bytes", "kda_fwd", "kda_fwd_k1", "kda_fwd_k2", "kda_fwd_k2_state", "kda_recurrent_fwd",
    "kda_varlen_fill_tables", "kda_selftest_bounded_wait", "kda_fwd_static_scratch",
    "kda_fwd_static_scratch_status", "kda_state_fold", "kda_state_fold_ex", "kda_state_fold_peer", "kda_peer_push", "kda_fwd_k2_state_push", "kda_fwd_k2_after_flags",
    "kda_flag_wait", "kda_peer_enable", "kda_ipc_export", "kda_ipc_open", "kda_ipc_close",
    "kda_fwd_status", "kda_fwd_k2_choice", "kda_last_launch_count", "kda_last_error", "kda_version",
)


class KdaFwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("g", ctypes.c_void_p),
        ("beta", ctypes.c_void_p), ("A_log", ctypes.c_void_p), ("dt_bias", ctypes.c_void_p),
        ("h0", ctypes.c_void_p), ("o", ctypes.c_void_p), ("ht", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("g_out", ctypes.c_void_p), ("ainv_out", ctypes.c_void_p),
        ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("g_dtype", ctypes.c_int32),
        ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3), ("v_stride", ctypes.c_int64 * 3),
        ("g_stride", ctypes.c_int64 * 3), ("o_stride", ctypes.c_int64 * 3), ("beta_stride", ctypes.c_int64 * 3),
        ("scale", ctypes.c_float), ("lower_bound", ctypes.c_float), ("flags", ctypes.c_uint32),
        ("k2_vsplit", ctypes.c_int32), ("k2_variant", ctypes.c_int32),
        ("n_seqs", ctypes.c_int32), ("chunk_table", ctypes.c_void_p), ("seq_table", ctypes.c_void_p),
        ("n_chunks", ctypes.c_int32), ("Hq", ctypes.c_int32),
    ]


class KdaFoldArgs(ctypes.Structure):
    _fields_ = [
        ("mq", ctypes.c_void_p), ("seg_stride", ctypes.c_int64), ("chain_stride", ctypes.c_int64),
        ("h0", ctypes.c_void_p), ("h0_stride", ctypes.c_int64),
        ("s_in", ctypes.c_void_p), ("final_out", ctypes.c_void_p), ("final_stride", ctypes.c_int64),
        ("n_chains", ctypes.c_int32), ("n_seg", ctypes.c_int32), ("use_q", ctypes.c_int32),
        ("status", ctypes.c_void_p),
    ]


MAX_PEERS = 16
ERR_UNSUPPORTED = -4


class KdaPeerPushArgs(ctypes.Structure):
    _fields_ = [
        ("src", ctypes.c_void_p), ("dst", ctypes.c_void_p * MAX_PEERS), ("flag", ctypes.c_void_p * MAX_PEERS),
        ("counter", ctypes.c_void_p), ("slice_floats", ctypes.c_int64), ("dst_offset_floats", ctypes.c_int64),
        ("world", ctypes.c_int32), ("epoch", ctypes.c_int32),
    ]


class KdaFoldPeerArgs(ctypes.Structure):
    _fields_ = [
        ("wait_flags", ctypes.c_void_p), ("n_wait", ctypes.c_int32), ("epoch", ctypes.c_int32),
        ("s_in_seg", ctypes.c_void_p * (MAX_PEERS + 1)), ("signal", ctypes.c_void_p * MAX_PEERS),
        ("n_signal", ctypes.c_int32), ("counter", ctypes.c_void_p),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            "%s is missing: build it with `python -m kda_ascendc_b200.build` "
            "(there is no CPU or PyTorch fallback for the KDA kernels)" % LIB_PATH)
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.kda_fwd_workspace_bytes.restype = ctypes.c_size_t
    lib.kda_fwd_workspace_bytes.argtypes = [ctypes.c_int32] * 3
    for name in ("kda_fwd", "kda_fwd_k1", "kda_fwd_k2", "kda_fwd_static_scratch", "kda_recurrent_fwd"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(KdaFwdArgs), ctypes.c_void_p]
    lib.kda_fwd_k2_state.restype = ctypes.c_int
    lib.kda_fwd_k2_state.argtypes = [ctypes.POINTER(KdaFwdArgs), ctypes.c_int, ctypes.c_void_p]
    lib.kda_state_fold.restype = ctypes.c_int
    lib.kda_state_fold.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.kda_state_fold_ex.restype = ctypes.c_int
    lib.kda_state_fold_ex.argtypes = [ctypes.POINTER(KdaFoldArgs), ctypes.c_void_p]
    lib.kda_state_fold_peer.restype = ctypes.c_int
    lib.kda_state_fold_peer.argtypes = [ctypes.POINTER(KdaFoldArgs), ctypes.POINTER(KdaFoldPeerArgs), ctypes.c_void_p]
    lib.kda_fwd_k2_state_push.restype = ctypes.c_int
    lib.kda_fwd_k2_state_push.argtypes = [ctypes.POINTER(KdaFwdArgs), ctypes.POINTER(KdaPeerPushArgs), ctypes.c_void_p]
    lib.kda_fwd_k2_after_flags.restype = ctypes.c_int
    lib.kda_fwd_k2_after_flags.argtypes = [ctypes.POINTER(KdaFwdArgs), ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.kda_peer_push.restype = ctypes.c_int
    lib.kda_peer_push.argtypes = [ctypes.POINTER(KdaPeerPushArgs), ctypes.c_void_p]
    lib.kda_peer_enable.restype = ctypes.c_int
    lib.kda_peer_enable.argtypes = [ctypes.c_int32]
    lib.kda_ipc_export.restype = ctypes.c_int
    lib.kda_ipc_export.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]
    lib.kda_ipc_open.restype = ctypes.c_int
    lib.kda_ipc_open.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]
    lib.kda_ipc_close.restype = ctypes.c_int
    lib.kda_ipc_close.argtypes = [ctypes.c_void_p]
    lib.kda_flag_wait.restype = ctypes.c_int
    lib.kda_flag_wait.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.kda_selftest_bounded_wait.restype = ctypes.c_int
    lib.kda_selftest_bounded_wait.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.kda_varlen_fill_tables.restype = ctypes.c_int
    lib.kda_varlen_fill_tables.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, ctypes.c_int32,
                                           ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    lib.kda_fwd_k2_choice.restype = ctypes.c_int
    lib.kda_fwd_k2_choice.argtypes = [ctypes.POINTER(KdaFwdArgs), ctypes.c_int, ctypes.c_int,
                                      ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    lib.kda_fwd_status.restype = ctypes.c_int
    lib.kda_fwd_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
    lib.kda_fwd_static_scratch_status.restype = ctypes.c_int
    lib.kda_fwd_static_scratch_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
    lib.kda_last_launch_count.restype = ctypes.c_int
    lib.kda_last_error.restype = ctypes.c_char_p
    lib.kda_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def last_error() -> str:
    return load().kda_last_error().decode("utf-8", "replace")
