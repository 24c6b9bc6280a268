"""ctypes binding of ``include/megaattn_b200.h``.

There is no fallback: if the shared library is missing (and cannot be built) or a symbol
is absent, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

MA_MAX_TP = 8
MA_FLAG_FA_ONLY = 1
MA_FLAG_DRAIN_FIRST = 2
MA_FLAG_TILE_ORDER = 4
MA_FLAG_AR_ONLY = 8
MA_FLAG_NO_AR = 16
MA_FLAG_OPROJ_ONLY = 32
MA_FLAG_AR_P2P = 64

MA_OK = 0
MA_ERR_INVALID = -1
MA_ERR_CUDA = -2
MA_ERR_NOT_SM100 = -3
MA_ERR_DEVICE_TIMEOUT = -4
MA_ERR_CAPACITY = -5

EXPORTS = ("ma_query_device", "ma_plan_create", "ma_launch", "ma_plan_set_inputs", "ma_read_status",
           "ma_plan_destroy", "ma_strerror", "ma_fused_prefill_noalloc", "ma_residual_rmsnorm", "ma_rope_qk")

MA_NOALLOC_OSCRATCH_BYTES = 16 << 20
MA_NOALLOC_MAX_BATCH = 512
MA_NOALLOC_MAX_ROW_TILES = 512
MA_NOALLOC_MAX_SLOTS = 4096


class DevInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "cc_major", "cc_minor", "num_sms", "max_smem_optin",
        "kernel_threads", "kernel_smem_bytes", "kernel_regs", "max_ctas")]


class PlanDesc(C.Structure):
    _fields_ = (
        [(n, C.c_int32) for n in (
            "device", "tp_size", "rank", "H_local", "H_kv", "D", "hidden",
            "super_group_n_tiles", "max_row_tiles", "max_batch", "max_tot_q", "max_tot_k")]
        + [("softmax_scale", C.c_float), ("wait_limit_ms", C.c_uint32)]
        + [(n, C.c_uint64) for n in (
            "Q", "K", "V", "W_o", "o_scratch", "csym",
            "ctrl", "sync_ctrl", "actv", "head_ready", "oproj_queue",
            "ready_count", "ready_bits", "ar_done_bits", "nvl_signal",
            "cu_q", "cu_k", "fa_b", "fa_mb", "status", "csym_multicast")]
        + [("peer_ready_count", C.c_uint64 * MA_MAX_TP),
           ("peer_ready_bits", C.c_uint64 * MA_MAX_TP),
           ("peer_nvl_signal", C.c_uint64 * MA_MAX_TP),
           ("page_table", C.c_uint64), ("cache_seqlens", C.c_uint64),
           ("max_pages_per_seq", C.c_int32), ("reserved0", C.c_int32),
           ("fa_order", C.c_uint64),
           ("peer_csym", C.c_uint64 * MA_MAX_TP),
           ("audit", C.c_uint64)]
    )


class LaunchArgs(C.Structure):
    _fields_ = [("w_fa", C.c_int32), ("w_oproj", C.c_int32), ("w_ar", C.c_int32),
                ("num_ctas", C.c_int32), ("flags", C.c_uint32)]


class Status(C.Structure):
    _fields_ = [("code", C.c_uint32), ("site", C.c_uint32), ("cta", C.c_uint32),
                ("aux", C.c_uint32)]


class NoAllocArgs(C.Structure):
    _fields_ = [("H_local", C.c_int32), ("H_kv", C.c_int32), ("hidden", C.c_int32),
                ("super_group_n_tiles", C.c_int32), ("num_batch", C.c_int32),
                ("w_fa", C.c_int32), ("w_oproj", C.c_int32), ("num_ctas", C.c_int32),
                ("softmax_scale", C.c_float), ("wait_limit_ms", C.c_uint32),
                ("seqlens_q", C.POINTER(C.c_int32)), ("seqlens_k", C.POINTER(C.c_int32)),
                ("Q", C.c_uint64), ("K", C.c_uint64), ("V", C.c_uint64), ("W_o", C.c_uint64),
                ("out", C.c_uint64), ("status_out", C.POINTER(Status))]


class RmsNormArgs(C.Structure):
    _fields_ = [("csym", C.c_uint64), ("residual_in", C.c_uint64), ("weight", C.c_uint64),
                ("residual_out", C.c_uint64), ("normed_out", C.c_uint64),
                ("cu_q", C.c_uint64), ("fa_b", C.c_uint64), ("fa_mb", C.c_uint64),
                ("num_row_tiles", C.c_int32), ("hidden", C.c_int32), ("row_pitch", C.c_int32),
                ("eps", C.c_float)]


class RopeArgs(C.Structure):
    _fields_ = [("q", C.c_uint64), ("k", C.c_uint64), ("cu_q", C.c_uint64), ("cu_k", C.c_uint64),
                ("token_batch", C.c_uint64), ("inv_freq", C.c_uint64), ("tot_q", C.c_int32),
                ("H_local", C.c_int32), ("H_kv", C.c_int32), ("reserved0", C.c_int32)]


def _load(path=None, audit=False):
    path = path or (_build.LIB_AUDIT if audit else _build.LIB)
    if not os.path.exists(path) or _build._stale(path):
        try:
            _build.build(audit=audit)     # under a file lock, into a temporary file, then renamed
        except Exception as exc:  # no nvcc on this machine: use what is there, if anything
            if not os.path.exists(path):
                raise ImportError(f"{os.path.basename(path)} is missing and cannot be built: {exc}")
    lib = C.CDLL(path)
    for name in EXPORTS:
        getattr(lib, name)     # AttributeError if the library does not export it
    lib.ma_query_device.argtypes = [C.c_int, C.POINTER(DevInfo)]
    lib.ma_query_device.restype = C.c_int
    lib.ma_plan_create.argtypes = [C.POINTER(PlanDesc), C.POINTER(C.c_void_p)]
    lib.ma_plan_create.restype = C.c_int
    lib.ma_launch.argtypes = [C.c_void_p, C.POINTER(LaunchArgs), C.c_void_p]
    lib.ma_launch.restype = C.c_int
    lib.ma_plan_set_inputs.argtypes = [C.c_void_p] + [C.c_uint64] * 4 + [C.c_int64] * 3
    lib.ma_plan_set_inputs.restype = C.c_int
    lib.ma_read_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(Status)]
    lib.ma_read_status.restype = C.c_int
    lib.ma_plan_destroy.argtypes = [C.c_void_p]
    lib.ma_plan_destroy.restype = None
    lib.ma_fused_prefill_noalloc.argtypes = [C.POINTER(NoAllocArgs), C.c_void_p]
    lib.ma_fused_prefill_noalloc.restype = C.c_int
    lib.ma_residual_rmsnorm.argtypes = [C.POINTER(RmsNormArgs), C.c_void_p]
    lib.ma_residual_rmsnorm.restype = C.c_int
    lib.ma_rope_qk.argtypes = [C.POINTER(RopeArgs), C.c_void_p]
    lib.ma_rope_qk.restype = C.c_int
    lib.ma_strerror.argtypes = [C.c_int]
    lib.ma_strerror.restype = C.c_char_p
    return lib


lib = _load()
_audit_lib = None


def audit_lib():
    """The audit build of the library (same ABI, compiled with -DMA_AUDIT: the kernel counts
    executions per task into ``ma_plan_desc.audit``).  Loaded on first use; tests only."""
    global _audit_lib
    if _audit_lib is None:
        _audit_lib = _load(audit=True)
    return _audit_lib


def strerror(code: int) -> str:
    return lib.ma_strerror(int(code)).decode()


def check(code: int, what: str):
    if code != MA_OK:
        raise RuntimeError(f"{what}: {strerror(code)} ({code})")
