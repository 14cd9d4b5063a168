"""ctypes binding of the C ABI declared in `include/flb200_attn.h`.

The shared library is the product: there is no Python, PyTorch or CPU
implementation behind these calls.  `load()` raises if the library has not been
built (`python -m flashlight_b200.build`).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# FLB200_LIBRARY selects another build of the same ABI (e.g. one compiled with tracing)
LIB_PATH = Path(os.environ.get("FLB200_LIBRARY") or Path(__file__).resolve().parent / "libflb200.so")

# flb200_status
OK = 0
E_BAD_ARG = -1
E_UNSUPPORTED = -2
E_MISALIGNED = -3
E_WORKSPACE = -4
E_ARCH = -5
E_LAUNCH = -6
E_TIMEOUT = -7

SCORE_NONE, SCORE_ALIBI, SCORE_SOFTCAP, SCORE_BIAS = 0, 1, 2, 3
PW_IDENTITY, PW_RELU, PW_TANH, PW_SIGMOID = 0, 1, 2, 3
MASK_NONE, MASK_CAUSAL, MASK_SLIDING, MASK_PREFIX, MASK_DOCUMENT = 0, 1, 2, 3, 4

ABI_VERSION = 3
NOALLOC_SCRATCH_BYTES = 1 << 20


class AttnParams(C.Structure):
    """Mirror of `flb200_attn_params` (field order and types must match the header)."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("diff", C.c_int32),
        ("N", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("L", C.c_int32),
        ("S", C.c_int32), ("E", C.c_int32), ("Ev", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("scale", C.c_float),
        ("score_mod", C.c_int32),
        ("alibi_heads", C.c_int32),
        ("softcap", C.c_float),
        ("bias", C.c_void_p * 2),
        ("bias_stride", (C.c_int64 * 4) * 2),
        ("bias_inner", C.c_int32),
        ("mask", C.c_int32),
        ("causal", C.c_int32),
        ("window", C.c_int32),
        ("prefix_len", C.c_void_p),
        ("prefix_scalar", C.c_int32),
        ("document_id", C.c_void_p),
        ("doc_stride_n", C.c_int64),
        ("diff_lambda", C.c_float),
        ("diff_rms_norm", C.c_int32),
        ("diff_rms_eps", C.c_float),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("block_map_ready", C.c_int32),
        ("status", C.c_void_p),
        ("lse", C.c_void_p),
        ("lse_stride", C.c_int64 * 2),
        ("wait_limit_us", C.c_uint32),
        ("status_host", C.c_void_p),
        ("alibi_head0", C.c_int32),
        ("product_chain", C.c_int32),
        ("pointwise", C.c_int32),
        ("k_keys_contiguous", C.c_int32),
    ]


class AttnBwdParams(C.Structure):
    """Mirror of `flb200_attn_bwd_params`."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("N", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("L", C.c_int32), ("S", C.c_int32), ("E", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("dout", C.c_void_p),
        ("lse", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3), ("do_stride", C.c_int64 * 3),
        ("dq_stride", C.c_int64 * 3), ("dk_stride", C.c_int64 * 3), ("dv_stride", C.c_int64 * 3),
        ("lse_stride", C.c_int64 * 2),
        ("scale", C.c_float),
        ("causal", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("status_host", C.c_void_p),
        ("wait_limit_us", C.c_uint32),
    ]


class IpaPackParams(C.Structure):
    """Mirror of `flb200_ipa_pack_params`."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("rows_q", C.c_int32), ("rows_k", C.c_int32),
        ("C", C.c_int32), ("P_qk", C.c_int32), ("P_v", C.c_int32), ("point_dim", C.c_int32),
        ("q_scalar", C.c_void_p), ("k_scalar", C.c_void_p), ("v_scalar", C.c_void_p),
        ("q_points", C.c_void_p), ("k_points", C.c_void_p), ("v_points", C.c_void_p),
        ("a", C.c_float),
        ("E", C.c_int32), ("Ev", C.c_int32),
        ("q_aug", C.c_void_p), ("k_aug", C.c_void_p), ("v_aug", C.c_void_p),
    ]


EXPORTS = (
    "flb200_abi_version",
    "flb200_strerror",
    "flb200_attn_validate",
    "flb200_attn_workspace_bytes",
    "flb200_build_block_map",
    "flb200_attn_fwd",
    "flb200_attn_fwd_noalloc",
    "flb200_selftest_wait_timeout",
    "flb200_attn_bwd_workspace_bytes",
    "flb200_attn_bwd",
    "flb200_selftest_bwd_wait_timeout",
    "flb200_ipa_pack",
    "flb200_decode_status",
    "flb200_launch_count",
)

_lib = None


def load() -> C.CDLL:
    """Load `libflb200.so` once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flashlight_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    P = C.POINTER(AttnParams)
    lib.flb200_abi_version.restype = C.c_uint32
    lib.flb200_abi_version.argtypes = []
    lib.flb200_strerror.restype = C.c_char_p
    lib.flb200_strerror.argtypes = [C.c_int]
    lib.flb200_attn_validate.restype = C.c_int
    lib.flb200_attn_validate.argtypes = [P]
    lib.flb200_attn_workspace_bytes.restype = C.c_size_t
    lib.flb200_attn_workspace_bytes.argtypes = [P]
    lib.flb200_build_block_map.restype = C.c_int
    lib.flb200_build_block_map.argtypes = [P, C.c_void_p]
    lib.flb200_attn_fwd.restype = C.c_int
    lib.flb200_attn_fwd.argtypes = [P, C.c_void_p]
    lib.flb200_attn_fwd_noalloc.restype = C.c_int
    lib.flb200_attn_fwd_noalloc.argtypes = [P, C.c_void_p]
    lib.flb200_selftest_wait_timeout.restype = C.c_int
    lib.flb200_selftest_wait_timeout.argtypes = [P, C.c_void_p]
    PB = C.POINTER(AttnBwdParams)
    lib.flb200_attn_bwd_workspace_bytes.restype = C.c_size_t
    lib.flb200_attn_bwd_workspace_bytes.argtypes = [PB]
    lib.flb200_attn_bwd.restype = C.c_int
    lib.flb200_attn_bwd.argtypes = [PB, C.c_void_p]
    lib.flb200_selftest_bwd_wait_timeout.restype = C.c_int
    lib.flb200_selftest_bwd_wait_timeout.argtypes = [PB, C.c_void_p]
    lib.flb200_ipa_pack.restype = C.c_int
    lib.flb200_ipa_pack.argtypes = [C.POINTER(IpaPackParams), C.c_void_p]
    lib.flb200_decode_status.restype = C.c_int
    lib.flb200_decode_status.argtypes = [C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.flb200_launch_count.restype = C.c_uint64
    lib.flb200_launch_count.argtypes = []
    if lib.flb200_abi_version() != ABI_VERSION:
        raise RuntimeError("libflb200.so was built from a different header (ABI version mismatch)")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().flb200_strerror(code).decode()


def new_params() -> AttnParams:
    p = AttnParams()
    p.struct_size = C.sizeof(AttnParams)
    return p
