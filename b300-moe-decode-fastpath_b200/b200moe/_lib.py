"""ctypes binding of libb200moe.so (declarations: include/b200moe.h).

This is the only place the Python side touches native code.  It takes the
place of the reference's pybind11 module ``fastpath._C`` (csrc/bindings.cpp:24-99),
but the boundary is a plain C ABI: device pointers as integers, sizes, and the
CUDA stream handle.  A missing library is an error, never a fallback.
"""

from __future__ import annotations

import ctypes
import json
import os
import threading
from pathlib import Path
from typing import Mapping

LIBRARY_NAME = "libb200moe.so"
ABI_VERSION = 5

STATUS_BAD_EXPERT_ID = 0x1
STATUS_PIPE_TIMEOUT = 0x2
STATUS_PEER_TIMEOUT = 0x4

FLAG_PDL = 0x1
FLAG_LOCAL_EXPERTS = 0x2
FLAG_F32_OUTPUT = 0x4
FLAG_FP8_WEIGHTS = 0x8
FLAG_HOST_IO = 0x10
FLAG_SKIP_COMBINE = 0x20
FLAG_EP_PUSH = 0x40
FLAG_NVFP4_WEIGHTS = 0x80
FLAG_EP_AFTER_PUSH = 0x100

STATIC_ROUTING_MAX_ASSIGNMENTS = 4096

TUNE_STAGE_KB = 1
TUNE_L2_PROMOTION = 2
TUNE_EVICT_FIRST = 3
TUNE_SMALL_CALL_MAX = 4
TUNE_DOWN_TARGET = 5
TUNE_DOWN_SPLITS = 6
TUNE_FP8_SEG_ROWS = 7
TUNE_NVFP4_PREFETCH = 8
TUNE_NVFP4_ISSUERS = 9
TUNE_GEMM_OVERLAP = 10

EXPORTS = (
    "b200moe_abi_version",
    "b200moe_build_info",
    "b200moe_error_string",
    "b200moe_scratch_bytes",
    "b200moe_routing",
    "b200moe_routing_static",
    "b200moe_gather",
    "b200moe_gate_up_swiglu",
    "b200moe_down",
    "b200moe_combine",
    "b200moe_forward",
    "b200moe_dispatch",
    "b200moe_dispatch_scratch_bytes",
    "b200moe_combine_bf16",
    "b200moe_ep_reduce",
    "b200moe_ep_combine_reduce",
    "b200moe_ep_push_max_blocks",
    "b200moe_ep_push",
    "b200moe_status_ptr",
    "b200moe_nvfp4_available",
    "b200moe_nvfp4_scale_bytes",
    "b200moe_nvfp4_quantize",
    "b200moe_nvfp4_rows_to_planes",
    "b200moe_tune",
    "b200moe_router_topk",
    "b200moe_fp8_quantize_rows",
    "b200moe_fp8_dequantize_rows",
)


class B200MoeArgs(ctypes.Structure):
    """Mirror of ``struct B200MoeArgs`` in include/b200moe.h (field order matters)."""

    _fields_ = [
        ("hidden_states", ctypes.c_void_p),
        ("expert_indices", ctypes.c_void_p),
        ("expert_weights", ctypes.c_void_p),
        ("gate_up_weight", ctypes.c_void_p),
        ("down_weight", ctypes.c_void_p),
        ("num_tokens", ctypes.c_int32),
        ("top_k", ctypes.c_int32),
        ("num_experts", ctypes.c_int32),
        ("hidden_size", ctypes.c_int32),
        ("intermediate_size", ctypes.c_int32),
        ("rows_cap", ctypes.c_int32),
        ("expert_counts", ctypes.c_void_p),
        ("expert_offsets", ctypes.c_void_p),
        ("expert_offsets_i32", ctypes.c_void_p),
        ("permutation", ctypes.c_void_p),
        ("reverse_mapping", ctypes.c_void_p),
        ("permuted_token_indices", ctypes.c_void_p),
        ("permuted_expert_indices", ctypes.c_void_p),
        ("permuted_weights", ctypes.c_void_p),
        ("permuted_hidden", ctypes.c_void_p),
        ("swiglu_output", ctypes.c_void_p),
        ("expert_output", ctypes.c_void_p),
        ("scratch", ctypes.c_void_p),
        ("scratch_bytes", ctypes.c_size_t),
        ("output", ctypes.c_void_p),
        ("flags", ctypes.c_uint32),
        ("expert_id_base", ctypes.c_int32),
        ("ep_wait_flags", ctypes.c_void_p),
        ("ep_world", ctypes.c_int32),
        ("ep_epoch", ctypes.c_uint32),
        ("ep_wait_limit_us", ctypes.c_uint32),
        ("gate_up_scale", ctypes.c_void_p),
        ("down_scale", ctypes.c_void_p),
        ("gate_up_block_scale", ctypes.c_void_p),
        ("down_block_scale", ctypes.c_void_p),
    ]


class B200MoeEpReduceArgs(ctypes.Structure):
    """Mirror of ``struct B200MoeEpReduceArgs`` in include/b200moe.h."""

    _fields_ = [
        ("partial_ptrs", ctypes.POINTER(ctypes.c_void_p)),
        ("flag_ptrs", ctypes.POINTER(ctypes.c_void_p)),
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("num_tokens", ctypes.c_int32),
        ("hidden_size", ctypes.c_int32),
        ("epoch", ctypes.c_uint32),
        ("wait_limit_us", ctypes.c_uint32),
        ("output", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("flags", ctypes.c_uint32),
        ("first_token", ctypes.c_int32),
        ("block_counter", ctypes.c_void_p),
        ("inbox_ptrs", ctypes.POINTER(ctypes.c_void_p)),
        ("inbox_cap_tokens", ctypes.c_int32),
        ("tokens_per_rank", ctypes.c_int32),
    ]


class B200MoeEpPushArgs(ctypes.Structure):
    """Mirror of ``struct B200MoeEpPushArgs`` in include/b200moe.h."""

    _fields_ = [
        ("hidden_states", ctypes.c_void_p),
        ("expert_indices", ctypes.c_void_p),
        ("expert_weights", ctypes.c_void_p),
        ("hidden_dst", ctypes.POINTER(ctypes.c_void_p)),
        ("indices_dst", ctypes.POINTER(ctypes.c_void_p)),
        ("weights_dst", ctypes.POINTER(ctypes.c_void_p)),
        ("flag_ptrs", ctypes.POINTER(ctypes.c_void_p)),
        ("block_counter", ctypes.c_void_p),
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("tokens_local", ctypes.c_int32),
        ("top_k", ctypes.c_int32),
        ("hidden_size", ctypes.c_int32),
        ("epoch", ctypes.c_uint32),
    ]


EP_MAX_WORLD = 8

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


def library_path() -> Path:
    override = os.environ.get("B200MOE_SO")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / LIBRARY_NAME


def _declare(lib: ctypes.CDLL) -> None:
    args_p = ctypes.POINTER(B200MoeArgs)
    lib.b200moe_abi_version.restype = ctypes.c_int
    lib.b200moe_abi_version.argtypes = []
    lib.b200moe_build_info.restype = ctypes.c_int
    lib.b200moe_build_info.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.b200moe_error_string.restype = ctypes.c_char_p
    lib.b200moe_error_string.argtypes = [ctypes.c_int]
    lib.b200moe_scratch_bytes.restype = ctypes.c_int
    lib.b200moe_scratch_bytes.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_size_t)]
    for name in (
        "b200moe_routing",
        "b200moe_routing_static",
        "b200moe_gather",
        "b200moe_gate_up_swiglu",
        "b200moe_down",
        "b200moe_combine",
        "b200moe_forward",
        "b200moe_dispatch",
    ):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [args_p, ctypes.c_void_p]
    lib.b200moe_dispatch_scratch_bytes.restype = ctypes.c_int
    lib.b200moe_dispatch_scratch_bytes.argtypes = [ctypes.c_int, ctypes.c_int,
                                                   ctypes.POINTER(ctypes.c_size_t)]
    lib.b200moe_ep_reduce.restype = ctypes.c_int
    lib.b200moe_ep_reduce.argtypes = [ctypes.POINTER(B200MoeEpReduceArgs), ctypes.c_void_p]
    lib.b200moe_ep_combine_reduce.restype = ctypes.c_int
    lib.b200moe_ep_combine_reduce.argtypes = [args_p, ctypes.POINTER(B200MoeEpReduceArgs),
                                              ctypes.c_void_p]
    lib.b200moe_ep_push_max_blocks.restype = ctypes.c_int
    lib.b200moe_ep_push_max_blocks.argtypes = [ctypes.POINTER(ctypes.c_int)]
    lib.b200moe_combine_bf16.restype = ctypes.c_int
    lib.b200moe_combine_bf16.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
    ]
    lib.b200moe_ep_push.restype = ctypes.c_int
    lib.b200moe_ep_push.argtypes = [ctypes.POINTER(B200MoeEpPushArgs), ctypes.c_void_p]
    lib.b200moe_status_ptr.restype = ctypes.c_int
    lib.b200moe_status_ptr.argtypes = [
        ctypes.c_void_p,
        ctypes.c_size_t,
        ctypes.POINTER(ctypes.c_void_p),
    ]
    lib.b200moe_nvfp4_available.restype = ctypes.c_int
    lib.b200moe_nvfp4_available.argtypes = []
    lib.b200moe_nvfp4_scale_bytes.restype = ctypes.c_int
    lib.b200moe_nvfp4_scale_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.POINTER(ctypes.c_size_t)]
    lib.b200moe_nvfp4_quantize.restype = ctypes.c_int
    lib.b200moe_nvfp4_quantize.argtypes = [
        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
    ]
    lib.b200moe_nvfp4_rows_to_planes.restype = ctypes.c_int
    lib.b200moe_nvfp4_rows_to_planes.argtypes = [
        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_void_p,
    ]
    lib.b200moe_router_topk.restype = ctypes.c_int
    lib.b200moe_router_topk.argtypes = [
        ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
    ]
    lib.b200moe_fp8_quantize_rows.restype = ctypes.c_int
    lib.b200moe_fp8_quantize_rows.argtypes = [
        ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_void_p,
    ]
    lib.b200moe_fp8_dequantize_rows.restype = ctypes.c_int
    lib.b200moe_fp8_dequantize_rows.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p,
        ctypes.c_void_p,
    ]
    lib.b200moe_tune.restype = ctypes.c_int
    lib.b200moe_tune.argtypes = [ctypes.c_int, ctypes.c_int]


def load() -> ctypes.CDLL:
    """Load the native library once; raise ``RuntimeError`` when it is absent.

    Same policy as the reference's ``_load_goal_1b_extension``
    (fastpath/b300_moe.py:394-401): a compiled backend that cannot be loaded is
    an error, not a reason to run something else.
    """

    global _library
    if _library is not None:
        return _library
    with _lock:
        if _library is not None:
            return _library
        path = library_path()
        if not path.exists():
            raise RuntimeError(
                f"{LIBRARY_NAME} is missing at {path}; build it for sm_100a with "
                "`python b300-moe-decode-fastpath_b200/build.py` (there is no fallback path)"
            )
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise RuntimeError(f"could not load {path}: {error}") from error
        missing = [name for name in EXPORTS if not hasattr(lib, name)]
        if missing:
            raise RuntimeError(f"{path} lacks required exports: {', '.join(missing)}")
        _declare(lib)
        version = lib.b200moe_abi_version()
        if version != ABI_VERSION:
            raise RuntimeError(f"{path} has ABI version {version}, expected {ABI_VERSION}")
        _library = lib
        return lib


def available() -> bool:
    """Whether the native library can be loaded (mirrors ``cuda_extension_available``)."""

    try:
        load()
    except RuntimeError:
        return False
    return True


def error_string(code: int) -> str:
    text = load().b200moe_error_string(int(code))
    return text.decode() if text else f"error {code}"


def check(code: int, what: str) -> None:
    """Raise for a non-zero return code of a native call."""

    if code == 0:
        return
    message = f"{what} failed: {error_string(code)} (code {code})"
    if code < 0:
        raise ValueError(message)
    raise RuntimeError(message)


def build_info() -> Mapping[str, object]:
    """The library's build attestation (mirrors ``fastpath._C.build_info()``)."""

    lib = load()
    buffer = ctypes.create_string_buffer(1024)
    lib.b200moe_build_info(buffer, len(buffer))
    return json.loads(buffer.value.decode())


def dispatch_scratch_bytes(rows_cap: int, num_experts: int) -> int:
    size = ctypes.c_size_t(0)
    check(load().b200moe_dispatch_scratch_bytes(rows_cap, num_experts, ctypes.byref(size)),
          "b200moe_dispatch_scratch_bytes")
    return int(size.value)


def scratch_bytes(
    max_tokens: int, top_k: int, num_experts: int, hidden_size: int, intermediate_size: int
) -> int:
    size = ctypes.c_size_t(0)
    code = load().b200moe_scratch_bytes(
        max_tokens, top_k, num_experts, hidden_size, intermediate_size, ctypes.byref(size)
    )
    check(code, "b200moe_scratch_bytes")
    return int(size.value)
