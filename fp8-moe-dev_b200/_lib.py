"""ctypes binding of the C ABI declared in include/moe_fp8_b200.h.

The library is the product: if it is missing or fails to load this module raises, there
is no Python or CPU fallback behind it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libmoe_fp8_b200.so"

OK = 0
ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_CAPACITY, ERR_DEVICE, ERR_UNSUPPORTED = -1, -2, -3, -4, -5
OPT_REFERENCE_PRUNING, OPT_EXACT_SILU, OPT_STAGE_TIMING = 1, 2, 3
OPT_STOP_AFTER_STAGE, OPT_DECODE_KERNEL, OPT_EXPERT_STRIDE, OPT_WAIT_LIMIT_US = 4, 5, 6, 7
OPT_WEIGHT_PRELAYOUT = 8
OPT_SMALL_BATCH_RING = 9
DECODE_MAX_TOKENS = 8

BUF = dict(
    expert_count=0, expert_offset=1, topk_idx=2, topk_weight=3, pair_count=4, pair_code=5, pair_weight=6,
    num_tiles=7, row_token=8, a1=9, sfa1=10, a2=11, sfa2=12, y=13, status=14, decode_timeline=15, exchange_timeline=16,
    pair_row=17,
)

EXPORTS = [
    "moe_fp8_b200_version", "moe_fp8_b200_workspace_bytes", "moe_fp8_b200_row_capacity",
    "moe_fp8_b200_create", "moe_fp8_b200_destroy", "moe_fp8_b200_last_error", "moe_fp8_b200_set_option",
    "moe_fp8_b200_run", "moe_fp8_b200_run_host", "moe_fp8_b200_check", "moe_fp8_b200_read_intermediate",
    "moe_fp8_b200_reference_policy", "moe_fp8_b200_stage_times", "moe_fp8_b200_route_noalloc",
    "moe_fp8_b200_exchange_bytes", "moe_fp8_b200_run_reduce_scatter", "moe_fp8_b200_quantize_hidden",
    "moe_fp8_b200_run_unfinalized", "moe_fp8_b200_finalize", "moe_fp8_b200_run_host_async",
    "moe_fp8_b200_host_wait", "moe_fp8_b200_set_expert_map", "moe_fp8_b200_inject_device_status",
    "moe_fp8_b200_exchange_regions", "moe_fp8_b200_copy_rows_h2d",
    "moe_fp8_b200_invalidate_weights", "moe_fp8_b200_copy_device", "moe_fp8_b200_signal_peers",
    "moe_fp8_b200_wait_peers", "moe_fp8_b200_create_shaped", "moe_fp8_b200_workspace_bytes_shaped",
    "moe_fp8_b200_get_shape",
]
NOALLOC_MAX_TOKENS = 4096


class Args(C.Structure):
    """moe_fp8_b200_args"""
    _fields_ = [
        ("routing_logits", C.c_void_p), ("routing_bias", C.c_void_p), ("hidden_states", C.c_void_p),
        ("hidden_states_scale", C.c_void_p), ("gemm1_weights", C.c_void_p), ("gemm1_weights_scale", C.c_void_p),
        ("gemm2_weights", C.c_void_p), ("gemm2_weights_scale", C.c_void_p), ("local_expert_offset", C.c_int64),
        ("routed_scaling_factor", C.c_double), ("output", C.c_void_p), ("num_tokens", C.c_int32),
    ]


class Shape(C.Structure):
    """moe_fp8_b200_shape"""
    _fields_ = [("hidden", C.c_int32), ("intermediate", C.c_int32), ("top_k", C.c_int32), ("n_group", C.c_int32),
                ("topk_group", C.c_int32)]


class Exchange(C.Structure):
    """moe_fp8_b200_exchange"""
    _fields_ = [("peer_buffers", C.c_void_p * 8), ("buffer_bytes", C.c_size_t), ("rank", C.c_int32),
                ("world", C.c_int32), ("epoch", C.c_uint32), ("capacity_tokens", C.c_int32)]


class Unfinalized(C.Structure):
    """moe_fp8_b200_unfinalized"""
    _fields_ = [("y", C.c_void_p), ("expert_offset", C.c_void_p), ("pair_count", C.c_void_p),
                ("pair_code", C.c_void_p), ("pair_weight", C.c_void_p), ("row_capacity", C.c_int32)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python fp8-moe-dev_b200/build.py` "
            "(the layer has no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    H = C.c_void_p
    lib.moe_fp8_b200_version.restype = C.c_int
    lib.moe_fp8_b200_workspace_bytes.restype = C.c_size_t
    lib.moe_fp8_b200_workspace_bytes.argtypes = [C.c_int, C.c_int]
    lib.moe_fp8_b200_row_capacity.restype = C.c_int
    lib.moe_fp8_b200_row_capacity.argtypes = [C.c_int, C.c_int]
    lib.moe_fp8_b200_create.restype = C.c_int
    lib.moe_fp8_b200_create.argtypes = [C.POINTER(H), C.c_int, C.c_int, C.c_int]
    lib.moe_fp8_b200_create_shaped.restype = C.c_int
    lib.moe_fp8_b200_create_shaped.argtypes = [C.POINTER(H), C.c_int, C.c_int, C.c_int, C.POINTER(Shape)]
    lib.moe_fp8_b200_workspace_bytes_shaped.restype = C.c_size_t
    lib.moe_fp8_b200_workspace_bytes_shaped.argtypes = [C.c_int, C.c_int, C.POINTER(Shape)]
    lib.moe_fp8_b200_get_shape.restype = C.c_int
    lib.moe_fp8_b200_get_shape.argtypes = [H, C.POINTER(Shape)]
    lib.moe_fp8_b200_destroy.restype = C.c_int
    lib.moe_fp8_b200_destroy.argtypes = [H]
    lib.moe_fp8_b200_last_error.restype = C.c_char_p
    lib.moe_fp8_b200_last_error.argtypes = [H]
    lib.moe_fp8_b200_set_option.restype = C.c_int
    lib.moe_fp8_b200_set_option.argtypes = [H, C.c_int, C.c_int]
    for name in ("moe_fp8_b200_run", "moe_fp8_b200_run_host"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [H, C.POINTER(Args), C.c_void_p]
    lib.moe_fp8_b200_exchange_bytes.restype = C.c_size_t
    lib.moe_fp8_b200_exchange_bytes.argtypes = [C.c_int, C.c_int]
    lib.moe_fp8_b200_copy_device.restype = C.c_int
    lib.moe_fp8_b200_copy_device.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                             C.c_void_p]
    for name in ("moe_fp8_b200_signal_peers", "moe_fp8_b200_wait_peers"):
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = [H, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_size_t, C.c_uint32, C.c_void_p]
    lib.moe_fp8_b200_invalidate_weights.restype = C.c_int
    lib.moe_fp8_b200_invalidate_weights.argtypes = [H]
    lib.moe_fp8_b200_copy_rows_h2d.restype = C.c_int
    lib.moe_fp8_b200_copy_rows_h2d.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                               C.c_void_p]
    lib.moe_fp8_b200_exchange_regions.restype = C.c_int
    lib.moe_fp8_b200_exchange_regions.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    lib.moe_fp8_b200_run_reduce_scatter.restype = C.c_int
    lib.moe_fp8_b200_run_reduce_scatter.argtypes = [H, C.POINTER(Args), C.POINTER(Exchange), C.c_void_p]
    lib.moe_fp8_b200_quantize_hidden.restype = C.c_int
    lib.moe_fp8_b200_quantize_hidden.argtypes = [H, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.moe_fp8_b200_run_unfinalized.restype = C.c_int
    lib.moe_fp8_b200_run_unfinalized.argtypes = [H, C.POINTER(Args), C.POINTER(Unfinalized), C.c_void_p]
    lib.moe_fp8_b200_finalize.restype = C.c_int
    lib.moe_fp8_b200_finalize.argtypes = [H, C.c_int, C.c_void_p, C.c_void_p]
    lib.moe_fp8_b200_run_host_async.restype = C.c_int
    lib.moe_fp8_b200_run_host_async.argtypes = [H, C.POINTER(Args), C.c_void_p, C.POINTER(C.c_int64)]
    lib.moe_fp8_b200_host_wait.restype = C.c_int
    lib.moe_fp8_b200_host_wait.argtypes = [H, C.c_int64]
    lib.moe_fp8_b200_set_expert_map.restype = C.c_int
    lib.moe_fp8_b200_set_expert_map.argtypes = [H, C.POINTER(C.c_int32)]
    lib.moe_fp8_b200_inject_device_status.restype = C.c_int
    lib.moe_fp8_b200_inject_device_status.argtypes = [H, C.c_int, C.c_uint, C.c_void_p]
    lib.moe_fp8_b200_check.restype = C.c_int
    lib.moe_fp8_b200_check.argtypes = [H, C.c_void_p]
    lib.moe_fp8_b200_read_intermediate.restype = C.c_int
    lib.moe_fp8_b200_read_intermediate.argtypes = [H, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
    lib.moe_fp8_b200_route_noalloc.restype = C.c_int
    lib.moe_fp8_b200_route_noalloc.argtypes = [
        C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_double, C.c_int32, C.c_void_p, C.c_void_p,
        C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]
    lib.moe_fp8_b200_stage_times.restype = C.c_int
    lib.moe_fp8_b200_stage_times.argtypes = [H, C.POINTER(C.c_float), C.POINTER(C.c_int)]
    lib.moe_fp8_b200_reference_policy.restype = C.c_int
    lib.moe_fp8_b200_reference_policy.argtypes = [C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_float)]
    _lib = lib
    return lib


def reference_policy(num_tokens: int) -> dict:
    """The reference's T-keyed dispatch policy as resolved by the library (host only)."""
    flags = (C.c_int32 * 5)()
    fracs = (C.c_float * 3)()
    rc = load().moe_fp8_b200_reference_policy(int(num_tokens), flags, fracs)
    if rc != OK:
        raise RuntimeError(f"moe_fp8_b200_reference_policy failed: {rc}")
    return dict(prune=flags[0], skip_zero_weight=flags[1], keep_limit=flags[2], drop_third=flags[3],
                renorm=flags[4], drop_third_frac=fracs[0], drop_second_frac_2=fracs[1],
                drop_second_frac_ge3=fracs[2])
