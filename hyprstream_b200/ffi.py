"""ctypes binding of libhs_attn.so — the same C ABI (include/hs_attn.h) a Rust `-sys` crate would bind.

There is no fallback: if the shared library is missing, importing this module raises.  Build it
with ``python hyprstream_b200/csrc/build.py``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhs_attn.so")

HS_OK = 0
HS_ERR_ARG, HS_ERR_UNSUPPORTED, HS_ERR_DEVICE, HS_ERR_WORKSPACE = -1, -2, -3, -4
HS_ERR_POOL_EXHAUSTED, HS_ERR_CACHE_OVERFLOW, HS_ERR_CACHE_EMPTY = -5, -6, -7
KV_BF16, KV_INT8, KV_NF4, KV_FP4 = 0, 1, 2, 3
SCALE_F32, SCALE_F16 = 0, 1
DTYPE_BF16, DTYPE_F16, DTYPE_F32 = 0, 1, 2
DEVERR_KV_WRITE_RANGE, DEVERR_ROPE_RANGE, DEVERR_DECODE_RANGE, DEVERR_WAIT_TIMEOUT = 1, 2, 4, 8
STEP_SYNC, SHARD_PUSH_ONLY, SCHED_DEVICE_OBJECTS = 1, 1, 1


class HsError(RuntimeError):
    """A non-zero status from the C ABI; `.status` holds the code (negative: argument, positive: CUDA)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"hs_attn status {status}: {message}")
        self.status = status


class GdnLayerParams(ctypes.Structure):
    """struct hs_gdn_layer_params."""
    _fields_ = [("conv_weight", c_void_p), ("neg_a_exp", c_void_p), ("dt_bias", c_void_p), ("norm_weight", c_void_p), ("norm_eps", c_float),
                ("n_k_heads", c_int32), ("n_v_heads", c_int32), ("head_k_dim", c_int32), ("head_v_dim", c_int32), ("kernel_size", c_int32)]


class GdnLayerIO(ctypes.Structure):
    """struct hs_gdn_layer_io."""
    _fields_ = [("mixed_qkv", c_void_p), ("z", c_void_p), ("a_in", c_void_p), ("b_in", c_void_p), ("conv_state", c_void_p),
                ("rec_state", c_void_p), ("y", c_void_p)]


class QwenAttnParams(ctypes.Structure):
    """struct hs_qwen_attn_params."""
    _fields_ = [("q_norm_weight", c_void_p), ("k_norm_weight", c_void_p), ("norm_eps", c_float), ("sin", c_void_p), ("cos", c_void_p),
                ("n_positions", c_int32), ("rotary_dim", c_int32), ("n_q_heads", c_int32), ("n_kv_heads", c_int32), ("head_dim", c_int32),
                ("softmax_scale", c_float)]


class QwenAttnIO(ctypes.Structure):
    """struct hs_qwen_attn_io."""
    _fields_ = [("q_proj", c_void_p), ("k_proj", c_void_p), ("v_proj", c_void_p), ("view", c_void_p), ("positions", c_void_p),
                ("dst_pos", c_void_p), ("seq_lens", c_void_p), ("out", c_void_p)]


class SchedPlan(ctypes.Structure):
    """struct hs_sched_plan."""
    _fields_ = [("n_prefill", c_int32), ("prefill_ids", POINTER(c_int64)), ("prefill_lens", POINTER(c_int32)), ("prefill_caches", POINTER(c_void_p)),
                ("n_decode", c_int32), ("decode_ids", POINTER(c_int64)), ("decode_caches", POINTER(c_void_p)), ("host_dst_pos", POINTER(c_int32)),
                ("view", c_void_p), ("dst_pos", c_void_p), ("seq_lens", c_void_p),
                ("n_deferred", c_int32), ("n_stalled", c_int32), ("n_waiting", c_int32), ("n_running", c_int32)]


class SchedStats(ctypes.Structure):
    """struct hs_sched_stats_t."""
    _fields_ = [("n_waiting", c_int32), ("n_running", c_int32), ("pages_free", c_int32), ("reserved", c_int32),
                ("n_admitted", c_int64), ("n_retired", c_int64), ("n_deferred", c_int64), ("n_stalled", c_int64), ("n_steps", c_int64)]


class KVView(ctypes.Structure):
    """struct hs_kv_view."""
    _fields_ = [
        ("kind", c_int32), ("scale_dtype", c_int32), ("block", c_int32), ("n_kv_heads", c_int32),
        ("head_dim", c_int32), ("page_tokens", c_int32), ("pages_per_seq", c_int32), ("reserved", c_int32),
        ("k_pages", c_void_p), ("v_pages", c_void_p), ("k_scale_pages", c_void_p), ("v_scale_pages", c_void_p),
    ]


if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python hyprstream_b200/csrc/build.py` (there is no CPU fallback)")

lib = ctypes.CDLL(LIB_PATH)

_SIGS = {
    "hs_attn_version": (c_int32, []),
    "hs_attn_device_check": (c_int32, [c_int32]),
    "hs_attn_last_error": (c_char_p, []),
    "hs_attn_take_device_error": (c_int32, [POINTER(c_int32)]),
    "hs_attn_inject_device_error": (c_int32, [c_int32]),
    "hs_attn_set_profiling": (c_int32, [c_int32]),
    "hs_attn_last_kernel_ms": (c_int32, [POINTER(c_float)]),
    "hs_attn_launch_count": (c_int64, []),
    "hs_quantize_blockwise": (c_int32, [c_int32, c_void_p, c_int32, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "hs_dequantize_blockwise": (c_int32, [c_int32, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_int32, c_void_p]),
    "hs_rope_apply": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "hs_qk_norm_rope": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_int32, c_void_p, c_void_p, c_void_p,
                                  c_int32, c_int32, c_int64, c_int32, c_int32, c_void_p]),
    "hs_kv_quantize_write": (c_int32, [POINTER(KVView), c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "hs_kv_norm_rope_quantize_write": (c_int32, [POINTER(KVView), c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_float, c_int32, c_void_p, c_void_p,
                                                 c_int32, c_int32, c_void_p, c_void_p]),
    "hs_kv_gather_dequantize": (c_int32, [POINTER(KVView), c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "hs_attn_decode_workspace_bytes": (c_int64, [c_int32, c_int32, c_int32]),
    "hs_attn_decode": (c_int32, [c_void_p, POINTER(KVView), c_void_p, c_int32, c_int32, c_float, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "hs_attn_decode_static_max_bytes": (c_int64, []),
    "hs_attn_decode_static": (c_int32, [c_void_p, POINTER(KVView), c_void_p, c_int32, c_int32, c_float, c_void_p, c_void_p, c_void_p]),
    "hs_attn_decode_append": (c_int32, [c_void_p, c_void_p, c_void_p, POINTER(KVView), c_void_p, c_void_p, c_int32, c_int32, c_float, c_void_p, c_void_p,
                                        c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "hs_attn_decode_step": (c_int32, [POINTER(KVView), c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_float, c_void_p, c_void_p,
                                      c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "hs_shard_group_create": (c_int32, [c_int32] * 5 + [POINTER(c_void_p)]),
    "hs_shard_group_handle_bytes": (c_int32, []),
    "hs_shard_group_export": (c_int32, [c_void_p, c_void_p]),
    "hs_shard_group_connect": (c_int32, [c_void_p, c_void_p]),
    "hs_shard_group_connect_local": (c_int32, [POINTER(c_void_p), c_int32]),
    "hs_shard_group_set_wait_ms": (c_int32, [c_void_p, c_int32]),
    "hs_shard_group_epoch": (c_int32, [c_void_p]),
    "hs_shard_group_destroy": (None, [c_void_p]),
    "hs_attn_decode_sharded": (c_int32, [c_void_p, c_void_p, POINTER(KVView), c_void_p, c_int32, c_int32, c_float, c_void_p, c_void_p, c_void_p,
                                         c_int64, c_int32, c_void_p]),
    "hs_cache_snapshot": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p]),
    "hs_view_is_current": (c_int32, [c_void_p]),
    "hs_attn_prefill_causal": (c_int32, [c_void_p] * 5 + [c_int32] * 6 + [c_float, c_void_p]),
    "hs_gdn_recurrent": (c_int32, [c_void_p] * 7 + [c_int32] * 6 + [c_void_p]),
    "hs_gdn_chunk_prefill": (c_int32, [c_void_p] * 7 + [c_int32] * 6 + [c_void_p]),
    "hs_gdn_prologue": (c_int32, [c_void_p] * 3 + [c_int32] + [c_void_p] * 9 + [c_int32] * 7 + [c_void_p]),
    "hs_gdn_epilogue": (c_int32, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int32, c_void_p]),
    "hs_gdn_layer_workspace_bytes": (c_int64, [c_void_p, c_int32, c_int32]),
    "hs_gdn_layer_forward": (c_int32, [c_void_p] * 7 + [c_int32] * 3 + [c_void_p, c_void_p, c_int64, c_void_p]),
    "hs_qwen_attn_layer_workspace_bytes": (c_int64, [c_void_p, c_int32, c_int32]),
    "hs_qwen_attn_layer_forward": (c_int32, [c_void_p] * 4 + [POINTER(KVView)] + [c_void_p] * 3 + [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_void_p]),
    "hs_qwen_block_workspace_bytes": (c_int64, [c_void_p, c_int32, c_void_p, c_int32, c_int32]),
    "hs_qwen_block_forward": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_int64, c_void_p]),
    "hs_sched_create": (c_int32, [c_void_p, c_int32, c_int32, POINTER(c_void_p)]),
    "hs_sched_destroy": (None, [c_void_p]),
    "hs_sched_submit": (c_int32, [c_void_p, c_int64, c_int32, c_int32]),
    "hs_sched_plan_step": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p]),
    "hs_sched_commit_step": (c_int32, [c_void_p, c_void_p, c_int32]),
    "hs_sched_cancel": (c_int32, [c_void_p, c_int64]),
    "hs_sched_stats": (c_int32, [c_void_p, c_void_p]),
    "hs_host_set_allocator": (c_int32, [c_void_p, c_void_p]),
    "hs_pool_create": (c_int32, [c_int32] * 7 + [POINTER(c_void_p)]),
    "hs_pool_destroy": (None, [c_void_p]),
    "hs_pool_num_free": (c_int32, [c_void_p]),
    "hs_cache_create": (c_int32, [c_int32] * 6 + [POINTER(c_void_p)]),
    "hs_cache_create_paged": (c_int32, [c_int32, c_void_p, c_int64, POINTER(c_void_p)]),
    "hs_cache_destroy": (None, [c_void_p]),
    "hs_cache_update": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int32, c_int32, c_void_p]),
    "hs_cache_get": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "hs_cache_reserve": (c_int32, [c_void_p, c_int32]),
    "hs_cache_clear": (c_int32, [c_void_p]),
    "hs_cache_truncate_to": (c_int32, [c_void_p, c_int32]),
    "hs_cache_seq_pos": (c_int32, [c_void_p]),
    "hs_cache_set_seq_pos": (c_int32, [c_void_p, c_int32]),
    "hs_cache_capacity": (c_int32, [c_void_p]),
    "hs_cache_num_pages": (c_int32, [c_void_p]),
    "hs_cache_memory_usage": (c_int64, [c_void_p]),
    "hs_cache_offload_bytes": (c_int64, [c_void_p]),
    "hs_cache_offload": (c_int32, [c_void_p, c_void_p, c_int64, c_void_p]),
    "hs_cache_restore": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "hs_view_create": (c_int32, [POINTER(c_void_p), c_int32, POINTER(c_void_p)]),
    "hs_view_get": (c_void_p, [c_void_p]),
    "hs_view_destroy": (None, [c_void_p]),
    "hs_attn_merge_partials": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int32, c_void_p, c_void_p, c_void_p]),
    "hs_attn_merge_partials_strided": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p, c_void_p]),
}


def exported_symbols() -> list[str]:
    """Every entry point include/hs_attn.h declares (checked against the header by the CPU tests)."""
    return sorted(_SIGS)


for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    msg = lib.hs_attn_last_error()
    return msg.decode() if msg else ""


def check(status: int) -> None:
    if status != HS_OK:
        raise HsError(status, last_error())


def take_device_error() -> int:
    flags = c_int32(0)
    check(lib.hs_attn_take_device_error(ctypes.byref(flags)))
    return flags.value


def set_profiling(on: bool) -> None:
    check(lib.hs_attn_set_profiling(1 if on else 0))


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib.hs_attn_launch_count())


def last_kernel_ms() -> float:
    ms = c_float(0.0)
    check(lib.hs_attn_last_kernel_ms(ctypes.byref(ms)))
    return ms.value
