"""ctypes binding of ``libdartkv_b200.so`` (the C ABI declared in ``include/dartkv_b200.h``).

The shared library is the product: there is no Python or CPU fallback.  If it has
not been built, importing this module raises with the build command.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

import torch

from .build import LIB_PATH

F32, F16, BF16 = 0, 1, 2
DENSE_PAGE, QUANTIZED_PAGE, MIXED_PAGE = 0, 1, 2
DIV_TRUE, DIV_RECIPROCAL = 0, 1
DEQUANT_PER_OP, DEQUANT_FP32, DEQUANT_FUSED = 0, 1, 2
SCORE_MAGNITUDE, SCORE_VARIANCE = 0, 1
OK, EINVAL, ECUDA, ELIMIT = 0, -1, -2, -3

DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
CODE_DTYPE = {v: k for k, v in DTYPE_CODE.items()}

#: every symbol ``include/dartkv_b200.h`` declares
EXPORTS = (
    "dartkv_last_error", "dartkv_version", "dartkv_launch_count", "dartkv_pack", "dartkv_unpack", "dartkv_quantize", "dartkv_dequantize",
    "dartkv_channel_scores", "dartkv_select_channels", "dartkv_quantize_key_mixed", "dartkv_dequantize_key_mixed",
    "dartkv_cache_geometry", "dartkv_cache_append", "dartkv_cache_materialize", "dartkv_decode_workspace_bytes",
    "dartkv_decode_attention", "dartkv_decode_plan", "dartkv_decode_status", "dartkv_builtin_scratch_bytes",
    "dartkv_decode_attention_builtin_scratch", "dartkv_shard_range", "dartkv_decode_split_override",
    "dartkv_lifecycle_plan", "dartkv_cache_append_step", "dartkv_decode_attention_scatter",
    "dartkv_decode_attention_padded", "dartkv_cache_append_device_planned",
)


class CacheDesc(Structure):
    """Mirror of ``dartkv_cache_desc``."""

    _fields_ = [
        ("batch", c_int32), ("kv_heads", c_int32), ("head_dim", c_int32),
        ("dtype", c_int32), ("md_dtype", c_int32),
        ("page_size", c_int32), ("key_group", c_int32), ("value_group", c_int32),
        ("key_bits", c_int32), ("value_bits", c_int32),
        ("key_mode", c_int32), ("promoted", c_int32),
        ("sink_tokens", c_int32), ("ring_tokens", c_int32),
        ("max_key_pages", c_int32), ("max_value_tokens", c_int32),
        ("key_page_bytes", c_int32),
        ("key_off_high", c_int32), ("key_off_index", c_int32), ("key_off_scale", c_int32), ("key_off_zero", c_int32),
        ("value_row_bytes", c_int32), ("value_groups", c_int32), ("regular_pages", c_int32),
        ("k_sink", c_void_p), ("v_sink", c_void_p), ("k_ring", c_void_p), ("v_ring", c_void_p),
        ("k_pages", c_void_p), ("v_codes", c_void_p), ("v_meta", c_void_p),
        ("page_start", c_void_p), ("page_tokens", c_void_p), ("state", c_void_p),
    ]


class DecodePlanInfo(Structure):
    """Mirror of ``dartkv_decode_plan_info``."""

    _fields_ = [
        ("kernel", c_int32), ("quads", c_int32), ("stream_blocks", c_int32), ("total_splits", c_int32),
        ("units", c_int64), ("generic_splits", c_int32), ("generic_chunk", c_int32),
    ]


class LifecycleConfig(Structure):
    """Mirror of ``dartkv_lifecycle_config``."""

    _fields_ = [("page_size", c_int32), ("sink_tokens", c_int32), ("local_tokens", c_int32),
                ("value_local_tokens", c_int32), ("hold_partial_pages", c_int32)]


class LifecycleStateC(Structure):
    """Mirror of ``dartkv_lifecycle_state``."""

    _fields_ = [("seen", c_int32), ("k_packed_end", c_int32), ("v_packed_end", c_int32), ("key_pages", c_int32)]


MAX_PEERS = 8


class PeerScatter(Structure):
    """Mirror of ``dartkv_peer_scatter``."""

    _fields_ = [("world_size", c_int32), ("rank", c_int32), ("dst_row_begin", c_int32), ("dst_head_begin", c_int32),
                ("dst_heads_total", c_int32), ("epoch", ctypes.c_uint32), ("out", c_void_p * MAX_PEERS),
                ("flags", c_void_p * MAX_PEERS)]


class Shard(Structure):
    """Mirror of ``dartkv_shard``."""

    _fields_ = [
        ("row_begin", c_int32), ("row_end", c_int32), ("head_begin", c_int32), ("head_end", c_int32),
        ("batch_groups", c_int32), ("head_groups", c_int32), ("rows_padded", c_int32), ("reserved", c_int32),
    ]


class AppendPlan(Structure):
    """Mirror of ``dartkv_append_plan``."""

    _fields_ = [
        ("chunk_start", c_int32), ("chunk_tokens", c_int32), ("sink_copy", c_int32),
        ("first_page", c_int32), ("num_pages", c_int32), ("page_token_start", c_int32),
        ("last_page_tokens", c_int32), ("value_begin", c_int32), ("value_end", c_int32),
        ("ring_begin", c_int32), ("reserved", c_int32),
        ("seen_after", c_int32), ("k_packed_end_after", c_int32), ("v_packed_end_after", c_int32),
        ("key_pages_after", c_int32), ("requantize_last_page", c_int32),
    ]


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. Build it with "
            "`python -m dartkv_b200.build` (needs nvcc; cross-compiles for sm_100a without a GPU)."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.dartkv_last_error.restype = c_char_p
    lib.dartkv_version.restype = c_int
    lib.dartkv_launch_count.restype = ctypes.c_longlong
    p, i64, i32 = c_void_p, c_int64, c_int
    lib.dartkv_pack.argtypes = [p, i64, i64, i32, p, p]
    lib.dartkv_unpack.argtypes = [p, i64, i64, i32, i64, p, p]
    lib.dartkv_quantize.argtypes = [p, i32, i64, i64, i64, i64, i64, i64, i32, i32, i32, i32, p, p, p, p, p]
    lib.dartkv_dequantize.argtypes = [p, p, p, i32, i64, i64, i64, i32, i32, i32, p, i32, i64, i64, i64, p]
    lib.dartkv_channel_scores.argtypes = [p, i32, i64, i64, i64, i64, i64, i32, p, p]
    lib.dartkv_select_channels.argtypes = [p, i32, i64, i64, i32, p, p]
    lib.dartkv_quantize_key_mixed.argtypes = [p, i32, i64, i64, i64, i64, i64, i32, p, i32, i32, p, p, p, p, p, p]
    lib.dartkv_dequantize_key_mixed.argtypes = [p, p, p, p, p, i32, i64, i64, i64, i32, i32, i32, p, i32, p]
    lib.dartkv_cache_geometry.argtypes = [POINTER(CacheDesc)]
    lib.dartkv_cache_append.argtypes = [POINTER(CacheDesc), POINTER(AppendPlan), p, p, i64, i64, i64, p, p, p]
    lib.dartkv_cache_materialize.argtypes = [POINTER(CacheDesc), i32, c_int32, c_int32, i32, p, i32, p]
    lib.dartkv_decode_workspace_bytes.argtypes = [POINTER(CacheDesc), i32, i32]
    lib.dartkv_decode_workspace_bytes.restype = c_int64
    lib.dartkv_decode_attention.argtypes = [POINTER(CacheDesc), p, i32, i32, c_float, i32, i32, p, i64, p, p]
    lib.dartkv_decode_attention_padded.argtypes = [POINTER(CacheDesc), p, i32, i32, c_float, i32, i32, p, p, i64, p, p]
    lib.dartkv_decode_attention_scatter.argtypes = [POINTER(CacheDesc), p, i32, i32, c_float, i32, i32, p, i64, p,
                                                    POINTER(PeerScatter), p]
    lib.dartkv_decode_status.argtypes = [p, POINTER(c_int), p]
    lib.dartkv_decode_plan.argtypes = [POINTER(CacheDesc), i32, i32, i32, i32, POINTER(DecodePlanInfo)]
    lib.dartkv_builtin_scratch_bytes.restype = c_int64
    lib.dartkv_decode_split_override.argtypes = [c_char_p]
    lib.dartkv_lifecycle_plan.argtypes = [POINTER(LifecycleConfig), POINTER(LifecycleStateC), i32, POINTER(AppendPlan)]
    lib.dartkv_cache_append_step.argtypes = [POINTER(CacheDesc), POINTER(LifecycleConfig), POINTER(LifecycleStateC), p, p,
                                             i32, i64, i64, i64, p, p, POINTER(AppendPlan), p]
    lib.dartkv_cache_append_device_planned.argtypes = [POINTER(CacheDesc), POINTER(LifecycleConfig), p, p, i32, i64, i64, i64,
                                                       p, p]
    lib.dartkv_shard_range.argtypes = [i32, i32, i32, i32, POINTER(Shard)]
    lib.dartkv_decode_attention_builtin_scratch.argtypes = [POINTER(CacheDesc), p, i32, i32, c_float, i32, i32, p, p]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if fn.restype is c_int and name not in ("dartkv_version",):
            fn.restype = c_int
    return lib


LIB = _load()


class DartKVError(RuntimeError):
    pass


def last_error() -> str:
    return (LIB.dartkv_last_error() or b"").decode("utf-8", "replace")


def check(rc: int, exc=None) -> None:
    """Raise for a failed C call.  -1 (bad argument) maps to ValueError like the reference's checks."""

    if rc == 0:
        return
    message = last_error()
    if exc is not None:
        raise exc(message)
    if rc == -1:
        raise ValueError(message)
    raise DartKVError(f"dartkv_b200 call failed ({rc}): {message}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """The kernels only exist for CUDA: refuse CPU tensors loudly instead of falling back."""

    device = None
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(
                "dartkv_b200 runs on CUDA tensors only (B200 kernels; there is no CPU fallback), "
                f"got a tensor on {t.device}"
            )
        if device is None:
            device = t.device
        elif t.device != device:
            raise ValueError("all tensors must be on the same CUDA device")
    return device


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int:
    """Handle of the current stream of ``device`` (the raw query skips building a Stream object)."""

    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(device: torch.device):
    """Context that makes ``device`` current for the launches inside it; free when it already is."""

    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()
