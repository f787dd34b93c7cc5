"""B200-native token sampling behind the flash-gordon `fg_sampler` C API.

The product is `lib/libfgsampler.so` (hand-written CUDA for sm_100a + a C17
host layer, C ABI declared in `include/`).  This package is the thin Python
side: it loads the library with ctypes, mirrors the C structs, and wraps device
memory that PyTorch allocated.  There is no Python or CPU implementation of the
sampling arithmetic here; if the library is missing, importing the bindings
raises.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, Structure, byref, c_bool, c_char, c_float, c_int, c_uint32,
                    c_uint64, c_void_p)
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE_DIR / "lib" / "libfgsampler.so"

FG_OK = 0
FG_ERR_ARGUMENT = 2
FG_ERR_IO = 3
FG_ERR_FORMAT = 4
FG_ERR_MISMATCH = 5
FG_ERR_OOM = 6
FG_ERR_UNAVAILABLE = 7
FG_ERR_LIMIT = 8
FG_ERR_INTERRUPTED = 9

FG_CUDA_F32 = 0
FG_CUDA_BF16 = 1
FG_CUDA_SAMPLE_ASYNC = 1
FG_CUDA_SAMPLE_ALLOW_NO_TOPK = 2
PADDING_ID = 0xFFFFFFFF
MAX_CANDIDATES = 64


class FgError(Structure):
    """fg_error (include/fg.h)."""
    _fields_ = [("code", c_int), ("message", c_char * 512)]

    def text(self) -> str:
        return self.message.decode("utf-8", "replace")


class SamplerConfig(Structure):
    """fg_sampler_config (include/fg_sampler.h): 40 bytes."""
    _fields_ = [
        ("temperature", c_float), ("top_p", c_float), ("top_k", c_uint32),
        ("presence_penalty", c_float), ("frequency_penalty", c_float),
        ("repetition_penalty", c_float), ("min_p", c_float), ("seed", c_uint64),
    ]

    @classmethod
    def make(cls, temperature=1.0, top_p=0.95, top_k=20, presence=0.0, frequency=0.0,
             repetition=1.0, seed=0x9E3779B97F4A7C15) -> "SamplerConfig":
        return cls(temperature, top_p, top_k, presence, frequency, repetition, 0.0, seed)


class SamplerState(Structure):
    _fields_ = [("state", c_uint64)]


class SampleDebug(Structure):
    _fields_ = [("candidate_count", c_void_p), ("candidate_ids", c_void_p),
                ("candidate_scores", c_void_p), ("raw_probability", c_void_p),
                ("tempered_probability", c_void_p)]


class SampleArgs(Structure):
    """fg_cuda_sample_args (include/fg_cuda_sampler.h)."""
    _fields_ = [
        ("logits", c_void_p), ("dtype", c_uint32), ("rows", c_uint32), ("vocab", c_uint32),
        ("flags", c_uint32), ("row_stride", c_uint64), ("history_tokens", c_void_p),
        ("history_offsets", c_void_p), ("history_max", c_uint32), ("config_count", c_uint32),
        ("configs", POINTER(SamplerConfig)), ("uniforms", c_void_p), ("tokens", c_void_p),
        ("token_logits", c_void_p), ("row_status", c_void_p), ("debug", POINTER(SampleDebug)),
    ]


assert ctypes.sizeof(SamplerConfig) == 40
assert ctypes.sizeof(FgError) == 516


class FgStatusError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"fg_status {status}: {message}")
        self.status = status
        self.message = message


_library = None


def load_library() -> ctypes.CDLL:
    """The C-ABI library; raises if it has not been built (no fallback exists)."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise RuntimeError(
            f"{LIBRARY_PATH} is missing: build it with `python -m flash_gordon_b200.build` "
            "(the sampler has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    P, E = c_void_p, POINTER(FgError)
    CFG = POINTER(SamplerConfig)
    u32, u64 = c_uint32, c_uint64
    sig = {
        # fg.h
        "fg_align_up_u64": (u64, [u64, u64]),
        "fg_is_aligned_u64": (c_bool, [u64, u64]),
        # fg_sampler.h
        "fg_sampler_config_greedy": (None, [CFG]),
        "fg_sampler_config_defaults": (None, [CFG]),
        "fg_sampler_config_validate": (c_int, [CFG, E]),
        "fg_sampler_state_init": (None, [POINTER(SamplerState), u64]),
        "fg_sampler_uniform": (c_float, [POINTER(SamplerState)]),
        "fg_sampler_select": (c_int, [CFG, P, P, u32, c_float, POINTER(u32), POINTER(c_float), E]),
        "fg_sampler_penalties_active": (c_bool, [CFG]),
        "fg_sampler_apply_penalties": (None, [P, P, P, u32, CFG]),
        "fg_sampler_last_status": (c_int, []),
        # fg_cuda_sampler.h
        "fg_cuda_context_create": (c_int, [c_int, POINTER(P), E]),
        "fg_cuda_context_destroy": (None, [P]),
        "fg_cuda_context_set_stream": (c_int, [P, P, E]),
        "fg_cuda_context_reset_stream": (c_int, [P, E]),
        "fg_cuda_context_stream": (P, [P]),
        "fg_cuda_context_device": (c_int, [P]),
        "fg_cuda_context_sm_count": (u32, [P]),
        "fg_cuda_context_launches": (u64, [P]),
        "fg_cuda_context_set_splits": (c_int, [P, u32, E]),
        "fg_cuda_context_set_path": (c_int, [P, u32, E]),
        "fg_cuda_context_scratch_bytes": (u64, [P]),
        "fg_cuda_begin": (c_int, [P, E]),
        "fg_cuda_end": (c_int, [P, E]),
        "fg_cuda_batch_active": (c_bool, [P]),
        "fg_cuda_tensor_create": (c_int, [P, u64, POINTER(P), E]),
        "fg_cuda_tensor_view": (c_int, [P, u64, u64, POINTER(P), E]),
        "fg_cuda_tensor_wrap": (c_int, [P, P, u64, POINTER(P), E]),
        "fg_cuda_tensor_destroy": (None, [P]),
        "fg_cuda_tensor_bytes": (u64, [P]),
        "fg_cuda_tensor_device_pointer": (P, [P]),
        "fg_cuda_tensor_write": (c_int, [P, u64, P, u64, E]),
        "fg_cuda_tensor_read": (c_int, [P, u64, P, u64, E]),
        "fg_cuda_apply_penalties": (c_int, [P, P, P, u32, c_float, c_float, c_float, E]),
        "fg_cuda_argmax_reduce": (c_int, [P, P, P, P, P, u32, POINTER(u32), E]),
        "fg_cuda_topk_select": (c_int, [P, P, P, P, P, u32, u32, POINTER(u32), E]),
        "fg_cuda_topk_reduce": (c_int, [P, P, P, P, P, u32, POINTER(u32), E]),
        "fg_cuda_router_topk": (c_int, [P, P, P, P, u32, u32, u32, E]),
        "fg_cuda_history_reset": (c_int, [P, P, u32, P, u32, E]),
        "fg_cuda_history_increment": (c_int, [P, P, u32, u32, E]),
        "fg_cuda_sample_batch": (c_int, [P, POINTER(SampleArgs), E]),
        "fg_cuda_sample_batch_host": (c_int, [P, POINTER(SampleArgs), E]),
        "fg_cuda_sample_batch_static": (c_int, [c_int, P, POINTER(SampleArgs), E]),
        "fg_cuda_shard_topk": (c_int, [P, POINTER(SampleArgs), u32, u32, u32, P, P, E]),
        "fg_cuda_merge_select": (c_int, [P, POINTER(SampleArgs), P, P, u32, u32, P, P, E]),
        "fg_dist_unique_id": (c_int, [P, E]),
        "fg_dist_create": (c_int, [P, u32, u32, P, u32, POINTER(P), E]),
        "fg_dist_destroy": (None, [P]),
        "fg_dist_ranks": (u32, [P]),
        "fg_dist_rank": (u32, [P]),
        "fg_dist_shard_span": (None, [u32, u32, u32, POINTER(u32), POINTER(u32)]),
        "fg_dist_sample_vocab_sharded": (c_int, [P, POINTER(SampleArgs), u32, u32, E]),
        "fg_dist_sample_vocab_sharded_fused": (c_int, [P, POINTER(SampleArgs), u32, u32, E]),
        "fg_dist_gather_rows": (c_int, [P, P, P, P, u32, P, P, P, E]),
        "fg_cuda_output_executor_create": (c_int, [P, u32, u32, u32, POINTER(P), E]),
        "fg_cuda_output_executor_destroy": (None, [P]),
        "fg_cuda_output_set_session": (None, [P, u32]),
        "fg_cuda_output_session": (u32, [P]),
        "fg_cuda_output_history_length": (u32, [P, u32]),
        "fg_cuda_output_history_reset": (c_int, [P, P, u32, E]),
        "fg_cuda_output_history_increment": (c_int, [P, u32, E]),
        "fg_cuda_output_greedy": (c_int, [P, P, POINTER(u32), POINTER(c_float), E]),
        "fg_cuda_output_sample": (c_int, [P, P, CFG, c_float, POINTER(u32), POINTER(c_float), E]),
        "fg_cuda_output_sample_sessions": (c_int, [P, POINTER(SampleArgs), P, E]),
        # test seam of the ring kernel (csrc/host/fg_host_internal.h; not in the public headers)
        "fg_cuda_internal_ring_controls": (c_int, [P, u32, u32, u32, u32, u32]),
    }
    for name, (restype, argtypes) in sig.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _library = lib
    return lib


def _check(status: int, err: FgError) -> None:
    if status != FG_OK:
        raise FgStatusError(status, err.text())


def config_array(configs) -> "ctypes.Array":
    """A contiguous C array from one SamplerConfig or a sequence of them."""
    if isinstance(configs, SamplerConfig):
        configs = [configs]
    array = (SamplerConfig * len(configs))()
    for i, cfg in enumerate(configs):
        array[i] = cfg
    return array


def uniform_stream(seed: int, count: int) -> list[float]:
    """`count` draws of the library's xorshift64* stream (fg_sampler_uniform)."""
    lib = load_library()
    state = SamplerState()
    lib.fg_sampler_state_init(byref(state), seed)
    return [lib.fg_sampler_uniform(byref(state)) for _ in range(count)]


from .api import Context, Tensor  # noqa: E402

__all__ = [
    "Context", "Tensor", "SamplerConfig", "SamplerState", "SampleArgs", "SampleDebug", "FgError",
    "FgStatusError", "load_library", "config_array", "uniform_stream", "LIBRARY_PATH",
]
