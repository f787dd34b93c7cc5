"""TEST INFRASTRUCTURE — ctypes access to the CPU oracle.

Only tests, the smoke check and the benchmark's CPU-baseline legs import this.
`load("port")` opens oracle/libfgoracle.so (this repository's restatement of
the reference's sampler), `load("reference")` opens oracle/_ref/libfgref.so
(the same pipeline linked against the reference's own objects; present only
where it was built from a mounted reference tree).
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, Structure, byref, c_bool, c_char, c_char_p, c_double, c_float, c_int, c_uint32, c_uint64, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_PATH = HERE / "libfgoracle.so"
REFERENCE_PATH = HERE / "_ref" / "libfgref.so"
PADDING_ID = 0xFFFFFFFF


class OracleError(Structure):
    _fields_ = [("code", c_int), ("message", c_char * 512)]


class OracleConfig(Structure):
    _fields_ = [
        ("temperature", c_float), ("top_p", c_float), ("top_k", c_uint32),
        ("presence_penalty", c_float), ("frequency_penalty", c_float),
        ("repetition_penalty", c_float), ("min_p", c_float), ("seed", c_uint64),
    ]

    @classmethod
    def of(cls, other) -> "OracleConfig":
        return cls(other.temperature, other.top_p, other.top_k, other.presence_penalty,
                   other.frequency_penalty, other.repetition_penalty, other.min_p, other.seed)


class OracleState(Structure):
    _fields_ = [("state", c_uint64)]


class OracleCandidates(Structure):
    _fields_ = [("count", c_uint32), ("ids", c_uint32 * 64), ("scores", c_float * 64),
                ("raw_probability", c_double * 64), ("tempered_probability", c_double * 64),
                ("nucleus", c_uint32), ("edge_margin", c_double)]


_handles: dict[str, ctypes.CDLL] = {}


def available(kind: str) -> bool:
    return (PORT_PATH if kind == "port" else REFERENCE_PATH).exists()


def load(kind: str = "port") -> ctypes.CDLL:
    if kind in _handles:
        return _handles[kind]
    path = PORT_PATH if kind == "port" else REFERENCE_PATH
    if kind == "port" and not path.exists():
        subprocess.run(["make", "-C", str(HERE), "libfgoracle.so"], check=True, capture_output=True)
    if not path.exists():
        raise FileNotFoundError(f"{path} has not been built")
    lib = ctypes.CDLL(str(path))
    P, E, CFG = c_void_p, POINTER(OracleError), POINTER(OracleConfig)
    u32, u64 = c_uint32, c_uint64
    sig = {
        "fgo_kind": (c_char_p, []),
        "fg_sampler_config_greedy": (None, [CFG]),
        "fg_sampler_config_defaults": (None, [CFG]),
        "fg_sampler_config_validate": (c_int, [CFG, E]),
        "fg_sampler_state_init": (None, [POINTER(OracleState), u64]),
        "fg_sampler_uniform": (c_float, [POINTER(OracleState)]),
        "fg_sampler_select": (c_int, [CFG, P, P, u32, c_float, POINTER(u32), POINTER(c_float), E]),
        "fg_sampler_penalties_active": (c_bool, [CFG]),
        "fg_sampler_apply_penalties": (None, [P, P, P, u32, CFG]),
        "fg_output_better": (c_bool, [c_float, u32, c_float, u32]),
        "fg_output_combine": (None, [c_float, u32, c_float, u32, POINTER(c_float), POINTER(u32)]),
        "fgo_history_counts": (c_int, [P, u32, P, u32, E]),
        "fgo_apply_penalties_shader": (None, [P, P, u32, c_float, c_float, c_float]),
        "fgo_argmax_reduce": (u32, [P, P, P, P, u32]),
        "fgo_topk_select": (u32, [P, P, P, P, u32, u32]),
        "fgo_topk_reduce": (u32, [P, P, P, P, u32]),
        "fgo_router_topk": (c_int, [P, u32, u32, P, P]),
        "fgo_select_general": (c_int, [CFG, c_bool, P, P, u32, c_float, POINTER(u32),
                                       POINTER(c_float), POINTER(u32), POINTER(c_double), E]),
        "fgo_sample_batch": (c_int, [P, u32, u32, u32, u64, P, P, CFG, u32, c_bool, P, P, P, P,
                                     POINTER(OracleCandidates), u32]),
        "fgo_shard_topk": (c_int, [P, u32, u32, u32, u64, u32, u32, P, P, CFG, u32, u32, P, P, P]),
        "fgo_merge_select": (c_int, [P, P, u32, u32, u32, P, P, CFG, u32, P, P, P, P,
                                     POINTER(OracleCandidates)]),
    }
    for name, (restype, argtypes) in sig.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _handles[kind] = lib
    return lib


def _ptr(array):
    return None if array is None else array.ctypes.data_as(c_void_p)


def _configs(configs):
    if not isinstance(configs, (list, tuple)):
        configs = [configs]
    array = (OracleConfig * len(configs))()
    for i, cfg in enumerate(configs):
        array[i] = OracleConfig.of(cfg)
    return array


def uniform_stream(lib, seed: int, count: int) -> np.ndarray:
    state = OracleState()
    lib.fg_sampler_state_init(byref(state), seed)
    return np.array([lib.fg_sampler_uniform(byref(state)) for _ in range(count)], dtype=np.float32)


def select(lib, config, scores, ids, uniform: float):
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    cfg = OracleConfig.of(config)
    token, logit, err = c_uint32(0), c_float(0.0), OracleError()
    status = lib.fg_sampler_select(byref(cfg), _ptr(scores), _ptr(ids), len(scores), uniform,
                                   byref(token), byref(logit), byref(err))
    return status, token.value, logit.value, err.message.decode()


def select_general(lib, config, scores, ids, uniform: float, allow_no_topk: bool = True):
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    cfg = OracleConfig.of(config)
    token, logit, nucleus, margin, err = c_uint32(0), c_float(0.0), c_uint32(0), c_double(0), OracleError()
    status = lib.fgo_select_general(byref(cfg), allow_no_topk, _ptr(scores), _ptr(ids), len(scores),
                                    uniform, byref(token), byref(logit), byref(nucleus),
                                    byref(margin), byref(err))
    return status, token.value, logit.value, nucleus.value, margin.value


def apply_penalties(lib, scores, ids, counts, config) -> np.ndarray:
    out = np.array(scores, dtype=np.float32, copy=True)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    counts = np.ascontiguousarray(counts, dtype=np.uint32)
    cfg = OracleConfig.of(config)
    lib.fg_sampler_apply_penalties(_ptr(out), _ptr(ids), _ptr(counts), len(out), byref(cfg))
    return out


def history_counts(lib, vocab: int, history):
    history = np.ascontiguousarray(history, dtype=np.uint32)
    counts = np.zeros(vocab, dtype=np.uint32)
    err = OracleError()
    status = lib.fgo_history_counts(_ptr(counts), vocab, _ptr(history), len(history), byref(err))
    return status, counts


def argmax_reduce(lib, scores, ids=None):
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    ids = None if ids is None else np.ascontiguousarray(ids, dtype=np.uint32)
    groups = (len(scores) + 4095) // 4096
    out_scores = np.zeros(groups, dtype=np.float32)
    out_ids = np.zeros(groups, dtype=np.uint32)
    lib.fgo_argmax_reduce(_ptr(out_scores), _ptr(out_ids), _ptr(scores), _ptr(ids), len(scores))
    return out_scores, out_ids


def topk_select(lib, scores, ids, k: int):
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    ids = None if ids is None else np.ascontiguousarray(ids, dtype=np.uint32)
    groups = (len(scores) + 1023) // 1024
    out_scores = np.zeros(groups * k, dtype=np.float32)
    out_ids = np.zeros(groups * k, dtype=np.uint32)
    lib.fgo_topk_select(_ptr(out_scores), _ptr(out_ids), _ptr(scores), _ptr(ids), len(scores), k)
    return out_scores, out_ids


def topk_reduce(lib, scores, ids=None):
    """Sorted top-512 of every 4096-element tile (fg_vk_topk_reduce)."""
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    ids = None if ids is None else np.ascontiguousarray(ids, dtype=np.uint32)
    groups = (len(scores) + 4095) // 4096
    out_scores = np.zeros(groups * 512, dtype=np.float32)
    out_ids = np.zeros(groups * 512, dtype=np.uint32)
    produced = lib.fgo_topk_reduce(_ptr(out_scores), _ptr(out_ids), _ptr(scores), _ptr(ids), len(scores))
    return out_scores[:produced], out_ids[:produced]


def router_topk(lib, logits, k: int, reference: bool = False):
    """(status, ids, weights) of one token's router logits; `reference` calls the reference's
    own fg_q38_router_topk (only in the reference build of the oracle)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    ids = np.zeros(k, dtype=np.uint32)
    weights = np.zeros(k, dtype=np.float32)
    if reference:
        fn = lib.fg_q38_router_topk
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, POINTER(OracleError)]
        status = fn(_ptr(logits), len(logits), k, _ptr(ids), _ptr(weights), byref(OracleError()))
    else:
        status = lib.fgo_router_topk(_ptr(logits), len(logits), k, _ptr(ids), _ptr(weights))
    return status, ids, weights


def sample_batch(lib, logits: np.ndarray, configs, uniforms=None, history_tokens=None,
                 history_offsets=None, allow_no_topk: bool = False, threads: int = 1,
                 want_candidates: bool = False, vocab: int | None = None):
    """logits: [rows, stride] float32, or uint16 holding bf16 bit patterns."""
    rows, stride = logits.shape
    vocab = stride if vocab is None else vocab
    dtype = 1 if logits.dtype == np.uint16 else 0
    logits = np.ascontiguousarray(logits)
    cfgs = _configs(configs)
    uniforms = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float32)
    if history_tokens is not None:
        history_tokens = np.ascontiguousarray(history_tokens, dtype=np.uint32)
        history_offsets = np.ascontiguousarray(history_offsets, dtype=np.uint64)
    tokens = np.zeros(rows, dtype=np.uint32)
    token_logits = np.zeros(rows, dtype=np.float32)
    row_status = np.zeros(rows, dtype=np.uint32)
    cands = (OracleCandidates * rows)() if want_candidates else None
    status = lib.fgo_sample_batch(_ptr(logits), dtype, rows, vocab, stride, _ptr(history_tokens),
                                  _ptr(history_offsets), cfgs, len(cfgs), allow_no_topk,
                                  _ptr(uniforms), _ptr(tokens), _ptr(token_logits), _ptr(row_status),
                                  cands, threads)
    return status, tokens, token_logits, row_status, cands


def shard_topk(lib, logits: np.ndarray, configs, vocab_offset: int, vocab_total: int, k_shard: int,
               history_tokens=None, history_offsets=None):
    rows, stride = logits.shape
    dtype = 1 if logits.dtype == np.uint16 else 0
    logits = np.ascontiguousarray(logits)
    cfgs = _configs(configs)
    if history_tokens is not None:
        history_tokens = np.ascontiguousarray(history_tokens, dtype=np.uint32)
        history_offsets = np.ascontiguousarray(history_offsets, dtype=np.uint64)
    scores = np.zeros((rows, k_shard), dtype=np.float32)
    ids = np.zeros((rows, k_shard), dtype=np.uint32)
    row_status = np.zeros(rows, dtype=np.uint32)
    status = lib.fgo_shard_topk(_ptr(logits), dtype, rows, stride, stride, vocab_offset, vocab_total,
                                _ptr(history_tokens), _ptr(history_offsets), cfgs, len(cfgs), k_shard,
                                _ptr(scores), _ptr(ids), _ptr(row_status))
    return status, scores, ids, row_status


def merge_select(lib, scores: np.ndarray, ids: np.ndarray, shard_first, shard_width, configs,
                 uniforms=None, want_candidates: bool = False):
    """scores / ids: [shards, rows, k_shard]."""
    shards, rows, k_shard = scores.shape
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    first = np.ascontiguousarray(shard_first, dtype=np.uint32)
    width = np.ascontiguousarray(shard_width, dtype=np.uint32)
    cfgs = _configs(configs)
    uniforms = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float32)
    tokens = np.zeros(rows, dtype=np.uint32)
    token_logits = np.zeros(rows, dtype=np.float32)
    row_status = np.zeros(rows, dtype=np.uint32)
    cands = (OracleCandidates * rows)() if want_candidates else None
    status = lib.fgo_merge_select(_ptr(scores), _ptr(ids), shards, rows, k_shard, _ptr(first),
                                  _ptr(width), cfgs, len(cfgs), _ptr(uniforms), _ptr(tokens),
                                  _ptr(token_logits), _ptr(row_status), cands)
    return status, tokens, token_logits, row_status, cands
