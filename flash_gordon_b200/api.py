"""Python mirror of the C operators: same names, same argument meaning.

`Context` wraps an fg_cuda_context bound to PyTorch's current stream, so the
kernels order themselves with the torch ops that produced the logits.  Torch is
used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_float, c_uint32, c_void_p
from dataclasses import dataclass

import torch

from . import (FG_CUDA_BF16, FG_CUDA_F32, FG_CUDA_SAMPLE_ALLOW_NO_TOPK, FG_CUDA_SAMPLE_ASYNC, FG_OK,
               MAX_CANDIDATES, FgError, FgStatusError, SampleArgs, SampleDebug, SamplerConfig,
               config_array, load_library)


def _pointer(tensor: torch.Tensor | None):
    return None if tensor is None else c_void_p(tensor.data_ptr())


@dataclass
class SampleResult:
    tokens: torch.Tensor        # uint32 bits in an int32 tensor
    token_logits: torch.Tensor  # fp32
    row_status: torch.Tensor    # int32 fg_status per row
    status: int                 # status of the lowest failing row
    message: str
    debug: dict | None = None


class Tensor:
    """fg_cuda_tensor handle (owned allocation, view, or wrapped torch memory)."""

    def __init__(self, context: "Context", handle: c_void_p, keepalive=None):
        self.context = context
        self.handle = handle
        self._keepalive = keepalive

    def __del__(self):
        # a tensor must not outlive its context (the C handle points into it)
        if getattr(self, "handle", None) and getattr(self.context, "handle", None):
            self.context.lib.fg_cuda_tensor_destroy(self.handle)
        self.handle = None

    @property
    def nbytes(self) -> int:
        return self.context.lib.fg_cuda_tensor_bytes(self.handle)

    def write(self, data: bytes | torch.Tensor, offset: int = 0) -> None:
        if isinstance(data, torch.Tensor):
            data = data.contiguous().cpu().numpy().tobytes()
        err = FgError()
        buf = ctypes.create_string_buffer(data, len(data))
        status = self.context.lib.fg_cuda_tensor_write(self.handle, offset, buf, len(data), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())

    def read(self, nbytes: int | None = None, offset: int = 0) -> bytes:
        nbytes = self.nbytes - offset if nbytes is None else nbytes
        buf = ctypes.create_string_buffer(nbytes)
        err = FgError()
        status = self.context.lib.fg_cuda_tensor_read(self.handle, offset, buf, nbytes, byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        return buf.raw


class Context:
    """fg_cuda_context on `device`, enqueueing on torch's current stream."""

    def __init__(self, device: int | None = None, use_torch_stream: bool = True):
        self.lib = load_library()
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device = device
        handle = c_void_p()
        err = FgError()
        status = self.lib.fg_cuda_context_create(device, byref(handle), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        self.handle = handle
        if use_torch_stream:
            self.bind_torch_stream()

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.fg_cuda_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def bind_torch_stream(self) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        err = FgError()
        status = self.lib.fg_cuda_context_set_stream(self.handle, c_void_p(stream), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())

    @property
    def sm_count(self) -> int:
        return self.lib.fg_cuda_context_sm_count(self.handle)

    @property
    def launches(self) -> int:
        return self.lib.fg_cuda_context_launches(self.handle)

    @property
    def scratch_bytes(self) -> int:
        return self.lib.fg_cuda_context_scratch_bytes(self.handle)

    def set_splits(self, splits: int) -> None:
        err = FgError()
        status = self.lib.fg_cuda_context_set_splits(self.handle, splits, byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())

    def ring_controls(self, deal: int = 0, wait_polls: int = 0, withhold: tuple[int, int] | None = None) -> None:
        """Test seam of the ring kernel: how work is dealt out (0 planner, 1 whole rows,
        2 tiles), the poll budget of its device-side waits (0 = default), and one tile
        (CTA, request number of its warp 0) that is never fetched, so that a wait runs out."""
        armed, cta, issue = (0, 0, 0) if withhold is None else (1, withhold[0], withhold[1])
        status = self.lib.fg_cuda_internal_ring_controls(self.handle, deal, wait_polls, armed, cta, issue)
        if status != FG_OK:
            raise FgStatusError(status, "invalid ring controls")

    def set_path(self, path: int) -> None:
        """0 automatic, 1 register-prefetch kernel, 2 shared-memory ring kernel, 3 ring where rows allow."""
        err = FgError()
        status = self.lib.fg_cuda_context_set_path(self.handle, path, byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())

    def begin(self) -> None:
        err = FgError()
        status = self.lib.fg_cuda_begin(self.handle, byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())

    def end(self) -> None:
        err = FgError()
        status = self.lib.fg_cuda_end(self.handle, byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())

    # ------------------------------------------------------------- tensors
    def tensor(self, nbytes: int) -> Tensor:
        handle = c_void_p()
        err = FgError()
        status = self.lib.fg_cuda_tensor_create(self.handle, nbytes, byref(handle), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        return Tensor(self, handle)

    def tensor_from(self, data: torch.Tensor) -> Tensor:
        """Owned device tensor initialised from a host torch tensor (tests)."""
        raw = data.contiguous().cpu().numpy().tobytes()
        out = self.tensor(max(len(raw), 1))
        if raw:
            out.write(raw)
        return out

    def wrap(self, data: torch.Tensor) -> Tensor:
        handle = c_void_p()
        err = FgError()
        nbytes = data.numel() * data.element_size()
        status = self.lib.fg_cuda_tensor_wrap(self.handle, c_void_p(data.data_ptr()), nbytes,
                                              byref(handle), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        return Tensor(self, handle, keepalive=data)

    def view(self, base: Tensor, offset: int, nbytes: int) -> Tensor:
        handle = c_void_p()
        err = FgError()
        status = self.lib.fg_cuda_tensor_view(base.handle, offset, nbytes, byref(handle), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        return Tensor(self, handle, keepalive=base)

    # ---------------------------------------------------- device operators
    def apply_penalties(self, logits: Tensor, counts: Tensor, values: int, presence: float,
                        frequency: float, repetition: float) -> int:
        err = FgError()
        return self.lib.fg_cuda_apply_penalties(self.handle, logits.handle, counts.handle, values,
                                                presence, frequency, repetition, byref(err))

    def argmax_reduce(self, out_scores: Tensor, out_ids: Tensor, in_scores: Tensor,
                      in_ids: Tensor | None, count: int) -> tuple[int, int]:
        produced = c_uint32(0)
        err = FgError()
        status = self.lib.fg_cuda_argmax_reduce(
            self.handle, out_scores.handle, out_ids.handle, in_scores.handle,
            in_ids.handle if in_ids is not None else None, count, byref(produced), byref(err))
        return status, produced.value

    def topk_select(self, out_scores: Tensor, out_ids: Tensor, in_scores: Tensor,
                    in_ids: Tensor | None, count: int, k: int) -> tuple[int, int]:
        produced = c_uint32(0)
        err = FgError()
        status = self.lib.fg_cuda_topk_select(
            self.handle, out_scores.handle, out_ids.handle, in_scores.handle,
            in_ids.handle if in_ids is not None else None, count, k, byref(produced), byref(err))
        return status, produced.value

    def topk_reduce(self, out_scores: Tensor, out_ids: Tensor, in_scores: Tensor, in_ids: Tensor | None,
                    count: int) -> tuple[int, int]:
        produced = c_uint32(0)
        err = FgError()
        status = self.lib.fg_cuda_topk_reduce(
            self.handle, out_scores.handle, out_ids.handle, in_scores.handle,
            in_ids.handle if in_ids is not None else None, count, byref(produced), byref(err))
        return status, produced.value

    def router_topk(self, selected: Tensor, gates: Tensor, logits: Tensor, experts: int, tokens: int,
                    k: int) -> tuple[int, str]:
        err = FgError()
        status = self.lib.fg_cuda_router_topk(self.handle, selected.handle, gates.handle, logits.handle,
                                              experts, tokens, k, byref(err))
        return status, err.text()

    def history_reset(self, counts: Tensor, vocab: int, history) -> int:
        array = (c_uint32 * max(len(history), 1))(*history)
        err = FgError()
        return self.lib.fg_cuda_history_reset(self.handle, counts.handle, vocab, array,
                                              len(history), byref(err))

    def history_increment(self, counts: Tensor, vocab: int, token: int) -> int:
        err = FgError()
        return self.lib.fg_cuda_history_increment(self.handle, counts.handle, vocab, token, byref(err))

    # -------------------------------------------------------- fused batched
    def _args(self, logits, configs, uniforms, history_tokens, history_offsets, history_max,
              vocab, flags, outputs, debug_struct):
        if logits.dtype == torch.float32:
            dtype = FG_CUDA_F32
        elif logits.dtype == torch.bfloat16:
            dtype = FG_CUDA_BF16
        else:
            raise TypeError("logits must be float32 or bfloat16")
        if logits.dim() != 2 or logits.stride(1) != 1:
            raise ValueError("logits must be a 2-D tensor with unit column stride")
        rows = logits.shape[0]
        vocab = logits.shape[1] if vocab is None else vocab
        cfgs = config_array(configs)
        tokens, token_logits, row_status = outputs
        args = SampleArgs()
        args.logits = logits.data_ptr()
        args.dtype = dtype
        args.rows = rows
        args.vocab = vocab
        args.flags = flags
        args.row_stride = logits.stride(0) if rows > 1 else max(logits.stride(0), vocab)
        args.history_tokens = history_tokens.data_ptr() if history_tokens is not None else None
        args.history_offsets = history_offsets.data_ptr() if history_offsets is not None else None
        args.history_max = history_max
        args.config_count = len(cfgs)
        args.configs = ctypes.cast(cfgs, POINTER(SamplerConfig))
        args.uniforms = uniforms.data_ptr() if uniforms is not None else None
        args.tokens = tokens.data_ptr() if tokens is not None else None
        args.token_logits = token_logits.data_ptr() if token_logits is not None else None
        args.row_status = row_status.data_ptr()
        args.debug = ctypes.pointer(debug_struct) if debug_struct is not None else None
        return args, cfgs

    def sample_batch(self, logits: torch.Tensor, configs, uniforms: torch.Tensor | None = None,
                     history_tokens: torch.Tensor | None = None,
                     history_offsets: torch.Tensor | None = None, history_max: int = 0,
                     vocab: int | None = None, allow_no_topk: bool = False,
                     asynchronous: bool = False, debug: bool = False, out=None,
                     check: bool = False) -> SampleResult:
        """fg_cuda_sample_batch on device tensors.

        logits [rows, >=vocab] fp32/bf16; history_tokens int32 (uint32 ids),
        history_offsets int64 [rows+1]; uniforms fp32 [rows]."""
        rows = logits.shape[0]
        device = logits.device
        if out is None:
            out = (torch.empty(rows, dtype=torch.int32, device=device),
                   torch.empty(rows, dtype=torch.float32, device=device),
                   torch.empty(rows, dtype=torch.int32, device=device))
        dbg_struct, dbg = None, None
        if debug:
            dbg = {
                "count": torch.zeros(rows, dtype=torch.int32, device=device),
                "ids": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.int32, device=device),
                "scores": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.float32, device=device),
                "raw": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.float64, device=device),
                "tempered": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.float64, device=device),
            }
            dbg_struct = SampleDebug(dbg["count"].data_ptr(), dbg["ids"].data_ptr(),
                                     dbg["scores"].data_ptr(), dbg["raw"].data_ptr(),
                                     dbg["tempered"].data_ptr())
        flags = (FG_CUDA_SAMPLE_ASYNC if asynchronous else 0) | \
                (FG_CUDA_SAMPLE_ALLOW_NO_TOPK if allow_no_topk else 0)
        args, keep = self._args(logits, configs, uniforms, history_tokens, history_offsets,
                                history_max, vocab, flags, out, dbg_struct)
        err = FgError()
        status = self.lib.fg_cuda_sample_batch(self.handle, byref(args), byref(err))
        del keep
        if check and status != FG_OK:
            raise FgStatusError(status, err.text())
        return SampleResult(out[0], out[1], out[2], status, err.text(), dbg)

    def prepared_sample(self, logits, configs, uniforms, history_tokens, history_offsets,
                        history_max, out, allow_no_topk: bool = False, asynchronous: bool = True):
        """Builds the argument block once; the returned callable re-issues the same
        fg_cuda_sample_batch call (decode loops call it once per step)."""
        flags = (FG_CUDA_SAMPLE_ASYNC if asynchronous else 0) | \
                (FG_CUDA_SAMPLE_ALLOW_NO_TOPK if allow_no_topk else 0)
        args, keep = self._args(logits, configs, uniforms, history_tokens, history_offsets,
                                history_max, None, flags, out, None)
        err = FgError()
        call, handle, args_ref, err_ref = self.lib.fg_cuda_sample_batch, self.handle, byref(args), byref(err)

        def issue() -> int:
            status = call(handle, args_ref, err_ref)
            if status != FG_OK:
                raise FgStatusError(status, err.text())
            return status

        issue.keepalive = (args, keep, err, logits, uniforms, history_tokens, history_offsets, out)
        return issue

    def sample_batch_host(self, logits: torch.Tensor, configs, uniforms: torch.Tensor | None,
                          history_tokens: torch.Tensor | None, history_offsets: torch.Tensor | None,
                          history_max: int, out=None, allow_no_topk: bool = False) -> SampleResult:
        """fg_cuda_sample_batch_host: every tensor lives in host memory."""
        rows = logits.shape[0]
        if out is None:
            out = (torch.empty(rows, dtype=torch.int32), torch.empty(rows, dtype=torch.float32),
                   torch.empty(rows, dtype=torch.int32))
        flags = FG_CUDA_SAMPLE_ALLOW_NO_TOPK if allow_no_topk else 0
        args, keep = self._args(logits, configs, uniforms, history_tokens, history_offsets,
                                history_max, None, flags, out, None)
        err = FgError()
        status = self.lib.fg_cuda_sample_batch_host(self.handle, byref(args), byref(err))
        del keep
        return SampleResult(out[0], out[1], out[2], status, err.text(), None)

    def shard_topk(self, logits: torch.Tensor, configs, vocab_offset: int, vocab_total: int,
                   k_shard: int, history_tokens=None, history_offsets=None, history_max: int = 0,
                   out=None, asynchronous: bool = False):
        """fg_cuda_shard_topk: returns (scores [rows,k], ids [rows,k] int32, row_status, status)."""
        rows = logits.shape[0]
        device = logits.device
        if out is None:
            out = (torch.empty(rows, k_shard, dtype=torch.float32, device=device),
                   torch.empty(rows, k_shard, dtype=torch.int32, device=device))
        row_status = torch.empty(rows, dtype=torch.int32, device=device)
        flags = FG_CUDA_SAMPLE_ASYNC if asynchronous else 0
        args, keep = self._args(logits, configs, None, history_tokens, history_offsets, history_max,
                                None, flags, (None, None, row_status), None)
        err = FgError()
        status = self.lib.fg_cuda_shard_topk(self.handle, byref(args), vocab_offset, vocab_total,
                                             k_shard, c_void_p(out[0].data_ptr()),
                                             c_void_p(out[1].data_ptr()), byref(err))
        del keep
        return out[0], out[1], row_status, status

    def merge_select(self, candidate_scores: torch.Tensor, candidate_ids: torch.Tensor, rows: int,
                     shards: int, k_shard: int, shard_first, shard_width, configs,
                     uniforms: torch.Tensor | None, debug: bool = False,
                     asynchronous: bool = False) -> SampleResult:
        """fg_cuda_merge_select over [shards][rows][k_shard] candidates."""
        device = candidate_scores.device
        out = (torch.empty(rows, dtype=torch.int32, device=device),
               torch.empty(rows, dtype=torch.float32, device=device),
               torch.empty(rows, dtype=torch.int32, device=device))
        dbg_struct, dbg = None, None
        if debug:
            dbg = {
                "count": torch.zeros(rows, dtype=torch.int32, device=device),
                "ids": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.int32, device=device),
                "scores": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.float32, device=device),
                "raw": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.float64, device=device),
                "tempered": torch.zeros(rows, MAX_CANDIDATES, dtype=torch.float64, device=device),
            }
            dbg_struct = SampleDebug(dbg["count"].data_ptr(), dbg["ids"].data_ptr(),
                                     dbg["scores"].data_ptr(), dbg["raw"].data_ptr(),
                                     dbg["tempered"].data_ptr())
        cfgs = config_array(configs)
        args = SampleArgs()
        args.rows = rows
        args.flags = FG_CUDA_SAMPLE_ASYNC if asynchronous else 0
        args.config_count = len(cfgs)
        args.configs = ctypes.cast(cfgs, POINTER(SamplerConfig))
        args.uniforms = uniforms.data_ptr() if uniforms is not None else None
        args.tokens = out[0].data_ptr()
        args.token_logits = out[1].data_ptr()
        args.row_status = out[2].data_ptr()
        args.debug = ctypes.pointer(dbg_struct) if dbg_struct is not None else None
        first = (c_uint32 * shards)(*shard_first)
        width = (c_uint32 * shards)(*shard_width)
        err = FgError()
        status = self.lib.fg_cuda_merge_select(
            self.handle, byref(args), c_void_p(candidate_scores.data_ptr()),
            c_void_p(candidate_ids.data_ptr()), shards, k_shard, first, width, byref(err))
        return SampleResult(out[0], out[1], out[2], status, err.text(), dbg)


def select(config: SamplerConfig, scores, ids, uniform: float):
    """fg_sampler_select on host lists; returns (status, token, logit, message)."""
    lib = load_library()
    n = len(scores)
    score_array = (c_float * max(n, 1))(*scores)
    id_array = (c_uint32 * max(n, 1))(*ids)
    token, logit, err = c_uint32(0), c_float(0.0), FgError()
    status = lib.fg_sampler_select(byref(config), score_array, id_array, n, uniform, byref(token),
                                   byref(logit), byref(err))
    return status, token.value, logit.value, err.text()


class OutputExecutor:
    """fg_cuda_output_executor: session slots whose token histories stay on the GPU between
    decode steps (the reference's fg_output executor, include/fg_output.h:42-66)."""

    def __init__(self, context: Context, vocab: int, session_slots: int, history_capacity: int):
        self.context = context
        self.lib = context.lib
        self.vocab = vocab
        handle = c_void_p()
        err = FgError()
        status = self.lib.fg_cuda_output_executor_create(context.handle, vocab, session_slots,
                                                         history_capacity, byref(handle), byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        self.handle = handle

    def close(self) -> None:
        if getattr(self, "handle", None) and getattr(self.context, "handle", None):
            self.lib.fg_cuda_output_executor_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_session(self, slot: int) -> None:
        self.lib.fg_cuda_output_set_session(self.handle, slot)

    @property
    def session(self) -> int:
        return self.lib.fg_cuda_output_session(self.handle)

    def history_length(self, slot: int) -> int:
        return self.lib.fg_cuda_output_history_length(self.handle, slot)

    def history_reset(self, history) -> int:
        array = (c_uint32 * max(len(history), 1))(*history)
        err = FgError()
        return self.lib.fg_cuda_output_history_reset(self.handle, array, len(history), byref(err))

    def history_increment(self, token: int) -> int:
        return self.lib.fg_cuda_output_history_increment(self.handle, token, byref(FgError()))

    def sample(self, logits: Tensor, config: SamplerConfig, uniform: float):
        """fg_cuda_output_sample: (status, token, logit, message) for the current session."""
        token, logit, err = c_uint32(0), c_float(0.0), FgError()
        status = self.lib.fg_cuda_output_sample(self.handle, logits.handle, byref(config), uniform,
                                                byref(token), byref(logit), byref(err))
        return status, token.value, logit.value, err.text()

    def greedy(self, logits: Tensor):
        token, logit, err = c_uint32(0), c_float(0.0), FgError()
        status = self.lib.fg_cuda_output_greedy(self.handle, logits.handle, byref(token), byref(logit), byref(err))
        return status, token.value, logit.value, err.text()

    def sample_sessions(self, logits: torch.Tensor, configs, uniforms: torch.Tensor | None, slots,
                        allow_no_topk: bool = False) -> SampleResult:
        """fg_cuda_output_sample_sessions: one decode step, row r in session slots[r]."""
        rows = logits.shape[0]
        device = logits.device
        out = (torch.empty(rows, dtype=torch.int32, device=device),
               torch.empty(rows, dtype=torch.float32, device=device),
               torch.empty(rows, dtype=torch.int32, device=device))
        flags = FG_CUDA_SAMPLE_ALLOW_NO_TOPK if allow_no_topk else 0
        args, keep = self.context._args(logits, configs, uniforms, None, None, 0, None, flags, out, None)
        slot_array = (c_uint32 * rows)(*slots)
        err = FgError()
        status = self.lib.fg_cuda_output_sample_sessions(self.handle, byref(args), slot_array, byref(err))
        del keep
        return SampleResult(out[0], out[1], out[2], status, err.text(), None)
