"""fg_cuda_sample_batch_static — the entry point for callers that may not allocate GPU
memory (a process whose own arena already holds the whole device, or a decode loop
that cannot take the stall an allocation may cause).  Its scratch is an array inside
the library, shared by all calls, so the test makes two calls in a row with
different inputs and checks each against the context-based entry point, bit for bit.
Collected last on purpose: a run that stops at the first failure has then already
run every other test."""
import ctypes
from ctypes import POINTER, byref, c_void_p

import numpy as np
import pytest
import torch

from flash_gordon_b200 import (FG_CUDA_BF16, FG_CUDA_F32, FG_ERR_ARGUMENT, FG_ERR_LIMIT, FG_ERR_UNAVAILABLE, FG_OK,
                               FgError, SampleArgs, SamplerConfig, config_array, synth)
from helpers import as_u32, assert_rows_equal, random_workload, run_oracle

pytestmark = pytest.mark.gpu


def call_static(library, w, out, stream=0, flags=0):
    cfgs = config_array(w.configs)
    args = SampleArgs()
    args.logits = w.logits.data_ptr()
    args.dtype = FG_CUDA_BF16 if w.logits.dtype == torch.bfloat16 else FG_CUDA_F32
    args.rows, args.vocab = w.rows, w.vocab
    args.row_stride = w.logits.stride(0)
    args.history_tokens = w.history_tokens.data_ptr() if w.history_tokens is not None else None
    args.history_offsets = w.history_offsets.data_ptr() if w.history_offsets is not None else None
    args.history_max = w.history_max
    args.config_count = len(cfgs)
    args.configs = ctypes.cast(cfgs, POINTER(SamplerConfig))
    args.uniforms = w.uniforms.data_ptr()
    args.flags = flags
    args.tokens, args.token_logits, args.row_status = (t.data_ptr() for t in out)
    err = FgError()
    status = library.fg_cuda_sample_batch_static(0, c_void_p(stream), byref(args), byref(err))
    return status, err.text()


def fresh_outputs(rows):
    return (torch.full((rows,), -1, dtype=torch.int32, device="cuda"),
            torch.full((rows,), -1.0, dtype=torch.float32, device="cuda"),
            torch.full((rows,), -1, dtype=torch.int32, device="cuda"))


def test_static_scratch_entry_matches_the_context_entry_twice(library, context):
    shared = SamplerConfig.make(temperature=0.9, top_p=0.9, top_k=40, presence=0.3, frequency=0.4,
                                repetition=1.1)
    per_row = [SamplerConfig.make(temperature=0.0 if r % 4 == 0 else 0.6 + 0.05 * r, top_p=0.8,
                                  top_k=1 + 3 * r, frequency=0.1 * (r % 3), repetition=1.0 + 0.02 * r)
               for r in range(20)]
    # few rows, so every row is shared by several CTAs and the hand-off scratch is in play;
    # the second call has other sizes, so stale contents of the first would show
    first = random_workload(24, 40_000, 600, [shared], 71, quantize=0.25, specials=2).to("cuda")
    second = random_workload(20, 33_333, 900, per_row, 72, quantize=0.5).to("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for w in (first, second):
        want = context.sample_batch(w.logits, w.configs, w.uniforms, w.history_tokens, w.history_offsets,
                                    w.history_max)
        torch.cuda.synchronize()
        out = fresh_outputs(w.rows)
        status, message = call_static(library, w, out, stream)
        assert status == FG_OK, message
        torch.cuda.synchronize()
        assert np.array_equal(as_u32(out[2]), as_u32(want.row_status))
        ok = as_u32(want.row_status) == FG_OK
        assert ok.any()
        assert np.array_equal(as_u32(out[0])[ok], as_u32(want.tokens)[ok])
        assert np.array_equal(out[1].cpu().numpy().view(np.uint32)[ok],
                              want.token_logits.cpu().numpy().view(np.uint32)[ok])


class _Result:
    """The outputs of the static entry in the shape the comparison helpers take."""

    def __init__(self, out, status):
        self.tokens, self.token_logits, self.row_status = out
        ok = as_u32(out[2])
        failing = np.nonzero(ok)[0]
        self.status = int(ok[failing[0]]) if failing.size else status


def test_static_scratch_entry_against_the_oracle_without_allocating(library, context):
    """The entry's own results against the CPU oracle (not only against the other entry
    point), for fp32 and bf16 rows, and the promise itself: free device memory is the same
    before and after the calls (the first call on the device has been made by then)."""
    cfg = SamplerConfig.make(temperature=0.8, top_p=0.9, top_k=33, presence=0.2, frequency=0.3, repetition=1.05)
    cases = [random_workload(12, 30_000, 500, [cfg], 81, quantize=0.25, specials=2),
             random_workload(9, 20_001, 300, [cfg], 82, quantize=0.5, dtype=torch.bfloat16)]
    warm = cases[0].to("cuda")
    assert call_static(library, warm, fresh_outputs(warm.rows))[0] == FG_OK  # first call: symbol lookup
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for w in cases:
        want = run_oracle(w)
        on_gpu = w.to("cuda")
        out = fresh_outputs(w.rows)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        for _ in range(2):
            status, message = call_static(library, on_gpu, out, stream)
            assert status == FG_OK, message
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the entry that allocates nothing allocated"
        assert_rows_equal(_Result(out, 0), want, f"static entry, {w.logits.dtype}")


def test_static_scratch_entry_rejects_what_does_not_fit(library):
    cfg = SamplerConfig.make()
    w = synth.Workload("tiny", torch.zeros(2, 64, device="cuda"), [cfg], torch.zeros(2, device="cuda"),
                       None, None, 0)
    out = fresh_outputs(2)
    assert call_static(library, w, out)[0] == FG_OK
    torch.cuda.synchronize()
    # more rows than the built-in scratch can track: a clear refusal, nothing launched
    cfgs = config_array([cfg])
    args = SampleArgs()
    args.logits = w.logits.data_ptr()
    args.dtype = FG_CUDA_F32
    args.rows, args.vocab, args.row_stride = 1_200_000, 64, 0
    args.config_count = 1
    args.configs = ctypes.cast(cfgs, POINTER(SamplerConfig))
    args.uniforms = out[1].data_ptr()
    args.tokens, args.token_logits, args.row_status = (t.data_ptr() for t in out)
    err = FgError()
    assert library.fg_cuda_sample_batch_static(0, None, byref(args), byref(err)) == FG_ERR_ARGUMENT
    args.row_stride = 64  # now well-formed, but 1.2 M rows need more than 4 MiB of counters
    status = library.fg_cuda_sample_batch_static(0, None, byref(args), byref(err))
    assert status == FG_ERR_LIMIT and "scratch" in err.text()
    # sizes whose history structure forces several CTAs per row while the hand-off of that many
    # does not fit the scratch: the entry must say so and return (it used to replan forever).
    # Only the arguments are read: nothing is launched, so the pointers may be small buffers.
    penalised = config_array([SamplerConfig.make(temperature=0.9, top_p=0.9, top_k=20, frequency=0.5)])
    args.rows, args.vocab, args.row_stride = 2100, 151_936, 151_936
    args.history_max = 262_144
    tokens = torch.zeros(8, dtype=torch.int32, device="cuda")
    offsets = torch.zeros(8, dtype=torch.int64, device="cuda")
    args.history_tokens, args.history_offsets = tokens.data_ptr(), offsets.data_ptr()
    args.configs = ctypes.cast(penalised, POINTER(SamplerConfig))
    status = library.fg_cuda_sample_batch_static(0, None, byref(args), byref(err))
    assert status == FG_ERR_LIMIT and "fits both" in err.text()
    # rows without a top-k cut are offered by the context entry only, and the text says so
    w5 = synth.Workload("nucleus", torch.zeros(2, 64, device="cuda"), [SamplerConfig.make(1.0, 0.9, 0)],
                        torch.zeros(2, device="cuda"), None, None, 0, allow_no_topk=True)
    status, message = call_static(library, w5, fresh_outputs(2), flags=2)
    assert status == FG_ERR_UNAVAILABLE and "fg_cuda_sample_batch" in message
