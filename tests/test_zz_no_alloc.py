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

from flash_gordon_b200 import (FG_CUDA_F32, FG_ERR_ARGUMENT, FG_ERR_LIMIT, FG_OK, FgError, SampleArgs,
                               SamplerConfig, config_array, synth)
from helpers import as_u32, random_workload

pytestmark = pytest.mark.gpu


def call_static(library, w, out, stream=0):
    cfgs = config_array(w.configs)
    args = SampleArgs()
    args.logits = w.logits.data_ptr()
    args.dtype = FG_CUDA_F32
    args.rows, args.vocab = w.rows, w.vocab
    args.row_stride = w.logits.stride(0)
    args.history_tokens = w.history_tokens.data_ptr() if w.history_tokens is not None else None
    args.history_offsets = w.history_offsets.data_ptr() if w.history_offsets is not None else None
    args.history_max = w.history_max
    args.config_count = len(cfgs)
    args.configs = ctypes.cast(cfgs, POINTER(SamplerConfig))
    args.uniforms = w.uniforms.data_ptr()
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


def test_static_scratch_entry_rejects_what_does_not_fit(library):
    cfg = SamplerConfig.make()
    w = synth.Workload("tiny", torch.zeros(2, 64, device="cuda"), [cfg], torch.zeros(2, device="cuda"),
                       None, None, 0)
    out = fresh_outputs(2)
    assert call_static(library, w, out)[0] == FG_OK
    torch.cuda.synchronize()
    # more rows than the built-in scratch can track: a clear refusal, nothing launched
    huge = synth.Workload("huge", torch.zeros(2, 64, device="cuda").expand(2, 64), [cfg],
                          torch.zeros(2, device="cuda"), None, None, 0)
    cfgs = config_array([cfg])
    args = SampleArgs()
    args.logits = huge.logits.data_ptr()
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
