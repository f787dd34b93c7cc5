"""Parity of the fused batched path (fg_cuda_sample_batch) with the CPU oracle:
token ids, the penalised logit of the pick and per-row status bit for bit;
probabilities within 1e-5 relative."""
import itertools

import numpy as np
import pytest
import torch

from flash_gordon_b200 import (FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_ERR_LIMIT, FG_ERR_MISMATCH, FG_OK,
                               SamplerConfig, synth)
from helpers import (as_u32, assert_candidates_close, assert_rows_equal, random_workload, run_gpu,
                     run_oracle)

pytestmark = pytest.mark.gpu

PROBABILITY_RTOL = 1e-5


@pytest.fixture(params=["ring_if_possible", "registers"], autouse=True)
def kernel_path(context, request):
    """Every case runs twice: through the shared-memory ring kernel wherever rows are
    16-byte aligned, and pinned to the register-prefetch kernel."""
    context.set_path(3 if request.param == "ring_if_possible" else 1)
    yield request.param
    context.set_path(0)


def test_config1_greedy_single_row(context):
    w = synth.config1()
    expected = run_oracle(w, want_candidates=True)
    assert expected[0] == FG_OK
    for splits in (0, 1, 5, 16):
        context.set_splits(splits)
        assert_rows_equal(run_gpu(context, w), expected, f"config1 splits={splits}")
    context.set_splits(0)


def test_config2_topk_topp_presence(context):
    w = synth.config2()
    expected = run_oracle(w, want_candidates=True)
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "config2")
    assert_candidates_close(result, expected, PROBABILITY_RTOL, "config2")


def test_config3_reduced_rows(context):
    w = synth.config3(rows=48)
    expected = run_oracle(w, want_candidates=True)
    for splits in (0, 1, 4, 7):
        context.set_splits(splits)
        result = run_gpu(context, w, debug=True)
        assert_rows_equal(result, expected, f"config3 splits={splits}")
        assert_candidates_close(result, expected, PROBABILITY_RTOL, f"config3 splits={splits}")
    context.set_splits(0)


def test_config4_bf16_unsharded(context):
    w = synth.config4(rows=32)
    expected = run_oracle(w, want_candidates=True)
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "config4 unsharded")
    assert_candidates_close(result, expected, PROBABILITY_RTOL, "config4 unsharded")


VOCABS = [1, 2, 31, 32, 33, 255, 256, 257, 1023, 1024, 1025, 4095, 4096, 4097, 18992]


@pytest.mark.parametrize("vocab", VOCABS)
def test_sizes_sweep(context, vocab):
    seed = 1000 + vocab
    for k, history, rows in [(1, 0, 1), (2, 1, 2), (20, 64, 3), (50, 512, 5), (64, 4096, 2)]:
        cfg = SamplerConfig.make(temperature=0.9, top_p=0.9, top_k=k, presence=0.7, frequency=0.3,
                                 repetition=1.3)
        w = random_workload(rows, vocab, history, [cfg], seed + k, quantize=0.5, specials=min(3, vocab))
        expected = run_oracle(w, want_candidates=True)
        for splits in (0, 1, 3):
            context.set_splits(splits)
            result = run_gpu(context, w, debug=True)
            label = f"V={vocab} k={k} H={history} rows={rows} splits={splits}"
            assert_rows_equal(result, expected, label)
            assert_candidates_close(result, expected, PROBABILITY_RTOL, label)
    context.set_splits(0)


@pytest.mark.parametrize("vocab,rows", [(151_936, 5), (248_320, 3)])
def test_large_vocab_heavy_ties(context, vocab, rows):
    cfg = SamplerConfig.make(temperature=1.0, top_p=0.95, top_k=50, frequency=0.5, repetition=1.05)
    w = random_workload(rows, vocab, 4096, [cfg], 77, quantize=1.0, specials=5, uniform_history=False)
    expected = run_oracle(w, want_candidates=True)
    for splits in (0, 1, 2, 16):
        context.set_splits(splits)
        result = run_gpu(context, w, debug=True)
        assert_rows_equal(result, expected, f"ties V={vocab} splits={splits}")
        assert_candidates_close(result, expected, PROBABILITY_RTOL, f"ties V={vocab} splits={splits}")
    context.set_splits(0)


def test_all_equal_and_sorted_rows(context):
    """Worst cases for a streaming select: every value ties, or every later value is larger."""
    vocab = 20_000
    flat = torch.full((1, vocab), 1.0)
    rising = torch.arange(vocab, dtype=torch.float32).reshape(1, vocab) * 0.001
    falling = rising.flip(1).contiguous()
    logits = torch.cat([flat, rising, falling], 0)
    cfg = SamplerConfig.make(temperature=1.0, top_p=1.0, top_k=64)
    w = synth.Workload("edges", logits, [cfg], torch.tensor([0.0, 0.5, 0.999]), None, None, 0)
    expected = run_oracle(w, want_candidates=True)
    for splits in (1, 2, 5):
        context.set_splits(splits)
        result = run_gpu(context, w, debug=True)
        assert_rows_equal(result, expected, f"edges splits={splits}")
        assert_candidates_close(result, expected, PROBABILITY_RTOL, f"edges splits={splits}")
    context.set_splits(0)


def test_per_row_configs_mixed_modes(context):
    rows, vocab = 12, 5000
    configs = []
    for r in range(rows):
        if r % 3 == 0:
            configs.append(SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1,
                                              repetition=1.0 + 0.1 * (r % 2)))
        else:
            configs.append(SamplerConfig.make(temperature=0.5 + 0.1 * r, top_p=0.5 + 0.04 * r,
                                              top_k=1 + 5 * r, presence=0.1 * r - 0.5,
                                              frequency=0.2 * (r % 4) - 0.3, repetition=0.8 + 0.05 * r))
    w = random_workload(rows, vocab, 300, configs, 5)
    expected = run_oracle(w, want_candidates=True)
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "mixed")
    assert_candidates_close(result, expected, PROBABILITY_RTOL, "mixed")


def test_greedy_nonfinite_is_an_error(context):
    vocab = 9000
    base = torch.randn(4, vocab)
    base[0, 4567] = float("nan")
    base[1, 10] = float("-inf")
    base[1, 8000] = float("inf")
    base[2, 1] = 50.0
    plain = SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1)
    w = synth.Workload("wild", base, [plain], None, None, None, 0)
    expected = run_oracle(w)
    assert list(expected[3]) == [FG_ERR_MISMATCH, FG_ERR_MISMATCH, FG_OK, FG_OK]
    for splits in (1, 4):
        context.set_splits(splits)
        result = run_gpu(context, w)
        assert_rows_equal(result, expected, "wild greedy")
        assert result.status == FG_ERR_MISMATCH
        # the offending id is reported, as in "invalid output finalist at token %u"
        assert as_u32(result.tokens)[0] == 4567 and as_u32(result.tokens)[1] == 10
    context.set_splits(0)
    penalised = SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1, presence=1.0)
    w2 = random_workload(4, vocab, 50, [penalised], 9)
    w2.logits[3, 77] = float("nan")
    expected2 = run_oracle(w2)
    assert expected2[3][3] == FG_ERR_FORMAT
    assert_rows_equal(run_gpu(context, w2), expected2, "wild penalised greedy")


def test_sampled_rows_drop_nonfinite_and_fail_without_finite(context):
    vocab = 3000
    logits = torch.randn(3, vocab)
    logits[0, ::2] = float("nan")
    logits[1, :] = float("inf")
    logits[2, :] = float("-inf")
    logits[2, 5] = 1.0
    cfg = SamplerConfig.make(temperature=1.0, top_p=1.0, top_k=40)
    w = synth.Workload("drop", logits, [cfg], torch.tensor([0.3, 0.3, 0.3]), None, None, 0)
    expected = run_oracle(w, want_candidates=True)
    assert list(expected[3]) == [FG_OK, FG_ERR_FORMAT, FG_OK]
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "drop")
    assert_candidates_close(result, expected, PROBABILITY_RTOL, "drop")


def test_unaligned_rows_and_strides(context):
    cfg = SamplerConfig.make(temperature=0.8, top_p=0.9, top_k=30, presence=0.4, frequency=0.2)
    for dtype in (torch.float32, torch.bfloat16):
        w = random_workload(4, 5003, 200, [cfg], 31, dtype=dtype, stride=5003 + 7)
        expected = run_oracle(w, want_candidates=True)
        wd = w.to("cuda")
        wide = torch.zeros(4, 5010, dtype=dtype, device="cuda")
        wide[:, :5003] = wd.logits
        strided = wide[:, :5003]
        assert strided.stride(0) == 5010
        result = context.sample_batch(strided, wd.configs, wd.uniforms, wd.history_tokens,
                                      wd.history_offsets, wd.history_max, debug=True)
        assert_rows_equal(result, expected, f"stride {dtype}")
        assert_candidates_close(result, expected, PROBABILITY_RTOL, f"stride {dtype}")


def test_history_errors(context):
    cfg = SamplerConfig.make(temperature=1.0, top_p=0.9, top_k=10, presence=1.0)
    w = random_workload(3, 4000, 100, [cfg], 3)
    w.history_tokens[int(w.history_offsets[1])] = 4000  # first token of row 1 is out of range
    if int(w.history_offsets[2]) == int(w.history_offsets[1]):
        pytest.skip("row 1 drew an empty history")
    expected = run_oracle(w)
    assert expected[3][1] == FG_ERR_FORMAT
    assert_rows_equal(run_gpu(context, w), expected, "bad history token")
    # a history longer than the caller's bound is refused for that row
    w2 = random_workload(2, 4000, 100, [cfg], 4)
    wd = w2.to("cuda")
    result = context.sample_batch(wd.logits, wd.configs, wd.uniforms, wd.history_tokens,
                                  wd.history_offsets, 10)
    assert as_u32(result.row_status)[0] == FG_ERR_LIMIT


def test_argument_errors(context):
    cfg = SamplerConfig.make()
    logits = torch.randn(2, 100, device="cuda")
    uniforms = torch.rand(2, device="cuda")
    bad = SamplerConfig.make(top_k=65)
    assert context.sample_batch(logits, [bad], uniforms).status == FG_ERR_ARGUMENT
    no_topk = SamplerConfig.make(top_k=0)
    assert context.sample_batch(logits, [no_topk], uniforms).status == FG_ERR_ARGUMENT
    assert context.sample_batch(logits, [cfg], None).status == FG_ERR_ARGUMENT
    assert context.sample_batch(logits, [cfg, cfg, cfg], uniforms).status == FG_ERR_ARGUMENT
    assert context.sample_batch(logits, [cfg], uniforms).status == FG_OK


def test_repeatable_and_canaries(context):
    """Two runs give identical bits, and nothing is written outside the outputs."""
    w = synth.config3(rows=16, history=1024).to("cuda")
    rows = w.rows
    guard = 0x5A5A5A5A
    pads = [torch.full((rows + 64,), guard, dtype=torch.int32, device="cuda") for _ in range(3)]
    outs = (pads[0][32:32 + rows], pads[1][32:32 + rows].view(torch.float32), pads[2][32:32 + rows])
    first = context.sample_batch(w.logits, w.configs, w.uniforms, w.history_tokens, w.history_offsets,
                                 w.history_max, out=outs)
    snapshot = [t.clone() for t in outs]
    second = context.sample_batch(w.logits, w.configs, w.uniforms, w.history_tokens,
                                  w.history_offsets, w.history_max, out=outs)
    assert first.status == FG_OK and second.status == FG_OK
    for a, b in zip(snapshot, outs):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    for pad in pads:
        assert bool((pad[:32] == guard).all()) and bool((pad[32 + rows:] == guard).all())


def test_host_entry_matches_device_entry(context):
    w = synth.config2(rows=8, vocab=20_000)
    expected = run_oracle(w)
    result = context.sample_batch_host(w.logits, w.configs, w.uniforms, w.history_tokens,
                                       w.history_offsets, w.history_max)
    assert_rows_equal(result, expected, "host entry")
