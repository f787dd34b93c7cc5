"""Edge cases of the persistent ring kernel (pinned with path = ring), against the oracle:
lists that overflow, histories that cover the best logits, many rows per CTA with both
pairs of lists in use, rows the kernel must skip, bf16, shard mode, broken histories."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from flash_gordon_b200 import (FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_ERR_LIMIT, FG_OK, Context,
                               SamplerConfig, synth)
from helpers import (as_u32, assert_candidates_close, assert_rows_equal, oracle_kind, random_workload,
                     run_gpu, run_oracle)

pytestmark = pytest.mark.gpu

PATH_AUTO, PATH_RING = 0, 2
PROBABILITY_RTOL = 1e-5  # probabilities: fp64 on both sides, exp() from different libraries


@pytest.fixture(scope="module")
def context():
    ctx = Context(0)
    ctx.set_path(PATH_RING)
    yield ctx
    ctx.set_path(PATH_AUTO)


def csr(histories):
    tokens = torch.tensor([t for h in histories for t in h], dtype=torch.int32)
    offsets = torch.tensor(np.cumsum([0] + [len(h) for h in histories]), dtype=torch.int64)
    return tokens, offsets, max(len(h) for h in histories)


def test_history_covers_the_best_logits(context):
    """Every row's best several hundred logits are in its history with assorted counts, so
    hundreds of ids are put aside and the lists overflow more than once."""
    rows, vocab = 6, 40_000
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(rows, vocab, generator=g) * 2.0
    histories = []
    for r in range(rows):
        best = torch.topk(logits[r], 300 + 100 * r).indices.tolist()
        history = []
        for j, token in enumerate(best):
            history += [token] * (1 + (j * 7 + r) % 5)
        extra = torch.randint(0, vocab, (500,), generator=g).tolist()
        order = torch.randperm(len(history) + len(extra), generator=g).tolist()
        merged = history + extra
        histories.append([merged[i] for i in order])
    tokens, offsets, longest = csr(histories)
    for cfg in (SamplerConfig.make(1.0, 0.95, 64, presence=0.2, frequency=0.3, repetition=1.1),
                SamplerConfig.make(0.7, 0.9, 20, presence=1.5),
                SamplerConfig.make(0.0, 1.0, 1, frequency=0.4, repetition=1.3)):
        w = synth.Workload("covered", logits, [cfg], torch.linspace(0.01, 0.99, rows), tokens, offsets,
                           longest)
        expected = run_oracle(w, want_candidates=True)
        result = run_gpu(context, w, debug=True)
        assert_rows_equal(result, expected, "covered")
        assert_candidates_close(result, expected, PROBABILITY_RTOL, "covered")


def test_rising_rows_with_history(context):
    """Every later value is larger (each tile overflows the list) and a third of the ids are
    in the history."""
    rows, vocab = 3, 30_000
    base = torch.arange(vocab, dtype=torch.float32) * 0.01
    logits = torch.stack([base, base.flip(0), torch.full((vocab,), 2.5)])
    histories = [list(range(0, vocab, 3)), list(range(1, vocab, 3)) * 2, list(range(0, vocab, 5))]
    tokens, offsets, longest = csr(histories)
    cfg = SamplerConfig.make(1.0, 1.0, 64, presence=0.5, frequency=0.25, repetition=1.2)
    w = synth.Workload("rising", logits, [cfg], torch.tensor([0.0, 0.5, 0.999]), tokens, offsets, longest)
    expected = run_oracle(w, want_candidates=True)
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "rising")
    assert_candidates_close(result, expected, PROBABILITY_RTOL, "rising")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_many_rows_per_cta_mixed_rows(context, dtype):
    """More rows than CTAs several times over: both pairs of lists are in use, rows differ in
    mode, k and history length, and every seventh row has no top-k cut (it is another kernel's)."""
    rows, vocab = 1500, 8192 + 264
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(rows, vocab, generator=g) * 3.0).to(dtype)
    configs, histories = [], []
    for r in range(rows):
        if r % 7 == 3:
            configs.append(SamplerConfig.make(0.9, 0.8, 0, presence=0.1))
        elif r % 5 == 0:
            configs.append(SamplerConfig.make(0.0, 1.0, 1, repetition=1.0 + 0.05 * (r % 3)))
        else:
            configs.append(SamplerConfig.make(0.6 + 0.01 * (r % 40), 0.5 + 0.01 * (r % 50), 1 + r % 64,
                                              presence=0.1 * (r % 4), frequency=0.05 * (r % 6),
                                              repetition=1.0 + 0.02 * (r % 5)))
        length = (r * 37) % 900
        histories.append(torch.randint(0, vocab, (length,), generator=g).tolist())
    tokens, offsets, longest = csr(histories)
    w = synth.Workload("many", logits, configs, torch.rand(rows, generator=g), tokens, offsets, longest,
                       allow_no_topk=True)
    expected = run_oracle(w)
    result = run_gpu(context, w)
    assert_rows_equal(result, expected, f"many {dtype}")


def test_broken_histories_fail_their_rows_only(context):
    rows, vocab = 8, 12_000
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(rows, vocab, generator=g)
    histories = [torch.randint(0, vocab, (200,), generator=g).tolist() for _ in range(rows)]
    histories[2][17] = vocab          # outside the vocabulary
    histories[5][0] = 2**31 - 1
    tokens, offsets, longest = csr(histories)
    cfg = SamplerConfig.make(1.0, 0.9, 40, presence=0.3, frequency=0.1)
    w = synth.Workload("broken", logits, [cfg], torch.rand(rows, generator=g), tokens, offsets, longest)
    expected = run_oracle(w)
    result = run_gpu(context, w)
    assert_rows_equal(result, expected, "broken")
    status = as_u32(result.row_status)
    assert status[2] == FG_ERR_FORMAT and status[5] == FG_ERR_FORMAT
    assert (np.delete(status, [2, 5]) == FG_OK).all()
    # a history longer than the caller's bound fails the row with the limit status
    short = synth.Workload("bound", logits, [cfg], torch.rand(rows, generator=g), tokens, offsets, 150)
    result = run_gpu(context, short)
    assert (as_u32(result.row_status) == FG_ERR_LIMIT).all()


def test_shard_candidates_through_the_ring(context):
    """fg_cuda_shard_topk on a column span with a vocabulary offset: ids are global, history
    tokens outside the span do not count."""
    import oracle
    rows, span, first, total, k = 9, 18_992, 37_984, 151_936, 64
    g = torch.Generator().manual_seed(21)
    logits = (torch.randn(rows, span, generator=g) * 4.0).to(torch.bfloat16)
    histories = [torch.randint(0, total, (3000,), generator=g).tolist() for _ in range(rows)]
    tokens, offsets, longest = csr(histories)
    cfg = SamplerConfig.make(0.8, 0.9, 64, presence=0.4, frequency=0.2, repetition=1.05)
    lib = oracle.load(oracle_kind())
    _, want_scores, want_ids, want_status = oracle.shard_topk(
        lib, logits.view(torch.int16).numpy().view(np.uint16), [cfg], first, total, k,
        tokens.numpy().view(np.uint32), offsets.numpy().view(np.uint64))
    scores, ids, row_status, status = context.shard_topk(
        logits.cuda(), [cfg], first, total, k, tokens.cuda(), offsets.cuda(), longest)
    torch.cuda.synchronize()
    assert status == FG_OK
    assert np.array_equal(as_u32(row_status), want_status)
    assert np.array_equal(as_u32(ids), want_ids.reshape(rows, k))
    assert np.array_equal(scores.cpu().numpy().view(np.uint32),
                          want_scores.reshape(rows, k).view(np.uint32))


@pytest.mark.parametrize("deal", [1, 2])
def test_both_ways_of_dealing_out_rows(context, deal):
    """Whole rows round-robin and equal runs of tiles (rows shared between CTAs, parts merged
    by the last to finish) give the same bits, for more rows than CTAs and for fewer."""
    for rows, vocab, history in ((700, 9_000, 300), (40, 151_936, 2_000), (3, 151_936, 64)):
        cfgs = [SamplerConfig.make(0.0 if r % 6 == 0 else 0.9, 0.9, 1 + (r * 5) % 64, presence=0.2 * (r % 2),
                                   frequency=0.1 * (r % 4), repetition=1.0 + 0.03 * (r % 3))
                for r in range(rows)]
        w = random_workload(rows, vocab, history, cfgs, 1000 + rows, quantize=0.125, specials=1)
        expected = run_oracle(w)
        context.ring_controls(deal=deal)
        try:
            result = run_gpu(context, w)
        finally:
            context.ring_controls()
        assert_rows_equal(result, expected, f"deal {deal}, {rows} rows")


def test_a_wait_that_runs_out_fails_rows_not_the_gpu(context):
    """One tile of CTA 0 is never asked for, and the waits give up after a few thousand polls:
    the kernel comes back, the rows of that CTA end with FG_ERR_LIMIT, the others are sampled,
    and the next call on the same context works."""
    rows, vocab = 600, 20_000
    cfg = SamplerConfig.make(0.8, 0.9, 30, presence=0.2, frequency=0.1)
    w = random_workload(rows, vocab, 200, [cfg], 77)
    expected = run_oracle(w)
    context.ring_controls(deal=1, wait_polls=3000, withhold=(0, 5))
    try:
        result = run_gpu(context, w)
    finally:
        context.ring_controls()
    status = as_u32(result.row_status)
    assert result.status == FG_ERR_LIMIT and "wait" in result.message
    failed = np.nonzero(status == FG_ERR_LIMIT)[0]
    assert failed.size > 0 and set(np.unique(status)) == {FG_OK, FG_ERR_LIMIT}
    sms = context.sm_count
    assert all(r % sms == 0 for r in failed), "only CTA 0's rows (0, SMs, 2 SMs, ...) may fail"
    ok = status == FG_OK
    assert np.array_equal(as_u32(result.tokens)[ok], expected[1][ok])
    again = run_gpu(context, w)
    assert_rows_equal(again, expected, "after the timeout")


def test_ring_refuses_what_it_cannot_take(context):
    """Pinned to the ring, a batch with a penalty that can raise a logit, or with rows that do
    not start on 16 bytes, is an argument error (automatic choice falls back instead)."""
    rows, vocab = 4, 4100
    logits = torch.randn(rows, vocab).cuda()
    tokens = torch.randint(0, vocab, (rows * 10,), dtype=torch.int32).cuda()
    offsets = (torch.arange(rows + 1, dtype=torch.int64) * 10).cuda()
    uniforms = torch.rand(rows).cuda()
    raising = SamplerConfig.make(1.0, 0.9, 10, presence=-0.5)
    assert context.sample_batch(logits, [raising], uniforms, tokens, offsets, 10).status == FG_ERR_ARGUMENT
    odd = torch.randn(rows, vocab + 1).cuda()[:, 1:]  # rows start 4 bytes off, stride vocab + 1
    assert context.sample_batch(odd, [SamplerConfig.make(1.0, 0.9, 10)], uniforms, None, None,
                                0).status == FG_ERR_ARGUMENT
    context.set_path(PATH_AUTO)
    try:
        result = context.sample_batch(logits, [raising], uniforms, tokens, offsets, 10)
        torch.cuda.synchronize()
        assert result.status == FG_OK
    finally:
        context.set_path(PATH_RING)


def test_shapes_the_planner_treats_differently(context):
    """Through the automatic choice: a few rows of more than a million logits (dealt out in tiles
    and merged), the same with a history (its bitmap does not fit beside the ring: the other
    kernel), long rows in a small batch, many one-tile rows, a ragged one-tile row."""
    context.set_path(PATH_AUTO)
    try:
        for rows, vocab, history, cfg in (
                (3, 1_200_000, 0, SamplerConfig.make(0.9, 0.9, 50)),
                (2, 1_200_004, 0, SamplerConfig.make(0.0, 1.0, 1)),
                (5, 1_100_000, 300, SamplerConfig.make(0.8, 0.9, 40, presence=0.2, frequency=0.1)),
                (40, 300_000, 500, SamplerConfig.make(0.8, 0.9, 64, presence=0.2, frequency=0.1, repetition=1.1)),
                (600, 2048, 100, SamplerConfig.make(0.8, 0.9, 20, presence=0.2)),
                (7, 2052, 0, SamplerConfig.make(1.0, 0.95, 64))):
            w = random_workload(rows, vocab, history, [cfg], 4242 + rows, specials=1)
            assert_rows_equal(run_gpu(context, w), run_oracle(w), f"{rows} x {vocab}")
    finally:
        context.set_path(PATH_RING)

