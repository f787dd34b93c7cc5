"""Device operators against the behaviour the reference's own Vulkan tests pin
(tests/test_fg_vk.c of the reference: output_argmax at line 1340,
generation_topk_selector at 1274-1338) and against the CPU oracle."""
import math

import numpy as np
import pytest
import torch

import oracle
from flash_gordon_b200 import FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_OK

pytestmark = pytest.mark.gpu

NAN = float("nan")
REFERENCE_VOCAB = 248_320


def _floats(raw: bytes) -> np.ndarray:
    return np.frombuffer(raw, dtype=np.float32)


def _words(raw: bytes) -> np.ndarray:
    return np.frombuffer(raw, dtype=np.uint32)


def _argmax_cascade(context, scores: np.ndarray, ids: np.ndarray | None):
    """The loop of src/output.c:565 of the reference: reduce until one finalist."""
    count = len(scores)
    groups = (count + 4095) // 4096
    source_scores = context.tensor_from(torch.from_numpy(scores))
    source_ids = None if ids is None else context.tensor_from(torch.from_numpy(ids.view(np.int32)))
    scratch = [(context.tensor(groups * 4), context.tensor(groups * 4)) for _ in range(2)]
    slot = 0
    context.begin()
    while count > 1:
        status, produced = context.argmax_reduce(scratch[slot][0], scratch[slot][1], source_scores,
                                                 source_ids, count)
        assert status == FG_OK
        source_scores, source_ids = scratch[slot]
        count = produced
        slot ^= 1
    context.end()
    return _floats(source_scores.read(4))[0], _words(source_ids.read(4))[0]


@pytest.mark.parametrize("explicit_ids", [True, False])
def test_output_argmax_tie_then_nan(context, explicit_ids):
    scores = -np.arange(REFERENCE_VOCAB, dtype=np.float32)
    ids = np.arange(REFERENCE_VOCAB, dtype=np.uint32) if explicit_ids else None
    scores[12345] = 100.0
    scores[23456] = 100.0
    value, token = _argmax_cascade(context, scores, ids)
    assert token == 12345 and value == 100.0          # tie -> smaller id
    scores[45678] = NAN
    value, token = _argmax_cascade(context, scores, ids)
    assert token == 45678 and not math.isfinite(value)  # a NaN wins the argmax order


def test_generation_topk_selector(context):
    scores = np.array([1, 9, 7, 9, 3, 8, 2, 7, 6, 5, 4, 0, -1, -2, -3, -4, -5, -6, NAN], dtype=np.float32)
    ids = np.arange(19, dtype=np.uint32)
    t_scores = context.tensor_from(torch.from_numpy(scores))
    t_ids = context.tensor_from(torch.from_numpy(ids.view(np.int32)))
    out_scores, out_ids = context.tensor(16), context.tensor(16)
    assert context.topk_select(out_scores, out_ids, t_scores, t_ids, 19, 0)[0] == FG_ERR_ARGUMENT
    assert context.topk_select(out_scores, out_ids, t_scores, t_ids, 19, 65)[0] == FG_ERR_ARGUMENT

    def run(k, source=t_scores):
        context.begin()
        status, produced = context.topk_select(out_scores, out_ids, source, t_ids, 19, k)
        context.end()
        assert status == FG_OK and produced == k
        return _floats(out_scores.read(4 * k)).copy(), _words(out_ids.read(4 * k)).copy()

    got_scores, got_ids = run(4)
    assert sorted(got_ids.tolist()) == [1, 2, 3, 5]
    assert all(got_scores[i] == scores[got_ids[i]] for i in range(4))
    again_scores, again_ids = run(4)
    assert np.array_equal(got_ids, again_ids) and np.array_equal(got_scores, again_scores)
    one_score, one_id = run(1)
    assert one_id[0] == 1 and one_score[0] == 9.0        # ids 1 and 3 tie at 9: smaller id
    shortage = np.full(19, NAN, dtype=np.float32)
    shortage[1], shortage[3] = 9.0, 8.0
    short_scores, short_ids = run(4, context.tensor_from(torch.from_numpy(shortage)))
    assert short_ids[0] != 0xFFFFFFFF and short_ids[1] != 0xFFFFFFFF
    assert short_ids[2] == 0xFFFFFFFF and not math.isfinite(short_scores[2])


def test_topk_cascade_matches_oracle(context, port):
    """The cascade of src/output.c:681-700 of the reference, pass by pass."""
    rng = np.random.default_rng(3)
    for count, k in [(1, 1), (1023, 5), (1024, 64), (1025, 20), (5000, 50), (151_936, 50)]:
        scores = np.round(rng.normal(0, 3, count), 1).astype(np.float32)
        scores[rng.integers(0, count, 5)] = np.nan
        scores[rng.integers(0, count, 2)] = np.inf
        cur_scores, cur_ids, n = scores, None, count
        t_scores = context.tensor_from(torch.from_numpy(scores))
        t_ids = None
        while True:
            want_scores, want_ids = oracle.topk_select(port, cur_scores[:n], cur_ids if cur_ids is None else cur_ids[:n], k)
            groups = (n + 1023) // 1024
            out_scores, out_ids = context.tensor(groups * k * 4), context.tensor(groups * k * 4)
            status, produced = context.topk_select(out_scores, out_ids, t_scores, t_ids, n, k)
            assert status == FG_OK and produced == groups * k
            got_scores = _floats(out_scores.read()).copy()
            got_ids = _words(out_ids.read()).copy()
            assert np.array_equal(got_ids, want_ids), f"count={count} k={k} n={n}"
            assert np.array_equal(got_scores.view(np.uint32), want_scores.view(np.uint32))
            cur_scores, cur_ids, n = want_scores, want_ids, produced
            t_scores, t_ids = out_scores, out_ids
            if produced <= k:
                break


def test_argmax_reduce_matches_oracle(context, port):
    rng = np.random.default_rng(8)
    for count in [1, 2, 4095, 4096, 4097, 100_000]:
        scores = np.round(rng.normal(0, 2, count)).astype(np.float32)
        if count > 10:
            scores[count // 2] = -np.inf if count % 2 else np.nan
        ids = rng.permutation(count).astype(np.uint32)
        want_scores, want_ids = oracle.argmax_reduce(port, scores, ids)
        groups = len(want_ids)
        out_scores, out_ids = context.tensor(groups * 4), context.tensor(groups * 4)
        status, produced = context.argmax_reduce(
            out_scores, out_ids, context.tensor_from(torch.from_numpy(scores)),
            context.tensor_from(torch.from_numpy(ids.view(np.int32))), count)
        assert status == FG_OK and produced == groups
        got_ids = _words(out_ids.read())
        got_scores = _floats(out_scores.read())
        assert np.array_equal(got_ids, want_ids)
        same = (got_scores.view(np.uint32) == want_scores.view(np.uint32)) | (np.isnan(got_scores) & np.isnan(want_scores))
        assert same.all()


def test_apply_penalties_operator(context, port):
    rng = np.random.default_rng(21)
    values = 151_936
    logits = rng.normal(0, 3, values).astype(np.float32)
    counts = (rng.random(values) < 0.03).astype(np.uint32) * rng.integers(1, 9, values).astype(np.uint32)
    ids = np.arange(values, dtype=np.uint32)
    t_logits = context.tensor_from(torch.from_numpy(logits))
    t_counts = context.tensor_from(torch.from_numpy(counts.view(np.int32)))
    assert context.apply_penalties(t_logits, t_counts, 0, 0.1, 0.1, 1.0) == FG_ERR_ARGUMENT
    assert context.apply_penalties(t_logits, t_counts, values, 0.1, 0.1, 0.0) == FG_ERR_ARGUMENT
    assert context.apply_penalties(t_logits, t_counts, values, NAN, 0.1, 1.0) == FG_ERR_ARGUMENT
    assert context.apply_penalties(t_logits, t_counts, values + 1, 0.1, 0.1, 1.0) == FG_ERR_ARGUMENT
    from flash_gordon_b200 import SamplerConfig
    cfg = SamplerConfig.make(presence=0.7, frequency=0.3, repetition=1.2)
    want = oracle.apply_penalties(port, logits, ids, counts, cfg)
    assert context.apply_penalties(t_logits, t_counts, values, 0.7, 0.3, 1.2) == FG_OK
    got = _floats(t_logits.read())
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # views: penalise only a window (the executor passes a per-session slice of its table)
    window = context.view(t_logits, 4096 * 4, 1000 * 4)
    window_counts = context.view(t_counts, 4096 * 4, 1000 * 4)
    assert context.apply_penalties(window, window_counts, 1001, 0.7, 0.3, 1.2) == FG_ERR_ARGUMENT
    assert context.apply_penalties(window, window_counts, 1000, 0.0, 0.0, 1.0) == FG_OK


def test_history_table(context, port):
    vocab = 1000
    counts = context.tensor(vocab * 4)
    history = [3, 3, 7, 999, 3, 0]
    assert context.history_reset(counts, vocab, history) == FG_OK
    status, want = oracle.history_counts(port, vocab, history)
    assert status == FG_OK
    assert np.array_equal(_words(counts.read()), want)
    assert context.history_increment(counts, vocab, 7) == FG_OK
    assert context.history_increment(counts, vocab, 1000) == FG_ERR_ARGUMENT
    context.begin(); context.end()
    want[7] += 1
    assert np.array_equal(_words(counts.read()), want)
    assert context.history_reset(counts, vocab, [1, 2, 1000]) == FG_ERR_FORMAT
    assert context.history_reset(counts, vocab, []) == FG_OK
    assert not _words(counts.read()).any()
