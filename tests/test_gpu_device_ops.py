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


# ---- sorted top-512 per tile (fg_vk_topk_reduce) and router top-k: the kernels next door ----

def test_topk_reduce_chunked_sizes(context, port):
    """tests/test_fg_vk.c:1231-1272 of the reference restated: 39 sizes from 1 to 8200 with zeros,
    NaN and both infinities sprinkled in; every output bit-equal to the oracle's."""
    from test_cpu_oracle import reduce_chunked_inputs
    everything = reduce_chunked_inputs(8200)
    ids = np.arange(8200, dtype=np.uint32)
    for count in (1, 2, 7, 63, 64, 65, 100, 127, 128, 129, 192, 320, 448, 511, 512, 513, 576, 640, 704, 768, 1000,
                  1024, 1088, 1090, 1091, 1152, 1216, 2048, 2112, 3000, 4032, 4096, 4097, 4160, 4224, 5000, 8000,
                  8192, 8200):
        want_scores, want_ids = oracle.topk_reduce(port, everything[:count], ids[:count])
        groups = (count + 4095) // 4096
        out_scores, out_ids = context.tensor(groups * 512 * 4), context.tensor(groups * 512 * 4)
        in_scores = context.tensor_from(torch.from_numpy(everything[:count].copy()))
        for explicit in (True, False):
            in_ids = context.tensor_from(torch.from_numpy(ids[:count].view(np.int32).copy())) if explicit else None
            status, produced = context.topk_reduce(out_scores, out_ids, in_scores, in_ids, count)
            assert status == FG_OK and produced == len(want_scores), count
            got_scores = np.frombuffer(out_scores.read(produced * 4), dtype=np.uint32)
            got_ids = np.frombuffer(out_ids.read(produced * 4), dtype=np.uint32)
            assert np.array_equal(got_ids, want_ids), count
            assert np.array_equal(got_scores, want_scores.view(np.uint32)), count


def test_topk_reduce_vocabulary_cascade_puts_the_nan_first(context):
    """tests/test_fg_vk.c:1202 of the reference: the cascade over 248,320 scores; a NaN sorts
    first, then the three spikes."""
    scores = -np.arange(REFERENCE_VOCAB, dtype=np.float32)
    scores[12345], scores[23456], scores[34567], scores[45678] = 100.0, 99.0, 98.0, np.nan
    first = (REFERENCE_VOCAB + 4095) // 4096 * 512
    source_scores = context.tensor_from(torch.from_numpy(scores))
    source_ids = None
    scratch = [(context.tensor(first * 4), context.tensor(first * 4)) for _ in range(2)]
    count, slot = REFERENCE_VOCAB, 0
    while count > 512:
        status, count = context.topk_reduce(scratch[slot][0], scratch[slot][1], source_scores, source_ids, count)
        assert status == FG_OK
        source_scores, source_ids = scratch[slot]
        slot ^= 1
    assert count == 512
    top_scores = np.frombuffer(source_scores.read(16), dtype=np.float32)
    top_ids = np.frombuffer(source_ids.read(16), dtype=np.uint32)
    assert top_ids.tolist() == [45678, 12345, 23456, 34567] and not np.isfinite(top_scores[0])
    assert top_scores[1:].tolist() == [100.0, 99.0, 98.0]
    assert context.topk_reduce(scratch[0][0], scratch[0][1], source_scores, source_ids, 0)[0] == FG_ERR_ARGUMENT


def test_router_topk_matches_the_reference_s_cpu_statement(context, port):
    """fg_q38_router_topk (src/q38_math.c:48-64): ids bit-exact, gate weights within 1e-6
    relative (exp() comes from another library here)."""
    rng = np.random.default_rng(5)
    experts, tokens, k = 512, 37, 10
    logits = (rng.standard_normal((tokens, experts)) * 2.0).astype(np.float32)
    logits[3, 100:110] = logits[3, 5]       # ties: smaller ids first
    logits[9, :] = 0.25                      # all equal
    logits[11, 7] = -np.inf                  # a -inf expert simply never wins
    device_logits = context.tensor_from(torch.from_numpy(logits))
    selected, gates = context.tensor(tokens * k * 4), context.tensor(tokens * k * 4)
    status, message = context.router_topk(selected, gates, device_logits, experts, tokens, k)
    assert status == FG_OK, message
    got_ids = np.frombuffer(selected.read(), dtype=np.uint32).reshape(tokens, k)
    got_weights = np.frombuffer(gates.read(), dtype=np.float32).reshape(tokens, k)
    for t in range(tokens):
        want_status, want_ids, want_weights = oracle.router_topk(port, logits[t], k)
        assert want_status == FG_OK and np.array_equal(got_ids[t], want_ids), t
        np.testing.assert_allclose(got_weights[t], want_weights, rtol=1e-6, atol=0)
    # a NaN or +Inf logit: that token's outputs are blanked and the call says which token
    logits[20, 3] = np.nan
    status, message = context.router_topk(selected, gates, context.tensor_from(torch.from_numpy(logits)),
                                          experts, tokens, k)
    assert status == FG_ERR_FORMAT and "token 20" in message
    got_ids = np.frombuffer(selected.read(), dtype=np.uint32).reshape(tokens, k)
    assert (got_ids[20] == 0xFFFFFFFF).all() and (got_ids[19] != 0xFFFFFFFF).all()
    assert context.router_topk(selected, gates, device_logits, experts, tokens, 33)[0] == FG_ERR_ARGUMENT
