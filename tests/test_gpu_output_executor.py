"""The stateful executor (fg_cuda_output_*): sessions decode step after step, every step's
tokens are checked against the CPU oracle run on the histories as they stand, and the
histories grow exactly as the reference's executor grows them (src/output.c:742, 752: a
token joins its session's history when it was picked with penalties active)."""
import numpy as np
import pytest
import torch

from flash_gordon_b200 import FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_ERR_MISMATCH, FG_OK, SamplerConfig, synth
from flash_gordon_b200.api import OutputExecutor
from helpers import as_u32, run_oracle

pytestmark = pytest.mark.gpu


def oracle_step(logits, configs, uniforms, histories):
    tokens = torch.tensor([t for h in histories for t in h], dtype=torch.int32)
    offsets = torch.tensor(np.cumsum([0] + [len(h) for h in histories]), dtype=torch.int64)
    longest = max([len(h) for h in histories] + [1])
    w = synth.Workload("step", logits, configs, uniforms, tokens, offsets, longest)
    return run_oracle(w)


@pytest.mark.parametrize("vocab", [151_936, 9_001])  # (9,001 fp32 rows are not 16-byte aligned: the other kernel)
def test_sixty_four_steps_of_eight_sessions(context, vocab):
    rows, steps, slots = 8, 64, 11
    g = torch.Generator().manual_seed(vocab)
    configs = [SamplerConfig.make(0.0 if r == 3 else 0.8 + 0.05 * r, 0.9, 1 + 7 * r, presence=0.3 * (r % 3),
                                  frequency=0.25 * (r % 2), repetition=1.0 + 0.05 * (r % 4))
               for r in range(rows)]
    configs[5] = SamplerConfig.make(1.0, 0.95, 20)                  # no penalties: history never grows
    configs[6] = SamplerConfig.make(0.9, 0.9, 30, presence=-0.5)     # can raise a logit: token lists, other kernel
    session_of = [9, 2, 7, 0, 4, 1, 10, 3]
    executor = OutputExecutor(context, vocab, slots, 512)
    histories = {s: [] for s in range(slots)}
    prompts = {9: torch.randint(0, vocab, (300,), generator=g).tolist(), 2: [5, 5, 5, 6], 4: [vocab - 1] * 40}
    for slot, prompt in prompts.items():
        executor.set_session(slot)
        assert executor.history_reset(prompt) == FG_OK
        histories[slot] = list(prompt)
    base = torch.randn(rows, vocab, generator=g) * 2.0
    for step in range(steps):
        # logits that favour what was picked before, so that penalised ids keep competing
        logits = base + 0.3 * torch.randn(rows, vocab, generator=g)
        for r in range(rows):
            recent = histories[session_of[r]][-6:]
            if recent:
                logits[r, recent] += 2.5
        uniforms = torch.rand(rows, generator=g)
        want = oracle_step(logits, configs, uniforms, [histories[s] for s in session_of])
        got = executor.sample_sessions(logits.cuda(), configs, uniforms.cuda(), session_of)
        assert got.status == want[0], (step, got.message)
        assert np.array_equal(as_u32(got.row_status), want[3]), step
        assert np.array_equal(as_u32(got.tokens), want[1]), step
        assert np.array_equal(got.token_logits.cpu().numpy().view(np.uint32), want[2].view(np.uint32)), step
        for r in range(rows):
            active = (configs[r].presence_penalty != 0 or configs[r].frequency_penalty != 0
                      or configs[r].repetition_penalty != 1)
            if active and want[3][r] == FG_OK:
                histories[session_of[r]].append(int(want[1][r]))
    for slot in range(slots):
        assert executor.history_length(slot) == len(histories[slot]), slot
    assert executor.history_length(1) == 0  # session of the unpenalised row
    executor.close()


def test_one_row_calls_follow_the_reference_s_executor(context):
    vocab = 30_000
    executor = OutputExecutor(context, vocab, 2, 64)
    g = torch.Generator().manual_seed(3)
    row = torch.randn(vocab, generator=g) * 3.0
    row[123], row[77] = 30.0, 29.5
    logits = context.tensor_from(row)
    # greedy: argmax of the raw logits, history untouched (src/output.c:560-599)
    assert executor.greedy(logits)[:2] == (FG_OK, 123)
    assert executor.history_length(0) == 0
    # penalised greedy: the pick joins the history, so the next step moves on (src/output.c:727-744)
    cfg = SamplerConfig.make(0.0, 1.0, 1, presence=1.0)
    assert executor.sample(logits, cfg, 0.0)[:2] == (FG_OK, 123)
    assert executor.history_length(0) == 1
    status, token, value, _ = executor.sample(logits, cfg, 0.0)
    assert (status, token) == (FG_OK, 77) and value == np.float32(29.5)
    status, token, value, _ = executor.sample(logits, cfg, 0.0)   # both seen now: 30 - 1 beats 29.5 - 1
    assert (status, token) == (FG_OK, 123) and value == np.float32(29.0)
    # the other session has its own history
    executor.set_session(1)
    assert executor.session == 1 and executor.sample(logits, cfg, 0.0)[:2] == (FG_OK, 123)
    executor.set_session(7)  # outside the table: ignored, as in the reference
    assert executor.session == 1
    # history_reset replaces, history_increment adds; a token outside the vocabulary is refused
    assert executor.history_reset([123, 123, 77]) == FG_OK and executor.history_length(1) == 3
    frequency = SamplerConfig.make(0.0, 1.0, 1, frequency=1.0)
    status, token, value, _ = executor.sample(logits, frequency, 0.0)   # 30 - 2 = 28 < 29.5 - 1 = 28.5
    assert (status, token) == (FG_OK, 77) and value == np.float32(28.5)
    assert executor.history_increment(vocab) == FG_ERR_FORMAT
    assert executor.history_reset([1, vocab, 2]) == FG_ERR_FORMAT and executor.history_length(1) == 4
    assert executor.history_reset(list(range(65))) == FG_ERR_ARGUMENT   # longer than the capacity
    # a NaN wins the argmax order and is rejected (src/output.c:593)
    row[5] = float("nan")
    bad = context.tensor_from(row)
    assert executor.greedy(bad)[0] == FG_ERR_MISMATCH
    assert executor.sample(bad, cfg, 0.0)[0] == FG_ERR_FORMAT
    executor.close()
