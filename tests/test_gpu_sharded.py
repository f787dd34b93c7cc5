"""Vocabulary-sharded sampling on one GPU: the shards are run one after another
through fg_cuda_shard_topk, stacked the way an all-gather would leave them and
merged by fg_cuda_merge_select.  The result must equal the CPU oracle's sharded
path and the unsharded path on the same rows."""
import numpy as np
import pytest
import torch

import oracle
from flash_gordon_b200 import FG_ERR_ARGUMENT, FG_ERR_MISMATCH, FG_OK, SamplerConfig, synth
from flash_gordon_b200.dist import shard_span
from helpers import (as_u32, assert_candidates_close, assert_rows_equal, logits_to_numpy, oracle_kind,
                     random_workload, run_oracle)

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["ring_if_possible", "registers"], autouse=True)
def kernel_path(context, request):
    context.set_path(3 if request.param == "ring_if_possible" else 1)
    yield request.param
    context.set_path(0)


def run_sharded(context, w, shards, k_shard, debug=False):
    wd = w.to("cuda")
    rows, vocab = wd.rows, wd.vocab
    scores, ids, spans = [], [], []
    for s in range(shards):
        first, width = shard_span(vocab, shards, s)
        part = wd.logits[:, first:first + width].contiguous()
        sc, idx, row_status, status = context.shard_topk(part, wd.configs, first, vocab, k_shard,
                                                         wd.history_tokens, wd.history_offsets,
                                                         wd.history_max)
        assert status == FG_OK
        scores.append(sc)
        ids.append(idx)
        spans.append((first, width))
    all_scores, all_ids = torch.stack(scores).contiguous(), torch.stack(ids).contiguous()
    result = context.merge_select(all_scores, all_ids, rows, shards, k_shard, [s[0] for s in spans],
                                  [s[1] for s in spans], wd.configs, wd.uniforms, debug=debug)
    return result, all_scores, all_ids, spans


def oracle_sharded(w, shards, k_shard):
    lib = oracle.load(oracle_kind())
    logits = logits_to_numpy(w.logits)
    tokens = offsets = None
    if w.history_tokens is not None:
        tokens = w.history_tokens.numpy().view(np.uint32)
        offsets = w.history_offsets.numpy().view(np.uint64)
    parts, spans = [], []
    for s in range(shards):
        first, width = shard_span(w.vocab, shards, s)
        parts.append(oracle.shard_topk(lib, np.ascontiguousarray(logits[:, first:first + width]), w.configs,
                                       first, w.vocab, k_shard, tokens, offsets))
        spans.append((first, width))
    scores = np.stack([p[1] for p in parts])
    ids = np.stack([p[2] for p in parts])
    merged = oracle.merge_select(lib, scores, ids, [s[0] for s in spans], [s[1] for s in spans], w.configs,
                                 w.uniforms.numpy(), want_candidates=True)
    return merged, scores, ids


def test_config4_bf16_eight_shards(context):
    w = synth.config4(rows=24)
    result, got_scores, got_ids, _ = run_sharded(context, w, 8, 64, debug=True)
    merged, want_scores, want_ids = oracle_sharded(w, 8, 64)
    assert np.array_equal(as_u32(got_ids), want_ids)
    assert np.array_equal(got_scores.cpu().numpy().view(np.uint32), want_scores.view(np.uint32))
    assert_rows_equal(result, merged, "config4 sharded vs sharded oracle")
    assert_candidates_close(result, merged, 1e-5, "config4 sharded")
    assert_rows_equal(result, run_oracle(w), "config4 sharded vs unsharded oracle")


def test_sharded_with_penalties_and_ties(context):
    cfg = SamplerConfig.make(temperature=0.9, top_p=0.85, top_k=40, presence=0.6, frequency=0.3,
                             repetition=1.15)
    w = random_workload(6, 10_007, 700, [cfg], 17, quantize=0.5, specials=4)
    for shards, k_shard in [(2, 40), (4, 64), (7, 50)]:
        result, _, _, _ = run_sharded(context, w, shards, k_shard, debug=True)
        merged, _, _ = oracle_sharded(w, shards, k_shard)
        assert_rows_equal(result, merged, f"shards={shards}")
        assert_candidates_close(result, merged, 1e-5, f"shards={shards}")
        assert_rows_equal(result, run_oracle(w), f"shards={shards} vs unsharded")


def test_sharded_greedy_fold(context):
    cfg = SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1)
    w = random_workload(5, 8192, 0, [cfg], 23, quantize=1.0)
    result, _, _, _ = run_sharded(context, w, 4, 8)
    merged, _, _ = oracle_sharded(w, 4, 8)
    assert_rows_equal(result, merged, "greedy sharded")
    assert_rows_equal(result, run_oracle(w), "greedy sharded vs unsharded")


def test_sharded_greedy_rows_with_nan_or_inf_fail_like_unsharded_ones(context):
    """A NaN/Inf anywhere in a greedy row wins the argmax order and is then rejected
    (src/runtime.c:2458-2463 for the split head, src/output.c:593 unsharded): the shard that
    holds it must hand it on, whichever kernel samples the shard."""
    cfg = SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1)
    w = random_workload(9, 8192, 0, [cfg], 29, quantize=1.0, specials=3)
    w.logits[4] = torch.round(torch.randn(8192) * 3.0)  # one clean row among them
    unsharded = run_oracle(w)
    assert (unsharded[3] == FG_ERR_MISMATCH).sum() >= 4 and unsharded[3][4] == FG_OK
    result, _, _, _ = run_sharded(context, w, 4, 8)  # (the fixture runs both kernels)
    merged, _, _ = oracle_sharded(w, 4, 8)
    assert_rows_equal(result, merged, "greedy sharded with specials")
    assert np.array_equal(as_u32(result.row_status), unsharded[3]), "sharded status != unsharded status"
    bad = unsharded[3] != FG_OK
    assert np.array_equal(as_u32(result.tokens)[bad], unsharded[1][bad]), "the rejected finalist's id"


def test_span_check_and_argument_errors(context):
    w = synth.config4(rows=4, vocab=8000)
    result, scores, ids, spans = run_sharded(context, w, 4, 64)
    assert result.status == FG_OK
    ids[1, 2, 0] = 5  # an id outside shard 1's span (src/runtime.c:2451-2456 of the reference)
    wd = w.to("cuda")
    bad = context.merge_select(scores, ids, 4, 4, 64, [s[0] for s in spans], [s[1] for s in spans],
                               wd.configs, wd.uniforms)
    assert bad.status == FG_ERR_MISMATCH
    assert as_u32(bad.row_status).tolist() == [0, 0, FG_ERR_MISMATCH, 0]
    # the union of shard lists only holds the global top-k up to k_shard
    small = context.merge_select(scores[:, :, :16].contiguous(), ids[:, :, :16].contiguous(), 4, 4, 16,
                                 [s[0] for s in spans], [s[1] for s in spans], wd.configs, wd.uniforms)
    assert small.status == FG_ERR_ARGUMENT
    part = wd.logits[:, :2000].contiguous()
    assert context.shard_topk(part, wd.configs, 7000, 8000, 64)[3] == FG_ERR_ARGUMENT  # span past the end
    assert context.shard_topk(part, wd.configs, 0, 8000, 65)[3] == FG_ERR_ARGUMENT
