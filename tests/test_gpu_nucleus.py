"""Rows sampled without a top-k cut (top_k == 0 under FG_CUDA_SAMPLE_ALLOW_NO_TOPK):
top-p over the whole vocabulary.  The reference's select stops at 64 candidates, so
the oracle here is the repository's generalisation of it (fgo_select_general): same
order, same fp64 formulas, any number of candidates.  The GPU accumulates masses as
2^-40 fixed point instead of left-to-right doubles; ids agree unless top_p or the
draw lies within ~1e-11 of an edge of the CDF, which these seeds do not hit."""
import numpy as np
import pytest
import torch

from flash_gordon_b200 import FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_OK, SamplerConfig, synth
from helpers import as_u32, assert_rows_equal, random_workload, run_gpu, run_oracle

pytestmark = pytest.mark.gpu


def test_config5_reduced_rows(context):
    w = synth.config5(rows=6)
    expected = run_oracle(w)
    assert expected[0] == FG_OK
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "config5")
    sizes = as_u32(result.debug["count"])
    assert (sizes > 20_000).all(), sizes  # near-flat logits: the nucleus spans tens of thousands


def test_config5_a_wave_of_rows_with_their_edge_margins(context, capsys):
    """More rows than the GPU has SMs (the kernel is one CTA per SM), full vocabulary, the
    benchmark's 32,768-token histories.  The oracle also reports, per row, how far top_p and
    the draw lie from the nearest edge of the cumulative distribution (in units of the total
    mass): ids can only differ where that is within the rounding of a sum -- about 1e-12 for
    the 2^-40 fixed point here, 1e-16 per term for the oracle's doubles -- so the smallest
    margin of the run is printed and must be far above it."""
    w = synth.config5(rows=160)
    expected = run_oracle(w, want_candidates=True)
    assert expected[0] == FG_OK
    margins = np.array([c.edge_margin for c in expected[4]])
    sizes = np.array([c.nucleus for c in expected[4]])
    with capsys.disabled():
        print(f"\nconfig5, {w.rows} rows: smallest edge margin {margins.min():.3e} (median {np.median(margins):.3e}), "
              f"nucleus {sizes.min()}..{sizes.max()} tokens")
    assert margins.min() > 1e-10
    result = run_gpu(context, w, debug=True)
    assert_rows_equal(result, expected, "config5, 160 rows")
    assert np.array_equal(as_u32(result.debug["count"]), sizes)


def test_on_an_edge_the_pick_is_the_oracle_s_or_its_neighbour(context):
    """3000 equal logits and top_p = 0.75: the cut falls exactly on an edge of the cumulative
    distribution (2250 / 3000).  The oracle's running sum of 1/3000 in doubles and an exact
    sum may part ways there by one candidate, and that is all they may part by."""
    vocab = 3000
    logits = torch.full((3, vocab), 0.5)
    cfg = SamplerConfig.make(temperature=1.0, top_p=0.75, top_k=0)
    uniforms = torch.tensor([0.99999994, 0.5, 0.0])
    w = synth.Workload("edge", logits, [cfg], uniforms, None, None, 0, allow_no_topk=True)
    expected = run_oracle(w, want_candidates=True)
    assert min(c.edge_margin for c in expected[4]) < 1e-12   # it is on the edge
    result = run_gpu(context, w)
    assert result.status == FG_OK
    got = as_u32(result.tokens).astype(np.int64)
    assert (np.abs(got - expected[1].astype(np.int64)) <= 1).all(), (got, expected[1])
    assert got[2] == 0 and abs(int(got[0]) - 2249) <= 1


@pytest.mark.parametrize("temperature,top_p", [(1.0, 0.9), (0.7, 0.5), (1.2, 0.99), (2.0, 1.0), (0.3, 0.05)])
def test_random_rows_with_ties_and_specials(context, temperature, top_p):
    cfg = SamplerConfig.make(temperature=temperature, top_p=top_p, top_k=0, presence=0.4, frequency=0.3,
                             repetition=1.2)
    for vocab, rows, quantize in [(5000, 6, 0.25), (40_000, 4, 0.0), (151_936, 2, 0.5), (33, 3, 1.0), (1, 2, 0.0)]:
        w = random_workload(rows, vocab, 300, [cfg], 500 + vocab, quantize=quantize, specials=min(3, vocab - 1))
        w.allow_no_topk = True
        expected = run_oracle(w)
        assert_rows_equal(run_gpu(context, w), expected, f"V={vocab} T={temperature} p={top_p}")


def test_extreme_draws_and_flat_rows(context):
    vocab = 3000
    logits = torch.cat([torch.full((2, vocab), 0.5), torch.randn(2, vocab)], 0)
    # 0.7501, not 0.75: with 3000 equal weights 0.75 is itself an edge of the CDF, where the
    # reference's running sum of 1/3000 and exact arithmetic may legitimately part ways
    cfg = SamplerConfig.make(temperature=1.0, top_p=0.7501, top_k=0)
    uniforms = torch.tensor([0.0, 0.99999994, 0.0, 0.99999994])
    w = synth.Workload("flat", logits, [cfg], uniforms, None, None, 0, allow_no_topk=True)
    expected = run_oracle(w)
    assert expected[1][0] == 0            # all equal: the draw 0 picks id 0 ...
    assert expected[1][1] == 2250         # ... and the largest draw the last id inside the nucleus
    assert_rows_equal(run_gpu(context, w), expected, "flat")


def test_mixed_batch_and_bf16(context):
    rows, vocab = 9, 20_000
    configs = []
    for r in range(rows):
        if r % 3 == 0:
            configs.append(SamplerConfig.make(temperature=0.9, top_p=0.9, top_k=0, frequency=0.2))
        elif r % 3 == 1:
            configs.append(SamplerConfig.make(temperature=0.8, top_p=0.9, top_k=30, presence=0.5))
        else:
            configs.append(SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1, repetition=1.1))
    for dtype in (torch.float32, torch.bfloat16):
        w = random_workload(rows, vocab, 500, configs, 77, dtype=dtype)
        w.allow_no_topk = True
        assert_rows_equal(run_gpu(context, w), run_oracle(w), f"mixed {dtype}")


def test_errors(context):
    vocab = 500
    logits = torch.randn(2, vocab)
    logits[1, :] = float("nan")
    cfg = SamplerConfig.make(temperature=1.0, top_p=0.9, top_k=0)
    w = synth.Workload("nan", logits, [cfg], torch.tensor([0.5, 0.5]), None, None, 0, allow_no_topk=True)
    expected = run_oracle(w)
    assert list(expected[3]) == [FG_OK, FG_ERR_FORMAT]
    assert_rows_equal(run_gpu(context, w), expected, "nan row")
    # without the flag top_k == 0 stays invalid, as in the reference's validate
    wd = w.to("cuda")
    assert context.sample_batch(wd.logits, wd.configs, wd.uniforms).status == FG_ERR_ARGUMENT
