"""The CPU oracle against what pins it: the reference's own known answers
(tests/test_sampler.c and the combine tests of tests/test_fg_vk.c:4021-4155 of
the reference, restated), the committed golden vectors that were generated from
the reference's objects, and — where oracle/_ref was built — the reference
objects themselves on random inputs."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLDEN = json.loads((Path(__file__).parent / "golden" / "sampler_golden.json").read_text())
KINDS = ["port"] + (["reference"] if oracle.available("reference") else [])


class Cfg:
    def __init__(self, temperature=1.0, top_p=0.95, top_k=20, presence=0.0, frequency=0.0,
                 repetition=1.0, min_p=0.0, seed=0x9E3779B97F4A7C15):
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.presence_penalty, self.frequency_penalty = presence, frequency
        self.repetition_penalty, self.min_p, self.seed = repetition, min_p, seed


def cfg_from_list(values) -> Cfg:
    values = [float(v) if i not in (2, 7) else int(float(v)) for i, v in enumerate(values)]
    return Cfg(*values)


def from_bits(words) -> np.ndarray:
    return np.array(words, dtype=np.uint32).view(np.float32)


def validate(lib, cfg) -> int:
    return lib.fg_sampler_config_validate(oracle.OracleConfig.of(cfg), oracle.OracleError())


@pytest.mark.parametrize("kind", KINDS)
def test_reference_sampler_known_answers(kind):
    """tests/test_sampler.c:10-54 of the reference, check for check."""
    lib = oracle.load(kind)
    cfg = oracle.OracleConfig()
    lib.fg_sampler_config_defaults(cfg)
    assert (cfg.temperature, cfg.top_k) == (1.0, 20) and abs(cfg.top_p - 0.95) < 1e-7
    assert validate(lib, cfg) == 0
    assert validate(lib, Cfg(presence=2.0, frequency=-2.0)) == 0
    for bad in (Cfg(presence=2.01), Cfg(presence=-2.01), Cfg(frequency=2.01), Cfg(frequency=-2.01),
                Cfg(repetition=0.0), Cfg(min_p=0.1), Cfg(top_k=65)):
        assert validate(lib, bad) == 2
    assert validate(lib, Cfg(temperature=0.7, top_p=0.8, top_k=20, presence=1.5)) == 0
    lib.fg_sampler_config_greedy(cfg)
    assert cfg.temperature == 0.0
    assert np.array_equal(oracle.uniform_stream(lib, 42, 4), oracle.uniform_stream(lib, 42, 4))
    scores, ids = [5.0, 4.0, 3.0], [9, 3, 1]
    a = oracle.select(lib, Cfg(1.0, 1.0, 2), scores, ids, 0.3)
    assert a[0] == 0 and a[1] != 1
    assert oracle.select(lib, Cfg(1.0, 1.0, 3), scores, ids, 0.8)[:2] == (0, 3)
    assert oracle.select(lib, Cfg(0.1, 1.0, 3), scores, ids, 0.8)[:2] == (0, 9)
    assert oracle.select(lib, Cfg(0.1, 0.5, 3), scores, ids, 0.99)[:2] == (0, 9)
    assert oracle.select(lib, Cfg(0.01, 1.0, 3), scores, ids, 0.99)[:2] == (0, 9)
    assert oracle.select(lib, Cfg(0.0, 1.0, 1), [1.0, 1.0], [8, 2], 0.5)[:2] == (0, 2)
    assert not lib.fg_sampler_penalties_active(oracle.OracleConfig.of(Cfg(0.0, 1.0, 1)))
    got = oracle.apply_penalties(lib, [4.0, -4.0, 3.0], [1, 2, 3], [0, 2, 3, 0],
                                 Cfg(0.0, 1.0, 1, presence=1.0, frequency=0.5, repetition=2.0))
    assert got.tolist() == [2.0 - 2.0, -8.0 - 2.5, 3.0]


@pytest.mark.parametrize("kind", KINDS)
def test_golden_vectors(kind):
    lib = oracle.load(kind)
    for entry in GOLDEN["uniform"]:
        got = oracle.uniform_stream(lib, entry["seed"], 16).view(np.uint32).tolist()
        assert got == entry["bits"]
    for entry in GOLDEN["validate"]:
        assert validate(lib, cfg_from_list(entry["config"])) == entry["status"], entry
    for i, entry in enumerate(GOLDEN["select"]):
        status, token, logit, _ = oracle.select(lib, cfg_from_list(entry["config"]),
                                                from_bits(entry["scores"]), entry["ids"],
                                                float(from_bits([entry["uniform"]])[0]))
        assert status == entry["status"], i
        if status == 0:
            assert token == entry["token"], i
            assert np.float32(logit).view(np.uint32) == entry["logit"], i
    for entry in GOLDEN["penalties"]:
        got = oracle.apply_penalties(lib, from_bits(entry["scores"]), entry["ids"], entry["counts"],
                                     cfg_from_list(entry["config"]))
        assert got.view(np.uint32).tolist() == entry["out"]
    values, ids = from_bits(GOLDEN["better"]["values"]), GOLDEN["better"]["ids"]
    table = iter(GOLDEN["better"]["table"])
    for a in values:
        for ai in ids:
            for b in values:
                for bi in ids:
                    assert int(lib.fg_output_better(float(a), ai, float(b), bi)) == int(next(table))
    pipe = GOLDEN["pipeline"]
    logits = from_bits(pipe["logits"]).reshape(pipe["rows"], pipe["vocab"])
    for case in pipe["cases"]:
        status, tokens, token_logits, row_status, _ = oracle.sample_batch(
            lib, logits, [cfg_from_list(case["config"])], from_bits(pipe["uniforms"]),
            np.array(pipe["history_tokens"], dtype=np.uint32),
            np.array(pipe["history_offsets"], dtype=np.uint64))
        assert status == case["status"] and row_status.tolist() == case["row_status"]
        ok = row_status == 0
        assert tokens[ok].tolist() == np.array(case["tokens"])[ok].tolist()
        assert token_logits.view(np.uint32)[ok].tolist() == np.array(case["token_logits"])[ok].tolist()


@pytest.mark.skipif(not oracle.available("reference"), reason="oracle/_ref was not built here")
def test_port_matches_reference_objects_on_random_inputs():
    port, ref = oracle.load("port"), oracle.load("reference")
    rng = np.random.default_rng(7)
    for trial in range(400):
        count = int(rng.integers(1, 65))
        scores = rng.normal(0, 3, count).astype(np.float32)
        if trial % 2:
            scores = np.round(scores * 2) / 2
        if trial % 9 == 0:
            scores[rng.integers(0, count)] = np.nan
        ids = rng.integers(0, 50, count).astype(np.uint32)  # duplicates on purpose
        cfg = Cfg(float(rng.choice([0.0, 0.3, 1.0, 1.7])), float(rng.choice([0.2, 0.9, 1.0])),
                  int(rng.integers(1, 65)))
        u = float(np.float32(rng.random()))
        assert oracle.select(port, cfg, scores, ids, u) == oracle.select(ref, cfg, scores, ids, u)
        counts = rng.integers(0, 3, 50).astype(np.uint32)
        pcfg = Cfg(presence=float(rng.uniform(-2, 2)), frequency=float(rng.uniform(-2, 2)),
                   repetition=float(rng.uniform(0.1, 3)))
        a = oracle.apply_penalties(port, scores, ids, counts, pcfg)
        b = oracle.apply_penalties(ref, scores, ids, counts, pcfg)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    for seed in (0, 1, 99, 2**63):
        assert np.array_equal(oracle.uniform_stream(port, seed, 64), oracle.uniform_stream(ref, seed, 64))


@pytest.mark.parametrize("kind", KINDS)
def test_split_combine_is_order_independent(kind):
    """tests/test_fg_vk.c:4107-4155 of the reference: four slice maxima folded in
    three orders equal the flat argmax, with ties, NaN, infinities, all-equal."""
    lib = oracle.load(kind)
    count, way = 10240, 2560
    for trial in range(8):
        scores = (np.sin((np.arange(count) + 1.0) * (trial + 1.0) * 0.0027) * 2.0).astype(np.float32)
        if trial == 1:
            scores[10] = scores[count - 1] = 5.0
        elif trial == 2:
            scores[way * 2 + 7] = np.nan
        elif trial == 3:
            scores[way] = scores[way * 3 + 3] = np.inf
        elif trial == 4:
            scores[:] = 1.0
        elif trial == 5:
            scores[0] = np.nan
        elif trial == 6:
            scores[way - 1] = 4.0
        elif trial == 7:
            scores[way] = scores[way + 1] = scores[way * 2] = 5.0

        def fold(pairs):
            best, best_id = pairs[0]
            for value, ident in pairs[1:]:
                if lib.fg_output_better(float(value), int(ident), float(best), int(best_id)):
                    best, best_id = value, ident
            return best, best_id

        flat = fold([(scores[i], i) for i in range(count)])
        slices = [fold([(scores[i], i) for i in range(w * way, (w + 1) * way)]) for w in range(4)]
        for order in ([0, 1, 2, 3], [3, 1, 0, 2], [2, 0, 3, 1]):
            got = fold([slices[i] for i in order])
            assert got[1] == flat[1]
            assert got[0] == flat[0] or (math.isnan(got[0]) and math.isnan(flat[0]))
        # the cascade of argmax tiles agrees with the flat fold
        tile_scores, tile_ids = oracle.argmax_reduce(lib, scores)
        final_scores, final_ids = oracle.argmax_reduce(lib, tile_scores, tile_ids)
        assert final_ids[0] == flat[1]


@pytest.mark.parametrize("kind", KINDS)
def test_topk_cascade_equals_global_order(kind):
    """The tile cascade of src/output.c:681-700 keeps exactly the k best finite
    entries under (score descending, id ascending)."""
    lib = oracle.load(kind)
    rng = np.random.default_rng(12)
    for count, k in [(19, 4), (1024, 64), (5000, 20), (40_000, 50)]:
        scores = np.round(rng.normal(0, 2, count), 1).astype(np.float32)
        scores[rng.integers(0, count, 4)] = np.nan
        cur_scores, cur_ids, n = scores, None, count
        while True:
            cur_scores, cur_ids = oracle.topk_select(lib, cur_scores[:n], cur_ids if cur_ids is None else cur_ids[:n], k)
            n = len(cur_ids)
            if n <= k:
                break
        finite = np.nonzero(np.isfinite(scores))[0]
        order = sorted(finite.tolist(), key=lambda i: (-scores[i], i))[:k]
        assert cur_ids[:len(order)].tolist() == order


@pytest.mark.parametrize("kind", KINDS)
def test_generalised_select_equals_reference_select_on_its_domain(kind):
    lib = oracle.load(kind)
    rng = np.random.default_rng(3)
    for trial in range(200):
        count = int(rng.integers(1, 65))
        scores = np.round(rng.normal(0, 3, count), 1).astype(np.float32)
        ids = rng.permutation(1000)[:count].astype(np.uint32)
        cfg = Cfg(float(rng.choice([0.0, 0.5, 1.0])), float(rng.choice([0.3, 0.9, 1.0])),
                  int(rng.integers(1, 65)))
        u = float(np.float32(rng.random()))
        want = oracle.select(lib, cfg, scores, ids, u)
        got = oracle.select_general(lib, cfg, scores, ids, u)
        assert got[0] == want[0] and got[1] == want[1]
        assert np.float32(got[2]).view(np.uint32) == np.float32(want[2]).view(np.uint32)


def test_sharded_oracle_equals_unsharded():
    lib = oracle.load("port")
    rng = np.random.default_rng(44)
    rows, vocab, shards, k_shard = 6, 4000, 4, 64
    logits = np.round(rng.normal(0, 3, (rows, vocab)), 1).astype(np.float32)
    lengths = rng.integers(0, 100, rows)
    offsets = np.zeros(rows + 1, dtype=np.uint64)
    offsets[1:] = np.cumsum(lengths)
    tokens = rng.integers(0, vocab, int(offsets[-1])).astype(np.uint32)
    uniforms = rng.random(rows).astype(np.float32)
    cfg = Cfg(0.8, 0.9, 40, presence=0.5, frequency=0.25, repetition=1.2)
    want = oracle.sample_batch(lib, logits, [cfg], uniforms, tokens, offsets)
    width = vocab // shards
    parts = [oracle.shard_topk(lib, logits[:, s * width:(s + 1) * width].copy(), [cfg], s * width, vocab,
                               k_shard, tokens, offsets) for s in range(shards)]
    scores = np.stack([p[1] for p in parts])
    ids = np.stack([p[2] for p in parts])
    got = oracle.merge_select(lib, scores, ids, [s * width for s in range(shards)], [width] * shards,
                              [cfg], uniforms)
    assert got[0] == want[0] == 0
    assert np.array_equal(got[1], want[1])
    assert np.array_equal(got[2].view(np.uint32), want[2].view(np.uint32))
    ids[1, 2, 0] = 5  # an id outside shard 1's span fails that row (src/runtime.c:2451-2456)
    bad = oracle.merge_select(lib, scores, ids, [s * width for s in range(shards)], [width] * shards,
                              [cfg], uniforms)
    assert bad[3][2] == 5 and bad[3][0] == 0


def _reduce_before(a, ai, b, bi):
    """tests/test_fg_vk.c:1223-1229 of the reference (topk_before)."""
    ap, bp = ai == 0xFFFFFFFF, bi == 0xFFFFFFFF
    if ap or bp:
        return (not ap) and bp
    an, bn = not np.isfinite(a), not np.isfinite(b)
    if an or bn:
        return an if an != bn else ai < bi
    return a > b or (a == b and ai < bi)


def reduce_chunked_inputs(count):
    """The input generator of tests/test_fg_vk.c:1243-1252 (zeros, NaN, +-Inf sprinkled in)."""
    scores = np.zeros(count, dtype=np.float32)
    seed = 12345
    for i in range(count):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        value = np.float32(((seed >> 8) % 2000) * 0.5)
        if i % 97 == 0:
            value = np.float32(0.0)
        if i % 257 == 0:
            value = np.float32(np.nan)
        if i % 389 == 0:
            value = np.float32(np.inf)
        if i % 521 == 0:
            value = np.float32(-np.inf)
        scores[i] = value
    return scores


def test_sorted_top512_oracle_has_the_reference_tests_properties(port):
    """tests/test_fg_vk.c:1231-1272 (topk_reduce_chunked) and :1202 (output_topk), on the oracle's
    restatement of shaders/fg_topk_reduce_v2.comp."""
    everything = reduce_chunked_inputs(8200)
    for count in (1, 2, 7, 63, 64, 65, 100, 511, 512, 513, 1000, 1024, 1091, 2048, 4032, 4096, 4097, 5000,
                  8192, 8200):
        scores = everything[:count]
        got_scores, got_ids = oracle.topk_reduce(port, scores)
        groups = (count + 4095) // 4096
        expected = count if groups == 1 and count < 512 else groups * 512
        assert len(got_scores) == expected, count
        for i in range(expected):
            group, within = divmod(i, 512)
            remaining = max(count - group * 4096, 0)
            valid = min(remaining, 512)
            if within >= valid:
                assert got_scores[i] == -np.inf and got_ids[i] == 0xFFFFFFFF
                continue
            ident = int(got_ids[i])
            assert ident < count and got_scores[i:i + 1].view(np.uint32)[0] == scores[ident:ident + 1].view(np.uint32)[0]
            if within + 1 < valid:
                assert not _reduce_before(got_scores[i + 1], int(got_ids[i + 1]), got_scores[i], ident), (count, i)
    # the vocabulary-sized cascade: a NaN sorts first, then the three spikes
    vocab = 248_320
    scores = -np.arange(vocab, dtype=np.float32)
    scores[12345], scores[23456], scores[34567], scores[45678] = 100.0, 99.0, 98.0, np.nan
    cur_scores, cur_ids = scores, None
    while len(cur_scores) > 512:
        cur_scores, cur_ids = oracle.topk_reduce(port, cur_scores, cur_ids)
    assert cur_ids[:4].tolist() == [45678, 12345, 23456, 34567] and not np.isfinite(cur_scores[0])
    assert cur_scores[1:4].tolist() == [100.0, 99.0, 98.0]


def test_router_topk_port_equals_the_reference(port):
    rng = np.random.default_rng(77)
    have_reference = oracle.available("reference")
    ref = oracle.load("reference") if have_reference else None
    for trial in range(60):
        count = [512, 512, 64, 17][trial % 4]
        k = [10, 10, 8, 17][trial % 4]
        logits = (rng.standard_normal(count) * (0.1 + trial % 5)).astype(np.float32)
        if trial % 3 == 0:
            logits[rng.integers(0, count, 6)] = logits[3]  # ties: the smaller id wins
        status, ids, weights = oracle.router_topk(port, logits, k)
        assert status == 0 and len(set(ids.tolist())) == k
        order = sorted(range(count), key=lambda i: (-logits[i], i))[:k]
        assert ids.tolist() == order
        assert abs(float(weights.sum()) - 1.0) < 1e-5
        if have_reference:
            ref_status, ref_ids, ref_weights = oracle.router_topk(ref, logits, k, reference=True)
            assert ref_status == status and np.array_equal(ref_ids, ids)
            assert np.array_equal(ref_weights.view(np.uint32), weights.view(np.uint32))
    bad = np.zeros(16, dtype=np.float32)
    bad[3] = np.nan
    assert oracle.router_topk(port, bad, 4)[0] == 4  # FG_ERR_FORMAT, src/q38_math.c:61
