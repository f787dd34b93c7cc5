"""Generates tests/golden/sampler_golden.json from the REFERENCE's own objects.

Run where the reference tree is mounted:

    make -C oracle reference REFERENCE=<path of the reference tree>
    python tests/golden/make_golden.py

It drives oracle/_ref/libfgref.so (the reference's src/sampler.c, src/util.c and
the comparator of src/output.c, compiled unchanged, plus this repository's
pipeline around them) on small seeded inputs and records inputs and outputs as
bit patterns.  The fixture travels with the repository; the reference does not.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402


class Cfg:
    def __init__(self, temperature=1.0, top_p=0.95, top_k=20, presence=0.0, frequency=0.0,
                 repetition=1.0, min_p=0.0, seed=0x9E3779B97F4A7C15):
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.presence_penalty, self.frequency_penalty = presence, frequency
        self.repetition_penalty, self.min_p, self.seed = repetition, min_p, seed

    def as_list(self):
        return [self.temperature, self.top_p, self.top_k, self.presence_penalty,
                self.frequency_penalty, self.repetition_penalty, self.min_p, self.seed]


def bits(a) -> list[int]:
    return np.asarray(a, dtype=np.float32).view(np.uint32).tolist()


def main() -> None:
    ref = oracle.load("reference")
    assert ref.fgo_kind() == b"reference"
    rng = np.random.default_rng(20260915)
    out: dict = {"generator": "tests/golden/make_golden.py", "source": "reference objects"}

    # xorshift64* streams (src/sampler.c:62-73)
    out["uniform"] = [{"seed": seed, "bits": bits(oracle.uniform_stream(ref, seed, 16))}
                      for seed in (0, 1, 42, 0x9E3779B97F4A7C15, 2**64 - 1)]

    # validation table (src/sampler.c:24-38)
    table = []
    for fields in [dict(), dict(presence=2.0, frequency=-2.0), dict(presence=2.01), dict(presence=-2.01),
                   dict(frequency=2.01), dict(frequency=-2.01), dict(repetition=0.0), dict(min_p=0.1),
                   dict(temperature=0.7, top_p=0.8, top_k=20, presence=1.5), dict(top_k=65),
                   dict(top_k=0), dict(top_p=0.0), dict(top_p=1.0), dict(top_p=1.0001),
                   dict(temperature=-0.0), dict(temperature=-1e-9), dict(temperature=float("nan")),
                   dict(temperature=float("inf")), dict(repetition=float("inf")),
                   dict(repetition=1e-30), dict(top_k=64), dict(min_p=-0.0)]:
        cfg = Cfg(**fields)
        err = oracle.OracleError()
        status = ref.fg_sampler_config_validate(oracle.OracleConfig.of(cfg), err)
        table.append({"config": [str(x) for x in cfg.as_list()], "status": int(status)})
    out["validate"] = table

    # select (src/sampler.c:80-122)
    selects = []
    for trial in range(120):
        count = int(rng.integers(1, 65))
        scores = rng.normal(0, 3, count).astype(np.float32)
        if trial % 3 == 0:
            scores = np.round(scores)
        if trial % 5 == 0:
            scores[rng.integers(0, count)] = np.nan
        if trial % 7 == 0:
            scores[rng.integers(0, count)] = np.inf
        if trial % 11 == 0:
            scores[:] = np.nan
        ids = rng.permutation(200_000)[:count].astype(np.uint32)
        cfg = Cfg(temperature=float(rng.choice([0.0, 0.01, 0.5, 0.7, 1.0, 2.0])),
                  top_p=float(rng.choice([0.1, 0.5, 0.8, 0.95, 1.0])), top_k=int(rng.integers(1, 65)))
        u = float(np.float32(rng.random()))
        if trial % 13 == 0:
            u = 1.5
        status, token, logit, _ = oracle.select(ref, cfg, scores, ids, u)
        selects.append({"config": cfg.as_list(), "scores": bits(scores), "ids": ids.tolist(),
                        "uniform": bits([u])[0], "status": status, "token": token,
                        "logit": bits([logit])[0]})
    out["select"] = selects

    # penalties (src/sampler.c:46-60)
    penalties = []
    for presence, frequency, repetition in [(0, 0, 1), (1.5, 0, 1), (0, 0.5, 1), (0, 0, 1.05), (0.5, 0.5, 1),
                                            (-2, 2, 0.5), (0.3, -0.7, 1.9), (1.0, 0.5, 2.0)]:
        n = 200
        scores = rng.normal(0, 4, n).astype(np.float32)
        scores[:5] = [0.0, -0.0, 1e-40, -1e-40, np.inf]
        ids = rng.integers(0, 60, n).astype(np.uint32)
        counts = rng.integers(0, 4, 60).astype(np.uint32)
        counts[7] = 4_000_000_000
        cfg = Cfg(presence=presence, frequency=frequency, repetition=repetition)
        got = oracle.apply_penalties(ref, scores, ids, counts, cfg)
        penalties.append({"config": cfg.as_list(), "scores": bits(scores), "ids": ids.tolist(),
                          "counts": counts.tolist(), "out": bits(got)})
    out["penalties"] = penalties

    # argmax total order (src/output.c:484-498)
    values = [0.0, -0.0, 1.0, -1.0, 5.0, float("nan"), float("inf"), float("-inf")]
    idsx = [0, 1, 7, 0xFFFFFFFF]
    better = []
    for a in values:
        for ai in idsx:
            for b in values:
                for bi in idsx:
                    better.append(int(ref.fg_output_better(a, ai, b, bi)))
    out["better"] = {"values": bits(values), "ids": idsx, "table": "".join(map(str, better))}

    # whole rows through the pipeline linked against the reference objects
    rows, vocab = 8, 3000
    logits = np.round(rng.normal(0, 3, (rows, vocab)) * 8).astype(np.float32) / 8
    logits[1, 5] = np.nan
    logits[2, 17] = np.inf
    lengths = rng.integers(0, 200, rows)
    offsets = np.zeros(rows + 1, dtype=np.uint64)
    offsets[1:] = np.cumsum(lengths)
    tokens = rng.integers(0, vocab, int(offsets[-1])).astype(np.uint32)
    uniforms = rng.random(rows).astype(np.float32)
    pipeline = []
    for cfg in [Cfg(temperature=0.0, top_p=1.0, top_k=1, repetition=1.1),
                Cfg(temperature=0.7, top_p=0.8, top_k=20, presence=1.5),
                Cfg(temperature=1.0, top_p=0.95, top_k=50, frequency=0.5, repetition=1.05),
                Cfg(temperature=1.2, top_p=0.99, top_k=64, presence=0.5, frequency=0.5),
                Cfg(temperature=0.0, top_p=1.0, top_k=1)]:
        status, toks, tls, row_status, _ = oracle.sample_batch(ref, logits, [cfg], uniforms, tokens, offsets)
        pipeline.append({"config": cfg.as_list(), "status": int(status), "tokens": toks.tolist(),
                         "token_logits": bits(tls), "row_status": row_status.tolist()})
    out["pipeline"] = {"rows": rows, "vocab": vocab, "logits": bits(logits.ravel()),
                       "history_tokens": tokens.tolist(), "history_offsets": offsets.tolist(),
                       "uniforms": bits(uniforms), "cases": pipeline}

    path = Path(__file__).resolve().parent / "sampler_golden.json"
    path.write_text(json.dumps(out, separators=(",", ":")))
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
