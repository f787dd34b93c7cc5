"""The fg_sampler.h entry points through the C ABI, on the reference's own
known answers (tests/test_sampler.c:28-54 of the reference) and against the CPU
oracle on random candidate sets.  select and apply_penalties run on the GPU."""
import ctypes
import math
from ctypes import byref, c_float, c_uint32

import numpy as np
import pytest

import oracle
from flash_gordon_b200 import (FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_OK, FgError, SamplerConfig,
                               load_library)
from flash_gordon_b200.api import select

pytestmark = pytest.mark.gpu


def test_reference_select_known_answers(context):
    scores, ids = [5.0, 4.0, 3.0], [9, 3, 1]
    cfg = SamplerConfig.make(temperature=1.0, top_p=1.0, top_k=2)
    a = select(cfg, scores, ids, 0.3)
    b = select(cfg, scores, ids, 0.3)
    assert a[0] == FG_OK and a[:3] == b[:3] and a[1] != 1          # top-k 2 never picks id 1
    cfg.top_k = 3
    assert select(cfg, scores, ids, 0.8)[:2] == (FG_OK, 3)
    cfg.temperature = 0.1
    assert select(cfg, scores, ids, 0.8)[:2] == (FG_OK, 9)          # low temperature
    cfg.top_p = 0.5
    assert select(cfg, scores, ids, 0.99)[:2] == (FG_OK, 9)         # top-p cut
    cfg.top_p, cfg.temperature = 1.0, 0.01
    assert select(cfg, scores, ids, 0.99)[:2] == (FG_OK, 9)
    cfg.temperature, cfg.top_k = 0.0, 1
    assert select(cfg, [1.0, 1.0], [8, 2], 0.5)[:2] == (FG_OK, 2)   # tie -> smaller id


def test_reference_penalties_known_answer(context, library):
    cfg = SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1, presence=1.0, frequency=0.5,
                             repetition=2.0)
    scores = (c_float * 3)(4.0, -4.0, 3.0)
    ids = (c_uint32 * 3)(1, 2, 3)
    counts = (c_uint32 * 4)(0, 2, 3, 0)
    library.fg_sampler_apply_penalties(scores, ids, counts, 3, byref(cfg))
    assert library.fg_sampler_last_status() == FG_OK
    assert list(scores) == [2.0 - 2.0, -8.0 - 2.5, 3.0]


def test_select_error_behaviour(context, library):
    cfg = SamplerConfig.make()
    assert select(cfg, [], [], 0.5)[0] == FG_ERR_ARGUMENT
    assert select(cfg, [0.0] * 65, list(range(65)), 0.5)[0] == FG_ERR_ARGUMENT
    status, _, _, message = select(cfg, [math.nan, math.inf], [1, 2], 0.5)
    assert status == FG_ERR_FORMAT and message == "sampler received no finite candidates"
    bad = SamplerConfig.make(top_k=0)
    status, _, _, message = select(bad, [1.0], [1], 0.5)
    assert status == FG_ERR_ARGUMENT and message == "invalid sampler controls"
    # an earlier error record is kept and its code returned (src/sampler.c:85-86 of the reference)
    err = FgError()
    err.code = 7
    err.message = b"earlier failure"
    token, logit = c_uint32(0), c_float(0)
    status = library.fg_sampler_select(byref(cfg), None, None, 0, 0.5, byref(token), byref(logit),
                                       byref(err))
    assert status == 7 and err.text() == "earlier failure"
    err = FgError()
    status = library.fg_sampler_select(byref(cfg), None, None, 0, 0.5, byref(token), byref(logit),
                                       byref(err))
    assert status == FG_ERR_ARGUMENT and err.text() == "invalid sampler candidates"


def test_select_matches_oracle_on_random_sets(context, port):
    rng = np.random.default_rng(11)
    for trial in range(300):
        count = int(rng.integers(1, 65))
        scores = rng.normal(0, 3, count).astype(np.float32)
        if trial % 3 == 0:
            scores = np.round(scores)                      # ties
        if trial % 5 == 0:
            scores[rng.integers(0, count)] = np.nan
        if trial % 7 == 0:
            scores[rng.integers(0, count)] = -np.inf
        ids = rng.permutation(100_000)[:count].astype(np.uint32)
        cfg = SamplerConfig.make(temperature=float(rng.choice([0.0, 0.01, 0.5, 1.0, 2.0])),
                                 top_p=float(rng.choice([0.1, 0.5, 0.9, 1.0])),
                                 top_k=int(rng.integers(1, 65)))
        u = float(rng.random(dtype=np.float32)) if trial % 11 else 1.5
        want = oracle.select(port, cfg, scores, ids, u)
        got = select(cfg, scores.tolist(), ids.tolist(), u)
        assert got[0] == want[0], f"trial {trial}"
        if want[0] == FG_OK:
            assert got[1] == want[1], f"trial {trial}: token"
            assert np.float32(got[2]).view(np.uint32) == np.float32(want[2]).view(np.uint32)


def test_apply_penalties_matches_oracle(context, library, port):
    rng = np.random.default_rng(5)
    for presence, frequency, repetition in [(0, 0, 1), (1.5, 0, 1), (0, 0.5, 1), (0, 0, 1.05),
                                            (0.5, 0.5, 1), (-2, 2, 0.5), (0.3, -0.7, 1.9)]:
        cfg = SamplerConfig.make(presence=presence, frequency=frequency, repetition=repetition)
        n = 5000
        scores = rng.normal(0, 4, n).astype(np.float32)
        scores[:6] = [0.0, -0.0, 1e-40, -1e-40, np.inf, np.nan]
        ids = rng.integers(0, 800, n).astype(np.uint32)
        counts = rng.integers(0, 4, 800).astype(np.uint32)
        counts[5] = 4_000_000_000
        want = oracle.apply_penalties(port, scores, ids, counts, cfg)
        got = scores.copy()
        library.fg_sampler_apply_penalties(got.ctypes.data_as(ctypes.c_void_p),
                                           ids.ctypes.data_as(ctypes.c_void_p),
                                           counts.ctypes.data_as(ctypes.c_void_p), n, byref(cfg))
        assert library.fg_sampler_last_status() == FG_OK
        # NaN payloads are not part of the contract (x86 keeps the operand's, the GPU
        # returns the canonical quiet NaN); everything else must agree bit for bit
        both_nan = np.isnan(got) & np.isnan(want)
        assert np.array_equal(got.view(np.uint32)[~both_nan], want.view(np.uint32)[~both_nan])


def test_the_reference_s_own_sampler_test_passes_against_this_library():
    """tests/test_sampler.c of the reference, compiled unchanged against include/ and linked
    with libfgsampler (`make -C oracle drop-in REFERENCE=...`, done where the reference tree is
    mounted; the binary travels with the repository).  All its checks must pass."""
    import subprocess
    from pathlib import Path
    binary = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "test_sampler_dropin"
    if not binary.exists():
        pytest.skip("oracle/_ref/test_sampler_dropin is built only where the reference tree is mounted")
    done = subprocess.run([str(binary)], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
