"""Shared by the parity tests: run a workload through the CPU oracle and through
the CUDA library, and compare."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from flash_gordon_b200 import FG_OK


def logits_to_numpy(logits: torch.Tensor) -> np.ndarray:
    logits = logits.detach().cpu().contiguous()
    if logits.dtype == torch.bfloat16:
        return logits.view(torch.int16).numpy().view(np.uint16)
    return logits.numpy()


def oracle_kind() -> str:
    """The checker the GPU parity tests use: the reference's own sampler objects where
    that build is present (it travels with the repository), else this repository's
    port of them (the CPU tests hold the two equal)."""
    return "reference" if oracle.available("reference") else "port"


def run_oracle(workload, kind: str | None = None, threads: int = 8, want_candidates: bool = False):
    lib = oracle.load(kind or oracle_kind())
    tokens = offsets = None
    if workload.history_tokens is not None:
        tokens = workload.history_tokens.cpu().numpy().view(np.uint32)
        offsets = workload.history_offsets.cpu().numpy().view(np.uint64)
    uniforms = None if workload.uniforms is None else workload.uniforms.cpu().numpy()
    return oracle.sample_batch(lib, logits_to_numpy(workload.logits), workload.configs, uniforms,
                               tokens, offsets, workload.allow_no_topk, threads, want_candidates)


def run_gpu(context, workload, debug: bool = False, **kwargs):
    w = workload.to("cuda")
    result = context.sample_batch(w.logits, w.configs, w.uniforms, w.history_tokens,
                                  w.history_offsets, w.history_max,
                                  allow_no_topk=w.allow_no_topk, debug=debug, **kwargs)
    torch.cuda.synchronize()
    return result


def as_u32(tensor: torch.Tensor) -> np.ndarray:
    return tensor.cpu().numpy().view(np.uint32)


def assert_rows_equal(result, expected, label: str = ""):
    """Bit-exact: status, token id and the penalised logit of the pick, per row."""
    status, tokens, token_logits, row_status, _ = expected
    got_status = as_u32(result.row_status)
    assert np.array_equal(got_status, row_status), f"{label}: row status differs"
    assert result.status == status, f"{label}: call status {result.status} != {status}"
    ok = row_status == FG_OK
    got_tokens = as_u32(result.tokens)
    bad = np.nonzero(got_tokens[ok] != tokens[ok])[0]
    assert bad.size == 0, f"{label}: {bad.size} token ids differ, first rows {np.nonzero(ok)[0][bad[:5]]}"
    got_bits = result.token_logits.cpu().numpy().view(np.uint32)
    want_bits = token_logits.view(np.uint32)
    assert np.array_equal(got_bits[ok], want_bits[ok]), f"{label}: token logits differ in bits"


def assert_candidates_close(result, expected, rel: float = 1e-5, label: str = ""):
    """Candidate ids and penalised logits bit-exact; probabilities within `rel`."""
    cands = expected[4]
    row_status = expected[3]
    count = as_u32(result.debug["count"])
    ids = as_u32(result.debug["ids"])
    scores = result.debug["scores"].cpu().numpy().view(np.uint32)
    raw = result.debug["raw"].cpu().numpy()
    tempered = result.debug["tempered"].cpu().numpy()
    for r in range(len(row_status)):
        if row_status[r] != FG_OK:
            continue
        n = cands[r].count
        assert count[r] == n, f"{label} row {r}: {count[r]} candidates, oracle {n}"
        want_ids = np.array(cands[r].ids[:n], dtype=np.uint32)
        want_scores = np.array(cands[r].scores[:n], dtype=np.float32).view(np.uint32)
        assert np.array_equal(ids[r, :n], want_ids), f"{label} row {r}: candidate ids"
        assert np.array_equal(scores[r, :n], want_scores), f"{label} row {r}: candidate logits"
        want_raw = np.array(cands[r].raw_probability[:n])
        want_temp = np.array(cands[r].tempered_probability[:n])
        np.testing.assert_allclose(raw[r, :n], want_raw, rtol=rel, atol=0, err_msg=f"{label} row {r} raw")
        np.testing.assert_allclose(tempered[r, :n], want_temp, rtol=rel, atol=0,
                                   err_msg=f"{label} row {r} tempered")


def random_workload(rows, vocab, history, configs, seed, quantize=0.0, specials=0, dtype=torch.float32,
                    stride=None, uniform_history=True):
    """Random rows; `quantize` > 0 rounds logits to that grid (many exact ties);
    `specials` sprinkles that many NaN / +Inf / -Inf / +-0 per row."""
    from flash_gordon_b200.synth import Workload
    g = torch.Generator().manual_seed(seed)
    stride = vocab if stride is None else stride
    storage = torch.randn(rows, stride, generator=g) * 3.0
    if quantize:
        storage = torch.round(storage / quantize) * quantize
    if specials:
        values = torch.tensor([float("nan"), float("inf"), float("-inf"), 0.0, -0.0, 1e-40, -1e-40])
        for r in range(rows):
            where = torch.randint(0, vocab, (specials,), generator=g)
            what = values[torch.randint(0, len(values), (specials,), generator=g)]
            storage[r, where] = what
    storage = storage.to(dtype)
    logits = storage[:, :vocab]
    tokens = offsets = None
    if history:
        lengths = torch.randint(0, history + 1, (rows,), generator=g)
        lengths[0] = history
        offsets = torch.zeros(rows + 1, dtype=torch.int64)
        offsets[1:] = torch.cumsum(lengths, 0)
        total = int(offsets[-1])
        if uniform_history:
            tokens = torch.randint(0, vocab, (total,), generator=g, dtype=torch.int32)
        else:  # heavy repeats
            tokens = (torch.randint(0, vocab, (total,), generator=g) % max(1, vocab // 50)).to(torch.int32)
    uniforms = torch.rand(rows, generator=g)
    return Workload("random", logits, list(configs), uniforms, tokens, offsets, history)
