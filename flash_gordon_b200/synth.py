"""Seeded synthetic sampling workloads.

The reference measures this path on no public suite and ships no recorded
logits, so every test and benchmark input is synthetic: the five shapes and
value distributions below follow the configurations the benchmark is defined
on (vocabulary 151,936; Gaussian / Gumbel logits; uniform or Zipf histories).
`rows`, `vocab` and `history` can be scaled down for tests; the distributions
stay the same.  Everything is generated with a seeded torch generator on
`device`, so the oracle and the GPU path see identical bits.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from . import SamplerConfig

VOCAB = 151_936
DEFAULT_SEED = 0x9E3779B97F4A7C15


@dataclass
class Workload:
    name: str
    logits: torch.Tensor                 # [rows, vocab] fp32 or bf16
    configs: list                        # one SamplerConfig (shared) or one per row
    uniforms: torch.Tensor | None        # [rows] fp32
    history_tokens: torch.Tensor | None  # int32 CSR payload
    history_offsets: torch.Tensor | None # int64 [rows + 1]
    history_max: int
    allow_no_topk: bool = False
    meta: dict = field(default_factory=dict)

    @property
    def rows(self) -> int:
        return self.logits.shape[0]

    @property
    def vocab(self) -> int:
        return self.logits.shape[1]

    def algorithmic_bytes_per_row(self) -> int:
        """Logits once + the row's history + its uniform + (token, logit) out."""
        history = self.history_max * 4 if self.history_tokens is not None else 0
        return self.vocab * self.logits.element_size() + history + 4 + 8

    def to(self, device) -> "Workload":
        move = lambda t: None if t is None else t.to(device)
        return Workload(self.name, move(self.logits), self.configs, move(self.uniforms),
                        move(self.history_tokens), move(self.history_offsets), self.history_max,
                        self.allow_no_topk, dict(self.meta))

    def slice_rows(self, begin: int, end: int) -> "Workload":
        """Rows [begin, end) as an independent workload (row partitioning)."""
        tokens = offsets = None
        if self.history_tokens is not None:
            first = int(self.history_offsets[begin])
            last = int(self.history_offsets[end])
            tokens = self.history_tokens[first:last]
            offsets = self.history_offsets[begin:end + 1] - first
        configs = self.configs if len(self.configs) == 1 else self.configs[begin:end]
        uniforms = None if self.uniforms is None else self.uniforms[begin:end]
        return Workload(self.name, self.logits[begin:end], configs, uniforms, tokens, offsets,
                        self.history_max, self.allow_no_topk, dict(self.meta))


def _generator(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def xorshift_uniforms(seed: int, count: int) -> list[float]:
    """`count` draws of the sampler's xorshift64* stream (src/sampler.c:62-73 of the
    reference: seed 0 becomes the default seed; x ^= x >> 12, x ^= x << 25, x ^= x >> 27;
    the top 24 bits of x * 2685821657736338717 scaled by 2^-24).  Written out here so that
    generating inputs never loads the native library; tests/test_cpu_abi.py holds it equal
    to fg_sampler_uniform."""
    mask = (1 << 64) - 1
    x = (seed & mask) or DEFAULT_SEED
    out = []
    for _ in range(count):
        x ^= x >> 12
        x = (x ^ (x << 25)) & mask
        x ^= x >> 27
        out.append((((x * 2685821657736338717) & mask) >> 40) / 16777216.0)
    return out


def _uniforms(rows: int, seed: int, device) -> torch.Tensor:
    # one draw per row on the host, as the reference's coordinator does once per token
    return torch.tensor(xorshift_uniforms(seed, rows), dtype=torch.float32, device=device)


def _zipf_history(rows: int, length: int, vocab: int, exponent: float, g, device):
    ranks = torch.arange(1, vocab + 1, dtype=torch.float64, device=device)
    weights = ranks.pow(-exponent)
    weights = (weights / weights.sum()).to(torch.float32)
    drawn = torch.multinomial(weights, rows * length, replacement=True, generator=g)
    # ranks -> ids through a fixed seeded permutation, so popular ids are spread out
    permutation = torch.randperm(vocab, generator=g, device=device)
    tokens = permutation[drawn].to(torch.int32)
    offsets = torch.arange(0, rows + 1, dtype=torch.int64, device=device) * length
    return tokens, offsets


def _uniform_history(rows: int, length: int, vocab: int, g, device):
    tokens = torch.randint(0, vocab, (rows * length,), generator=g, device=device, dtype=torch.int32)
    offsets = torch.arange(0, rows + 1, dtype=torch.int64, device=device) * length
    return tokens, offsets


def config1(device="cpu", vocab: int = VOCAB, history: int = 64, seed: int = 101) -> Workload:
    """One row ~ N(0, 3^2) with +12 added at 8 seeded positions; repetition 1.1 over a
    uniform history; greedy."""
    g = _generator(device, seed)
    logits = torch.randn(1, vocab, generator=g, device=device) * 3.0
    spikes = torch.randperm(vocab, generator=g, device=device)[:8]
    logits[0, spikes] += 12.0
    tokens, offsets = _uniform_history(1, history, vocab, g, device)
    cfg = SamplerConfig.make(temperature=0.0, top_p=1.0, top_k=1, repetition=1.1)
    return Workload("config1", logits, [cfg], None, tokens, offsets, history,
                    meta={"spike": "+12 added at 8 seeded ids", "seed": seed})


def config2(device="cpu", rows: int = 64, vocab: int = VOCAB, history: int = 512,
            seed: int = 202) -> Workload:
    """N(0, 3^2); 5% of rows carry one dominant spike; T 0.7, top-k 20, top-p 0.8,
    presence 1.5 over a Zipf(1.1) history."""
    g = _generator(device, seed)
    logits = torch.randn(rows, vocab, generator=g, device=device) * 3.0
    spiked = max(1, math.ceil(rows * 0.05))
    which = torch.randperm(rows, generator=g, device=device)[:spiked]
    where = torch.randint(0, vocab, (spiked,), generator=g, device=device)
    logits[which, where] += 20.0
    tokens, offsets = _zipf_history(rows, history, vocab, 1.1, g, device)
    cfg = SamplerConfig.make(temperature=0.7, top_p=0.8, top_k=20, presence=1.5)
    return Workload("config2", logits, [cfg], _uniforms(rows, DEFAULT_SEED, device), tokens,
                    offsets, history, meta={"seed": seed})


def config3(device="cpu", rows: int = 1024, vocab: int = VOCAB, history: int = 4096,
            seed: int = 303) -> Workload:
    """Gumbel(0,1) + N(0, 2^2); frequency 0.5 and repetition 1.05 over a Zipf(1.0)
    history; T 1.0, top-k 50, top-p 0.95."""
    g = _generator(device, seed)
    logits = torch.randn(rows, vocab, generator=g, device=device) * 2.0
    u = torch.rand(rows, vocab, generator=g, device=device).clamp_(1e-20, 1.0)
    logits -= torch.log(-torch.log(u))
    del u
    tokens, offsets = _zipf_history(rows, history, vocab, 1.0, g, device)
    cfg = SamplerConfig.make(temperature=1.0, top_p=0.95, top_k=50, frequency=0.5, repetition=1.05)
    return Workload("config3", logits, [cfg], _uniforms(rows, DEFAULT_SEED, device), tokens,
                    offsets, history, meta={"seed": seed})


def config4(device="cpu", rows: int = 256, vocab: int = VOCAB, seed: int = 404) -> Workload:
    """bf16 ~ N(0, 4^2), to be split by columns across GPUs; T 0.8, top-p 0.9,
    merged top-k 64; no penalties."""
    g = _generator(device, seed)
    logits = (torch.randn(rows, vocab, generator=g, device=device) * 4.0).to(torch.bfloat16)
    cfg = SamplerConfig.make(temperature=0.8, top_p=0.9, top_k=64)
    return Workload("config4", logits, [cfg], _uniforms(rows, DEFAULT_SEED, device), None, None, 0,
                    meta={"seed": seed, "k_shard": 64})


def config5(device="cpu", rows: int = 4096, vocab: int = VOCAB, history: int = 32768,
            seed: int = 505) -> Workload:
    """Near-flat N(0, 0.5^2); T 1.2, top-p 0.99, no top-k cut; presence 0.5 and
    frequency 0.5 over a uniform history."""
    g = _generator(device, seed)
    logits = torch.randn(rows, vocab, generator=g, device=device) * 0.5
    tokens, offsets = _uniform_history(rows, history, vocab, g, device)
    cfg = SamplerConfig.make(temperature=1.2, top_p=0.99, top_k=0, presence=0.5, frequency=0.5)
    return Workload("config5", logits, [cfg], _uniforms(rows, DEFAULT_SEED, device), tokens,
                    offsets, history, allow_no_topk=True, meta={"seed": seed})


CONFIGS = {"config1": config1, "config2": config2, "config3": config3, "config4": config4,
           "config5": config5}
