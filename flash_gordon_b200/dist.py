"""Multi-GPU plumbing for the two ways the sampling path spreads over GPUs.

One process per GPU, `torch.distributed` for the plumbing.

* Row partition: rows are independent, so each rank samples a contiguous block
  of rows and nothing is exchanged on the data path (an optional all-gather of
  the 12 bytes of result per row is provided for callers that want every
  result everywhere).

* Vocabulary shards: each rank owns a contiguous span of columns of every row
  (what a tensor-parallel lm_head leaves behind).  A rank keeps the `k_shard`
  best finite (logit, global id) pairs of its span per row, the pairs are
  all-gathered, and every rank merges them and samples.  The reference does the
  same for greedy decoding with one pair per slice (src/output.c:320-344,
  src/runtime.c:2437-2466, spans from src/protocol.c:93-105); here a slice sends
  k_shard pairs so that top-k / top-p sampling works too.

The compute steps go through a small backend interface so the exchange logic can
be exercised on CPU ranks (gloo) with a stand-in backend.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def row_block(rows: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block of `rows` owned by `rank`; the first rows % world ranks get one more."""
    base, extra = divmod(rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_span(vocab: int, shards: int, shard: int) -> tuple[int, int]:
    """(first column, width) of `shard`: equal widths, the last one takes the remainder
    (the rule of src/protocol.c:99-103 of the reference for its 4-way split)."""
    width = vocab // shards
    first = shard * width
    return first, (vocab - first) if shard + 1 == shards else width


def gather_rows(tokens: torch.Tensor, token_logits: torch.Tensor, row_status: torch.Tensor,
                group=None):
    """All ranks' row results concatenated in rank order (blocks may differ by one row)."""
    world = dist.get_world_size(group)
    packed = torch.stack([tokens.to(torch.int32), token_logits.view(torch.int32),
                          row_status.to(torch.int32)], dim=1).contiguous()
    counts = torch.zeros(world, dtype=torch.int64, device=packed.device)
    counts[dist.get_rank(group)] = packed.shape[0]
    dist.all_reduce(counts, group=group)
    longest = int(counts.max())
    padded = torch.zeros(longest, 3, dtype=torch.int32, device=packed.device)
    padded[:packed.shape[0]] = packed
    everyone = torch.empty(world, longest, 3, dtype=torch.int32, device=packed.device)
    # flat views: the backends agree on 1-D concatenation
    dist.all_gather_into_tensor(everyone.view(-1), padded.view(-1), group=group)
    parts = [everyone[r, :int(counts[r])] for r in range(world)]
    merged = torch.cat(parts, dim=0)
    return merged[:, 0].contiguous(), merged[:, 1].contiguous().view(torch.float32), merged[:, 2].contiguous()


class CudaBackend:
    """The two compute steps of the sharded path on this rank's GPU."""

    def __init__(self, context):
        self.context = context

    def shard_topk(self, logits, configs, vocab_offset, vocab_total, k_shard, history_tokens,
                   history_offsets, history_max):
        scores, ids, row_status, status = self.context.shard_topk(
            logits, configs, vocab_offset, vocab_total, k_shard, history_tokens, history_offsets,
            history_max, asynchronous=True)
        return scores, ids, row_status

    def merge_select(self, scores, ids, rows, shards, k_shard, first, width, configs, uniforms):
        return self.context.merge_select(scores, ids, rows, shards, k_shard, first, width, configs,
                                         uniforms)


@dataclass
class ShardedResult:
    tokens: torch.Tensor
    token_logits: torch.Tensor
    row_status: torch.Tensor
    status: int
    shard_status: torch.Tensor


def sample_vocab_sharded(backend, logits_shard: torch.Tensor, configs, uniforms: torch.Tensor,
                         vocab_total: int, k_shard: int = 64, history_tokens=None,
                         history_offsets=None, history_max: int = 0, group=None) -> ShardedResult:
    """Every rank calls this with its column span of the same rows; every rank gets
    the same tokens.  The spans follow `shard_span` in rank order."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = logits_shard.shape[0]
    first, width = shard_span(vocab_total, world, rank)
    if logits_shard.shape[1] != width:
        raise ValueError(f"rank {rank} holds {logits_shard.shape[1]} columns, its span has {width}")
    scores, ids, shard_status = backend.shard_topk(logits_shard, configs, first, vocab_total, k_shard,
                                                   history_tokens, history_offsets, history_max)
    # one exchange: (fp32 logit, int32 global id) pairs, 8 bytes each, as one buffer
    mine = torch.stack([scores.view(torch.int32), ids.view(torch.int32)], dim=0).contiguous()
    everyone = torch.empty(world, 2, rows, k_shard, dtype=torch.int32, device=mine.device)
    dist.all_gather_into_tensor(everyone.view(-1), mine.view(-1), group=group)
    all_scores = everyone[:, 0].contiguous().view(torch.float32)  # [shard][row][k]
    all_ids = everyone[:, 1].contiguous()
    spans = [shard_span(vocab_total, world, s) for s in range(world)]
    merged = backend.merge_select(all_scores, all_ids, rows, world, k_shard, [s[0] for s in spans],
                                  [s[1] for s in spans], configs, uniforms)
    return ShardedResult(merged.tokens, merged.token_logits, merged.row_status, merged.status,
                         shard_status)
