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


FG_ERR_LIMIT = 8  # include/fg.h


@dataclass
class ShardedResult:
    tokens: torch.Tensor
    token_logits: torch.Tensor
    row_status: torch.Tensor
    status: int
    shard_status: torch.Tensor
    message: str = ""


def sample_vocab_sharded(backend, logits_shard: torch.Tensor, configs, uniforms: torch.Tensor,
                         vocab_total: int, k_shard: int = 64, history_tokens=None,
                         history_offsets=None, history_max: int = 0, group=None) -> ShardedResult:
    """The sharded path with torch.distributed doing the exchange (any backend, so CPU ranks
    over gloo can run it with a stand-in for the two compute steps).  Every rank calls this
    with its column span of the same rows; every rank gets the same tokens.  The spans follow
    `shard_span` in rank order.  GPU ranks normally use `Communicator` instead, which does
    the same through the library's own NCCL communicator without any copy in between."""
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
    try:
        dist.all_gather_into_tensor(everyone.view(-1), mine.view(-1), group=group)
    except RuntimeError as error:
        # a rank that never joined: the group's timeout ends the exchange, and the step fails
        # closed with the status the reference gives a partial that misses its deadline
        # (src/runtime.c:2379-2435)
        failed = torch.full((rows,), FG_ERR_LIMIT, dtype=torch.int32)
        result = ShardedResult(torch.full((rows,), -1, dtype=torch.int32), torch.zeros(rows), failed,
                               FG_ERR_LIMIT, shard_status)
        result.message = f"not every rank joined the exchange: {error}"
        return result
    all_scores = everyone[:, 0].contiguous().view(torch.float32)  # [shard][row][k]
    all_ids = everyone[:, 1].contiguous()
    spans = [shard_span(vocab_total, world, s) for s in range(world)]
    merged = backend.merge_select(all_scores, all_ids, rows, world, k_shard, [s[0] for s in spans],
                                  [s[1] for s in spans], configs, uniforms)
    return ShardedResult(merged.tokens, merged.token_logits, merged.row_status, merged.status,
                         shard_status)


class Communicator:
    """fg_dist: this process's membership in the library's own NCCL communicator, bound to a
    Context (its GPU and stream).  torch.distributed is used once, to carry the 128-byte
    communicator id from rank 0 to the others."""

    def __init__(self, context, group=None, timeout_ms: int = 0, ranks: int | None = None,
                 rank: int | None = None, unique_id: bytes | None = None):
        """Joins the ranks of `group` (default: torch.distributed's world).  A caller without
        torch.distributed passes `ranks`, `rank` and the `unique_id` rank 0 made with
        `Communicator.make_unique_id` (a single rank needs neither)."""
        import ctypes
        from . import FG_OK, FgError, FgStatusError
        self.context = context
        self.lib = context.lib
        err = FgError()
        if ranks is None:
            self.ranks = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
            mine = self.make_unique_id(context.lib) if self.rank == 0 else bytes(128)
            carrier = torch.tensor(list(mine), dtype=torch.uint8)
            if dist.get_backend(group) == "nccl":
                carrier = carrier.to(torch.device("cuda", context.device))
            dist.broadcast(carrier, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            unique_id = bytes(carrier.cpu().tolist())
        else:
            self.ranks, self.rank = ranks, 0 if rank is None else rank
            if unique_id is None:
                if self.ranks != 1:
                    raise ValueError("more than one rank needs rank 0's unique id")
                unique_id = self.make_unique_id(context.lib)
        id_bytes = (ctypes.c_ubyte * 128)(*unique_id)
        handle = ctypes.c_void_p()
        status = self.lib.fg_dist_create(context.handle, self.ranks, self.rank, id_bytes, timeout_ms,
                                         ctypes.byref(handle), ctypes.byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        self.handle = handle

    @staticmethod
    def make_unique_id(lib) -> bytes:
        """fg_dist_unique_id: the 128 bytes rank 0 hands to every other rank."""
        import ctypes
        from . import FG_OK, FgError, FgStatusError
        id_bytes = (ctypes.c_ubyte * 128)()
        err = FgError()
        status = lib.fg_dist_unique_id(id_bytes, ctypes.byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        return bytes(id_bytes)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.fg_dist_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sample_vocab_sharded(self, logits_shard: torch.Tensor, configs, uniforms: torch.Tensor,
                             vocab_total: int, k_shard: int = 64, history_tokens=None, history_offsets=None,
                             history_max: int = 0, out=None, asynchronous: bool = False, fused: bool = False):
        """fg_dist_sample_vocab_sharded: shard top-k, one all-gather, merge and select.  `fused`:
        fg_dist_sample_vocab_sharded_fused, where the shard kernel stores its candidates straight
        into every rank's window and the merge kernel waits for them (no collective kernel)."""
        import ctypes
        from . import FG_CUDA_SAMPLE_ASYNC, FgError
        from .api import SampleResult
        rows = logits_shard.shape[0]
        device = logits_shard.device
        if out is None:
            out = (torch.empty(rows, dtype=torch.int32, device=device),
                   torch.empty(rows, dtype=torch.float32, device=device),
                   torch.empty(rows, dtype=torch.int32, device=device))
        args, keep = self.context._args(logits_shard, configs, uniforms, history_tokens, history_offsets,
                                        history_max, None, FG_CUDA_SAMPLE_ASYNC if asynchronous else 0, out, None)
        err = FgError()
        call = self.lib.fg_dist_sample_vocab_sharded_fused if fused else self.lib.fg_dist_sample_vocab_sharded
        status = call(self.handle, ctypes.byref(args), vocab_total, k_shard, ctypes.byref(err))
        del keep
        return SampleResult(out[0], out[1], out[2], status, err.text(), None)

    def prepared_sample_vocab_sharded(self, logits_shard: torch.Tensor, configs, uniforms: torch.Tensor,
                                      vocab_total: int, k_shard: int, out, history_tokens=None,
                                      history_offsets=None, history_max: int = 0, fused: bool = False):
        """Builds the argument block once; the returned callable re-issues the same asynchronous
        fg_dist_sample_vocab_sharded(_fused) call and returns its status (decode loops call it
        once per token)."""
        import ctypes
        from . import FG_CUDA_SAMPLE_ASYNC, FgError
        args, keep = self.context._args(logits_shard, configs, uniforms, history_tokens, history_offsets,
                                        history_max, None, FG_CUDA_SAMPLE_ASYNC, out, None)
        err = FgError()
        call = self.lib.fg_dist_sample_vocab_sharded_fused if fused else self.lib.fg_dist_sample_vocab_sharded
        handle, args_ref, err_ref = self.handle, ctypes.byref(args), ctypes.byref(err)

        def issue() -> int:
            return call(handle, args_ref, vocab_total, k_shard, err_ref)

        issue.keep = (keep, args, err, logits_shard, uniforms, out)
        return issue

    def gather_rows(self, tokens: torch.Tensor, token_logits: torch.Tensor, row_status: torch.Tensor):
        """fg_dist_gather_rows: every rank's `rows` results on every rank, in rank order."""
        import ctypes
        from . import FG_OK, FgError, FgStatusError
        rows = tokens.shape[0]
        device = tokens.device
        everyone = (torch.empty(self.ranks * rows, dtype=torch.int32, device=device),
                    torch.empty(self.ranks * rows, dtype=torch.float32, device=device),
                    torch.empty(self.ranks * rows, dtype=torch.int32, device=device))
        err = FgError()
        P = ctypes.c_void_p
        status = self.lib.fg_dist_gather_rows(self.handle, P(tokens.data_ptr()), P(token_logits.data_ptr()),
                                              P(row_status.data_ptr()), rows, P(everyone[0].data_ptr()),
                                              P(everyone[1].data_ptr()), P(everyone[2].data_ptr()),
                                              ctypes.byref(err))
        if status != FG_OK:
            raise FgStatusError(status, err.text())
        return everyone
