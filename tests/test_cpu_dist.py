"""The multi-rank host logic on CPU ranks (gloo, world size 2): block and span
arithmetic, the candidate exchange layout of the vocabulary-sharded path and the
gather of row-partitioned results.  The compute steps are stood in for by the CPU
oracle; what is under test is the plumbing around them."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from flash_gordon_b200.dist import gather_rows, row_block, sample_vocab_sharded, shard_span  # noqa: E402


def test_blocks_and_spans_tile_their_ranges():
    for rows, world in [(1024, 8), (1000, 7), (3, 8), (64, 1)]:
        cursor = 0
        for rank in range(world):
            begin, end = row_block(rows, world, rank)
            assert begin == cursor and end >= begin
            cursor = end
        assert cursor == rows
    for vocab, shards in [(151_936, 8), (248_320, 4), (1001, 3)]:
        cursor = 0
        for s in range(shards):
            first, width = shard_span(vocab, shards, s)
            assert first == cursor and width > 0
            cursor += width
        assert cursor == vocab
    assert shard_span(151_936, 8, 3) == (3 * 18_992, 18_992)


class OracleBackend:
    """Stand-in for the GPU steps, same interface as flash_gordon_b200.dist.CudaBackend."""

    def __init__(self):
        import oracle
        self.oracle = oracle
        self.lib = oracle.load("port")

    def shard_topk(self, logits, configs, vocab_offset, vocab_total, k_shard, history_tokens,
                   history_offsets, history_max):
        tokens = None if history_tokens is None else history_tokens.numpy().view(np.uint32)
        offsets = None if history_offsets is None else history_offsets.numpy().view(np.uint64)
        _, scores, ids, row_status = self.oracle.shard_topk(
            self.lib, logits.contiguous().numpy(), configs, vocab_offset, vocab_total, k_shard, tokens, offsets)
        return (torch.from_numpy(scores), torch.from_numpy(ids.view(np.int32)),
                torch.from_numpy(row_status.view(np.int32)))

    def merge_select(self, scores, ids, rows, shards, k_shard, first, width, configs, uniforms):
        from flash_gordon_b200.api import SampleResult
        status, tokens, logits, row_status, _ = self.oracle.merge_select(
            self.lib, scores.numpy(), ids.numpy().view(np.uint32), first, width, configs, uniforms.numpy())
        return SampleResult(torch.from_numpy(tokens.view(np.int32)), torch.from_numpy(logits),
                            torch.from_numpy(row_status.view(np.int32)), status, "")


def _worker(rank, world, port, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_gordon_b200 import SamplerConfig
        from helpers import random_workload, run_oracle
        cfg = SamplerConfig.make(temperature=0.8, top_p=0.9, top_k=30, presence=0.4, frequency=0.2,
                                 repetition=1.1)
        w = random_workload(7, 5001, 300, [cfg], 99, quantize=0.5, specials=2)
        want = run_oracle(w, threads=1)
        # vocabulary shards: every rank ends up with the unsharded answer
        first, width = shard_span(w.vocab, world, rank)
        out = sample_vocab_sharded(OracleBackend(), w.logits[:, first:first + width].contiguous(), w.configs,
                                   w.uniforms, w.vocab, 64, w.history_tokens, w.history_offsets, w.history_max)
        assert out.status == want[0], (out.status, want[0])
        assert np.array_equal(out.tokens.numpy().view(np.uint32), want[1])
        assert np.array_equal(out.token_logits.numpy().view(np.uint32), want[2].view(np.uint32))
        # row partition: each rank samples its block, the gather restores row order
        begin, end = row_block(w.rows, world, rank)
        mine = w.slice_rows(begin, end)
        part = run_oracle(mine, threads=1)
        tokens, logits, status = gather_rows(torch.from_numpy(part[1].view(np.int32)), torch.from_numpy(part[2]),
                                             torch.from_numpy(part[3].view(np.int32)))
        assert np.array_equal(tokens.numpy().view(np.uint32), want[1])
        assert np.array_equal(logits.numpy().view(np.uint32), want[2].view(np.uint32))
        assert np.array_equal(status.numpy().view(np.uint32), want[3])
    except Exception as error:  # surfaced by the parent
        failures.put(f"rank {rank}: {error!r}")
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_sharded_and_partitioned():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    failures = context.Queue()
    workers = [context.Process(target=_worker, args=(rank, 2, port, failures)) for rank in range(2)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=240)
        assert not worker.is_alive(), "a rank hung"
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    assert not problems, problems
    assert all(worker.exitcode == 0 for worker in workers)


def _no_show_worker(rank, world, port, outcomes):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    try:
        from flash_gordon_b200 import SamplerConfig
        from helpers import random_workload
        w = random_workload(3, 2000, 0, [SamplerConfig.make(0.8, 0.9, 20)], 3)
        first, width = shard_span(w.vocab, world, rank)
        if rank == 1:
            import time
            time.sleep(8)  # the rank that never calls the exchange
            outcomes.put((rank, "absent"))
            return
        out = sample_vocab_sharded(OracleBackend(), w.logits[:, first:first + width].contiguous(), w.configs,
                                   w.uniforms, w.vocab, 64)
        outcomes.put((rank, out.status, out.row_status.tolist(), out.message))
    except Exception as error:
        outcomes.put((rank, f"raised {error!r}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_never_joins_ends_the_step_with_the_limit_status():
    """Host-side fault: rank 1 never calls the exchange.  Rank 0 must come back within the
    group's timeout with FG_ERR_LIMIT on every row (the reference: a partial that misses its
    deadline, src/runtime.c:2379-2435) instead of waiting forever.  No GPU is involved."""
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    outcomes = context.Queue()
    workers = [context.Process(target=_no_show_worker, args=(rank, 2, port, outcomes)) for rank in range(2)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=120)
        assert not worker.is_alive(), "a rank hung"
    seen = {}
    while not outcomes.empty():
        item = outcomes.get()
        seen[item[0]] = item[1:]
    assert seen[1] == ("absent",)
    status, row_status, message = seen[0]
    assert status == 8 and set(row_status) == {8} and "joined" in message  # FG_ERR_LIMIT
