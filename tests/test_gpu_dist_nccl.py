"""The library's own multi-GPU layer (fg_dist_*: an NCCL communicator behind the C ABI).
One rank on one GPU exercises the whole sharded call -- shard top-k written as pairs,
all-gather, merge over the gathered layout -- on any box.  Two ranks on two GPUs run the
vocabulary-sharded path with its one all-gather and the row-partitioned path, each checked
against the CPU oracle (skipped on a single-GPU box; the same exchange logic also runs on
CPU ranks in test_cpu_dist.py)."""
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

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flash_gordon_b200 import Context, synth
        from flash_gordon_b200.dist import Communicator, row_block, shard_span
        from helpers import run_oracle
        context = Context(rank)
        communicator = Communicator(context)
        # config 4: bf16 columns split across the ranks, shard top-64, all-gather, merge
        w = synth.config4(rows=32)
        want = run_oracle(w, threads=4)
        first, width = shard_span(w.vocab, world, rank)
        mine = w.logits[:, first:first + width].contiguous().cuda()
        out = communicator.sample_vocab_sharded(mine, w.configs, w.uniforms.cuda(), w.vocab, 64)
        torch.cuda.synchronize()
        assert out.status == want[0] == 0, out.message
        assert np.array_equal(out.tokens.cpu().numpy().view(np.uint32), want[1])
        assert np.array_equal(out.token_logits.cpu().numpy().view(np.uint32), want[2].view(np.uint32))
        # the same with the exchange fused into the kernels (stores into the peers' windows), three
        # times over so that both halves of the windows and a second use of one are exercised
        for attempt in range(3):
            fused = communicator.sample_vocab_sharded(mine, w.configs, w.uniforms.cuda(), w.vocab, 64, fused=True)
            assert fused.status == 0, fused.message
            assert np.array_equal(fused.tokens.cpu().numpy().view(np.uint32), want[1]), attempt
            assert np.array_equal(fused.token_logits.cpu().numpy().view(np.uint32), want[2].view(np.uint32))
        # with penalties and a history: ids are global, every shard filters the history to its span
        w2 = synth.config2(rows=16, history=256)
        want2 = run_oracle(w2, threads=4)
        mine2 = w2.logits[:, first:first + width].contiguous().cuda()
        out2 = communicator.sample_vocab_sharded(mine2, w2.configs, w2.uniforms.cuda(), w2.vocab, 64,
                                                 w2.history_tokens.cuda(), w2.history_offsets.cuda(),
                                                 w2.history_max)
        assert out2.status == 0, out2.message
        assert np.array_equal(out2.tokens.cpu().numpy().view(np.uint32), want2[1])
        # config 3 rows partitioned: no collective on the data path, results gathered afterwards
        w3 = synth.config3(rows=24, history=512)
        want3 = run_oracle(w3, threads=4)
        begin, end = row_block(w3.rows, world, rank)
        part = w3.slice_rows(begin, end).to("cuda")
        got = context.sample_batch(part.logits, part.configs, part.uniforms, part.history_tokens,
                                   part.history_offsets, part.history_max)
        tokens, logits, status = communicator.gather_rows(got.tokens, got.token_logits, got.row_status)
        assert np.array_equal(tokens.cpu().numpy().view(np.uint32), want3[1])
        assert np.array_equal(logits.cpu().numpy().view(np.uint32), want3[2].view(np.uint32))
        assert not status.any()
        communicator.close()
        context.close()
    except Exception as error:
        failures.put(f"rank {rank}: {error!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_sharded_and_partitioned():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    failures = context.Queue()
    workers = [context.Process(target=_worker, args=(rank, 2, port, failures)) for rank in range(2)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=600)
        assert not worker.is_alive(), "a rank hung"
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    assert not problems, problems
    assert all(worker.exitcode == 0 for worker in workers)


def test_one_rank_runs_the_whole_sharded_call(context):
    """ranks = 1: the shard is the whole vocabulary; the call still writes pairs, goes through
    ncclAllGather on a one-rank communicator and merges the gathered layout."""
    from flash_gordon_b200 import FG_OK, SamplerConfig, synth
    from flash_gordon_b200.dist import Communicator
    from helpers import assert_rows_equal, random_workload, run_oracle
    communicator = Communicator(context, ranks=1)
    try:
        for w in (synth.config4(rows=20, vocab=30_000),
                  random_workload(12, 20_000, 400, [SamplerConfig.make(0.8, 0.9, 40, presence=0.3,
                                                                       frequency=0.2, repetition=1.1)], 5,
                                  quantize=0.25, specials=2),
                  random_workload(7, 9_000, 0, [SamplerConfig.make(0.0, 1.0, 1)], 6, specials=1)):
            wd = w.to("cuda")
            result = communicator.sample_vocab_sharded(wd.logits, wd.configs, wd.uniforms, w.vocab, 64,
                                                       wd.history_tokens, wd.history_offsets, wd.history_max)
            torch.cuda.synchronize()
            want = run_oracle(w)
            # (a greedy row with a NaN/Inf is rejected as the split head does: MISMATCH, as unsharded)
            assert_rows_equal(result, want, w.name)
            # and with the exchange fused into the two kernels: the shard kernel stores into the
            # (one) rank's window and counts itself in, the merge kernel waits for the counters
            for attempt in range(3):
                fused = communicator.sample_vocab_sharded(wd.logits, wd.configs, wd.uniforms, w.vocab, 64,
                                                          wd.history_tokens, wd.history_offsets, wd.history_max,
                                                          fused=True)
                torch.cuda.synchronize()
                assert_rows_equal(fused, want, f"{w.name}, fused exchange, call {attempt}")
        # the prepared form (argument block built once, asynchronous calls back to back), both ways
        w = synth.config4(rows=24, vocab=40_000)
        wd = w.to("cuda")
        want = run_oracle(w)
        out = (torch.empty(24, dtype=torch.int32, device="cuda"), torch.empty(24, dtype=torch.float32, device="cuda"),
               torch.empty(24, dtype=torch.int32, device="cuda"))
        for fused in (False, True):
            issue = communicator.prepared_sample_vocab_sharded(wd.logits, wd.configs, wd.uniforms, w.vocab, 64, out,
                                                               fused=fused)
            for _ in range(4):
                out[0].fill_(-7)
                assert issue() == FG_OK
            torch.cuda.synchronize()
            assert np.array_equal(out[0].cpu().numpy().view(np.uint32), want[1]), fused
            assert np.array_equal(out[1].cpu().numpy().view(np.uint32), want[2].view(np.uint32)), fused
            assert int(out[2].max()) == 0
        wd = synth.config4(rows=4, vocab=8_000).to("cuda")
        short = communicator.sample_vocab_sharded(wd.logits[:, :4000].contiguous(), wd.configs, wd.uniforms,
                                                  8_000, 64)
        assert short.status != FG_OK and "span" in short.message  # the rank's columns must be its span
    finally:
        communicator.close()
