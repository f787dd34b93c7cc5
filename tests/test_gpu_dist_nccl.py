"""Two ranks, two GPUs, NCCL: the vocabulary-sharded path with its one all-gather and the
row-partitioned path, each checked against the CPU oracle.  Skipped on a single-GPU box
(the same exchange logic runs on CPU ranks in test_cpu_dist.py)."""
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
        from flash_gordon_b200.dist import CudaBackend, gather_rows, row_block, sample_vocab_sharded, shard_span
        from helpers import run_oracle
        context = Context(rank)
        # config 4: bf16 columns split across the ranks, shard top-64, all-gather, merge
        w = synth.config4(rows=32)
        want = run_oracle(w, threads=4)
        first, width = shard_span(w.vocab, world, rank)
        mine = w.logits[:, first:first + width].contiguous().cuda()
        out = sample_vocab_sharded(CudaBackend(context), mine, w.configs, w.uniforms.cuda(), w.vocab, 64)
        torch.cuda.synchronize()
        assert out.status == want[0] == 0
        assert np.array_equal(out.tokens.cpu().numpy().view(np.uint32), want[1])
        assert np.array_equal(out.token_logits.cpu().numpy().view(np.uint32), want[2].view(np.uint32))
        # config 3 rows partitioned: no collective on the data path, results gathered afterwards
        w3 = synth.config3(rows=24, history=512)
        want3 = run_oracle(w3, threads=4)
        begin, end = row_block(w3.rows, world, rank)
        part = w3.slice_rows(begin, end).to("cuda")
        got = context.sample_batch(part.logits, part.configs, part.uniforms, part.history_tokens,
                                   part.history_offsets, part.history_max)
        tokens, logits, status = gather_rows(got.tokens, got.token_logits, got.row_status)
        assert np.array_equal(tokens.cpu().numpy().view(np.uint32), want3[1])
        assert np.array_equal(logits.cpu().numpy().view(np.uint32), want3[2].view(np.uint32))
        assert not status.any()
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
