"""world_size-2 run of the multi-GPU host logic on CPU (gloo): row sharding and
the vocabulary-sharded candidate exchange.  The kernels are replaced by the CPU
oracle here — this file checks ranges, record layout, the all-gather shape and
the merge rule, not the CUDA code."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def ordered_key(values):
    bits = (values.astype(np.float32) + np.float32(0.0)).view(np.uint32)
    return np.where(bits & 0x80000000, ~bits, bits | 0x80000000).astype(np.uint32)


def make_records(values, indices):
    """The 64-bit candidate record of include/moe_b200_sampler.h."""
    return (ordered_key(values).astype(np.uint64) << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - indices.astype(np.uint64))


def _worker(rank, world, port, rows, vocab, top_k, queue):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as graft
    from oracle import oracle as oracle_module

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    graft.load_package()
    parallel = __import__("ncnn_moe_runtime_b200.parallel", fromlist=["x"])
    oracle = oracle_module.port()
    rng = np.random.default_rng(1234)           # every rank builds the same full matrix, then keeps its part
    logits = np.round(rng.standard_normal((rows, vocab)).astype(np.float32) * 4) / 4
    uniforms = rng.random(rows).astype(np.float32)

    # --- vocabulary sharding: local stable Top-K records, all-gather, merge ---------
    begin, end = parallel.vocab_shard_range(vocab, world, rank)
    local = np.zeros((rows, top_k), dtype=np.uint64)
    for r in range(rows):
        order = oracle.topk_order(logits[r, begin:end], top_k)
        local[r, :order.size] = make_records(logits[r, begin:end][order], order.astype(np.int64) + begin)
    gathered = parallel.all_gather_candidates(torch.from_numpy(local.view(np.int64))).numpy().view(np.uint64)
    assert gathered.shape == (world, rows, top_k)
    merged_ids = []
    for r in range(rows):
        records = gathered[:, r, :].reshape(-1)
        records = np.sort(records[records != 0])[::-1][:top_k]     # larger record = earlier rank
        merged_ids.append((np.uint64(0xFFFFFFFF) - (records & np.uint64(0xFFFFFFFF))).astype(np.int64))
    expected_ids = [oracle.topk_order(logits[r], top_k).astype(np.int64) for r in range(rows)]
    ok_vocab = all(np.array_equal(a, b) for a, b in zip(merged_ids, expected_ids))

    # --- row sharding: no collective on the data path; results concatenate ----------
    row_begin, row_end = parallel.shard_range(rows, world, rank)
    mine = oracle.sample_batch(logits[row_begin:row_end], np.full(row_end - row_begin, 0.8, np.float32), np.full(row_end - row_begin, 20, np.uint32),
                               np.full(row_end - row_begin, 0.9, np.float32), np.zeros(row_end - row_begin, np.float32), uniforms[row_begin:row_end], threads=1)
    pieces = [None] * world
    dist.all_gather_object(pieces, (row_begin, mine["token"]))
    tokens = np.concatenate([p[1] for p in sorted(pieces, key=lambda p: p[0])])
    whole = oracle.sample_batch(logits, np.full(rows, 0.8, np.float32), np.full(rows, 20, np.uint32), np.full(rows, 0.9, np.float32),
                                np.zeros(rows, np.float32), uniforms, threads=1)
    ok_rows = np.array_equal(tokens, whole["token"])
    # --- a count every rank derives from its own clock is agreed before it is used ----
    ok_rows = ok_rows and parallel.agree_on_maximum(10 + 5 * rank) == 10 + 5 * (world - 1)
    queue.put((rank, ok_vocab, ok_rows))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_row_and_vocab_sharding():
    import torch.multiprocessing as mp

    context = mp.get_context("spawn")
    queue = context.Queue()
    port = _free_port()
    world = 2
    processes = [context.Process(target=_worker, args=(rank, world, port, 7, 3001, 24, queue)) for rank in range(world)]
    for process in processes:
        process.start()
    results = [queue.get(timeout=180) for _ in range(world)]
    for process in processes:
        process.join(timeout=60)
        assert process.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] and r[2] for r in results)
