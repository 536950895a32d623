"""Host logic of the two multi-GPU forms, on CPU: token-balanced sequence partition, page-pool
compaction, and the KV-range exchange (world_size-2 gloo ranks, oracle standing in for the kernels)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200 import sharding
from single_gpu_inference_lab_b200.workloads import make_inputs


def test_lpt_partition_balances_tokens():
    w = make_inputs("qwen2.5-7b-b256", seed=0, shrink=0.125)
    lens = w.seq_lens.tolist()
    for world in (1, 2, 4, 8):
        parts = sharding.lpt_partition(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(256))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.05 * sum(lens) / world + max(lens)


def test_shard_sequences_is_a_pure_relabelling():
    w = make_inputs("qwen2.5-7b-b256", seed=0, batch=32, shrink=0.05)
    full = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    seen = []
    for rank in range(4):
        local, rows = sharding.shard_sequences(w, rank, 4)
        seen += rows
        assert local.key_cache.shape[0] == sum(-(-int(n) // 16) for n in local.seq_lens)
        out = oracle.reference(
            local.query, local.key_cache, local.value_cache, local.block_table.long(), local.seq_lens, w.k_scale, w.v_scale
        )
        assert torch.equal(out.view(torch.int16), full[rows].view(torch.int16))
    assert sorted(seen) == list(range(32))


def test_kv_range_bounds_cover_the_sequence_once():
    for msl in (1, 16, 17, 4096, 131072, 1000):
        for world in (1, 2, 4, 8):
            covered = 0
            for r in range(world):
                lo, hi = sharding.kv_range_bounds(msl, r, world)
                assert lo % 16 == 0
                if hi > lo:
                    assert lo == covered
                    covered = hi
            assert covered >= msl


def _oracle_partial(local, split_size):
    o, m, l = oracle.split_partials(
        local.query, local.key_cache, local.value_cache, local.block_table.long(), local.seq_lens,
        local.k_scale, local.v_scale, split_size=max(local.max_seq_len, 16), num_splits=1,
    )
    return torch.cat([o[:, :, 0], m, l], dim=-1)


def _oracle_merge(gathered, like):
    return oracle.merge_packed(gathered)


def _worker(rank, world, port, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        w = make_inputs("llama3-8b-long-b4", seed=0, batch=3, shrink=1 / 128)
        lens = w.seq_lens.clone()
        lens[1] = 300  # ends inside rank 0's range: rank 1 holds nothing of it
        lens[2] = 777
        w.seq_lens = lens
        local = sharding.shard_kv_range(w, rank, world)
        out = sharding.kv_range_decode(local, partial_fn=_oracle_partial, merge_fn=_oracle_merge)
        ref = oracle.reference_fp32(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
        result_queue.put((rank, float((out - ref).abs().max()), int(local.seq_lens.sum())))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_kv_range_exchange_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=100) for _ in procs)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert [r[0] for r in results] == [0, 1]
    for _, err, _ in results:
        assert err < 1e-5
    assert results[0][2] + results[1][2] == 1024 + 300 + 777
