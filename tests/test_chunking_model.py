"""Invariants of the balanced kernel's work partition, on the host-side model of its arithmetic
(tests/chunking_model.py restates csrc/paged_decode_balanced.cuh `Chunking`)."""

import random

import pytest

from chunking_model import ChunkPlan, pairs_of
from single_gpu_inference_lab_b200.workloads import make_inputs


def lengths(case: str):
    rng = random.Random(5)
    if case == "uniform-long":
        return [rng.randint(512, 4096) for _ in range(64)], 2
    if case == "log-uniform":
        return [max(1, round(2 ** rng.uniform(0, 13))) for _ in range(256)], 4
    if case == "few-very-long":
        return [131072] * 4, 8
    if case == "tiny":
        return [1, 17, 33, 0, 5], 2
    if case == "with-empty":
        return [0, 700, 0, 0, 4000, 31, 0], 1
    raise KeyError(case)


@pytest.mark.parametrize("case", ["uniform-long", "log-uniform", "few-very-long", "tiny", "with-empty"])
@pytest.mark.parametrize("kv_start", [0, 48, 50])
def test_partition_invariants(case, kv_start):
    lens, hkv = lengths(case)
    plan = ChunkPlan(lens, hkv, kv_start=kv_start)
    total = plan.prefix[-1]
    # chunks tile the pair list without gap or overlap
    cursor = 0
    for c in range(plan.groups):
        lo, hi = plan.pair_range(c)
        assert lo == cursor and hi >= lo
        cursor = hi
    assert cursor == total
    # chunk_of inverts start_of
    for c in range(plan.groups):
        assert plan.chunk_of(plan.start_of(c)) == c
        if plan.start_of(c + 1) > plan.start_of(c):
            assert plan.chunk_of(plan.start_of(c + 1) - 1) == c
    # what the merge kernel derives per sequence is what the chunk kernel wrote
    slots = set()
    for b, n in enumerate(plan.pairs):
        pieces = plan.pieces_of(b)
        assert sum(p.last_pair - p.first_pair + 1 for p in pieces) == n
        for p, q in zip(pieces, pieces[1:]):
            assert q.first_pair == p.last_pair + 1 and q.group == p.group + 1
        for p in pieces:
            assert p.last_pair >= p.first_pair, "a chunk inside a sequence is never empty"
            if p.slot is not None:
                assert p.slot not in slots, "two pieces share a workspace slot"
                slots.add(p.slot)
        if len(pieces) == 1:
            assert pieces[0].slot is None  # finished by its warp, nothing for the merge kernel
    assert all(0 <= s < 2 * plan.groups for s in slots)


def test_cost_balance_on_the_batch_256_workload():
    w = make_inputs("qwen2.5-7b-b256", seed=0, device="cpu", shrink=1.0)
    hkv = w.key_cache.shape[2]
    plan = ChunkPlan(w.seq_lens.tolist(), hkv)
    assert plan.groups == 148 * 8 // hkv
    costs = [plan.start_of(c + 1) - plan.start_of(c) for c in range(plan.groups)]
    assert max(costs) - min(costs) <= 1
    # bytes differ more than cost does: groups that meet many short sequences stream fewer pairs
    pairs = [hi - lo for lo, hi in (plan.pair_range(c) for c in range(plan.groups))]
    assert max(pairs) <= plan.base // 2 + 1 and min(pairs) >= (plan.base - 2 * 40) // 2
    assert sum(pairs) == sum(pairs_of(int(n)) for n in w.seq_lens)
