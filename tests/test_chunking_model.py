"""Invariants of the balanced kernel's work partition, on the host-side model of its arithmetic
(tests/chunking_model.py restates csrc/paged_decode_balanced.cuh `Chunking` / `chunk_range`)."""

import random

import pytest

from chunking_model import ChunkPlan, pages_of, pairs_of
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
    # every page of every sequence is attended by exactly one chunk, in order
    seen = []
    for c in range(plan.groups):
        r = plan.chunk_range(c)
        assert r.end_pair >= r.first_pair
        got = plan.pages_of_chunk(c)
        assert got or r.end_pair == r.first_pair or plan.groups == 1 or all(n == 0 for n in plan.pages)
        seen += got
    expected = [(b, page) for b, n in enumerate(plan.pages) for page in range(n)]
    assert seen == expected
    # neighbouring chunks share a pair exactly when the boundary splits it
    for c in range(plan.groups - 1):
        a, b = plan.chunk_range(c), plan.chunk_range(c + 1)
        assert a.tail_split == b.head_split
        assert b.first_pair == a.end_pair - (1 if a.tail_split else 0)
    # chunk_of inverts start_of
    for c in range(plan.groups):
        assert plan.chunk_of(plan.start_of(c)) == c
        if plan.start_of(c + 1) > plan.start_of(c):
            assert plan.chunk_of(plan.start_of(c + 1) - 1) == c
    # what the merge derives per sequence is what the chunk kernel attended and wrote
    by_chunk = {c: plan.pages_of_chunk(c) for c in range(plan.groups)}
    slots = set()
    for b, n in enumerate(plan.pages):
        pieces = plan.pieces_of(b)
        assert sum(p.last_page - p.first_page + 1 for p in pieces) == n
        for p, q in zip(pieces, pieces[1:]):
            assert q.first_page == p.last_page + 1 and q.group == p.group + 1
        for p in pieces:
            assert p.last_page >= p.first_page, "a chunk inside a sequence is never empty"
            assert [page for (s, page) in by_chunk[p.group] if s == b] == list(range(p.first_page, p.last_page + 1))
            if p.slot is not None:
                assert p.slot not in slots, "two pieces share a workspace slot"
                slots.add(p.slot)
        if len(pieces) == 1:
            assert pieces[0].slot is None  # finished by its warp, nothing to merge
    assert all(0 <= s < 2 * plan.groups for s in slots)


def test_cost_balance_on_the_batch_256_workload():
    w = make_inputs("qwen2.5-7b-b256", seed=0, device="cpu", shrink=1.0)
    hkv = w.key_cache.shape[2]
    plan = ChunkPlan(w.seq_lens.tolist(), hkv)
    assert plan.groups == 148 * 8 // hkv
    costs = [plan.start_of(c + 1) - plan.start_of(c) for c in range(plan.groups)]
    assert max(costs) - min(costs) <= 1
    # bytes differ more than cost does: groups that meet many short sequences attend fewer pages
    pages = [len(plan.pages_of_chunk(c)) for c in range(plan.groups)]
    assert max(pages) <= plan.base + 1 and min(pages) >= plan.base - 2 * 40
    assert sum(pages) == sum(pages_of(int(n)) for n in w.seq_lens)
    assert plan.prefix[-1] == sum(pairs_of(int(n)) for n in w.seq_lens)


def test_page_balance_on_the_batch_64_workload():
    """With boundaries at page granularity no chunk of a batch of long sequences attends more than
    one page above the mean, and chunks differ only by what the sequence starts inside them cost."""
    w = make_inputs("qwen2.5-coder-3b-b64", seed=0, device="cpu")
    plan = ChunkPlan(w.seq_lens.tolist(), w.key_cache.shape[2])
    pages = [len(plan.pages_of_chunk(c)) for c in range(plan.groups)]
    assert max(pages) <= plan.base + 1
    assert max(pages) - min(pages) <= 2 * plan.piece_cost + 1
