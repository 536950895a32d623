"""KV-range exchange inside the kernels, on ONE GPU: the ranks' objects live in one process and
their calls are issued one after another on one stream, so every flag a merge kernel looks at
was released by a kernel that has already completed (nothing spins on a running kernel).  The
decode kernels store their packed rows into every "rank's" receive buffer and release the step's
flags; the exchange merge kernel checks the flags and merges.  Held against the CPU oracle.

The expiry case: a rank that is not asked to store never releases its flag; the other ranks'
merge kernels give up after the wait limit, set device status 4 and leave their output alone, and
the next complete step is right again.
"""

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import make_inputs
from helpers import assert_within_gate

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
EARLY = 32


def _workspace(local, split):
    from single_gpu_inference_lab_b200 import l20_paged_split_kv as m

    return m.allocate_l20_paged_split_kv_workspace(local.query, max(local.max_seq_len, 1), split_size=split)


def _setup(world, name, **kw):
    from single_gpu_inference_lab_b200 import sharding

    w = make_inputs(name, **kw)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    locals_ = [sharding.shard_kv_range(w, r, world).to(DEV) for r in range(world)]
    b, hq, d = w.query.shape
    ranks = sharding.KvRangeExchange.emulate(world, b, hq, d, DEV)
    return w, exp, locals_, ranks


@pytest.mark.parametrize("world,flags,planned", [(1, 0, False), (2, 0, False), (2, EARLY, True), (3, EARLY, False), (8, 0, True)])
def test_exchange_matches_oracle_over_several_steps(built_libs, world, flags, planned):
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    w, exp, locals_, ranks = _setup(world, "llama3-8b-long-b4", seed=3, batch=3, shrink=1 / 32)
    split = 256
    wss = [_workspace(l, split) for l in locals_]
    plans = [
        cabi.plan_decode(l.query, l.key_cache, l.value_cache, l.block_table, l.seq_lens, max_seq_len=l.max_seq_len,
                         split_size=split, workspace=ws) if planned else None
        for l, ws in zip(locals_, wss)
    ]
    try:
        for step in range(4):  # both halves of the buffers twice, the row counter reset three times
            outs = [torch.full_like(l.query, float("nan")) for l in locals_]
            for x, l, ws, plan in zip(ranks, locals_, wss, plans):
                x.decode(l, split_size=split, workspace=ws, plan=plan, flags=flags)
            for x, o in zip(ranks, outs):
                x.merge(o)
            assert cabi.device_status() == 0
            for r, o in enumerate(outs):
                assert_within_gate(o, exp, f"world {world} step {step} rank {r}")
                assert torch.equal(o, outs[0]), "every rank merges the same records"
    finally:
        for x in ranks:
            x.close()


def test_exchange_with_uneven_lengths_and_empty_ranges(built_libs):
    """Sequences that end before a rank's range begins give that rank empty rows (m = -inf), which
    it still has to publish; a batch large enough for several chunks per sequence and for the
    merge kernel's rows as well."""
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    world = 4
    w = make_inputs("qwen2.5-coder-3b-b64", seed=5, batch=12, shrink=0.5)
    lens = w.seq_lens.clone()
    lens[0] = 1
    lens[1] = 17
    lens[5] = 130
    w.seq_lens = lens
    from single_gpu_inference_lab_b200 import sharding

    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    locals_ = [sharding.shard_kv_range(w, r, world).to(DEV) for r in range(world)]
    b, hq, d = w.query.shape
    ranks = sharding.KvRangeExchange.emulate(world, b, hq, d, DEV)
    try:
        for step in range(3):
            outs = [torch.full_like(l.query, float("nan")) for l in locals_]
            for x, l in zip(ranks, locals_):
                x.decode(l, split_size=128, workspace=_workspace(l, 128), flags=EARLY)
            for x, o in zip(ranks, outs):
                x.merge(o)
            assert cabi.device_status() == 0
            for r, o in enumerate(outs):
                assert_within_gate(o, exp, f"step {step} rank {r}")
    finally:
        for x in ranks:
            x.close()


def test_exchange_steps_replayed_from_a_cuda_graph(built_libs):
    """The step's tag is device-resident: one captured step (every rank's decode, every rank's
    merge) is right on every replay, fresh KV each time."""
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    w, exp, locals_, ranks = _setup(2, "llama3-8b-long-b4", seed=6, batch=2, shrink=1 / 32)
    split = 256
    wss = [_workspace(l, split) for l in locals_]
    outs = [torch.empty_like(l.query) for l in locals_]
    try:
        def one_step():
            for x, l, ws in zip(ranks, locals_, wss):
                x.decode(l, split_size=split, workspace=ws, flags=EARLY)
            for x, o in zip(ranks, outs):
                x.merge(o)

        one_step()  # an odd number of eager steps first: replays then begin on the other half
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side), torch.cuda.graph(g, stream=side):
            one_step()
            one_step()
            one_step()
        for replay in range(4):
            for o in outs:
                o.fill_(float("nan"))
            g.replay()
            torch.cuda.synchronize()
            assert cabi.device_status() == 0
            for r, o in enumerate(outs):
                assert_within_gate(o, exp, f"replay {replay} rank {r}")
    finally:
        for x in ranks:
            x.close()


def test_exchange_refusals(built_libs):
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    w, exp, locals_, ranks = _setup(2, "qwen2.5-coder-3b-b64", seed=2, batch=4, shrink=0.1)
    l, x = locals_[0], ranks[0]
    ws = _workspace(l, 128)
    common = dict(k_scale=l.k_scale, v_scale=l.v_scale, max_seq_len=l.max_seq_len, split_size=128, workspace=ws)
    try:
        broken = cabi.Exchange.from_buffer_copy(x.struct)
        broken.control = None
        with pytest.raises(RuntimeError, match="control words"):
            cabi.paged_decode_fp8_e4m3_split_out(l.query, l.key_cache, l.value_cache, l.block_table, l.seq_lens, exchange=broken, **common)
        with pytest.raises(RuntimeError, match="exchange: needs the balanced kernel"):
            cabi.paged_decode_fp8_e4m3_split_out(l.query, l.key_cache, l.value_cache, l.block_table, l.seq_lens, exchange=x.struct,
                                                 flags=cabi.PFD_FLAG_FIXED_SPLITS, **common)
        with pytest.raises(RuntimeError, match="allocation-free"):
            cabi.paged_decode_fp8_e4m3_split_out_noalloc(l.query, l.key_cache, l.value_cache, l.block_table, l.seq_lens,
                                                         exchange=x.struct, output=torch.empty_like(l.query), **common)
        assert cabi.device_status() == 0
    finally:
        for r in ranks:
            r.close()


def test_a_rank_that_does_not_publish_ends_the_wait_with_a_status(built_libs):
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    w, exp, locals_, ranks = _setup(2, "llama3-8b-long-b4", seed=4, batch=2, shrink=1 / 32)
    split = 256
    wss = [_workspace(l, split) for l in locals_]

    def step(skip=None):
        outs = [torch.full_like(l.query, 7.0) for l in locals_]
        for r, (x, l, ws) in enumerate(zip(ranks, locals_, wss)):
            if r != skip:
                x.decode(l, split_size=split, workspace=ws)
        for x, o in zip(ranks, outs):
            x.merge(o)  # every rank, or the ranks' step counts part
        return outs

    try:
        outs = step()
        assert cabi.device_status() == 0
        assert_within_gate(outs[0], exp, "before")
        cabi.set_wait_limit_ns(2_000_000)  # 2 ms
        try:
            outs = step(skip=1)  # rank 1 is not asked to store: its flag never arrives
            assert cabi.device_status() == 4
            assert all(bool((o == 7.0).all()) for o in outs), "nothing is merged when a flag is missing"
            assert cabi.device_status() == 0, "reading the status clears it"
        finally:
            cabi.set_wait_limit_ns(200_000_000)  # the library's default
        outs = step()  # the context is still usable and the next complete step is right
        assert cabi.device_status() == 0
        for o in outs:
            assert_within_gate(o, exp, "after")
    finally:
        for x in ranks:
            x.close()


@pytest.mark.parametrize("seed", range(6))
def test_exchange_on_random_batches(built_libs, seed):
    """Random worlds, batches, head geometries and lengths (some shorter than a rank's range start),
    plan and early-metadata flag at random; three steps each."""
    from single_gpu_inference_lab_b200 import cabi, sharding

    cabi.load()
    gen = torch.Generator().manual_seed(900 + seed)
    world = [2, 3, 4, 5, 7, 8][seed]
    name = ["qwen2.5-coder-3b-b64", "qwen2.5-7b-b256", "llama3-8b-long-b4"][seed % 3]
    batch = int(torch.randint(1, 20, (1,), generator=gen))
    w = make_inputs(name, seed=seed, batch=batch, shrink=[0.3, 0.1, 1 / 64][seed % 3])
    lens = w.seq_lens.clone()
    for i in range(0, batch, 3):
        lens[i] = int(torch.randint(1, int(w.max_seq_len) + 1, (1,), generator=gen))
    w.seq_lens = lens
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    locals_ = [sharding.shard_kv_range(w, r, world).to(DEV) for r in range(world)]
    b, hq, d = w.query.shape
    ranks = sharding.KvRangeExchange.emulate(world, b, hq, d, DEV)
    split = 128
    flags = EARLY if seed % 2 else 0
    try:
        wss = [_workspace(l, split) for l in locals_]
        plans = [cabi.plan_decode(l.query, l.key_cache, l.value_cache, l.block_table, l.seq_lens, max_seq_len=l.max_seq_len,
                                  split_size=split, workspace=ws) if seed % 3 == 0 else None for l, ws in zip(locals_, wss)]
        for step in range(3):
            outs = [torch.full_like(l.query, float("nan")) for l in locals_]
            for x, l, ws, plan in zip(ranks, locals_, wss, plans):
                x.decode(l, split_size=split, workspace=ws, plan=plan, flags=flags)
            for x, o in zip(ranks, outs):
                x.merge(o)
            assert cabi.device_status() == 0
            for r, o in enumerate(outs):
                assert_within_gate(o, exp, f"seed {seed} world {world} step {step} rank {r}")
    finally:
        for x in ranks:
            x.close()
