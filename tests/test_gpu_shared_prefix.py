"""Shared-prefix decode (dense tcgen05 prefix pass + split-KV suffix pass + merge) against the
CPU oracle, through the C ABI.  The oracle needs no notion of a shared prefix: it is only a
property of the block tables (every row names the same prefix pages)."""

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import make_inputs

from helpers import assert_within_gate

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def cabi(built_libs):
    from single_gpu_inference_lab_b200 import cabi as module

    module.load()
    return module


def run_shared(cabi, w, split, query=None):
    g = w.to(DEV)
    q = g.query if query is None else query.to(DEV)
    chunks = -(-w.prefix_len // 256)
    slots = chunks + max(1, -(-(w.max_seq_len - w.prefix_len) // split))
    b, hq, d = q.shape
    ws = (
        torch.full((b, hq, slots, d), float("nan"), device=DEV),
        torch.full((b, hq, slots), float("nan"), device=DEV),
        torch.full((b, hq, slots), float("nan"), device=DEV),
    )
    out = torch.full_like(q, float("nan"))
    cabi.shared_prefix_decode_fp8_e4m3(
        q, g.key_cache, g.value_cache, g.block_table, g.seq_lens, prefix_len=w.prefix_len,
        k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=w.max_seq_len, split_size=split, output=out, workspace=ws,
    )
    torch.cuda.synchronize()
    assert cabi.device_status() == 0, "a bounded device-side wait gave up"
    return out, ws, chunks


@pytest.mark.parametrize("batch,shrink", [(8, 0.125), (20, 0.25), (64, 1.0)])
def test_shared_prefix_decode_matches_oracle(cabi, batch, shrink):
    w = make_inputs("shared-prefix-b64", seed=0, batch=batch, shrink=shrink)
    # the grouping the dispatch relies on: one group spanning the batch
    groups = oracle.find_shared_prefix_groups(w.block_table, [w.prefix_len] * batch, min_batch=1, min_prefix_length=16)
    assert groups == [list(range(batch))]
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    for split in (128, 512):
        out, _, _ = run_shared(cabi, w, split)
        assert_within_gate(out, exp, f"batch={batch} shrink={shrink} split={split}")


def test_prefix_chunks_match_oracle_partials(cabi):
    """Slots [0, chunks) of the workspace hold (o, m, l) of 256-token prefix chunks."""
    w = make_inputs("shared-prefix-b64", seed=3, batch=10, shrink=0.25)  # prefix 1024 = 4 chunks
    out, ws, chunks = run_shared(cabi, w, 256)
    head = make_inputs("shared-prefix-b64", seed=3, batch=10, shrink=0.25)
    head.seq_lens = torch.full_like(head.seq_lens, w.prefix_len)
    o, m, l = oracle.split_partials(
        head.query, head.key_cache, head.value_cache, head.block_table.long(), head.seq_lens, head.k_scale, head.v_scale,
        split_size=256, num_splits=chunks,
    )
    po, pm, ps = (t[:, :, :chunks].cpu() for t in ws)
    assert torch.allclose(pm, m, atol=2e-3, rtol=1e-3)
    c = torch.exp(pm - m)
    assert torch.allclose(ps * c, l, atol=1e-2, rtol=5e-3)
    assert torch.allclose(po * c[..., None], o, atol=2e-2, rtol=1e-2)


def test_requests_without_suffix_and_fp16_query(cabi):
    w = make_inputs("shared-prefix-b64", seed=5, batch=12, shrink=0.125)
    lens = w.seq_lens.clone()
    lens[::3] = w.prefix_len  # every third request has no private suffix at all
    w.seq_lens = lens
    w.max_seq_len = int(lens.max())
    q16 = w.query.to(torch.float16)
    exp = oracle.reference(q16, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    out, _, _ = run_shared(cabi, w, 128, query=q16)
    assert_within_gate(out, exp, "fp16, some empty suffixes")


def test_shared_prefix_argument_checks(cabi):
    w = make_inputs("shared-prefix-b64", seed=0, batch=8, shrink=0.125).to(DEV)
    out = torch.empty_like(w.query)
    ws = (torch.empty(8, 16, 1, 128, device=DEV), torch.empty(8, 16, 1, device=DEV), torch.empty(8, 16, 1, device=DEV))
    common = dict(k_scale=w.k_scale, v_scale=w.v_scale, max_seq_len=w.max_seq_len, split_size=128, output=out, workspace=ws)
    before = cabi.launch_count()
    with pytest.raises(RuntimeError, match="needs .* slots"):
        cabi.shared_prefix_decode_fp8_e4m3(w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens, prefix_len=w.prefix_len, **common)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        cabi.shared_prefix_decode_fp8_e4m3(w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens, prefix_len=100, **common)
    assert cabi.launch_count() == before


def test_dispatch_module_end_to_end(built_libs, monkeypatch):
    """The reference-shaped entry: gate (env switch, one group spanning the batch) + op + trace."""
    from single_gpu_inference_lab_b200 import l20_shared_prefix_decode_dispatch as d

    w = make_inputs("shared-prefix-b64", seed=2, batch=16, shrink=0.25)  # prefix 1024
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    prefix = [w.prefix_len] * 16
    monkeypatch.delenv("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", raising=False)
    assert d.maybe_l20_shared_prefix_paged_decode(
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, prefix, k_scale=g.k_scale, v_scale=g.v_scale) is None
    monkeypatch.setenv("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", "1")
    # default gate wants prefix >= 4096: this batch's prefix is 1024
    assert not d.should_dispatch_l20_shared_prefix_paged_decode(g.query, g.key_cache, g.block_table, prefix)
    assert d.should_dispatch_l20_shared_prefix_paged_decode(g.query, g.key_cache, g.block_table, prefix, min_prefix_length=1024)
    out = d.shared_paged_prefix_paged_suffix_gqa_decode_attention_fp8(
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, w.prefix_len,
        k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=w.max_seq_len, suffix_split_size=128)
    torch.cuda.synchronize()
    assert_within_gate(out, exp, "dispatch module")
    # a batch whose rows do not share the chain is refused by the gate
    other = g.block_table.clone()
    other[5, 0] = other[6, 1]
    assert not d.should_dispatch_l20_shared_prefix_paged_decode(g.query, g.key_cache, other, prefix, min_prefix_length=1024)


def _random_grouped_table(gen, batch, cols, n_groups, prefix_pages, loners):
    """A block table in which `n_groups` sets of rows share their first pages (each set its own
    chain and prefix length), `loners` rows share nothing, and everything is shuffled."""
    table = torch.randint(0, 1 << 20, (batch, cols), generator=gen, dtype=torch.int32)
    lengths = torch.zeros(batch, dtype=torch.int32)
    order = torch.randperm(batch, generator=gen).tolist()
    free = order[loners:]
    per = len(free) // max(n_groups, 1)
    for g in range(n_groups):
        rows = free[g * per:(g + 1) * per] if g < n_groups - 1 else free[g * per:]
        pages = prefix_pages[g % len(prefix_pages)]
        chain = torch.randint(0, 1 << 20, (pages,), generator=gen, dtype=torch.int32)
        for r in rows:
            table[r, :pages] = chain
            lengths[r] = pages * 16
    for r in order[:loners]:
        lengths[r] = prefix_pages[0] * 16  # same length as a group, different chain
    return table, lengths


@pytest.mark.parametrize("seed", range(6))
def test_device_grouping_equals_the_oracle_on_random_tables(built_libs, seed):
    from single_gpu_inference_lab_b200 import l20_paged_decode as ops

    gen = torch.Generator().manual_seed(100 + seed)
    batch = [8, 37, 64, 200, 513, 2048][seed]
    cols = [40, 64, 300, 128, 96, 48][seed]
    n_groups = [1, 3, 4, 7, 20, 60][seed]
    pages = [[8], [4, 9, 30], [256, 17], [64], [5, 6, 7, 90], [16, 33]][seed]
    table, lengths = _random_grouped_table(gen, batch, cols, n_groups, pages, loners=batch // 5)
    if seed == 2:  # near misses: one block of the chain differs, at its start, middle and end
        grouped = [r for r in range(batch) if lengths[r] == 256 * 16][:3]
        for r, col in zip(grouped, (0, 128, 255)):
            table[r, col] += 1
    if seed == 3:  # the same chain under two prefix lengths is two groups
        same = [r for r in range(batch) if lengths[r] > 0][:40]
        for r in same[:20]:
            table[r] = table[same[0]]
            lengths[r] = 64 * 16
        for r in same[20:]:
            table[r] = table[same[0]]
            lengths[r] = 32 * 16
    for min_batch, min_prefix in ((1, 16), (2, 64), (8, 16), (8, 4096)):
        want = oracle.find_shared_prefix_groups(table, lengths, min_batch=min_batch, min_prefix_length=min_prefix)
        found = ops.group_shared_prefixes(table.to(DEV), prefix_lengths=lengths.to(DEV), min_batch=min_batch,
                                          min_prefix_len=min_prefix, max_groups=batch)
        torch.cuda.synchronize()
        assert found.to_lists() == want, (seed, min_batch, min_prefix)
        row_group = found.row_group.cpu().tolist()
        row_prefix = found.row_prefix_len.cpu().tolist()
        for gi, rows in enumerate(want):
            assert all(row_group[r] == gi and row_prefix[r] == int(lengths[r]) for r in rows)
        in_groups = {r for rows in want for r in rows}
        assert all(row_group[r] == -1 and row_prefix[r] == 0 for r in range(batch) if r not in in_groups)


def test_device_grouping_discovers_the_prefixes_and_caps_the_groups(built_libs):
    from single_gpu_inference_lab_b200 import l20_paged_decode as ops
    from single_gpu_inference_lab_b200 import l20_shared_prefix_decode_dispatch as d

    w = make_inputs("shared-prefix-b64", seed=4, batch=24, shrink=0.25)  # prefix 1024, private suffixes of 0..8 pages
    g = w.to(DEV)
    # discovery: keyed on the first 512 tokens' pages, extended as far as every member agrees
    found = ops.group_shared_prefixes(g.block_table, seq_lens=g.seq_lens, min_batch=8, min_prefix_len=512)
    assert found.to_lists() == [list(range(24))]
    assert found.group_prefix_len.cpu().tolist()[0] == 1024
    assert found.row_prefix_len.cpu().tolist() == [1024] * 24
    # a member that leaves the common chain early shortens the group's prefix to where it leaves
    table = w.block_table.clone()
    table[5, 40] += 3  # page 40 = tokens 640..655
    found = ops.group_shared_prefixes(table.to(DEV), seq_lens=g.seq_lens, min_batch=8, min_prefix_len=512)
    assert found.to_lists() == [list(range(24))] and found.group_prefix_len.cpu().tolist()[0] == 640
    # ... and one that differs inside the key pages is no member
    table[7, 3] += 1
    found = ops.group_shared_prefixes(table.to(DEV), seq_lens=g.seq_lens, min_batch=8, min_prefix_len=512)
    assert found.to_lists() == [[r for r in range(24) if r != 7]] and found.row_group.cpu().tolist()[7] == -1
    # a short member bounds the prefix by the whole pages it has filled
    lens = g.seq_lens.clone()
    lens[2] = 700
    found = ops.group_shared_prefixes(g.block_table, seq_lens=lens, min_batch=8, min_prefix_len=512)
    assert found.group_prefix_len.cpu().tolist()[0] == 688
    uniform = ops.group_shared_prefixes(g.block_table, uniform_prefix_len=w.prefix_len, min_batch=8, min_prefix_len=512)
    assert uniform.to_lists() == [list(range(24))]
    # the list-returning mirror of the reference function runs the same kernels for a CUDA table
    assert d.find_l20_shared_prefix_groups(g.block_table, [w.prefix_len] * 24, min_batch=8, min_prefix_length=512) == [list(range(24))]
    # capacity: with room for one group only the first (by first member) comes out
    table = w.block_table.clone()
    table[12:, 0] += 7  # rows 12.. form a second group
    both = oracle.find_shared_prefix_groups(table, [w.prefix_len] * 24, min_batch=8, min_prefix_length=512)
    assert len(both) == 2
    capped = ops.group_shared_prefixes(table.to(DEV), uniform_prefix_len=w.prefix_len, min_batch=8, min_prefix_len=512, max_groups=1)
    assert capped.to_lists() == both[:1]
    assert capped.row_group.cpu().tolist()[12:] == [-1] * 12


def _mixed_batch(seed, prefix_a, prefix_b):
    """24 requests: rows 0-9 share a prefix of `prefix_a` tokens, rows 10-17 another of `prefix_b`
    tokens in other pages, rows 18-23 share nothing."""
    w = make_inputs("shared-prefix-b64", seed=seed, batch=24, shrink=0.25)  # every row: the same 1024-token prefix
    gen = torch.Generator().manual_seed(seed)
    table = w.block_table.clone()
    pages = w.key_cache.shape[0]
    chain_b = torch.randperm(pages, generator=gen)[: -(-prefix_b // 16)].to(torch.int32)
    for r in range(10, 18):
        table[r, : chain_b.numel()] = chain_b
    for r in range(18, 24):
        table[r, :64] = torch.randperm(pages, generator=gen)[:64].to(torch.int32)
    lengths = torch.tensor([prefix_a] * 10 + [prefix_b] * 8 + [prefix_a] * 6, dtype=torch.int32)
    w.block_table = table
    w.seq_lens = torch.maximum(w.seq_lens, lengths + 1)
    w.max_seq_len = int(w.seq_lens.max())
    return w, lengths


@pytest.mark.parametrize("prefix_a,prefix_b,bound,min_batch", [
    (1024, 512, None, 8),     # two groups + six requests in none
    (1024, 528, None, 8),     # a prefix that ends inside a 256-token chunk
    (1000, 520, None, 8),     # lengths that are no multiple of 16: used up to the page boundary
    (1024, 512, 768, 8),      # a bound below the longer prefix: the rest goes through the split-KV pass
    (1024, 512, None, 16),    # no group is large enough: everything through the split-KV pass
    (1024, 512, 0, 8),        # a bound of zero: no dense pass at all
])
def test_grouped_decode_of_a_mixed_batch_matches_the_oracle(cabi, prefix_a, prefix_b, bound, min_batch):
    w, lengths = _mixed_batch(11, prefix_a, prefix_b)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    groups, max_groups = cabi.group_shared_prefixes(g.block_table, prefix_lengths=lengths.to(DEV), min_batch=min_batch, min_prefix_len=256)
    split = 128
    cap = w.max_seq_len if bound is None else min(bound, w.max_seq_len)
    slots = -(-cap // 256) + -(-w.max_seq_len // split)
    b, hq, d = g.query.shape
    ws = (
        torch.full((b, hq, slots, d), float("nan"), device=DEV),
        torch.full((b, hq, slots), float("nan"), device=DEV),
        torch.full((b, hq, slots), float("nan"), device=DEV),
    )
    for step in range(2):  # the same groups buffer serves every layer of a model step
        out = torch.full_like(g.query, float("nan"))
        cabi.shared_prefix_decode_grouped_fp8_e4m3(
            g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, groups=groups, max_groups=max_groups,
            max_prefix_len=bound, k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=w.max_seq_len, split_size=split,
            output=out, workspace=ws)
        torch.cuda.synchronize()
        assert cabi.device_status() == 0
        assert_within_gate(out, exp, f"grouped decode step {step}")


def test_grouped_decode_through_the_dispatcher_and_its_workspace_check(built_libs):
    from single_gpu_inference_lab_b200 import l20_paged_decode as ops

    w, lengths = _mixed_batch(12, 1024, 512)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    found = ops.group_shared_prefixes(g.block_table, prefix_lengths=lengths.to(DEV), min_batch=8, min_prefix_len=256)
    assert found.to_lists() == [list(range(10)), list(range(10, 18))]
    b, hq, d = g.query.shape
    slots = -(-w.max_seq_len // 256) + -(-w.max_seq_len // 128)
    ws = (torch.empty(b, hq, slots, d, device=DEV), torch.empty(b, hq, slots, device=DEV), torch.empty(b, hq, slots, device=DEV))
    out = torch.empty_like(g.query)
    ops.shared_prefix_decode_grouped_fp8_e4m3(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, *ws, out,
                                              g.k_scale, g.v_scale, w.max_seq_len, 128, found)
    torch.cuda.synchronize()
    assert_within_gate(out, exp, "grouped decode through torch.ops")
    small = tuple(t[:, :, : slots - 1].contiguous() for t in ws)
    with pytest.raises(RuntimeError, match="needs"):
        ops.shared_prefix_decode_grouped_fp8_e4m3(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, *small, out,
                                                  g.k_scale, g.v_scale, w.max_seq_len, 128, found)


@pytest.mark.parametrize("seed", range(8))
def test_grouped_decode_on_random_batches_matches_the_oracle(cabi, seed):
    """Random batches: 1-4 groups of random sizes and prefix lengths (discovered on the device from
    the table and the lengths), requests in no group, random suffixes, both head geometries."""
    gen = torch.Generator().manual_seed(500 + seed)
    hq, hkv = [(16, 2), (28, 4), (8, 8), (32, 8)][seed % 4]
    batch = int(torch.randint(9, 70, (1,), generator=gen))
    n_groups = int(torch.randint(1, 5, (1,), generator=gen))
    pages = 4096
    d = 128
    key = torch.randn(pages, 16, hkv, d, generator=gen)
    value = torch.randn(pages, 16, hkv, d, generator=gen)
    from single_gpu_inference_lab_b200.workloads import quantize_per_head

    kc, ks = quantize_per_head(key)
    vc, vs = quantize_per_head(value)
    cols = 80
    table = torch.randint(0, pages, (batch, cols), generator=gen, dtype=torch.int32)
    lens = torch.randint(1, cols * 16 + 1, (batch,), generator=gen, dtype=torch.int32)
    order = torch.randperm(batch, generator=gen).tolist()
    per = max(batch // (n_groups + 1), 1)
    expect_groups = 0
    for g in range(n_groups):
        rows = order[g * per:(g + 1) * per]
        prefix_pages = int(torch.randint(17, 60, (1,), generator=gen))  # 272 .. 944 tokens, min_prefix_len is 256
        chain = torch.randint(0, pages, (prefix_pages,), generator=gen, dtype=torch.int32)
        for r in rows:
            table[r, :prefix_pages] = chain
            lens[r] = int(torch.randint(prefix_pages * 16, cols * 16 + 1, (1,), generator=gen))
        expect_groups += len(rows) >= 8
    q = torch.randn(batch, hq, d, generator=gen).to(torch.bfloat16)
    exp = oracle.reference(q, kc, vc, table.long(), lens, ks, vs)
    dev = lambda t: t.to(DEV)
    gq, gkc, gvc, gt, gl, gks, gvs = map(dev, (q, kc, vc, table, lens, ks, vs))
    groups, max_groups = cabi.group_shared_prefixes(gt, seq_lens=gl, min_batch=8, min_prefix_len=256, max_groups=4)
    max_len = int(lens.max())
    split = 256
    slots = -(-max_len // 256) + -(-max_len // split)
    ws = (torch.full((batch, hq, slots, d), float("nan"), device=DEV), torch.full((batch, hq, slots), float("nan"), device=DEV),
          torch.full((batch, hq, slots), float("nan"), device=DEV))
    out = torch.full_like(gq, float("nan"))
    cabi.shared_prefix_decode_grouped_fp8_e4m3(gq, gkc, gvc, gt, gl, groups=groups, max_groups=max_groups, k_scale=gks, v_scale=gvs,
                                               max_seq_len=max_len, split_size=split, output=out, workspace=ws)
    torch.cuda.synchronize()
    assert cabi.device_status() == 0
    assert int(groups[3]) >= expect_groups  # (chance agreement of random pages aside, at least the planted groups)
    assert_within_gate(out, exp, f"random grouped batch {seed}: batch {batch}, {n_groups} planted groups, {hq}/{hkv} heads")


def test_grouped_decode_with_a_suffix_bound_and_its_violation(cabi):
    """With a true bound on the grouped requests' suffixes the split-KV grid has few splits, and the
    requests in no group cover their whole context with as many, longer, ones; a bound that a
    grouped request exceeds is reported through the device status (5), not swallowed."""
    w, lengths = _mixed_batch(13, 1024, 512)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    groups, max_groups = cabi.group_shared_prefixes(g.block_table, prefix_lengths=lengths.to(DEV), min_batch=8, min_prefix_len=256)
    split = 64
    bound = w.max_seq_len - 512  # group B's prefix is the shortest
    slots = -(-w.max_seq_len // 256) + -(-bound // split)
    b, hq, d = g.query.shape
    ws = (torch.full((b, hq, slots, d), float("nan"), device=DEV), torch.full((b, hq, slots), float("nan"), device=DEV),
          torch.full((b, hq, slots), float("nan"), device=DEV))
    common = dict(groups=groups, max_groups=max_groups, k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=w.max_seq_len,
                  split_size=split, workspace=ws)
    out = torch.full_like(g.query, float("nan"))
    cabi.shared_prefix_decode_grouped_fp8_e4m3(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, output=out,
                                               max_suffix_len=bound, **common)
    torch.cuda.synchronize()
    assert cabi.device_status() == 0
    assert_within_gate(out, exp, "grouped decode with a suffix bound")
    cabi.shared_prefix_decode_grouped_fp8_e4m3(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, output=out,
                                               max_suffix_len=64, **common)
    torch.cuda.synchronize()
    assert cabi.device_status() == 5


@pytest.fixture
def suffix_form(cabi):
    """Forces one of the two forms of the split-KV pass behind the dense pass; restores the choice."""
    yield cabi.set_suffix_form
    cabi.set_suffix_form(-1)


@pytest.mark.parametrize("form", [0, 1])
def test_both_forms_of_the_suffix_pass_match_the_oracle(cabi, suffix_form, form):
    """The split-KV pass over the suffixes runs either after the dense prefix pass (eight-warp
    CTAs) or beside it (two-warp CTAs, of which only one waits for the dense pass before the grid
    completes): same results, whichever the library would choose by itself."""
    suffix_form(form)
    for batch, shrink, splits in ((20, 0.25, (64, 128, 512)), (64, 1.0, (128, 192))):
        w = make_inputs("shared-prefix-b64", seed=3, batch=batch, shrink=shrink)
        exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
        for split in splits:
            for rep in range(2):
                out, _, _ = run_shared(cabi, w, split)
                assert_within_gate(out, exp, f"form={form} batch={batch} split={split} rep={rep}")
    w, lengths = _mixed_batch(14, 1024, 512)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    groups, max_groups = cabi.group_shared_prefixes(g.block_table, prefix_lengths=lengths.to(DEV), min_batch=8, min_prefix_len=256)
    slots = -(-w.max_seq_len // 256) + -(-w.max_seq_len // 128)
    b, hq, d = g.query.shape
    ws = (torch.full((b, hq, slots, d), float("nan"), device=DEV), torch.full((b, hq, slots), float("nan"), device=DEV),
          torch.full((b, hq, slots), float("nan"), device=DEV))
    out = torch.full_like(g.query, float("nan"))
    cabi.shared_prefix_decode_grouped_fp8_e4m3(
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, groups=groups, max_groups=max_groups,
        k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=w.max_seq_len, split_size=128, output=out, workspace=ws)
    torch.cuda.synchronize()
    assert cabi.device_status() == 0
    assert_within_gate(out, exp, f"form={form}: mixed batch (requests in no group attend from token 0)")


def _full_size_batch_in_three_groups(seed):
    """64 requests behind 4096-token prefixes: three groups of 17 (136 rows of 8 heads each: one
    full 128-row tile and a ragged one) and 13 requests that share nothing."""
    w = make_inputs("shared-prefix-b64", seed=seed, batch=64)
    gen = torch.Generator().manual_seed(seed)
    pages = w.key_cache.shape[0]
    table = w.block_table.clone()
    prefix_pages = w.prefix_len // 16
    for first in (17, 34):
        chain = torch.randint(0, pages, (prefix_pages,), generator=gen, dtype=torch.int32)
        table[first:first + 17, :prefix_pages] = chain
    for r in range(51, 64):
        table[r, :prefix_pages] = torch.randint(0, pages, (prefix_pages,), generator=gen, dtype=torch.int32)
    w.block_table = table
    return w


@pytest.mark.parametrize("hint", [False, True])
def test_grouped_decode_with_more_tiles_than_tile_slots(cabi, hint):
    """At full size the dense pass's grid is one CTA per SM wide and gets no spare tile slots:
    three groups with a ragged tile each make six tiles for four slots, so CTAs take a second tile
    in turn.  With the all-in-groups hint set although 13 requests are in no group (a caller's
    mistake) the result is still right."""
    w = _full_size_batch_in_three_groups(21)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    groups, max_groups = cabi.group_shared_prefixes(g.block_table, seq_lens=g.seq_lens, min_batch=8, min_prefix_len=4096, max_groups=4)
    torch.cuda.synchronize()
    assert groups[3:5].tolist() == [3, 51]
    split = 128
    bound = w.max_seq_len - 4096
    slots = w.prefix_len // 256 + -(-bound // split)
    b, hq, d = g.query.shape
    ws = (torch.full((b, hq, slots, d), float("nan"), device=DEV), torch.full((b, hq, slots), float("nan"), device=DEV),
          torch.full((b, hq, slots), float("nan"), device=DEV))
    for step in range(2):
        out = torch.full_like(g.query, float("nan"))
        cabi.shared_prefix_decode_grouped_fp8_e4m3(
            g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, groups=groups, max_groups=max_groups,
            max_prefix_len=w.prefix_len, max_suffix_len=bound, k_scale=g.k_scale, v_scale=g.v_scale, max_seq_len=w.max_seq_len,
            split_size=split, output=out, workspace=ws, flags=cabi.PFD_FLAG_ALL_IN_GROUPS if hint else 0)
        torch.cuda.synchronize()
        assert cabi.device_status() == 0
        assert_within_gate(out, exp, f"three groups of 17, hint={hint}, step {step}")
