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
