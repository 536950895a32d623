"""Host logic of the shared-prefix dispatch (CPU): grouping equals the oracle's restatement of
the reference function; the gate is closed without the switch / without a GPU."""

import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200 import l20_shared_prefix_decode_dispatch as d
from single_gpu_inference_lab_b200.workloads import make_inputs


def test_grouping_matches_reference_restatement():
    w = make_inputs("shared-prefix-b64", seed=0, batch=12, shrink=0.125)
    table = w.block_table.clone()
    table[3, 1] += 1
    table[7, 0] = table[8, 2]
    for lengths in ([w.prefix_len] * 12, [w.prefix_len] * 6 + [w.prefix_len - 16] * 6):
        for min_batch in (1, 4, 8):
            got = d.find_l20_shared_prefix_groups(table, lengths, min_batch=min_batch, min_prefix_length=64)
            want = oracle.find_shared_prefix_groups(table, lengths, min_batch=min_batch, min_prefix_length=64)
            assert got == want
    assert d.shared_prefix_block_key(table[0], 33) == (33, tuple(int(x) for x in table[0, :3]))


def test_gate_is_closed_by_default(monkeypatch):
    w = make_inputs("shared-prefix-b64", seed=0, batch=8, shrink=0.125)
    monkeypatch.delenv("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", raising=False)
    assert not d.l20_shared_prefix_decode_enabled()
    assert not d.should_dispatch_l20_shared_prefix_paged_decode(w.query, w.key_cache, w.block_table, [w.prefix_len] * 8)
    monkeypatch.setenv("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", "1")
    assert d.l20_shared_prefix_decode_enabled()
    # CPU tensors: still closed (no fallback path exists)
    assert not d.should_dispatch_l20_shared_prefix_paged_decode(w.query, w.key_cache, w.block_table, [w.prefix_len] * 8)


def test_trace_line(tmp_path, monkeypatch):
    path = tmp_path / "trace.jsonl"
    monkeypatch.setenv("VLLM_L20_SHARED_PREFIX_DECODE_TRACE", str(path))
    d.l20_shared_prefix_trace("l20_shared_prefix_paged_decode_run", batch=8, prefix_length=4096)
    import json

    rec = json.loads(path.read_text().strip())
    assert rec["event"] == "l20_shared_prefix_paged_decode_run" and rec["batch"] == 8 and "ts" in rec


def test_workspace_slots():
    q = torch.zeros(4, 16, 128, dtype=torch.bfloat16)
    po, pm, ps, out = d.allocate_shared_prefix_workspace(q, 4096 + 300, 4096, suffix_split_size=128)
    assert po.shape == (4, 16, 16 + 3, 128) and pm.shape == (4, 16, 19) and out.shape == q.shape
