"""The per-model-step state of the decode hook: the first layer of a step computes the plan, the
shared-prefix groups and the workspace, the other layers reuse them; a step with groups goes
through the grouped shared-prefix operator and leaves the reference's trace records."""

import json
from types import SimpleNamespace

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import make_inputs

from helpers import assert_within_gate

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _fresh(monkeypatch, **env):
    from single_gpu_inference_lab_b200 import l20_decode_step as mod

    for k in ("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", "VLLM_L20_SHARED_PREFIX_FORCE", "VLLM_L20_SHARED_PREFIX_DECODE_TRACE",
              "VLLM_L20_PAGED_NO_PLAN"):
        monkeypatch.delenv(k, raising=False)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    mod._SWITCHES = None
    mod._BUFFERS.clear()
    return mod


def test_plan_and_workspace_are_made_once_per_step_and_shared_by_the_layers(built_libs, monkeypatch):
    mod = _fresh(monkeypatch)
    from single_gpu_inference_lab_b200 import l20_paged_split_kv as m

    w = make_inputs("qwen2.5-coder-3b-b64", seed=31, batch=16, shrink=0.25)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    layers = [(g.key_cache, g.value_cache), (g.key_cache.clone(), g.value_cache.clone())]
    steps = []
    for _ in range(2):  # two model steps: new metadata object, same persistent buffers
        meta = SimpleNamespace(l20_step=None)
        for kc, vc in layers:
            step = mod.l20_decode_step(meta, g.query, kc, vc, g.block_table, g.seq_lens, w.max_seq_len)
            assert step is meta.l20_step and step.plan is not None and step.groups is None
            out = m.l20_paged_split_kv_attention_fp8(g.query, kc, vc, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
                                                     max_seq_len=w.max_seq_len, split_size=512, workspace=step.workspace,
                                                     metadata_stable=True, plan=step.plan, output=torch.empty_like(g.query))
            torch.cuda.synchronize()
            assert_within_gate(out, exp, "planned layer")
        steps.append(meta.l20_step)
    assert steps[0] is not steps[1]
    assert steps[0].plan.data_ptr() == steps[1].plan.data_ptr(), "the plan buffer is persistent (a CUDA graph replays into it)"
    assert steps[0].workspace[0].data_ptr() == steps[1].workspace[0].data_ptr()


def test_a_step_with_shared_prefix_groups_takes_the_grouped_operator_and_is_traced(built_libs, monkeypatch, tmp_path):
    trace = tmp_path / "trace.jsonl"
    mod = _fresh(monkeypatch, VLLM_ENABLE_L20_SHARED_PREFIX_DECODE="1", VLLM_L20_SHARED_PREFIX_DECODE_TRACE=str(trace))
    w = make_inputs("shared-prefix-b64", seed=32, batch=16)  # 4096 shared tokens + private suffixes
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    meta = SimpleNamespace(l20_step=None)
    for _layer in range(2):
        step = mod.l20_decode_step(meta, g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, w.max_seq_len)
        assert step.groups is not None and step.group_sizes == [16]
        assert step.all_in_groups and step.one_prefix == 4096  # one group spans the batch: the single-group operator runs
        out = mod.l20_grouped_decode(step, g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, g.k_scale, g.v_scale,
                                     w.max_seq_len, torch.empty_like(g.query))
        torch.cuda.synchronize()
        assert_within_gate(out, exp, "grouped layer")
    records = [json.loads(line) for line in trace.read_text().splitlines()]
    assert [r["event"] for r in records] == ["shared_prefix_decode_candidate", "l20_shared_prefix_paged_decode_run",
                                             "l20_shared_prefix_paged_decode_run"]  # (read before the second batch below)
    assert records[0]["eligible"] is True and records[0]["group_sizes"] == [16] and records[0]["batch"] == 16
    # two groups of eight: the grouped operator, with the word that no request is outside the groups
    gen = torch.Generator().manual_seed(5)
    pages = w.key_cache.shape[0]
    w.block_table = w.block_table.clone()
    w.block_table[8:, : w.prefix_len // 16] = torch.randint(0, pages, (w.prefix_len // 16,), generator=gen, dtype=torch.int32)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    meta = SimpleNamespace(l20_step=None)
    step = mod.l20_decode_step(meta, g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, w.max_seq_len)
    assert step.group_sizes == [8, 8] and step.all_in_groups and step.one_prefix == 0
    out = mod.l20_grouped_decode(step, g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, g.k_scale, g.v_scale,
                                 w.max_seq_len, torch.empty_like(g.query))
    torch.cuda.synchronize()
    assert_within_gate(out, exp, "two groups of eight")
    # a batch without groups: the step keeps to the ordinary operator
    other = make_inputs("qwen2.5-coder-3b-b64", seed=33, batch=16).to(DEV)
    meta = SimpleNamespace(l20_step=None)
    step = mod.l20_decode_step(meta, other.query, other.key_cache, other.value_cache, other.block_table, other.seq_lens,
                               other.max_seq_len)
    assert step.groups is None
