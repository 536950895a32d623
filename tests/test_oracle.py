"""The CPU oracle against the golden vectors made by the reference's own torch code
(tests/golden/make_golden.py), plus its internal consistency (split partials + LSE merge)."""

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import GEOMETRIES, make_inputs

from helpers import digest, smoke_recipe


def _case_inputs(case):
    return make_inputs(case["workload"], seed=0, device="cpu", batch=case["batch"], shrink=case["shrink"])


@pytest.mark.parametrize(
    "name",
    ["cfg1-qwen0.5b-b8", "cfg2-coder3b-b4", "cfg3-qwen7b-b24", "cfg4-llama8b-b2", "cfg5-prefix-b8"],
)
def test_oracle_reproduces_reference_outputs_bit_for_bit(golden, name):
    case = golden["cases"][name]
    w = _case_inputs(case)
    assert digest(w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens, w.k_scale, w.v_scale) == case[
        "inputs_sha256"
    ], "seeded input generation changed; regenerate tests/golden with make_golden.py"
    out = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    assert out.dtype == case["output"].dtype
    assert torch.equal(out.view(torch.int16), case["output"].view(torch.int16))


def test_oracle_reproduces_reference_smoke_recipe(golden):
    for key, case in golden["smoke"].items():
        q, kc, vc, table, lens, ks, vs = smoke_recipe(
            case["batch"], case["context"], case["q_heads"], case["kv_heads"], oracle.quantize_fp8_e4m3
        )
        assert ks == case["k_scale"] and vs == case["v_scale"], key
        assert digest(kc, vc) == case["cache_sha256"], key
        out = oracle.reference(q, kc, vc, table.long(), lens, ks, vs)
        assert torch.equal(out.view(torch.int16), case["output"].view(torch.int16)), key


@pytest.mark.parametrize(
    "name", ["kv16-cfg2-coder3b-b4-bf16", "kv16-cfg3-qwen7b-b24-bf16", "kv16-cfg4-llama8b-b2-fp16"]
)
def test_kv16_oracle_reproduces_reference_outputs_bit_for_bit(golden, name):
    """The non-quantised sibling against reference() of scripts/smoke_cuda_paged_decode_op.py."""
    case = golden["kv16"][name]
    dtype = getattr(torch, case["dtype"])
    w = make_inputs(case["workload"], seed=0, device="cpu", batch=case["batch"], shrink=case["shrink"],
                    query_dtype=dtype, kv_dtype=dtype)
    assert digest(w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens) == case["inputs_sha256"]
    out = oracle.reference_kv16(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens)
    assert out.dtype == dtype and torch.equal(out.view(torch.int16), case["output"].view(torch.int16))


def test_per_head_quantisation_matches_per_tensor_recipe_on_one_head():
    torch.manual_seed(3)
    x = torch.randn(5, 16, 1, 64)
    q_t, s_t = oracle.quantize_fp8_e4m3(x)
    q_h, s_h = oracle.quantize_fp8_e4m3_per_head(x)
    # the per-tensor scale is a Python double, the per-head one float32: equal to fp32 rounding
    assert abs(float(s_h[0]) - s_t) <= 1e-6 * s_t
    same = (q_t.view(torch.uint8) == q_h.view(torch.uint8)).float().mean().item()
    assert same > 0.999


@pytest.mark.parametrize("split_size", [16, 64, 512])
def test_split_partials_merge_equals_reference(split_size):
    w = make_inputs("qwen2.5-0.5b-b8", seed=1, device="cpu", batch=3, shrink=0.25)
    num_splits = -(-w.max_seq_len // split_size)
    o, m, l = oracle.split_partials(
        w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale,
        split_size=split_size, num_splits=num_splits,
    )
    merged = oracle.merge_partials(o, m, l)
    ref = oracle.reference_fp32(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    assert torch.allclose(merged, ref, atol=2e-6, rtol=1e-5)
    packed = torch.cat([o, m[..., None], l[..., None]], dim=-1).permute(2, 0, 1, 3).contiguous()
    assert torch.allclose(oracle.merge_packed(packed), ref, atol=2e-6, rtol=1e-5)


def test_resolve_slots_expression():
    table = torch.tensor([[5, 2, 9], [1, 0, 0]], dtype=torch.int32)
    lens = torch.tensor([33, 3], dtype=torch.int32)
    slots = oracle.resolve_slots(table, lens, 40)
    assert slots.shape == (2, 40)
    assert slots[0, 0] == 80 and slots[0, 15] == 95 and slots[0, 16] == 32 and slots[0, 32] == 144
    assert (slots[0, 33:] == -1).all() and (slots[1, 3:] == -1).all() and slots[1, 2] == 18


def test_shared_prefix_grouping():
    w = make_inputs("shared-prefix-b64", seed=0, device="cpu", batch=10, shrink=0.125)
    groups = oracle.find_shared_prefix_groups(w.block_table, [w.prefix_len] * 10, min_batch=8, min_prefix_length=w.prefix_len)
    assert groups == [list(range(10))]
    table = w.block_table.clone()
    table[3, 0] += 1
    groups = oracle.find_shared_prefix_groups(table, [w.prefix_len] * 10, min_batch=8, min_prefix_length=w.prefix_len)
    assert groups == [[0, 1, 2, 4, 5, 6, 7, 8, 9]]
    assert oracle.find_shared_prefix_groups(table, [w.prefix_len] * 10, min_batch=8, min_prefix_length=w.prefix_len + 1) == []
    with pytest.raises(ValueError):
        oracle.find_shared_prefix_groups(table[0], [1])


def test_workload_geometries_and_determinism():
    assert set(GEOMETRIES) == {
        "qwen2.5-0.5b-b8", "qwen2.5-coder-3b-b64", "qwen2.5-7b-b256", "llama3-8b-long-b4", "shared-prefix-b64",
    }
    a = make_inputs("qwen2.5-0.5b-b8", seed=0)
    b = make_inputs("qwen2.5-0.5b-b8", seed=0)
    assert digest(a.query, a.key_cache, a.block_table) == digest(b.query, b.key_cache, b.block_table)
    assert a.query.shape == (8, 14, 64) and a.key_cache.shape[1:] == (16, 2, 64)
    assert int(a.seq_lens.min()) >= 128 and int(a.seq_lens.max()) <= 1024
    # every physical page is used exactly once across the batch
    pages = []
    for r in range(8):
        pages += a.block_table[r, : -(-int(a.seq_lens[r]) // 16)].tolist()
    assert sorted(pages) == list(range(a.key_cache.shape[0]))
    assert a.kv_bytes == int(a.seq_lens.sum()) * 2 * 64 * 2
    c = make_inputs("qwen2.5-7b-b256", seed=0, shrink=0.125)
    assert c.query.shape == (256, 28, 128) and int(c.seq_lens.min()) >= 1 and int(c.seq_lens.max()) <= 1024
    s = make_inputs("shared-prefix-b64", seed=0, batch=6, shrink=0.125)
    pp = s.prefix_len // 16
    assert (s.block_table[:, :pp] == s.block_table[0, :pp]).all()
