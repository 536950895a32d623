"""The producer step (rotary embedding + paged KV append, optionally quantised to FP8):
the CPU oracle against the reference's own outputs, and the CUDA kernel against the oracle --
bit for bit -- and against the decode operator that consumes what it wrote."""

import pytest
import torch

from oracle import paged_decode_oracle as decode_oracle
from oracle import rope_kv_oracle as oracle

from helpers import assert_within_gate

DEV = "cuda:0"


def golden_inputs(case):
    """The seeded inputs tests/golden/make_golden.py fed to the reference's rope_kv_reference."""
    tokens, hkv, d, rot = case["tokens"], case["kv_heads"], case["head_dim"], case["rotary_dim"]
    dtype = getattr(torch, case["dtype"])
    gen = torch.Generator().manual_seed(41)
    k = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    v = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    angle = torch.rand(tokens, rot // 2, generator=gen) * 6.2831853
    slots = torch.randperm(4 * tokens, generator=gen)[:tokens]
    return k, v, torch.cos(angle), torch.sin(angle), slots, dtype


def test_oracle_reproduces_reference_rope_kv_outputs_bit_for_bit(golden):
    for name, case in golden["rope"].items():
        k, v, cos, sin, slots, dtype = golden_inputs(case)
        tokens, hkv, d = k.shape
        # the reference writes a flat [slots, Hkv, D] cache from per-token cos / sin rows: the same thing
        # as a one-token-per-block paged cache and a cos_sin table indexed by the token number
        table = torch.cat([cos, sin], dim=1)
        kc = torch.zeros(4 * tokens, 1, hkv, d, dtype=dtype)
        _, _, kc2, vc2 = oracle.rope_and_cache(
            torch.zeros(tokens, hkv, d, dtype=dtype), k, v, torch.arange(tokens), table, True, kc, torch.zeros_like(kc), slots
        )
        assert torch.equal(kc2[:, 0].view(torch.int16), case["key_cache"].view(torch.int16)), name
        assert torch.equal(vc2[:, 0].view(torch.int16), case["value_cache"].view(torch.int16)), name


def paged_golden_inputs(case):
    """The seeded inputs tests/golden/make_golden.py fed to the reference's paged_rope_kv_reference
    (src/l20_stack/ops/triton_rope_kv.py:176-205): same recipe as paged_rope_inputs there."""
    seqs, tokens, hkv, d, rot = case["seqs"], case["tokens"], case["kv_heads"], case["head_dim"], case["rotary_dim"]
    dtype = getattr(torch, case["dtype"])
    gen = torch.Generator().manual_seed(43)
    k = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    v = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    angle = torch.rand(tokens, rot // 2, generator=gen) * 6.2831853
    max_blocks = 6
    table = torch.randperm(seqs * max_blocks, generator=gen).reshape(seqs, max_blocks)
    flat = torch.randperm(seqs * max_blocks * 16, generator=gen)[:tokens]
    sequence_ids, positions = flat // (max_blocks * 16), flat % (max_blocks * 16)
    # what an engine hands the operator: the slot of every token, resolved through the block table
    slots = table[sequence_ids, positions // 16] * 16 + positions % 16
    cos_sin = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1)  # one row per token, indexed by token number
    return k, v, cos_sin, slots, table.numel(), dtype


def check_against_paged_golden(case, kc, vc, slots, name):
    from helpers import digest

    assert torch.equal(kc[slots // 16, slots % 16].view(torch.int16), case["key_rows"].view(torch.int16)), name
    assert torch.equal(vc[slots // 16, slots % 16].view(torch.int16), case["value_rows"].view(torch.int16)), name
    assert digest(kc) == case["key_cache_sha256"] and digest(vc) == case["value_cache_sha256"], name


def test_oracle_reproduces_reference_paged_rope_kv_outputs_bit_for_bit(golden):
    for name, case in golden["rope_paged"].items():
        k, v, cos_sin, slots, blocks, dtype = paged_golden_inputs(case)
        tokens, hkv, d = k.shape
        kc = torch.zeros(blocks, 16, hkv, d, dtype=dtype)
        _, _, kc2, vc2 = oracle.rope_and_cache(torch.zeros(tokens, hkv, d, dtype=dtype), k, v, torch.arange(tokens), cos_sin,
                                               True, kc, torch.zeros_like(kc), slots)
        check_against_paged_golden(case, kc2, vc2, slots, name)


@pytest.mark.gpu
def test_kernel_reproduces_reference_paged_rope_kv_outputs_bit_for_bit(built_libs, golden):
    from single_gpu_inference_lab_b200 import l20_rope_kv

    for name, case in golden["rope_paged"].items():
        k, v, cos_sin, slots, blocks, dtype = paged_golden_inputs(case)
        tokens, hkv, d = k.shape
        kc = torch.zeros(blocks, 16, hkv, d, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        q = torch.zeros(tokens, hkv, d, dtype=dtype, device=DEV)
        l20_rope_kv.l20_rope_and_cache(q, k.to(DEV), v.to(DEV), torch.arange(tokens, device=DEV), cos_sin.to(DEV), True,
                                       kc, vc, slots.to(DEV))
        torch.cuda.synchronize()
        check_against_paged_golden(case, kc.cpu(), vc.cpu(), slots, name)


def make_step(seed, tokens, hq, hkv, d, rot, dtype, cache_dtype, table_dtype, block_size=16):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(tokens, hq, d, generator=gen).to(dtype)
    k = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    v = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    max_pos = 512
    angle = torch.rand(max_pos, rot // 2, generator=gen) * 6.2831853
    cos_sin = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).to(table_dtype)
    positions = torch.randint(0, max_pos, (tokens,), generator=gen)
    blocks = 2 * tokens // block_size + 3
    slots = torch.randperm(blocks * block_size, generator=gen)[:tokens]
    slots[tokens // 2] = -1  # a padded token: rotated, not stored
    if cache_dtype == torch.float8_e4m3fn:
        kc = torch.full((blocks, block_size, hkv, d), 0x11, dtype=torch.uint8).view(torch.float8_e4m3fn)
        vc = torch.full((blocks, block_size, hkv, d), 0x22, dtype=torch.uint8).view(torch.float8_e4m3fn)
        ks = torch.rand(hkv, generator=gen) * 0.02 + 0.003
        vs = torch.rand(hkv, generator=gen) * 0.02 + 0.003
    else:
        kc = torch.full((blocks, block_size, hkv, d), 7.0, dtype=dtype)
        vc = torch.full((blocks, block_size, hkv, d), -7.0, dtype=dtype)
        ks = vs = None
    return q, k, v, positions, cos_sin, kc, vc, slots, ks, vs


@pytest.mark.gpu
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("cache", ["same", "fp8"])
def test_kernel_matches_oracle_bit_for_bit(built_libs, is_neox, cache):
    from single_gpu_inference_lab_b200 import l20_rope_kv

    for seed, (tokens, hq, hkv, d, rot, dtype, table_dtype) in enumerate([
        (64, 16, 2, 128, 128, torch.bfloat16, torch.float32),
        (5, 28, 4, 128, 64, torch.float16, torch.float16),
        (256, 14, 2, 64, 64, torch.bfloat16, torch.bfloat16),
        (1, 32, 8, 128, 32, torch.float16, torch.float32),
        (33, 8, 8, 128, 128, torch.float16, torch.float16),  # the vectorised kernel in fp16 with an fp16 table
        (700, 16, 2, 128, 128, torch.bfloat16, torch.float32),
    ]):
        cache_dtype = torch.float8_e4m3fn if cache == "fp8" else dtype
        q, k, v, pos, cs, kc, vc, slots, ks, vs = make_step(seed, tokens, hq, hkv, d, rot, dtype, cache_dtype, table_dtype)
        eq, ek, ekc, evc = oracle.rope_and_cache(q, k, v, pos, cs, is_neox, kc, vc, slots, ks, vs)
        g = [t.to(DEV) for t in (q, k, v, pos, cs, kc, vc, slots)]
        gq, gk, gv, gpos, gcs, gkc, gvc, gslots = g
        l20_rope_kv.l20_rope_and_cache(gq, gk, gv, gpos, gcs, is_neox, gkc, gvc, gslots,
                                       k_scale=None if ks is None else ks.to(DEV), v_scale=None if vs is None else vs.to(DEV))
        torch.cuda.synchronize()
        what = f"tokens={tokens} hq={hq} hkv={hkv} d={d} rot={rot} {dtype} neox={is_neox} cache={cache}"
        assert torch.equal(gq.cpu().view(torch.int16), eq.view(torch.int16)), "query " + what
        assert torch.equal(gk.cpu().view(torch.int16), ek.view(torch.int16)), "key " + what
        as_bits = (lambda t: t.view(torch.uint8)) if cache == "fp8" else (lambda t: t.view(torch.int16))
        assert torch.equal(as_bits(gkc.cpu()), as_bits(ekc)), "key cache " + what
        assert torch.equal(as_bits(gvc.cpu()), as_bits(evc)), "value cache " + what


@pytest.mark.gpu
def test_append_then_decode_equals_the_oracles(built_libs):
    """One decode step of a small model layer: append the new token of every sequence with the
    producer kernel, then attend with the FP8 decode operator; compare with the two CPU oracles
    chained the same way."""
    from single_gpu_inference_lab_b200 import l20_paged_split_kv, l20_rope_kv
    from single_gpu_inference_lab_b200.workloads import make_inputs

    w = make_inputs("qwen2.5-coder-3b-b64", seed=12, batch=12, shrink=0.2)
    batch, hq, d = w.query.shape
    hkv = w.key_cache.shape[2]
    gen = torch.Generator().manual_seed(3)
    # the new token of each sequence overwrites its last position
    positions = (w.seq_lens.long() - 1)
    slots = w.block_table[torch.arange(batch), positions // 16].long() * 16 + positions % 16
    q = torch.randn(batch, hq, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(batch, hkv, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(batch, hkv, d, generator=gen).to(torch.bfloat16)
    angle = torch.arange(int(positions.max()) + 1)[:, None] * (1e4 ** (-torch.arange(0, d, 2) / d))[None, :]
    cos_sin = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).float()
    eq, _, ekc, evc = oracle.rope_and_cache(q, k, v, positions, cos_sin, True, w.key_cache, w.value_cache, slots,
                                            w.k_scale, w.v_scale)
    exp = decode_oracle.reference(eq, ekc, evc, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    gq, gk, gv = q.to(DEV), k.to(DEV), v.to(DEV)
    l20_rope_kv.l20_rope_and_cache(gq, gk, gv, positions.to(DEV), cos_sin.to(DEV), True, g.key_cache, g.value_cache,
                                   slots.to(DEV), k_scale=g.k_scale, v_scale=g.v_scale)
    out = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
        gq, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
        max_seq_len=w.max_seq_len, split_size=256)
    torch.cuda.synchronize()
    assert torch.equal(g.key_cache.cpu().view(torch.uint8), ekc.view(torch.uint8))
    assert_within_gate(out, exp, "append + decode")
    # The same step with a plan and the caller's word that the kernel in front of the decode call
    # writes K/V only at each sequence's last position (kv_stable): the balanced kernel may then
    # fetch older pages before the append has completed, and must still see the new token.
    w2 = make_inputs("qwen2.5-coder-3b-b64", seed=12, batch=64, shrink=0.5)
    batch = w2.query.shape[0]
    positions = (w2.seq_lens.long() - 1)
    slots = w2.block_table[torch.arange(batch), positions // 16].long() * 16 + positions % 16
    q = torch.randn(batch, hq, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(batch, hkv, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(batch, hkv, d, generator=gen).to(torch.bfloat16)
    angle = torch.arange(int(positions.max()) + 1)[:, None] * (1e4 ** (-torch.arange(0, d, 2) / d))[None, :]
    cos_sin = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).float()
    eq, _, ekc, evc = oracle.rope_and_cache(q, k, v, positions, cos_sin, True, w2.key_cache, w2.value_cache, slots,
                                            w2.k_scale, w2.v_scale)
    exp = decode_oracle.reference(eq, ekc, evc, w2.block_table.long(), w2.seq_lens, w2.k_scale, w2.v_scale)
    g = w2.to(DEV)
    kc0, vc0 = g.key_cache.clone(), g.value_cache.clone()
    ws = l20_paged_split_kv.allocate_l20_paged_split_kv_workspace(g.query, w2.max_seq_len, split_size=512)
    plan = l20_paged_split_kv.plan_l20_paged_split_kv(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens,
                                                      max_seq_len=w2.max_seq_len, split_size=512, workspace=ws)
    cs, pos, sl = cos_sin.to(DEV), positions.to(DEV), slots.to(DEV)
    for rep in range(8):
        g.key_cache.copy_(kc0)
        g.value_cache.copy_(vc0)
        gq, gk, gv = q.to(DEV), k.to(DEV), v.to(DEV)
        l20_rope_kv.l20_rope_and_cache(gq, gk, gv, pos, cs, True, g.key_cache, g.value_cache, sl,
                                       k_scale=g.k_scale, v_scale=g.v_scale)
        out = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
            gq, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
            max_seq_len=w2.max_seq_len, split_size=512, workspace=ws, plan=plan, metadata_stable=True, kv_stable=True)
        torch.cuda.synchronize()
        assert_within_gate(out, exp, f"append + planned decode with early K/V, repetition {rep}")


def test_wrapper_argument_errors_without_a_gpu():
    from single_gpu_inference_lab_b200 import l20_rope_kv

    q = torch.zeros(2, 4, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="requires an SM100 GPU"):
        l20_rope_kv.l20_rope_and_cache(q, q, q, torch.zeros(2, dtype=torch.long), torch.zeros(8, 128), True,
                                       torch.zeros(1, 16, 4, 128, dtype=torch.bfloat16),
                                       torch.zeros(1, 16, 4, 128, dtype=torch.bfloat16), torch.zeros(2, dtype=torch.long))
