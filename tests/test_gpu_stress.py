"""Randomised cases and graph replay with changing metadata (the reference's counterpart is
scripts/stress_cuda_paged_decode.py: 100 ragged cases, then CUDA-graph capture and replays).

Both operators (FP8 caches, 16-bit caches) on random geometries, lengths, layouts and kv_start,
each against the CPU oracle; then one captured call replayed while the sequence lengths, the
block table and the query are rewritten in place between replays -- what an engine that records
its decode step does."""

import random

import pytest
import torch

from oracle import paged_decode_oracle as oracle

from helpers import assert_within_gate

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def cabi(built_libs):
    from single_gpu_inference_lab_b200 import cabi as module

    module.load()
    return module


def random_case(rng: random.Random, kv16: bool):
    hkv = rng.choice([1, 2, 3, 4, 6, 8])
    group = rng.choice([1, 2, 4, 7, 8])
    hq = hkv * group
    batch = rng.choice([1, 2, 3, 5, 17, 40])
    longest = rng.choice([16, 33, 200, 1500])
    lens = torch.tensor([rng.randint(0 if rng.random() < 0.1 else 1, longest) for _ in range(batch)], dtype=torch.int32)
    if int(lens.max()) == 0:
        lens[0] = 1
    pages_per = (int(lens.max()) + 15) // 16
    spare = rng.randint(0, 3)
    total = batch * pages_per + spare
    gen = torch.Generator().manual_seed(rng.randrange(1 << 30))
    table = torch.randperm(total, generator=gen)[: batch * pages_per].to(torch.int32).reshape(batch, pages_per)
    dtype = rng.choice([torch.bfloat16, torch.float16])
    q = torch.randn(batch, hq, 128, generator=gen).to(dtype)
    k = torch.randn(total, 16, hkv, 128, generator=gen)
    v = torch.randn(total, 16, hkv, 128, generator=gen)
    if kv16:
        return q, k.to(dtype), v.to(dtype), table, lens, None, None
    kc, ks = oracle.quantize_fp8_e4m3_per_head(k)
    vc, vs = oracle.quantize_fp8_e4m3_per_head(v)
    return q, kc, vc, table, lens, ks, vs


def expected(q, kc, vc, table, lens, ks, vs, kv_start=0):
    """fp32 reference with zero rows where nothing is attended."""
    rows = []
    for b in range(q.shape[0]):
        if int(lens[b]) <= kv_start:
            rows.append(torch.zeros(q.shape[1], q.shape[2]))
            continue
        one = slice(b, b + 1)
        if ks is None:
            rows.append(oracle.reference_kv16(q[one], kc, vc, table[one].long(), lens[one], kv_start=kv_start)[0].float())
        else:
            rows.append(oracle.reference_fp32(q[one], kc, vc, table[one].long(), lens[one], ks, vs, kv_start=kv_start)[0])
    return torch.stack(rows).to(q.dtype)


@pytest.mark.parametrize("kv16", [False, True])
def test_random_cases(cabi, kv16):
    rng = random.Random(2024 + kv16)
    for case in range(100):
        q, kc, vc, table, lens, ks, vs = random_case(rng, kv16)
        hkv = kc.shape[2]
        kv_start = rng.choice([0, 0, 0, 5, 16, 37]) if int(lens.max()) > 40 else 0
        exp = expected(q, kc, vc, table, lens, ks, vs, kv_start)
        g = [t.to(DEV) for t in (q, kc, vc, table, lens)]
        if rng.random() < 0.5:  # head-major cache memory behind the same logical view
            g[1] = g[1].permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
            g[2] = g[2].permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        rows = cabi.balanced_workspace_rows(q.shape[1], hkv)
        splits = max(1, -(-rows // (q.shape[0] * q.shape[1])), -(-int(lens.max()) // 512))
        ws = (
            torch.full((q.shape[0], q.shape[1], splits, 128), float("nan"), device=DEV),
            torch.full((q.shape[0], q.shape[1], splits), float("nan"), device=DEV),
            torch.full((q.shape[0], q.shape[1], splits), float("nan"), device=DEV),
            None,
        )
        out = torch.full_like(g[0], float("nan"))
        flags = rng.choice([0, 32])  # with and without early metadata reads
        planned = rng.random() < 0.7  # both kernels read a plan, or derive the split themselves
        fused = planned and rng.random() < 0.5  # pieces combined inside the balanced kernel (one launch)
        what = (f"case {case}: kv16={kv16} B={q.shape[0]} Hq={q.shape[1]} Hkv={hkv} max={int(lens.max())} "
                f"kv_start={kv_start} flags={flags} planned={planned} fused={fused}")
        plan = None
        if planned:
            plan = cabi.plan_decode(*g, max_seq_len=int(lens.max()), split_size=512, workspace=ws, kv_start=kv_start)
            if flags:  # the plan kernel must not be the kernel right in front of an early-metadata call
                torch.cuda.synchronize()
            if fused:
                flags |= 64
        if kv16:
            cabi.paged_decode_kv16_split_out(*g, max_seq_len=int(lens.max()), split_size=512, output=out, workspace=ws,
                                             kv_start=kv_start, flags=flags, plan=plan)
        else:
            cabi.paged_decode_fp8_e4m3_split_out(*g, k_scale=ks.to(DEV), v_scale=vs.to(DEV), max_seq_len=int(lens.max()),
                                                 split_size=512, output=out, workspace=ws, kv_start=kv_start, flags=flags,
                                                 plan=plan)
        torch.cuda.synchronize()
        assert cabi.device_status() == 0, what
        assert cabi.last_path() == ((6 if kv16 else 5) if fused else (4 if kv16 else 3)), what
        assert_within_gate(out, exp, what)


@pytest.mark.parametrize("planned", [False, True, "fused"])
@pytest.mark.parametrize("kv16", [False, True])
def test_graph_replay_with_metadata_rewritten_in_place(built_libs, kv16, planned):
    from single_gpu_inference_lab_b200 import l20_paged_split_kv as m

    torch.manual_seed(5)
    batch, hq, hkv, max_len = 24, 16, 2, 900
    pages_per = (max_len + 15) // 16
    total = batch * pages_per
    dtype = torch.bfloat16
    k = torch.randn(total, 16, hkv, 128)
    v = torch.randn(total, 16, hkv, 128)
    if kv16:
        kc, vc, ks, vs = k.to(dtype), v.to(dtype), None, None
    else:
        kc, ks = oracle.quantize_fp8_e4m3_per_head(k)
        vc, vs = oracle.quantize_fp8_e4m3_per_head(v)
    # persistent device buffers, as an engine keeps them
    q = torch.zeros(batch, hq, 128, dtype=dtype, device=DEV)
    table = torch.zeros(batch, pages_per, dtype=torch.int32, device=DEV)
    lens = torch.ones(batch, dtype=torch.int32, device=DEV)
    gk, gv = kc.to(DEV), vc.to(DEV)
    gks, gvs = (None, None) if kv16 else (ks.to(DEV), vs.to(DEV))
    ws = m.allocate_l20_paged_split_kv_workspace(q, max_len, split_size=512, num_kv_heads=hkv)

    plan_buf = m.plan_l20_paged_split_kv(q, gk, gv, table, lens, max_seq_len=max_len, split_size=512, workspace=ws) if planned else None
    filler = torch.zeros(1 << 16, device=DEV)

    def call():
        # what an engine records per step: the plan from the step's metadata, other work, then
        # the layers' attention calls (two of them here) that share the plan
        plan = None
        if planned:
            plan = m.plan_l20_paged_split_kv(q, gk, gv, table, lens, max_seq_len=max_len, split_size=512, workspace=ws,
                                             plan=plan_buf)
            filler.add_(1.0)
        for _ in range(2):
            if kv16:
                m.l20_paged_split_kv_attention(q, gk, gv, table, lens, split_size=512, workspace=ws, max_seq_len=max_len,
                                               metadata_stable=True, plan=plan, single_launch=planned == "fused")
            else:
                m.l20_paged_split_kv_attention_fp8(q, gk, gv, table, lens, k_scale=gks, v_scale=gvs,
                                                   max_seq_len=max_len, split_size=512, workspace=ws, metadata_stable=True,
                                                   plan=plan, single_launch=planned == "fused")

    call()  # lazy initialisation outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    gen = torch.Generator().manual_seed(9)
    for step in range(40):
        new_lens = torch.randint(0 if step % 4 == 3 else 1, max_len + 1, (batch,), generator=gen).to(torch.int32)
        if step == 5:
            new_lens[:] = max_len
        new_table = torch.randperm(total, generator=gen).to(torch.int32).reshape(batch, pages_per)
        new_q = torch.randn(batch, hq, 128, generator=gen).to(dtype)
        q.copy_(new_q); table.copy_(new_table); lens.copy_(new_lens)
        ws[3].fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        exp = expected(new_q, kc, vc, new_table, new_lens, ks, vs)
        assert_within_gate(ws[3], exp, f"replay {step} kv16={kv16}")


@pytest.mark.parametrize("flags,d", [(8, 128), (1, 128), (0, 64)])
def test_random_cases_fixed_split_grid(cabi, flags, d):
    """The same for the fixed-split grid (TMA and plain loads) and head_dim 64, small split sizes."""
    rng = random.Random(77 + flags + d)
    for case in range(30):
        q, kc, vc, table, lens, ks, vs = random_case(rng, False)
        if d == 64:
            q, kc, vc = q[..., :64].contiguous(), kc[..., :64].contiguous(), vc[..., :64].contiguous()
        hkv = kc.shape[2]
        kv_start = rng.choice([0, 0, 5, 16, 37]) if int(lens.max()) > 40 else 0
        exp = expected(q, kc, vc, table, lens, ks, vs, kv_start)
        split = rng.choice([16, 64, 256, 1024])
        call_flags = flags | rng.choice([0, 32])  # with and without early metadata reads
        g = [t.to(DEV) for t in (q, kc, vc, table, lens)]
        splits = max(1, -(-(int(lens.max()) - kv_start) // split))
        ws = (
            torch.full((q.shape[0], q.shape[1], splits, d), float("nan"), device=DEV),
            torch.full((q.shape[0], q.shape[1], splits), float("nan"), device=DEV),
            torch.full((q.shape[0], q.shape[1], splits), float("nan"), device=DEV),
            None,
        )
        out = torch.full_like(g[0], float("nan"))
        what = f"case {case}: flags={call_flags} d={d} B={q.shape[0]} Hq={q.shape[1]} Hkv={hkv} max={int(lens.max())} kv_start={kv_start} split={split}"
        cabi.paged_decode_fp8_e4m3_split_out(*g, k_scale=ks.to(DEV), v_scale=vs.to(DEV), max_seq_len=int(lens.max()),
                                             split_size=split, output=out, workspace=ws, kv_start=kv_start, flags=call_flags)
        torch.cuda.synchronize()
        assert cabi.device_status() == 0, what
        assert cabi.last_path() == (1 if (flags & 1 or d == 64) else 2), what
        assert_within_gate(out, exp, what)
