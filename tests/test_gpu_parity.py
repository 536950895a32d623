"""Parity of the CUDA path against the CPU oracle, through the C ABI (ctypes).

Gate (on bf16 / fp16 outputs): |a - b| <= 2e-3 + 1e-2 * |b| element-wise; gather indices
bit-exact.  Every test here needs a B200.
"""

import math

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import make_inputs

from helpers import assert_within_gate, smoke_recipe

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def cabi(built_libs):
    from single_gpu_inference_lab_b200 import cabi as module

    module.load()
    return module


PATH_LDG, PATH_TMA, PATH_BALANCED, PATH_FUSED = 1, 2, 3, 5
EARLY = 32  # PFD_FLAG_EARLY_METADATA: what the benchmark and the vLLM hook pass
SINGLE = 64  # PFD_FLAG_SINGLE_LAUNCH: pieces combined inside the balanced kernel (needs a plan)
EARLY_KV = 256  # PFD_FLAG_EARLY_KV: with EARLY and a plan, pages other than a sequence's last are streamed before the wait
PLAN = 1 << 20  # not a library flag: the test helpers call pfd_plan_decode first and pass the plan
FUSED = PLAN | SINGLE


def workspace(q, max_seq_len, split_size, dtype=torch.float32, kv_start=0, poison=True, min_rows=0):
    """(partial_output, partial_max, partial_sum, None) with one slot per split, or as many as
    it takes to hold ``min_rows`` rows (the capacity the balanced persistent kernel asks for)."""
    b, hq, d = q.shape
    s = max(1, -(-(max_seq_len - kv_start) // split_size), -(-min_rows // (b * hq)))
    fill = float("nan") if poison else 0.0
    return (
        torch.full((b, hq, s, d), fill, device=q.device, dtype=dtype),
        torch.full((b, hq, s), fill, device=q.device, dtype=torch.float32),
        torch.full((b, hq, s), fill, device=q.device, dtype=torch.float32),
        None,
    )


def expected_path(cabi, q, num_kv_heads, flags, partial_dtype=torch.float32):
    """Which kernels a call must have launched.  flags 0: the library's choice, i.e. the balanced
    persistent kernel for head_dim 128 with at most 8 query heads per kv head and an f32 workspace
    that is large enough (PLAN: both kernels read a plan; FUSED: the balanced kernel alone); 8:
    fixed-split grid with TMA; 1: with plain loads."""
    _, hq, d = q.shape
    if flags & 1 or d != 128:
        return PATH_LDG
    if flags & (8 | 2) or partial_dtype != torch.float32 or hq // num_kv_heads > 8:
        return PATH_TMA
    return PATH_FUSED if (flags & FUSED) == FUSED else PATH_BALANCED


def balanced(path):
    return path in (PATH_BALANCED, PATH_FUSED)


def make_plan(cabi, want, flags, q, kc, vc, table, lens, ws, msl, split_size, kv_start=0):
    """The plan of a call that asks for one (PLAN) and runs the balanced kernel (None otherwise)."""
    if not (flags & PLAN) or not balanced(want):
        return None
    return cabi.plan_decode(q, kc, vc, table, lens, max_seq_len=msl, split_size=split_size, workspace=ws, kv_start=kv_start)


def run(cabi, w, split_size, *, flags=0, kv_start=0, partial_dtype=torch.float32, packed=False,
        k_scale=None, v_scale=None, max_seq_len=None):
    """w: PagedDecodeInputs on the GPU. Returns output (and packed partial if asked)."""
    q = w.query
    hkv = w.key_cache.shape[2]
    msl = w.max_seq_len if max_seq_len is None else max_seq_len
    want = expected_path(cabi, q, hkv, flags, partial_dtype)
    rows = cabi.balanced_workspace_rows(q.shape[1], hkv) if balanced(want) else 0
    ws = workspace(q, msl, split_size, partial_dtype, kv_start, min_rows=rows)
    out = torch.full_like(q, float("nan"))
    pk = torch.full((q.shape[0], q.shape[1], q.shape[2] + 2), float("nan"), device=q.device) if packed else None
    plan = make_plan(cabi, want, flags, q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, ws, msl, split_size, kv_start)
    flags &= ~PLAN
    cabi.paged_decode_fp8_e4m3_split_out(
        q, w.key_cache, w.value_cache, w.block_table, w.seq_lens,
        k_scale=w.k_scale if k_scale is None else k_scale,
        v_scale=w.v_scale if v_scale is None else v_scale,
        max_seq_len=msl, split_size=split_size, output=None if packed else out, packed_output=pk,
        workspace=ws, kv_start=kv_start, flags=flags, plan=plan,
    )
    torch.cuda.synchronize()
    assert cabi.device_status() == 0, "a bounded device-side wait gave up"
    assert cabi.last_path() == want, f"flags={flags}: path {cabi.last_path()}, expected {want}"
    return pk if packed else out


def expected(w, **kw):
    return oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale, **kw)


# ---------------------------------------------------------------- golden fixtures
@pytest.mark.parametrize(
    "name", ["cfg1-qwen0.5b-b8", "cfg2-coder3b-b4", "cfg3-qwen7b-b24", "cfg4-llama8b-b2", "cfg5-prefix-b8"]
)
@pytest.mark.parametrize("flags", [PLAN, FUSED, 8, 1, 0, PLAN | EARLY, FUSED | EARLY, PLAN | EARLY | EARLY_KV, FUSED | EARLY | EARLY_KV])
def test_against_committed_reference_outputs(cabi, golden, name, flags):
    case = golden["cases"][name]
    w = make_inputs(case["workload"], seed=0, device="cpu", batch=case["batch"], shrink=case["shrink"])
    for split in (64, 512):
        out = run(cabi, w.to(DEV), split, flags=flags)
        assert_within_gate(out, case["output"], f"{name} split={split}")


def test_reference_smoke_recipe_fp16_query_scalar_scales(cabi, golden):
    for key, case in golden["smoke"].items():
        q, kc, vc, table, lens, ks, vs = smoke_recipe(
            case["batch"], case["context"], case["q_heads"], case["kv_heads"], oracle.quantize_fp8_e4m3
        )
        q, kc, vc, table, lens = (t.to(DEV) for t in (q, kc, vc, table, lens))
        out = torch.empty_like(q)
        ws = workspace(q, case["context"], 128)
        cabi.paged_decode_fp8_e4m3_split_out(
            q, kc, vc, table, lens, k_scale=ks, v_scale=vs, max_seq_len=case["context"], split_size=128,
            output=out, workspace=ws,
        )
        torch.cuda.synchronize()
        assert_within_gate(out, case["output"], key)


# ---------------------------------------------------------------- the five configurations
def test_config1_full_size(cabi):
    w = make_inputs("qwen2.5-0.5b-b8", seed=0)
    exp = expected(w)
    for split in (16, 128, 1024):
        for flags in (0, EARLY):
            assert_within_gate(run(cabi, w.to(DEV), split, flags=flags), exp, f"cfg1 split={split} flags={flags}")


def test_config2_full_size(cabi):
    w = make_inputs("qwen2.5-coder-3b-b64", seed=0)
    exp = expected(w)
    for split, flags in ((256, PLAN), (512, 0), (896, 0), (512, 8), (1024, 1), (512, EARLY), (896, EARLY | 8), (256, EARLY | 1), (512, PLAN | EARLY), (512, FUSED), (256, FUSED | EARLY), (512, PLAN | EARLY | EARLY_KV), (256, EARLY | EARLY_KV)):
        assert_within_gate(run(cabi, w.to(DEV), split, flags=flags), exp, f"cfg2 split={split} flags={flags}")


def test_config3_full_size_log_uniform_lengths(cabi):
    w = make_inputs("qwen2.5-7b-b256", seed=0)
    assert int(w.seq_lens.min()) <= 4
    exp = expected(w)
    for flags in (0, PLAN, FUSED, 8, EARLY, EARLY | 8, PLAN | EARLY, FUSED | EARLY, PLAN | EARLY | EARLY_KV):
        assert_within_gate(run(cabi, w.to(DEV), 512, flags=flags), exp, f"cfg3 flags={flags}")


def test_config4_long_context_sampled_rows_and_split_invariance(cabi):
    """Full 4 x 131072 tokens on the GPU.  The oracle is run on one sequence compacted to its
    own pages (the whole-cache dequantisation of the reference function would need ~10 GB);
    split invariance covers the rest."""
    w = make_inputs("llama3-8b-long-b4", seed=0, device=DEV)
    out_a = run(cabi, w, 2048, flags=PLAN)
    out_b = run(cabi, w, 512, flags=8)
    out_c = run(cabi, w, 16384)
    out_d = run(cabi, w, 2048, flags=EARLY)
    out_f = run(cabi, w, 2048, flags=PLAN | EARLY)
    out_h = run(cabi, w, 2048, flags=PLAN | EARLY | EARLY_KV)
    assert_within_gate(out_f, out_a, "planned, early metadata vs not")
    assert_within_gate(out_h, out_a, "planned, early metadata and early K/V vs not")
    out_g = run(cabi, w, 2048, flags=FUSED | EARLY)
    assert_within_gate(out_g, out_a, "pieces combined inside the balanced kernel vs the merge kernel")
    out_e = run(cabi, w, 1024, flags=EARLY | 8)
    assert_within_gate(out_d, out_a, "early metadata vs not")
    assert_within_gate(out_e, out_a, "early metadata, fixed split 1024 vs 2048")
    assert_within_gate(out_b, out_a, "split 512 vs 2048")
    assert_within_gate(out_c, out_a, "split 8192 vs 2048")
    b = 2
    pages = w.block_table[b].long().cpu()
    kc = w.key_cache[pages.to(DEV)].cpu()
    vc = w.value_cache[pages.to(DEV)].cpu()
    table = torch.arange(pages.numel(), dtype=torch.int64)[None]
    exp = oracle.reference(
        w.query[b : b + 1].cpu(), kc, vc, table, w.seq_lens[b : b + 1].cpu(), w.k_scale.cpu(), w.v_scale.cpu()
    )
    assert_within_gate(out_a[b : b + 1], exp, "cfg4 row 2")


def test_config5_shared_prefix_full_size(cabi):
    w = make_inputs("shared-prefix-b64", seed=0)
    exp = expected(w)
    for flags in (0, PLAN, FUSED, 8, EARLY, EARLY | 8, PLAN | EARLY):
        assert_within_gate(run(cabi, w.to(DEV), 512, flags=flags), exp, f"cfg5 flags={flags}")


# ---------------------------------------------------------------- edge cases
@pytest.mark.parametrize("d,hq,hkv", [(128, 16, 2), (64, 14, 2), (128, 28, 4), (128, 32, 8), (128, 16, 16), (128, 16, 1)])
def test_every_short_context_length(cabi, d, hq, hkv):
    """ctx = 1 .. 70 in one batch: ragged tails, single page, page boundary +-1."""
    torch.manual_seed(11)
    lens = torch.arange(1, 71, dtype=torch.int32)
    b = lens.numel()
    pages_per = 5
    table = torch.randperm(b * pages_per).to(torch.int32).reshape(b, pages_per)
    kc, ks = oracle.quantize_fp8_e4m3_per_head(torch.randn(b * pages_per, 16, hkv, d))
    vc, vs = oracle.quantize_fp8_e4m3_per_head(torch.randn(b * pages_per, 16, hkv, d))
    q = torch.randn(b, hq, d).to(torch.bfloat16)
    exp = oracle.reference(q, kc, vc, table.long(), lens, ks, vs)
    for split in (16, 32, 64, 512):
        for flags in (PLAN, FUSED, 0, 8, 1, 2, EARLY, EARLY | 8, EARLY | 1, PLAN | EARLY, FUSED | EARLY):
            out = torch.full_like(q, float("nan"), device=DEV)
            want = expected_path(cabi, q, hkv, flags)
            rows = cabi.balanced_workspace_rows(hq, hkv) if balanced(want) else 0
            ws = workspace(q.to(DEV), 70, split, min_rows=rows)
            g = [t.to(DEV) for t in (q, kc, vc, table, lens)]
            plan = make_plan(cabi, want, flags, *g, ws, 70, split)
            cabi.paged_decode_fp8_e4m3_split_out(
                *g, k_scale=ks.to(DEV), v_scale=vs.to(DEV),
                max_seq_len=70, split_size=split, output=out, workspace=ws, flags=flags & ~PLAN, plan=plan,
            )
            torch.cuda.synchronize()
            assert cabi.last_path() == want, f"flags={flags}"
            assert_within_gate(out, exp, f"d={d} hq={hq} hkv={hkv} split={split} flags={flags}")


def test_unused_slots_may_hold_nan_bytes(cabi):
    """Slots past seq_len inside the last page (and unused pages) are never trusted: fill
    them with the e4m3 NaN pattern."""
    w = make_inputs("qwen2.5-coder-3b-b64", seed=5, batch=6, shrink=0.1)
    exp = expected(w)
    kc = w.key_cache.clone().view(torch.uint8)
    vc = w.value_cache.clone().view(torch.uint8)
    for b in range(6):
        n = int(w.seq_lens[b])
        if n % 16:
            page = int(w.block_table[b, n // 16])
            kc[page, n % 16 :] = 0x7F
            vc[page, n % 16 :] = 0xFF
    w.key_cache, w.value_cache = kc.view(torch.float8_e4m3fn), vc.view(torch.float8_e4m3fn)
    for flags in (PLAN, FUSED, 0, 8, 1):
        assert_within_gate(run(cabi, w.to(DEV), 64, flags=flags), exp, "nan slots")


def test_max_seq_len_larger_than_every_sequence_and_empty_splits(cabi):
    w = make_inputs("qwen2.5-0.5b-b8", seed=2, shrink=0.25)
    exp = expected(w)
    wide = torch.zeros(8, 40, dtype=torch.int32)
    wide[:, : w.block_table.shape[1]] = w.block_table
    w.block_table = wide
    out = run(cabi, w.to(DEV), 64, max_seq_len=640)
    assert_within_gate(out, exp, "msl=640")


def test_consumer_right_behind_the_call_sees_finished_rows(cabi):
    """Stream order without a host synchronisation: a kernel enqueued right behind the call (here a
    copy of the output) must see finished rows.  The merge grid is a programmatic dependent of the
    partial grid; when every one of its rows is already final it must still not complete early.
    Cases: one short sequence (one warp group, nothing to merge), and lengths that all fit one
    split while max_seq_len asks for several."""
    torch.manual_seed(3)
    hq, hkv, d, pages = 16, 2, 128, 8
    for batch, ctx, msl, flags in ((1, 64, 64, 0), (1, 64, 64, EARLY), (3, 60, 640, 8), (3, 60, 640, EARLY | 8), (1, 64, 64, FUSED), (2, 640, 640, FUSED | EARLY), (2, 640, 640, PLAN | EARLY)):
        lens = torch.full((batch,), ctx, dtype=torch.int32)
        table = torch.randperm(batch * 40).to(torch.int32).reshape(batch, 40)
        kc, ks = oracle.quantize_fp8_e4m3_per_head(torch.randn(batch * 40, 16, hkv, d))
        vc, vs = oracle.quantize_fp8_e4m3_per_head(torch.randn(batch * 40, 16, hkv, d))
        q = torch.randn(batch, hq, d).to(torch.bfloat16)
        exp = oracle.reference(q, kc, vc, table.long(), lens, ks, vs)
        g = [t.to(DEV) for t in (q, kc, vc, table, lens, ks, vs)]
        want = expected_path(cabi, q, hkv, flags)
        rows = cabi.balanced_workspace_rows(hq, hkv) if balanced(want) else 0
        ws = workspace(g[0], msl, 64, min_rows=rows)
        plan = make_plan(cabi, want, flags, *g[:5], ws, msl, 64)
        torch.cuda.synchronize()
        out = torch.empty_like(g[0])
        copies = []
        for _ in range(200):
            out.fill_(float("nan"))
            cabi.paged_decode_fp8_e4m3_split_out(
                g[0], g[1], g[2], g[3], g[4], k_scale=g[5], v_scale=g[6], max_seq_len=msl, split_size=64,
                output=out, workspace=ws, flags=flags & ~PLAN, plan=plan)
            copies.append(out.clone())
        torch.cuda.synchronize()
        assert cabi.last_path() == want
        for c in copies:
            assert_within_gate(c, exp, f"batch={batch} ctx={ctx} max_seq_len={msl} flags={flags}")


def test_zero_length_sequence_gives_zeros(cabi):
    w = make_inputs("qwen2.5-0.5b-b8", seed=2, shrink=0.25)
    lens = w.seq_lens.clone()
    lens[3] = 0
    w.seq_lens = lens
    exp = expected(w)  # softmax over nothing is NaN in torch; the operator writes zeros there
    out = run(cabi, w.to(DEV), 64)
    assert (out[3] == 0).all()
    keep = [0, 1, 2, 4, 5, 6, 7]
    assert_within_gate(out[keep], exp[keep], "others")


@pytest.mark.parametrize("layout", ["hnd", "interleaved_kv", "padded_pages"])
def test_strided_cache_layouts(cabi, layout):
    """The reference's Triton path honours cache strides (l20_paged_split_kv.py:665-668);
    vLLM hands it `kv_cache.unbind(1)` views.  Same logical [pages,16,Hkv,D] view, other memory."""
    w = make_inputs("qwen2.5-coder-3b-b64", seed=7, batch=5, shrink=0.1)
    exp = expected(w)
    g = w.to(DEV)
    if layout == "hnd":
        g.key_cache = g.key_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        g.value_cache = g.value_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    elif layout == "interleaved_kv":
        both = torch.stack([g.key_cache.view(torch.uint8), g.value_cache.view(torch.uint8)], dim=1)
        k, v = both.view(torch.float8_e4m3fn).unbind(1)
        g.key_cache, g.value_cache = k, v
    else:
        pages, _, hkv, d = g.key_cache.shape
        big = torch.zeros(pages, 16, hkv + 1, d, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
        big2 = big.clone()
        big[:, :, :hkv] = g.key_cache
        big2[:, :, :hkv] = g.value_cache
        g.key_cache, g.value_cache = big[:, :, :hkv], big2[:, :, :hkv]
    assert not g.key_cache.is_contiguous()
    for flags in (PLAN, FUSED, 0, 8, 1):
        assert_within_gate(run(cabi, g, 64, flags=flags), exp, layout)


@pytest.mark.parametrize("pdtype", [torch.float32, torch.float16, torch.bfloat16])
def test_partial_workspace_dtypes(cabi, pdtype):
    """The reference keeps partial outputs in the query dtype (l20_paged_split_kv.py:24-26);
    callers that pass such a workspace still work (looser: one extra rounding per split)."""
    w = make_inputs("qwen2.5-coder-3b-b64", seed=3, batch=4, shrink=0.25)
    exp = expected(w)
    out = run(cabi, w.to(DEV), 128, partial_dtype=pdtype)
    if pdtype == torch.float32:
        assert_within_gate(out, exp, str(pdtype))
    else:
        assert torch.allclose(out.float().cpu(), exp.float(), atol=2e-2, rtol=2e-2)


def test_kv_start_suffix_pass_and_packed_partials_merge(cabi):
    """Prefix part + suffix part, each returned as packed (o, m, l), merged by pfd_merge_packed
    == attention over the whole range.  kv_start both page-aligned and not."""
    w = make_inputs("shared-prefix-b64", seed=4, batch=9, shrink=0.125)
    exp = expected(w)
    g = w.to(DEV)
    for cut in (w.prefix_len, w.prefix_len - 5, 3):
        head = g.to(DEV)
        head.seq_lens = torch.clamp(g.seq_lens, max=cut)
        p0 = run(cabi, head, 128, packed=True, max_seq_len=cut, flags=FUSED if cut == 3 else 0)
        p1 = run(cabi, g, 128, packed=True, kv_start=cut, flags=(FUSED if cut == 3 else PLAN) if cut % 2 else 8)
        out = torch.empty_like(g.query)
        cabi.merge_packed(torch.stack([p0, p1]).contiguous(), out)
        torch.cuda.synchronize()
        assert_within_gate(out, exp, f"cut={cut}")
        # the suffix alone equals the oracle restricted to [cut, len)
        has_suffix = (w.seq_lens > cut).nonzero().flatten().tolist()
        if has_suffix:
            sub = oracle.reference_fp32(
                w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale, kv_start=cut
            )
            o, m, l = p1[..., :-2], p1[..., -2], p1[..., -1]
            got = (o / l[..., None]).cpu()
            assert torch.allclose(got[has_suffix], sub[has_suffix], atol=2e-3, rtol=1e-2)
        empty = (w.seq_lens <= cut).nonzero().flatten().tolist()
        for b in empty:
            assert (p1[b, :, :-2] == 0).all() and torch.isneginf(p1[b, :, -2]).all() and (p1[b, :, -1] == 0).all()


def test_partials_match_oracle_split_semantics(cabi):
    """partial_max (natural log units), partial_sum and un-normalised partial_output of every
    live split equal the oracle's restatement of the reference partial kernel."""
    w = make_inputs("qwen2.5-0.5b-b8", seed=6, batch=4, shrink=0.5)
    split = 64
    ns = -(-w.max_seq_len // split)
    o, m, l = oracle.split_partials(
        w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale,
        split_size=split, num_splits=ns,
    )
    g = w.to(DEV)
    ws = workspace(g.query, w.max_seq_len, split, poison=False)
    out = torch.empty_like(g.query)
    cabi.paged_decode_fp8_e4m3_split_out(
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
        max_seq_len=w.max_seq_len, split_size=split, output=out, workspace=ws, flags=2,
    )
    torch.cuda.synchronize()
    po, pm, ps = (t.cpu() for t in ws[:3])
    for b in range(4):
        live = -(-int(w.seq_lens[b]) // split)
        assert torch.allclose(pm[b, :, :live], m[b, :, :live], atol=2e-3, rtol=1e-3)
        # rescale both to a common max before comparing sums / outputs
        c = torch.exp(pm[b, :, :live] - m[b, :, :live])
        assert torch.allclose(ps[b, :, :live] * c, l[b, :, :live], atol=1e-3, rtol=5e-3)
        assert torch.allclose(po[b, :, :live] * c[..., None], o[b, :, :live], atol=5e-3, rtol=1e-2)


def test_gather_indices_bit_exact(cabi):
    for name, kw in [("qwen2.5-0.5b-b8", {}), ("qwen2.5-7b-b256", {}), ("shared-prefix-b64", {})]:
        w = make_inputs(name, seed=0, shrink=0.25 if name != "qwen2.5-0.5b-b8" else 1.0)
        want = oracle.resolve_slots(w.block_table, w.seq_lens, w.max_seq_len)
        got = cabi.resolve_slots(w.block_table.to(DEV), w.seq_lens.to(DEV), w.max_seq_len)
        torch.cuda.synchronize()
        assert got.dtype == torch.int64 and torch.equal(got.cpu(), want), name


def test_block_table_permutation_invariance_and_idempotence(cabi):
    """Relocating every page (new permutation, caches moved accordingly) must not change a bit
    of the output; neither must running the same step twice into a reused workspace."""
    w = make_inputs("qwen2.5-coder-3b-b64", seed=8, batch=8, shrink=0.2).to(DEV)
    a = run(cabi, w, 128, flags=8)
    a2 = run(cabi, w, 128, flags=8)
    assert torch.equal(a.view(torch.int16), a2.view(torch.int16))
    pages = w.key_cache.shape[0]
    perm = torch.randperm(pages, device=DEV)
    moved = w.to(DEV)
    kc = torch.empty_like(w.key_cache.view(torch.uint8))
    vc = torch.empty_like(kc)
    kc[perm] = w.key_cache.view(torch.uint8)
    vc[perm] = w.value_cache.view(torch.uint8)
    moved.key_cache, moved.value_cache = kc.view(torch.float8_e4m3fn), vc.view(torch.float8_e4m3fn)
    moved.block_table = perm[w.block_table.long()].to(torch.int32)
    b = run(cabi, moved, 128, flags=8)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # the balanced path sums warps in a fixed order too: same bits run to run and after relocation
    c1, c2, c3 = run(cabi, w, 128, flags=0), run(cabi, w, 128, flags=0), run(cabi, moved, 128, flags=0)
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))
    assert torch.equal(c1.view(torch.int16), c3.view(torch.int16))
    # combined inside the balanced kernel the pieces of a cut sequence are folded in a fixed order as well
    c1, c2, c3 = run(cabi, w, 128, flags=FUSED), run(cabi, w, 128, flags=FUSED), run(cabi, moved, 128, flags=FUSED)
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))
    assert torch.equal(c1.view(torch.int16), c3.view(torch.int16))


def test_linearity_in_v_scale_and_scale_folding(cabi):
    w = make_inputs("qwen2.5-0.5b-b8", seed=9, batch=4, shrink=0.5).to(DEV)
    a = run(cabi, w, 64)
    b = run(cabi, w, 64, v_scale=w.v_scale * 2)
    assert torch.equal((a.float() * 2).to(torch.bfloat16).view(torch.int16), b.view(torch.int16))


def test_a_wait_that_nothing_satisfies_runs_out_and_sets_the_status_word(cabi):
    """Every device-side wait is bounded in time.  The self-test kernel arms a barrier for bytes
    that no copy delivers: the wait gives up after the limit, the kernel finishes, the error word
    reads 1 once and then 0 again, and the next decode call runs as usual."""
    assert cabi.device_status() == 0
    for limit_ns in (200_000, 3_000_000):
        waited = cabi.selftest_bounded_wait(limit_ns)
        assert limit_ns <= waited < limit_ns + 2_000_000, (limit_ns, waited)
        assert cabi.device_status() == 1
        assert cabi.device_status() == 0
    w = make_inputs("qwen2.5-coder-3b-b64", seed=12, batch=4, shrink=0.25)
    assert_within_gate(run(cabi, w.to(DEV), 128), expected(w), "decode after an expired wait")


# ---------------------------------------------------------------- dispatcher op (torch.ops) surface
def test_torch_op_reference_signature_and_wrapper_module(built_libs, golden):
    from single_gpu_inference_lab_b200 import l20_paged_decode, l20_paged_split_kv

    key, case = next(iter(golden["smoke"].items()))
    q, kc, vc, table, lens, ks, vs = smoke_recipe(
        case["batch"], case["context"], case["q_heads"], case["kv_heads"], oracle.quantize_fp8_e4m3
    )
    q, kc, vc, table, lens = (t.to(DEV) for t in (q, kc, vc, table, lens))
    splits = -(-case["context"] // 128)
    # exactly the call of scripts/smoke_cuda_paged_fp8_decode_op.py:89-111 (fp16 partial workspace)
    partial = torch.empty(case["batch"], case["q_heads"], splits, 128, device=DEV, dtype=torch.float16)
    maxima = torch.empty(case["batch"], case["q_heads"], splits, device=DEV)
    sums = torch.empty_like(maxima)
    output = torch.empty_like(q)
    actual = torch.ops.l20_stack.paged_decode_fp8_e4m3_split_out(
        q, kc, vc, table, lens, partial, maxima, sums, output, ks, vs, case["context"], 128
    )
    torch.cuda.synchronize()
    assert actual.data_ptr() == output.data_ptr()
    torch.testing.assert_close(actual.cpu(), case["output"], rtol=2e-2, atol=2e-2)  # the reference smoke's own gate
    # module-level wrapper with allocator, fp32 partials, bf16 query, per-head scales
    w = make_inputs("qwen2.5-coder-3b-b64", seed=0, batch=4, shrink=0.25)
    exp = expected(w)
    g = w.to(DEV)
    out = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
        max_seq_len=w.max_seq_len, split_size=256,
    )
    torch.cuda.synchronize()
    assert_within_gate(out, exp, "wrapper")
    with pytest.raises(RuntimeError, match="workspace shape does not match"):
        l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
            g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=1.0, v_scale=1.0,
            max_seq_len=w.max_seq_len, split_size=256,
            workspace=l20_paged_split_kv.allocate_l20_paged_split_kv_workspace(g.query[:2], 16, split_size=256),
        )
    with pytest.raises(RuntimeError, match="split_size must be a multiple of 16"):
        l20_paged_decode.paged_decode_fp8_e4m3_split_out(
            q, kc, vc, table, lens, partial, maxima, sums, output, ks, vs, case["context"], 100
        )
    assert l20_paged_decode.resolve_slots(table, lens, case["context"]).shape == (case["batch"], case["context"])


def test_cuda_graph_capture_and_replay(built_libs):
    """The op makes no host sync and no allocation, so it captures (the reference switches its
    hook off while capturing, install_l20_fp8_paged_decode.py:72; its fp16 sibling is graph
    tested in scripts/stress_cuda_paged_decode.py:129-167)."""
    from single_gpu_inference_lab_b200 import l20_paged_split_kv as m

    w = make_inputs("qwen2.5-coder-3b-b64", seed=1, batch=4, shrink=0.25)
    exp = expected(w)
    g = w.to(DEV)
    ws = m.allocate_l20_paged_split_kv_workspace(g.query, w.max_seq_len, split_size=128)
    m.l20_paged_split_kv_attention_fp8(
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
        max_seq_len=w.max_seq_len, split_size=128, workspace=ws,
    )
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    ws[3].zero_()
    with torch.cuda.graph(graph):
        m.l20_paged_split_kv_attention_fp8(
            g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
            max_seq_len=w.max_seq_len, split_size=128, workspace=ws,
        )
    for _ in range(3):
        ws[3].zero_()
        graph.replay()
    torch.cuda.synchronize()
    assert_within_gate(ws[3], exp, "graph replay")
