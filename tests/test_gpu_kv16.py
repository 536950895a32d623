"""Parity of the non-quantised sibling (fp16 / bf16 K/V caches) against the CPU oracle, through
the C ABI and the dispatcher op.  Gate as for the FP8 path: |a - b| <= 2e-3 + 1e-2 * |b|."""

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import make_inputs

from helpers import assert_within_gate

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PATH_KV16 = 4
PATH_KV16_FUSED = 6


@pytest.fixture(scope="module")
def cabi(built_libs):
    from single_gpu_inference_lab_b200 import cabi as module

    module.load()
    return module


def workspace(q, splits, dtype=torch.float32):
    b, hq, d = q.shape
    return (
        torch.full((b, hq, splits, d), float("nan"), device=q.device, dtype=dtype),
        torch.full((b, hq, splits), float("nan"), device=q.device),
        torch.full((b, hq, splits), float("nan"), device=q.device),
        None,
    )


def run(cabi, w, *, splits=None, partial_dtype=torch.float32, kv_start=0, packed=False, flags=0, planned=False):
    """planned: pfd_plan_decode first, then the call with that plan; "fused": with
    PFD_FLAG_SINGLE_LAUNCH on top (pieces combined inside the balanced kernel)."""
    if planned == "fused":
        flags |= 64
    q = w.query
    hkv = w.key_cache.shape[2]
    if splits is None:  # room for every warp group
        splits = max(1, -(-cabi.balanced_workspace_rows(q.shape[1], hkv) // (q.shape[0] * q.shape[1])))
    out = torch.full_like(q, float("nan"))
    pk = torch.full((q.shape[0], q.shape[1], q.shape[2] + 2), float("nan"), device=q.device) if packed else None
    ws = workspace(q, splits, partial_dtype)
    plan = None
    if planned:
        plan = cabi.plan_decode(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, max_seq_len=w.max_seq_len,
                                split_size=512, workspace=ws, kv_start=kv_start)
    cabi.paged_decode_kv16_split_out(
        q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, max_seq_len=w.max_seq_len, split_size=512,
        output=None if packed else out, packed_output=pk, workspace=ws,
        kv_start=kv_start, flags=flags, plan=plan,
    )
    torch.cuda.synchronize()
    assert cabi.device_status() == 0, "a bounded device-side wait gave up"
    assert cabi.last_path() == (PATH_KV16_FUSED if planned == "fused" and partial_dtype == torch.float32 else PATH_KV16)
    return pk if packed else out


def expected(w, **kw):
    return oracle.reference_kv16(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, **kw)


@pytest.mark.parametrize(
    "name", ["kv16-cfg2-coder3b-b4-bf16", "kv16-cfg3-qwen7b-b24-bf16", "kv16-cfg4-llama8b-b2-fp16"]
)
def test_against_committed_reference_outputs(cabi, golden, name):
    case = golden["kv16"][name]
    dtype = getattr(torch, case["dtype"])
    w = make_inputs(case["workload"], seed=0, device="cpu", batch=case["batch"], shrink=case["shrink"],
                    query_dtype=dtype, kv_dtype=dtype)
    for splits in (None, 1, 3):  # full capacity; the smallest legal workspaces (few warp groups)
        for planned in (False, True, "fused"):
            assert_within_gate(run(cabi, w.to(DEV), splits=splits, planned=planned), case["output"],
                               f"{name} splits={splits} planned={planned}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_config2_and_config3_full_size(cabi, dtype):
    for name in ("qwen2.5-coder-3b-b64", "qwen2.5-7b-b256"):
        w = make_inputs(name, seed=0, query_dtype=dtype, kv_dtype=dtype)
        exp = expected(w)
        assert_within_gate(run(cabi, w.to(DEV)), exp, f"{name} {dtype}")
        assert_within_gate(run(cabi, w.to(DEV), planned=True, flags=32), exp, f"{name} {dtype} planned")
        assert_within_gate(run(cabi, w.to(DEV), planned=True, flags=32 | 256), exp, f"{name} {dtype} planned, early K/V")
        assert_within_gate(run(cabi, w.to(DEV), planned="fused", flags=32), exp, f"{name} {dtype} fused")


@pytest.mark.parametrize("hq,hkv", [(16, 2), (28, 4), (32, 8), (8, 8), (12, 2)])
def test_every_short_context_length(cabi, hq, hkv):
    """ctx = 1 .. 70 in one batch: ragged tails, single page, page boundary +-1."""
    torch.manual_seed(11)
    lens = torch.arange(1, 71, dtype=torch.int32)
    b, pages_per, d = lens.numel(), 5, 128
    table = torch.randperm(b * pages_per).to(torch.int32).reshape(b, pages_per)
    for dtype in (torch.bfloat16, torch.float16):
        kc = torch.randn(b * pages_per, 16, hkv, d).to(dtype)
        vc = torch.randn(b * pages_per, 16, hkv, d).to(dtype)
        # slots past the end of a sequence may hold anything: poison them
        for s in range(b):
            n = int(lens[s])
            if n % 16:
                page = int(table[s, n // 16])
                kc[page, n % 16 :] = float("nan")
                vc[page, n % 16 :] = float("inf")
        q = torch.randn(b, hq, d).to(dtype)
        exp = oracle.reference_kv16(q, kc, vc, table.long(), lens)
        out = torch.full_like(q, float("nan"), device=DEV)
        cabi.paged_decode_kv16_split_out(
            q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), lens.to(DEV), max_seq_len=70, split_size=64,
            output=out, workspace=workspace(q.to(DEV), 8),
        )
        torch.cuda.synchronize()
        assert_within_gate(out, exp, f"hq={hq} hkv={hkv} {dtype}")


def test_hnd_layout_partial_dtypes_kv_start_and_packed_output(cabi):
    w = make_inputs("qwen2.5-coder-3b-b64", seed=7, batch=6, shrink=0.2, kv_dtype=torch.bfloat16)
    exp = expected(w)
    g = w.to(DEV)
    g.key_cache = g.key_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    g.value_cache = g.value_cache.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert not g.key_cache.is_contiguous()
    assert_within_gate(run(cabi, g), exp, "hnd")
    assert_within_gate(run(cabi, g, planned=True), exp, "hnd planned")
    assert_within_gate(run(cabi, g, planned="fused"), exp, "hnd fused")
    for pdtype in (torch.float16, torch.bfloat16):  # the reference keeps partials in the query dtype
        for planned in (False, "fused"):  # a plan is ignored for 16-bit partials
            out = run(cabi, g, partial_dtype=pdtype, planned=planned)
            assert torch.allclose(out.float().cpu(), exp.float(), atol=2e-2, rtol=2e-2)
    # suffix only, as packed (o, m, l)
    cut = 100
    pk2 = run(cabi, g, kv_start=cut, packed=True, planned="fused")
    pk = run(cabi, g, kv_start=cut, packed=True)
    assert torch.allclose((pk2[..., :-2] / pk2[..., -1:]).nan_to_num(), (pk[..., :-2] / pk[..., -1:]).nan_to_num(), atol=1e-5, rtol=1e-4)
    sub = oracle.reference_kv16(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, kv_start=cut)
    has = (w.seq_lens > cut).nonzero().flatten().tolist()
    got = (pk[..., :-2] / pk[..., -1:]).cpu()
    assert torch.allclose(got[has].float(), sub[has].float(), atol=4e-3, rtol=2e-2)


def test_dispatcher_op_with_the_reference_smoke_call(built_libs):
    """The call of scripts/smoke_cuda_paged_decode_op.py:49-80: seed 17, fp16, 12 q / 2 kv heads,
    fp16 partial workspace with ceil(context / 64) splits."""
    from single_gpu_inference_lab_b200 import l20_paged_decode, l20_paged_split_kv  # noqa: F401

    for batch, context in ((1, 129), (3, 1000), (1, 50)):  # the last: one request, one split, 12 workspace rows
        torch.manual_seed(17)
        pages_per = (context + 15) // 16
        pages = batch * pages_per
        table = torch.randperm(pages, dtype=torch.int32).reshape(batch, pages_per)
        lens = torch.full((batch,), context, dtype=torch.int32)
        q = torch.randn(batch, 12, 128, dtype=torch.float16)
        kc = torch.randn(pages, 16, 2, 128, dtype=torch.float16)
        vc = torch.randn_like(kc)
        exp = oracle.reference_kv16(q, kc, vc, table.long(), lens)
        splits = (context + 63) // 64
        q, kc, vc, table, lens = (t.to(DEV) for t in (q, kc, vc, table, lens))
        partial = torch.empty(batch, 12, splits, 128, device=DEV, dtype=torch.float16)
        maxima = torch.empty(batch, 12, splits, device=DEV)
        sums = torch.empty_like(maxima)
        output = torch.empty_like(q)
        actual = torch.ops.l20_stack.paged_decode_split_out(q, kc, vc, table, lens, partial, maxima, sums, output, context, 64)
        torch.cuda.synchronize()
        assert actual.data_ptr() == output.data_ptr()
        torch.testing.assert_close(actual.cpu(), exp, rtol=2e-2, atol=2e-2)  # the reference smoke's own gate
        out2 = l20_paged_split_kv.l20_paged_split_kv_attention(q, kc, vc, table, lens, split_size=64)
        torch.cuda.synchronize()
        assert_within_gate(out2, exp, "wrapper with its own workspace")


def test_indptr_indices_addressing_matches_block_table(cabi, built_libs):
    """FlashInfer's addressing (flat page list + indptr) gives the bits the block table gives,
    for the 16-bit operator (C ABI and dispatcher op) and for the FP8 operator's balanced path."""
    from single_gpu_inference_lab_b200 import l20_paged_decode

    w16 = make_inputs("qwen2.5-7b-b256", seed=3, batch=40, shrink=0.25, kv_dtype=torch.bfloat16).to(DEV)
    w8 = make_inputs("qwen2.5-7b-b256", seed=3, batch=40, shrink=0.25).to(DEV)
    for w, call in ((w16, cabi.paged_decode_kv16_split_out), (w8, cabi.paged_decode_fp8_e4m3_split_out)):
        q = w.query
        pages = (w.seq_lens.cpu() + 15) // 16
        indptr = torch.zeros(q.shape[0] + 1, dtype=torch.int32)
        indptr[1:] = torch.cumsum(pages, 0)
        indices = torch.cat([w.block_table[b, : int(pages[b])].cpu() for b in range(q.shape[0])]).to(torch.int32)
        splits = -(-cabi.balanced_workspace_rows(q.shape[1], w.key_cache.shape[2]) // (q.shape[0] * q.shape[1]))
        outs = []
        for table, ptr in ((w.block_table, None), (indices.to(DEV), indptr.to(DEV))):
            out = torch.full_like(q, float("nan"))
            call(q, w.key_cache, w.value_cache, table, w.seq_lens, k_scale=w.k_scale, v_scale=w.v_scale,
                 max_seq_len=w.max_seq_len, split_size=512, output=out, workspace=workspace(q, splits),
                 page_indptr=ptr)
            torch.cuda.synchronize()
            assert cabi.device_status() == 0
            outs.append(out)
        assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
        if w is w16:
            assert_within_gate(outs[1], expected(w), "indptr addressing")
            ws = workspace(q, splits)
            out = torch.full_like(q, float("nan"))
            l20_paged_decode.paged_decode_split_indices_out(
                q, w.key_cache, w.value_cache, indptr.to(DEV), indices.to(DEV), w.seq_lens, ws[0], ws[1], ws[2], out,
                w.max_seq_len, 512)
            torch.cuda.synchronize()
            assert torch.equal(out.view(torch.int16), outs[0].view(torch.int16))
    # a call that cannot take the balanced path refuses the addressing instead of misreading the list
    small = workspace(w8.query, -(-w8.max_seq_len // 512))
    with pytest.raises(RuntimeError, match="page_indptr addressing needs the balanced kernel"):
        cabi.paged_decode_fp8_e4m3_split_out(
            w8.query, w8.key_cache, w8.value_cache, indices.to(DEV), w8.seq_lens, k_scale=w8.k_scale, v_scale=w8.v_scale,
            max_seq_len=w8.max_seq_len, split_size=512, output=torch.empty_like(w8.query), workspace=small,
            page_indptr=indptr.to(DEV), flags=8)
