"""The allocation-free entry point (split-KV partials in the array built into the library, for
hosts that cannot allocate a workspace: all HBM already given to the KV cache, or no tensor
allocator at all) against the ordinary entry point, through the C ABI.

Collected last on purpose: a failure here cannot hide a failure elsewhere under ``-x``.
"""

import ctypes

import pytest
import torch

from oracle import paged_decode_oracle as oracle
from single_gpu_inference_lab_b200.workloads import make_inputs

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _both(cabi, w, split):
    q = w.query
    dev = q.device
    splits = -(-w.max_seq_len // split)
    ws = (
        torch.empty(q.shape[0], q.shape[1], splits, q.shape[2], device=dev),
        torch.empty(q.shape[0], q.shape[1], splits, device=dev),
        torch.empty(q.shape[0], q.shape[1], splits, device=dev),
    )
    common = dict(k_scale=w.k_scale, v_scale=w.v_scale, max_seq_len=w.max_seq_len, split_size=split)
    want = torch.full_like(q, float("nan"))
    cabi.paged_decode_fp8_e4m3_split_out(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, output=want, workspace=ws, **common)
    got = torch.full_like(q, float("nan"))
    cabi.paged_decode_fp8_e4m3_split_out_noalloc(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, output=got, **common)
    torch.cuda.synchronize(dev)
    return got, want


def _within_gate(got, want):
    err = (got.float().cpu() - want.float().cpu()).abs()
    return bool((err <= 2e-3 + 1e-2 * want.float().cpu().abs()).all()), err.max().item()


def test_noalloc_entry_matches_workspace_entry_on_two_calls_in_a_row(built_libs):
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    # first call: many splits per sequence; second call: other geometry, fewer and differently
    # placed partials, so anything left in the shared array by the first call is stale for it
    # and both are held against the CPU oracle, not only against each other
    first = make_inputs("qwen2.5-coder-3b-b64", seed=21, batch=16, shrink=0.5)
    second = make_inputs("qwen2.5-0.5b-b8", seed=22)
    for w, split in ((first, 64), (second, 128)):
        exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
        got, want = _both(cabi, w.to(DEV), split)
        assert torch.isfinite(got.float()).all()
        ok, worst = _within_gate(got, want)
        assert ok, worst
        ok, worst = _within_gate(got, exp)
        assert ok, worst


def test_noalloc_entry_on_a_second_device(built_libs):
    """Every device that loads the library has its own copy of the array and its own address of
    it: the first call on another device must look that address up, not reuse device 0's."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    w = make_inputs("qwen2.5-coder-3b-b64", seed=24, batch=8, shrink=0.25)
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        got, want = _both(cabi, w.to(dev), 64)
        ok, worst = _within_gate(got, exp)
        assert ok, (dev, worst)


def test_noalloc_entry_without_partials_and_its_refusals(built_libs):
    """A request whose longest sequence fits one split touches no scratch and is never refused for
    size; indptr addressing and partial-only runs are refused with their own messages."""
    from single_gpu_inference_lab_b200 import cabi

    lib = cabi.load()
    w = make_inputs("qwen2.5-7b-b256", seed=25, batch=256, shrink=0.06)  # 256 x 28 rows, lengths <= 492
    exp = oracle.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens, w.k_scale, w.v_scale)
    g = w.to(DEV)
    assert 256 * 28 * 130 * 4 * 4 > cabi.NOALLOC_SCRATCH_BYTES  # four splits would not fit ...
    got = torch.full_like(g.query, float("nan"))
    cabi.paged_decode_fp8_e4m3_split_out_noalloc(  # ... one split needs none
        g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale, v_scale=g.v_scale,
        max_seq_len=w.max_seq_len, split_size=512, output=got)
    torch.cuda.synchronize()
    ok, worst = _within_gate(got, exp)
    assert ok, worst
    before = cabi.launch_count()
    indptr = torch.zeros(257, dtype=torch.int32, device=DEV)
    for kw, text in ((dict(page_indptr=indptr), b"page_indptr"), (dict(flags=4), b"PARTIAL_ONLY")):
        args = cabi.decode_args(g.query, g.key_cache, g.value_cache, g.block_table, g.seq_lens, k_scale=g.k_scale,
                                v_scale=g.v_scale, max_seq_len=w.max_seq_len, split_size=512, output=got, **kw)
        assert lib.pfd_paged_decode_fp8_e4m3_split_out_noalloc(ctypes.byref(args)) == -2
        assert text in lib.pfd_last_error()
    assert cabi.launch_count() == before


def test_noalloc_entry_refuses_requests_beyond_its_array(built_libs):
    from single_gpu_inference_lab_b200 import cabi

    lib = cabi.load()
    w = make_inputs("qwen2.5-coder-3b-b64", seed=23, batch=64, shrink=1.0).to(DEV)
    out = torch.empty_like(w.query)
    before = cabi.launch_count()
    args = cabi.decode_args(
        w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens, k_scale=w.k_scale, v_scale=w.v_scale,
        max_seq_len=w.max_seq_len, split_size=16, output=out,
    )
    need = 64 * 16 * -(-w.max_seq_len // 16) * 130 * 4
    assert need > cabi.NOALLOC_SCRATCH_BYTES
    rc = lib.pfd_paged_decode_fp8_e4m3_split_out_noalloc(ctypes.byref(args))
    assert rc == -2 and b"scratch" in lib.pfd_last_error()
    assert cabi.launch_count() == before
