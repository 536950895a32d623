"""The allocation-free entry point (split-KV partials in the array built into the library, for
hosts that cannot allocate a workspace: all HBM already given to the KV cache, or no tensor
allocator at all) against the ordinary entry point, through the C ABI.

Collected last on purpose: a failure here cannot hide a failure elsewhere under ``-x``.
"""

import ctypes

import pytest
import torch

from single_gpu_inference_lab_b200.workloads import make_inputs

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _both(cabi, w, split):
    q = w.query
    splits = -(-w.max_seq_len // split)
    ws = (
        torch.empty(q.shape[0], q.shape[1], splits, q.shape[2], device=DEV),
        torch.empty(q.shape[0], q.shape[1], splits, device=DEV),
        torch.empty(q.shape[0], q.shape[1], splits, device=DEV),
    )
    common = dict(k_scale=w.k_scale, v_scale=w.v_scale, max_seq_len=w.max_seq_len, split_size=split)
    want = torch.full_like(q, float("nan"))
    cabi.paged_decode_fp8_e4m3_split_out(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, output=want, workspace=ws, **common)
    got = torch.full_like(q, float("nan"))
    cabi.paged_decode_fp8_e4m3_split_out_noalloc(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, output=got, **common)
    torch.cuda.synchronize()
    return got, want


def test_noalloc_entry_matches_workspace_entry_on_two_calls_in_a_row(built_libs):
    from single_gpu_inference_lab_b200 import cabi

    cabi.load()
    # first call: many splits per sequence; second call: other geometry, fewer and differently
    # placed partials, so anything left in the shared array by the first call is stale for it
    first = make_inputs("qwen2.5-coder-3b-b64", seed=21, batch=16, shrink=0.5).to(DEV)
    second = make_inputs("qwen2.5-0.5b-b8", seed=22).to(DEV)
    for w, split in ((first, 64), (second, 128)):
        got, want = _both(cabi, w, split)
        assert torch.isfinite(got.float()).all()
        err = (got.float() - want.float()).abs()
        assert (err <= 2e-3 + 1e-2 * want.float().abs()).all(), err.max().item()


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
