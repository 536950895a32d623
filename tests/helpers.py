"""Shared helpers of the test-suite (input digests, tolerance gate, smoke recipe)."""

from __future__ import annotations

import hashlib

import torch

ATOL = 2e-3  # max-abs gate on bf16 outputs
RTOL = 1e-2  # max-rel gate on bf16 outputs


def digest(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        elif t.dtype in (torch.bfloat16, torch.float16):
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def assert_within_gate(actual: torch.Tensor, expected: torch.Tensor, what: str = "") -> float:
    """``|a - b| <= 2e-3 + 1e-2 * |b|`` element-wise on the (bf16/fp16) outputs; returns max-abs."""
    a, b = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.isfinite(a).all(), f"{what}: non-finite output"
    err = (a - b).abs()
    bound = ATOL + RTOL * b.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"{what}: max_abs={err.max().item():.3e}, exceeds gate by {worst:.3e}"
    return err.max().item()


def smoke_recipe(batch: int, context: int, q_heads: int, kv_heads: int, quantize):
    """Input recipe of the reference smoke (scripts/smoke_cuda_paged_fp8_decode_op.py:71-88)
    on the CPU generator: seed 29, uniform context, fp16 query, per-tensor scales."""
    torch.manual_seed(29)
    pages_per_request = (context + 15) // 16
    pages = batch * pages_per_request
    table = torch.randperm(pages).to(torch.int32).reshape(batch, pages_per_request)
    seq_lens = torch.full((batch,), context, dtype=torch.int32)
    query = torch.randn(batch, q_heads, 128, dtype=torch.float16)
    key_bf16 = torch.randn(pages, 16, kv_heads, 128, dtype=torch.bfloat16)
    value_bf16 = torch.randn_like(key_bf16)
    key_cache, k_scale = quantize(key_bf16)
    value_cache, v_scale = quantize(value_bf16)
    return query, key_cache, value_cache, table, seq_lens, k_scale, v_scale
