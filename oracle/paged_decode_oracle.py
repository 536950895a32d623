"""CPU oracle for paged FP8-e4m3 KV-cache GQA decode attention.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke
entry and the benchmark's CPU-baseline / reference arm may import it; the
operator itself never does and has no CPU fallback.

It is a device-agnostic restatement (plain torch, CPU) of the reference
project's own torch implementation of this path:

* ``quantize_fp8_e4m3``        <- scripts/smoke_cuda_paged_fp8_decode_op.py:13-19
* ``reference``                <- scripts/smoke_cuda_paged_fp8_decode_op.py:22-41
* ``split_partials`` / ``merge_partials``
                               <- integrations/vllm/l20_paged_split_kv.py:134-239
                                  (partial) and :459-488 (LSE reduce), also
                                  integrations/vllm/cuda/l20_paged_decode.cu:424-463
* ``resolve_slots``            <- the gather expression of the reference,
                                  scripts/smoke_cuda_paged_fp8_decode_op.py:29-33
* ``find_shared_prefix_groups``<- integrations/vllm/l20_shared_prefix_decode_dispatch.py:41-76

Parity is pinned: ``tests/golden/make_golden.py`` imports the reference's own
``reference()`` / ``quantize_fp8_e4m3`` from its source tree, runs them on seeded
inputs and stores the outputs under ``tests/golden/``; ``tests/test_oracle.py``
requires this restatement to reproduce those outputs bit for bit.

The only generalisations over the reference function are (a) tensors stay on
the device of ``query`` instead of a hard-coded "cuda", (b) ``k_scale`` /
``v_scale`` may be a float (per tensor, as in the reference) or a ``[Hkv]``
tensor (per kv head), (c) an optional explicit softmax scale and ``kv_start``.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Sequence, Union

import torch

PAGE_SIZE = 16
Scale = Union[float, torch.Tensor]


def quantize_fp8_e4m3(tensor: torch.Tensor) -> tuple[torch.Tensor, float]:
    """Per-tensor e4m3 quantisation (smoke_cuda_paged_fp8_decode_op.py:13-19)."""
    finfo = torch.finfo(torch.float8_e4m3fn)
    scale = max(float(tensor.float().abs().max()) / finfo.max, 1.0e-12)
    quantized = (tensor.float() / scale).clamp(finfo.min, finfo.max).to(
        torch.float8_e4m3fn
    )
    return quantized, scale


def quantize_fp8_e4m3_per_head(tensor: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Same recipe with one scale per kv head of a ``[pages, 16, Hkv, D]`` cache."""
    finfo = torch.finfo(torch.float8_e4m3fn)
    amax = tensor.float().abs().amax(dim=(0, 1, 3))
    scale = (amax / finfo.max).clamp_min(1.0e-12)
    quantized = (
        (tensor.float() / scale[None, None, :, None])
        .clamp(finfo.min, finfo.max)
        .to(torch.float8_e4m3fn)
    )
    return quantized, scale.to(torch.float32)


def _broadcast_scale(scale: Scale, like: torch.Tensor):
    if isinstance(scale, torch.Tensor) and scale.ndim >= 1:
        return scale.to(torch.float32).reshape(1, 1, -1, 1)
    return float(scale)


def dequantize(cache: torch.Tensor, scale: Scale) -> torch.Tensor:
    """``(fp8.float() * scale).to(float16)`` -- the reference rounds the
    dequantised cache to fp16 before any maths (smoke...:23-24)."""
    return (cache.float() * _broadcast_scale(scale, cache)).to(torch.float16)


def resolve_slots(
    block_table: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int | None = None
) -> torch.Tensor:
    """Integer slot index ``page * 16 + offset`` the path gathers for every
    (sequence, token); ``-1`` beyond the sequence.  Same expression as the
    reference's gather (``physical = table[b, t // 16]; offsets = t % 16``)."""
    batch = block_table.shape[0]
    if max_seq_len is None:
        max_seq_len = int(seq_lens.max()) if batch else 0
    token = torch.arange(max_seq_len, dtype=torch.int64)
    slots = torch.full((batch, max_seq_len), -1, dtype=torch.int64)
    for b in range(batch):
        length = int(seq_lens[b])
        t = token[:length]
        slots[b, :length] = block_table[b, t // PAGE_SIZE].to(torch.int64) * PAGE_SIZE + t % PAGE_SIZE
    return slots


def reference_fp32(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_scale: Scale,
    v_scale: Scale,
    *,
    sm_scale: float | None = None,
    kv_start: int = 0,
) -> torch.Tensor:
    """The reference computation, returned before the final cast (fp32)."""
    key_dequant = dequantize(key_cache, k_scale)
    value_dequant = dequantize(value_cache, v_scale)
    scale = query.shape[-1] ** -0.5 if sm_scale is None else float(sm_scale)
    outputs = []
    for batch in range(query.shape[0]):
        length = int(seq_lens[batch])
        token = torch.arange(kv_start, length, device=query.device)
        physical = table[batch, token // PAGE_SIZE]
        offsets = token % PAGE_SIZE
        keys = key_dequant[physical, offsets]
        values = value_dequant[physical, offsets]
        kv_heads = keys.shape[1]
        group = query.shape[1] // kv_heads
        keys = keys.repeat_interleave(group, dim=1)
        values = values.repeat_interleave(group, dim=1)
        scores = torch.einsum("hd,thd->ht", query[batch].float(), keys.float()) * scale
        probs = scores.softmax(dim=-1)
        outputs.append(torch.einsum("ht,thd->hd", probs, values.float()))
    return torch.stack(outputs)


def reference(query, key_cache, value_cache, table, seq_lens, k_scale, v_scale, **kw):
    """Restatement of ``reference()`` (smoke_cuda_paged_fp8_decode_op.py:22-41):
    dequantise -> fp16 rounding -> fp32 einsum / softmax / einsum -> query dtype."""
    return reference_fp32(
        query, key_cache, value_cache, table, seq_lens, k_scale, v_scale, **kw
    ).to(query.dtype)


def reference_kv16(query, key_cache, value_cache, table, seq_lens, *, kv_start: int = 0) -> torch.Tensor:
    """The non-quantised sibling: restatement of ``reference()`` of
    scripts/smoke_cuda_paged_decode_op.py:13-30 (caches in the query's fp16 / bf16 type, no
    scales): per sequence gather ``table[b, t // 16]``, ``t % 16``; fp32 einsum / softmax /
    einsum; cast to the query dtype."""
    scale = query.shape[-1] ** -0.5
    outputs = []
    for batch in range(query.shape[0]):
        length = int(seq_lens[batch])
        token = torch.arange(kv_start, length, device=query.device)
        physical = table[batch, token // PAGE_SIZE]
        offsets = token % PAGE_SIZE
        keys = key_cache[physical, offsets]
        values = value_cache[physical, offsets]
        kv_heads = keys.shape[1]
        group = query.shape[1] // kv_heads
        keys = keys.repeat_interleave(group, dim=1)
        values = values.repeat_interleave(group, dim=1)
        scores = torch.einsum("hd,thd->ht", query[batch].float(), keys.float()) * scale
        probs = scores.softmax(dim=-1)
        outputs.append(torch.einsum("ht,thd->hd", probs, values.float()))
    return torch.stack(outputs).to(query.dtype)


def split_partials(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_scale: Scale,
    v_scale: Scale,
    *,
    split_size: int,
    num_splits: int,
    kv_start: int = 0,
    sm_scale: float | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-split ``(o unnormalised, m, l)`` in fp32 with the semantics of the
    reference's partial kernels (l20_paged_split_kv.py:134-239): split ``s``
    covers tokens ``[kv_start + s*split, kv_start + (s+1)*split) ∩ [0, seq_len)``;
    an empty split stores ``(0, -inf, 0)`` (:226-239)."""
    key_dequant = dequantize(key_cache, k_scale).float()
    value_dequant = dequantize(value_cache, v_scale).float()
    batch, q_heads, head_dim = query.shape
    scale = head_dim ** -0.5 if sm_scale is None else float(sm_scale)
    out = torch.zeros(batch, q_heads, num_splits, head_dim)
    mx = torch.full((batch, q_heads, num_splits), float("-inf"))
    sm = torch.zeros(batch, q_heads, num_splits)
    for b in range(batch):
        length = int(seq_lens[b])
        for s in range(num_splits):
            lo = kv_start + s * split_size
            hi = min(lo + split_size, length)
            if lo >= hi:
                continue
            token = torch.arange(lo, hi)
            physical = table[b, token // PAGE_SIZE]
            offsets = token % PAGE_SIZE
            keys = key_dequant[physical, offsets]
            values = value_dequant[physical, offsets]
            group = q_heads // keys.shape[1]
            keys = keys.repeat_interleave(group, dim=1)
            values = values.repeat_interleave(group, dim=1)
            scores = torch.einsum("hd,thd->ht", query[b].float(), keys) * scale
            m = scores.max(dim=-1).values
            p = torch.exp(scores - m[:, None])
            mx[b, :, s] = m
            sm[b, :, s] = p.sum(dim=-1)
            out[b, :, s] = torch.einsum("ht,thd->hd", p, values)
    return out, mx, sm


def merge_partials(
    partial_output: torch.Tensor, partial_max: torch.Tensor, partial_sum: torch.Tensor
) -> torch.Tensor:
    """LSE merge over the split axis (l20_paged_split_kv.py:459-488):
    ``M = max_s m_s; c_s = exp(m_s - M); out = sum c_s o_s / sum c_s l_s``."""
    global_max = partial_max.max(dim=-1, keepdim=True).values
    correction = torch.exp(partial_max - global_max)
    correction = torch.where(torch.isneginf(partial_max), torch.zeros_like(correction), correction)
    denominator = (partial_sum * correction).sum(dim=-1)
    numerator = (partial_output * correction[..., None]).sum(dim=-2)
    return numerator / denominator[..., None]


def merge_packed(packed: torch.Tensor) -> torch.Tensor:
    """Merge ``[N, B, Hq, D+2]`` packed partials (``o`` unnormalised, then
    ``m``, then ``l``), the cross-GPU exchange format of a KV-range split."""
    o = packed[..., :-2].permute(1, 2, 0, 3)
    m = packed[..., -2].permute(1, 2, 0)
    l = packed[..., -1].permute(1, 2, 0)
    return merge_partials(o, m, l)


def find_shared_prefix_groups(
    block_tables: torch.Tensor,
    prefix_lengths: Sequence[int] | torch.Tensor,
    *,
    min_batch: int = 8,
    min_prefix_length: int = 4096,
    page_size: int = PAGE_SIZE,
) -> list[list[int]]:
    """Group request indices by identical (prefix length, prefix block chain)
    (l20_shared_prefix_decode_dispatch.py:41-76)."""
    if block_tables.ndim != 2:
        raise ValueError("block_tables must have shape [B, max_pages]")
    lengths = [int(x) for x in (prefix_lengths.tolist() if isinstance(prefix_lengths, torch.Tensor) else prefix_lengths)]
    if len(lengths) != block_tables.shape[0]:
        raise ValueError("prefix_lengths must have one entry per request")
    groups: dict[tuple[int, tuple[int, ...]], list[int]] = defaultdict(list)
    for index, prefix_length in enumerate(lengths):
        if prefix_length < min_prefix_length:
            continue
        pages = (prefix_length + page_size - 1) // page_size
        key = (prefix_length, tuple(int(x) for x in block_tables[index, :pages].tolist()))
        groups[key].append(index)
    return [indices for indices in groups.values() if len(indices) >= min_batch]
