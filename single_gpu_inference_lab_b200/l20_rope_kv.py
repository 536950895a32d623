"""Fused rotary embedding + paged KV-cache append, B200 build, with FP8-e4m3 caches.

Same call as the reference's vLLM operator ``l20_rope_and_cache``
(integrations/vllm/l20_rope_kv.py:256-328): Q and K are rotated in place and K, V are written
to the NHD cache at ``slot_mapping``.  The reference refuses quantised caches (":273-274,
"quantized KV cache is not supported"); here ``key_cache`` / ``value_cache`` may also be
``torch.float8_e4m3fn`` (or ``uint8``), in which case ``k_scale`` / ``v_scale`` -- per-layer
floats or ``[Hkv]`` float32 tensors, the scales the decode operator dequantises with -- are
required.  One CUDA kernel behind ``torch.ops.l20_stack.rope_and_cache``; no Triton, no fallback.
"""

from __future__ import annotations

import torch

from .l20_paged_split_kv import REQUIRED_CAPABILITY, _on_required_gpu, _scale_vector


def l20_rope_and_cache(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    positions: torch.Tensor,
    cos_sin_cache: torch.Tensor,
    is_neox: bool,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    *,
    k_scale: float | torch.Tensor | None = None,
    v_scale: float | torch.Tensor | None = None,
) -> None:
    if not _on_required_gpu(query):
        raise RuntimeError("l20_rope_and_cache requires an SM100 GPU")
    if query.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("l20_rope_and_cache supports FP16 and BF16")
    if key.dtype != query.dtype or value.dtype != query.dtype:
        raise RuntimeError("Q, K, and V must use the same dtype")
    quantised = key_cache.dtype in (torch.float8_e4m3fn, torch.uint8)
    if not quantised and (key_cache.dtype != query.dtype or value_cache.dtype != query.dtype):
        raise RuntimeError("the caches must be FP8-e4m3 or have the query's dtype")
    if query.ndim != 3 or key.ndim != 3 or value.ndim != 3:
        raise RuntimeError("Q, K, and V must be [tokens, heads, head_dim]")
    if key.shape != value.shape or query.shape[0] != key.shape[0]:
        raise RuntimeError("Q, K, and V shapes are incompatible")
    if key_cache.ndim != 4 or value_cache.shape != key_cache.shape:
        raise RuntimeError("cache must use NHD [blocks, block, heads, dim]")
    if key_cache.shape[2:] != key.shape[1:]:
        raise RuntimeError("cache head shape must match K/V")
    if positions.numel() != query.shape[0] or slot_mapping.numel() != query.shape[0]:
        raise RuntimeError("positions and slot_mapping must match token count")
    rotary_dim = cos_sin_cache.shape[1]
    if rotary_dim <= 0 or rotary_dim > query.shape[2] or rotary_dim % 2:
        raise RuntimeError("invalid cos_sin_cache rotary dimension")
    scales = (None, None)
    if quantised:
        if k_scale is None or v_scale is None:
            raise RuntimeError("FP8 caches need k_scale and v_scale")
        hkv = key.shape[1]

        def vec(s):
            if isinstance(s, torch.Tensor):
                return s.to(device=query.device, dtype=torch.float32).reshape(-1).expand(hkv).contiguous()
            return _scale_vector(s, hkv, query.device)

        scales = (vec(k_scale), vec(v_scale))
    from . import l20_paged_decode  # noqa: F401  (loads the operator library)

    torch.ops.l20_stack.rope_and_cache(
        query, key, value, positions, cos_sin_cache, bool(is_neox), key_cache, value_cache, slot_mapping, *scales
    )


__all__ = ["l20_rope_and_cache", "REQUIRED_CAPABILITY"]
