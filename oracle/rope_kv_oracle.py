"""CPU oracle of the producer step (rotary embedding + paged KV append).  TEST INFRASTRUCTURE:
only tests may import it; the product path never does.

``rope_and_cache`` restates, in torch on the CPU,

* the half-rotation (NeoX) arithmetic and the cache write of the reference's
  ``rope_kv_reference`` (src/l20_stack/ops/triton_rope_kv.py:147-173): products and sums in
  fp32, the result cast to the tensor's 16-bit type, K and V stored at their cache positions --
  pinned bit for bit to that function's outputs by ``tests/golden`` (key ``rope``);
* what the reference's vLLM operator adds (integrations/vllm/l20_rope_kv.py:26-253): the same
  rotation applied to Q in place, the interleaved (GPT-J) pairing when ``is_neox`` is false,
  ``slot_mapping`` addressing (block * block_size + offset, negative = skip), a
  ``[max_position, rotary_dim]`` cos/sin table indexed by ``positions``;
* and, beyond the reference (which refuses quantised caches), FP8-e4m3 caches: the rotated and
  16-bit-rounded key (and the value) divided by the per-kv-head scale in fp32, clamped to
  +-448, cast to ``float8_e4m3fn`` -- the inverse of what the decode oracle does.
  These two items have no reference output to be pinned to: parity unpinned beyond the formulas.
"""

from __future__ import annotations

import torch


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, is_neox: bool) -> torch.Tensor:
    """x [T, H, D]; cos, sin [T, rotary_dim / 2] -> rotated copy in x's dtype."""
    half = cos.shape[1]
    out = x.clone()
    if is_neox:
        first, second = x[:, :, :half].float(), x[:, :, half : 2 * half].float()
    else:
        first, second = x[:, :, 0 : 2 * half : 2].float(), x[:, :, 1 : 2 * half : 2].float()
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    y1 = (first * c - second * s).to(x.dtype)
    y2 = (second * c + first * s).to(x.dtype)
    if is_neox:
        out[:, :, :half], out[:, :, half : 2 * half] = y1, y2
    else:
        out[:, :, 0 : 2 * half : 2], out[:, :, 1 : 2 * half : 2] = y1, y2
    return out


def quantize(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x [T, Hkv, D] 16-bit, scale [Hkv] -> e4m3 bytes."""
    return (x.float() / scale.float().view(1, -1, 1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def rope_and_cache(query, key, value, positions, cos_sin_cache, is_neox, key_cache, value_cache, slot_mapping,
                   k_scale=None, v_scale=None):
    """Returns (query', key', key_cache', value_cache'); nothing is modified in place."""
    half = cos_sin_cache.shape[1] // 2
    rows = cos_sin_cache[positions.long()]
    cos, sin = rows[:, :half], rows[:, half:]
    q2, k2 = rotate(query, cos, sin, is_neox), rotate(key, cos, sin, is_neox)
    kc, vc = key_cache.clone(), value_cache.clone()
    keep = slot_mapping >= 0
    block_size = kc.shape[1]
    blocks, offsets = slot_mapping[keep] // block_size, slot_mapping[keep] % block_size
    if kc.dtype in (torch.float8_e4m3fn, torch.uint8):
        kq, vq = quantize(k2[keep], k_scale), quantize(value[keep], v_scale)
        kc.view(torch.uint8)[blocks, offsets] = kq.view(torch.uint8)
        vc.view(torch.uint8)[blocks, offsets] = vq.view(torch.uint8)
    else:
        kc[blocks, offsets] = k2[keep]
        vc[blocks, offsets] = value[keep]
    return q2, k2, kc, vc
