"""Seeded synthetic decode-step inputs for the paged FP8-KV decode path.

The reference project's own smoke and benchmark scripts build their inputs the
same way -- ``torch.randn`` data quantised with ``amax / 448`` and a
``torch.randperm`` block table (scripts/smoke_cuda_paged_fp8_decode_op.py:71-88,
scripts/benchmark_cuda_paged_fp8_decode.py:76-97); the shared-prefix layout
follows scripts/benchmark_shared_paged_prefix_suffix_decode_attention.py:76-122
(identical prefix rows in every block-table row, private suffix pages).

Five named geometries are provided:

=====================  ====  ====  ====  =====  ==========================
name                   Hq    Hkv   D     batch  context lengths
=====================  ====  ====  ====  =====  ==========================
``qwen2.5-0.5b-b8``    14    2     64    8      uniform int [128, 1024]
``qwen2.5-coder-3b-b64``  16  2    128   64     uniform int [512, 4096]
``qwen2.5-7b-b256``    28    4     128   256    log-uniform [1, 8192]
``llama3-8b-long-b4``  32    8     128   4      131072 each
``shared-prefix-b64``  16    2     128   64     4096 shared + U[0, 512]
=====================  ====  ====  ====  =====  ==========================
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

PAGE_SIZE = 16
FP8_MAX = 448.0


@dataclass
class PagedDecodeInputs:
    """One decode step's operands.  ``key_cache`` / ``value_cache`` are
    ``[pages, 16, Hkv, D]`` ``float8_e4m3fn`` (the reference op's NHD layout)."""

    name: str
    query: torch.Tensor
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    block_table: torch.Tensor
    seq_lens: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    max_seq_len: int
    prefix_len: int = 0
    meta: dict = field(default_factory=dict)

    @property
    def sm_scale(self) -> float:
        return self.query.shape[-1] ** -0.5

    @property
    def kv_bytes(self) -> int:
        """Algorithmic KV bytes of one step: every K and V byte of every live
        token once, ``sum_b ctx_b * Hkv * D * 2`` times the bytes per cache element."""
        hkv, d = self.key_cache.shape[2], self.key_cache.shape[3]
        return int(self.seq_lens.sum().item()) * hkv * d * 2 * self.key_cache.element_size()

    def to(self, device) -> "PagedDecodeInputs":
        moved = {
            k: (v.to(device) if isinstance(v, torch.Tensor) else v)
            for k, v in self.__dict__.items()
        }
        return PagedDecodeInputs(**moved)


GEOMETRIES = {
    "qwen2.5-0.5b-b8": dict(q_heads=14, kv_heads=2, head_dim=64, batch=8),
    "qwen2.5-coder-3b-b64": dict(q_heads=16, kv_heads=2, head_dim=128, batch=64),
    "qwen2.5-7b-b256": dict(q_heads=28, kv_heads=4, head_dim=128, batch=256),
    "llama3-8b-long-b4": dict(q_heads=32, kv_heads=8, head_dim=128, batch=4),
    "shared-prefix-b64": dict(q_heads=16, kv_heads=2, head_dim=128, batch=64),
}


def quantize_per_head(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``[pages, 16, Hkv, D]`` -> (e4m3 cache, ``[Hkv]`` scale = amax / 448)."""
    amax = x.abs().amax(dim=(0, 1, 3))
    scale = (amax / FP8_MAX).clamp_min(1.0e-12).to(torch.float32)
    q = (x / scale[None, None, :, None]).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def _context_lengths(name: str, batch: int, gen: torch.Generator, shrink: float) -> torch.Tensor:
    def scaled(v: int) -> int:
        return max(1, int(round(v * shrink)))

    if name == "qwen2.5-0.5b-b8":
        return torch.randint(scaled(128), scaled(1024) + 1, (batch,), generator=gen)
    if name == "qwen2.5-coder-3b-b64":
        return torch.randint(scaled(512), scaled(4096) + 1, (batch,), generator=gen)
    if name == "qwen2.5-7b-b256":
        hi = scaled(8192)
        u = torch.rand(batch, generator=gen, dtype=torch.float64)
        return torch.exp(u * math.log(hi)).round().clamp_(1, hi).to(torch.int64)
    if name == "llama3-8b-long-b4":
        return torch.full((batch,), scaled(131072), dtype=torch.int64)
    raise KeyError(name)


def make_inputs(
    name: str,
    *,
    seed: int = 0,
    device: str | torch.device = "cpu",
    batch: int | None = None,
    shrink: float = 1.0,
    query_dtype: torch.dtype = torch.bfloat16,
    kv_dtype: torch.dtype | None = None,
) -> PagedDecodeInputs:
    """Build one seeded decode step.

    ``kv_dtype`` (fp16 / bf16) builds the caches of the non-quantised sibling operator
    instead: N(0, 1) values stored as they are, both scales one.

    Index data (lengths, block table) always comes from a CPU generator seeded
    with ``seed`` so that it is identical everywhere.  K/V/q values come from a
    generator on ``device``: on ``"cpu"`` the whole input is reproducible bit
    for bit on any machine (what the parity tests and golden fixtures use); on
    a CUDA device generation of the large configurations takes milliseconds
    instead of minutes (what the benchmark uses).  ``shrink`` scales context
    lengths and ``batch`` overrides the batch, for parity tests that must stay
    small enough for the CPU oracle.
    """
    geo = dict(GEOMETRIES[name])
    if batch is not None:
        geo["batch"] = batch
    hq, hkv, d, bsz = geo["q_heads"], geo["kv_heads"], geo["head_dim"], geo["batch"]
    cpu_gen = torch.Generator(device="cpu").manual_seed(seed)
    dev = torch.device(device)
    dev_gen = cpu_gen if dev.type == "cpu" else torch.Generator(device=dev).manual_seed(seed)

    prefix_len = 0
    if name == "shared-prefix-b64":
        prefix_len = max(PAGE_SIZE, int(round(4096 * shrink)) // PAGE_SIZE * PAGE_SIZE)
        suffix = torch.randint(0, int(round(512 * shrink)) + 1, (bsz,), generator=cpu_gen)
        lens = prefix_len + suffix
        prefix_pages = prefix_len // PAGE_SIZE
        suffix_pages = (suffix + PAGE_SIZE - 1) // PAGE_SIZE
        total_pages = prefix_pages + int(suffix_pages.sum())
        max_pages = prefix_pages + int(suffix_pages.max())
        physical = torch.randperm(total_pages, generator=cpu_gen).to(torch.int32)
        table = torch.zeros(bsz, max_pages, dtype=torch.int32)
        table[:, :prefix_pages] = physical[:prefix_pages]
        cursor = prefix_pages
        for b in range(bsz):
            n = int(suffix_pages[b])
            table[b, prefix_pages : prefix_pages + n] = physical[cursor : cursor + n]
            cursor += n
    else:
        lens = _context_lengths(name, bsz, cpu_gen, shrink)
        pages_per = (lens + PAGE_SIZE - 1) // PAGE_SIZE
        total_pages = int(pages_per.sum())
        max_pages = int(pages_per.max())
        physical = torch.randperm(total_pages, generator=cpu_gen).to(torch.int32)
        table = torch.zeros(bsz, max_pages, dtype=torch.int32)
        cursor = 0
        for b in range(bsz):
            n = int(pages_per[b])
            table[b, :n] = physical[cursor : cursor + n]
            cursor += n

    shape = (total_pages, PAGE_SIZE, hkv, d)
    if kv_dtype is not None:
        key_cache = torch.randn(shape, generator=dev_gen, device=dev, dtype=torch.float32).to(kv_dtype)
        value_cache = torch.randn(shape, generator=dev_gen, device=dev, dtype=torch.float32).to(kv_dtype)
        k_scale = v_scale = torch.ones(hkv, device=dev, dtype=torch.float32)
    else:
        key_cache, k_scale = quantize_per_head(
            torch.randn(shape, generator=dev_gen, device=dev, dtype=torch.float32)
        )
        value_cache, v_scale = quantize_per_head(
            torch.randn(shape, generator=dev_gen, device=dev, dtype=torch.float32)
        )
    query = torch.randn(bsz, hq, d, generator=dev_gen, device=dev, dtype=torch.float32).to(query_dtype)
    return PagedDecodeInputs(
        name=name,
        query=query,
        key_cache=key_cache,
        value_cache=value_cache,
        block_table=table.to(dev),
        seq_lens=lens.to(torch.int32).to(dev),
        k_scale=k_scale,
        v_scale=v_scale,
        max_seq_len=int(lens.max()),
        prefix_len=prefix_len,
        meta=dict(geo, total_pages=total_pages, seed=seed, shrink=shrink),
    )
