"""Opt-in dispatch of shared-prefix decode attention, B200 build, FP8 paged KV.

Mirror of the reference's integrations/vllm/l20_shared_prefix_decode_dispatch.py for the fully
paged form (prefix and suffix both in the paged cache): same switch
``VLLM_ENABLE_L20_SHARED_PREFIX_DECODE``, same trace switch
``VLLM_L20_SHARED_PREFIX_DECODE_TRACE``, same grouping key (prefix length + the prefix's block
chain, :41-76), same conservative gate (one group spanning the whole batch, batch >= 8,
prefix >= 4096, :122-159).  Differences: the gate asks for sm_100 and an e4m3 cache (the
reference's gate rejects quantised caches, :138-141), and the work is done by the dense
tcgen05 prefix pass + split-KV suffix pass + merge of ``l20_stack::shared_prefix_decode_fp8_e4m3``
instead of three Triton kernels (src/l20_stack/ops/triton_decode_attention.py:1310-1458).
"""

from __future__ import annotations

import json
import os
import time
from collections import defaultdict
from pathlib import Path
from typing import Sequence

import torch

PREFIX_CHUNK = 256  # prefix tokens per CTA of the dense pass


def l20_shared_prefix_decode_enabled() -> bool:
    return os.getenv("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", "0") == "1"


def l20_shared_prefix_trace(event: str, **fields) -> None:
    path = os.getenv("VLLM_L20_SHARED_PREFIX_DECODE_TRACE")
    if not path:
        return
    payload = {"event": event, "ts": time.time(), **fields}
    try:
        with Path(path).open("a", encoding="utf-8") as trace_file:
            trace_file.write(json.dumps(payload, sort_keys=True) + "\n")
    except OSError:
        return


def _to_int_list(values: torch.Tensor | Sequence[int]) -> list[int]:
    if isinstance(values, torch.Tensor):
        return [int(item) for item in values.detach().cpu().tolist()]
    return [int(item) for item in values]


def shared_prefix_block_key(
    block_table_row: torch.Tensor, prefix_length: int, *, page_size: int = 16
) -> tuple[int, tuple[int, ...]]:
    pages = (int(prefix_length) + page_size - 1) // page_size
    blocks = block_table_row[:pages].detach().cpu().tolist()
    return int(prefix_length), tuple(int(block) for block in blocks)


def find_l20_shared_prefix_groups(
    block_tables: torch.Tensor,
    prefix_lengths: torch.Tensor | Sequence[int],
    *,
    min_batch: int = 8,
    min_prefix_length: int = 4096,
    page_size: int = 16,
) -> list[list[int]]:
    """Group request indices by identical prefix length and block chain."""
    if block_tables.ndim != 2:
        raise ValueError("block_tables must have shape [B, max_pages]")
    lengths = _to_int_list(prefix_lengths)
    if len(lengths) != block_tables.shape[0]:
        raise ValueError("prefix_lengths must have one entry per request")
    table = block_tables.detach().cpu()  # one copy for the whole batch
    groups: dict[tuple[int, tuple[int, ...]], list[int]] = defaultdict(list)
    for index, prefix_length in enumerate(lengths):
        if prefix_length < min_prefix_length:
            continue
        groups[shared_prefix_block_key(table[index], prefix_length, page_size=page_size)].append(index)
    return [indices for indices in groups.values() if len(indices) >= min_batch]


def should_dispatch_l20_shared_prefix_paged_decode(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    block_tables: torch.Tensor,
    prefix_lengths: torch.Tensor | Sequence[int],
    *,
    page_size: int = 16,
    min_batch: int = 8,
    min_prefix_length: int = 4096,
) -> bool:
    if not l20_shared_prefix_decode_enabled():
        return False
    if not torch.cuda.is_available() or not query.is_cuda:
        return False
    if torch.cuda.get_device_capability(query.device) != (10, 0):
        return False
    if torch.cuda.is_current_stream_capturing():
        return False  # the grouping below copies the block table to the host
    if query.dtype not in (torch.float16, torch.bfloat16):
        return False
    if key_cache.dtype != torch.float8_e4m3fn:
        return False
    if query.ndim != 3 or key_cache.ndim != 4:
        return False
    if block_tables.ndim != 2 or block_tables.shape[0] != query.shape[0]:
        return False
    if query.shape[0] < min_batch:
        return False
    if query.shape[-1] != 128 or key_cache.shape[-1] != 128:
        return False
    if key_cache.shape[1] != page_size or page_size != 16:
        return False
    lengths = _to_int_list(prefix_lengths)
    if not lengths or lengths[0] % page_size:
        return False
    groups = find_l20_shared_prefix_groups(
        block_tables, lengths, min_batch=min_batch, min_prefix_length=min_prefix_length, page_size=page_size
    )
    return len(groups) == 1 and len(groups[0]) == query.shape[0]


def allocate_shared_prefix_workspace(query: torch.Tensor, max_seq_len: int, prefix_length: int, *, suffix_split_size: int = 512):
    """``(partial_output, partial_max, partial_sum, output)`` with one slot per 256-token prefix
    chunk plus one per suffix split."""
    batch, num_q_heads, head_dim = query.shape
    slots = -(-prefix_length // PREFIX_CHUNK) + max(1, -(-(max_seq_len - prefix_length) // suffix_split_size))
    shape = (batch, num_q_heads, slots)
    return (
        torch.empty((*shape, head_dim), device=query.device, dtype=torch.float32),
        torch.empty(shape, device=query.device, dtype=torch.float32),
        torch.empty(shape, device=query.device, dtype=torch.float32),
        torch.empty_like(query),
    )


def shared_paged_prefix_paged_suffix_gqa_decode_attention_fp8(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    prefix_length: int,
    *,
    k_scale: torch.Tensor | float,
    v_scale: torch.Tensor | float,
    max_seq_len: int | None = None,
    suffix_split_size: int = 512,
    output: torch.Tensor | None = None,
    workspace=None,
) -> torch.Tensor:
    """FP8 counterpart of ``shared_paged_prefix_paged_suffix_gqa_decode_attention``
    (src/l20_stack/ops/triton_decode_attention.py:1310-1458): every request attends the same
    ``prefix_length`` tokens (same pages in every block-table row) plus its own suffix."""
    from . import l20_paged_decode as ops

    if max_seq_len is None:
        max_seq_len = int(seq_lens.max().item())
    num_kv_heads = key_cache.shape[2]
    if workspace is None:
        workspace = allocate_shared_prefix_workspace(query, max_seq_len, prefix_length, suffix_split_size=suffix_split_size)
    partial_output, partial_max, partial_sum, workspace_output = workspace[:4]
    if output is None:
        output = workspace_output

    def as_vec(s):
        if isinstance(s, torch.Tensor) and s.dtype == torch.float32 and s.shape == (num_kv_heads,) and s.device == query.device:
            return s
        if isinstance(s, torch.Tensor):
            return s.to(device=query.device, dtype=torch.float32).reshape(-1).expand(num_kv_heads).contiguous()
        return torch.full((num_kv_heads,), float(s), device=query.device, dtype=torch.float32)

    return ops.shared_prefix_decode_fp8_e4m3(
        query, key_cache, value_cache, block_tables, seq_lens, partial_output, partial_max, partial_sum, output,
        as_vec(k_scale), as_vec(v_scale), max_seq_len, suffix_split_size, int(prefix_length),
    )


def maybe_l20_shared_prefix_paged_decode(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    prefix_lengths: torch.Tensor | Sequence[int],
    *,
    k_scale: torch.Tensor | float,
    v_scale: torch.Tensor | float,
    page_size: int = 16,
    suffix_split_size: int = 512,
    max_seq_len: int | None = None,
    workspace=None,
):
    """Return the shared-prefix output for a fully paged prefix and suffix, or None when the
    conservative gate fails (the caller then takes its ordinary decode path)."""
    if not should_dispatch_l20_shared_prefix_paged_decode(
        query, key_cache, block_tables, prefix_lengths, page_size=page_size
    ):
        return None
    prefix_length = _to_int_list(prefix_lengths)[0]
    out = shared_paged_prefix_paged_suffix_gqa_decode_attention_fp8(
        query, key_cache, value_cache, block_tables, seq_lens, prefix_length, k_scale=k_scale, v_scale=v_scale,
        max_seq_len=max_seq_len, suffix_split_size=suffix_split_size, workspace=workspace,
    )
    l20_shared_prefix_trace(
        "l20_shared_prefix_paged_decode_run", batch=int(query.shape[0]), prefix_length=int(prefix_length),
        q_heads=int(query.shape[1]), kv_heads=int(key_cache.shape[2]),
    )
    return out
