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
from typing import Optional, Sequence

import torch

PREFIX_CHUNK = 256  # prefix tokens per work item of the dense pass
_SWITCH = "VLLM_ENABLE_L20_SHARED_PREFIX_DECODE"
_TRACE = "VLLM_L20_SHARED_PREFIX_DECODE_TRACE"


def l20_shared_prefix_decode_enabled() -> bool:
    """The reference's opt-in switch (l20_shared_prefix_decode_dispatch.py:18-19)."""
    return os.environ.get(_SWITCH, "0") == "1"


def l20_shared_prefix_trace(event: str, **fields) -> None:
    """Append one JSON line ``{"event", "ts", **fields}`` to the file the trace switch names, as
    the reference's trace does (:22-31); a trace that cannot be written is dropped silently."""
    target = os.environ.get(_TRACE)
    if not target:
        return
    record = dict(fields, event=event, ts=time.time())
    try:
        with open(target, "a", encoding="utf-8") as sink:
            print(json.dumps(record, sort_keys=True), file=sink)
    except OSError:
        pass


def _lengths_on_host(values) -> list[int]:
    if isinstance(values, torch.Tensor):
        values = values.detach().to("cpu").tolist()
    return list(map(int, values))


def shared_prefix_block_key(block_table_row: torch.Tensor, prefix_length: int, *, page_size: int = 16):
    """The grouping key of one request: its prefix length and the block ids that hold the prefix."""
    n_pages = -(-int(prefix_length) // page_size)
    return int(prefix_length), tuple(map(int, block_table_row[:n_pages].detach().to("cpu").tolist()))


def find_l20_shared_prefix_groups(
    block_tables: torch.Tensor,
    prefix_lengths,
    *,
    min_batch: int = 8,
    min_prefix_length: int = 4096,
    page_size: int = 16,
) -> list[list[int]]:
    """Requests with the same prefix length whose prefixes sit in the same blocks, as lists of
    request indices (groups ordered by first member, groups below ``min_batch`` and prefixes below
    ``min_prefix_length`` left out): the reference function of the same name (:41-76).

    A block table on the GPU is grouped there (``group_shared_prefixes``: hash, verify, number --
    the table itself never leaves the device, only the small result is read back for this
    list-returning interface); a table in host memory is grouped with ``torch.unique`` over the
    prefix columns, one call per distinct prefix length."""
    if block_tables.ndim != 2:
        raise ValueError("block_tables must have shape [B, max_pages]")
    lengths = _lengths_on_host(prefix_lengths)
    batch = block_tables.shape[0]
    if len(lengths) != batch:
        raise ValueError("prefix_lengths must have one entry per request")
    if block_tables.is_cuda and page_size == 16 and block_tables.dtype == torch.int32 and batch <= 2048:
        from . import l20_paged_decode as ops

        found = ops.group_shared_prefixes(
            block_tables, prefix_lengths=torch.tensor(lengths, dtype=torch.int32, device=block_tables.device),
            min_batch=min_batch, min_prefix_len=max(int(min_prefix_length), 1), max_groups=max(batch, 1),
        )
        return found.to_lists()
    table = block_tables.detach().to("cpu")
    by_first_member: dict[int, list[int]] = {}
    for length in sorted(set(x for x in lengths if x >= min_prefix_length)):
        members = torch.tensor([i for i, x in enumerate(lengths) if x == length], dtype=torch.long)
        n_pages = -(-length // page_size)
        _, klass = torch.unique(table[members, :n_pages], dim=0, return_inverse=True)
        for k in klass.unique().tolist():
            rows = members[klass == k].tolist()
            if len(rows) >= min_batch:
                by_first_member[rows[0]] = rows
    return [by_first_member[first] for first in sorted(by_first_member)]


def _why_not(query, key_cache, block_tables, prefix_lengths, page_size, min_batch, min_prefix_length) -> Optional[str]:
    """None when the conservative single-group dispatch applies, else the first reason it does not
    (the conditions of the reference's gate, :122-159, with sm_100 and an e4m3 cache in place of
    its sm_89 / unquantised ones)."""
    if not l20_shared_prefix_decode_enabled():
        return "switch"
    if not (torch.cuda.is_available() and query.is_cuda):
        return "device"
    if torch.cuda.get_device_capability(query.device) != (10, 0):
        return "arch"
    if torch.cuda.is_current_stream_capturing():
        return "capturing"  # this gate reads the grouping result on the host
    if query.dtype not in (torch.float16, torch.bfloat16) or key_cache.dtype != torch.float8_e4m3fn:
        return "dtype"
    shapes_ok = (
        query.ndim == 3 and key_cache.ndim == 4 and block_tables.ndim == 2
        and block_tables.shape[0] == query.shape[0]
        and query.shape[-1] == 128 and key_cache.shape[-1] == 128
        and key_cache.shape[1] == page_size == 16
    )
    if not shapes_ok:
        return "shape"
    if query.shape[0] < min_batch:
        return "batch"
    lengths = _lengths_on_host(prefix_lengths)
    if not lengths or lengths[0] % page_size:
        return "prefix_alignment"
    groups = find_l20_shared_prefix_groups(
        block_tables, lengths, min_batch=min_batch, min_prefix_length=min_prefix_length, page_size=page_size
    )
    if len(groups) != 1 or len(groups[0]) != query.shape[0]:
        return "groups"
    return None


def should_dispatch_l20_shared_prefix_paged_decode(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    block_tables: torch.Tensor,
    prefix_lengths,
    *,
    page_size: int = 16,
    min_batch: int = 8,
    min_prefix_length: int = 4096,
) -> bool:
    return _why_not(query, key_cache, block_tables, prefix_lengths, page_size, min_batch, min_prefix_length) is None


def choose_suffix_split_size(batch: int, num_kv_heads: int, max_suffix_len: int, *, resident_ctas: int = 444) -> int:
    """Split size of the suffix pass of the shared-prefix operators.  The suffix kernel's work
    items are (request, kv head, split); private suffixes are short, so with the reference's
    constant 512 (install hook, :117) a work item is one latency chain of a few page pairs and
    there are too few of them: the pass then lasts as long as the dense pass it accompanies (10 us
    on the batch of 64 with suffixes up to 512 tokens).  As many equal splits per request as make
    about one wave of resident CTAs (3 per SM on 148 SMs), but two to four of them, in multiples
    of 64 tokens (whole page pairs for each warp of a CTA), is what the measurements ask for, in us
    per step with suffixes up to 511 tokens behind a prefix of 4096:
    batch 64: 512 -> 25.1, 256 -> 19.4, 192 -> 18.1, 160 -> 18.2, 128 -> 17.6, 96 -> 20.1, 64 -> 18.9;
    batch 256: 512 -> 61.9, 256 -> 59.8, 128 -> 62.3;  batch 128: 512 -> 37.0, 256 -> 34.1, 128 -> 34.2;
    batches 32 to 96: within 0.3 us from 128 to 512;  batch 16: 512 -> 14.0, 128 -> 14.4, 64 -> 14.5."""
    if max_suffix_len <= 0:
        return 64
    splits = -(-int(resident_ctas) // max(int(batch) * int(num_kv_heads), 1))
    splits = min(4, max(2, splits))
    size = -(-(-(-int(max_suffix_len) // splits)) // 64) * 64
    return int(min(512, max(64, size)))


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
    suffix_split_size: int | None = 512,
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
    if suffix_split_size is None:  # (the reference's default is the constant 512)
        suffix_split_size = choose_suffix_split_size(query.shape[0], num_kv_heads, max_seq_len - int(prefix_length))
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
    suffix_split_size: int | None = None,
    max_seq_len: int | None = None,
    workspace=None,
):
    """Return the shared-prefix output for a fully paged prefix and suffix, or None when the
    conservative gate fails (the caller then takes its ordinary decode path)."""
    if not should_dispatch_l20_shared_prefix_paged_decode(
        query, key_cache, block_tables, prefix_lengths, page_size=page_size
    ):
        return None
    prefix_length = _lengths_on_host(prefix_lengths)[0]
    out = shared_paged_prefix_paged_suffix_gqa_decode_attention_fp8(
        query, key_cache, value_cache, block_tables, seq_lens, prefix_length, k_scale=k_scale, v_scale=v_scale,
        max_seq_len=max_seq_len, suffix_split_size=suffix_split_size, workspace=workspace,
    )
    l20_shared_prefix_trace(
        "l20_shared_prefix_paged_decode_run", batch=int(query.shape[0]), prefix_length=int(prefix_length),
        q_heads=int(query.shape[1]), kv_heads=int(key_cache.shape[2]),
    )
    return out
