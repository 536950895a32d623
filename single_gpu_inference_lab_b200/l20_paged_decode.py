"""Dispatcher-backed entry points of the B200 paged-decode operator.

Mirror of the reference wrapper module integrations/vllm/l20_paged_decode.py: the library
sits next to this file as ``l20_paged_decode_ops.so`` and is loaded at import (:11-17,
:116-117), the wrappers forward to ``torch.ops.l20_stack.*`` (:48-77) and fake (meta)
implementations are registered for tracing (:80-113).  A missing library is an error: there
is no eager or CPU fallback.
"""

from __future__ import annotations

from pathlib import Path
from typing import Optional, Union

import torch

_LOADED = False

# flag bits of the superset op (PFD_FLAG_* of include/paged_fp8_decode.h)
FLAG_NO_TMA = 1
FLAG_NO_DIRECT_OUT = 2
FLAG_PARTIAL_ONLY = 4
FLAG_FIXED_SPLITS = 8
FLAG_EARLY_METADATA = 32
FLAG_SINGLE_LAUNCH = 64
FLAG_EARLY_KV = 256


def load_library(path: Optional[Union[str, Path]] = None) -> None:
    global _LOADED
    library = (
        Path(path)
        if path is not None
        else Path(__file__).with_name("l20_paged_decode_ops.so")
    )
    if not library.exists():
        raise RuntimeError(
            f"{library} is missing (build it with `python -m single_gpu_inference_lab_b200.build`); "
            "the paged FP8 decode operator has no fallback implementation"
        )
    torch.ops.load_library(str(library))
    _LOADED = True


def paged_decode_split_out(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    output: torch.Tensor,
    max_seq_len: int,
    split_size: int,
) -> torch.Tensor:
    """The non-quantised sibling: caches in the query's fp16 / bf16 type.  Same call as the
    reference wrapper (l20_paged_decode.py:20-45); returns ``output``."""
    return torch.ops.l20_stack.paged_decode_split_out(
        query, key_cache, value_cache, block_table, seq_lens,
        partial_output, partial_max, partial_sum, output, max_seq_len, split_size,
    )


def paged_decode_split_out_v2(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    output: torch.Tensor,
    max_seq_len: int,
    split_size: int,
    *,
    flags: int = 0,
    plan: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """The non-quantised sibling with ``FLAG_*`` bits and an optional ``plan`` (see ``plan_decode``)."""
    torch.ops.l20_stack.paged_decode_split_out_v2(
        query, key_cache, value_cache, block_table, seq_lens,
        partial_output, partial_max, partial_sum, output, max_seq_len, split_size, flags, plan,
    )
    return output


def paged_decode_split_indices_out(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    page_indptr: torch.Tensor,
    page_indices: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    output: torch.Tensor,
    max_seq_len: int,
    split_size: int,
) -> torch.Tensor:
    """The fp16 / bf16 cache operator with FlashInfer's page addressing: the pages of sequence
    ``b`` are ``page_indices[page_indptr[b] : page_indptr[b + 1]]`` (reference launcher
    integrations/vllm/cuda/l20_paged_decode.cu:600-649, exported through pybind only)."""
    torch.ops.l20_stack.paged_decode_split_indices_out(
        query, key_cache, value_cache, page_indptr, page_indices, seq_lens,
        partial_output, partial_max, partial_sum, output, max_seq_len, split_size,
    )
    return output


def paged_decode_fp8_e4m3_split_out(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    output: torch.Tensor,
    k_scale: float,
    v_scale: float,
    max_seq_len: int,
    split_size: int,
) -> torch.Tensor:
    """Same call as the reference wrapper (l20_paged_decode.py:48-77); returns ``output``."""
    return torch.ops.l20_stack.paged_decode_fp8_e4m3_split_out(
        query,
        key_cache,
        value_cache,
        block_table,
        seq_lens,
        partial_output,
        partial_max,
        partial_sum,
        output,
        float(k_scale),
        float(v_scale),
        max_seq_len,
        split_size,
    )


def paged_decode_fp8_e4m3_split_out_v2(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: Optional[torch.Tensor],
    partial_max: Optional[torch.Tensor],
    partial_sum: Optional[torch.Tensor],
    output: Optional[torch.Tensor],
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    max_seq_len: int,
    split_size: int,
    *,
    packed_output: Optional[torch.Tensor] = None,
    sm_scale: float = 0.0,
    kv_start: int = 0,
    flags: int = 0,
    plan: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """Superset op: ``[Hkv]`` scale tensors (per layer and kv head), explicit softmax scale
    (0 = ``D**-0.5``), first attended token ``kv_start`` and, instead of or besides
    ``output``, a packed fp32 ``[B, Hq, D + 2]`` ``(o, m, l)`` for cross-GPU merging.
    ``flags`` are the ``FLAG_*`` bits above.  ``plan`` is the buffer ``plan_decode`` filled for the
    same lengths, block table and workspace (``FLAG_SINGLE_LAUNCH`` needs one)."""
    torch.ops.l20_stack.paged_decode_fp8_e4m3_split_out_v2(
        query,
        key_cache,
        value_cache,
        block_table,
        seq_lens,
        partial_output,
        partial_max,
        partial_sum,
        output,
        packed_output,
        k_scale,
        v_scale,
        float(sm_scale),
        max_seq_len,
        split_size,
        kv_start,
        flags,
        plan,
    )
    return output


def plan_decode(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    max_seq_len: int,
    split_size: int,
    *,
    kv_start: int = 0,
    plan: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Work split of a model step's decode-attention calls (``pfd_plan_decode``): one small
    kernel over the lengths and the block table, whose result every layer's call of the step
    reuses (``plan=``).  The caches and the workspace are passed for their geometry only; FP8
    caches plan for ``paged_decode_fp8_e4m3_split_out_v2``, caches in the query's type for the
    non-quantised sibling.  Raises when the call would not run the balanced kernel."""
    if plan is None:
        words = torch.ops.l20_stack.plan_bytes(query.shape[0], key_cache.shape[2]) // 4
        plan = torch.empty(words, dtype=torch.int32, device=query.device)
    torch.ops.l20_stack.plan_decode(
        query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum, plan,
        max_seq_len, split_size, kv_start,
    )
    return plan


def shared_prefix_decode_fp8_e4m3(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    output: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    max_seq_len: int,
    split_size: int,
    prefix_len: int,
    *,
    sm_scale: float = 0.0,
) -> torch.Tensor:
    """Decode step of a batch whose block-table rows all start with the same ``prefix_len // 16``
    pages: dense tcgen05 pass over the shared prefix, split-KV pass over the private suffixes,
    one merge.  The workspace needs ``ceil(prefix_len / 256) + ceil((max_seq_len - prefix_len) /
    split_size)`` slots on its split axis."""
    torch.ops.l20_stack.shared_prefix_decode_fp8_e4m3(
        query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum, output,
        k_scale, v_scale, float(sm_scale), max_seq_len, split_size, prefix_len,
    )
    return output


def shared_prefix_decode_grouped_fp8_e4m3(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    partial_output: torch.Tensor,
    partial_max: torch.Tensor,
    partial_sum: torch.Tensor,
    output: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    max_seq_len: int,
    split_size: int,
    groups: "PrefixGroups",
    *,
    max_prefix_len: Optional[int] = None,
    max_suffix_len: Optional[int] = None,
    sm_scale: float = 0.0,
    all_in_groups: bool = False,
) -> torch.Tensor:
    """Decode step of a batch with any number of shared-prefix groups plus requests in none
    (``groups`` from ``group_shared_prefixes``, read on the device): dense tcgen05 pass per group,
    split-KV pass from each request's own start, one merge.  ``max_suffix_len`` bounds what a
    request in a group has behind its prefix (``max_seq_len`` minus the grouping's
    ``min_prefix_len`` is always a true bound; ``None`` = the whole context): the split-KV grid is
    sized for it and requests in no group get as many, longer, splits.  The workspace needs
    ``ceil(min(max_prefix_len, max_seq_len) / 256) + ceil(min(max_suffix_len, max_seq_len) /
    split_size)`` slots.  ``all_in_groups`` (``PFD_FLAG_ALL_IN_GROUPS``): the caller has read
    ``groups.buffer[4]`` and it equals the batch; the split-KV pass may then run beside the dense
    pass instead of behind it (a hint about speed only)."""
    torch.ops.l20_stack.shared_prefix_decode_grouped_fp8_e4m3(
        query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum, output,
        k_scale, v_scale, float(sm_scale), max_seq_len, split_size, groups.buffer, groups.max_groups,
        int(max_seq_len if max_prefix_len is None else max_prefix_len), int(max_suffix_len or 0), bool(all_in_groups),
    )
    return output


class PrefixGroups:
    """Device-resident result of ``group_shared_prefixes`` (layout of ``pfd_group_shared_prefixes``
    in include/paged_fp8_decode.h).  The views below alias the buffer; reading them on the host
    (``to_lists``) is for tests and traces, the decode path consumes the buffer on the device."""

    HEADER = 8

    def __init__(self, buffer: torch.Tensor, batch: int, max_groups: int):
        self.buffer, self.batch, self.max_groups = buffer, batch, max_groups
        b, g, h = batch, max_groups, self.HEADER
        self.row_prefix_len = buffer[h:h + b]
        self.row_group = buffer[h + b:h + 2 * b]
        self.group_offsets = buffer[h + 2 * b:h + 2 * b + g + 1]
        self.group_prefix_len = buffer[h + 2 * b + g + 1:h + 2 * b + 2 * g + 1]
        self.group_rows = buffer[h + 2 * b + 2 * g + 1:h + 3 * b + 2 * g + 1]

    def to_lists(self) -> list[list[int]]:
        """The groups as lists of request indices (one device-to-host copy of the small buffer)."""
        host = self.buffer[: self.HEADER + 3 * self.batch + 2 * self.max_groups + 1].cpu()
        view = PrefixGroups(host, self.batch, self.max_groups)
        n = int(host[3])
        off = view.group_offsets.tolist()
        rows = view.group_rows.tolist()
        return [rows[off[g]:off[g + 1]] for g in range(n)]


def group_shared_prefixes(
    block_table: torch.Tensor,
    *,
    prefix_lengths: Optional[torch.Tensor] = None,
    uniform_prefix_len: int = 0,
    seq_lens: Optional[torch.Tensor] = None,
    min_batch: int = 8,
    min_prefix_len: int = 4096,
    max_groups: Optional[int] = None,
    buffer: Optional[torch.Tensor] = None,
) -> PrefixGroups:
    """Shared-prefix groups of a decode batch, found on the device without a host copy: same key
    and filters as the reference's ``find_l20_shared_prefix_groups``
    (integrations/vllm/l20_shared_prefix_decode_dispatch.py:41-76), any number of groups.  The
    prefix length of a request comes from ``prefix_lengths`` (int32, device), else from
    ``uniform_prefix_len``; with neither the prefixes are discovered from the table and
    ``seq_lens``: requests that agree on their first ``min_prefix_len`` tokens' pages form a group
    whose prefix is as long as all of them agree, in whole filled pages."""
    batch = block_table.shape[0]
    if max_groups is None:
        max_groups = max(1, batch // max(1, min_batch))
    if buffer is None:
        words = torch.ops.l20_stack.prefix_groups_bytes(batch, max_groups) // 4
        buffer = torch.empty(words, dtype=torch.int32, device=block_table.device)
    torch.ops.l20_stack.group_shared_prefixes(
        block_table, prefix_lengths, int(uniform_prefix_len), seq_lens, int(min_batch), int(min_prefix_len),
        int(max_groups), buffer,
    )
    return PrefixGroups(buffer, batch, max_groups)


def merge_packed_partials(packed: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
    """LSE-merge ``[parts, B, Hq, D + 2]`` packed partials into ``output [B, Hq, D]``."""
    torch.ops.l20_stack.merge_packed_partials(packed, output)
    return output


def resolve_slots(block_table: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int) -> torch.Tensor:
    """Cache slot (``page * 16 + offset``) the kernels resolve per (sequence, token); -1 past the end."""
    slots = torch.empty(block_table.shape[0], max_seq_len, dtype=torch.int64, device=block_table.device)
    torch.ops.l20_stack.resolve_slots(block_table, seq_lens, slots)
    return slots


def _register_fake() -> None:
    @torch.library.register_fake("l20_stack::paged_decode_split_out")
    def _(query, key_cache, value_cache, block_table, seq_lens, partial_output, partial_max, partial_sum,
          output, max_seq_len, split_size):
        return output

    @torch.library.register_fake("l20_stack::paged_decode_split_indices_out")
    def _(query, key_cache, value_cache, page_indptr, page_indices, seq_lens, partial_output, partial_max,
          partial_sum, output, max_seq_len, split_size):
        return None

    @torch.library.register_fake("l20_stack::paged_decode_fp8_e4m3_split_out")
    def _paged_decode_fp8_e4m3_split_out_fake(
        query,
        key_cache,
        value_cache,
        block_table,
        seq_lens,
        partial_output,
        partial_max,
        partial_sum,
        output,
        k_scale,
        v_scale,
        max_seq_len,
        split_size,
    ):
        return output

    @torch.library.register_fake("l20_stack::paged_decode_fp8_e4m3_split_out_v2")
    def _paged_decode_fp8_e4m3_split_out_v2_fake(*args):
        return None

    @torch.library.register_fake("l20_stack::paged_decode_split_out_v2")
    def _paged_decode_split_out_v2_fake(*args):
        return None

    @torch.library.register_fake("l20_stack::plan_decode")
    def _plan_decode_fake(*args):
        return None

    @torch.library.register_fake("l20_stack::shared_prefix_decode_fp8_e4m3")
    def _shared_prefix_decode_fake(*args):
        return None

    @torch.library.register_fake("l20_stack::merge_packed_partials")
    def _merge_packed_partials_fake(packed, output):
        return None

    @torch.library.register_fake("l20_stack::shared_prefix_decode_grouped_fp8_e4m3")
    def _shared_prefix_decode_grouped_fake(*args):
        return None

    @torch.library.register_fake("l20_stack::group_shared_prefixes")
    def _group_shared_prefixes_fake(*args):
        return None

    @torch.library.register_fake("l20_stack::resolve_slots")
    def _resolve_slots_fake(block_table, seq_lens, slots):
        return None


load_library()
_register_fake()
