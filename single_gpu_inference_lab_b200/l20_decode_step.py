"""What the decode hook computes once per model step and every attention layer of the step reuses.

The block table and the sequence lengths of a decode step are the same for all layers, so
anything derived from them alone is derived once, by the first layer that runs:

* the **plan** of the balanced kernel (``plan_l20_paged_split_kv``): how the step's KV is cut into
  chunks, which the kernels then read instead of re-deriving it in every layer;
* the **shared-prefix groups** of the batch (``group_shared_prefixes``), found on the device; with
  ``VLLM_ENABLE_L20_SHARED_PREFIX_DECODE=1`` (the reference's switch,
  integrations/vllm/l20_shared_prefix_decode_dispatch.py:18-19) a step that has groups goes
  through the grouped shared-prefix operator, and ``VLLM_L20_SHARED_PREFIX_DECODE_TRACE`` gets the
  reference's candidate record (:245-315) plus one run record per step;
* the **workspace**, one per shape for the whole model instead of one per layer (the layers run
  one after another on one stream).

The hook keeps the result on the step's metadata object (a new one per step), so a new step
starts fresh.  All buffers are persistent per shape, which is what a CUDA graph needs: while
vLLM records a decode graph the plan kernel is recorded in front of the first layer and replays
with the graph.  Deciding whether a step HAS groups needs one four-byte read per step on the
host; while a graph is being recorded that read is impossible, and the grouped path is then taken
only under ``VLLM_L20_SHARED_PREFIX_FORCE=1`` (it is correct for any batch, groups or none).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

MIN_GROUP_BATCH = 8
MIN_PREFIX_TOKENS = 4096
MAX_GROUPS = 4
PREFIX_CHUNK = 256


@dataclass
class DecodeStep:
    workspace: tuple
    plan: Optional[torch.Tensor] = None
    groups: object = None              # PrefixGroups when this step takes the grouped path
    prefix_workspace: Optional[tuple] = None
    suffix_split: int = 512            # split size of the grouped path's split-KV pass
    max_suffix: int = 0                # what a request in a group can have behind its prefix
    group_sizes: Optional[list] = None
    all_in_groups: bool = False        # no request of the step is outside the groups (read on the host)
    one_prefix: int = 0                # > 0: one group spans the batch with this prefix (read on the host):
                                       # the single-group operator runs, which needs no table lookups


_BUFFERS: dict = {}
_SWITCHES: Optional[dict] = None


def _switches() -> dict:
    global _SWITCHES
    if _SWITCHES is None:
        _SWITCHES = {
            "shared_prefix": os.environ.get("VLLM_ENABLE_L20_SHARED_PREFIX_DECODE", "0") == "1",
            "shared_prefix_force": os.environ.get("VLLM_L20_SHARED_PREFIX_FORCE", "0") == "1",
            "trace": os.environ.get("VLLM_L20_SHARED_PREFIX_DECODE_TRACE"),
            "no_plan": os.environ.get("VLLM_L20_PAGED_NO_PLAN", "0") == "1",
        }
    return _SWITCHES


def _persistent(key, make):
    buf = _BUFFERS.get(key)
    if buf is None:
        buf = _BUFFERS[key] = make()
    return buf


def l20_decode_step(meta, query, key_cache, value_cache, block_tables, seq_lens, max_seq_len: int, *,
                    split_size: int = 512, fp8: bool = True) -> DecodeStep:
    """The step's shared state: computed by the first layer of a step, kept on ``meta.l20_step``."""
    step = getattr(meta, "l20_step", None)
    if step is not None:
        return step
    from . import l20_paged_decode as ops
    from .l20_paged_split_kv import allocate_l20_paged_split_kv_workspace, plan_l20_paged_split_kv

    sw = _switches()
    batch, q_heads, head_dim = query.shape
    kv_heads = key_cache.shape[2]
    shape = (query.device, batch, q_heads, kv_heads, head_dim, -(-max_seq_len // split_size), query.dtype)
    workspace = _persistent(("ws",) + shape,
                            lambda: allocate_l20_paged_split_kv_workspace(query, max_seq_len, split_size=split_size))
    step = DecodeStep(workspace=workspace)
    planned = head_dim == 128 and q_heads <= 8 * kv_heads and batch <= 2048 and not sw["no_plan"]
    if planned:
        plan_buffer = _persistent(("plan",) + shape, lambda: torch.empty(
            torch.ops.l20_stack.plan_bytes(batch, kv_heads) // 4, dtype=torch.int32, device=query.device))
        try:
            step.plan = plan_l20_paged_split_kv(query, key_cache, value_cache, block_tables, seq_lens,
                                                max_seq_len=max_seq_len, split_size=split_size, workspace=workspace,
                                                plan=plan_buffer)
        except RuntimeError:
            step.plan = None  # this shape does not run the balanced kernel: the calls go without a plan
    capturing = torch.cuda.is_current_stream_capturing()
    if fp8 and sw["shared_prefix"] and head_dim == 128 and MIN_GROUP_BATCH <= batch <= 2048 and max_seq_len >= MIN_PREFIX_TOKENS \
            and (not capturing or sw["shared_prefix_force"]):
        # every group the buffer has room for costs idle CTAs in each layer's dense pass: room for a few
        max_groups = max(1, min(batch // MIN_GROUP_BATCH, MAX_GROUPS))
        groups_buffer = _persistent(("groups", query.device, batch, max_groups), lambda: torch.empty(
            torch.ops.l20_stack.prefix_groups_bytes(batch, max_groups) // 4, dtype=torch.int32, device=query.device))
        groups = ops.group_shared_prefixes(block_tables, seq_lens=seq_lens, min_batch=MIN_GROUP_BATCH,
                                           min_prefix_len=MIN_PREFIX_TOKENS, max_groups=max_groups, buffer=groups_buffer)
        take = sw["shared_prefix_force"]
        if not capturing:
            sizes = [len(g) for g in groups.to_lists()] if sw["trace"] else None
            # the one host read of the step: groups found, requests in them, prefix length of the first group
            pick = _persistent(("pick", query.device, batch, max_groups), lambda: torch.tensor(
                [3, 4, groups.HEADER + 2 * batch + max_groups + 1], dtype=torch.int64, device=query.device))
            found, grouped, first_prefix = groups.buffer.index_select(0, pick).tolist()
            take = take or found > 0
            step.all_in_groups = grouped == batch
            if found == 1 and grouped == batch and first_prefix >= MIN_PREFIX_TOKENS:
                step.one_prefix = min(first_prefix // 16 * 16, (max_seq_len - 1) // 16 * 16)
            if sw["trace"]:
                from .l20_shared_prefix_decode_dispatch import l20_shared_prefix_trace

                lens = seq_lens.tolist()
                l20_shared_prefix_trace(
                    "shared_prefix_decode_candidate", eligible=bool(found > 0), batch=int(batch), q_heads=int(q_heads),
                    kv_heads=int(kv_heads), head_dim=int(head_dim), page_size=16,
                    candidate_prefix=(min(lens) // 16) * 16 if lens else 0, max_seq_len=int(max_seq_len),
                    min_seq_len=min(lens) if lens else 0, group_sizes=sizes,
                )
                step.group_sizes = sizes
        if take:
            from .l20_shared_prefix_decode_dispatch import choose_suffix_split_size

            # grouped requests attend at most max_seq_len - MIN_PREFIX_TOKENS tokens behind their prefix
            step.max_suffix = max(max_seq_len - MIN_PREFIX_TOKENS, 16)
            step.suffix_split = choose_suffix_split_size(
                batch, kv_heads, max_seq_len - step.one_prefix if step.one_prefix else step.max_suffix)
            slots = -(-max_seq_len // PREFIX_CHUNK) + -(-step.max_suffix // step.suffix_split)
            step.groups = groups
            step.prefix_workspace = _persistent(("pws", query.device, batch, q_heads, slots), lambda: (
                torch.empty(batch, q_heads, slots, head_dim, device=query.device, dtype=torch.float32),
                torch.empty(batch, q_heads, slots, device=query.device, dtype=torch.float32),
                torch.empty(batch, q_heads, slots, device=query.device, dtype=torch.float32),
            ))
    try:
        meta.l20_step = step
    except AttributeError:
        pass  # metadata without the field: every layer then computes its own (still correct)
    return step


def l20_grouped_decode(step: DecodeStep, query, key_cache, value_cache, block_tables, seq_lens, k_scale, v_scale,
                       max_seq_len: int, output, *, split_size: int = 512):
    """One layer of a step that takes the grouped shared-prefix path."""
    from . import l20_paged_decode as ops
    from .l20_paged_split_kv import _scale_vector

    kv_heads = key_cache.shape[2]

    def vec(s):
        if isinstance(s, torch.Tensor) and s.dtype == torch.float32 and s.shape == (kv_heads,) and s.device == query.device:
            return s
        if isinstance(s, torch.Tensor):
            return s.to(device=query.device, dtype=torch.float32).reshape(-1).expand(kv_heads).contiguous()
        return _scale_vector(float(s), kv_heads, query.device)

    po, pm, ps = step.prefix_workspace
    if step.one_prefix:
        # one group spanning the batch: the reference's case (l20_shared_prefix_decode_dispatch.py:122-159);
        # the single-group operator reads no group table (2 us per layer less on the batch of 64)
        ops.shared_prefix_decode_fp8_e4m3(query, key_cache, value_cache, block_tables, seq_lens, po, pm, ps, output,
                                          vec(k_scale), vec(v_scale), max_seq_len, step.suffix_split, step.one_prefix)
    else:
        ops.shared_prefix_decode_grouped_fp8_e4m3(query, key_cache, value_cache, block_tables, seq_lens, po, pm, ps, output,
                                                  vec(k_scale), vec(v_scale), max_seq_len, step.suffix_split, step.groups,
                                                  max_suffix_len=step.max_suffix, all_in_groups=step.all_in_groups)
    sw = _switches()
    if sw["trace"]:
        from .l20_shared_prefix_decode_dispatch import l20_shared_prefix_trace

        l20_shared_prefix_trace("l20_shared_prefix_paged_decode_run", batch=int(query.shape[0]), q_heads=int(query.shape[1]),
                                kv_heads=int(kv_heads), max_seq_len=int(max_seq_len), group_sizes=step.group_sizes)
    return output
