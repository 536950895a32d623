"""Paged split-KV GQA decode attention over an FP8-e4m3 KV cache, B200 build.

Same public surface as the module the reference's vLLM hook copies into
``vllm/v1/attention/ops/`` (integrations/vllm/l20_paged_split_kv.py):

* ``allocate_l20_paged_split_kv_workspace(query, max_seq_len, *, split_size=512)``  (:14-30)
* ``l20_paged_split_kv_attention_fp8(query, key_cache, value_cache, block_table, seq_lens, *,
  k_scale, v_scale, max_seq_len=None, split_size=512, output=None, workspace=None)`` (:597-695)
* ``should_use_l20_paged_fp8_split_kv(batch, max_seq_len)``                          (:705-709)
* ``l20_paged_split_kv_attention(...)`` / ``should_use_l20_paged_split_kv``: the fp16 / bf16
  cache siblings (:491-594, :698-702)

with the same ``RuntimeError`` texts where the condition still exists.  Differences, all
supersets: bf16 or fp16 queries, head_dim 64 or 128, any number of splits (the reference
stops at 16, :635-636), ``k_scale`` / ``v_scale`` either floats or ``[Hkv]`` float32 tensors,
fp32 partials (the reference keeps partial sums in the query dtype, :24-26), strided caches in
any (page, token, head) order.  The two Triton launches are replaced by one call of the
``l20_stack`` CUDA operator; there is no Triton, FlashInfer or CPU path behind it.
"""

from __future__ import annotations

import torch

REQUIRED_CAPABILITY = (10, 0)


def _next_power_of_two(value: int) -> int:
    return 1 << (max(int(value), 1) - 1).bit_length()


def _cdiv(a: int, b: int) -> int:
    return -(-int(a) // int(b))


_OPS = None
_CAPABILITY: dict = {}
_SCALE_VECTORS: dict = {}


def _ops():
    global _OPS
    if _OPS is None:
        from . import l20_paged_decode  # loads l20_paged_decode_ops.so or raises

        _OPS = l20_paged_decode
    return _OPS


def _on_required_gpu(tensor: torch.Tensor) -> bool:
    """Capability gate, looked up once per device (this runs once per layer and decode step)."""
    if not tensor.is_cuda:
        return False
    key = tensor.device.index
    if key not in _CAPABILITY:
        _CAPABILITY[key] = torch.cuda.get_device_capability(tensor.device) == REQUIRED_CAPABILITY
    return _CAPABILITY[key]


def _scale_vector(value: float, num_kv_heads: int, device: torch.device) -> torch.Tensor:
    """``[Hkv]`` float32 tensor filled with a per-layer Python-float scale, built once per
    (device, heads, value): no fill kernel on the per-step path."""
    key = (device.index, num_kv_heads, float(value))
    vec = _SCALE_VECTORS.get(key)
    if vec is None:
        if len(_SCALE_VECTORS) > 4096:
            _SCALE_VECTORS.clear()
        vec = _SCALE_VECTORS[key] = torch.full((num_kv_heads,), float(value), device=device, dtype=torch.float32)
    return vec


BALANCED_WARPS_PER_SM = 8  # warps of the balanced persistent kernel on every SM
BALANCED_MAX_GROUP = 8      # query heads per kv head it handles


def balanced_workspace_splits(query: torch.Tensor, num_kv_heads: int | None = None) -> int:
    """Smallest split axis ``S`` with which a ``[B, Hq, S]`` workspace can hold the pieces of the
    balanced persistent kernel: two slots of ``Hq`` rows for every group of ``Hkv`` warps, i.e.
    ``2 * (8 * SMs // Hkv) * Hq`` rows (``pfd_balanced_workspace_rows``).  Without
    ``num_kv_heads`` the bound for the largest supported GQA ratio is used (about 10 MB of fp32
    rows on a 148-SM part, whatever the batch)."""
    batch, num_q_heads, _ = query.shape
    sms = torch.cuda.get_device_properties(query.device).multi_processor_count if query.is_cuda else 148
    warps = sms * BALANCED_WARPS_PER_SM
    if num_kv_heads:
        rows = 2 * (warps // int(num_kv_heads)) * num_q_heads
    else:
        rows = 2 * warps * min(BALANCED_MAX_GROUP, num_q_heads)
    return _cdiv(rows, max(batch * num_q_heads, 1))


def allocate_l20_paged_split_kv_workspace(
    query: torch.Tensor,
    max_seq_len: int,
    *,
    split_size: int = 512,
    num_kv_heads: int | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(partial_output [B,Hq,S,D] f32, partial_max [B,Hq,S] f32, partial_sum, output)`` as in
    the reference (:14-30), where ``S = next_pow2(ceil(max_seq_len / split_size))`` (:21-22).
    Here ``S`` is also at least ``balanced_workspace_splits(query)``, which only matters for
    small batches: with that capacity the operator runs its balanced persistent kernel, which
    treats the workspace as a flat list of rows and needs no tuning of ``split_size``."""
    batch, num_q_heads, head_dim = query.shape
    num_splits = _next_power_of_two(_cdiv(max_seq_len, split_size))
    if head_dim == 128:
        num_splits = max(num_splits, balanced_workspace_splits(query, num_kv_heads))
    partial_shape = (batch, num_q_heads, num_splits)
    return (
        torch.empty((*partial_shape, head_dim), device=query.device, dtype=torch.float32),
        torch.empty(partial_shape, device=query.device, dtype=torch.float32),
        torch.empty(partial_shape, device=query.device, dtype=torch.float32),
        torch.empty_like(query),
    )


def choose_split_size(batch: int, num_kv_heads: int, max_seq_len: int, *, seq_lens=None,
                      sm_count: int = 148, ctas_per_sm: int = 3, minimum: int = 128, step: int = 64) -> int:
    """Split size for the fixed-split grid, from host-side knowledge only (no device read).

    The kernel likes exactly one wave of live (sequence, kv head, split) work items: a second,
    partly filled wave costs about as much as the first.  With ``target`` = token-heads per
    resident CTA slot, the smallest multiple of ``step`` whose item count fits the
    ``sm_count * ctas_per_sm`` slots is used if it is at most ``1.5 * target``; batches with more
    (sequence, kv head) pairs than slots cannot fit one wave, they get ``0.8 * target`` (a few
    waves of small items, measured best on B200).  ``seq_lens`` (host ints, e.g. the engine's
    CPU copy of the sequence lengths) makes the count exact; without it every sequence is
    taken as ``max_seq_len`` long."""
    slots = sm_count * ctas_per_sm
    lens = [int(x) for x in seq_lens] if seq_lens is not None else [int(max_seq_len)] * int(batch)
    lens = [n for n in lens if n > 0] or [1]
    longest = max(max_seq_len, max(lens))
    target = max(1.0, num_kv_heads * sum(lens) / slots)

    def round_up(x: float) -> int:
        return max(minimum, _cdiv(int(x), step) * step)

    split = round_up(target)
    while split < longest and split <= 1.5 * target:
        if num_kv_heads * sum(_cdiv(n, split) for n in lens) <= slots:
            return int(split)
        split += step
    if num_kv_heads * len(lens) <= slots and split >= longest:
        return int(round_up(longest))  # one item per pair already fits
    return int(min(round_up(0.8 * target), round_up(longest)))


def l20_paged_split_kv_attention_fp8(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    *,
    k_scale: float | torch.Tensor,
    v_scale: float | torch.Tensor,
    max_seq_len: int | None = None,
    split_size: int = 512,
    output: torch.Tensor | None = None,
    workspace: tuple[torch.Tensor, ...] | None = None,
    metadata_stable: bool = False,
    plan: torch.Tensor | None = None,
    single_launch: bool = False,
    kv_stable: bool = False,
) -> torch.Tensor:
    """``metadata_stable=True`` (not in the reference) tells the operator that the kernel
    running before it on the stream does not write ``block_table``, ``seq_lens`` or ``plan`` --
    true for every layer of a model step, whose metadata is built once -- so that it may read
    them while that kernel drains (``PFD_FLAG_EARLY_METADATA``).  ``plan`` (not in the reference
    either) is the result of ``plan_l20_paged_split_kv`` for the same step: the kernels then read
    their work split instead of deriving it; ``single_launch`` (needs a plan) makes the balanced
    kernel combine the pieces of cut sequences itself, one launch instead of two
    (``PFD_FLAG_SINGLE_LAUNCH``; the slower of the two on B200).  ``kv_stable=True`` (with
    ``metadata_stable`` and a plan): that kernel also writes K/V only into the last page of each
    sequence -- a decode step's cache append -- so every other page may be streamed while it
    drains (``PFD_FLAG_EARLY_KV``)."""
    if not _on_required_gpu(query):
        raise RuntimeError("requires an SM100 GPU")
    if query.ndim != 3 or key_cache.ndim != 4 or value_cache.shape != key_cache.shape:
        raise RuntimeError("expected Q=[B,H,D], cache=[pages,page,Hkv,D]")
    if key_cache.dtype != torch.float8_e4m3fn or value_cache.dtype != key_cache.dtype:
        raise RuntimeError("key/value cache must use torch.float8_e4m3fn")
    batch, num_q_heads, head_dim = query.shape
    _, page_size, num_kv_heads, cache_dim = key_cache.shape
    if (
        head_dim not in (64, 128)
        or cache_dim != head_dim
        or page_size != 16
        or num_q_heads % num_kv_heads
        or num_q_heads // num_kv_heads > 16
        or block_table.shape[0] != batch
        or seq_lens.numel() != batch
    ):
        raise RuntimeError("requires compatible head_dim=64/128 GQA tensors")
    if max_seq_len is None:
        max_seq_len = int(seq_lens.max().item())
    num_splits = _next_power_of_two(_cdiv(max_seq_len, split_size))
    partial_shape = (batch, num_q_heads, num_splits)
    if workspace is None:
        workspace = allocate_l20_paged_split_kv_workspace(query, max_seq_len, split_size=split_size)
    partial_output, partial_max, partial_sum, workspace_output = workspace[:4]
    if output is None:
        output = workspace_output
    if (
        partial_output.shape[:2] != partial_shape[:2]
        or partial_output.shape[2] < num_splits
        or partial_output.shape[3] != head_dim
        or partial_max.shape != partial_output.shape[:3]
        or partial_sum.shape != partial_output.shape[:3]
        or output.shape != query.shape
    ):
        raise RuntimeError("paged split-KV workspace shape does not match the request")
    ops = _ops()
    if isinstance(k_scale, torch.Tensor) or isinstance(v_scale, torch.Tensor) or metadata_stable or plan is not None:
        def as_vec(s):
            if isinstance(s, torch.Tensor):
                if s.dtype == torch.float32 and s.device == query.device and s.shape == (num_kv_heads,) and s.is_contiguous():
                    return s  # the common case costs nothing
                return s.to(device=query.device, dtype=torch.float32).reshape(-1).expand(num_kv_heads).contiguous()
            return _scale_vector(s, num_kv_heads, query.device)

        ops.paged_decode_fp8_e4m3_split_out_v2(
            query, key_cache, value_cache, block_table, seq_lens,
            partial_output, partial_max, partial_sum, output,
            as_vec(k_scale), as_vec(v_scale), max_seq_len, split_size,
            flags=(ops.FLAG_EARLY_METADATA if metadata_stable else 0) | (ops.FLAG_SINGLE_LAUNCH if single_launch else 0)
            | (ops.FLAG_EARLY_KV if kv_stable and metadata_stable else 0),
            plan=plan,
        )
        return output
    return ops.paged_decode_fp8_e4m3_split_out(
        query, key_cache, value_cache, block_table, seq_lens,
        partial_output, partial_max, partial_sum, output,
        float(k_scale), float(v_scale), max_seq_len, split_size,
    )


def l20_paged_split_kv_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    *,
    split_size: int = 512,
    workspace: tuple[torch.Tensor, ...] | None = None,
    max_seq_len: int | None = None,
    output: torch.Tensor | None = None,
    metadata_stable: bool = False,
    plan: torch.Tensor | None = None,
    single_launch: bool = False,
    kv_stable: bool = False,
) -> torch.Tensor:
    """The non-quantised sibling (reference :491-594): K/V caches in the query's fp16 / bf16
    type.  ``metadata_stable`` / ``plan`` / ``single_launch`` / ``kv_stable`` as for the FP8 wrapper.  ``page_granular`` / ``grouped_gqa`` of the reference select between its Triton kernel
    variants and have no counterpart here.  ``max_seq_len`` (not in the reference, which always
    reads it back from the device, :517) avoids that host synchronisation."""
    if not _on_required_gpu(query):
        raise RuntimeError("requires an SM100 GPU")
    if query.ndim != 3 or key_cache.ndim != 4 or value_cache.shape != key_cache.shape:
        raise RuntimeError("expected Q=[B,H,D], cache=[pages,page,Hkv,D]")
    batch, num_q_heads, head_dim = query.shape
    _, page_size, num_kv_heads, cache_dim = key_cache.shape
    if (
        head_dim != 128
        or cache_dim != head_dim
        or page_size != 16
        or num_q_heads % num_kv_heads
        or num_q_heads // num_kv_heads > 8
        or block_table.shape[0] != batch
        or seq_lens.numel() != batch
        or key_cache.dtype != query.dtype
        or value_cache.dtype != query.dtype
    ):
        raise RuntimeError("requires compatible head_dim=128 GQA tensors")
    if max_seq_len is None:
        max_seq_len = int(seq_lens.max().item())
    if workspace is None:
        workspace = allocate_l20_paged_split_kv_workspace(query, max_seq_len, split_size=split_size,
                                                          num_kv_heads=num_kv_heads)
    partial_output, partial_max, partial_sum, workspace_output = workspace[:4]
    if output is None:
        output = workspace_output
    if (
        partial_output.shape[:2] != (batch, num_q_heads)
        or partial_output.shape[3] != head_dim
        or partial_max.shape != partial_output.shape[:3]
        or partial_sum.shape != partial_output.shape[:3]
        or output.shape != query.shape
    ):
        raise RuntimeError("paged split-KV workspace shape does not match the request")
    ops = _ops()
    if metadata_stable or plan is not None:
        return ops.paged_decode_split_out_v2(
            query, key_cache, value_cache, block_table, seq_lens,
            partial_output, partial_max, partial_sum, output, max_seq_len, split_size,
            flags=(ops.FLAG_EARLY_METADATA if metadata_stable else 0) | (ops.FLAG_SINGLE_LAUNCH if single_launch else 0)
            | (ops.FLAG_EARLY_KV if kv_stable and metadata_stable else 0),
            plan=plan,
        )
    return ops.paged_decode_split_out(
        query, key_cache, value_cache, block_table, seq_lens,
        partial_output, partial_max, partial_sum, output, max_seq_len, split_size,
    )


def plan_l20_paged_split_kv(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    *,
    max_seq_len: int,
    split_size: int = 512,
    workspace: tuple[torch.Tensor, ...],
    plan: torch.Tensor | None = None,
) -> torch.Tensor | None:
    """Once per model step (not in the reference, whose kernels need no work split): the plan the
    decode calls of all layers of the step share -- pass it as ``plan=`` to
    ``l20_paged_split_kv_attention_fp8`` / ``l20_paged_split_kv_attention``.  One small kernel
    over the lengths and the block table; ``plan`` reuses a buffer.  Returns ``None`` for
    geometries the balanced kernel does not take (their calls need no plan)."""
    _, num_q_heads, head_dim = query.shape
    num_kv_heads = key_cache.shape[2]
    if head_dim != 128 or num_q_heads // num_kv_heads > BALANCED_MAX_GROUP or workspace[0].dtype != torch.float32:
        return None
    return _ops().plan_decode(
        query, key_cache, value_cache, block_table, seq_lens, workspace[0], workspace[1], workspace[2],
        max_seq_len, split_size, plan=plan,
    )


def should_use_l20_paged_split_kv(batch: int, max_seq_len: int) -> bool:
    # Same policy as the reference (:698-702): off until a serving A/B says otherwise.
    del batch, max_seq_len
    return False


def should_use_l20_paged_fp8_split_kv(batch: int, max_seq_len: int) -> bool:
    # Same policy as the reference (:705-709): production dispatch stays off until a serving
    # A/B on the target GPU says otherwise; VLLM_L20_FP8_PAGED_FORCE=1 bypasses this.
    del batch, max_seq_len
    return False
