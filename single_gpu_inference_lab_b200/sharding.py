"""Multi-GPU forms of the paged FP8 decode step (one process per GPU).

The reference project is single-GPU by design and has no collective anywhere; the two forms
below are the natural shardings of its operator:

* **sequence sharding** -- a batch is split by sequence, every rank owns the pages, block-table
  rows, query rows and output rows of its sequences.  No data-path communication at all.
  ``lpt_partition`` balances *tokens*, not sequence counts.
* **KV-range sharding** -- every sequence's pages are dealt out in contiguous page ranges, one
  range per rank; each rank runs the ordinary operator on its range, which yields packed
  ``[B, Hq, D + 2]`` fp32 records (``o`` un-normalised, ``m``, ``l``), every rank needs every
  rank's records and applies the same LSE merge the single-GPU split-KV path uses (reference
  maths: integrations/vllm/l20_paged_split_kv.py:459-488).  Two forms of the exchange:
  ``KvRangeExchange`` -- the decode kernels store their rows straight into every rank's receive
  buffer over NVLink and tag each row with the step, the merge kernel waits (bounded) for the
  tags: no collective call; and ``kv_range_decode`` -- ``packed_output`` plus one
  ``all_gather_into_tensor``, the fallback where peer mappings are not to be had (and on CPU
  ranks in tests).

Nothing here falls back to a CPU implementation: the default compute callbacks are the CUDA
operator; tests on CPU ranks inject their own.
"""

from __future__ import annotations

from dataclasses import replace
from typing import Callable, Optional

import torch
import torch.distributed as dist

from .workloads import PAGE_SIZE, PagedDecodeInputs


def lpt_partition(lengths, world_size: int) -> list[list[int]]:
    """Longest-processing-time-first assignment of sequences to ranks by context length.
    Returns, per rank, the sorted list of sequence indices."""
    lengths = [int(x) for x in lengths]
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    loads = [0] * world_size
    parts: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (loads[k], k))
        parts[r].append(i)
        loads[r] += lengths[i]
    return [sorted(p) for p in parts]


def compact_rows(inputs: PagedDecodeInputs, rows, page_lo, page_hi, seq_lens) -> PagedDecodeInputs:
    """Keep block-table columns [page_lo, page_hi) of ``rows`` and move the pages they name into
    a dense local pool (local ids in order of first use)."""
    table = inputs.block_table[rows][:, page_lo:page_hi].cpu().long()
    lens = seq_lens.cpu().long()
    used = []
    local = torch.zeros_like(table)
    remap: dict[int, int] = {}
    for r in range(table.shape[0]):
        n = -(-int(lens[r]) // PAGE_SIZE)
        for c in range(n):
            page = int(table[r, c])
            if page not in remap:
                remap[page] = len(used)
                used.append(page)
            local[r, c] = remap[page]
    if not used:
        used = [0]
    index = torch.tensor(used, dtype=torch.long, device=inputs.key_cache.device)
    return replace(
        inputs,
        query=inputs.query[rows],
        key_cache=inputs.key_cache[index].contiguous(),
        value_cache=inputs.value_cache[index].contiguous(),
        block_table=local.to(torch.int32).to(inputs.block_table.device),
        seq_lens=lens.to(torch.int32).to(inputs.seq_lens.device),
        max_seq_len=int(lens.max()) if lens.numel() else 0,
    )


def shard_sequences(inputs: PagedDecodeInputs, rank: int, world_size: int) -> tuple[PagedDecodeInputs, list[int]]:
    """This rank's sequences (token-balanced) with a compacted local page pool."""
    rows = lpt_partition(inputs.seq_lens.tolist(), world_size)[rank]
    idx = torch.tensor(rows, dtype=torch.long)
    return compact_rows(inputs, idx, 0, inputs.block_table.shape[1], inputs.seq_lens.cpu()[idx]), rows


def kv_range_bounds(max_seq_len: int, rank: int, world_size: int) -> tuple[int, int]:
    """Token range [lo, hi) of rank ``rank``: whole pages, ceil(pages / world) pages per rank."""
    pages = -(-max_seq_len // PAGE_SIZE)
    per = -(-pages // world_size)
    return rank * per * PAGE_SIZE, min((rank + 1) * per, pages) * PAGE_SIZE


def shard_kv_range(inputs: PagedDecodeInputs, rank: int, world_size: int) -> PagedDecodeInputs:
    """Every sequence's tokens [lo, hi) of this rank as a local cache, local block table and
    local lengths (0 for sequences that end before ``lo``).  The query stays replicated."""
    lo, hi = kv_range_bounds(inputs.max_seq_len, rank, world_size)
    lens = (inputs.seq_lens.cpu().long() - lo).clamp(0, max(hi - lo, 0))
    rows = torch.arange(inputs.query.shape[0])
    hi_page = max(hi // PAGE_SIZE, lo // PAGE_SIZE + 1)
    return compact_rows(inputs, rows, lo // PAGE_SIZE, hi_page, lens)


def _cuda_partial(local: PagedDecodeInputs, split_size: int, workspace=None, packed=None) -> torch.Tensor:
    from . import l20_paged_decode as ops
    from .l20_paged_split_kv import allocate_l20_paged_split_kv_workspace

    q = local.query
    if packed is None:
        packed = torch.empty(q.shape[0], q.shape[1], q.shape[2] + 2, device=q.device, dtype=torch.float32)
    ws = workspace or allocate_l20_paged_split_kv_workspace(q, max(local.max_seq_len, 1), split_size=split_size)
    ops.paged_decode_fp8_e4m3_split_out_v2(
        q, local.key_cache, local.value_cache, local.block_table, local.seq_lens, ws[0], ws[1], ws[2], None,
        local.k_scale, local.v_scale, local.max_seq_len, split_size, packed_output=packed,
    )
    return packed


def _cuda_merge(gathered: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    from . import l20_paged_decode as ops

    return ops.merge_packed_partials(gathered, torch.empty_like(like))


def kv_range_decode(
    local: PagedDecodeInputs,
    *,
    split_size: int = 2048,
    group: Optional[dist.ProcessGroup] = None,
    partial_fn: Callable[[PagedDecodeInputs, int], torch.Tensor] = _cuda_partial,
    merge_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor] = _cuda_merge,
    gather_buffer: Optional[torch.Tensor] = None,
    workspace=None,
    packed_buffer: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One decode step of a KV-range-sharded batch: local packed partial, one all-gather of
    ``[B, Hq, D + 2]`` fp32 per rank, LSE merge on every rank.  Returns ``[B, Hq, D]``.
    ``workspace`` / ``packed_buffer`` / ``gather_buffer`` let a caller reuse its allocations."""
    if partial_fn is _cuda_partial:
        packed = _cuda_partial(local, split_size, workspace, packed_buffer)
    else:
        packed = partial_fn(local, split_size).contiguous()
    world = dist.get_world_size(group)
    if gather_buffer is None:
        gather_buffer = torch.empty((world, *packed.shape), device=packed.device, dtype=packed.dtype)
    # concatenation along dim 0 is the layout every backend accepts; [world*B,...] == [world,B,...]
    dist.all_gather_into_tensor(gather_buffer.view(-1, *packed.shape[1:]), packed, group=group)
    return merge_fn(gather_buffer, local.query)


class KvRangeExchange:
    """Receive buffers and peer mappings of the in-kernel KV-range exchange
    (``pfd_exchange`` of include/paged_fp8_decode.h) for a fixed ``[B, Hq, D]`` step shape.

    ``KvRangeExchange.create`` is the multi-process form: every rank allocates its own memory,
    the ranks swap CUDA IPC handles over the process group (host side, once) and map each
    other's.  ``KvRangeExchange.emulate`` builds all ranks' objects inside ONE process on one
    device, for tests that issue the ranks' calls one after another on one stream.
    """

    def __init__(self, rank: int, world: int, rows: int, head_dim: int, bases: list[int], owned: int,
                 opened: list[int], device: torch.device):
        from . import cabi

        self.rank, self.world, self.rows, self.head_dim = rank, world, rows, head_dim
        self.device = device
        self._owned, self._opened = owned, opened
        _, control_off = cabi.exchange_geometry(world, rows, head_dim)
        x = cabi.Exchange()
        x.world, x.rank = world, rank
        for r in range(world):
            x.recv[r] = bases[r]
        x.control = bases[rank] + control_off
        self.struct = x

    @classmethod
    def create(cls, batch: int, num_q_heads: int, head_dim: int, device, group=None) -> "KvRangeExchange":
        from . import cabi

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        rows = batch * num_q_heads
        nbytes, _ = cabi.exchange_geometry(world, rows, head_dim)
        with torch.cuda.device(device):
            base, handle = cabi.exchange_alloc(nbytes)
            handles: list = [None] * world
            dist.all_gather_object(handles, handle, group=group)
            bases, opened = [], []
            for r in range(world):
                if r == rank:
                    bases.append(base)
                else:
                    bases.append(cabi.exchange_open(handles[r]))
                    opened.append(bases[-1])
        return cls(rank, world, rows, head_dim, bases, base, opened, torch.device(device))

    @classmethod
    def emulate(cls, world: int, batch: int, num_q_heads: int, head_dim: int, device) -> list["KvRangeExchange"]:
        from . import cabi

        rows = batch * num_q_heads
        nbytes, _ = cabi.exchange_geometry(world, rows, head_dim)
        with torch.cuda.device(device):
            bases = [cabi.exchange_alloc(nbytes)[0] for _ in range(world)]
        return [cls(r, world, rows, head_dim, bases, bases[r], [], torch.device(device)) for r in range(world)]

    def decode(self, local: PagedDecodeInputs, *, split_size: int, workspace, plan=None, flags: int = 0) -> None:
        """This rank's range through the operator; its packed rows go to every rank."""
        from . import cabi

        cabi.paged_decode_fp8_e4m3_split_out(
            local.query, local.key_cache, local.value_cache, local.block_table, local.seq_lens,
            k_scale=local.k_scale, v_scale=local.v_scale, max_seq_len=local.max_seq_len, split_size=split_size,
            workspace=workspace, plan=plan, flags=flags, exchange=self.struct,
        )

    def merge(self, output: torch.Tensor) -> torch.Tensor:
        """Wait (bounded) for every rank's rows of the current step and merge them into ``output``."""
        from . import cabi

        cabi.exchange_merge(self.struct, output)
        return output

    def close(self) -> None:
        from . import cabi

        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._opened:
                cabi.exchange_close(p)
            self._opened = []
            if self._owned:
                cabi.exchange_free(self._owned)
                self._owned = 0


def kv_range_decode_exchange(
    local: PagedDecodeInputs, exchange: KvRangeExchange, *, split_size: int = 2048, workspace=None, plan=None,
    flags: int = 0, output: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One decode step of a KV-range-sharded batch with the exchange inside the kernels: two calls,
    no collective, nothing per step on the host (the step count lives on the device, so the pair
    can be captured in a CUDA graph and replayed).  Every rank must call it once per step.
    Returns ``[B, Hq, D]``."""
    from .l20_paged_split_kv import allocate_l20_paged_split_kv_workspace

    if workspace is None:
        workspace = allocate_l20_paged_split_kv_workspace(local.query, max(local.max_seq_len, 1), split_size=split_size)
    if output is None:
        output = torch.empty_like(local.query)
    exchange.decode(local, split_size=split_size, workspace=workspace, plan=plan, flags=flags)
    return exchange.merge(output)
