#!/usr/bin/env python3
"""Benchmark of the paged FP8-KV GQA decode-attention step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One *step* is one decode-attention layer-step over one synthetic batch.  Metric: KV bytes read
per second (``sum_b ctx_b * Hkv * D * 2`` bytes per step), microseconds per layer-step beside
it.  Rank 0 prints ONE JSON line.

* ``value``        device-resident operands, CUDA events around K back-to-back steps replayed from
                   CUDA graphs; successive steps use different KV pools so that every step reads
                   from HBM, not L2.  Median of ``repeats`` such K-step runs.
* ``correct`` / ``max_abs_error``  the exact call that is timed (same flags, split, workspace,
                   plan, pool 0), run once before the timing and checked against the CPU oracle
                   on a bounded sample of sequences (gate ``|a-b| <= 2e-3 + 1e-2 |b|``).
* ``roofline``     the dominant kernel alone (merge skipped) against the measured HBM copy peak;
                   ``traffic`` is read from ``profiles/traffic.json`` (ncu captures).
* ``isolated``     the same step with an unrelated ordinary kernel launched between steps, i.e.
                   without the overlap of one step's prologue with the previous step's tail that
                   programmatic dependent launch gives back-to-back decode calls.
* ``e2e``          the call a serving hook makes (``l20_paged_split_kv_attention_fp8``) with the
                   step's query / block table / sequence lengths copied from pinned host memory
                   and the output copied back, every step.  The KV cache is the resident state of
                   the serving engine and stays on the device.
* ``per_config``   (N = 1) the other four configurations, each with the same fields in short.
* ``sharded``      (N > 1) the two sharded forms: the batch of 256 split by sequence over the
                   ranks (no communication) and the long-context batch split by KV range (packed
                   partials exchanged, merged on every rank), with the one-GPU figure measured in
                   the same run on rank 0 and the time of exchange + merge alone.
* ``cpu_baseline`` the CPU oracle (torch restatement of the reference's own torch path) timed
                   on this host's cores on the same batch.
* ``--impl reference`` times only that CPU path and prints its own line.

With N > 1 the headline is one batch per GPU, the same batch (seed) on every rank, no data-path
collective ("weak").  ``--strong`` / ``--workload llama3-8b-long-b4`` make a sharded form the
headline instead.  ``--kv-dtype bf16|fp16`` times the non-quantised sibling operator; ``--flags``
are the ``PFD_FLAG_*`` bits of the timed calls (default 32: early metadata reads; 288 adds early
K/V streaming).  ``--with-producer`` adds ``with_producer``: the fused RoPE + FP8 append of each
request's new token in front of every decode call, as in a model layer.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024
DEFAULT_WORKLOAD = "qwen2.5-coder-3b-b64"
ALL_WORKLOADS = ("qwen2.5-0.5b-b8", "qwen2.5-coder-3b-b64", "qwen2.5-7b-b256", "llama3-8b-long-b4", "shared-prefix-b64")
KERNEL_NAMES = {1: "paged_decode_fp8_partial_ldg_kernel", 2: "paged_decode_fp8_partial_tma_kernel",
                3: "paged_decode_fp8_chunk_kernel", 4: "paged_decode_fp8_chunk_kernel<KV16>",
                5: "paged_decode_fp8_chunk_kernel<FUSED>", 6: "paged_decode_fp8_chunk_kernel<KV16,FUSED>"}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=600)
    p.add_argument("--warmup", type=int, default=30)
    p.add_argument("--repeats", type=int, default=5, help="K-step runs; the median is reported")
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default=DEFAULT_WORKLOAD)
    p.add_argument("--split-size", type=int, default=0, help="0 = choose from the geometry")
    p.add_argument("--pools", type=int, default=0, help="distinct KV pools rotated through (0 = enough to exceed L2 x3)")
    p.add_argument("--kv-dtype", choices=["fp8", "bf16", "fp16"], default="fp8",
                   help="fp8: the e4m3 path (headline); bf16 / fp16: the non-quantised sibling operator, "
                        "caches and query in that type (single GPU, batch-sharded or weak scaling only)")
    p.add_argument("--exchange", choices=("peer", "nccl"), default="peer",
                   help="KV-range mode on several GPUs: 'peer' = the decode kernels store their packed rows into "
                        "every rank's receive buffer and the merge kernel waits for them (the all-gather form is "
                        "measured beside it); 'nccl' = packed_output + all_gather_into_tensor + merge only")
    p.add_argument("--graph-collective", action="store_true",
                   help="KV-range mode on several GPUs: replay the step, exchange included, from a CUDA graph "
                        "instead of launching every step eagerly")
    p.add_argument("--flags", type=int, default=32,
                   help="PFD_FLAG_* bits of the timed calls; default PFD_FLAG_EARLY_METADATA: the block table "
                        "and sequence lengths do not change between the timed layer-steps")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-per-config", action="store_true", help="skip the per_config / sharded sections")
    p.add_argument("--no-shared-prefix", action="store_true",
                   help="shared-prefix-b64 only: use the ordinary decode path instead of the dense tcgen05 prefix pass")
    p.add_argument("--single-launch", action="store_true",
                   help="with the plan: combine the pieces of cut sequences inside the balanced kernel (PFD_FLAG_SINGLE_LAUNCH)")
    p.add_argument("--no-plan", action="store_true",
                   help="do not plan the step: every call derives its work split itself")
    p.add_argument("--with-producer", action="store_true",
                   help="also time producer + decode: the fused RoPE + FP8 append of each request's new token in front of "
                        "every decode call, as in a model layer (reported as `with_producer`)")
    p.add_argument("--producer-step", action="store_true",
                   help="time the step in front of decode attention instead (rotary embedding + FP8 quantise + paged "
                        "KV append, l20_rope_and_cache) and print its own JSON line")
    p.add_argument("--grouped-prefix", action="store_true",
                   help="shared-prefix-b64 only: find the groups on the device (once, as per model step) and run the "
                        "grouped shared-prefix entry instead of the single-group one")
    p.add_argument("--strong", action="store_true",
                   help="N > 1: shard ONE batch by sequence over the ranks (token-balanced) instead of one batch per rank")
    return p.parse_args()


def measured_peak() -> tuple[float, str]:
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(peaks["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic(workload: str, kernel: str):
    """dram bytes read + written per launch of `kernel` on `workload`, from the tracked summary of
    the ncu captures (None when there is no capture of that pair)."""
    try:
        table = json.loads((ROOT / "profiles" / "traffic.json").read_text())
    except Exception:
        return None
    for row in table.get("captures", []):
        if row.get("workload") == workload and row.get("kernel") == kernel:
            return int(row["dram_bytes_read"]) + int(row["dram_bytes_write"])
    return None


def bind_to_own_cores(local_rank: int, local_world: int) -> list[int]:
    """Give every rank of the node its own slice of the host cores, so that the per-step host
    path of one rank (copies, launches, stream sync) is not scheduled on another rank's cores."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = max(1, len(cores) // max(local_world, 1))
        mine = cores[local_rank * per:(local_rank + 1) * per] or cores
        os.sched_setaffinity(0, mine)
        return mine
    except Exception:
        return []


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed loops run."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        n = self._nvml
        names = {
            "hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(n, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
                get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self._h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self._period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# --------------------------------------------------------------------------- CPU oracle legs
def cpu_reference_run(w, sample_rows: int, repeats: int):
    """Time the CPU oracle on the first ``sample_rows`` sequences (their pages compacted into
    a cache of their own first, outside the timed region); returns (GB/s, seconds, bytes)."""
    from oracle import paged_decode_oracle as oracle
    from single_gpu_inference_lab_b200 import sharding

    torch.set_num_threads(os.cpu_count() or 1)
    rows = torch.arange(sample_rows)
    sub = sharding.compact_rows(w, rows.to(w.query.device), 0, w.block_table.shape[1], w.seq_lens.cpu()[rows]).to("cpu")
    table = sub.block_table.long()
    hkv, d = sub.key_cache.shape[2], sub.key_cache.shape[3]
    nbytes = int(sub.seq_lens.sum()) * hkv * d * 2 * sub.key_cache.element_size()
    best = float("inf")
    for attempt in range(repeats + 1):  # the first pass is the warm-up
        t0 = time.perf_counter()
        if sub.key_cache.dtype == torch.float8_e4m3fn:
            oracle.reference(sub.query, sub.key_cache, sub.value_cache, table, sub.seq_lens, sub.k_scale, sub.v_scale)
        else:
            oracle.reference_kv16(sub.query, sub.key_cache, sub.value_cache, table, sub.seq_lens)
        dt = time.perf_counter() - t0
        if attempt > 0 or repeats == 0:
            best = min(best, dt)
    return nbytes / best / 1e9, best, nbytes


def check_against_oracle(w, out: torch.Tensor, token_budget: int = 150_000) -> tuple[bool, float, str]:
    """Compare ``out`` (the timed call's result) with the CPU oracle on a bounded sample of
    sequences: the first, the last, the longest and the shortest, then more until the budget of
    tokens is spent.  The checker only: nothing here is timed."""
    from oracle import paged_decode_oracle as oracle
    from single_gpu_inference_lab_b200 import sharding

    lens = w.seq_lens.cpu().long()
    batch = lens.numel()
    order = [0, batch - 1, int(lens.argmax()), int(lens.argmin())] + list(range(1, batch - 1))
    rows, spent = [], 0
    for b in order:
        if b in rows or int(lens[b]) == 0:
            continue
        if rows and spent + int(lens[b]) > token_budget:
            continue
        rows.append(b)
        spent += int(lens[b])
        if spent >= token_budget:
            break
    idx = torch.tensor(sorted(rows))
    sub = sharding.compact_rows(w, idx.to(w.query.device), 0, w.block_table.shape[1], lens[idx]).to("cpu")
    if sub.key_cache.dtype == torch.float8_e4m3fn:
        exp = oracle.reference(sub.query, sub.key_cache, sub.value_cache, sub.block_table.long(), sub.seq_lens,
                               sub.k_scale, sub.v_scale)
    else:
        exp = oracle.reference_kv16(sub.query, sub.key_cache, sub.value_cache, sub.block_table.long(), sub.seq_lens)
    got = out[idx.to(out.device)].float().cpu()
    err = (got - exp.float()).abs()
    ok = bool(torch.isfinite(got).all()) and bool((err <= 2e-3 + 1e-2 * exp.float().abs()).all())
    return ok, float(err.max()), f"{len(rows)} of {batch} sequences ({spent} tokens)"


def run_reference_arm(args, rank: int) -> int:
    """The reference's own CPU torch path for this operator (its ``reference()`` restated in
    oracle/), all host threads, on a bounded sample of the workload.  Rank 0 only."""
    if rank != 0:
        return 0
    from single_gpu_inference_lab_b200.workloads import make_inputs

    cores = os.cpu_count() or 1
    shrink = 1.0 / 32 if args.workload == "llama3-8b-long-b4" else 1.0
    w = make_inputs(args.workload, seed=0, device="cpu", shrink=shrink)
    batch = w.query.shape[0]
    sample_rows = batch
    torch.set_num_threads(cores)
    times = []
    nbytes = 0
    for i in range(args.warmup + args.steps):
        gbs, dt, nbytes = cpu_reference_run(w, sample_rows, 0)
        if i >= args.warmup:
            times.append(dt)
        if sum(times) > 150:  # bound the arm to a few minutes whatever K is
            break
    ms = 1e3 * sum(times) / len(times)
    value = nbytes / (ms * 1e-3) / 1e9
    sample = f"{sample_rows} of {batch} sequences of {args.workload}" + (f" with contexts scaled by {shrink}" if shrink != 1.0 else "")
    line = {
        "impl": "reference",
        "metric": "decode_attn_kv_read_gbs", "value": round(value, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "us_per_layer_step": round(ms * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 KV, bf16 q, fp32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "sample": sample, "kv_bytes_per_step": nbytes},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------- one workload on this rank
class Case:
    """One workload resident on this rank's GPU: inputs, rotating KV pools, workspace, plan and
    the timed call.  ``mode``: "batch" (this rank's own batch), "strong" (its share of one batch
    split by sequence), "kv-range" (its KV range of every sequence, packed partials exchanged)."""

    def __init__(self, args, workload: str, dev, rank: int, world: int, mode: str, seed: int = 0):
        from single_gpu_inference_lab_b200 import cabi, l20_paged_split_kv, sharding
        from single_gpu_inference_lab_b200.workloads import make_inputs

        self.args, self.workload, self.dev, self.rank, self.world, self.mode = args, workload, dev, rank, world, mode
        self.cabi = cabi
        kv16 = {"fp8": None, "bf16": torch.bfloat16, "fp16": torch.float16}[args.kv_dtype]
        self.kv16 = kv16
        gen_kw = {} if kv16 is None else {"kv_dtype": kv16, "query_dtype": kv16}
        if mode == "kv-range":
            full_len = 131072
            lo, hi = sharding.kv_range_bounds(full_len, rank, world)
            w = make_inputs(workload, seed=seed + rank, device=dev, shrink=(hi - lo) / full_len)
        elif mode == "strong":
            full = make_inputs(workload, seed=seed, device=dev, **gen_kw)  # same batch on every rank
            w, _rows = sharding.shard_sequences(full, rank, world)
            del full
            torch.cuda.empty_cache()
        else:
            w = make_inputs(workload, seed=seed, device=dev, **gen_kw)
        self.w = w
        q = w.query
        self.batch, self.hq, self.d = q.shape
        self.hkv = w.key_cache.shape[2]
        self.kv_bytes = w.kv_bytes
        self.split = args.split_size or l20_paged_split_kv.choose_split_size(
            self.batch, self.hkv, w.max_seq_len, seq_lens=w.seq_lens.tolist())
        self.pool_bytes = 2 * w.key_cache.numel() * w.key_cache.element_size()
        pools = args.pools or max(2, -(-3 * L2_BYTES // self.pool_bytes) + 1)
        self.pools = min(pools, max(2, int(40e9 // self.pool_bytes)))
        self.kcs = [w.key_cache] + [w.key_cache.clone() for _ in range(self.pools - 1)]
        self.vcs = [w.value_cache] + [w.value_cache.clone() for _ in range(self.pools - 1)]
        self.shared_prefix = w.prefix_len > 0 and not args.no_shared_prefix and self.d == 128 and kv16 is None
        if self.shared_prefix and not args.split_size:
            from single_gpu_inference_lab_b200.l20_shared_prefix_decode_dispatch import choose_suffix_split_size

            self.split = choose_suffix_split_size(self.batch, self.hkv, w.max_seq_len - w.prefix_len)
        self.ws = l20_paged_split_kv.allocate_l20_paged_split_kv_workspace(q, w.max_seq_len, split_size=self.split)
        if self.shared_prefix:
            from single_gpu_inference_lab_b200 import l20_shared_prefix_decode_dispatch as spd

            self.spd = spd
            self.ws = spd.allocate_shared_prefix_workspace(q, w.max_seq_len, w.prefix_len, suffix_split_size=self.split)
        # --grouped-prefix: the groups are discovered on the device from the block table and the
        # lengths (once, as an engine does per model step); every timed layer-step reads them
        self.groups = None
        if self.shared_prefix and args.grouped_prefix:
            self.groups, self.max_groups = cabi.group_shared_prefixes(w.block_table, seq_lens=w.seq_lens, min_batch=8,
                                                                      min_prefix_len=4096, max_groups=4)
            # one host read per model step, as the decode hook does: are all requests in groups?
            self.group_flags = cabi.PFD_FLAG_ALL_IN_GROUPS if int(self.groups[4].item()) == self.batch else 0
            self.prefix_bound = (w.prefix_len + 255) // 256 * 256  # an engine knows how long its cached prefixes can be
            self.suffix_bound = max(w.max_seq_len - 4096, 16)  # true for any group the grouping call above can find
            self.split = choose_suffix_split_size(self.batch, self.hkv, self.suffix_bound) if not args.split_size else self.split
            slots = self.prefix_bound // 256 + -(-self.suffix_bound // self.split)
            self.ws = (torch.empty(self.batch, self.hq, slots, self.d, device=dev), torch.empty(self.batch, self.hq, slots, device=dev),
                       torch.empty(self.batch, self.hq, slots, device=dev), torch.empty_like(q))
            torch.cuda.synchronize()
        self.out = self.ws[3]
        self.flags = args.flags
        # The plan of the model step: block table and lengths are the same for every layer, so the
        # work split is computed once, outside the timed layer-steps, as an engine does per step.
        self.plan = None
        if not args.no_plan and not self.shared_prefix and self.d == 128 and self.hq // self.hkv <= 8 and not (self.flags & (1 | 2 | 8)):
            self.plan = cabi.plan_decode(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, max_seq_len=w.max_seq_len,
                                         split_size=self.split, workspace=self.ws)
            torch.cuda.synchronize()
            if args.single_launch:
                self.flags |= cabi.PFD_FLAG_SINGLE_LAUNCH
        kvr = mode == "kv-range"
        # KV-range mode on several GPUs: the decode kernels store their packed rows straight into
        # every rank's receive buffer ("peer"); the all-gather form is measured beside it.
        self.xch = None
        if kvr and world > 1 and args.exchange == "peer":
            self.xch = sharding.KvRangeExchange.create(self.batch, self.hq, self.d, dev)
        self.packed = torch.empty(self.batch, self.hq, self.d + 2, device=dev) if kvr else None
        self.gathered = torch.empty(world, self.batch, self.hq, self.d + 2, device=dev) if kvr else None
        self.filler = torch.zeros(1 << 14, device=dev)

    # -- the timed call
    def step(self, i: int, flags=None, exchange: bool = True, peer: bool = True):
        import torch.distributed as dist

        cabi, w = self.cabi, self.w
        flags = self.flags if flags is None else flags
        kc, vc = self.kcs[i % self.pools], self.vcs[i % self.pools]
        if self.kv16 is not None:
            cabi.paged_decode_kv16_split_out(
                w.query, kc, vc, w.block_table, w.seq_lens, max_seq_len=w.max_seq_len,
                split_size=self.split, output=self.out, workspace=self.ws, flags=flags, plan=self.plan)
            return
        if self.groups is not None:
            cabi.shared_prefix_decode_grouped_fp8_e4m3(
                w.query, kc, vc, w.block_table, w.seq_lens, groups=self.groups, max_groups=self.max_groups,
                max_prefix_len=self.prefix_bound, max_suffix_len=self.suffix_bound, k_scale=w.k_scale, v_scale=w.v_scale,
                max_seq_len=w.max_seq_len,
                split_size=self.split, output=self.out, workspace=self.ws, flags=self.group_flags)
            return
        if self.shared_prefix:
            cabi.shared_prefix_decode_fp8_e4m3(
                w.query, kc, vc, w.block_table, w.seq_lens, prefix_len=w.prefix_len,
                k_scale=w.k_scale, v_scale=w.v_scale, max_seq_len=w.max_seq_len, split_size=self.split, output=self.out,
                workspace=self.ws)
            return
        kvr = self.mode == "kv-range"
        if kvr and self.xch is not None and peer and exchange and not (flags & cabi.PFD_FLAG_PARTIAL_ONLY):
            cabi.paged_decode_fp8_e4m3_split_out(
                w.query, kc, vc, w.block_table, w.seq_lens, k_scale=w.k_scale, v_scale=w.v_scale,
                max_seq_len=w.max_seq_len, split_size=self.split, workspace=self.ws, flags=flags, plan=self.plan,
                exchange=self.xch.struct)
            cabi.exchange_merge(self.xch.struct, self.out)
            return
        cabi.paged_decode_fp8_e4m3_split_out(
            w.query, kc, vc, w.block_table, w.seq_lens, k_scale=w.k_scale, v_scale=w.v_scale,
            max_seq_len=w.max_seq_len, split_size=self.split, output=None if kvr else self.out,
            packed_output=self.packed, workspace=self.ws, flags=flags, plan=self.plan,
        )
        if kvr and exchange and not (flags & cabi.PFD_FLAG_PARTIAL_ONLY):
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered.view(-1, self.hq, self.d + 2), self.packed)
            else:
                self.gathered[0].copy_(self.packed)
            cabi.merge_packed(self.gathered, self.out)

    def step_allgather(self, i: int):
        """KV-range mode: the step with the packed partials exchanged by one all-gather."""
        self.step(i, peer=False)

    def exchange_only(self, i: int):
        """KV-range mode: the exchange of the packed partials and the merge, without the kernel."""
        import torch.distributed as dist

        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1, self.hq, self.d + 2), self.packed)
        else:
            self.gathered[0].copy_(self.packed)
        self.cabi.merge_packed(self.gathered, self.out)

    def isolated_step(self, i: int):
        """The step behind an unrelated ordinary kernel: no overlap with the previous step."""
        self.filler.add_(1.0)
        self.step(i)

    # -- timing helpers (device time, CUDA events on the launching stream, max over ranks)
    def barrier(self):
        import torch.distributed as dist

        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def _max_over_ranks(self, ms: float) -> float:
        import torch.distributed as dist

        t = torch.tensor([ms], device=self.dev)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_eager(self, fn, steps: int) -> float:
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        self.barrier()
        return self._max_over_ranks(e0.elapsed_time(e1) / steps)

    def timed_graph(self, fn, steps: int, repeats: int = 1, collective: bool = False) -> tuple[float, list[float]]:
        """ms per step with the K steps replayed from CUDA graphs (a graph of `chunk` consecutive
        steps replayed, plus one for the remainder) so that host launch overhead does not pace
        the device: exactly `steps` steps run inside each timed region.  Returns the median of
        `repeats` such regions and all of them."""
        if collective and self.world > 1 and not self.args.graph_collective:
            runs = [self.timed_eager(fn, steps) for _ in range(repeats)]  # the collective is launched eagerly
            return statistics.median(runs), runs
        chunk = min(steps, max(self.pools, (64 // self.pools) * self.pools))
        reps, rest = divmod(steps, chunk)
        side = torch.cuda.Stream()
        graphs = []
        with torch.cuda.stream(side):
            for count in (chunk, rest):
                if count == 0:
                    graphs.append(None)
                    continue
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(count):
                        fn(i)
                graphs.append(g)
        self.barrier()  # ranks whose kernels wait for one another start their replays together
        graphs[0].replay()
        runs = []
        for _ in range(repeats):
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graphs[0].replay()
            if graphs[1] is not None:
                graphs[1].replay()
            e1.record()
            self.barrier()
            runs.append(self._max_over_ranks(e0.elapsed_time(e1) / steps))
        return statistics.median(runs), runs

    def measure(self, steps: int, warmup: int, repeats: int, check: bool, isolated: bool = True) -> dict:
        """Warm up, check the timed call against the oracle, then time step / kernel / isolated."""
        cabi = self.cabi
        kvr = self.mode == "kv-range"
        for i in range(max(warmup, 3)):
            self.step(i)
        torch.cuda.synchronize()
        res = {}
        if check:
            self.out.fill_(float("nan"))
            self.step(0)
            torch.cuda.synchronize()
            res["status"] = cabi.device_status()
            if kvr and self.world > 1:
                res["correct"], res["max_abs_error"] = None, None
                res["checked"] = "KV-range shards hold independent data; parity of this mode is tests/test_multi_gpu.py"
            else:
                ok, err, what = check_against_oracle(self.w, self.out)
                res["correct"], res["max_abs_error"], res["checked"] = bool(ok and res["status"] == 0), err, what
        before = cabi.launch_count()
        self.step(0)
        res["launches_per_step"] = cabi.launch_count() - before
        res["path"] = cabi.last_path()
        ms_step, runs = self.timed_graph(self.step, steps, repeats, collective=kvr and self.xch is None)
        res["ms_step"], res["runs_us"] = ms_step, [round(r * 1e3, 3) for r in runs]
        single = self.shared_prefix or res["launches_per_step"] == 1
        if single:
            res["ms_kernel"] = ms_step
        else:
            res["ms_kernel"], _ = self.timed_graph(
                lambda i: self.step(i, self.flags | cabi.PFD_FLAG_PARTIAL_ONLY, exchange=False), steps, 1)
        if isolated:
            res["ms_isolated"], _ = self.timed_graph(self.isolated_step, steps, 1, collective=kvr and self.xch is None)
            ms_fill, _ = self.timed_graph(lambda i: self.filler.add_(1.0), steps, 1)
            res["ms_isolated"] = max(res["ms_isolated"] - ms_fill, 0.0)
        if kvr and self.xch is not None:
            res["ms_exchange"] = max(ms_step - res["ms_kernel"], 0.0)
            res["ms_step_allgather"], _ = self.timed_graph(self.step_allgather, steps, 1, collective=True)
            res["ms_exchange_allgather"], _ = self.timed_graph(self.exchange_only, steps, 1, collective=True)
            res["exchange_status"] = cabi.device_status()
        elif kvr:
            res["ms_exchange"], _ = self.timed_graph(self.exchange_only, steps, 1, collective=True)
        return res

    # -- producer + decode, as in a model layer: the new token of every request is rotated,
    # quantised and appended by the kernel in front of the decode call
    def init_producer(self):
        w, dev = self.w, self.w.query.device
        gen = torch.Generator(device="cpu").manual_seed(1)
        mk = lambda heads: torch.randn(self.batch, heads, self.d, generator=gen).to(w.query.dtype).to(dev)
        self.pq, self.pk, self.pv = mk(self.hq), mk(self.hkv), mk(self.hkv)
        pos = (w.seq_lens.long() - 1).clamp_min(0)
        self.ppos = pos.to(dev)
        rows = torch.arange(self.batch, device=dev)
        self.pslots = w.block_table[rows, (self.ppos // 16)].long() * 16 + self.ppos % 16
        angle = torch.rand(int(pos.max()) + 1, self.d // 2, generator=gen) * 6.2831853
        self.cos_sin = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).to(dev)

    def producer(self, i: int):
        from single_gpu_inference_lab_b200 import l20_rope_kv

        w = self.w
        l20_rope_kv.l20_rope_and_cache(self.pq, self.pk, self.pv, self.ppos, self.cos_sin, True, self.kcs[i % self.pools],
                                       self.vcs[i % self.pools], self.pslots, k_scale=w.k_scale, v_scale=w.v_scale)

    def measure_with_producer(self, steps: int, repeats: int) -> dict:
        self.init_producer()

        def both(i):
            self.producer(i)
            self.step(i)

        for i in range(3):
            both(i)
        torch.cuda.synchronize()
        ms_both, runs = self.timed_graph(both, steps, repeats)
        ms_prod, _ = self.timed_graph(self.producer, steps, 1)
        return {"us_per_layer_step": round(ms_both * 1e3, 3), "runs_us": [round(r * 1e3, 3) for r in runs],
                "producer_alone_us": round(ms_prod * 1e3, 3), "status": self.cabi.device_status(),
                "what": "fused RoPE + FP8 append of one new token per request (its last position), then the decode call; "
                        "the decode call's flags are the run's"}

    def kernel_name(self, path: int) -> str:
        if self.shared_prefix:
            return "shared_prefix_dense_kernel + paged_decode_fp8_partial_tma_kernel + paged_decode_merge_kernel"
        return KERNEL_NAMES.get(path, "?")

    def release(self):
        if self.xch is not None:
            self.barrier()  # no rank still stores into another's buffer
            self.xch.close()
            self.xch = None
        del self.kcs, self.vcs, self.ws, self.w
        torch.cuda.empty_cache()


def short_report(case: Case, res: dict, peak: float, world_bytes: float, world: int) -> dict:
    """The per-configuration fields of ``per_config`` / ``sharded``."""
    us = res["ms_step"] * 1e3
    gbs = world_bytes / (res["ms_step"] * 1e-3) / 1e9
    out = {
        "us_per_layer_step": round(us, 3), "kv_read_gbs": round(gbs, 1),
        "step_frac_of_hbm_peak": round(gbs / (peak * world), 4),
        "kernel": case.kernel_name(res["path"]), "kernel_us": round(res["ms_kernel"] * 1e3, 3),
        "kernel_frac_of_hbm_peak": round(case.kv_bytes / (res["ms_kernel"] * 1e-3) / 1e9 / peak, 4),
        "path": case.cabi.PATH_NAMES.get(res["path"], "?"), "launches_per_step": res["launches_per_step"],
        "kv_bytes_per_step_per_gpu": case.kv_bytes, "runs_us": res["runs_us"],
    }
    if "ms_isolated" in res:
        out["isolated_us_per_layer_step"] = round(res["ms_isolated"] * 1e3, 3)
    if "correct" in res:
        out["correct"], out["max_abs_error"], out["checked"] = res["correct"], res["max_abs_error"], res["checked"]
    if "ms_exchange" in res:
        out["exchange_and_merge_us"] = round(res["ms_exchange"] * 1e3, 3)
    if "ms_step_allgather" in res:
        out["exchange"] = ("inside the kernels: rows stored to every rank over NVLink as tagged 8-byte words, bounded "
                           "wait for them in the merge kernel; exchange_and_merge_us = step - decode kernels alone")
        out["exchange_status"] = res["exchange_status"]
        out["allgather_form"] = {"us_per_layer_step": round(res["ms_step_allgather"] * 1e3, 3),
                                 "exchange_and_merge_us": round(res["ms_exchange_allgather"] * 1e3, 3),
                                 "what": "packed_output + one NCCL all_gather_into_tensor + merge kernel, launched eagerly"}
    return out


def run_producer_step(args) -> int:
    """The producer step alone: T new tokens (one per request of a decode step, or a prefill
    chunk), qwen2.5-coder-3b geometry, FP8 caches with per-head scales.  Bytes moved per token:
    q, k read and written back, v read, cos / sin rows read, k and v written as e4m3."""
    from single_gpu_inference_lab_b200 import l20_rope_kv

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hq, hkv, d = 16, 2, 128
    gen = torch.Generator(device="cpu").manual_seed(0)
    rows = []
    for tokens in (64, 256, 1024, 4096, 16384):
        q = torch.randn(tokens, hq, d, generator=gen).to(torch.bfloat16).to(dev)
        k = torch.randn(tokens, hkv, d, generator=gen).to(torch.bfloat16).to(dev)
        v = torch.randn(tokens, hkv, d, generator=gen).to(torch.bfloat16).to(dev)
        angle = torch.rand(8192, d // 2, generator=gen) * 6.2831853
        cos_sin = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).to(dev)
        pos = torch.randint(0, 8192, (tokens,), generator=gen).to(dev)
        blocks = tokens // 16 + 64
        slots = torch.randperm(blocks * 16, generator=gen)[:tokens].to(dev)
        kc = torch.zeros(blocks, 16, hkv, d, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        vc = torch.zeros_like(kc)
        ks = torch.full((hkv,), 0.01, device=dev)
        vs = torch.full((hkv,), 0.01, device=dev)

        def call():
            l20_rope_kv.l20_rope_and_cache(q, k, v, pos, cos_sin, True, kc, vc, slots, k_scale=ks, v_scale=vs)

        for _ in range(5):
            call()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side), torch.cuda.graph(g, stream=side):
            for _ in range(20):
                call()
        torch.cuda.synchronize()
        g.replay()
        runs = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            runs.append(e0.elapsed_time(e1) / 20 * 1e3)
        us = statistics.median(runs)
        nbytes = tokens * ((hq + hkv) * d * 2 * 2 + hkv * d * 2 + d * 4 + 2 * hkv * d)
        rows.append({"tokens": tokens, "us_per_call": round(us, 3), "bytes_per_call": nbytes,
                     "gbs": round(nbytes / (us * 1e-6) / 1e9, 1)})
    peak, peak_kind = measured_peak()
    print(json.dumps({"metric": "rope_quant_append_us", "unit": "us", "geometry": {"q_heads": hq, "kv_heads": hkv, "head_dim": d},
                      "dtype": "bf16 q/k/v, fp32 cos/sin table, e4m3 caches, per-head scales", "kernel": "rope_quant_append_vec_kernel",
                      "timing": "20 calls per CUDA graph replay, CUDA events, median of 5; operands of the larger sizes exceed L2",
                      "hbm_peak_gbs": peak, "peak_source": peak_kind, "rows": rows}))
    return 0


def main() -> int:
    args = parse_args()
    if args.producer_step:
        return run_producer_step(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    if args.impl == "reference":
        return run_reference_arm(args, rank)
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the operator has no CPU path")
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    import torch.distributed as dist

    from single_gpu_inference_lab_b200 import cabi, l20_paged_split_kv, sharding

    cores = bind_to_own_cores(local_rank, local_world) if world > 1 else []
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cabi.load()
    peak, peak_kind = measured_peak()

    kv16 = args.kv_dtype != "fp8"
    if args.workload == "llama3-8b-long-b4" and not kv16:
        mode, scaling = "kv-range", "strong"
    elif args.strong and world > 1:
        mode, scaling = "strong", "strong"
    else:
        mode, scaling = "batch", "weak"
    case = Case(args, args.workload, dev, rank, world, mode)
    w, q = case.w, case.w.query

    # -------- e2e operands: the per-step inputs (q, block table, lengths) packed into ONE pinned host
    # buffer and copied with one transfer into a device buffer the operands are views of
    def aligned(n: int) -> int:
        return (n + 255) // 256 * 256

    q_bytes, t_bytes, l_bytes = q.numel() * q.element_size(), w.block_table.numel() * 4, w.seq_lens.numel() * 4
    off_t, off_l = aligned(q_bytes), aligned(q_bytes) + aligned(t_bytes)
    # two sets of buffers: the inputs of step i + 1 cross PCIe on a copy stream while step i computes
    host_in = torch.empty(off_l + aligned(l_bytes), dtype=torch.uint8).pin_memory()
    dev_ins = [torch.empty_like(host_in, device=dev) for _ in range(2)]

    def views(buf):
        return (buf[:q_bytes].view(q.dtype).view(q.shape),
                buf[off_t:off_t + t_bytes].view(torch.int32).view(w.block_table.shape),
                buf[off_l:off_l + l_bytes].view(torch.int32).view(w.seq_lens.shape))

    hq_v, ht_v, hl_v = views(host_in)
    hq_v.copy_(q.cpu()); ht_v.copy_(w.block_table.cpu()); hl_v.copy_(w.seq_lens.cpu())
    dev_views = [views(b) for b in dev_ins]
    host_outs = [torch.empty(q.shape, dtype=q.dtype).pin_memory() for _ in range(2)]
    h2d = q_bytes + t_bytes + l_bytes
    d2h = host_outs[0].numel() * host_outs[0].element_size()
    stream = torch.cuda.current_stream()
    copy_stream = torch.cuda.Stream()
    in_ready = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    split, pools, ws = case.split, case.pools, case.ws

    def e2e_call(i: int, dq, dtable, dlens):
        kc, vc = case.kcs[i % pools], case.vcs[i % pools]
        if mode == "kv-range":
            local = w.__class__(**{**w.__dict__, "query": dq, "block_table": dtable, "seq_lens": dlens,
                                   "key_cache": kc, "value_cache": vc})
            if world > 1 and case.xch is not None:
                res = sharding.kv_range_decode_exchange(local, case.xch, split_size=split, workspace=ws, output=case.out)
            elif world > 1:
                res = sharding.kv_range_decode(local, split_size=split, gather_buffer=case.gathered, workspace=ws,
                                               packed_buffer=case.packed)
            else:
                res = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
                    dq, kc, vc, dtable, dlens, k_scale=w.k_scale, v_scale=w.v_scale,
                    max_seq_len=w.max_seq_len, split_size=split, workspace=ws)
        elif case.kv16 is not None:
            res = l20_paged_split_kv.l20_paged_split_kv_attention(
                dq, kc, vc, dtable, dlens, split_size=split, workspace=ws, max_seq_len=w.max_seq_len)
        elif case.groups is not None:
            # the step's own block table and lengths arrive with the step: group them, then decode
            from single_gpu_inference_lab_b200 import l20_paged_decode as ops

            found = ops.group_shared_prefixes(dtable, seq_lens=dlens, min_batch=8, min_prefix_len=4096,
                                              max_groups=case.max_groups, buffer=case.groups)
            res = ops.shared_prefix_decode_grouped_fp8_e4m3(
                dq, kc, vc, dtable, dlens, ws[0], ws[1], ws[2], ws[3], w.k_scale, w.v_scale, w.max_seq_len, split, found,
                max_prefix_len=case.prefix_bound, max_suffix_len=case.suffix_bound,
                all_in_groups=int(found.buffer[4].item()) == dq.shape[0])
        elif case.shared_prefix:
            res = case.spd.shared_paged_prefix_paged_suffix_gqa_decode_attention_fp8(
                dq, kc, vc, dtable, dlens, w.prefix_len, k_scale=w.k_scale, v_scale=w.v_scale,
                max_seq_len=w.max_seq_len, suffix_split_size=split, workspace=ws)
        else:
            res = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
                dq, kc, vc, dtable, dlens, k_scale=w.k_scale, v_scale=w.v_scale,
                max_seq_len=w.max_seq_len, split_size=split, workspace=ws)
        return res

    def e2e_serial_step(i: int):
        """Copy in, compute, copy out, wait: nothing of one step overlaps the next."""
        dev_ins[0].copy_(host_in, non_blocking=True)
        host_outs[0].copy_(e2e_call(i, *dev_views[0]), non_blocking=True)
        stream.synchronize()  # the host consumes the step's result

    def stage_inputs(slot: int):
        """Host-to-device copy of one step's inputs, on the copy stream."""
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(out_ready[slot])  # the step that last read this buffer is done
            dev_ins[slot].copy_(host_in, non_blocking=True)
            in_ready[slot].record(copy_stream)

    counter = [0]

    def e2e_step(_i: int):
        """Every step has its own copy in, call, copy out and host read of its result, but the
        steps overlap as in an engine that schedules asynchronously: the inputs of step i + 1
        cross PCIe on the copy stream while step i computes, and the host reads the result of
        step i - 1 (waits for its copy out) after it has enqueued step i."""
        i = counter[0]
        counter[0] += 1
        slot = i & 1
        stream.wait_event(in_ready[slot])
        host_outs[slot].copy_(e2e_call(i, *dev_views[slot]), non_blocking=True)
        out_ready[slot].record(stream)
        stage_inputs(slot ^ 1)
        if i > 0:
            out_ready[slot ^ 1].synchronize()  # the host consumes the previous step's result

    def e2e_drain():
        out_ready[(counter[0] - 1) & 1].synchronize()

    # -------- the headline workload, under clock sampling
    with ClockSampler(local_rank) as clocks:
        res = case.measure(args.steps, args.warmup, args.repeats, check=True)
        for i in range(3):
            e2e_serial_step(i)
        ms_e2e_serial = case.timed_eager(e2e_serial_step, args.steps)
        stage_inputs(0)
        for i in range(4):
            e2e_step(i)
        e2e_drain()
        ms_e2e = case.timed_eager(e2e_step, args.steps)  # (the barrier behind the K steps waits for the last result)
        torch.cuda.synchronize()
        ms_eager = case.timed_eager(case.step, args.steps)
        with_producer = None
        if args.with_producer and mode == "batch" and case.kv16 is None and not case.shared_prefix and world == 1:
            with_producer = case.measure_with_producer(args.steps, 3)  # (last: it rewrites the pools' newest tokens)

    total_bytes = torch.tensor([float(case.kv_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total_bytes)
    total_bytes = float(total_bytes.item())
    ms_step, ms_kernel = res["ms_step"], res["ms_kernel"]
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e * 1e-3) / 1e9
    achieved = case.kv_bytes / (ms_kernel * 1e-3) / 1e9  # one GPU's kernel, one GPU's peak
    correct_all = torch.tensor([1.0 if res.get("correct") in (True, None) else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(correct_all, op=dist.ReduceOp.MIN)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = case.batch if mode != "kv-range" else 1
        repeats = 3 if case.kv_bytes < 5e8 else 1
        gbs, secs, nbytes = cpu_reference_run(w, rows, repeats)
        cpu_baseline = {
            "value": round(gbs, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{rows} of {case.batch} sequences, best of {repeats}, {secs * 1e3:.0f} ms per pass",
        }

    line = None
    if rank == 0:
        kernel_name = case.kernel_name(res["path"])
        short_kernel = kernel_name.split("<")[0] if res["path"] in KERNEL_NAMES else kernel_name
        line = {
            "metric": "decode_attn_kv_read_gbs", "value": round(value, 2), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "repeats": args.repeats,
            "ms_per_step": round(ms_step, 6), "us_per_layer_step": round(ms_step * 1e3, 3),
            "runs_us_per_layer_step": res["runs_us"],
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": ("fp8_e4m3 KV, bf16 q, fp32 accumulate" if not kv16
                      else f"{args.kv_dtype} KV and q, fp32 accumulate"), "data": "synthetic",
            "correct": bool(correct_all.item() > 0.5), "max_abs_error": res.get("max_abs_error"),
            "checked": res.get("checked"),
            "config": {
                "workload": args.workload, "batch_per_gpu": case.batch, "q_heads": case.hq, "kv_heads": case.hkv,
                "head_dim": case.d, "page_size": 16, "split_size": split, "max_seq_len": w.max_seq_len,
                "path": cabi.PATH_NAMES.get(res["path"], "?"), "flags": case.flags,
                "plan": ("computed once per model step (pfd_plan_decode), outside the timed layer-steps"
                         if case.plan is not None else "none"),
                "metadata": ("block_table and seq_lens are not rewritten between the timed layer-steps "
                             "(PFD_FLAG_EARLY_METADATA)") if case.flags & cabi.PFD_FLAG_EARLY_METADATA else "no promise",
                "kv_bytes_per_step_per_gpu": case.kv_bytes,
                **({"shared_prefix_tokens": w.prefix_len,
                    "unique_kv_bytes_per_step": int(w.prefix_len + (w.seq_lens - w.prefix_len).sum().item()) * case.hkv * case.d * 2,
                    "prefix_pass": "dense tcgen05 (TMEM accumulators), 128 rows x 256 tokens per CTA",
                    "groups": ("found on the device from the block table and the lengths (prefix lengths discovered), "
                               "grouped entry point") if case.groups is not None else "one group given by the caller"}
                   if case.shared_prefix else {}),
                "parallelism": (("kv-range split; packed partials stored to every rank by the decode kernels (peer stores of tagged words), merged on every rank"
                                 if args.exchange == "peer" else
                                 "kv-range split, packed partials exchanged (all-gather), merged on every rank") if mode == "kv-range" else
                                ("one batch sharded by sequence (token-balanced), no collective" if mode == "strong"
                                 else "the same batch on every GPU, no collective")) if world > 1 else "single GPU",
                "l2": f"{pools} KV pools of {case.pool_bytes / 1e6:.0f} MB rotated ({pools * case.pool_bytes / 1e6:.0f} MB > L2): every step reads cold KV",
                **({"host_cores_per_rank": len(cores)} if cores else {}),
            },
            "pct_of_hbm_peak": round(100 * value / (peak * world), 2),
            "roofline": {
                "bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": None if mode != "batch" else ncu_traffic(args.workload, short_kernel),
                "kernel": kernel_name, "us_per_launch": round(ms_kernel * 1e3, 3), "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": case.kv_bytes,
            },
            "isolated": {"us_per_layer_step": round(res["ms_isolated"] * 1e3, 3),
                         "what": "an unrelated ordinary kernel between steps (its own time subtracted): no overlap of a "
                                 "step's prologue with the previous step's tail"},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "us_per_layer_step": round(ms_e2e * 1e3, 3),
                    "pipeline": "two buffers, asynchronous scheduling: step i + 1's inputs are copied in on a second stream "
                                "while step i computes, and the host reads step i - 1's result after enqueueing step i; "
                                "every step has its own copy in, call, copy out and host read",
                    "serial_us_per_layer_step": round(ms_e2e_serial * 1e3, 3)},
            **({"with_producer": with_producer} if with_producer is not None else {}),
            "gpu_launches": int(res["launches_per_step"] * args.steps),
            "timing": "K steps replayed from CUDA graphs, CUDA events around the replays, median of `repeats` runs; eager launch loop beside it",
            "us_per_layer_step_eager_launch": round(ms_eager * 1e3, 3),
            "clocks": clocks.summary(),
        }
        if "ms_exchange" in res:
            line["exchange_and_merge_us"] = round(res["ms_exchange"] * 1e3, 3)
        if "ms_step_allgather" in res:
            line["exchange_status"] = res["exchange_status"]
            line["allgather_form"] = {"us_per_layer_step": round(res["ms_step_allgather"] * 1e3, 3),
                                      "exchange_and_merge_us": round(res["ms_exchange_allgather"] * 1e3, 3)}
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
    case.release()
    del case

    # -------- the other configurations (N = 1) / the two sharded forms (N > 1)
    extra_steps = max(40, min(args.steps, 200))
    if not args.no_per_config and not kv16 and args.workload == DEFAULT_WORKLOAD and mode == "batch":
        if world == 1:
            per_config = {}
            for name in ALL_WORKLOADS:
                if name == args.workload:
                    continue
                c = Case(args, name, dev, 0, 1, "kv-range" if name == "llama3-8b-long-b4" else "batch")
                r = c.measure(extra_steps, 5, 3, check=True, isolated=name != "llama3-8b-long-b4")
                per_config[name] = short_report(c, r, peak, c.kv_bytes, 1)
                c.release()
                del c
            line["per_config"] = per_config
        else:
            sharded = {}
            for name, smode in (("qwen2.5-7b-b256", "strong"), ("llama3-8b-long-b4", "kv-range")):
                c = Case(args, name, dev, rank, world, smode)
                r = c.measure(extra_steps, 5, 3, check=smode == "strong", isolated=False)
                tb = torch.tensor([float(c.kv_bytes)], device=dev, dtype=torch.float64)
                dist.all_reduce(tb)
                ok = torch.tensor([1.0 if r.get("correct") in (True, None) else 0.0], device=dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                rep = short_report(c, r, peak, float(tb.item()), world) if rank == 0 else None
                c.release()
                del c
                # the one-GPU figure of the same workload, measured in this run on rank 0 alone
                one = None
                if rank == 0:
                    c1 = Case(args, name, dev, 0, 1, "kv-range" if smode == "kv-range" else "batch")
                    r1 = c1.measure(extra_steps, 5, 1, check=False, isolated=False)
                    one = r1["ms_step"] * 1e3
                    c1.release()
                    del c1
                dist.barrier()
                if rank == 0:
                    if smode == "strong":
                        rep["correct"] = bool(ok.item() > 0.5)
                    rep["one_gpu_us_per_layer_step"] = round(one, 3)
                    rep["speedup_over_one_gpu"] = round(one / rep["us_per_layer_step"], 3)
                    rep["sharding"] = ("sequences split over the ranks by tokens (longest first), no communication"
                                       if smode == "strong" else
                                       "KV range of every sequence split over the ranks; packed (o, m, l) rows exchanged, merged on every rank")
                    sharded[name] = rep
            if rank == 0:
                line["sharded"] = sharded
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
