#!/usr/bin/env python3
"""Benchmark of the paged FP8-KV GQA decode-attention step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One *step* is one decode-attention layer-step over one synthetic batch (partial kernel +
LSE merge kernel).  Metric: KV bytes read per second (``sum_b ctx_b * Hkv * D * 2`` bytes per
step), with microseconds per layer-step beside it.  One JSON line is printed by rank 0.

* ``value``        device-resident operands, CUDA events around K back-to-back steps; successive
                   steps use different KV pools so that every step reads from HBM, not L2.
* ``roofline``     the split-KV partial kernel alone (same pools, merge skipped), against the
                   measured HBM copy peak.
* ``e2e``          the call a serving hook makes (``l20_paged_split_kv_attention_fp8``) with the
                   step's query / block table / sequence lengths copied from pinned host memory
                   and the output copied back, every step.  The KV cache is the resident state of
                   the serving engine and stays on the device.
* ``cpu_baseline`` the CPU oracle (torch restatement of the reference's own torch path) timed
                   on this host's cores on the same batch.
* ``--impl reference`` times only that CPU path and prints its own line.

With N > 1 every rank runs the same geometry on its own sequences (no data-path collective;
``--strong`` shards ONE batch by sequence instead); ``--workload llama3-8b-long-b4`` splits each
sequence's KV range over the ranks and merges the partials after one NCCL all-gather
(``--graph-collective`` replays that step, collective included, from a CUDA graph).
``--kv-dtype bf16|fp16`` times the non-quantised sibling operator on the same geometries;
``--flags`` are the ``PFD_FLAG_*`` bits of the timed calls (default: early metadata reads; add 8
for the fixed-split grid).
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (the bench's own seed-0 workloads, full size).
NCU_TRAFFIC_BYTES_PER_LAUNCH = {
    ("qwen2.5-coder-3b-b64", 3): 80_427_520 + 3_423_488,   # chunk kernel (mean of two launches)
    ("qwen2.5-7b-b256", 3): 224_103_040 + 7_126_144,       # chunk kernel
    ("qwen2.5-coder-3b-b64", 2): 80_438_016 + 3_118_592,   # fixed-split TMA kernel (--flags 40)
}

DEFAULT_WORKLOAD = "qwen2.5-coder-3b-b64"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=600)
    p.add_argument("--warmup", type=int, default=30)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default=DEFAULT_WORKLOAD)
    p.add_argument("--split-size", type=int, default=0, help="0 = choose from the geometry")
    p.add_argument("--pools", type=int, default=0, help="distinct KV pools rotated through (0 = enough to exceed L2 x3)")
    p.add_argument("--kv-dtype", choices=["fp8", "bf16", "fp16"], default="fp8",
                   help="fp8: the e4m3 path (headline); bf16 / fp16: the non-quantised sibling operator, "
                        "caches and query in that type (single GPU, batch-sharded or weak scaling only)")
    p.add_argument("--graph-collective", action="store_true",
                   help="KV-range mode on several GPUs: replay the step, all-gather included, from a CUDA graph "
                        "instead of launching every step eagerly")
    p.add_argument("--flags", type=int, default=32,
                   help="PFD_FLAG_* bits of the timed calls; default PFD_FLAG_EARLY_METADATA: the block table "
                        "and sequence lengths do not change between the timed layer-steps")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-shared-prefix", action="store_true",
                   help="shared-prefix-b64 only: use the ordinary decode path instead of the dense tcgen05 prefix pass")
    p.add_argument("--single-launch", action="store_true",
                   help="with the plan: combine the pieces of cut sequences inside the balanced kernel (PFD_FLAG_SINGLE_LAUNCH)")
    p.add_argument("--no-plan", action="store_true",
                   help="do not plan the step: every call derives its work split itself and a merge kernel follows")
    p.add_argument("--strong", action="store_true",
                   help="N > 1: shard ONE batch by sequence over the ranks (token-balanced) instead of one batch per rank")
    return p.parse_args()


def measured_peak() -> tuple[float, str]:
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(peaks["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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


def main() -> int:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference_arm(args, rank)
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the operator has no CPU path")
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    import torch.distributed as dist

    from single_gpu_inference_lab_b200 import cabi, l20_paged_split_kv, sharding
    from single_gpu_inference_lab_b200.workloads import make_inputs

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cabi.load()

    kv16 = {"fp8": None, "bf16": torch.bfloat16, "fp16": torch.float16}[args.kv_dtype]
    gen_kw = {} if kv16 is None else {"kv_dtype": kv16, "query_dtype": kv16}
    kv_range_mode = args.workload == "llama3-8b-long-b4" and kv16 is None
    # -------- inputs: every rank builds its own batch directly on its GPU
    if kv_range_mode:
        full_len = 131072
        lo, hi = sharding.kv_range_bounds(full_len, rank, world)
        w = make_inputs(args.workload, seed=rank, device=dev, shrink=(hi - lo) / full_len)
        scaling = "strong"
    elif args.strong and world > 1:
        full = make_inputs(args.workload, seed=0, device=dev, **gen_kw)  # same batch on every rank
        w, _rows = sharding.shard_sequences(full, rank, world)
        del full
        torch.cuda.empty_cache()
        scaling = "strong"
    else:
        w = make_inputs(args.workload, seed=rank, device=dev, **gen_kw)
        scaling = "weak"
    q = w.query
    batch, hq, d = q.shape
    hkv = w.key_cache.shape[2]
    kv_bytes = w.kv_bytes
    split = args.split_size or l20_paged_split_kv.choose_split_size(
        batch, hkv, w.max_seq_len, seq_lens=w.seq_lens.tolist())
    pool_bytes = 2 * w.key_cache.numel()
    pools = args.pools or max(2, -(-3 * L2_BYTES // pool_bytes) + 1)
    pools = min(pools, max(2, int(40e9 // pool_bytes)))
    kcs = [w.key_cache] + [w.key_cache.clone() for _ in range(pools - 1)]
    vcs = [w.value_cache] + [w.value_cache.clone() for _ in range(pools - 1)]
    shared_prefix = w.prefix_len > 0 and not args.no_shared_prefix and d == 128 and kv16 is None
    if shared_prefix and not args.split_size:
        split = 512
    ws = l20_paged_split_kv.allocate_l20_paged_split_kv_workspace(q, w.max_seq_len, split_size=split)
    if shared_prefix:
        from single_gpu_inference_lab_b200 import l20_shared_prefix_decode_dispatch as spd

        ws = spd.allocate_shared_prefix_workspace(q, w.max_seq_len, w.prefix_len, suffix_split_size=split)
    out = ws[3]
    # The plan of the model step: block table and lengths are the same for every layer, so the
    # work split is computed once, outside the timed layer-steps, as an engine does per step.
    plan = None
    if not args.no_plan and not shared_prefix and d == 128 and hq // hkv <= 8 and not (args.flags & (1 | 2 | 8)):
        plan = cabi.plan_decode(q, w.key_cache, w.value_cache, w.block_table, w.seq_lens, max_seq_len=w.max_seq_len,
                                split_size=split, workspace=ws)
        torch.cuda.synchronize()
        if args.single_launch:
            args.flags |= cabi.PFD_FLAG_SINGLE_LAUNCH
    packed = torch.empty(batch, hq, d + 2, device=dev) if kv_range_mode else None
    gathered = torch.empty(world, batch, hq, d + 2, device=dev) if kv_range_mode else None

    def step(i: int, flags: int = args.flags):
        if kv16 is not None:
            cabi.paged_decode_kv16_split_out(
                q, kcs[i % pools], vcs[i % pools], w.block_table, w.seq_lens, max_seq_len=w.max_seq_len,
                split_size=split, output=out, workspace=ws, flags=flags, plan=plan)
            return
        if shared_prefix:
            cabi.shared_prefix_decode_fp8_e4m3(
                q, kcs[i % pools], vcs[i % pools], w.block_table, w.seq_lens, prefix_len=w.prefix_len,
                k_scale=w.k_scale, v_scale=w.v_scale, max_seq_len=w.max_seq_len, split_size=split, output=out,
                workspace=ws)
            return
        cabi.paged_decode_fp8_e4m3_split_out(
            q, kcs[i % pools], vcs[i % pools], w.block_table, w.seq_lens, k_scale=w.k_scale, v_scale=w.v_scale,
            max_seq_len=w.max_seq_len, split_size=split, output=None if kv_range_mode else out,
            packed_output=packed, workspace=ws, flags=flags, plan=plan,
        )
        if kv_range_mode and not (flags & cabi.PFD_FLAG_PARTIAL_ONLY):
            if world > 1:
                dist.all_gather_into_tensor(gathered.view(-1, hq, d + 2), packed)
            else:
                gathered[0].copy_(packed)
            cabi.merge_packed(gathered, out)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps: int) -> float:
        """ms per step, CUDA events on the launching stream, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def timed_graph(fn, steps: int) -> float:
        """Same, with the K steps replayed from CUDA graphs (a graph of `chunk` consecutive
        steps replayed, plus one for the remainder) so that host launch overhead does not
        pace the device: exactly `steps` steps run inside the timed region."""
        if kv_range_mode and world > 1 and not args.graph_collective:
            return timed(fn, steps)  # the collective is launched eagerly
        chunk = min(steps, max(pools, (64 // pools) * pools))
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
        torch.cuda.synchronize()
        graphs[0].replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graphs[0].replay()
        if graphs[1] is not None:
            graphs[1].replay()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # -------- e2e operands: the per-step inputs (q, block table, lengths) packed into ONE pinned host
    # buffer and copied with one transfer into a device buffer the operands are views of
    def aligned(n: int) -> int:
        return (n + 255) // 256 * 256

    q_bytes, t_bytes, l_bytes = q.numel() * q.element_size(), w.block_table.numel() * 4, w.seq_lens.numel() * 4
    off_t, off_l = aligned(q_bytes), aligned(q_bytes) + aligned(t_bytes)
    host_in = torch.empty(off_l + aligned(l_bytes), dtype=torch.uint8).pin_memory()
    dev_in = torch.empty_like(host_in, device=dev)

    def views(buf):
        return (buf[:q_bytes].view(q.dtype).view(q.shape),
                buf[off_t:off_t + t_bytes].view(torch.int32).view(w.block_table.shape),
                buf[off_l:off_l + l_bytes].view(torch.int32).view(w.seq_lens.shape))

    hq_v, ht_v, hl_v = views(host_in)
    hq_v.copy_(q.cpu()); ht_v.copy_(w.block_table.cpu()); hl_v.copy_(w.seq_lens.cpu())
    dq, dtable, dlens = views(dev_in)
    host_out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    h2d = q_bytes + t_bytes + l_bytes
    d2h = host_out.numel() * host_out.element_size()
    stream = torch.cuda.current_stream()

    def e2e_step(i: int):
        dev_in.copy_(host_in, non_blocking=True)
        if kv_range_mode:
            local = w.__class__(**{**w.__dict__, "query": dq, "block_table": dtable, "seq_lens": dlens,
                                   "key_cache": kcs[i % pools], "value_cache": vcs[i % pools]})
            if world > 1:
                res = sharding.kv_range_decode(local, split_size=split, gather_buffer=gathered, workspace=ws, packed_buffer=packed)
            else:
                res = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
                    dq, kcs[i % pools], vcs[i % pools], dtable, dlens, k_scale=w.k_scale, v_scale=w.v_scale,
                    max_seq_len=w.max_seq_len, split_size=split, workspace=ws)
        elif kv16 is not None:
            res = l20_paged_split_kv.l20_paged_split_kv_attention(
                dq, kcs[i % pools], vcs[i % pools], dtable, dlens, split_size=split, workspace=ws,
                max_seq_len=w.max_seq_len)
        elif shared_prefix:
            res = spd.shared_paged_prefix_paged_suffix_gqa_decode_attention_fp8(
                dq, kcs[i % pools], vcs[i % pools], dtable, dlens, w.prefix_len, k_scale=w.k_scale, v_scale=w.v_scale,
                max_seq_len=w.max_seq_len, suffix_split_size=split, workspace=ws)
        else:
            res = l20_paged_split_kv.l20_paged_split_kv_attention_fp8(
                dq, kcs[i % pools], vcs[i % pools], dtable, dlens, k_scale=w.k_scale, v_scale=w.v_scale,
                max_seq_len=w.max_seq_len, split_size=split, workspace=ws)
        host_out.copy_(res, non_blocking=True)
        stream.synchronize()  # the host consumes the step's result

    # -------- warm-up, then the timed loops under clock sampling
    for i in range(max(args.warmup, 3)):
        step(i)
    for i in range(3):
        e2e_step(i)
    with ClockSampler(local_rank) as clocks:
        launches_before = cabi.launch_count()
        step(0)
        per_step = cabi.launch_count() - launches_before  # kernels of this library per step
        ms_step = timed_graph(step, args.steps)
        launches = per_step * args.steps                  # replayed from graphs inside the timed region
        path = cabi.last_path()
        fused = ((not kv_range_mode) and per_step == 1) or shared_prefix  # no single dominant kernel to time apart
        kernel_name = {1: "paged_decode_fp8_partial_ldg_kernel", 2: "paged_decode_fp8_partial_tma_kernel",
                       3: "paged_decode_fp8_chunk_kernel", 4: "paged_decode_fp8_chunk_kernel<KV16>",
                       5: "paged_decode_fp8_chunk_kernel", 6: "paged_decode_fp8_chunk_kernel<KV16>"}.get(path, "?")
        if shared_prefix:
            kernel_name = "shared_prefix_dense_kernel + paged_decode_fp8_partial_tma_kernel + paged_decode_merge_kernel"
        ms_kernel = timed_graph(step if fused else (lambda i: step(i, args.flags | cabi.PFD_FLAG_PARTIAL_ONLY)), args.steps)
        ms_e2e = timed(e2e_step, args.steps)
        ms_eager = timed(step, args.steps)

    # -------- aggregate over ranks
    total_bytes = torch.tensor([float(kv_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(total_bytes)
    total_bytes = float(total_bytes.item())
    peak, peak_kind = measured_peak()
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e * 1e-3) / 1e9
    achieved = kv_bytes / (ms_kernel * 1e-3) / 1e9  # one GPU's kernel, one GPU's peak

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = batch if not kv_range_mode else 1
        repeats = 3 if kv_bytes < 5e8 else 1
        gbs, secs, nbytes = cpu_reference_run(w, rows, repeats)
        cpu_baseline = {
            "value": round(gbs, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{rows} of {batch} sequences, best of {repeats}, {secs * 1e3:.0f} ms per pass",
        }

    if rank == 0:
        line = {
            "metric": "decode_attn_kv_read_gbs", "value": round(value, 2), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_step, 6), "us_per_layer_step": round(ms_step * 1e3, 3),
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": ("fp8_e4m3 KV, bf16 q, fp32 accumulate" if kv16 is None
                      else f"{args.kv_dtype} KV and q, fp32 accumulate"), "data": "synthetic",
            "config": {
                "workload": args.workload, "batch_per_gpu": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                "page_size": 16, "split_size": split, "max_seq_len": w.max_seq_len, "path": cabi.PATH_NAMES.get(path, "?"),
                "flags": args.flags,
                "metadata": ("block_table and seq_lens are not rewritten between the timed layer-steps "
                             "(PFD_FLAG_EARLY_METADATA)") if args.flags & cabi.PFD_FLAG_EARLY_METADATA else "no promise",
                "kv_bytes_per_step_per_gpu": kv_bytes,
                **({"shared_prefix_tokens": w.prefix_len,
                    "unique_kv_bytes_per_step": int(w.prefix_len + (w.seq_lens - w.prefix_len).sum().item()) * hkv * d * 2,
                    "prefix_pass": "dense tcgen05 (TMEM accumulators), 128 rows x 256 tokens per CTA"} if shared_prefix else {}),
                "parallelism": ("kv-range split + all-gather" if kv_range_mode else
                                ("one batch sharded by sequence (token-balanced), no collective" if args.strong
                                 else "one batch per GPU, no collective")) if world > 1 else "single GPU",
                "l2": f"{pools} KV pools of {pool_bytes / 1e6:.0f} MB rotated ({pools * pool_bytes / 1e6:.0f} MB > L2): every step reads cold KV",
            },
            "pct_of_hbm_peak": round(100 * value / (peak * world), 2),
            "roofline": {
                "bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": None if (args.strong or kv_range_mode) else NCU_TRAFFIC_BYTES_PER_LAUNCH.get((args.workload, path)),
                "kernel": kernel_name, "us_per_launch": round(ms_kernel * 1e3, 3), "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": kv_bytes,
            },
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "us_per_layer_step": round(ms_e2e * 1e3, 3)},
            "gpu_launches": int(launches),
            "timing": "K steps replayed from CUDA graphs, CUDA events around the replays; eager launch loop beside it",
            "us_per_layer_step_eager_launch": round(ms_eager * 1e3, 3),
            "clocks": clocks.summary(),
        }
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
