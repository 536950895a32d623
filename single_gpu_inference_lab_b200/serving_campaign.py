#!/usr/bin/env python3
"""Serving A/B campaign for the FP8 paged-decode hook on B200.

Port of the reference's campaign (scripts/run_vllm_l20_fp8_paged_campaign.sh:29-101, analysed by
scripts/analyze_vllm_serving.py): the same engine twice, hook off and hook on, over a grid of
concurrencies and prompt lengths, several runs per cell; inter-token latency decides, and the
hook's trace file says how often it ran.  Two ways to run it:

``serve``  the reference's way, for a host that has model weights and a tokenizer: ``vllm serve``
           from an overlay of the installed package with the hook installed (the installed package
           is not touched), FlashInfer backend, FP8 KV cache, then ``vllm bench serve`` with the
           random dataset per (concurrency, input length, run); every report must show all
           prompts completed.  Eager mode as in the reference (``--enforce-eager``), or with
           ``--cuda-graphs`` vLLM's default graphs and the hook kept on while they are recorded
           (``VLLM_L20_PAGED_CUDAGRAPH=1``; the reference always steps aside under capture).

           ``--dummy-weights`` makes this mode runnable on a host without model files: a Qwen2-shaped
           model directory is written (``--layers``, ``--q-heads``, ``--kv-heads``, ``--intermediate``) with a
           synthetic word-level tokenizer whose decode / encode round trip is exact, and the server
           draws the weights (``--load-format dummy``).  Latencies are then those of the shape, the
           generated text means nothing.

``dummy``  for a host without weights (this build's GPU boxes have no network): the in-process
           engine of ``vllm_live_check.py --ab`` -- a Qwen2-shaped model with re-drawn random
           weights -- once per cell; batch = concurrency, all prompts of the given length, decode
           steps timed with the prefill subtracted.  No HTTP server, no request arrival process:
           it measures the decode step inside the engine, not queueing.

Both write ``<output-dir>/summary.json``: per cell and engine the median of the runs, plus the
hook-on / hook-off ratio; ``serve`` cells carry ITL / TPOT / TTFT percentiles, ``dummy`` cells
milliseconds per decode step.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import signal
import statistics
import subprocess
import sys
import time
import urllib.request
from pathlib import Path

PKG = Path(__file__).resolve().parent


def _ints(text: str) -> list[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def build_overlay(work: Path) -> Path:
    """A copy-on-write view of the installed vLLM with the decode hook installed; returns the
    directory to put on PYTHONPATH."""
    import importlib.util

    sys.path.insert(0, str(PKG.parent))
    from single_gpu_inference_lab_b200 import install_l20_fp8_paged_decode as installer
    from single_gpu_inference_lab_b200 import vllm_live_check as live

    spec = importlib.util.find_spec("vllm")
    if spec is None or not spec.submodule_search_locations:
        raise RuntimeError("vLLM is not installed")
    src = work / "vllm_src"
    if src.exists():
        shutil.rmtree(src)
    live.overlay(Path(list(spec.submodule_search_locations)[0]), src / "vllm", live.COPIED_PATHS)
    installer.main(["--vllm-source-dir", str(src)])
    return src


def write_dummy_model(path: Path, *, layers: int, q_heads: int, kv_heads: int, intermediate: int, vocab: int = 32000) -> Path:
    """A model directory a server can start from without any downloaded file: the config of a
    Qwen2-shaped model and a word-level tokenizer over ``vocab`` made-up words (ids 0-3: unk, bos,
    eos, pad; id i: the word "w<i>"), for which ``encode(decode(ids)) == ids`` -- the random
    dataset of ``vllm bench serve`` builds its prompts by decoding random ids."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from .vllm_live_check import write_model_config

    write_model_config(path, layers=layers, q_heads=q_heads, kv_heads=kv_heads, intermediate=intermediate)
    config = json.loads((path / "config.json").read_text())
    config["vocab_size"] = vocab
    (path / "config.json").write_text(json.dumps(config))
    specials = ["<unk>", "<bos>", "<eos>", "<pad>"]
    assert config["bos_token_id"] == 1 and config["eos_token_id"] == 2
    words = {s: i for i, s in enumerate(specials)}
    words.update({f"w{i}": i for i in range(len(specials), vocab)})
    tok = Tokenizer(models.WordLevel(words, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<bos>", eos_token="<eos>",
                            pad_token="<pad>").save_pretrained(str(path))
    return path


def wait_for_server(port: int, proc: subprocess.Popen, log: Path, seconds: int = 900) -> None:
    deadline = time.time() + seconds
    while time.time() < deadline:
        if proc.poll() is not None:
            raise RuntimeError(f"vllm serve exited with code {proc.returncode}; see {log}")
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                if r.status == 200:
                    return
        except OSError:
            time.sleep(5)
    raise RuntimeError(f"vllm serve did not come up within {seconds} s; see {log}")


def run_serve_arm(args, src: Path, out: Path, hook_on: bool) -> dict:
    """One engine of the reference's campaign: server up, the grid of bench runs, server down."""
    out.mkdir(parents=True, exist_ok=True)
    trace = out / "l20-fp8-paged-trace.jsonl"
    trace.unlink(missing_ok=True)
    flag = "1" if hook_on else "0"
    env = dict(os.environ, PYTHONPATH=str(src) + os.pathsep + os.environ.get("PYTHONPATH", ""),
               VLLM_ENABLE_L20_FP8_PAGED_DECODE=flag, VLLM_L20_FP8_PAGED_FORCE=flag,
               VLLM_L20_FP8_PAGED_TRACE=str(trace), VLLM_USE_FLASHINFER_SAMPLER="0")
    if args.cuda_graphs and hook_on:
        env["VLLM_L20_PAGED_CUDAGRAPH"] = "1"
    serve = [sys.executable, "-m", "vllm.entrypoints.cli.main", "serve", args.model, "--served-model-name", args.served_name,
             "--host", "127.0.0.1", "--port", str(args.port), "--attention-backend", "FLASHINFER",
             "--no-enable-prefix-caching", "--kv-cache-dtype", "fp8", "--calculate-kv-scales",
             "--max-num-seqs", str(max(args.concurrencies)), "--max-model-len", str(args.max_model_len)]
    if not args.cuda_graphs:
        serve.append("--enforce-eager")
    if args.dummy_weights:
        serve += ["--load-format", "dummy"]
    log = out / "server.log"
    with log.open("w") as sink:
        server = subprocess.Popen(serve, env=env, stdout=sink, stderr=subprocess.STDOUT, start_new_session=True)
    cells = {}
    try:
        wait_for_server(args.port, server, log)
        for conc in args.concurrencies:
            for inp in args.inputs:
                reports = []
                for run in range(1, args.runs + 1):
                    name = f"c{conc}-i{inp}-r{run}.json"
                    subprocess.run(
                        [sys.executable, "-m", "vllm.entrypoints.cli.main", "bench", "serve", "--backend", "vllm",
                         "--base-url", f"http://127.0.0.1:{args.port}", "--model", args.served_name, "--tokenizer", args.model,
                         "--dataset-name", "random", "--random-input-len", str(inp), "--random-output-len", str(args.output_tokens),
                         "--num-prompts", str(args.num_prompts), "--num-warmups", "3", "--max-concurrency", str(conc),
                         "--disable-tqdm", "--ignore-eos", "--temperature", "0", "--percentile-metrics", "ttft,tpot,itl,e2el",
                         "--metric-percentiles", "50,95,99", "--save-result", "--result-dir", str(out), "--result-filename", name],
                        env=env, check=True)
                    report = json.loads((out / name).read_text())
                    if report.get("completed") != args.num_prompts or report.get("failed") != 0:
                        raise RuntimeError(f"invalid benchmark report {out / name}: completed={report.get('completed')} "
                                           f"failed={report.get('failed')}")
                    reports.append(report)
                keys = ("median_itl_ms", "p95_itl_ms", "p99_itl_ms", "median_tpot_ms", "median_ttft_ms", "output_throughput")
                cells[f"c{conc}-i{inp}"] = {k: statistics.median(r[k] for r in reports if k in r) for k in keys
                                            if any(k in r for r in reports)}
    finally:
        try:
            os.killpg(server.pid, signal.SIGTERM)  # the process group this function started, nothing else
        except ProcessLookupError:
            pass
        server.wait(timeout=120)
    hits = sum(1 for _ in trace.open()) if trace.exists() else 0
    return {"cells": cells, "hook_hits": hits}


def run_dummy_cells(args, out: Path) -> dict:
    """The grid through the in-process engine of vllm_live_check --ab (stock and hooked per cell)."""
    cells = {}
    for conc in args.concurrencies:
        for inp in args.inputs:
            runs = []
            for run in range(1, args.runs + 1):
                cmd = [sys.executable, "-m", "single_gpu_inference_lab_b200.vllm_live_check", "--ab", "--batch", str(conc),
                       "--prompt-len", str(inp), "--new-tokens", str(args.output_tokens), "--layers", str(args.layers),
                       "--workdir", str(out / f"c{conc}-i{inp}-r{run}")]
                if args.cuda_graphs:
                    cmd.append("--cuda-graphs")
                proc = subprocess.run(cmd, capture_output=True, text=True, cwd=str(PKG.parent), timeout=3600)
                lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
                if proc.returncode != 0 or not lines:
                    raise RuntimeError(f"cell c{conc}-i{inp} run {run} failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-2000:]}")
                runs.append(json.loads(lines[-1]))
            stock = statistics.median(r["stock_ms_per_decode_step"] for r in runs)
            hook = statistics.median(r["hook_ms_per_decode_step"] for r in runs)
            cells[f"c{conc}-i{inp}"] = {"stock_ms_per_decode_step": stock, "hook_ms_per_decode_step": hook,
                                        "hook_over_stock": round(hook / stock, 4), "runs": len(runs)}
    return cells


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("mode", choices=["serve", "dummy"])
    parser.add_argument("--output-dir", required=True)
    parser.add_argument("--model", help="serve: model directory or name (weights and tokenizer)")
    parser.add_argument("--served-name", default="l20-campaign")
    parser.add_argument("--port", type=int, default=int(os.environ.get("PORT", "8000")))
    parser.add_argument("--inputs", type=_ints, default=_ints(os.environ.get("INPUTS", "4096")))
    parser.add_argument("--concurrencies", type=_ints, default=_ints(os.environ.get("CONCURRENCIES", "8")))
    parser.add_argument("--runs", type=int, default=int(os.environ.get("RUNS", "2")))
    parser.add_argument("--num-prompts", type=int, default=int(os.environ.get("NUM_PROMPTS", "32")))
    parser.add_argument("--output-tokens", type=int, default=int(os.environ.get("OUTPUT_TOKENS", "32")))
    parser.add_argument("--max-model-len", type=int, default=int(os.environ.get("MAX_MODEL_LEN", "8192")))
    parser.add_argument("--layers", type=int, default=36, help="dummy, serve --dummy-weights: layers of the random-weight model")
    parser.add_argument("--dummy-weights", action="store_true",
                        help="serve: write a Qwen2-shaped model directory with a synthetic tokenizer and let the server draw the weights")
    parser.add_argument("--q-heads", type=int, default=16)
    parser.add_argument("--kv-heads", type=int, default=2)
    parser.add_argument("--intermediate", type=int, default=4096)
    parser.add_argument("--cuda-graphs", action="store_true")
    args = parser.parse_args(argv)
    out = Path(args.output_dir).resolve()
    out.mkdir(parents=True, exist_ok=True)
    summary = {"mode": args.mode, "engine_mode": "cuda graphs" if args.cuda_graphs else "eager", "inputs": args.inputs,
               "concurrencies": args.concurrencies, "runs": args.runs, "output_tokens": args.output_tokens}
    if args.mode == "dummy":
        summary["cells"] = run_dummy_cells(args, out)
    else:
        if args.dummy_weights:
            args.model = str(write_dummy_model(out / "model", layers=args.layers, q_heads=args.q_heads,
                                               kv_heads=args.kv_heads, intermediate=args.intermediate))
            summary["weights"] = "dummy"
        if not args.model:
            parser.error("serve needs --model or --dummy-weights")
        src = build_overlay(out)
        off = run_serve_arm(args, src, out / "hook-off", hook_on=False)
        on = run_serve_arm(args, src, out / "hook-on", hook_on=True)
        cells = {}
        for cell, base in off["cells"].items():
            hooked = on["cells"].get(cell, {})
            cells[cell] = {"hook_off": base, "hook_on": hooked,
                           "median_itl_ratio": (round(hooked["median_itl_ms"] / base["median_itl_ms"], 4)
                                                if "median_itl_ms" in base and "median_itl_ms" in hooked else None)}
        summary.update(cells=cells, hook_hits=on["hook_hits"], hook_hits_with_hook_off=off["hook_hits"])
    (out / "summary.json").write_text(json.dumps(summary, indent=1, sort_keys=True))
    print(json.dumps(summary))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
