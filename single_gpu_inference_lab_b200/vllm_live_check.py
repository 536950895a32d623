#!/usr/bin/env python3
"""Run the hook inside a live vLLM engine and compare it with the stock FlashInfer decode.

What it does, on a B200 with vLLM installed and no model files at hand:

1. builds an overlay of the installed ``vllm`` package in a work directory (symlinks, except
   ``v1/attention/backends/flashinfer.py`` and ``v1/attention/ops/``, which are copies) and
   runs ``install_l20_fp8_paged_decode.py`` on it -- the installed package is not touched;
2. writes the config of a small Qwen2-shaped model (4 layers, 16 query / 2 KV heads of 128) and
   lets vLLM create it with ``load_format="dummy"``; the weights are then re-drawn at a
   realistic scale from a fixed seed, so that attention matters to the logits;
3. generates greedily from 8 random prompts of 300-1500 tokens, twice, each in a fresh
   process: stock, and with the hook's switches set (``--kv-cache-dtype fp8``: the FP8
   operator; ``auto``: the fp16 / bf16 sibling);
4. prints one JSON line: hook hits counted from the trace file, how many generated tokens agree
   step by step, and the largest difference of the top-3 log-probabilities over the agreeing
   steps (sequences are compared up to their first different token).

With ``--ab`` it times decoding instead (the miniature of the reference's serving A/B campaign,
scripts/run_vllm_l20_fp8_paged_campaign.sh): a model of ``--layers`` layers of the same shape,
``--batch`` prompts of ``--prompt-len`` tokens, ``--new-tokens`` greedy tokens; per engine the
time of a 1-token generation is subtracted from that of a (1 + new-tokens)-token generation
(best of two each), which leaves the decode steps; eager mode, so launch overheads of the whole
model are in both numbers.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

PKG = Path(__file__).resolve().parent
COPIED_PATHS = ("v1/attention/backends/flashinfer.py", "v1/attention/ops")

CHILD = r'''
import json, math, os, random, time
import torch
from vllm import LLM, SamplingParams

llm = LLM(model=os.environ["LIVE_MODEL"], load_format="dummy", skip_tokenizer_init=True,
          enforce_eager=os.environ.get("LIVE_GRAPHS", "0") != "1",
          kv_cache_dtype=os.environ["LIVE_KV"], block_size=16, dtype="bfloat16",
          max_model_len=int(os.environ.get("LIVE_MAX_LEN", "4096")), max_num_seqs=int(os.environ.get("LIVE_BATCH", "64")),
          gpu_memory_utilization=float(os.environ.get("LIVE_MEM", "0.3")), seed=0,
          enable_prefix_caching=os.environ.get("LIVE_SHARED_PREFIX", "0") == "1",
          **({"compilation_config": {"pass_config": {"fuse_rope_kvcache": True}, "splitting_ops": []}}  # (the pass wants an unsplit graph)
             if os.environ.get("LIVE_ROPE_FUSION", "0") == "1" else {}),
          attention_config={"backend": "FLASHINFER",
                            **({} if os.environ.get("LIVE_TRTLLM_AUTO", "0") == "1" else {"use_trtllm_attention": False})})


def reinit(model):
    g = torch.Generator(device="cuda").manual_seed(1234)
    for name, p in sorted(model.named_parameters()):
        if p.dim() == 1:
            p.data.fill_(0.0 if name.endswith("bias") else 1.0)
        else:
            p.data.copy_(torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32).mul_(0.02))
    return True


AB = int(os.environ.get("LIVE_AB", "0"))
if AB:
    batch, plen, new = (int(os.environ[k]) for k in ("LIVE_BATCH", "LIVE_PROMPT_LEN", "LIVE_NEW_TOKENS"))
    rng = random.Random(0)
    if os.environ.get("LIVE_LOGUNIFORM", "0") == "1":  # lengths log-uniform in [16, plen]
        lens = [max(16, int(round(math.exp(rng.uniform(math.log(16), math.log(plen)))))) for _ in range(batch)]
    else:
        lens = [plen] * batch
    prompts = [{"prompt_token_ids": [rng.randrange(10, 31000) for _ in range(n)]} for n in lens]
    def timed(max_tokens):
        best = 1e9
        for _ in range(2):
            t0 = time.time()
            llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_tokens, detokenize=False, ignore_eos=True),
                         use_tqdm=False)
            best = min(best, time.time() - t0)
        return best
    timed(2)  # warm-up of every code path
    t1, tn = timed(1), timed(1 + new)
    print("LIVE_RESULT " + json.dumps({"prefill_seconds": t1, "total_seconds": tn,
                                       "ms_per_decode_step": (tn - t1) / new * 1e3}))
    raise SystemExit(0)

llm.apply_model(reinit)
rng = random.Random(0)
if os.environ.get("LIVE_SHARED_PREFIX", "0") == "1":
    # 16 requests behind one 4200-token prefix: a first request computes (and caches) the prefix's
    # blocks, the others then start from the same physical blocks -- a shared-prefix decode batch
    common = [rng.randrange(10, 31000) for _ in range(4200)]
    llm.generate([{"prompt_token_ids": common}], SamplingParams(temperature=0.0, max_tokens=1, detokenize=False), use_tqdm=False)
    prompts = [{"prompt_token_ids": common + [rng.randrange(10, 31000) for _ in range(rng.randrange(20, 200))]} for _ in range(16)]
else:
    prompts = [{"prompt_token_ids": [rng.randrange(10, 31000) for _ in range(rng.randrange(300, 1500))]} for _ in range(8)]
params = SamplingParams(temperature=0.0, max_tokens=12, logprobs=3, detokenize=False, ignore_eos=True)
t0 = time.time()
outs = llm.generate(prompts, params)
seconds = time.time() - t0
result = []
for o in outs:
    c = o.outputs[0]
    result.append([
        {"token": int(tok), "top": sorted(((int(k), float(v.logprob)) for k, v in lp.items()), key=lambda x: -x[1])[:3]}
        for tok, lp in zip(c.token_ids, c.logprobs)
    ])
print("LIVE_RESULT " + json.dumps({"seconds": seconds, "outputs": result}))
'''


def overlay(real: Path, dst: Path, copy_rel) -> None:
    """``dst`` mirrors ``real`` with symlinks; the entries ``copy_rel`` (and the directories
    that lead to them) are real copies."""
    copy_rel = [Path(p) for p in copy_rel]

    def build(rdir: Path, ddir: Path, rel: Path) -> None:
        ddir.mkdir(parents=True, exist_ok=True)
        for entry in rdir.iterdir():
            erel, target = rel / entry.name, ddir / entry.name
            if any(c == erel for c in copy_rel):
                if entry.is_dir():
                    shutil.copytree(entry, target, dirs_exist_ok=True)
                else:
                    shutil.copy2(entry, target)
            elif entry.is_dir() and any(erel in c.parents for c in copy_rel):
                build(entry, target, erel)
            elif not target.exists():
                target.symlink_to(entry)

    build(real, dst, Path("."))


def write_model_config(path: Path, layers: int = 4, q_heads: int = 16, kv_heads: int = 2,
                       intermediate: int = 4096) -> None:
    path.mkdir(parents=True, exist_ok=True)
    config = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 128 * q_heads,
        "num_attention_heads": q_heads, "num_key_value_heads": kv_heads, "num_hidden_layers": layers,
        "intermediate_size": intermediate,
        "vocab_size": 32000, "max_position_embeddings": 32768, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 1,
        "eos_token_id": 2, "use_sliding_window": False,
    }
    (path / "config.json").write_text(json.dumps(config))


def run_engine(work: Path, kv: str, extra_env: dict, log: Path) -> dict:
    env = dict(os.environ)
    env.update(extra_env)
    env["PYTHONPATH"] = str(work / "vllm_src") + os.pathsep + env.get("PYTHONPATH", "")
    env["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
    env["LIVE_MODEL"] = str(work / "model")
    env["LIVE_KV"] = kv
    proc = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=1200)
    log.write_text(proc.stdout[-20000:] + "\n==== stderr\n" + proc.stderr[-20000:])
    for line in proc.stdout.splitlines():
        if line.startswith("LIVE_RESULT "):
            return json.loads(line[len("LIVE_RESULT "):])
    raise RuntimeError(f"the engine run failed (exit code {proc.returncode}); see {log}")


def shared_prefix_summary(trace: Path) -> dict:
    """Counts of the shared-prefix trace: candidate records (one per model step), how many found a
    group, the group sizes seen, and layer calls of the grouped operator."""
    records = [json.loads(line) for line in trace.read_text().splitlines()] if trace.exists() else []
    candidates = [r for r in records if r["event"] == "shared_prefix_decode_candidate"]
    sizes = sorted({tuple(r.get("group_sizes") or ()) for r in candidates if r.get("eligible")})
    return {"shared_prefix_steps": len(candidates), "shared_prefix_steps_with_groups": sum(1 for r in candidates if r.get("eligible")),
            "shared_prefix_group_sizes": [list(s) for s in sizes],
            "shared_prefix_layer_calls": sum(1 for r in records if r["event"] == "l20_shared_prefix_paged_decode_run")}


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--kv-cache-dtype", choices=["fp8", "auto"], default="fp8")
    parser.add_argument("--workdir", help="where the overlay, the model config and the logs go (default: a new temporary directory)")
    parser.add_argument("--ab", action="store_true", help="time decode steps, stock against hooked")
    parser.add_argument("--layers", type=int, default=36)
    parser.add_argument("--batch", type=int, default=64)
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--new-tokens", type=int, default=32)
    parser.add_argument("--q-heads", type=int, default=16, help="with --ab: query heads of 128 (hidden size = 128 x this)")
    parser.add_argument("--kv-heads", type=int, default=2)
    parser.add_argument("--intermediate", type=int, default=4096)
    parser.add_argument("--stock-auto", action="store_true",
                        help="with --ab: a third engine with use_trtllm_attention left to vLLM's own choice")
    parser.add_argument("--log-uniform", action="store_true", help="with --ab: prompt lengths log-uniform in [16, prompt-len]")
    parser.add_argument("--rope-hook", action="store_true",
                        help="also install the producer hook (install_l20_rope_kv.py) and switch vLLM's "
                             "fuse_rope_kvcache pass on in the hooked engine: rotary embedding + KV append then run "
                             "through l20_rope_and_cache, decode through the decode hook; implies --cuda-graphs "
                             "(the pass belongs to vLLM's compilation)")
    parser.add_argument("--shared-prefix", action="store_true",
                        help="16 requests behind one cached 4200-token prefix (prefix caching on in both engines); the "
                             "hooked engine also gets VLLM_ENABLE_L20_SHARED_PREFIX_DECODE=1, so its decode steps find "
                             "the group on the device and run the grouped shared-prefix operator; eager mode")
    parser.add_argument("--cuda-graphs", action="store_true",
                        help="let vLLM compile and record CUDA graphs (both engines), and keep the hook on while "
                             "it records (VLLM_L20_PAGED_CUDAGRAPH=1); hook hits are then counted at recording time")
    args = parser.parse_args(argv)
    if args.rope_hook:
        args.cuda_graphs = True

    spec = importlib.util.find_spec("vllm")  # located, not imported
    if spec is None or not spec.submodule_search_locations:
        raise RuntimeError("vLLM is not installed")
    work = Path(args.workdir) if args.workdir else Path(tempfile.mkdtemp(prefix="l20-live-"))
    work.mkdir(parents=True, exist_ok=True)
    if (work / "vllm_src").exists():
        shutil.rmtree(work / "vllm_src")
    copied = COPIED_PATHS + (("config/compilation.py",) if args.rope_hook else ())
    overlay(Path(list(spec.submodule_search_locations)[0]), work / "vllm_src" / "vllm", copied)
    sys.path.insert(0, str(PKG.parent))
    from single_gpu_inference_lab_b200 import install_l20_fp8_paged_decode as installer

    installer.main(["--vllm-source-dir", str(work / "vllm_src")])
    if args.rope_hook:
        from single_gpu_inference_lab_b200 import install_l20_rope_kv as rope_installer

        rope_installer.main(["--vllm-source-dir", str(work / "vllm_src")])
    if args.ab:
        write_model_config(work / "model", args.layers, args.q_heads, args.kv_heads, args.intermediate)
    else:
        write_model_config(work / "model")

    kv = args.kv_cache_dtype
    if args.ab:
        shape = {"LIVE_AB": "1", "LIVE_BATCH": str(args.batch), "LIVE_PROMPT_LEN": str(args.prompt_len),
                 "LIVE_NEW_TOKENS": str(args.new_tokens), "LIVE_GRAPHS": "1" if args.cuda_graphs else "0",
                 "LIVE_LOGUNIFORM": "1" if args.log_uniform else "0", "LIVE_MEM": "0.5",
                 "LIVE_MAX_LEN": str(max(4096, args.prompt_len + args.new_tokens + 16))}
        on = ({"VLLM_ENABLE_L20_FP8_PAGED_DECODE": "1", "VLLM_L20_FP8_PAGED_FORCE": "1"} if kv == "fp8"
              else {"VLLM_ENABLE_L20_PAGED_DECODE": "1", "VLLM_L20_PAGED_FORCE": "1"})
        stock = run_engine(work, kv, shape, work / f"{kv}_ab_stock.log")
        if args.cuda_graphs:
            on["VLLM_L20_PAGED_CUDAGRAPH"] = "1"
        hooked = run_engine(work, kv, {**shape, **on}, work / f"{kv}_ab_hook.log")
        auto = None
        if args.stock_auto:  # what vLLM picks by itself on this GPU (may be the TRTLLM-gen decode, which the hook never sees)
            auto = run_engine(work, kv, {**shape, "LIVE_TRTLLM_AUTO": "1"}, work / f"{kv}_ab_stock_auto.log")
        print(json.dumps({
            **({"stock_auto_backend_ms_per_decode_step": round(auto["ms_per_decode_step"], 4)} if auto else {}),
            "kv_cache_dtype": kv, "layers": args.layers, "q_heads": args.q_heads, "kv_heads": args.kv_heads,
            "batch": args.batch, "prompt_len": args.prompt_len, "log_uniform_lengths": args.log_uniform,
            "new_tokens": args.new_tokens, "mode": "cuda graphs" if args.cuda_graphs else "eager",
            "stock_ms_per_decode_step": round(stock["ms_per_decode_step"], 4),
            "hook_ms_per_decode_step": round(hooked["ms_per_decode_step"], 4),
            "stock_prefill_s": round(stock["prefill_seconds"], 4), "hook_prefill_s": round(hooked["prefill_seconds"], 4),
        }))
        return 0
    trace = work / f"trace_{kv}.jsonl"
    trace.unlink(missing_ok=True)
    graphs = {"LIVE_GRAPHS": "1"} if args.cuda_graphs else {}
    prefix_trace = work / f"prefix_trace_{kv}.jsonl"
    prefix_trace.unlink(missing_ok=True)
    if args.shared_prefix:
        graphs.update(LIVE_SHARED_PREFIX="1", LIVE_MAX_LEN="8192", LIVE_MEM="0.4")
    stock = run_engine(work, kv, graphs, work / f"{kv}_stock.log")
    switches = (
        {"VLLM_ENABLE_L20_FP8_PAGED_DECODE": "1", "VLLM_L20_FP8_PAGED_FORCE": "1", "VLLM_L20_FP8_PAGED_TRACE": str(trace)}
        if kv == "fp8"
        else {"VLLM_ENABLE_L20_PAGED_DECODE": "1", "VLLM_L20_PAGED_FORCE": "1", "VLLM_L20_PAGED_TRACE": str(trace)}
    )
    if args.cuda_graphs:
        switches["VLLM_L20_PAGED_CUDAGRAPH"] = "1"
    rope_trace = work / f"rope_trace_{kv}.jsonl"
    rope_trace.unlink(missing_ok=True)
    if args.rope_hook:
        switches.update(LIVE_ROPE_FUSION="1", VLLM_L20_ROPE_KV_TRACE=str(rope_trace))
    if args.shared_prefix:
        switches.update(VLLM_ENABLE_L20_SHARED_PREFIX_DECODE="1", VLLM_L20_SHARED_PREFIX_DECODE_TRACE=str(prefix_trace))
    hooked = run_engine(work, kv, {**graphs, **switches}, work / f"{kv}_hook.log")

    hits = [json.loads(line) for line in trace.read_text().splitlines()] if trace.exists() else []
    compared = agree = 0
    worst = 0.0
    for a, b in zip(stock["outputs"], hooked["outputs"]):
        for sa, sb in zip(a, b):
            compared += 1
            if sa["token"] != sb["token"]:
                break
            agree += 1
            da, db = dict(sa["top"]), dict(sb["top"])
            worst = max([worst] + [abs(da[k] - db[k]) for k in da if k in db])
    print(json.dumps({
        "kv_cache_dtype": kv, "mode": "cuda graphs" if args.cuda_graphs else "eager", "hook_hits": len(hits),
        "hook_hits_beyond_warmup": sum(1 for h in hits if h["max_seq_len"] > 64),
        "generated_steps_compared": compared, "same_token": agree, "max_abs_logprob_diff": worst,
        **({"rope_hook_hits": sum(1 for _ in rope_trace.open()) if rope_trace.exists() else 0} if args.rope_hook else {}),
        **(shared_prefix_summary(prefix_trace) if args.shared_prefix else {}),
        "workdir": str(work),
    }))
    return 0 if hits and agree >= compared * 0.8 else 1


if __name__ == "__main__":
    raise SystemExit(main())
