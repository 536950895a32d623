#!/usr/bin/env python3
"""Generate the golden vectors that pin ``oracle/paged_decode_oracle.py``.

Runs the reference project's OWN torch implementation of the path --
``reference()`` and ``quantize_fp8_e4m3()`` of
``scripts/smoke_cuda_paged_fp8_decode_op.py`` (:13-41), imported from a checkout of that
project (``--reference-root``, or the ``REFERENCE_ROOT`` environment variable) -- on seeded CPU inputs and
stores inputs digests + outputs in ``tests/golden/paged_decode_golden.pt``.

The reference function hard-codes ``device="cuda"`` in one ``torch.arange`` call (:29); the
only change made here is to strip that keyword while the function runs, so everything stays
on the CPU.  Nothing of this file or of the reference tree is needed at test time: the
fixtures travel, the reference does not.

    python tests/golden/make_golden.py --reference-root <checkout of single-gpu-inference-lab>
"""

from __future__ import annotations

import argparse
import os
import contextlib
import hashlib
import importlib
import importlib.util
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))

from single_gpu_inference_lab_b200.workloads import make_inputs  # noqa: E402

CASES = [
    # (case name, workload, batch override, shrink)
    ("cfg1-qwen0.5b-b8", "qwen2.5-0.5b-b8", None, 1.0),
    ("cfg2-coder3b-b4", "qwen2.5-coder-3b-b64", 4, 0.25),
    ("cfg3-qwen7b-b24", "qwen2.5-7b-b256", 24, 0.125),
    ("cfg4-llama8b-b2", "llama3-8b-long-b4", 2, 1.0 / 64),
    ("cfg5-prefix-b8", "shared-prefix-b64", 8, 0.125),
]


def digest(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.detach().cpu().contiguous()
        if t.dtype in (torch.float8_e4m3fn,):
            t = t.view(torch.uint8)
        elif t.dtype in (torch.bfloat16, torch.float16):
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


@contextlib.contextmanager
def arange_on_cpu():
    real = torch.arange

    def shim(*args, **kwargs):
        kwargs.pop("device", None)
        return real(*args, **kwargs)

    torch.arange = shim
    try:
        yield
    finally:
        torch.arange = real


KV16_CASES = [
    # (case name, workload, batch, shrink, dtype): the non-quantised sibling
    ("kv16-cfg2-coder3b-b4-bf16", "qwen2.5-coder-3b-b64", 4, 0.25, torch.bfloat16),
    ("kv16-cfg3-qwen7b-b24-bf16", "qwen2.5-7b-b256", 24, 0.125, torch.bfloat16),
    ("kv16-cfg4-llama8b-b2-fp16", "llama3-8b-long-b4", 2, 1.0 / 64, torch.float16),
]


def load_reference(root: Path, script: str = "scripts/smoke_cuda_paged_fp8_decode_op.py"):
    path = root / script
    spec = importlib.util.spec_from_file_location("ref_smoke", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def smoke_recipe(ref, batch: int, context: int, q_heads: int, kv_heads: int):
    """The reference smoke's own input recipe (:71-88) on the CPU: seed 29, uniform context,
    fp16 query, bf16 K/V quantised per tensor."""
    torch.manual_seed(29)
    pages_per_request = (context + 15) // 16
    pages = batch * pages_per_request
    table = torch.randperm(pages).to(torch.int32).reshape(batch, pages_per_request)
    seq_lens = torch.full((batch,), context, dtype=torch.int32)
    query = torch.randn(batch, q_heads, 128, dtype=torch.float16)
    key_bf16 = torch.randn(pages, 16, kv_heads, 128, dtype=torch.bfloat16)
    value_bf16 = torch.randn_like(key_bf16)
    key_cache, k_scale = ref.quantize_fp8_e4m3(key_bf16)
    value_cache, v_scale = ref.quantize_fp8_e4m3(value_bf16)
    return query, key_cache, value_cache, table, seq_lens, k_scale, v_scale


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference-root", default=os.environ.get("REFERENCE_ROOT"), required="REFERENCE_ROOT" not in os.environ)
    parser.add_argument("--only-paged-rope", action="store_true",
                        help="add the paged producer cases to the existing file, leave the rest as it is")
    args = parser.parse_args()
    if args.only_paged_rope:
        return update_paged_rope_only(args.reference_root)
    ref = load_reference(Path(args.reference_root))
    golden: dict = {"torch": torch.__version__, "cases": {}, "smoke": {}}

    for name, workload, batch, shrink in CASES:
        w = make_inputs(workload, seed=0, device="cpu", batch=batch, shrink=shrink)
        with arange_on_cpu():
            out = ref.reference(
                w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens,
                w.k_scale.reshape(1, 1, -1, 1), w.v_scale.reshape(1, 1, -1, 1),
            )
        golden["cases"][name] = dict(
            workload=workload, batch=batch, shrink=shrink,
            inputs_sha256=digest(w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens, w.k_scale, w.v_scale),
            output=out.clone(),
        )
        print(name, tuple(out.shape), out.dtype, "tokens", int(w.seq_lens.sum()))

    for batch, context, hq, hkv in [(1, 257, 16, 8), (3, 100, 16, 2), (2, 513, 32, 8)]:
        q, kc, vc, table, lens, ks, vs = smoke_recipe(ref, batch, context, hq, hkv)
        with arange_on_cpu():
            out = ref.reference(q, kc, vc, table.long(), lens, ks, vs)
        golden["smoke"][f"b{batch}-c{context}-q{hq}-kv{hkv}"] = dict(
            batch=batch, context=context, q_heads=hq, kv_heads=hkv,
            k_scale=ks, v_scale=vs, cache_sha256=digest(kc, vc), output=out.clone(),
        )
        print("smoke", batch, context, hq, hkv, ks, vs)

    # the fp16 / bf16 sibling: reference() of scripts/smoke_cuda_paged_decode_op.py:13-30
    ref16 = load_reference(Path(args.reference_root), "scripts/smoke_cuda_paged_decode_op.py")
    golden["kv16"] = {}
    for name, workload, batch, shrink, dtype in KV16_CASES:
        w = make_inputs(workload, seed=0, device="cpu", batch=batch, shrink=shrink, query_dtype=dtype, kv_dtype=dtype)
        with arange_on_cpu():
            out = ref16.reference(w.query, w.key_cache, w.value_cache, w.block_table.long(), w.seq_lens)
        golden["kv16"][name] = dict(
            workload=workload, batch=batch, shrink=shrink, dtype=str(dtype).replace("torch.", ""),
            inputs_sha256=digest(w.query, w.key_cache, w.value_cache, w.block_table, w.seq_lens),
            output=out.clone(),
        )
        print(name, tuple(out.shape), out.dtype, "tokens", int(w.seq_lens.sum()))

    # the producer step: rope_kv_reference of src/l20_stack/ops/triton_rope_kv.py:147-173
    sys.path.insert(0, str(Path(args.reference_root) / "src"))  # the module imports its own package
    rope = importlib.import_module("l20_stack.ops.triton_rope_kv")
    golden["rope"] = {}
    for name, tokens, hkv, d, rot, dtype in [("t37-h2-d128-r128-bf16", 37, 2, 128, 128, torch.bfloat16),
                                             ("t64-h4-d128-r64-fp16", 64, 4, 128, 64, torch.float16),
                                             ("t9-h8-d64-r64-bf16", 9, 8, 64, 64, torch.bfloat16)]:
        gen = torch.Generator().manual_seed(41)
        k = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
        v = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
        angle = torch.rand(tokens, rot // 2, generator=gen) * 6.2831853
        cos, sin = torch.cos(angle), torch.sin(angle)
        slots = torch.randperm(4 * tokens, generator=gen)[:tokens]
        kc = torch.zeros(4 * tokens, hkv, d, dtype=dtype)
        vc = torch.zeros_like(kc)
        kc, vc = rope.rope_kv_reference(k, v, cos, sin, slots, kc, vc)
        golden["rope"][name] = dict(tokens=tokens, kv_heads=hkv, head_dim=d, rotary_dim=rot,
                                    dtype=str(dtype).replace("torch.", ""), key_cache=kc.clone(), value_cache=vc.clone())
        print("rope", name)

    add_paged_rope_cases(golden, rope)
    torch.save(golden, HERE / "paged_decode_golden.pt")
    print("wrote", HERE / "paged_decode_golden.pt")
    return 0


PAGED_ROPE_CASES = [("s5-t23-h2-d128-r128-bf16", 5, 23, 2, 128, 128, torch.bfloat16),
                    ("s3-t40-h4-d128-r64-fp16", 3, 40, 4, 128, 64, torch.float16),
                    ("s8-t8-h8-d64-r64-bf16", 8, 8, 8, 64, 64, torch.bfloat16)]


def paged_rope_inputs(name, seqs, tokens, hkv, d, rot, dtype):
    """Seeded inputs of one paged case (the test regenerates them from the same recipe): new
    tokens of `seqs` sequences at arbitrary positions, written through a block table into a
    [blocks, 16, Hkv, D] cache."""
    gen = torch.Generator().manual_seed(43)
    k = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    v = torch.randn(tokens, hkv, d, generator=gen).to(dtype)
    angle = torch.rand(tokens, rot // 2, generator=gen) * 6.2831853
    max_blocks = 6
    table = torch.randperm(seqs * max_blocks, generator=gen).reshape(seqs, max_blocks)
    # distinct (sequence, position) pairs, so that no two tokens write the same slot
    flat = torch.randperm(seqs * max_blocks * 16, generator=gen)[:tokens]
    sequence_ids, positions = flat // (max_blocks * 16), flat % (max_blocks * 16)
    return k, v, torch.cos(angle), torch.sin(angle), sequence_ids, positions, table


def add_paged_rope_cases(golden, rope):
    """paged_rope_kv_reference of src/l20_stack/ops/triton_rope_kv.py:176-205."""
    golden["rope_paged"] = {}
    for case in PAGED_ROPE_CASES:
        name, seqs, tokens, hkv, d, rot, dtype = case
        k, v, cos, sin, sequence_ids, positions, table = paged_rope_inputs(*case)
        kc = torch.zeros(table.numel(), 16, hkv, d, dtype=dtype)
        vc = torch.zeros_like(kc)
        kc, vc = rope.paged_rope_kv_reference(k, v, cos, sin, sequence_ids, positions, table, kc, vc)
        # the rows the reference wrote, plus digests of the whole caches (everything else stays zero)
        blocks, offsets = table[sequence_ids, positions // 16], positions % 16
        golden["rope_paged"][name] = dict(seqs=seqs, tokens=tokens, kv_heads=hkv, head_dim=d, rotary_dim=rot,
                                          dtype=str(dtype).replace("torch.", ""),
                                          key_rows=kc[blocks, offsets].clone(), value_rows=vc[blocks, offsets].clone(),
                                          key_cache_sha256=digest(kc), value_cache_sha256=digest(vc))
        print("rope paged", name)


def update_paged_rope_only(reference_root: str) -> int:
    """Add the paged producer cases to the committed file without regenerating the rest."""
    sys.path.insert(0, str(Path(reference_root) / "src"))
    rope = importlib.import_module("l20_stack.ops.triton_rope_kv")
    golden = torch.load(HERE / "paged_decode_golden.pt", weights_only=False)
    add_paged_rope_cases(golden, rope)
    torch.save(golden, HERE / "paged_decode_golden.pt")
    print("updated", HERE / "paged_decode_golden.pt")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
