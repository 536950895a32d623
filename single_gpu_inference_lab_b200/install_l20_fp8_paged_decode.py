#!/usr/bin/env python3
"""Install the gated B200 paged FP8 decode path into vLLM's FlashInfer backend.

Same role, command line and switches as the reference installer
(integrations/vllm/install_l20_fp8_paged_decode.py): it text-patches
``vllm/v1/attention/backends/flashinfer.py`` so that the FlashInfer *decode* branch sends
FP8-KV decode steps through ``l20_paged_split_kv_attention_fp8`` when

* ``VLLM_ENABLE_L20_FP8_PAGED_DECODE=1`` is set, the GPU is sm_100, the step is not being
  captured into a CUDA graph (unless ``VLLM_L20_PAGED_CUDAGRAPH=1``: the operator allocates
  nothing and synchronises nothing, so it can be recorded), the cache is a non-NVFP4 FP8 cache,
  head_dim is 64 or 128, and
* the policy ``should_use_l20_paged_fp8_split_kv`` agrees, or ``VLLM_L20_FP8_PAGED_FORCE=1``;

``VLLM_L20_FP8_PAGED_TRACE=<path>`` appends one JSON line per dispatched step with the
reference's keys.  ``--uninstall`` restores the backup ``flashinfer.py.l20-fp8-paged-backup``.

The same block also carries the non-quantised sibling, which the reference installs with a
second installer at the same call site (integrations/vllm/install_l20_paged_decode.py:95-170,
always on for a few shapes): here ``VLLM_ENABLE_L20_PAGED_DECODE=1`` sends decode steps over
fp16 / bf16 caches (head_dim 128, at most 8 query heads per KV head) through
``l20_paged_split_kv_attention`` when ``should_use_l20_paged_split_kv`` agrees or
``VLLM_L20_PAGED_FORCE=1``; ``VLLM_L20_PAGED_TRACE=<path>`` traces those steps.

What differs from the reference installer, because vLLM on sm_100 differs from vLLM on sm_89
(and because in eager mode the host time of this block is most of a layer's decode time):

* the switches, the GPU capability and the cache dtype are read once per attention layer and
  kept on it (the reference reads the environment on every call); the cache views are made
  once per cache buffer;

* it is self-sufficient: the reference FP8 installer only works after its fp16 sibling
  installer has added ``block_tables / seq_lens / max_seq_len`` to ``FIDecode`` and nested the
  decode call (install_l20_paged_decode.py:78-93, :160-168); this one adds the fields itself;
* it imports what its text uses (``os``, ``json``), which the reference text assumes;
* FlashInfer asks for the HND cache layout on sm_100, so the hook hands the operator a
  ``[pages, 16, Hkv, D]`` *view* of either layout (the kernels take strides);
* what depends on the step's block table and lengths alone -- the balanced kernel's work split
  (plan), the shared-prefix groups, the workspace -- is made once per model step by the first
  layer and kept on the step's ``FIDecode`` (``l20_decode_step.py``), not once per layer;
* with ``VLLM_ENABLE_L20_SHARED_PREFIX_DECODE=1`` (the reference's switch, which there only
  traces candidates: install_l20_shared_prefix_decode.py:92-110) a step whose batch has
  shared-prefix groups runs the grouped shared-prefix operator, and
  ``VLLM_L20_SHARED_PREFIX_DECODE_TRACE`` gets the candidate and run records;
* it copies the operator's modules and two shared libraries next to each other into
  ``vllm/v1/attention/ops/`` (the reference copies one Triton module).
"""

from __future__ import annotations

import argparse
import importlib.util
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent
BACKUP_SUFFIX = ".py.l20-fp8-paged-backup"
COPIED = (
    "l20_paged_split_kv.py",
    "l20_paged_decode.py",
    "l20_decode_step.py",
    "l20_shared_prefix_decode_dispatch.py",
    "l20_paged_decode_ops.so",
    "libpaged_fp8_decode.so",
)


def replace_once(source: str, old: str, new: str, label: str) -> str:
    if new in source:
        return source
    if old not in source:
        raise RuntimeError(f"cannot find patch point: {label}")
    return source.replace(old, new, 1)


def find_vllm_package(source_dir: str | None) -> Path:
    candidates = []
    if source_dir:
        candidates.append(Path(source_dir).expanduser().resolve() / "vllm")
    candidates.append(Path.cwd() / "vllm")
    spec = importlib.util.find_spec("vllm")  # located, not imported
    if spec is not None and spec.submodule_search_locations:
        candidates.append(Path(list(spec.submodule_search_locations)[0]))
    for candidate in candidates:
        if (candidate / "v1/attention/backends/flashinfer.py").exists():
            return candidate
    raise RuntimeError("cannot find vLLM source package")


IMPORT_OLD = "import torch\n"
IMPORT_NEW = "import torch\nimport json as l20_json\nimport os as l20_os\n"

FIDECODE_OLD = '''class FIDecode:
    """Metadata for the native FlashInfer decode pathway (non-TRTLLM)."""

    wrapper: BatchDecodeWithPagedKVCacheWrapper
'''
FIDECODE_NEW = '''class FIDecode:
    """Metadata for the native FlashInfer decode pathway (non-TRTLLM)."""

    wrapper: BatchDecodeWithPagedKVCacheWrapper
    block_tables: torch.Tensor | None = None
    seq_lens: torch.Tensor | None = None
    max_seq_len: int = 0
    l20_step: object | None = None  # what the first layer of a step computes for all of them
'''

CONSTRUCT_OLD = "attn_metadata.decode = FIDecode(wrapper=decode_wrapper)"
CONSTRUCT_NEW = """attn_metadata.decode = FIDecode(
                    wrapper=decode_wrapper,
                    block_tables=block_table_tensor[:num_decodes],
                    seq_lens=seq_lens[:num_decodes],
                    max_seq_len=max_seq_len,
                )"""

CALL_OLD = """                else:
                    decode_wrapper.run(
                        decode_query,
                        kv_cache_permute,
                        k_scale=layer._k_scale_float,
                        v_scale=layer._v_scale_float,
                        out=out_decode,
                        kv_cache_sf=kv_cache_sf,
                    )
"""

CALL_NEW = """                else:
                    # What cannot change while the engine runs is decided once per layer: the
                    # switches, the GPU, the cache dtype, the attention variant.
                    l20_static = getattr(self, "_l20_static_gate", None)
                    if l20_static is None:
                        l20_common = (
                            current_platform.get_device_capability()
                            == DeviceCapability(10, 0)
                            and self.window_left == -1
                            and not self.logits_soft_cap
                        )
                        l20_static = self._l20_static_gate = {
                            "fp8": l20_common
                            and l20_os.getenv("VLLM_ENABLE_L20_FP8_PAGED_DECODE", "0") == "1"
                            and not self.is_kvcache_nvfp4
                            and is_quantized_kv_cache(self.kv_cache_dtype),
                            "fp8_force": l20_os.getenv("VLLM_L20_FP8_PAGED_FORCE", "0") == "1",
                            "fp8_trace": l20_os.getenv("VLLM_L20_FP8_PAGED_TRACE"),
                            "kv16": l20_common
                            and l20_os.getenv("VLLM_ENABLE_L20_PAGED_DECODE", "0") == "1"
                            and not is_quantized_kv_cache(self.kv_cache_dtype),
                            "kv16_force": l20_os.getenv("VLLM_L20_PAGED_FORCE", "0") == "1",
                            "kv16_trace": l20_os.getenv("VLLM_L20_PAGED_TRACE"),
                            # the operator is capturable: VLLM_L20_PAGED_CUDAGRAPH=1 keeps the hook on
                            # while vLLM records its decode graphs (the reference always steps aside)
                            "graphs": l20_os.getenv("VLLM_L20_PAGED_CUDAGRAPH", "0") == "1",
                            # the kernel in front of a decode call (the cache write, a prefill
                            # kernel) writes K/V at most at the decode requests' last positions:
                            # with VLLM_L20_PAGED_EARLY_KV=1 older pages are streamed while it drains
                            "early_kv": l20_os.getenv("VLLM_L20_PAGED_EARLY_KV", "0") == "1",
                            "hnd": get_kv_cache_layout() == "HND",
                            "views": None,
                        }
                    l20_fp8_batch = decode_query.shape[0]
                    l20_fp8_max_seq = attn_metadata.decode.max_seq_len
                    l20_fp8_hnd = l20_static["hnd"]
                    l20_dynamic = (
                        (l20_static["fp8"] or l20_static["kv16"])
                        and (
                            l20_static["graphs"]
                            or not torch.cuda.is_current_stream_capturing()
                        )
                        and attn_metadata.decode.block_tables is not None
                        and l20_fp8_max_seq > 0
                        and decode_query.dim() == 3
                        and abs(self.scale - decode_query.shape[-1] ** -0.5) < 1e-6
                        and kv_cache_permute.dim() == 5
                        and kv_cache_permute.shape[1] == 2
                        and kv_cache_permute.shape[3 if l20_fp8_hnd else 2] == 16
                        and kv_cache_permute.shape[-1] == decode_query.shape[-1]
                    )
                    l20_fp8_enabled = (
                        l20_dynamic
                        and l20_static["fp8"]
                        and decode_query.shape[-1] in (64, 128)
                    )
                    if l20_fp8_enabled and not l20_static["fp8_force"]:
                        from vllm.v1.attention.ops.l20_paged_split_kv import (
                            should_use_l20_paged_fp8_split_kv,
                        )

                        l20_fp8_enabled = should_use_l20_paged_fp8_split_kv(
                            int(l20_fp8_batch),
                            int(l20_fp8_max_seq),
                        )
                    # the non-quantised sibling (fp16 / bf16 caches): VLLM_ENABLE_L20_PAGED_DECODE=1
                    l20_kv16_enabled = (
                        l20_dynamic
                        and l20_static["kv16"]
                        and decode_query.shape[-1] == 128
                        and decode_query.dtype in (torch.float16, torch.bfloat16)
                        and kv_cache_permute.dtype == decode_query.dtype
                        and decode_query.shape[1]
                        <= 8 * kv_cache_permute.shape[2 if l20_fp8_hnd else 3]
                    )
                    if l20_kv16_enabled and not l20_static["kv16_force"]:
                        from vllm.v1.attention.ops.l20_paged_split_kv import (
                            should_use_l20_paged_split_kv,
                        )

                        l20_kv16_enabled = should_use_l20_paged_split_kv(
                            int(l20_fp8_batch),
                            int(l20_fp8_max_seq),
                        )
                    if l20_fp8_enabled or l20_kv16_enabled:
                        from vllm.v1.attention.ops.l20_decode_step import (
                            l20_decode_step,
                            l20_grouped_decode,
                        )
                        from vllm.v1.attention.ops.l20_paged_split_kv import (
                            l20_paged_split_kv_attention,
                            l20_paged_split_kv_attention_fp8,
                        )

                        # logical [pages, 16, Hkv, D] views of the layer's cache, made once per buffer
                        l20_views = l20_static["views"]
                        if l20_views is None or l20_views[0] != kv_cache_permute.data_ptr():
                            key_cache, value_cache = kv_cache_permute.unbind(1)
                            if l20_fp8_hnd:
                                # [pages, Hkv, 16, D] -> logical [pages, 16, Hkv, D] view
                                key_cache = key_cache.permute(0, 2, 1, 3)
                                value_cache = value_cache.permute(0, 2, 1, 3)
                            if l20_fp8_enabled and key_cache.dtype == torch.uint8:
                                key_cache = key_cache.view(torch.float8_e4m3fn)
                                value_cache = value_cache.view(torch.float8_e4m3fn)
                            l20_views = l20_static["views"] = (
                                kv_cache_permute.data_ptr(),
                                key_cache,
                                value_cache,
                            )
                        key_cache, value_cache = l20_views[1], l20_views[2]
                        # once per model step, by its first layer: the work split (plan), the
                        # shared-prefix groups, and one workspace for all layers
                        l20_step = l20_decode_step(
                            attn_metadata.decode,
                            decode_query,
                            key_cache,
                            value_cache,
                            attn_metadata.decode.block_tables,
                            attn_metadata.decode.seq_lens,
                            l20_fp8_max_seq,
                            split_size=512,
                            fp8=bool(l20_fp8_enabled),
                        )
                    if l20_fp8_enabled and l20_step.groups is not None:
                        # VLLM_ENABLE_L20_SHARED_PREFIX_DECODE=1 and this step has shared-prefix groups
                        l20_grouped_decode(
                            l20_step,
                            decode_query,
                            key_cache,
                            value_cache,
                            attn_metadata.decode.block_tables,
                            attn_metadata.decode.seq_lens,
                            layer._k_scale_float,
                            layer._v_scale_float,
                            l20_fp8_max_seq,
                            out_decode.view_as(decode_query),
                            split_size=512,
                        )
                    elif l20_fp8_enabled:
                        l20_paged_split_kv_attention_fp8(
                            decode_query,
                            key_cache,
                            value_cache,
                            attn_metadata.decode.block_tables,
                            attn_metadata.decode.seq_lens,
                            k_scale=layer._k_scale_float,
                            v_scale=layer._v_scale_float,
                            max_seq_len=l20_fp8_max_seq,
                            split_size=512,
                            output=out_decode.view_as(decode_query),
                            workspace=l20_step.workspace,
                            metadata_stable=True,  # built once per model step
                            kv_stable=l20_static["early_kv"],
                            plan=l20_step.plan,
                        )
                        trace_path = l20_static["fp8_trace"]
                        if trace_path:
                            with open(trace_path, "a", encoding="utf-8") as trace_file:
                                trace_file.write(
                                    l20_json.dumps(
                                        {
                                            "event": "l20_fp8_paged_decode_run",
                                            "batch": int(l20_fp8_batch),
                                            "max_seq_len": int(l20_fp8_max_seq),
                                            "q_heads": int(decode_query.shape[1]),
                                            "kv_heads": int(key_cache.shape[2]),
                                        },
                                        sort_keys=True,
                                    )
                                    + "\\n"
                                )
                    elif l20_kv16_enabled:
                        l20_paged_split_kv_attention(
                            decode_query,
                            key_cache,
                            value_cache,
                            attn_metadata.decode.block_tables,
                            attn_metadata.decode.seq_lens,
                            split_size=512,
                            workspace=l20_step.workspace,
                            max_seq_len=l20_fp8_max_seq,
                            output=out_decode.view_as(decode_query),
                            metadata_stable=True,
                            kv_stable=l20_static["early_kv"],
                            plan=l20_step.plan,
                        )
                        trace_path = l20_static["kv16_trace"]
                        if trace_path:
                            with open(trace_path, "a", encoding="utf-8") as trace_file:
                                trace_file.write(
                                    l20_json.dumps(
                                        {
                                            "event": "l20_paged_decode_run",
                                            "batch": int(l20_fp8_batch),
                                            "max_seq_len": int(l20_fp8_max_seq),
                                            "q_heads": int(decode_query.shape[1]),
                                            "kv_heads": int(key_cache.shape[2]),
                                        },
                                        sort_keys=True,
                                    )
                                    + "\\n"
                                )
                    else:
                        decode_wrapper.run(
                            decode_query,
                            kv_cache_permute,
                            k_scale=layer._k_scale_float,
                            v_scale=layer._v_scale_float,
                            out=out_decode,
                            kv_cache_sf=kv_cache_sf,
                        )
"""


def patch_backend_source(source: str) -> str:
    """The four text edits, each applied once and idempotent."""
    source = replace_once(source, IMPORT_OLD, IMPORT_NEW, "torch import")
    source = replace_once(source, FIDECODE_OLD, FIDECODE_NEW, "FIDecode metadata")
    source = replace_once(source, CONSTRUCT_OLD, CONSTRUCT_NEW, "FIDecode construction")
    source = replace_once(source, CALL_OLD, CALL_NEW, "FlashInfer decode call")
    return source


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--vllm-source-dir")
    parser.add_argument("--uninstall", action="store_true")
    args = parser.parse_args(argv)

    package = find_vllm_package(args.vllm_source_dir)
    backend = package / "v1/attention/backends/flashinfer.py"
    backup = backend.with_suffix(BACKUP_SUFFIX)
    op_dir = package / "v1/attention/ops"
    if args.uninstall:
        if backup.exists():
            shutil.copy2(backup, backend)
        return 0
    missing = [name for name in COPIED if not (HERE / name).exists()]
    if missing:
        raise RuntimeError(
            "missing " + ", ".join(missing) + ": build the libraries first "
            "(python -m single_gpu_inference_lab_b200.build)"
        )
    patched = patch_backend_source(backend.read_text(encoding="utf-8"))
    if not backup.exists():
        shutil.copy2(backend, backup)
    for name in COPIED:
        shutil.copy2(HERE / name, op_dir)
    backend.write_text(patched, encoding="utf-8")
    print(package)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
