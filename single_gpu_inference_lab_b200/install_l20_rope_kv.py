#!/usr/bin/env python3
"""Install the fused RoPE + paged KV append into vLLM's FlashInfer backend, B200 build.

Same role and call site as the reference installer (integrations/vllm/install_l20_rope_kv.py):
vLLM's compilation pass ``fuse_rope_kvcache`` replaces "rotary embedding, then cache write" by
one call of the backend's ``do_rope_and_kv_cache_update`` when the backend says
``fused_rope_kvcache_supported()``.  The installer

* relaxes the guard in ``vllm/config/compilation.py`` that keeps the pass to ROCm (:48-62 there),
* gives the FlashInfer backend the two methods (:73-121 there), and
* copies the operator module and libraries into ``vllm/v1/attention/ops/``.

What differs from the reference:

* the gate asks for sm_100 instead of sm_89 and ACCEPTS FP8 caches -- the reference's gate is
  ``kv_cache_dtype == "auto"`` (:86, :182) because its operator refuses quantised caches
  (integrations/vllm/l20_rope_kv.py:273-274); this operator quantises with the layer's
  ``_k_scale`` / ``_v_scale``, the scales the decode operator dequantises with;
* FlashInfer keeps the cache in the HND layout on sm_100 and hands the method a logical
  ``[blocks, 2, 16, Hkv, D]`` tensor whose strides carry that layout: the operator takes strides;
* the Triton attention backend is left alone (the reference patches it too, :123-229): on sm_100
  an FP8 cache runs on the FlashInfer backend.

``VLLM_L20_ROPE_KV_TRACE=<path>`` appends one JSON line per call of the operator.
``--uninstall`` restores the backups (``*.l20-rope-backup``).  ``--vllm-source-dir`` points at a
vLLM checkout instead of the installed package.
"""

from __future__ import annotations

import argparse
import shutil
from pathlib import Path

from .install_l20_fp8_paged_decode import find_vllm_package, replace_once

HERE = Path(__file__).resolve().parent
BACKUP_SUFFIX = ".l20-rope-backup"
COPIED = (
    "l20_rope_kv.py",
    "l20_paged_split_kv.py",
    "l20_paged_decode.py",
    "l20_paged_decode_ops.so",
    "libpaged_fp8_decode.so",
)

GUARD_OLD = "if self.fuse_rope_kvcache and not current_platform.is_rocm():"
GUARD_NEW = "if (self.fuse_rope_kvcache and not current_platform.is_rocm()\n                and not current_platform.is_cuda()):"

IMPORT_OLD = "from vllm.v1.attention.ops.merge_attn_states import merge_attn_states\n"
IMPORT_NEW = IMPORT_OLD + "from vllm.v1.attention.ops.l20_rope_kv import l20_rope_and_cache\n"

METHODS_MARKER = "\n\ndef fast_plan_decode(\n"
METHODS = '''

    def fused_rope_kvcache_supported(self):
        capability = current_platform.get_device_capability()
        return (
            capability is not None
            and capability.to_int() == 100
            and not getattr(self, "is_kvcache_nvfp4", False)
            and (self.kv_cache_dtype == "auto" or is_quantized_kv_cache(self.kv_cache_dtype))
            and self.kv_sharing_target_layer_name is None
            and self.head_size <= 256
        )

    def do_rope_and_kv_cache_update(
        self,
        layer: torch.nn.Module,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        positions: torch.Tensor,
        cos_sin_cache: torch.Tensor,
        is_neox: bool,
        kv_cache: torch.Tensor,
        layer_slot_mapping: torch.Tensor,
    ) -> None:
        # logical [blocks, 16, Hkv, D] views of the layer's cache: vLLM hands this method the cache
        # in that shape whatever the physical layout (the strides carry it); a tensor that comes
        # head-major instead is turned into the same view
        key_cache, value_cache = kv_cache[:, 0], kv_cache[:, 1]
        if key_cache.shape[2] != key.shape[1] and key_cache.shape[1] == key.shape[1]:
            key_cache = key_cache.permute(0, 2, 1, 3)
            value_cache = value_cache.permute(0, 2, 1, 3)
        l20_fp8 = is_quantized_kv_cache(self.kv_cache_dtype)
        if l20_fp8 and key_cache.dtype == torch.uint8:
            key_cache = key_cache.view(torch.float8_e4m3fn)
            value_cache = value_cache.view(torch.float8_e4m3fn)
        l20_rope_and_cache(
            query,
            key,
            value,
            positions,
            cos_sin_cache,
            is_neox,
            key_cache,
            value_cache,
            layer_slot_mapping,
            k_scale=layer._k_scale if l20_fp8 else None,
            v_scale=layer._v_scale if l20_fp8 else None,
        )
        l20_trace = __import__("os").environ.get("VLLM_L20_ROPE_KV_TRACE")
        if l20_trace:
            with open(l20_trace, "a", encoding="utf-8") as l20_sink:
                l20_sink.write(
                    '{"event": "l20_rope_kv_run", "tokens": %d, "fp8_cache": %s}\\n'
                    % (int(query.shape[0]), "true" if l20_fp8 else "false")
                )
'''


def patch_config_source(source: str) -> str:
    source = replace_once(source, GUARD_OLD, GUARD_NEW, "CUDA config guard")
    return source.replace(
        "KV cache fusion currently only enabled on ROCm.",
        "KV cache fusion requires ROCm/AITER or the CUDA operator of this build.",
        1,
    )


def patch_backend_source(source: str) -> str:
    source = replace_once(source, IMPORT_OLD, IMPORT_NEW, "kernel import")
    return replace_once(source, METHODS_MARKER, METHODS + METHODS_MARKER, "FlashInfer methods")


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--vllm-source-dir")
    parser.add_argument("--uninstall", action="store_true")
    args = parser.parse_args(argv)

    package = find_vllm_package(args.vllm_source_dir)
    targets = {
        "config": package / "config/compilation.py",
        "backend": package / "v1/attention/backends/flashinfer.py",
    }
    backups = {name: path.with_suffix(path.suffix + BACKUP_SUFFIX) for name, path in targets.items()}
    if args.uninstall:
        for name, path in targets.items():
            if backups[name].exists():
                shutil.copy2(backups[name], path)
        return 0
    missing = [name for name in COPIED if not (HERE / name).exists()]
    if missing:
        raise RuntimeError("missing " + ", ".join(missing) + ": build the libraries first "
                           "(python -m single_gpu_inference_lab_b200.build)")
    patched = {
        "config": patch_config_source(targets["config"].read_text(encoding="utf-8")),
        "backend": patch_backend_source(targets["backend"].read_text(encoding="utf-8")),
    }
    for name, path in targets.items():
        if not backups[name].exists():
            shutil.copy2(path, backups[name])
    op_dir = package / "v1/attention/ops"
    for name in COPIED:
        shutil.copy2(HERE / name, op_dir)
    for name, path in targets.items():
        path.write_text(patched[name], encoding="utf-8")
    print(package)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
