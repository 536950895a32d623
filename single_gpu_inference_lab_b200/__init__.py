"""B200 (sm_100a) paged FP8-e4m3 KV-cache GQA decode attention.

A drop-in for one path of Kevin-Li-2025/single-gpu-inference-lab: the
``l20_stack::paged_decode_fp8_e4m3_split_out`` operator, its Python wrappers
(``l20_paged_decode``, ``l20_paged_split_kv``) and its vLLM install hook.

Importing this package does not load any native code; ``l20_paged_decode`` loads the
dispatcher library on import (as the reference module does) and ``cabi`` binds the C ABI
with ``ctypes``.  There is no CPU or eager fallback: a missing library raises.
"""

__all__ = ["build", "cabi", "l20_paged_decode", "l20_paged_split_kv", "workloads"]
__version__ = "0.1.0"
