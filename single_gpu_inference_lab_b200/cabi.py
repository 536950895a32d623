"""``ctypes`` binding of the C ABI in ``include/paged_fp8_decode.h``.

This is the route a non-PyTorch host takes; torch tensors are used here only as device
buffers whose ``data_ptr()`` / strides are handed over as plain integers.  The parity tests
call the kernels through this module.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_NAME = "libpaged_fp8_decode.so"

PFD_DTYPE_F32, PFD_DTYPE_F16, PFD_DTYPE_BF16 = 0, 1, 2
PFD_FLAG_NO_TMA = 1
PFD_FLAG_NO_DIRECT_OUT = 2
PFD_FLAG_PARTIAL_ONLY = 4
PFD_FLAG_FIXED_SPLITS = 8
PFD_FLAG_EARLY_METADATA = 32
PFD_FLAG_SINGLE_LAUNCH = 64
PFD_FLAG_ALL_IN_GROUPS = 128
PFD_FLAG_EARLY_KV = 256

EXPORTS = (
    "pfd_paged_decode_fp8_e4m3_split_out",
    "pfd_paged_decode_fp8_e4m3_split_out_noalloc",
    "pfd_paged_decode_kv16_split_out",
    "pfd_shared_prefix_decode_fp8_e4m3",
    "pfd_shared_prefix_decode_grouped_fp8_e4m3",
    "pfd_group_shared_prefixes",
    "pfd_prefix_groups_bytes",
    "pfd_merge_packed",
    "pfd_resolve_slots",
    "pfd_rope_quant_append",
    "pfd_balanced_workspace_rows",
    "pfd_plan_bytes",
    "pfd_plan_decode",
    "pfd_exchange_merge",
    "pfd_exchange_bytes",
    "pfd_exchange_control_offset",
    "pfd_exchange_alloc",
    "pfd_exchange_open",
    "pfd_exchange_close",
    "pfd_exchange_free",
    "pfd_device_status",
    "pfd_set_wait_limit_ns",
    "pfd_set_suffix_form",
    "pfd_selftest_bounded_wait",
    "pfd_last_path",
    "pfd_launch_count",
    "pfd_last_error",
    "pfd_abi_version",
)


class Exchange(C.Structure):
    """Mirror of ``pfd_exchange``: where the ranks of a KV-range exchange receive."""

    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("recv", C.c_void_p * 8),
        ("control", C.c_void_p),
    ]


class IpcHandle(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * 64)]


class DecodeArgs(C.Structure):
    """Mirror of ``pfd_decode_args`` (field order and types must match the header)."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("flags", C.c_uint32),
        ("batch", C.c_int32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("page_size", C.c_int32),
        ("max_seq_len", C.c_int32),
        ("split_size", C.c_int32),
        ("kv_start", C.c_int32),
        ("query_dtype", C.c_int32),
        ("partial_dtype", C.c_int32),
        ("sm_scale", C.c_float),
        ("k_scale", C.c_float),
        ("v_scale", C.c_float),
        ("workspace_splits", C.c_int32),
        ("query", C.c_void_p),
        ("q_stride_b", C.c_int64),
        ("q_stride_h", C.c_int64),
        ("key_cache", C.c_void_p),
        ("value_cache", C.c_void_p),
        ("num_pages", C.c_int64),
        ("k_stride_page", C.c_int64),
        ("k_stride_token", C.c_int64),
        ("k_stride_head", C.c_int64),
        ("v_stride_page", C.c_int64),
        ("v_stride_token", C.c_int64),
        ("v_stride_head", C.c_int64),
        ("block_table", C.c_void_p),
        ("bt_stride_b", C.c_int64),
        ("seq_lens", C.c_void_p),
        ("k_scale_per_head", C.c_void_p),
        ("v_scale_per_head", C.c_void_p),
        ("partial_output", C.c_void_p),
        ("partial_max", C.c_void_p),
        ("partial_sum", C.c_void_p),
        ("partial_stride_b", C.c_int64),
        ("partial_stride_h", C.c_int64),
        ("partial_stride_s", C.c_int64),
        ("output", C.c_void_p),
        ("o_stride_b", C.c_int64),
        ("o_stride_h", C.c_int64),
        ("packed_output", C.c_void_p),
        ("stream", C.c_void_p),
        ("page_indptr", C.c_void_p),
        ("plan", C.c_void_p),
        ("exchange", C.POINTER(Exchange)),
    ]


_lib = None


def library_path() -> Path:
    return Path(__file__).with_name(LIB_NAME)


def load() -> C.CDLL:
    """Load the C-ABI library (built in-tree by ``build.py``).  Raises if it is missing."""
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -m single_gpu_inference_lab_b200.build`; "
                "there is no fallback implementation"
            )
        lib = C.CDLL(str(path))
        lib.pfd_paged_decode_fp8_e4m3_split_out.argtypes = [C.POINTER(DecodeArgs)]
        lib.pfd_paged_decode_fp8_e4m3_split_out.restype = C.c_int
        lib.pfd_paged_decode_fp8_e4m3_split_out_noalloc.argtypes = [C.POINTER(DecodeArgs)]
        lib.pfd_paged_decode_fp8_e4m3_split_out_noalloc.restype = C.c_int
        lib.pfd_merge_packed.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]
        lib.pfd_merge_packed.restype = C.c_int
        lib.pfd_resolve_slots.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        lib.pfd_resolve_slots.restype = C.c_int
        lib.pfd_launch_count.restype = C.c_int64
        lib.pfd_last_error.restype = C.c_char_p
        lib.pfd_abi_version.restype = C.c_int
        _lib = lib
    return _lib


def _dtype_code(dtype: torch.dtype) -> int:
    return {torch.float32: PFD_DTYPE_F32, torch.float16: PFD_DTYPE_F16, torch.bfloat16: PFD_DTYPE_BF16}[dtype]


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(load().pfd_last_error().decode())


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def decode_args(
    query, key_cache, value_cache, block_table, seq_lens, *, k_scale, v_scale, max_seq_len,
    split_size, output=None, packed_output=None, workspace=None, kv_start=0, sm_scale=0.0, flags=0,
    page_indptr=None, plan=None, exchange=None,
) -> DecodeArgs:
    """Fill ``pfd_decode_args`` from torch tensors (device buffers).  With ``page_indptr``
    (int32 ``[B + 1]``) ``block_table`` is the flat list of page ids it indexes.  ``plan`` is the
    buffer ``plan_decode`` filled for the same inputs.  ``exchange`` is an ``Exchange`` whose
    ranks receive this call's packed rows instead of ``output`` / ``packed_output``."""
    a = DecodeArgs()
    a.struct_size = C.sizeof(DecodeArgs)
    a.flags = flags
    a.batch, a.num_q_heads, a.head_dim = query.shape
    a.num_kv_heads = key_cache.shape[2]
    a.page_size = key_cache.shape[1]
    a.max_seq_len = int(max_seq_len)
    a.split_size = int(split_size)
    a.kv_start = int(kv_start)
    a.query_dtype = _dtype_code(query.dtype)
    a.sm_scale = float(sm_scale)
    a.query = query.data_ptr()
    a.q_stride_b, a.q_stride_h = query.stride(0), query.stride(1)
    a.key_cache, a.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
    a.num_pages = key_cache.shape[0]
    a.k_stride_page, a.k_stride_token, a.k_stride_head = key_cache.stride()[:3]
    a.v_stride_page, a.v_stride_token, a.v_stride_head = value_cache.stride()[:3]
    a.block_table = block_table.data_ptr()
    a.bt_stride_b = block_table.stride(0) if page_indptr is None else 0
    if page_indptr is not None:
        a.page_indptr = page_indptr.data_ptr()
    a.seq_lens = seq_lens.data_ptr()
    if isinstance(k_scale, torch.Tensor):
        a.k_scale_per_head = k_scale.data_ptr()
    else:
        a.k_scale = float(k_scale)
    if isinstance(v_scale, torch.Tensor):
        a.v_scale_per_head = v_scale.data_ptr()
    else:
        a.v_scale = float(v_scale)
    if workspace is not None:
        po, pm, ps = workspace[:3]
        a.partial_output, a.partial_max, a.partial_sum = po.data_ptr(), pm.data_ptr(), ps.data_ptr()
        a.partial_dtype = _dtype_code(po.dtype)
        a.partial_stride_b, a.partial_stride_h, a.partial_stride_s = pm.stride()
        a.workspace_splits = po.shape[2]
    if output is not None:
        a.output = output.data_ptr()
        a.o_stride_b, a.o_stride_h = output.stride(0), output.stride(1)
    if packed_output is not None:
        a.packed_output = packed_output.data_ptr()
    if plan is not None:
        a.plan = plan.data_ptr()
    if exchange is not None:
        a.exchange = C.pointer(exchange)  # the pointer object keeps `exchange` alive with `a`
    a.stream = _stream(query)
    return a


def plan_bytes(batch: int, num_kv_heads: int) -> int:
    """Size of the plan buffer of ``plan_decode`` on the current device (``pfd_plan_bytes``)."""
    lib = load()
    lib.pfd_plan_bytes.argtypes = [C.c_int32, C.c_int32]
    lib.pfd_plan_bytes.restype = C.c_int64
    n = int(lib.pfd_plan_bytes(int(batch), int(num_kv_heads)))
    if n < 0:
        raise RuntimeError(lib.pfd_last_error().decode())
    return n


def plan_decode(query, key_cache, value_cache, block_table, seq_lens, *, plan=None, **kw) -> torch.Tensor:
    """``pfd_plan_decode``: the work split of a model step's decode calls, computed once from the
    lengths and the block table; pass the returned int32 buffer as ``plan=`` to the decode calls
    of every layer.  Keywords as for ``decode_args``."""
    kw.setdefault("k_scale", 1.0)
    kw.setdefault("v_scale", 1.0)
    args = decode_args(query, key_cache, value_cache, block_table, seq_lens, **kw)
    if plan is None:
        with torch.cuda.device(query.device):
            plan = torch.empty(plan_bytes(query.shape[0], key_cache.shape[2]) // 4, dtype=torch.int32, device=query.device)
    lib = load()
    lib.pfd_plan_decode.argtypes = [C.POINTER(DecodeArgs), C.c_int32, C.c_void_p, C.c_int64]
    lib.pfd_plan_decode.restype = C.c_int
    with torch.cuda.device(query.device):
        _check(lib.pfd_plan_decode(C.byref(args), key_cache.element_size(), plan.data_ptr(), plan.numel() * 4))
    return plan


def paged_decode_fp8_e4m3_split_out(query, key_cache, value_cache, block_table, seq_lens, **kw) -> None:
    """One layer-step through ``pfd_paged_decode_fp8_e4m3_split_out``; see ``decode_args``."""
    args = decode_args(query, key_cache, value_cache, block_table, seq_lens, **kw)
    with torch.cuda.device(query.device):
        _check(load().pfd_paged_decode_fp8_e4m3_split_out(C.byref(args)))


def paged_decode_kv16_split_out(query, key_cache, value_cache, block_table, seq_lens, **kw) -> None:
    """One layer-step over fp16 / bf16 caches (the query's dtype) through
    ``pfd_paged_decode_kv16_split_out``; same keywords as above, the scales are ignored."""
    if key_cache.dtype != query.dtype or value_cache.dtype != query.dtype:
        raise RuntimeError("K/V cache must have the query's dtype")
    kw.setdefault("k_scale", 1.0)
    kw.setdefault("v_scale", 1.0)
    args = decode_args(query, key_cache, value_cache, block_table, seq_lens, **kw)
    with torch.cuda.device(query.device):
        _check(load().pfd_paged_decode_kv16_split_out(C.byref(args)))


def shared_prefix_decode_fp8_e4m3(query, key_cache, value_cache, block_table, seq_lens, *, prefix_len, **kw) -> None:
    """One layer-step through ``pfd_shared_prefix_decode_fp8_e4m3``: dense tcgen05 pass over the
    prefix every request shares, split-KV pass over the private suffixes, one merge."""
    args = decode_args(query, key_cache, value_cache, block_table, seq_lens, **kw)
    lib = load()
    lib.pfd_shared_prefix_decode_fp8_e4m3.argtypes = [C.POINTER(DecodeArgs), C.c_int32]
    lib.pfd_shared_prefix_decode_fp8_e4m3.restype = C.c_int
    with torch.cuda.device(query.device):
        _check(lib.pfd_shared_prefix_decode_fp8_e4m3(C.byref(args), int(prefix_len)))


def group_shared_prefixes(block_table, *, prefix_lengths=None, uniform_prefix_len=0, seq_lens=None, min_batch=8,
                          min_prefix_len=4096, max_groups=None) -> tuple[torch.Tensor, int]:
    """``pfd_group_shared_prefixes``: (int32 groups buffer on the device, its max_groups)."""
    lib = load()
    lib.pfd_prefix_groups_bytes.argtypes = [C.c_int32, C.c_int32]
    lib.pfd_prefix_groups_bytes.restype = C.c_int64
    batch = block_table.shape[0]
    if max_groups is None:
        max_groups = max(1, batch // max(1, min_batch))
    nbytes = int(lib.pfd_prefix_groups_bytes(batch, max_groups))
    if nbytes < 0:
        raise RuntimeError(lib.pfd_last_error().decode())
    lib.pfd_group_shared_prefixes.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                              C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p]
    lib.pfd_group_shared_prefixes.restype = C.c_int
    with torch.cuda.device(block_table.device):
        groups = torch.empty(nbytes // 4, dtype=torch.int32, device=block_table.device)
        _check(lib.pfd_group_shared_prefixes(
            block_table.data_ptr(), block_table.stride(0), block_table.shape[1],
            None if prefix_lengths is None else prefix_lengths.data_ptr(), int(uniform_prefix_len),
            None if seq_lens is None else seq_lens.data_ptr(), batch, int(min_batch), int(min_prefix_len), int(max_groups),
            groups.data_ptr(), nbytes, _stream(block_table)))
    return groups, max_groups


def shared_prefix_decode_grouped_fp8_e4m3(query, key_cache, value_cache, block_table, seq_lens, *, groups, max_groups,
                                          max_prefix_len=None, max_suffix_len=None, **kw) -> None:
    """One layer-step through ``pfd_shared_prefix_decode_grouped_fp8_e4m3``: any number of
    shared-prefix groups plus requests in none, as the groups buffer on the device says."""
    args = decode_args(query, key_cache, value_cache, block_table, seq_lens, **kw)
    lib = load()
    lib.pfd_shared_prefix_decode_grouped_fp8_e4m3.argtypes = [C.POINTER(DecodeArgs), C.c_void_p, C.c_int32, C.c_int32, C.c_int32]
    lib.pfd_shared_prefix_decode_grouped_fp8_e4m3.restype = C.c_int
    bound = args.max_seq_len if max_prefix_len is None else int(max_prefix_len)
    with torch.cuda.device(query.device):
        _check(lib.pfd_shared_prefix_decode_grouped_fp8_e4m3(C.byref(args), groups.data_ptr(), int(max_groups), bound,
                                                             int(max_suffix_len or 0)))


NOALLOC_SCRATCH_BYTES = 8 * 1024 * 1024


def paged_decode_fp8_e4m3_split_out_noalloc(query, key_cache, value_cache, block_table, seq_lens, **kw) -> None:
    """One layer-step through ``pfd_paged_decode_fp8_e4m3_split_out_noalloc``: no ``workspace``
    argument, the split-KV partials live in the fixed array inside the library, for hosts that
    have no memory left to allocate one (an engine that gave all free HBM to its KV cache) or no
    allocator at all.  Raises when the request needs more than ``NOALLOC_SCRATCH_BYTES``.  Calls
    that overlap on the GPU share that array and must be serialised by the caller."""
    kw.pop("workspace", None)
    args = decode_args(query, key_cache, value_cache, block_table, seq_lens, **kw)
    with torch.cuda.device(query.device):
        _check(load().pfd_paged_decode_fp8_e4m3_split_out_noalloc(C.byref(args)))


def merge_packed(packed: torch.Tensor, output: torch.Tensor) -> None:
    parts, batch, heads, dp2 = packed.shape
    with torch.cuda.device(packed.device):
        _check(load().pfd_merge_packed(packed.data_ptr(), parts, batch * heads, dp2 - 2, output.data_ptr(),
                                       _dtype_code(output.dtype), _stream(packed)))


def exchange_geometry(world: int, rows: int, head_dim: int) -> tuple[int, int]:
    """(bytes of one rank's exchange memory, byte offset of its control words)
    (``pfd_exchange_bytes`` / ``pfd_exchange_control_offset``)."""
    lib = load()
    for fn in (lib.pfd_exchange_bytes, lib.pfd_exchange_control_offset):
        fn.argtypes = [C.c_int32, C.c_int64, C.c_int32]
        fn.restype = C.c_int64
    total = int(lib.pfd_exchange_bytes(world, rows, head_dim))
    if total < 0:
        raise RuntimeError(lib.pfd_last_error().decode())
    return total, int(lib.pfd_exchange_control_offset(world, rows, head_dim))


def exchange_alloc(nbytes: int) -> tuple[int, bytes]:
    """``pfd_exchange_alloc`` on the current device: (device pointer, 64-byte IPC handle)."""
    lib = load()
    lib.pfd_exchange_alloc.argtypes = [C.c_int64, C.POINTER(C.c_void_p), C.POINTER(IpcHandle)]
    lib.pfd_exchange_alloc.restype = C.c_int
    ptr, handle = C.c_void_p(), IpcHandle()
    _check(lib.pfd_exchange_alloc(int(nbytes), C.byref(ptr), C.byref(handle)))
    return int(ptr.value), bytes(handle.bytes)


def exchange_open(handle: bytes) -> int:
    """``pfd_exchange_open``: map another process's exchange memory; returns the peer pointer."""
    lib = load()
    lib.pfd_exchange_open.argtypes = [C.POINTER(IpcHandle), C.POINTER(C.c_void_p)]
    lib.pfd_exchange_open.restype = C.c_int
    h = IpcHandle()
    C.memmove(h.bytes, handle, 64)
    ptr = C.c_void_p()
    _check(lib.pfd_exchange_open(C.byref(h), C.byref(ptr)))
    return int(ptr.value)


def exchange_close(ptr: int) -> None:
    lib = load()
    lib.pfd_exchange_close.argtypes = [C.c_void_p]
    lib.pfd_exchange_close.restype = C.c_int
    _check(lib.pfd_exchange_close(C.c_void_p(ptr)))


def exchange_free(ptr: int) -> None:
    lib = load()
    lib.pfd_exchange_free.argtypes = [C.c_void_p]
    lib.pfd_exchange_free.restype = C.c_int
    _check(lib.pfd_exchange_free(C.c_void_p(ptr)))


def exchange_merge(exchange: Exchange, output: torch.Tensor) -> None:
    """``pfd_exchange_merge``: bounded wait, row by row, for every rank's rows of the running step,
    then the LSE merge of this rank's receive buffer into ``output [B, Hq, D]``."""
    lib = load()
    lib.pfd_exchange_merge.argtypes = [C.POINTER(Exchange), C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]
    lib.pfd_exchange_merge.restype = C.c_int
    rows = output.shape[0] * output.shape[1]
    with torch.cuda.device(output.device):
        _check(lib.pfd_exchange_merge(C.byref(exchange), rows, output.shape[2], output.data_ptr(),
                                      _dtype_code(output.dtype), _stream(output)))


def resolve_slots(block_table: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int) -> torch.Tensor:
    slots = torch.empty(block_table.shape[0], max_seq_len, dtype=torch.int64, device=block_table.device)
    with torch.cuda.device(block_table.device):
        _check(load().pfd_resolve_slots(block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
                                        block_table.shape[0], max_seq_len, slots.data_ptr(), _stream(block_table)))
    return slots


def device_status() -> int:
    """Synchronise and return (then clear) the kernels' error word; 0 means no bounded wait gave up."""
    value = C.c_int32(0)
    lib = load()
    lib.pfd_device_status.argtypes = [C.POINTER(C.c_int32)]
    lib.pfd_device_status.restype = C.c_int
    _check(lib.pfd_device_status(C.byref(value)))
    return int(value.value)


def set_suffix_form(form: int) -> None:
    """Tuning: form of the split-KV pass behind a dense prefix pass (``pfd_set_suffix_form``):
    -1 chosen per call, 0 always after that pass, 1 always beside it."""
    lib = load()
    lib.pfd_set_suffix_form.argtypes = [C.c_int32]
    lib.pfd_set_suffix_form.restype = C.c_int
    _check(lib.pfd_set_suffix_form(int(form)))


def set_wait_limit_ns(limit_ns: int) -> None:
    """How long a device-side wait may last before it gives up and sets the error word (``pfd_set_wait_limit_ns``)."""
    lib = load()
    lib.pfd_set_wait_limit_ns.argtypes = [C.c_uint64]
    lib.pfd_set_wait_limit_ns.restype = C.c_int
    _check(lib.pfd_set_wait_limit_ns(int(limit_ns)))


def selftest_bounded_wait(limit_ns: int) -> int:
    """Run the bounded-wait self-test kernel; returns the nanoseconds the wait lasted on the device.
    ``device_status()`` reads 1 afterwards."""
    lib = load()
    lib.pfd_selftest_bounded_wait.argtypes = [C.c_uint64, C.POINTER(C.c_uint64), C.c_void_p]
    lib.pfd_selftest_bounded_wait.restype = C.c_int
    waited = C.c_uint64(0)
    _check(lib.pfd_selftest_bounded_wait(int(limit_ns), C.byref(waited), torch.cuda.current_stream().cuda_stream))
    return int(waited.value)


PATH_NAMES = {0: "none", 1: "fixed-split grid (plain loads) + merge", 2: "fixed-split grid (TMA) + merge",
              3: "balanced persistent kernel + merge", 4: "balanced persistent kernel (16-bit caches) + merge",
              5: "balanced persistent kernel alone (pieces combined inside, one launch)",
              6: "balanced persistent kernel alone (16-bit caches, one launch)"}


def balanced_workspace_rows(num_q_heads: int, num_kv_heads: int) -> int:
    """Rows ``B * Hq * splits`` the workspace needs for the balanced persistent kernel on the current device."""
    lib = load()
    lib.pfd_balanced_workspace_rows.argtypes = [C.c_int32, C.c_int32]
    lib.pfd_balanced_workspace_rows.restype = C.c_int64
    rows = int(lib.pfd_balanced_workspace_rows(num_q_heads, num_kv_heads))
    if rows < 0:
        raise RuntimeError(lib.pfd_last_error().decode())
    return rows


def last_path() -> int:
    """PFD_PATH_* code of the kernels this thread's last decode call launched."""
    lib = load()
    lib.pfd_last_path.restype = C.c_int
    return int(lib.pfd_last_path())


def launch_count() -> int:
    return int(load().pfd_launch_count())
