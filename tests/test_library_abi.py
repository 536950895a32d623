"""The shared libraries build without a GPU, load, and export what include/*.h declares."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include/paged_fp8_decode.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pfd_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_functions()
    for required in ("pfd_paged_decode_fp8_e4m3_split_out", "pfd_merge_packed", "pfd_resolve_slots", "pfd_last_error"):
        assert required in names


def test_cabi_library_exports_every_declared_symbol(built_libs):
    lib = ctypes.CDLL(str(built_libs[0]))
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_ctypes_struct_matches_header_size(built_libs, tmp_path):
    """sizeof(pfd_decode_args) as compiled by the C compiler == ctypes mirror."""
    import subprocess

    from single_gpu_inference_lab_b200 import cabi

    src = tmp_path / "sz.c"
    src.write_text('#include "paged_fp8_decode.h"\n#include <stdio.h>\nint main(void){printf("%zu", sizeof(pfd_decode_args));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    size = int(subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout)
    assert size == ctypes.sizeof(cabi.DecodeArgs)
    assert cabi.load().pfd_abi_version() == 4


def test_argument_errors_are_reported_without_a_gpu(built_libs):
    from single_gpu_inference_lab_b200 import cabi

    lib = cabi.load()
    assert lib.pfd_paged_decode_fp8_e4m3_split_out(None) == -1
    assert b"NULL" in lib.pfd_last_error()
    a = cabi.DecodeArgs()
    a.struct_size = 8
    assert lib.pfd_paged_decode_fp8_e4m3_split_out(ctypes.byref(a)) == -1
    assert b"size mismatch" in lib.pfd_last_error()
    a.struct_size = ctypes.sizeof(cabi.DecodeArgs)
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim, a.page_size = 1, 16, 2, 96, 16
    assert lib.pfd_paged_decode_fp8_e4m3_split_out(ctypes.byref(a)) == -2
    assert b"head_dim" in lib.pfd_last_error()
    a.head_dim, a.num_kv_heads = 128, 3
    assert lib.pfd_paged_decode_fp8_e4m3_split_out(ctypes.byref(a)) == -1
    assert b"divisible" in lib.pfd_last_error()
    a.num_kv_heads, a.query_dtype, a.split_size = 2, 1, 40
    assert lib.pfd_paged_decode_fp8_e4m3_split_out(ctypes.byref(a)) == -1
    assert b"split_size must be a multiple of 16" in lib.pfd_last_error()
    assert lib.pfd_launch_count() == 0
    # the tuning switch of the shared-prefix suffix pass takes -1, 0 or 1 and needs no device
    for form in (0, 1, -1):
        cabi.set_suffix_form(form)
    with pytest.raises(RuntimeError, match="form must be"):
        cabi.set_suffix_form(2)


def test_suffix_split_policy():
    """Two to four splits per request, in multiples of 64 tokens, within [64, 512]."""
    from single_gpu_inference_lab_b200.l20_shared_prefix_decode_dispatch import choose_suffix_split_size as choose

    assert choose(64, 2, 511) == 128      # the batch-64 configuration: four splits
    assert choose(256, 2, 511) == 256     # many requests: still two splits each
    assert choose(8, 2, 511) == 128       # few requests: no more than four
    assert choose(64, 2, 100) == 64 and choose(64, 2, 0) == 64
    assert choose(64, 2, 8192) == 512     # long suffixes: the reference's constant is the cap
    for batch in (1, 7, 64, 500):
        for suffix in (1, 63, 64, 65, 700, 5000):
            size = choose(batch, 4, suffix)
            assert size % 64 == 0 and 64 <= size <= 512


def test_dispatcher_library_registers_the_reference_schema(built_libs):
    from single_gpu_inference_lab_b200 import l20_paged_decode  # noqa: F401  (loads the .so)

    schema = str(torch.ops.l20_stack.paged_decode_fp8_e4m3_split_out.default._schema)
    # same schema string as integrations/vllm/cuda/l20_paged_decode.cpp:128-135
    assert "Tensor(a!) partial_output, Tensor(b!) partial_max, Tensor(c!) partial_sum, Tensor(d!) output" in schema
    assert "float k_scale, float v_scale, int max_seq_len, int split_size) -> Tensor(d!)" in schema
    for name in ("paged_decode_fp8_e4m3_split_out_v2", "merge_packed_partials", "resolve_slots"):
        assert hasattr(torch.ops.l20_stack, name)


def test_fake_impl_returns_output_alias(built_libs):
    from torch._subclasses.fake_tensor import FakeTensorMode

    from single_gpu_inference_lab_b200 import l20_paged_decode

    with FakeTensorMode():
        q = torch.empty(2, 16, 128, dtype=torch.bfloat16, device="cuda")
        kc = torch.empty(8, 16, 2, 128, dtype=torch.float8_e4m3fn, device="cuda")
        table = torch.empty(2, 4, dtype=torch.int32, device="cuda")
        lens = torch.empty(2, dtype=torch.int32, device="cuda")
        po = torch.empty(2, 16, 1, 128, device="cuda")
        pm = torch.empty(2, 16, 1, device="cuda")
        out = torch.empty_like(q)
        got = l20_paged_decode.paged_decode_fp8_e4m3_split_out(q, kc, kc, table, lens, po, pm, pm.clone(), out, 1.0, 1.0, 64, 64)
        assert got.shape == out.shape and got.dtype == out.dtype


def test_no_cpu_fallback_wrappers_reject_cpu_tensors(built_libs):
    from single_gpu_inference_lab_b200 import l20_paged_split_kv as m

    q = torch.zeros(1, 16, 128, dtype=torch.bfloat16)
    kc = torch.zeros(2, 16, 2, 128).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="requires an SM100 GPU"):
        m.l20_paged_split_kv_attention_fp8(
            q, kc, kc, torch.zeros(1, 2, dtype=torch.int32), torch.ones(1, dtype=torch.int32), k_scale=1.0, v_scale=1.0
        )
    assert m.should_use_l20_paged_fp8_split_kv(8, 4096) is False
    assert m.should_use_l20_paged_fp8_split_kv(64, 131072) is False


def test_workspace_allocator_shapes():
    from single_gpu_inference_lab_b200 import l20_paged_split_kv as m

    q = torch.zeros(3, 16, 128, dtype=torch.bfloat16)
    # head_dim 64: the reference shape, S = next_pow2(ceil(4097 / 512)) = 16
    q64 = torch.zeros(3, 14, 64, dtype=torch.bfloat16)
    po, pm, ps, out = m.allocate_l20_paged_split_kv_workspace(q64, 4097, split_size=512)
    assert po.shape == (3, 14, 16, 64) and po.dtype == torch.float32
    assert pm.shape == ps.shape == (3, 14, 16) and out.shape == q64.shape and out.dtype == q64.dtype
    # head_dim 128: at least the rows the balanced kernel wants, 2 * (8 * 148 // Hkv) * Hq
    po, pm, ps, out = m.allocate_l20_paged_split_kv_workspace(q, 4097, split_size=512, num_kv_heads=2)
    assert po.shape[:2] == (3, 16) and po.shape[3] == 128 and pm.shape == ps.shape == po.shape[:3]
    assert po.shape[2] == -(-2 * (8 * 148 // 2) * 16 // (3 * 16)) and po.shape[2] >= 16
    big = torch.zeros(256, 28, 128, dtype=torch.bfloat16)
    assert m.allocate_l20_paged_split_kv_workspace(big, 8192, split_size=512)[0].shape == (256, 28, 16, 128)
    assert m.choose_split_size(64, 2, 4096) % 64 == 0
    s = m.choose_split_size(4, 8, 131072)  # 32 long segments: one wave of 444 slots
    assert s % 64 == 0 and 8 * 4 * -(-131072 // s) <= 444 < 8 * 4 * -(-131072 // (s - 64))
    assert m.choose_split_size(4, 2, 4096, seq_lens=[512, 4096, 2000, 100]) == 128  # tiny batch: the minimum
    many = [900] * 256  # more (sequence, kv head) pairs than slots: a few waves of small items
    s = m.choose_split_size(256, 4, 8192, seq_lens=many)
    assert 128 <= s <= 2048 and s % 64 == 0


def test_missing_libraries_fail_loudly_and_the_package_never_imports_the_oracle(tmp_path, monkeypatch):
    """No CPU or eager path stands behind the operator: without its shared libraries every entry
    point raises, and no module of the package reaches for the test oracle."""
    import re
    from pathlib import Path

    from single_gpu_inference_lab_b200 import cabi, l20_paged_decode

    monkeypatch.setattr(cabi, "_lib", None)
    monkeypatch.setattr(cabi, "library_path", lambda: tmp_path / "libpaged_fp8_decode.so")
    with pytest.raises(RuntimeError, match="there is no fallback implementation"):
        cabi.load()
    with pytest.raises(RuntimeError, match="has no fallback implementation"):
        l20_paged_decode.load_library(tmp_path / "l20_paged_decode_ops.so")
    package = Path(cabi.__file__).resolve().parent
    for source in list(package.glob("*.py")) + list((package / "csrc").glob("*")):
        text = source.read_text(errors="ignore")
        assert not re.search(r"^\s*(from|import)\s+oracle\b", text, re.M), source
