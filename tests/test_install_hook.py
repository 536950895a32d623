"""The vLLM hook installer against a copy of the installed vLLM FlashInfer backend (CPU only;
mirrors what the reference pins in tests/test_install_l20_fp8_paged_decode.py: switch names,
policy call, quantised-cache gate -- plus that the patched file still compiles)."""

import ast
import importlib.util
import shutil
from pathlib import Path

import pytest

from single_gpu_inference_lab_b200 import install_l20_fp8_paged_decode as installer


def _fake_tree(tmp_path: Path) -> Path:
    spec = importlib.util.find_spec("vllm")
    if spec is None or not spec.submodule_search_locations:
        pytest.skip("vLLM is not installed")
    real = Path(list(spec.submodule_search_locations)[0]) / "v1/attention/backends/flashinfer.py"
    if not real.exists():
        pytest.skip("this vLLM has no FlashInfer backend file")
    root = tmp_path / "src"
    (root / "vllm/v1/attention/backends").mkdir(parents=True)
    (root / "vllm/v1/attention/ops").mkdir(parents=True)
    shutil.copy2(real, root / "vllm/v1/attention/backends/flashinfer.py")
    return root


def test_install_is_idempotent_compiles_and_uninstalls(tmp_path, built_libs, capsys):
    root = _fake_tree(tmp_path)
    backend = root / "vllm/v1/attention/backends/flashinfer.py"
    original = backend.read_text()
    assert installer.main(["--vllm-source-dir", str(root)]) == 0
    assert capsys.readouterr().out.strip() == str(root / "vllm")
    patched = backend.read_text()
    assert patched != original
    ast.parse(patched)  # still valid Python
    for needle in (
        "VLLM_ENABLE_L20_FP8_PAGED_DECODE",
        "VLLM_L20_FP8_PAGED_FORCE",
        "VLLM_L20_FP8_PAGED_TRACE",
        "should_use_l20_paged_fp8_split_kv",
        "l20_decode_step(",
        "l20_grouped_decode(",
        "plan=l20_step.plan",
        "workspace=l20_step.workspace",
        "l20_step: object | None = None",
        "l20_paged_split_kv_attention_fp8",
        "is_quantized_kv_cache(self.kv_cache_dtype)",
        "DeviceCapability(10, 0)",
        "l20_fp8_paged_decode_run",
        "block_tables=block_table_tensor[:num_decodes]",
        # the non-quantised sibling shares the call site
        "VLLM_ENABLE_L20_PAGED_DECODE",
        "VLLM_L20_PAGED_FORCE",
        "VLLM_L20_PAGED_TRACE",
        "l20_paged_decode_run",
        "should_use_l20_paged_split_kv",
        "l20_paged_split_kv_attention(",
        "not is_quantized_kv_cache(self.kv_cache_dtype)",
        "metadata_stable=True",
    ):
        assert needle in patched, needle
    # the stock call survives as the fallback branch, exactly once more than the DCP call
    assert patched.count("decode_wrapper.run(") == original.count("decode_wrapper.run(")
    ops = root / "vllm/v1/attention/ops"
    for name in installer.COPIED:
        assert (ops / name).exists(), name
    backup = backend.with_suffix(installer.BACKUP_SUFFIX)
    assert backup.read_text() == original
    # second run: nothing changes
    assert installer.main(["--vllm-source-dir", str(root)]) == 0
    assert backend.read_text() == patched
    assert installer.main(["--vllm-source-dir", str(root), "--uninstall"]) == 0
    assert backend.read_text() == original


def test_missing_patch_point_is_reported(tmp_path):
    with pytest.raises(RuntimeError, match="cannot find patch point: FIDecode metadata"):
        installer.patch_backend_source("import torch\nclass Other:\n    pass\n")
    with pytest.raises(RuntimeError, match="cannot find vLLM source package"):
        installer.find_vllm_package.__wrapped__ if hasattr(installer.find_vllm_package, "__wrapped__") else None
        import os

        cwd = os.getcwd()
        os.chdir(tmp_path)
        try:
            real_find = importlib.util.find_spec
            importlib.util.find_spec = lambda name: None
            installer.find_vllm_package(str(tmp_path / "nowhere"))
        finally:
            importlib.util.find_spec = real_find
            os.chdir(cwd)


def test_replace_once_semantics():
    assert installer.replace_once("a b", "b", "c", "x") == "a c"
    assert installer.replace_once("a c", "b", "c", "x") == "a c"  # already applied
    with pytest.raises(RuntimeError, match="cannot find patch point: x"):
        installer.replace_once("a", "b", "zz", "x")


def test_live_check_overlay_leaves_the_installed_package_alone(tmp_path):
    """The overlay the live engine check patches: copies where the installer writes, symlinks
    elsewhere."""
    from single_gpu_inference_lab_b200 import vllm_live_check as live

    real = tmp_path / "real/vllm"
    (real / "v1/attention/backends").mkdir(parents=True)
    (real / "v1/attention/ops").mkdir(parents=True)
    (real / "model_executor").mkdir()
    (real / "__init__.py").write_text("x = 1\n")
    (real / "v1/attention/backends/flashinfer.py").write_text("stock\n")
    (real / "v1/attention/backends/other.py").write_text("other\n")
    (real / "v1/attention/ops/common.py").write_text("common\n")
    dst = tmp_path / "overlay/vllm"
    live.overlay(real, dst, live.COPIED_PATHS)
    assert (dst / "__init__.py").is_symlink() and (dst / "model_executor").is_symlink()
    assert (dst / "v1/attention/backends/other.py").is_symlink()
    patched = dst / "v1/attention/backends/flashinfer.py"
    assert not patched.is_symlink() and not (dst / "v1/attention/ops").is_symlink()
    patched.write_text("patched\n")
    (dst / "v1/attention/ops/new.py").write_text("new\n")
    assert (real / "v1/attention/backends/flashinfer.py").read_text() == "stock\n"
    assert not (real / "v1/attention/ops/new.py").exists()


def test_rope_hook_installs_compiles_and_uninstalls(tmp_path, built_libs, capsys):
    """The producer hook at the reference's call site (integrations/vllm/install_l20_rope_kv.py):
    config guard relaxed for CUDA, the two backend methods added with the sm_100 / FP8 gate."""
    from single_gpu_inference_lab_b200 import install_l20_rope_kv as rope_installer

    root = _fake_tree(tmp_path)
    spec = importlib.util.find_spec("vllm")
    real_config = Path(list(spec.submodule_search_locations)[0]) / "config/compilation.py"
    if not real_config.exists():
        pytest.skip("this vLLM has no config/compilation.py")
    (root / "vllm/config").mkdir(parents=True)
    shutil.copy2(real_config, root / "vllm/config/compilation.py")
    backend = root / "vllm/v1/attention/backends/flashinfer.py"
    config = root / "vllm/config/compilation.py"
    originals = backend.read_text(), config.read_text()
    assert rope_installer.main(["--vllm-source-dir", str(root)]) == 0
    capsys.readouterr()
    patched_backend, patched_config = backend.read_text(), config.read_text()
    ast.parse(patched_backend)
    ast.parse(patched_config)
    for needle in (
        "from vllm.v1.attention.ops.l20_rope_kv import l20_rope_and_cache",
        "def fused_rope_kvcache_supported(self):",
        "capability.to_int() == 100",
        "is_quantized_kv_cache(self.kv_cache_dtype)",
        "def do_rope_and_kv_cache_update(",
        "k_scale=layer._k_scale if l20_fp8 else None",
    ):
        assert needle in patched_backend, needle
    assert "and not current_platform.is_cuda()" in patched_config
    for name in rope_installer.COPIED:
        assert (root / "vllm/v1/attention/ops" / name).exists(), name
    assert rope_installer.main(["--vllm-source-dir", str(root)]) == 0  # idempotent
    assert backend.read_text() == patched_backend and config.read_text() == patched_config
    # both hooks together: the decode hook patches the same backend file
    assert installer.main(["--vllm-source-dir", str(root)]) == 0
    ast.parse(backend.read_text())
    assert rope_installer.main(["--vllm-source-dir", str(root), "--uninstall"]) == 0
    assert (backend.read_text(), config.read_text()) == originals
