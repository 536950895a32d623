"""Host logic of the serving campaign (CPU): the grid, the medians and the summary file, with
the engine runs replaced by canned results."""

import json
import subprocess
from types import SimpleNamespace

from single_gpu_inference_lab_b200 import serving_campaign as campaign


def test_dummy_mode_runs_the_grid_and_writes_medians(tmp_path, monkeypatch, capsys):
    calls = []

    def fake_run(cmd, **kw):
        calls.append(cmd)
        batch = int(cmd[cmd.index("--batch") + 1])
        run = len([c for c in calls if c[c.index("--batch") + 1] == str(batch) and c[c.index("--prompt-len") + 1] == cmd[cmd.index("--prompt-len") + 1]])
        line = json.dumps({"stock_ms_per_decode_step": 10.0 + run, "hook_ms_per_decode_step": 5.0 + run, "batch": batch})
        return SimpleNamespace(returncode=0, stdout="noise\n" + line + "\n", stderr="")

    monkeypatch.setattr(subprocess, "run", fake_run)
    rc = campaign.main(["dummy", "--output-dir", str(tmp_path), "--concurrencies", "8 64", "--inputs", "1024,4096", "--runs", "3",
                        "--cuda-graphs", "--layers", "4"])
    assert rc == 0
    assert len(calls) == 2 * 2 * 3 and all("--cuda-graphs" in c and "--ab" in c for c in calls)
    summary = json.loads((tmp_path / "summary.json").read_text())
    assert summary["engine_mode"] == "cuda graphs" and set(summary["cells"]) == {"c8-i1024", "c8-i4096", "c64-i1024", "c64-i4096"}
    cell = summary["cells"]["c64-i4096"]
    assert cell["stock_ms_per_decode_step"] == 12.0 and cell["hook_ms_per_decode_step"] == 7.0 and cell["runs"] == 3
    assert cell["hook_over_stock"] == round(7.0 / 12.0, 4)
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1]) == summary


def test_list_arguments():
    assert campaign._ints("8 16,32") == [8, 16, 32]


def test_dummy_model_directory_has_an_exact_tokenizer(tmp_path):
    """``serve --dummy-weights``: the directory loads offline and decode / encode is the identity on
    ids, which is what the random dataset of the serving benchmark relies on for its prompt lengths."""
    import random

    from transformers import AutoTokenizer

    path = campaign.write_dummy_model(tmp_path / "model", layers=2, q_heads=4, kv_heads=2, intermediate=256, vocab=5000)
    config = json.loads((path / "config.json").read_text())
    assert config["num_hidden_layers"] == 2 and config["vocab_size"] == 5000 and config["hidden_size"] == 512
    tok = AutoTokenizer.from_pretrained(str(path))
    assert len(tok) == 5000 and tok.bos_token_id == config["bos_token_id"] and tok.eos_token_id == config["eos_token_id"]
    rng = random.Random(0)
    ids = [rng.randrange(4, 5000) for _ in range(3000)]
    assert tok.encode(tok.decode(ids), add_special_tokens=False) == ids


def test_serve_mode_with_dummy_weights_builds_the_model_and_the_server_command(tmp_path, monkeypatch):
    seen = {}

    def fake_arm(args, src, out, hook_on):
        seen[hook_on] = args.model
        assert args.dummy_weights
        return {"cells": {"c8-i4096": {"median_itl_ms": 3.0 if hook_on else 4.0}}, "hook_hits": 7 if hook_on else 0}

    monkeypatch.setattr(campaign, "build_overlay", lambda work: work / "vllm_src")
    monkeypatch.setattr(campaign, "run_serve_arm", fake_arm)
    rc = campaign.main(["serve", "--output-dir", str(tmp_path), "--dummy-weights", "--layers", "2", "--q-heads", "4", "--intermediate", "256"])
    assert rc == 0
    summary = json.loads((tmp_path / "summary.json").read_text())
    assert summary["weights"] == "dummy" and summary["cells"]["c8-i4096"]["median_itl_ratio"] == 0.75 and summary["hook_hits"] == 7
    assert seen[True] == seen[False] == str(tmp_path / "model") and (tmp_path / "model" / "tokenizer.json").exists()
