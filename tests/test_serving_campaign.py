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
