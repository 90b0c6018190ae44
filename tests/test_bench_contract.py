"""The benchmark and entry-point contracts that can be checked without a GPU."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(torch.cuda.is_available(), reason="the no-GPU answer is only printed on a machine without one")
@pytest.mark.parametrize("impl", ["ours", "reference"])
def test_bench_answers_in_one_json_line_without_a_gpu(impl):
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", impl, "--steps", "1", "--warmup", "1"], cwd=ROOT,
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-500:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == impl and "no CUDA device" in line["unavailable"]


def test_bench_arguments_and_configs():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        args = bench.parse_args()
    finally:
        sys.argv = argv
    assert args.gpus == 1 and args.impl == "ours" and args.warmup >= 3 and args.steps >= 1  # the no-flag defaults
    assert {"cfg3", "cfg4", "cfg5", "cfg4-depth"} <= set(bench.CONFIGS)


def test_entry_point_module_has_build_and_smoke():
    spec = importlib.util.spec_from_file_location("graft_entry", ROOT / "__graft_entry__.py")
    entry = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(entry)
    assert callable(entry.build) and callable(entry.smoke)


def test_package_front_door_lists_and_dispatches_commands(capsys, monkeypatch):
    import importlib

    from lbi_b200 import __main__ as front

    assert front.main([]) == 0 and "train" in capsys.readouterr().out
    assert front.main(["nope"]) == 2
    for name, (module, _) in front.COMMANDS.items():
        assert callable(getattr(importlib.import_module(module), "main")), name
    monkeypatch.setenv("LBI_LAUNCH_QUIET", "1")
    assert front.main(["launch", "dense", "--dry-run"]) == 0
    assert "--variants dense" in capsys.readouterr().out
