from __future__ import annotations

import json

from tpu_cake_b200 import cli


def test_verify_schedule_and_render(capsys):
    assert cli.main(["verify-schedule", "--mesh-size", "8", "--m", "128", "--k", "1024", "--n", "1024"]) == 0
    hashes = json.loads(capsys.readouterr().out)
    assert len(hashes["distributed_sha256"]) == 64 and len(hashes["physical_sha256"]) == 64
    assert cli.main(["render-workload", "--physical"]) == 0
    assert '"tpu_schedule.collective"' in capsys.readouterr().out


def test_estimate_large_configuration(capsys):
    assert cli.main(["estimate", "--mesh-size", "8", "--m", "8192", "--k", "16384", "--n", "8192", "--scatter-dimension", "M"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["operations_per_device"] == 2 * 8192 * 2048 * 8192 and report["limiting_resource"] == "compute"
