"""Capacity-plan command line (no GPU, no run)."""
import json

from flextrain_b200 import plan_cli


def test_plan_for_70b_on_eight_gpus(capsys, tmp_path):
    out_file = tmp_path / "cfg.json"
    rc = plan_cli.main(["--model", "llama:llama3-70b", "--gpus", "8", "--hbm-gib", "176", "--dram-gib", "900",
                        "--emit", str(out_file)])
    assert rc == 0
    table = json.loads(capsys.readouterr().out)
    assert 900 < table["state_gib_total"] < 940
    split = table["split_ratio"]
    assert split["parameter"] == [1.0, 0.0] and split["optimizer"][0] > 0.9
    total = table["per_rank_gib"]["total"]
    assert total["hbm"] + table["working_set_gib"] < 176 and total["nvme"] < 1e-6
    cfg = json.load(open(out_file))
    assert cfg["batch_size"] == 16 and cfg["split_ratio"] == split
    from flextrain_b200.config import FlexTrainConfig
    FlexTrainConfig(cfg)                                   # the emitted file is a valid config


def test_plan_reports_what_does_not_fit(capsys):
    rc = plan_cli.main(["--model", "gpt:gpt3-175b", "--gpus", "8", "--hbm-gib", "176", "--dram-gib", "900"])
    assert rc == 1
    assert json.loads(capsys.readouterr().out)["split_ratio"] is None
    rc = plan_cli.main(["--model", "gpt:gpt3-175b", "--gpus", "8", "--hbm-gib", "176", "--dram-gib", "900",
                        "--nvme-gib", "4000"])
    assert rc == 0
    table = json.loads(capsys.readouterr().out)
    assert table["per_rank_gib"]["total"]["nvme"] > 10
