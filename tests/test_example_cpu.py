"""The example training script end to end on CPU: a run that is saved and resumed
continues exactly like an uninterrupted one; two ranks under the launcher; the
sample config parses."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "examples", "pretrain.py")


def _run(args, cwd, launcher=None, timeout=600):
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    env["OMP_NUM_THREADS"] = "2"
    cmd = [sys.executable] + (launcher or []) + [SCRIPT] + args
    proc = subprocess.run(cmd, cwd=cwd, env=env, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("{")][-1]
    return json.loads(line)


def test_save_resume_matches_uninterrupted_run(tmp_path):
    from flextrain_b200.data import TokenFile
    rng = np.random.default_rng(0)
    data = str(tmp_path / "tokens.u16")
    TokenFile.write(data, rng.integers(0, 1024, size=20000))
    common = ["--model", "llama:tiny", "--data", data, "--micro-batch-size", "1"]
    mfile = str(tmp_path / "metrics.jsonl")
    whole = _run(common + ["--steps", "5", "--metrics-file", mfile], str(tmp_path))
    rows = [json.loads(l) for l in open(mfile)]
    assert [r["step"] for r in rows] == [1, 2, 3, 4, 5] and [r["loss"] for r in rows] == whole["losses"]
    assert all(r["tokens_per_s"] > 0 for r in rows)
    ck = str(tmp_path / "ck")
    first = _run(common + ["--steps", "3", "--save-dir", ck], str(tmp_path))
    # one state file per rank, one file per unit (the checkpoint is written unit by unit)
    assert sorted(os.listdir(ck)) == ["rank0_data.json", "rank0_state.pt"] + [f"rank0_unit{u}.pt" for u in range(4)]
    second = _run(common + ["--steps", "2", "--resume", ck], str(tmp_path))
    assert second["steps_done"] == 5
    assert first["losses"] + second["losses"] == whole["losses"]


def test_two_ranks_gpt_under_the_launcher(tmp_path):
    port = 23000 + os.getpid() % 2000
    out = _run(["--model", "gpt:tiny", "--steps", "2", "--micro-batch-size", "1",
                "--micro-batches-per-rank", "1"], str(tmp_path),
               launcher=["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                         "--master-addr", "127.0.0.1", "--master-port", str(port)])
    assert out["steps_done"] == 2 and abs(out["first_loss"] - np.log(1024)) < 0.3


def test_sample_config_parses(fresh_runtime):
    from flextrain_b200.config import get_flextrain_config, init_flextrain_config
    with open(os.path.join(ROOT, "examples", "llama3_70b_8gpu.json")) as f:
        init_flextrain_config(json.load(f), log=False)
    cfg = get_flextrain_config()
    assert cfg.batch_size == 16 and cfg.micro_batch_size == 2
    assert cfg.split_ratio.optimizer[0] == 0.92


def test_custom_model_example_learns_and_offload_changes_nothing(tmp_path):
    script = os.path.join(ROOT, "examples", "custom_model.py")
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    env["OMP_NUM_THREADS"] = "2"

    def last_line(extra):
        proc = subprocess.run([sys.executable, script, "--device", "cpu", "--steps", "30"] + extra,
                              cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
        return [l for l in proc.stdout.splitlines() if l.startswith("first loss")][-1]

    resident = last_line([])
    offloaded = last_line(["--offload"])
    first, last = float(resident.split()[2]), float(resident.split()[5])
    assert last < 0.3 * first
    assert resident == offloaded                       # same numbers to the printed precision
