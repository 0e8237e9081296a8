"""Fused collective kernels across real GPUs (needs >= 2 devices on the box).
Each case runs as child processes, one per GPU, over NCCL; NVLS is switched off
and the kernels use plain peer loads, so a failing rank cannot fault its peers."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


_PORTS = {"n": 0}


def _next_port():
    """A different rendezvous port for every launch of this test process."""
    _PORTS["n"] += 1
    return 29400 + (os.getpid() * 7 + _PORTS["n"] * 13) % 1500


def _launch(case, nproc, extra_env=None):
    if case == "engine":
        return _launch_engine(nproc)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_next_port()),
           os.path.join(HERE, "_multi_gpu_worker.py"), case]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    if proc.returncode != 0:
        # the ranks' own tracebacks come before the launcher's summary: show the lines that name an error
        lines = (proc.stdout + proc.stderr).splitlines()
        named = [ln for ln in lines if "Error" in ln or "assert" in ln.lower() or "rank" in ln.lower()][:60]
        raise AssertionError("\n".join(named) + "\n--- tail ---\n" + proc.stderr[-2500:])


def _launch_engine(nproc):
    """The tiny Llama through the engine with the library collectives and with the fused
    kernels (two launches); the loss trajectories must agree."""
    import json
    import tempfile
    got = {}
    with tempfile.TemporaryDirectory() as d:
        for mode in ("engine_nccl", "engine_fused"):
            path = os.path.join(d, mode + ".json")
            _launch(mode, nproc, {"FT_TEST_LOSSES": path})
            with open(path) as f:
                got[mode] = json.load(f)
    a, b = got["engine_nccl"]["losses"], got["engine_fused"]["losses"]
    assert max(abs(x - y) for x, y in zip(a, b)) < 5e-3, (a, b)


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_gpus() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("case", ["rs_adam", "engine", "ag_gemm"])
def test_two_ranks(case):
    _launch(case, 2)


@pytest.mark.skipif(_gpus() < 4, reason="needs at least 4 GPUs")
@pytest.mark.parametrize("case", ["rs_adam", "engine", "ag_gemm"])
def test_four_ranks(case):
    _launch(case, 4)


@pytest.mark.skipif(_gpus() < 8, reason="needs 8 GPUs")
@pytest.mark.parametrize("case", ["rs_adam", "engine", "ag_gemm"])
def test_eight_ranks(case):
    _launch(case, 8)
