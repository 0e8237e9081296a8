"""Version record under the reference's module name (flextrain/git_version_info_installed.py:1-5,
written there by setup.py at install time).  Here the values are computed on import, so a
source checkout and an installed copy answer alike; ``env_report`` prints the same facts."""
import os
import subprocess

import torch

from . import __version__ as _base


def _git(*args) -> str:
    try:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        out = subprocess.run(["git", "-C", root, *args], capture_output=True, text=True, timeout=5)
        return out.stdout.strip() if out.returncode == 0 and out.stdout.strip() else "unknown"
    except (OSError, subprocess.SubprocessError):
        return "unknown"


git_hash = _git("rev-parse", "--short", "HEAD")
git_branch = _git("rev-parse", "--abbrev-ref", "HEAD")
version = f"{_base}+{git_hash}"
accelerator_name = "cuda"
_nccl = torch.cuda.nccl.version() if torch.cuda.is_available() else None
torch_info = {"version": ".".join(torch.__version__.split(".")[:2]),
              "bf16_support": bool(torch.cuda.is_available() and torch.cuda.is_bf16_supported()),
              "cuda_version": torch.version.cuda or "0.0",
              "nccl_version": ".".join(str(x) for x in _nccl[:2]) if _nccl else "0.0"}
