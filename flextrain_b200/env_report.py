"""Environment and build report: ``python -m flextrain_b200.env_report``.

Parity: the reference records the torch / CUDA / NCCL versions it was installed
against (setup.py:120-171, flextrain/git_version_info_installed.py:1-5) and each
op builder answers ``is_compatible`` (flextrain/ops/op_builder/builder.py).  Here
the same facts are gathered at run time into one dict: package and library
versions, compilers, state of the two native libraries (built, current with the
sources), host SIMD level, the NVMe engine's backend and, when a GPU is present,
its name, compute capability and memory.
"""
from __future__ import annotations

import json
import os
import platform
import sys
from typing import Any, Dict


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def _native_state() -> Dict[str, Any]:
    from .ops.op_builder import ALL_OPS
    from .ops.op_builder.builder import BuildError
    out = {}
    for name, cls in ALL_OPS.items():
        b = cls()
        entry = {"path": b.lib_path, "built": os.path.exists(b.lib_path), "current": b.is_current(),
                 "sources": len(b.sources)}
        try:
            entry["compiler"] = b.compiler()
        except BuildError as exc:
            entry["compiler"] = None
            entry["compiler_error"] = str(exc).splitlines()[0]
        out[name] = entry
    return out


def _nvme_backend() -> str:
    try:
        from .memory.nvme_swapper import NVMeEngine
        eng = NVMeEngine(queue_depth=4, threads=1)
        try:
            return eng.kind
        finally:
            eng.close()
    except Exception as exc:              # library not built or kernel refuses every backend
        return f"unavailable ({type(exc).__name__})"


def collect(probe_nvme: bool = True) -> Dict[str, Any]:
    """Everything the report prints, as a JSON-serialisable dict."""
    import torch

    from . import __version__
    from .ops.op_builder import cuda_home, nvcc_path
    flags = _cpu_flags()
    report: Dict[str, Any] = {
        "flextrain_b200": __version__,
        "python": platform.python_version(),
        "platform": platform.platform(),
        "torch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "nccl": None,
        "cuda_home": cuda_home(),
        "nvcc": nvcc_path(),
        "target_arch": "sm_100a",
        "host_simd": "avx512" if "avx512f" in flags else ("avx2" if "avx2" in flags else "scalar"),
        "host_cores": os.cpu_count(),
        "native": _native_state(),
        "gpus": [],
    }
    try:
        report["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception:
        pass
    if probe_nvme:
        report["nvme_backend"] = _nvme_backend()
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            report["gpus"].append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}",
                                   "sms": p.multi_processor_count,
                                   "memory_gib": round(p.total_memory / 2 ** 30, 1),
                                   "supported": (p.major, p.minor) == (10, 0)})
    return report


def format_report(report: Dict[str, Any]) -> str:
    lines = ["flextrain_b200 environment", "-" * 60]

    def row(key, value):
        lines.append(f"{key} {'.' * max(2, 28 - len(key))} {value}")

    for key in ("flextrain_b200", "python", "platform", "torch", "torch_cuda", "nccl", "cuda_home",
                "nvcc", "target_arch", "host_simd", "host_cores", "nvme_backend"):
        if key in report:
            row(key, report[key])
    for name, st in report["native"].items():
        state = "current" if st["current"] else ("stale" if st["built"] else "not built")
        row(f"lib{name}.so", f"{state}  ({st['sources']} sources, compiler {st['compiler']})")
    if not report["gpus"]:
        row("gpus", "none visible")
    for g in report["gpus"]:
        ok = "" if g["supported"] else "  [not sm_100: kernels will not load]"
        row(f"gpu {g['index']}", f"{g['name']} cc {g['capability']} {g['sms']} SMs {g['memory_gib']} GiB{ok}")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    report = collect(probe_nvme="--no-nvme" not in argv)
    print(json.dumps(report, indent=1) if "--json" in argv else format_report(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
