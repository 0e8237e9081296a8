"""In-tree native build: every shared object is compiled next to the package
with an explicit compiler command and loaded through ctypes.

Capability parity: flextrain/ops/op_builder/builder.py:1-860 (JIT builders for
the CPU Adam and async-IO ops).  Differences: there is one target GPU
(``-gencode arch=compute_100a,code=sm_100a``), objects are cached by a content
signature instead of ninja timestamps, the products live inside the package
directory so they travel with a source snapshot, and the C ABI needs no
PyTorch headers.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence

PKG_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REPO_ROOT = os.path.dirname(PKG_ROOT)
CSRC = os.path.join(REPO_ROOT, "csrc")
NATIVE_DIR = os.path.join(PKG_ROOT, "_native")

SM100A_GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
_LOCK = threading.Lock()
_LOADED: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _which(name: str, extra: Sequence[str] = ()) -> Optional[str]:
    found = shutil.which(name)
    if found:
        return found
    for d in extra:
        cand = os.path.join(d, name)
        if os.path.exists(cand):
            return cand
    return None


def host_cxx() -> str:
    """The system g++ (it ships libgomp); ``FLEXTRAIN_CXX`` overrides.  The
    generic ``CXX`` variable is ignored on purpose: toolchains that lack an
    OpenMP runtime are commonly exported through it."""
    if os.environ.get("FLEXTRAIN_CXX"):
        cxx = _which(os.environ["FLEXTRAIN_CXX"])
    else:
        cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else _which("g++")
    if not cxx:
        raise BuildError("no C++ compiler found (g++)")
    return cxx


def nvcc_path() -> Optional[str]:
    return _which("nvcc", ["/usr/local/cuda/bin"])


def cuda_home() -> Optional[str]:
    n = nvcc_path()
    return os.path.dirname(os.path.dirname(os.path.realpath(n))) if n else None


class MissingCUDAException(BuildError):
    pass


class CUDAMismatchException(BuildError):
    pass


DEFAULT_COMPUTE_CAPABILITIES = "10.0a"
MIN_CUDA_FOR_SM100A = (12, 8)


def installed_cuda_version():
    """(major, minor) of the nvcc that would build the kernels
    (flextrain/ops/op_builder/builder.py:50-64)."""
    nvcc = nvcc_path()
    if not nvcc:
        raise MissingCUDAException("nvcc not found: the CUDA kernels cannot be compiled")
    words = subprocess.check_output([nvcc, "-V"], universal_newlines=True).split()
    release = words[words.index("release") + 1].rstrip(",").split(".")
    return int(release[0]), int(release[1])


def get_default_compute_capabilities() -> str:
    """The reference builds for a list of architectures (6.0 ... 8.6,
    flextrain/ops/op_builder/builder.py:67-78); this package has exactly one target."""
    return DEFAULT_COMPUTE_CAPABILITIES


def assert_no_cuda_mismatch(name: str = "") -> bool:
    """The reference refuses an nvcc whose version differs from the CUDA PyTorch was built
    with, because its ops link against PyTorch (flextrain/ops/op_builder/builder.py:92-126).
    The libraries here have a C ABI and link neither PyTorch nor its CUDA runtime, so the only
    hard requirement is an nvcc that knows sm_100a."""
    have = installed_cuda_version()
    if have < MIN_CUDA_FOR_SM100A:
        raise CUDAMismatchException(
            f"{name or 'flextrain_b200'}: nvcc {have[0]}.{have[1]} cannot compile for sm_100a "
            f"(needs {MIN_CUDA_FOR_SM100A[0]}.{MIN_CUDA_FOR_SM100A[1]} or newer)")
    return True


class OpBuilder:
    """Compiles ``sources`` (relative to ``csrc/``) into ``_native/lib<name>.so``."""

    kind = "host"

    def __init__(self, name: str, sources: Sequence[str], extra_flags: Sequence[str] = (),
                 link_flags: Sequence[str] = (), headers: Sequence[str] = ()):
        self.name = name
        self.sources = [os.path.join(CSRC, s) for s in sources]
        self.headers = [os.path.join(CSRC, h) for h in headers]
        self.extra_flags = list(extra_flags)
        self.link_flags = list(link_flags)

    # ------------------------------------------------------------ commands
    def compiler(self) -> str:
        return host_cxx()

    def compile_cmd(self, src: str, obj: str) -> List[str]:
        return [self.compiler(), "-O3", "-std=c++17", "-fPIC", "-fopenmp", "-mavx2", "-mfma",
                "-mf16c", "-ffp-contract=off", "-Wall", "-Wno-unknown-pragmas",
                f"-I{CSRC}", *self.extra_flags, "-c", src, "-o", obj]

    def link_cmd(self, objs: Sequence[str], out: str) -> List[str]:
        return [self.compiler(), "-shared", "-fopenmp", *objs, "-o", out, "-lpthread",
                *self.link_flags]

    # ----------------------------------------------------------- signature
    @property
    def lib_path(self) -> str:
        return os.path.join(NATIVE_DIR, f"lib{self.name}.so")

    def signature(self) -> str:
        # paths enter relative to the repository so that a copy of the tree made
        # elsewhere (another checkout, a snapshot on a GPU box) still matches
        h = hashlib.sha256()
        for path in sorted(self.sources + self.headers):
            with open(path, "rb") as f:
                h.update(os.path.relpath(path, REPO_ROOT).encode())
                h.update(f.read())
        flags = " ".join(self.compile_cmd("S", "O") + self.link_cmd(["O"], "L"))
        h.update(flags.replace(REPO_ROOT, "<repo>").encode())
        return h.hexdigest()

    def is_current(self) -> bool:
        sig_path = self.lib_path + ".sig"
        if not (os.path.exists(self.lib_path) and os.path.exists(sig_path)):
            return False
        try:
            with open(sig_path) as f:
                return f.read().strip() == self.signature()
        except (OSError, BuildError):
            return False

    # --------------------------------------------------------------- build
    def _run(self, cmd: Sequence[str]):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"command failed ({proc.returncode}): {' '.join(cmd)}\n"
                             f"{proc.stdout}\n{proc.stderr}")
        return proc

    def build(self, force: bool = False, verbose: bool = False) -> str:
        import fcntl
        os.makedirs(NATIVE_DIR, exist_ok=True)
        # one builder at a time per tree: ranks of one job start together
        with _LOCK, open(os.path.join(NATIVE_DIR, f".{self.name}.lock"), "w") as lock_file:
            fcntl.flock(lock_file, fcntl.LOCK_EX)
            if not force and self.is_current():
                return self.lib_path
            obj_dir = os.path.join(NATIVE_DIR, "obj", self.name)
            os.makedirs(obj_dir, exist_ok=True)
            objs = [os.path.join(obj_dir, os.path.basename(s) + ".o") for s in self.sources]
            jobs = min(len(self.sources), max(1, (os.cpu_count() or 2) // 2))
            with ThreadPoolExecutor(jobs) as pool:
                results = list(pool.map(lambda so: self._run(self.compile_cmd(*so)),
                                        zip(self.sources, objs)))
            if verbose:
                for r in results:
                    sys.stderr.write(r.stderr)
            tmp = self.lib_path + f".tmp{os.getpid()}"
            self._run(self.link_cmd(objs, tmp))
            os.replace(tmp, self.lib_path)
            with open(self.lib_path + ".sig", "w") as f:
                f.write(self.signature())
            return self.lib_path

    def load(self, build_if_needed: bool = True) -> ctypes.CDLL:
        if self.name in _LOADED:
            return _LOADED[self.name]
        if not self.is_current():
            can_build = True
            try:
                self.compiler()
            except BuildError:
                can_build = False
            if build_if_needed and can_build:
                self.build()
            elif not os.path.exists(self.lib_path):
                raise BuildError(f"{self.lib_path} is missing and cannot be built here")
        lib = ctypes.CDLL(self.lib_path, mode=ctypes.RTLD_GLOBAL)
        _LOADED[self.name] = lib
        return lib


class CPUOpBuilder(OpBuilder):
    """Host-only library: g++ with OpenMP, no CUDA toolchain needed
    (flextrain/ops/op_builder/builder.py:620-642)."""


class CUDAOpBuilder(OpBuilder):
    """nvcc build for sm_100a only."""

    kind = "cuda"

    def compiler(self) -> str:
        n = nvcc_path()
        if not n:
            raise BuildError("nvcc not found")
        return n

    def compile_cmd(self, src: str, obj: str) -> List[str]:
        return [self.compiler(), "-ccbin", host_cxx(), *SM100A_GENCODE, "-O3", "-std=c++17",
                "-lineinfo",
                "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fopenmp",
                f"-I{CSRC}", *self.extra_flags, "-c", src, "-o", obj]

    def link_cmd(self, objs: Sequence[str], out: str) -> List[str]:
        return [self.compiler(), "-ccbin", host_cxx(), *SM100A_GENCODE, "-shared", "-Xcompiler",
                "-fPIC", "-Xcompiler", "-fopenmp", *objs, "-o", out,
                "-lpthread", "-ldl", *self.link_flags]
