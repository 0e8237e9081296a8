"""Builders for the native libraries of the package.

Capability parity: flextrain/ops/op_builder/__init__.py, cpu_adam.py, async_io.py.
``HostOpsBuilder`` holds the AVX-512 Adam, the NVMe engine and host copies;
``CudaOpsBuilder`` holds every sm_100a kernel plus the pinned pool and the
peer-memory plumbing.
"""
import glob
import os

from .builder import (BuildError, CPUOpBuilder, CSRC, CUDAOpBuilder, NATIVE_DIR, OpBuilder, cuda_home,
                      nvcc_path)


def _rel(pattern):
    return sorted(os.path.relpath(p, CSRC) for p in glob.glob(os.path.join(CSRC, pattern)))


class HostOpsBuilder(CPUOpBuilder):
    def __init__(self):
        super().__init__("ft_host", _rel("host/*.cpp"), headers=_rel("host/*.h"))


class CPUAdamBuilder(HostOpsBuilder):
    """The host library exports the Adam entry points (``ft_adam_*``)."""


class AsyncIOBuilder(HostOpsBuilder):
    """The host library exports the NVMe engine entry points (``ft_nvme_*``)."""


class CudaOpsBuilder(CUDAOpBuilder):
    def __init__(self):
        super().__init__("ft_cuda", _rel("kernels/*.cu") + _rel("comm/*.cu"),
                         headers=_rel("kernels/*.cuh") + _rel("comm/*.cuh") + _rel("kernels/*.h"))


ALL_OPS = {"ft_host": HostOpsBuilder, "ft_cuda": CudaOpsBuilder}


def build_all(force=False, verbose=False):
    paths = []
    for cls in ALL_OPS.values():
        paths.append(cls().build(force=force, verbose=verbose))
    return paths
