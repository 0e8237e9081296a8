"""Module path of the reference's NVMe-engine builder (flextrain/ops/op_builder/async_io.py:14-121).

The reference compiles its libaio extension on first use and probes for the libaio
development package.  Here the engine is part of the host library (raw io_uring system
calls with a linux-aio and a pread/pwrite fall-back, no user-space I/O library needed), so
``is_compatible`` only has to ask the running kernel which of the three it grants.
"""
from . import AsyncIOBuilder

__all__ = ["AsyncIOBuilder"]
