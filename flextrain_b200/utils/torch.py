"""PyTorch version helpers under the reference's module path (flextrain/utils/torch.py:1-63).

The reference selects between the old and new names of the flat collectives and asserts
at import time that the coalescing manager exists.  This package needs PyTorch 2.x, where
``all_gather_into_tensor`` / ``reduce_scatter_tensor`` always exist, so the getters return
them directly and nothing is asserted on import; the private ``_..._base`` names are still
tried last for callers that run this module against an older build.
"""
from __future__ import annotations

import re
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as tdist


def _major_minor(version: str) -> Tuple[int, int]:
    m = re.match(r"\s*(\d+)\.(\d+)", version)
    if not m:
        raise ValueError(f"not a version: {version!r}")
    return int(m.group(1)), int(m.group(2))


TORCH_MAJOR, TORCH_MINOR = _major_minor(torch.__version__)


def torch_version_eq(cmp_version: str) -> bool:
    return (TORCH_MAJOR, TORCH_MINOR) == _major_minor(cmp_version)


def torch_version_ge(cmp_version: str) -> bool:
    return (TORCH_MAJOR, TORCH_MINOR) >= _major_minor(cmp_version)


def _first(*names: str) -> Optional[Callable]:
    for name in names:
        fn = getattr(tdist, name, None)
        if fn is not None:
            return fn
    return None


def get_all_gather_function() -> Optional[Callable]:
    return _first("all_gather_into_tensor", "_all_gather_base")


def get_reduce_scatter_function() -> Optional[Callable]:
    return _first("reduce_scatter_tensor", "_reduce_scatter_base")


def get_coalescing_manager(group, device, reqs=None, async_op: bool = False):
    """Context manager that batches the collectives issued inside it into one launch."""
    build = tdist.distributed_c10d._coalescing_manager
    return build(group, device=device, async_ops=async_op)
