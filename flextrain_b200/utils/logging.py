"""Process-wide logger, a rank-0-only logger and small print helpers.

Parity: flextrain/utils/logging.py:1-55 (logger, rank0_logger, warning_once,
print_rank0, log_configuration).
"""
import functools
import logging
import os
import sys

_FORMAT = "[%(asctime)s] [%(levelname)s] [%(filename)s:%(lineno)d:%(funcName)s] %(message)s"


def _build_logger(name="FlexTrainB200", level=logging.INFO):
    lg = logging.getLogger(name)
    if lg.handlers:
        return lg
    lg.setLevel(os.environ.get("FLEXTRAIN_LOG_LEVEL", level))
    lg.propagate = False
    handler = logging.StreamHandler(stream=sys.stdout)
    handler.setFormatter(logging.Formatter(_FORMAT))
    lg.addHandler(handler)
    return lg


logger = _build_logger()


class _Rank0Logger:
    """Forwards to ``logger`` on rank 0 and swallows everything elsewhere.

    The rank is read from the ``RANK`` environment variable at call time so a
    process that learns its rank late (spawned test workers) still behaves.
    """

    def __getattr__(self, name):
        target = getattr(logger, name)
        if not callable(target):
            return target

        def call(*args, **kwargs):
            if int(os.environ.get("RANK", "0")) == 0:
                kwargs.setdefault("stacklevel", 2)
                return target(*args, **kwargs)
            return None

        return call


rank0_logger = _Rank0Logger()


@functools.lru_cache(None)
def warning_once(message: str):
    logger.warning(message)


def print_rank0(*args, **kwargs):
    if int(os.environ.get("RANK", "0")) == 0:
        print(*args, **kwargs, flush=True)


def log_configuration(config, name: str):
    """Pretty-print every public attribute of ``config`` on rank 0."""
    lines = [f"{name}:"]
    for key in sorted(vars(config)):
        if key.startswith("_"):
            continue
        dots = "." * max(2, 32 - len(key))
        lines.append(f"  {key} {dots} {getattr(config, key)}")
    rank0_logger.info("\n".join(lines))
