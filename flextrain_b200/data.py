"""Token sources and a prefetching micro-batch feeder for ``get_batch``.

The reference leaves data loading to its user (``get_batch`` is the first of
the six callbacks, flextrain/llm_func.py:8-49); its users take Megatron's
indexed-dataset loaders.  This module is the small piece a run on this engine
needs instead: a flat binary token file read through ``numpy.memmap``, random
fixed-length windows drawn per (seed, micro-batch counter, rank) so every rank
reads different data and a resumed run continues the same stream, and a feeder
that fills pinned host buffers on a worker thread and copies them to the GPU on
a side stream, one or more micro-batches ahead of the engine.

    feeder = MicroBatchFeeder(TokenFile("tokens.u16"), micro_batch_size=2, seq_len=4096,
                              device=dev, rank=rank, world=world)
    flextrain.set_llm_func(*make_llm_funcs(model, feeder))       # feeder() -> (tokens, labels)
"""
from __future__ import annotations

import collections
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Optional, Tuple

import numpy as np
import torch

_SUFFIX_DTYPES = {".u16": np.uint16, ".u32": np.uint32, ".i32": np.int32, ".i64": np.int64,
                  ".bin": np.uint16}


class TokenFile:
    """A flat array of token ids on disk (no header), memory-mapped read-only.
    The dtype comes from ``dtype`` or from the suffix (``.u16`` / ``.bin``: uint16,
    ``.u32``, ``.i32``, ``.i64``)."""

    def __init__(self, path: str, dtype=None):
        if dtype is None:
            dtype = _SUFFIX_DTYPES.get(os.path.splitext(path)[1])
            if dtype is None:
                raise ValueError(f"cannot tell the token dtype of {path}: pass dtype=")
        self.path = path
        self.tokens = np.memmap(path, dtype=dtype, mode="r")
        if self.tokens.size < 2:
            raise ValueError(f"{path} holds fewer than two tokens")

    def __len__(self) -> int:
        return int(self.tokens.size)

    def window(self, start: int, length: int) -> np.ndarray:
        if start < 0 or start + length > self.tokens.size:
            raise IndexError(f"window [{start}, {start + length}) outside a file of {self.tokens.size} tokens")
        return self.tokens[start:start + length]

    @staticmethod
    def write(path: str, tokens, dtype=None) -> "TokenFile":
        """Write ``tokens`` (any integer sequence) as a flat file and open it."""
        if dtype is None:
            dtype = _SUFFIX_DTYPES.get(os.path.splitext(path)[1], np.uint16)
        arr = np.asarray(tokens)
        if arr.size and (arr.min() < np.iinfo(dtype).min or arr.max() > np.iinfo(dtype).max):
            raise ValueError(f"token ids do not fit {np.dtype(dtype).name}")
        arr.astype(dtype).tofile(path)
        return TokenFile(path, dtype)


class SyntheticTokens:
    """Uniform random token ids (benchmarks, smoke runs)."""

    def __init__(self, vocab: int):
        if vocab < 2:
            raise ValueError("vocab must be at least 2")
        self.vocab = vocab


class _Slot:
    __slots__ = ("host", "event")

    def __init__(self, host):
        self.host = host
        self.event = None


class MicroBatchFeeder:
    """Callable returning ``(tokens [B, S], labels [B, S])`` int64 on ``device``,
    labels being the tokens shifted by one.  ``depth`` micro-batches are prepared
    ahead: a worker thread gathers the windows into pinned host buffers; on CUDA
    the host-to-device copy runs on its own stream and the caller's stream waits
    for it, so the copy overlaps whatever the engine has queued.

    Window ``b`` of micro-batch ``n`` on ``rank`` starts at a position drawn from a
    generator seeded with ``(seed, n, rank)``: the stream depends on nothing else,
    ``state_dict`` / ``load_state_dict`` therefore only carry ``n``."""

    def __init__(self, source, micro_batch_size: int, seq_len: int, device=None, rank: int = 0,
                 world: int = 1, seed: int = 0, depth: int = 2, pin: Optional[bool] = None):
        if micro_batch_size < 1 or seq_len < 1 or depth < 1:
            raise ValueError("micro_batch_size, seq_len and depth must be positive")
        if not 0 <= rank < world:
            raise ValueError("rank must lie in [0, world)")
        self.source = source
        self.mbs, self.seq = micro_batch_size, seq_len
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.rank, self.world, self.seed, self.depth = rank, world, seed, depth
        if isinstance(source, TokenFile) and len(source) < seq_len + 1:
            raise ValueError(f"{source.path} is shorter than one window of {seq_len + 1} tokens")
        cuda = self.device.type == "cuda"
        pin = cuda if pin is None else pin
        self._slots = []
        for _ in range(depth):
            host = torch.empty(micro_batch_size, seq_len + 1, dtype=torch.int64)
            self._slots.append(_Slot(host.pin_memory() if pin else host))
        self._stream = torch.cuda.Stream(device=self.device) if cuda else None
        self._pool = ThreadPoolExecutor(1, thread_name_prefix="ft-feeder")
        self._futures = collections.deque()
        self._next_fill = 0
        self.consumed = 0
        self.h2d_bytes = 0
        for _ in range(depth):
            self._schedule()

    # ----------------------------------------------------------- sampling
    def window_starts(self, n: int) -> np.ndarray:
        """Start offsets of the windows of micro-batch ``n`` on this rank."""
        gen = torch.Generator().manual_seed((self.seed * 1_000_003 + n) * 4099 + self.rank)
        hi = len(self.source) - self.seq
        return torch.randint(0, hi, (self.mbs,), generator=gen).numpy()

    def _fill(self, slot: _Slot, n: int) -> _Slot:
        if slot.event is not None:
            slot.event.synchronize()                # the previous copy out of this buffer is done
            slot.event = None
        if isinstance(self.source, SyntheticTokens):
            gen = torch.Generator().manual_seed((self.seed * 1_000_003 + n) * 4099 + self.rank)
            slot.host.copy_(torch.randint(0, self.source.vocab, (self.mbs, self.seq + 1), generator=gen))
        else:
            for b, start in enumerate(self.window_starts(n)):
                win = self.source.window(int(start), self.seq + 1)
                slot.host[b].copy_(torch.from_numpy(win.astype(np.int64, copy=False)))
        return slot

    def _schedule(self):
        n = self._next_fill
        self._next_fill += 1
        self._futures.append(self._pool.submit(self._fill, self._slots[n % self.depth], n))

    # ------------------------------------------------------------- feeding
    def __call__(self) -> Tuple[torch.Tensor, torch.Tensor]:
        slot = self._futures.popleft().result()
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                t = slot.host.to(self.device, non_blocking=True)
                slot.event = torch.cuda.Event()
                slot.event.record(self._stream)
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(slot.event)
            t.record_stream(cur)
            self.h2d_bytes += t.numel() * t.element_size()
        else:
            t = slot.host.clone()
        self.consumed += 1
        self._schedule()
        return t[:, :-1], t[:, 1:]

    # -------------------------------------------------------------- resume
    def state_dict(self) -> Dict[str, int]:
        return {"consumed": self.consumed, "seed": self.seed}

    def load_state_dict(self, state: Dict[str, int]):
        if state.get("seed", self.seed) != self.seed:
            raise ValueError("feeder state was written with a different seed")
        self._drain()
        self.consumed = self._next_fill = int(state["consumed"])
        for _ in range(self.depth):
            self._schedule()

    def _drain(self):
        while self._futures:
            self._futures.popleft().result()

    def close(self):
        self._drain()
        self._pool.shutdown(wait=True)
        if self._stream is not None:
            self._stream.synchronize()
