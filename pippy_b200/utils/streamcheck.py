"""Debug aid: a happens-before checker for buffers that several CUDA streams touch.

The package runs work on side streams (the data-parallel reducer's kernels, NCCL's communicator streams) over buffers
that the compute stream also reads and writes (the flat gradient buffer).  A missing ``wait_event`` there is a data
race that no test on small shapes is sure to catch, and compute-sanitizer's racecheck is not available everywhere.
With ``PIPPY_STREAM_CHECK=1`` (or ``enable()``) the code that launches side-stream work reports what it does here:

    tracker.write(name, stream)        work launched on ``stream`` writes buffer ``name``
    tracker.read(name, stream)         work launched on ``stream`` reads it
    tracker.ordered(first, then)       ``then`` was made to wait for everything launched so far on ``first``
                                       (an event recorded on ``first`` and waited for by ``then``)

and every access is checked against the last writer (and, for writes, the readers since): the accessing stream must
be that same stream or must have been ordered after it since the conflicting access was launched.  A violation raises
:class:`StreamOrderError` naming the buffer and the two streams.  Streams are identified by any hashable value (the
runtime uses ``torch.cuda.Stream.cuda_stream``; the unit tests use strings), so the checker itself runs without a GPU.
The reference has no such tool (it relies on NCCL's stream semantics and lock-step schedules).
"""
from __future__ import annotations

import os
from typing import Dict, Hashable, List, Optional, Tuple


class StreamOrderError(RuntimeError):
    """Two streams touched the same buffer without an ordering between them."""


class StreamTracker:
    def __init__(self) -> None:
        self._clock = 0
        # per stream: logical time of its latest launch
        self._launched: Dict[Hashable, int] = {}
        # (waiter, waited) -> the waited stream's logical time that the waiter is known to be ordered after
        self._seen: Dict[Tuple[Hashable, Hashable], int] = {}
        self._last_write: Dict[str, Tuple[Hashable, int]] = {}
        self._reads_since: Dict[str, List[Tuple[Hashable, int]]] = {}

    def _tick(self, stream: Hashable) -> int:
        self._clock += 1
        self._launched[stream] = self._clock
        return self._clock

    def ordered(self, first: Hashable, then: Hashable) -> None:
        """``then`` waits for all work launched on ``first`` so far; orderings ``first`` had itself carry over."""
        if first == then:
            return
        self._seen[(then, first)] = self._launched.get(first, 0)
        for (waiter, waited), t in list(self._seen.items()):
            if waiter == first:
                key = (then, waited)
                self._seen[key] = max(self._seen.get(key, 0), t)

    def _is_after(self, stream: Hashable, other: Hashable, when: int) -> bool:
        return stream == other or self._seen.get((stream, other), -1) >= when

    def read(self, name: str, stream: Hashable) -> None:
        lw = self._last_write.get(name)
        if lw is not None and not self._is_after(stream, lw[0], lw[1]):
            raise StreamOrderError(f"stream {stream!r} reads {name!r} without waiting for its writer on stream {lw[0]!r}")
        self._reads_since.setdefault(name, []).append((stream, self._tick(stream)))

    def write(self, name: str, stream: Hashable) -> None:
        lw = self._last_write.get(name)
        if lw is not None and not self._is_after(stream, lw[0], lw[1]):
            raise StreamOrderError(
                f"stream {stream!r} writes {name!r} without waiting for the previous writer on stream {lw[0]!r}")
        for rs, when in self._reads_since.get(name, []):
            if not self._is_after(stream, rs, when):
                raise StreamOrderError(f"stream {stream!r} overwrites {name!r} while stream {rs!r} may still read it")
        self._reads_since[name] = []
        self._last_write[name] = (stream, self._tick(stream))


_TRACKER: Optional[StreamTracker] = StreamTracker() if os.environ.get("PIPPY_STREAM_CHECK", "0") == "1" else None


def enable() -> StreamTracker:
    global _TRACKER
    if _TRACKER is None:
        _TRACKER = StreamTracker()
    return _TRACKER


def disable() -> None:
    global _TRACKER
    _TRACKER = None


def tracker() -> Optional[StreamTracker]:
    """The active tracker, or None when checking is off (the callers' fast path)."""
    return _TRACKER
