"""Optional per-kernel timing with CUDA events on the launching stream.

Off by default (zero overhead beyond one ``if``).  ``bench.py`` turns it on for a few
steps to obtain the average duration of every native launch, which is what the roofline
figures are computed from.
"""
from __future__ import annotations

import contextlib
from collections import defaultdict

_enabled = False
_records = []          # (name, start_event, end_event)
launch_count = 0       # native kernel launches since the last reset (always counted)


def enable(flag: bool = True) -> None:
    global _enabled
    _enabled = flag


def reset() -> None:
    global launch_count
    _records.clear()
    launch_count = 0


@contextlib.contextmanager
def kernel(name: str, stream=None):
    """Brackets one native launch."""
    global launch_count
    launch_count += 1
    if not _enabled:
        yield
        return
    import torch

    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    yield
    e.record()
    _records.append((name, s, e))


def summary() -> dict:
    """{kernel name: (launches, total milliseconds)}; synchronises."""
    import torch

    torch.cuda.synchronize()
    out = defaultdict(lambda: [0, 0.0])
    for name, s, e in _records:
        out[name][0] += 1
        out[name][1] += s.elapsed_time(e)
    return {k: tuple(v) for k, v in out.items()}
