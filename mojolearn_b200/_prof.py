"""Optional device timing of the classes of work inside a model step.

Off by default (a span is then a no-op). When enabled, every span records a CUDA event pair on the current stream
around the launches it encloses; `report()` synchronises and returns the summed microseconds and the number of
spans per class. Launch by launch only: events cannot be recorded into a captured graph this way, and the spans
serialise nothing (they measure the stream's own order), so the sum over classes is the step's device time.
"""
import collections

import torch

ENABLED = False
_records = collections.defaultdict(list)


class span(object):
    __slots__ = ("name", "e0")

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if ENABLED:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if ENABLED:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _records[self.name].append((self.e0, e1))
        return False


def enable(on=True):
    global ENABLED
    ENABLED = bool(on)
    if on:
        _records.clear()


def report():
    torch.cuda.synchronize()
    out = {name: {"us": 1e3 * sum(a.elapsed_time(b) for a, b in pairs), "spans": len(pairs)} for name, pairs in _records.items()}
    _records.clear()
    return out
