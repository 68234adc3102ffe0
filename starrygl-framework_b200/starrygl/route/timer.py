"""Named wall/device timers (reference: starrygl/route/timer.py:10-70).  CUDA events when a GPU is
present, ``perf_counter`` otherwise; times are in seconds."""
import time
from contextlib import contextmanager
from typing import Dict, List, Tuple

import torch


class _Event:
    def __init__(self):
        self.type = "cuda" if torch.cuda.is_available() else "cpu"
        self.inner = None

    def record(self):
        if self.type == "cuda":
            self.inner = torch.cuda.Event(enable_timing=True)
            self.inner.record()
        else:
            self.inner = time.perf_counter()

    def elapsed_time(self, other: "_Event") -> float:
        if self.type == "cuda":
            other.inner.synchronize()
            return self.inner.elapsed_time(other.inner) / 1000
        return other.inner - self.inner

    def synchronize(self):
        if self.type == "cuda":
            self.inner.synchronize()


class EventTimer:
    def __init__(self):
        self.elapsed_times: Dict[str, float] = {}
        self.record_events: Dict[str, List[Tuple[_Event, _Event]]] = {}

    @contextmanager
    def record(self, name: str = "_default_"):
        s, t = _Event(), _Event()
        s.record()
        yield
        t.record()
        self.record_events.setdefault(name, []).append((s, t))

    def reset(self):
        self.elapsed_times.clear()
        self.record_events.clear()

    def __getitem__(self, name: str) -> float:
        return self.get(name)

    def get(self, name: str = "_default_") -> float:
        value = self.elapsed_times.get(name, 0.0)
        for s, t in self.record_events.pop(name, []):
            value += s.elapsed_time(t)
        self.elapsed_times[name] = value
        return value
