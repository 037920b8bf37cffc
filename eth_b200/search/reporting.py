"""Search logging: progress lines, wall-clock timers and the ranked summary
(reference: eth/searching/reporting.py:24-106 timers, :324-409 top configs, :587-613 trend CSVs)."""
from __future__ import annotations

import os
import time


class SearchLog:
    def __init__(self, log_path=None, quiet=False):
        self.quiet = quiet
        self.file = None
        if log_path:
            os.makedirs(log_path, exist_ok=True)
            self.file = open(os.path.join(log_path, "search_trend.log"), "a")

    def write(self, msg: str) -> None:
        if not self.quiet:
            print(msg, flush=True)
        if self.file:
            self.file.write(msg + "\n")
            self.file.flush()


class Timers:
    def __init__(self):
        self.t = {}
        self.open = {}

    def start(self, name):
        self.open[name] = time.perf_counter()

    def stop(self, name):
        self.t[name] = self.t.get(name, 0.0) + time.perf_counter() - self.open.pop(name)

    def report(self):
        return dict(self.t)
