"""Search logging and result ranking.

`SearchLog` prints and files progress lines; `Ranking` keeps the best N distinct plans seen and
writes them out ordered (`top_configs/`), with a CSV of the ranking and a trend CSV of every
improvement over time (reference: eth/searching/reporting.py:324-409 top configs, :562-584 hybrid
top list, :587-613 trend CSVs). `Timers` accumulates wall-clock time per named phase of the search
and is reported in the summary (:24-106).
"""
from __future__ import annotations

import csv
import os
import time
from contextlib import contextmanager
from typing import Callable, List, Tuple


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
        self.seconds = {}

    @contextmanager
    def phase(self, name: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.seconds[name] = self.seconds.get(name, 0.0) + time.perf_counter() - t0

    def report(self):
        return {k: round(v, 4) for k, v in sorted(self.seconds.items())}


class Ranking:
    """Best `keep` plans by iteration time; plans with the same signature count once."""

    def __init__(self, keep: int, signature: Callable):
        self.keep, self.signature = max(1, keep), signature
        self.entries: List[Tuple[float, object]] = []
        self.trend: List[Tuple[float, float, float]] = []    # (seconds since start, iteration ms, samples/s)
        self.t0 = time.time()

    def offer(self, plan) -> bool:
        """True if `plan` is the new best."""
        sig = self.signature(plan)
        for i, (_, old) in enumerate(self.entries):
            if self.signature(old) == sig:
                if plan.iteration_us < old.iteration_us:
                    self.entries[i] = (plan.iteration_us, plan)
                break
        else:
            self.entries.append((plan.iteration_us, plan))
        self.entries.sort(key=lambda e: e[0])
        del self.entries[self.keep:]
        is_best = self.entries[0][1] is plan
        if is_best:
            self.trend.append((time.time() - self.t0, plan.iteration_us / 1e3, plan.throughput))
        return is_best

    @property
    def best(self):
        return self.entries[0][1] if self.entries else None

    def write_csvs(self, directory: str, stem: str) -> None:
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, f"{stem}_ranking.csv"), "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["rank", "iteration_ms", "samples_per_s", "pipelines", "stages", "micro_batch_sizes", "batch_sizes"])
            for rank, (_, plan) in enumerate(self.entries, 1):
                w.writerow([rank, f"{plan.iteration_us / 1e3:.3f}", f"{plan.throughput:.3f}", len(plan.pipelines),
                            "|".join(str(len(p.stages)) for p in plan.pipelines),
                            "|".join(str(p.mbs) for p in plan.pipelines), "|".join(map(str, plan.batch_sizes))])
        with open(os.path.join(directory, f"{stem}_trend.csv"), "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["seconds", "best_iteration_ms", "best_samples_per_s"])
            for sec, ms, rate in self.trend:
                w.writerow([f"{sec:.3f}", f"{ms:.3f}", f"{rate:.3f}"])
