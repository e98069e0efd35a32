"""Background sampler of device memory.

Parity: cubework/utils/profiling/memory_tracker.py:15-72 (thread sampling
``torch.cuda.max_memory_allocated`` on an interval, optional per-rank log file).
"""
import threading
import time

import torch


class MemoryTracker(object):

    def __init__(self, log_file=None, interval=1e-3):
        self.interval = interval
        self.log_file = log_file
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        fh = open(self.log_file, "w") if self.log_file else None
        t0 = time.time()
        while not self._stop.is_set():
            peak = torch.cuda.max_memory_allocated() if torch.cuda.is_available() else 0
            self.samples.append((time.time() - t0, peak))
            if fh:
                fh.write(f"{self.samples[-1][0]:.6f} {peak}\n")
            time.sleep(self.interval)
        if fh:
            fh.close()

    def start(self):
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return max((p for _, p in self.samples), default=0)
