"""Communication profiler.

Parity: cubework/utils/profiling/communication.py:16-168 — ``CommProfiler.start()/stop()/reset()``;
``stop()`` returns ``(ops, bytes, seconds)`` where bytes are *algorithm* bytes (all-reduce
``2(n-1)/n*S``, all-gather / reduce-scatter ``(n-1)/n*S``, broadcast / reduce ``S``).

Design: instead of rebinding ``torch.distributed`` functions, the collective wrappers of this package
report to the active profiler directly.  Every record holds a pair of CUDA events taken on the
issuing stream; nothing synchronises the host until ``stop()`` (or ``summary()``), where overlapping
records are merged into busy intervals so concurrent collectives are not double-counted.  Fused
compute+collective kernels report their own link bytes through :meth:`account`, with a pair of
events around the launch: their transfer is not a separate launch, so their time (``fused_seconds``
in :meth:`summary`) is the kernels' whole duration - product and exchange overlapped - and is kept
apart from the time of the stand-alone collectives.
"""
import time

import torch

from ...parallel import collective as _coll


class CommProfiler(object):

    def __init__(self):
        self.reset()
        self._active = False

    def reset(self):
        self.ops = 0
        self.volume = 0
        self.records = []       # (kind, bytes, start, end) with CUDA events or host times
        self.fused_bytes = 0
        self.fused_records = []  # (start event, end event) of fused compute+collective launches
        self.by_kind = {}

    # -- called by cubework_b200.parallel.collective ------------------------------------------
    def _open(self, kind, nbytes, tensor):
        self.ops += 1
        self.volume += nbytes
        k = self.by_kind.setdefault(kind, [0, 0])
        k[0] += 1
        k[1] += nbytes
        if tensor.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            rec = [kind, nbytes, ev, None, True]
        else:
            rec = [kind, nbytes, time.perf_counter(), None, False]
        self.records.append(rec)
        return rec

    def _close(self, rec):
        if rec[4]:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            rec[3] = ev
        else:
            rec[3] = time.perf_counter()

    def account(self, kind, nbytes, start=None, end=None):
        """Link bytes moved inside a fused kernel; ``start`` / ``end`` are CUDA events recorded around its launch."""
        if start is not None and end is not None:
            self.fused_records.append((start, end))
        self.ops += 1
        self.volume += nbytes
        self.fused_bytes += nbytes
        k = self.by_kind.setdefault(kind, [0, 0])
        k[0] += 1
        k[1] += nbytes

    # -- public API -------------------------------------------------------------------------------
    def start(self):
        self._active = True
        _coll._set_profiler(self)

    def _seconds(self):
        cuda_recs = [r for r in self.records if r[4] and r[3] is not None]
        host = sum(r[3] - r[2] for r in self.records if (not r[4]) and r[3] is not None)
        if not cuda_recs:
            return host
        torch.cuda.synchronize()
        base = cuda_recs[0][2]
        spans = sorted((base.elapsed_time(r[2]), base.elapsed_time(r[3])) for r in cuda_recs)
        busy, cur_s, cur_e = 0.0, spans[0][0], spans[0][1]
        for s, e in spans[1:]:
            if s > cur_e:
                busy += cur_e - cur_s
                cur_s, cur_e = s, e
            else:
                cur_e = max(cur_e, e)
        busy += cur_e - cur_s
        return host + busy / 1e3

    def stop(self):
        if self._active:
            _coll._set_profiler(None)
            self._active = False
        return self.ops, self.volume, self._seconds()

    def _fused_seconds(self):
        if not self.fused_records:
            return 0.0
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.fused_records) / 1e3

    def summary(self):
        secs = self._seconds()
        return dict(ops=self.ops, bytes=self.volume, seconds=secs, fused_bytes=self.fused_bytes,
                    fused_seconds=self._fused_seconds(),
                    algo_gbps=(self.volume - self.fused_bytes) / secs / 1e9 if secs > 0 else 0.0,
                    by_kind={k: tuple(v) for k, v in self.by_kind.items()})
