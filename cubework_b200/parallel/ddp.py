"""Data parallelism over the DATA group.

The reference wraps models in ``torch.nn.parallel.DistributedDataParallel(process_group=pm.DATA.group)``
(benchmark/gpt2/gpt2.py:382-383, vit/vit.py:419-421, opt/opt.py:562).  This wrapper does the same job
for the layers of this package: gradients are packed into flat buckets in reverse construction order;
a bucket's all-reduce is launched (asynchronously) the moment its last gradient has been accumulated,
so the reduction overlaps the rest of backward; a callback at the end of backward waits for the
buckets and scatters the averaged values back.  Collectives go through the package's wrappers, so the
communication profiler sees data-parallel traffic too (the reference's profiler cannot see DDP's).
"""
import torch
import torch.nn as nn
from torch.autograd import Variable

from .collective import all_reduce, broadcast
from .mesh import pm


class DataParallel(nn.Module):

    def __init__(self, module, bucket_bytes=256 << 20, mode=None, broadcast_params=True):
        super().__init__()
        self.module = module
        self.mode = mode or pm.DATA
        self.enabled = self.mode.is_initialized() and self.mode.world_size > 1
        self._buckets = []
        self._pending = []
        self._callback_queued = False
        self.require_sync = True
        if not self.enabled:
            return
        params = [p for p in module.parameters() if p.requires_grad]
        if broadcast_params:
            with torch.no_grad():
                for p in params:
                    broadcast(p.data, self.mode.rank_by_idx(0), self.mode)
        cur, cur_bytes, cur_key = [], 0, None
        for p in reversed(params):
            key = (p.dtype, p.device)
            nbytes = p.numel() * p.element_size()
            if cur and (key != cur_key or cur_bytes + nbytes > bucket_bytes):
                self._buckets.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_key = key
        if cur:
            self._buckets.append(cur)
        self._bucket_of = {}
        for bi, b in enumerate(self._buckets):
            for p in b:
                self._bucket_of[p] = bi
                p.register_post_accumulate_grad_hook(self._on_grad)
        self._ready = [0] * len(self._buckets)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def no_sync(self):
        """Context manager: skip gradient reduction (gradient accumulation micro-steps)."""
        outer = self

        class _Ctx:

            def __enter__(self):
                outer.require_sync = False

            def __exit__(self, *exc):
                outer.require_sync = True

        return _Ctx()

    def _on_grad(self, p):
        if not (self.enabled and self.require_sync):
            return
        bi = self._bucket_of[p]
        self._ready[bi] += 1
        if not self._callback_queued:
            Variable._execution_engine.queue_callback(self._finish)
            self._callback_queued = True
        if self._ready[bi] == len(self._buckets[bi]):
            self._launch(bi)

    def _launch(self, bi):
        ps = [p for p in self._buckets[bi] if p.grad is not None]
        if not ps:
            return
        flat = torch.cat([p.grad.reshape(-1) for p in ps])
        flat.div_(self.mode.world_size)
        flat, work = all_reduce(flat, self.mode, async_op=True)
        self._pending.append((ps, flat, work))

    def _finish(self):
        # buckets whose parameters did not all receive a gradient in this pass are reduced now
        for bi, n in enumerate(self._ready):
            if 0 < n < len(self._buckets[bi]):
                self._launch(bi)
        for ps, flat, work in self._pending:
            if work is not None:
                work.wait()
            off = 0
            for p in ps:
                n = p.numel()
                p.grad.copy_(flat[off:off + n].view_as(p.grad))
                off += n
        self._pending.clear()
        self._ready = [0] * len(self._buckets)
        self._callback_queued = False

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)
