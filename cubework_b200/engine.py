"""Training engine: the call a user makes to run one optimisation step.

Parity: the ``_train`` hot loop of benchmark/{gpt2,opt,vit}/train.py:44-184 — micro-batch loop with
gradient accumulation, autocast forward, loss, backward, gradient clipping, optimizer + scheduler step,
``zero_grad``.  Differences: inputs are copied host->device from pinned memory on a side stream one
step ahead; bf16 needs no ``GradScaler`` (fp16 still gets one); there is no per-micro-batch host
synchronisation — ``step`` returns the loss as a device tensor and ``loss.item()`` is the caller's
choice.
"""
import contextlib

import torch

from .parallel.common import synchronize as _sync_async_grads
from .parallel.ops_1d import PARTIAL_GRAD, reduce_partial_grads
from .utils.clip_grad import clip_grad_norm


class Trainer:

    def __init__(self, model, criterion, optimizer, lr_scheduler=None, *, amp_dtype=torch.bfloat16, clip=None,
                 accum_steps=1, forward_fn=None, device=None, scaler_kwargs=None, timer=None):
        """``forward_fn(model, batch) -> (outputs, targets)``; default feeds ``batch`` as kwargs minus
        ``labels`` and uses ``batch["labels"]`` as targets.  ``scaler_kwargs`` (``init_scale``, ``growth_factor``,
        ``backoff_factor``, ``growth_interval``) configure the loss scaler of fp16 runs (benchmark/gpt2/train.py:
        316-319, 340-347 in the reference).  ``timer`` (an object with ``start(name)`` / ``stop(name)``) receives
        the phases ``data``, ``fwd``, ``bwd`` and ``opt`` of every step (train.py:79-129)."""
        self.model, self.criterion, self.optimizer, self.lr_scheduler = model, criterion, optimizer, lr_scheduler
        self.amp_dtype, self.clip, self.accum_steps = amp_dtype, clip, accum_steps
        self.forward_fn = forward_fn or self._default_forward
        self.device = device or next(model.parameters()).device
        self.scaler = torch.amp.GradScaler("cuda", **(scaler_kwargs or {})) \
            if (amp_dtype == torch.float16 and self.device.type == "cuda") else None
        self.timer = timer
        self._copy_stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.h2d_bytes = 0
        self.steps = 0
        # replicated parameters applied to row-sharded activations (1D sequence_parallel): summed over the group
        self._partial_params = [p for p in model.parameters() if getattr(p, PARTIAL_GRAD, False)]
        self._params = list(model.parameters())      # walking the module tree every step costs host milliseconds
        self.status_interval = 16     # steps between reads of the kernels' host-mapped error word

    @staticmethod
    def _default_forward(model, batch):
        labels = batch["labels"]
        out = model(**{k: v for k, v in batch.items() if k != "labels"})
        if isinstance(out, tuple):
            out = out[0]
        return out, labels

    def to_device(self, batch):
        """Asynchronous host->device copy of a dict of (pinned) host tensors."""
        if self.device.type != "cuda":
            return batch
        moved = []

        def move(v):
            if torch.is_tensor(v) and v.device.type == "cpu":
                self.h2d_bytes += v.numel() * v.element_size()
                v = v.to(self.device, non_blocking=True)
                moved.append(v)
            elif isinstance(v, (tuple, list)):       # e.g. mixed-up labels: (labels, permuted labels, lambda)
                v = type(v)(move(x) for x in v)
            return v

        with torch.cuda.stream(self._copy_stream):
            out = {k: move(v) for k, v in batch.items()}
        torch.cuda.current_stream().wait_stream(self._copy_stream)
        for v in moved:
            v.record_stream(torch.cuda.current_stream())
        return out

    def _autocast(self):
        if self.amp_dtype is None or self.device.type != "cuda":
            return contextlib.nullcontext()
        return torch.autocast("cuda", dtype=self.amp_dtype)

    def step(self, batches):
        """One optimisation step over ``accum_steps`` micro-batches (a dict, or a list of dicts)."""
        if isinstance(batches, dict):
            batches = [batches]
        if not self.model.training:      # walking every submodule each step costs milliseconds of host time
            self.model.train()
        total = None
        n = len(batches)
        tm = self.timer
        for i, batch in enumerate(batches):
            if tm is not None:
                tm.start("data")
            batch = self.to_device(batch)
            if tm is not None:
                tm.stop("data")
            sync_ctx = contextlib.nullcontext()
            if i < n - 1 and hasattr(self.model, "no_sync"):
                sync_ctx = self.model.no_sync()
            with sync_ctx:
                if tm is not None:
                    tm.start("fwd")
                with self._autocast():
                    out, targets = self.forward_fn(self.model, batch)
                    loss = self.criterion(out, targets)
                if tm is not None:
                    tm.stop("fwd")
                    tm.start("bwd")
                scaled = loss / n if n > 1 else loss
                if self.scaler is not None:
                    self.scaler.scale(scaled).backward()
                else:
                    scaled.backward()
                if tm is not None:
                    tm.stop("bwd")
            total = loss.detach() if total is None else total + loss.detach()
        if tm is not None:
            tm.start("opt")
        _sync_async_grads(host_sync=False)
        if self._partial_params:
            reduce_partial_grads(self._partial_params)
        if self.scaler is not None:
            self.scaler.unscale_(self.optimizer)
        if self.clip is not None and self.clip > 0:
            clip_grad_norm(self._params, self.clip)
        if self.scaler is not None:
            self.scaler.step(self.optimizer)
            self.scaler.update()
        else:
            self.optimizer.step()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.optimizer.zero_grad(set_to_none=True)
        if tm is not None:
            tm.stop("opt")
        self.steps += 1
        if self.device.type == "cuda" and self.steps % self.status_interval == 0:
            self.check_device_status()
        return total / n if n > 1 else total

    def check_device_status(self):
        """Raise if a kernel of this package gave up on a bounded wait (a peer that never arrived, a stage that
        never landed) since the last check.  Reading the host-mapped word costs no synchronisation, so a failure
        is reported at the latest ``status_interval`` steps after it happened; a failed fused launch leaves its
        output incomplete, and the peer-memory workspaces are released so that the next fused call starts from
        fresh epochs."""
        from .ops import ext
        if not ext.loaded():
            return
        try:
            ext.check_status()
        except RuntimeError:
            from .parallel import symm
            symm.invalidate_all()
            raise

    @torch.no_grad()
    def evaluate(self, batch):
        if self.device.type == "cuda":
            self.check_device_status()
        self.model.eval()
        batch = self.to_device(batch)
        with self._autocast():
            out, targets = self.forward_fn(self.model, batch)
            loss = self.criterion(out, targets)
        return out, targets, loss
