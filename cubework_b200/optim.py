"""Fused optimizers.

Replaces ``torch.optim.AdamW`` (benchmark/gpt2/gpt2.py:440, vit/vit.py:477) and ``torch.optim.SGD``
(benchmark/opt/opt.py:623).  On CUDA one multi-tensor kernel updates the fp32 master parameter, its
moments and — when the parameter has a low-precision shadow used by the GEMMs — the shadow, so no
separate cast kernel runs in steady state.  Parameters that are themselves 16-bit (the pure 16-bit mode of
``benchmark/opt/train.py -O3``) take the formula path with fp32 arithmetic per update and no master copy.  An optional device-side ``grad_scale`` (e.g. the clipping
coefficient) is folded into the same pass.  On the host the update is the textbook formula and matches
``torch.optim`` bit-for-bit in fp32.
"""
import math

import torch

from . import ops
from .ops import ext


def _lowp_shadow(p):
    for dt in (torch.bfloat16, torch.float16):
        s = ops.peek_shadow(p, dt)
        if s is not None:
            return s
    return None


class FusedAdamW(torch.optim.Optimizer):

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None, grad_scale=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            todo = []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                todo.append(p)
            if not todo:
                continue
            step = self.state[todo[0]]["step"]
            if todo[0].is_cuda and ops.kernels_enabled() and all(self.state[p]["step"] == step for p in todo) \
                    and all(p.dtype == torch.float32 for p in todo):
                ext.require()
                shadows = [_lowp_shadow(p) for p in todo]
                ext.multi_adamw(todo, [p.grad for p in todo], [self.state[p]["exp_avg"] for p in todo],
                                [self.state[p]["exp_avg_sq"] for p in todo],
                                [s.tensor if s is not None else None for s in shadows], lr, beta1, beta2, eps, wd,
                                step, grad_scale)
                continue
            for p in todo:
                st = self.state[p]
                g = p.grad.float()
                if grad_scale is not None:
                    g = g * grad_scale.to(g.device)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                pf = p.float() if p.dtype != torch.float32 else p
                pf.mul_(1 - lr * wd)
                m.lerp_(g, 1 - beta1)
                v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                bc1 = 1 - beta1**st["step"]
                bc2 = 1 - beta2**st["step"]
                denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
                pf.addcdiv_(m, denom, value=-lr / bc1)
                if pf is not p:
                    p.copy_(pf)
        return loss


class FusedSGD(torch.optim.Optimizer):

    def __init__(self, params, lr=1e-3, momentum=0.0, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None, grad_scale=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            lr, mom, wd = group["lr"], group["momentum"], group["weight_decay"]
            todo = [p for p in group["params"] if p.grad is not None]
            if not todo:
                continue
            bufs = []
            for p in todo:
                st = self.state[p]
                if mom != 0 and "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                    st["fresh"] = True
                bufs.append(st.get("momentum_buffer"))
            if todo[0].is_cuda and ops.kernels_enabled() and all(p.dtype == torch.float32 for p in todo):
                ext.require()
                shadows = [_lowp_shadow(p) for p in todo]
                first = bool(mom != 0 and self.state[todo[0]].get("fresh", False))
                ext.multi_sgd(todo, [p.grad for p in todo], bufs if mom != 0 else None,
                              [s.tensor if s is not None else None for s in shadows], lr, mom, wd, first, grad_scale)
                for p in todo:
                    self.state[p]["fresh"] = False
                continue
            for p, buf in zip(todo, bufs):
                g = p.grad.float()
                if grad_scale is not None:
                    g = g * grad_scale.to(g.device)
                if wd != 0:
                    g = g.add(p.float(), alpha=wd)
                if mom != 0:
                    if self.state[p].get("fresh", False):
                        buf.copy_(g)
                        self.state[p]["fresh"] = False
                    else:
                        buf.mul_(mom).add_(g)
                    g = buf
                p.add_(g.to(p.dtype), alpha=-lr)
        return loss


def linear_warmup_schedule(optimizer, num_warmup_steps, num_training_steps):
    """Linear warm-up then linear decay to zero (the schedule the GPT-2 / OPT recipes use)."""

    def f(step):
        if step < num_warmup_steps:
            return float(step) / float(max(1, num_warmup_steps))
        return max(0.0, float(num_training_steps - step) / float(max(1, num_training_steps - num_warmup_steps)))

    return torch.optim.lr_scheduler.LambdaLR(optimizer, f)


def cosine_warmup_schedule(optimizer, num_warmup_steps, num_training_steps):
    """Linear warm-up then half-cosine decay (the ViT recipe)."""

    def f(step):
        if step < num_warmup_steps:
            return float(step) / float(max(1, num_warmup_steps))
        prog = float(step - num_warmup_steps) / float(max(1, num_training_steps - num_warmup_steps))
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * prog)))

    return torch.optim.lr_scheduler.LambdaLR(optimizer, f)
