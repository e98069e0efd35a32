"""Initializer factories for sharded tensors.

Parity: cubework/module/init.py:8-140 (``zeros_, ones_, uniform_, normal_, trunc_normal_,
kaiming_uniform_, kaiming_normal_, xavier_uniform_(a, scale, gain), xavier_normal_, lecun_uniform_,
lecun_normal_``).  A factory call returns ``initializer(tensor, fan_in=None, fan_out=None)``; layers
pass the *global* fan-in / fan-out because ``tensor`` is one shard of the logical weight.

Every initializer here is described by a distribution kind and a function from the fans to that
distribution's spread, so there is a single code path that draws the numbers.
"""
import math

import torch.nn as nn


class _ShardInit:
    """``kind`` in {const, uniform, normal, trunc}; ``spread(fan_in, fan_out)`` -> kind parameters."""

    def __init__(self, kind, spread, needs=()):
        self.kind, self.spread, self.needs = kind, spread, needs

    def __call__(self, tensor, fan_in=None, fan_out=None):
        if tensor.numel() == 0:
            return tensor
        fans = {"fan_in": fan_in, "fan_out": fan_out}
        for name in self.needs:
            if fans[name] is None:
                raise AssertionError(f"{name} is not provided")
        args = self.spread(fan_in, fan_out)
        if self.kind == "const":
            return nn.init.constant_(tensor, args)
        if self.kind == "uniform":
            lo, hi = args
            return nn.init.uniform_(tensor, lo, hi)
        if self.kind == "normal":
            mean, std = args
            return nn.init.normal_(tensor, mean, std)
        mean, std, lo, hi = args
        return nn.init.trunc_normal_(tensor, mean, std, lo, hi)


def zeros_():
    return _ShardInit("const", lambda fi, fo: 0.0)


def ones_():
    return _ShardInit("const", lambda fi, fo: 1.0)


def uniform_(a: float = 0.0, b: float = 1.0):
    return _ShardInit("uniform", lambda fi, fo: (a, b))


def normal_(mean: float = 0.0, std: float = 1.0):
    return _ShardInit("normal", lambda fi, fo: (mean, std))


def trunc_normal_(mean: float = 0.0, std: float = 1.0, a: float = -2.0, b: float = 2.0):
    return _ShardInit("trunc", lambda fi, fo: (mean, std, a, b))


def _kaiming_std(a, mode, nonlinearity):
    if mode not in ("fan_in", "fan_out"):
        raise ValueError(f"Invalid initialization mode '{mode}'")
    gain = nn.init.calculate_gain(nonlinearity, a)
    return (lambda fi, fo: gain / math.sqrt(fi if mode == "fan_in" else fo)), (mode, )


def kaiming_uniform_(a=0, mode="fan_in", nonlinearity="leaky_relu"):
    std, needs = _kaiming_std(a, mode, nonlinearity)
    return _ShardInit("uniform", lambda fi, fo: (-math.sqrt(3.0) * std(fi, fo), math.sqrt(3.0) * std(fi, fo)), needs)


def kaiming_normal_(a=0, mode="fan_in", nonlinearity="leaky_relu"):
    std, needs = _kaiming_std(a, mode, nonlinearity)
    return _ShardInit("normal", lambda fi, fo: (0.0, std(fi, fo)), needs)


def _xavier_std(scale, gain):
    # fan_out is optional: biases are initialised from the fan-in alone
    return lambda fi, fo: gain * math.sqrt(scale / float(fi + (fo or 0)))


def xavier_uniform_(a: float = math.sqrt(3.0), scale: float = 2.0, gain: float = 1.0):
    std = _xavier_std(scale, gain)
    return _ShardInit("uniform", lambda fi, fo: (-a * std(fi, fo), a * std(fi, fo)), ("fan_in", ))


def xavier_normal_(scale: float = 2.0, gain: float = 1.0):
    std = _xavier_std(scale, gain)
    return _ShardInit("normal", lambda fi, fo: (0.0, std(fi, fo)), ("fan_in", ))


def lecun_uniform_():
    return _ShardInit("uniform", lambda fi, fo: (-math.sqrt(3.0 / fi), math.sqrt(3.0 / fi)), ("fan_in", ))


def lecun_normal_():
    # 0.8796... is the std of a unit normal truncated to [-2, 2]
    return _ShardInit("trunc", lambda fi, fo: (0.0, math.sqrt(1.0 / fi) / 0.87962566103423978, -2.0, 2.0),
                      ("fan_in", ))
