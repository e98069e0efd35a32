"""RNG and device helpers.

Parity: cubework/utils/common.py:9-49 (``seed`` context manager, ``set_device``, ``set_seed``,
``get_current_device``, ``free_port``).  ``seed(mode)`` swaps in the RNG stream owned by a
``ParallelMode`` and, unlike the reference, stores the advanced state back on exit so successive
blocks draw fresh numbers; pass ``replay=True`` for the reference's replaying behaviour.  Works on
hosts without CUDA.
"""
import random
import socket
from contextlib import contextmanager

import numpy as np
import torch


@contextmanager
def seed(parallel_mode, replay: bool = False):
    use_cuda = torch.cuda.is_available() and parallel_mode.cuda_rng_state is not None
    cur = torch.get_rng_state()
    cur_cuda = torch.cuda.get_rng_state() if use_cuda else None
    try:
        torch.set_rng_state(parallel_mode.rng_state)
        if use_cuda:
            torch.cuda.set_rng_state(parallel_mode.cuda_rng_state)
        yield
    finally:
        if not replay:
            parallel_mode.set_rng_states(torch.get_rng_state(), torch.cuda.get_rng_state() if use_cuda else None)
        torch.set_rng_state(cur)
        if use_cuda:
            torch.cuda.set_rng_state(cur_cuda)


def set_device(local_rank):
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank % torch.cuda.device_count())


def set_seed(seed_):
    random.seed(seed_)
    np.random.seed(seed_ % (2**32))
    torch.manual_seed(seed_)


def get_current_device():
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]
