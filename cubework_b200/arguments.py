"""Framework flags appended to the caller's argparse parser.

Parity: cubework/arguments.py:1-21 (``--tensor_parallel/--tp``, ``--tensor_parallel_size/--tp_size``,
``--backend``, ``--seed``; result cached and returned by ``get_args``).  ``parse_args`` additionally
accepts an explicit ``argv`` list so tests and benchmarks do not have to edit ``sys.argv``.
"""
import argparse

_ARGS = None


def get_args():
    return _ARGS


def add_framework_flags(parser):
    have = {s for a in parser._actions for s in a.option_strings}
    if "--tensor_parallel" not in have:
        parser.add_argument("--tensor_parallel", "--tp", type=str, default=None, choices=["1d", "2d", "3d"])
    if "--tensor_parallel_size" not in have:
        parser.add_argument("--tensor_parallel_size", "--tp_size", type=int, default=None)
    if "--backend" not in have:
        parser.add_argument("--backend", type=str, default=None,
                            help="torch.distributed backend; default nccl with a GPU, gloo without")
    if "--seed" not in have:
        parser.add_argument("--seed", type=int, default=None)
    return parser


def parse_args(parser=None, argv=None):
    if parser is None:
        parser = argparse.ArgumentParser()
    add_framework_flags(parser)
    global _ARGS
    _ARGS = parser.parse_args(argv)
    return _ARGS


def set_args(ns):
    """Install an already-built namespace (used by programmatic launchers and tests)."""
    global _ARGS
    _ARGS = ns
    return _ARGS
