"""Spawn ``world_size`` CPU/gloo (or CUDA/NCCL) ranks on this host and run a check function in each.

Mirrors the launch style of the reference tests (tests/test_1d/test_1d.py:22-46: ``mp.spawn`` + a free
port + ``initialize_distributed``) but passes the framework flags as an ``argv`` list and defaults to
gloo so the suite runs without a GPU.
"""
import os
import traceback

import torch
import torch.multiprocessing as mp


def _worker(rank, world_size, port, fn, tp, tp_size, backend, fn_args, use_cuda):
    os.environ["RANK"] = str(rank)
    os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if not use_cuda:
        os.environ["CUDA_VISIBLE_DEVICES"] = ""
    torch.set_num_threads(1)
    import cubework_b200 as cube
    argv = []
    if tp is not None:
        argv += ["--tp", tp, "--tp_size", str(tp_size)]
    argv += ["--backend", backend]
    try:
        cube.initialize_distributed(argv=argv, timeout_s=120)
        fn(*fn_args)
    except Exception:
        traceback.print_exc()
        raise
    finally:
        try:
            cube.destroy_distributed()
        except Exception:
            pass


def run_dist(fn, world_size, tp=None, tp_size=None, backend="gloo", args=(), use_cuda=False):
    from cubework_b200.utils import free_port
    for attempt in range(4):
        port = free_port()
        try:
            mp.spawn(_worker, args=(world_size, port, fn, tp, tp_size or world_size, backend, args, use_cuda),
                     nprocs=world_size, join=True)
            return
        except Exception as e:     # the probed port can be taken again before rank 0 binds it: pick another
            if "address already in use" not in str(e).lower() or attempt == 3:
                raise


def chunk(x, n, dim, idx):
    return torch.chunk(x, n, dim=dim)[idx]


def check_close(a, b, rtol=1e-4, atol=1e-5, what=""):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if not torch.allclose(a, b, rtol=rtol, atol=atol):
        err = (a - b).abs().max().item()
        raise AssertionError(f"{what}: max abs err {err:.3e} (rtol={rtol}, atol={atol})")
