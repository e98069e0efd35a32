"""Per-group peer-memory workspaces and the dispatch of fused GEMM + collective launches.

A workspace is three ``cudaMalloc`` buffers per rank (staging for partial tiles, result tiles, flags),
exchanged as CUDA IPC handles over the group's gloo twin so every rank holds every peer's pointer.  Flags
carry a call epoch that only grows.  One workspace per process group; its fused launches are ordered by
the stream they run on.
"""
import os

import torch
import torch.distributed as dist

from ..ops import ext

TILE_BYTES = 128 * 256 * 2
_STAGE_BYTES = int(os.environ.get("CUBEWORK_B200_STAGE_MB", "160")) << 20
_RESULT_BYTES = int(os.environ.get("CUBEWORK_B200_RESULT_MB", "64")) << 20
_DONE_CAP = 1 << 16          # tiles per call
_COMM_CTAS = int(os.environ.get("CUBEWORK_B200_COMM_CTAS", "0"))
TRACE = None                  # optional int64 [148, 192, 2] CUDA tensor: per-CTA event trace of the next fused launches


class Workspace:

    def __init__(self, mode):
        m = ext.require()
        self.mode = mode
        self.n = mode.world_size
        self.me = mode.local_rank
        self.epoch = 0
        self.owned_cap = min(_RESULT_BYTES // TILE_BYTES, _STAGE_BYTES // (TILE_BYTES * self.n))
        flag_bytes = 4 * (_DONE_CAP * 8 + self.owned_cap * self.n * 8)
        self._local = []
        self._opened = []
        self.ptrs = {}
        for name, nbytes, zero in (("stage", _STAGE_BYTES, False), ("result", _RESULT_BYTES, False),
                                   ("flags", flag_bytes, True)):
            ptr, handle = m.ipc_alloc(nbytes, zero)
            self._local.append(ptr)
            handles = [None] * self.n
            dist.all_gather_object(handles, bytes(handle), group=mode.cpu_group)
            peers = []
            for r, h in enumerate(handles):
                if r == self.me:
                    peers.append(ptr)
                else:
                    q = m.ipc_open(h)
                    self._opened.append(q)
                    peers.append(q)
            self.ptrs[name] = peers
        torch.cuda.synchronize()
        dist.barrier(group=mode.cpu_group)

    def fits(self, M, N):
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        return tiles <= _DONE_CAP and (tiles + self.n - 1) // self.n <= self.owned_cap

    def close(self):
        m = ext.require()
        torch.cuda.synchronize()
        for q in self._opened:
            m.ipc_close(q)
        for p in self._local:
            m.ipc_free(p)
        self._opened, self._local = [], []


def workspace(mode):
    from . import symm
    ws = symm._WORKSPACES.get(mode.name)
    if ws is None:
        ws = Workspace(mode)
        symm._WORKSPACES[mode.name] = ws
    return ws


def _comm_ctas(M, N, K, n):
    """Communication CTAs out of the 148: more of them when the exchange outweighs the local product."""
    if _COMM_CTAS > 0:
        return _COMM_CTAS
    t_gemm = 2.0 * M * N * K / 1.4e15
    t_link = 2.0 * (n - 1) / n * M * N * 2 / 700e9
    frac = t_link / (t_link + t_gemm)
    return int(min(32, max(8, round(148 * frac * 0.15))))


def fused_gemm_all_reduce(a, b, trans_a, trans_b, mode, bias, out_dtype):
    if out_dtype != a.dtype or a.dtype != b.dtype:
        return None
    M = a.shape[1] if trans_a else a.shape[0]
    K = a.shape[0] if trans_a else a.shape[1]
    N = b.shape[0] if trans_b else b.shape[1]
    if N % 8 != 0 or a.shape[1] % 8 != 0 or b.shape[1] % 8 != 0 or mode.world_size > 8:
        return None
    from . import symm
    if not symm.prefer_fused(M, N, K, mode.world_size):
        return None
    ws = workspace(mode)
    if not ws.fits(M, N):
        return None
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    ws.epoch += 1
    m = ext.require()
    ext._count(1)
    m.fused_gemm_all_reduce(a, b, bool(trans_a), bool(trans_b), bias, out, ws.ptrs["stage"], ws.ptrs["result"],
                            ws.ptrs["flags"], _DONE_CAP, ws.me, ws.epoch, _comm_ctas(M, N, K, ws.n),
                            m.status_device_ptr(), TRACE)
    from . import collective
    if collective._profiler is not None:
        collective._profiler.account("fused_gemm_all_reduce", 2 * (ws.n - 1) * M * N * a.element_size() // ws.n)
    return out


def dispatch(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias, out_dtype, keep_gathered):
    live = lambda s: s is not None and s[0].world_size > 1
    if reduce is not None and reduce.world_size > 1 and not live(gather_a) and not live(gather_b) and not live(scatter):
        out = fused_gemm_all_reduce(a, b, trans_a, trans_b, reduce, bias, out_dtype or a.dtype)
        if out is None:
            return None
        return (out, a, b) if keep_gathered else out
    return None
