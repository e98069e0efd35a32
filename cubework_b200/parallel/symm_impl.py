"""Per-group peer-memory workspaces and the dispatch of fused GEMM + collective launches.

A workspace is a set of ``cudaMalloc`` regions per rank (staging for partial tiles, result tiles, gather
buffers, flags), each created at first use and exchanged as CUDA IPC handles over the group's gloo twin so
every rank holds every peer's pointer.  Flags carry a call epoch that only grows; gather and reduce-scatter
staging regions are used in two halves that alternate with the epoch.  One workspace per process group; its
fused launches are ordered by the stream they run on.
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
STATS = {"gemm_all_reduce": 0, "gather_gemm_scatter": 0}     # fused launches issued by this process
TRACE = None                  # optional int64 [148, 192, 2] CUDA tensor: per-CTA event trace of the next fused launches
GGS_TRACE = None              # optional int64 [148 * 3, 512, 2] CUDA tensor: the same for the gather/scatter kernel


class Workspace:
    """Peer-mapped regions of one process group, created on first use (region creation is collective: every
    rank of the group reaches it at the same call, because the decisions that lead here depend on shapes and
    settings only)."""

    def __init__(self, mode):
        ext.require()
        self.mode = mode
        self.n = mode.world_size
        self.me = mode.local_rank
        self.epoch = 0
        self.owned_cap = min(_RESULT_BYTES // TILE_BYTES, _STAGE_BYTES // (TILE_BYTES * self.n))
        self._local = []
        self._opened = []
        self.ptrs = {}

    def region(self, name, nbytes, zero=False):
        """Every rank's device pointer to the region ``name`` (allocated and exchanged at the first call)."""
        peers = self.ptrs.get(name)
        if peers is not None:
            return peers
        m = ext.require()
        ptr, handle = m.ipc_alloc(nbytes, zero)
        self._local.append(ptr)
        handles = [None] * self.n
        dist.all_gather_object(handles, bytes(handle), group=self.mode.cpu_group)
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
        dist.barrier(group=self.mode.cpu_group)
        return peers

    def halves(self, name, half_bytes):
        """Every rank's pointers to the two halves of a double-buffered region (cached lists: this is on the path
        of every fused call)."""
        key = name + "/halves"
        both = self.ptrs.get(key)
        if both is None:
            base = self.region(name, 2 * half_bytes)
            both = ([p for p in base], [p + half_bytes for p in base])
            self.ptrs[key] = both
        return both

    def all_reduce_regions(self):
        flag_bytes = 4 * (_DONE_CAP * 8 + self.owned_cap * self.n * 8)
        return (self.region("stage", _STAGE_BYTES), self.region("result", _RESULT_BYTES),
                self.region("flags", flag_bytes, True))

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
        self.ptrs = {}


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
    STATS["gemm_all_reduce"] += 1
    stage, result, flags = ws.all_reduce_regions()
    m.fused_gemm_all_reduce(a, b, bool(trans_a), bool(trans_b), bias, out, stage, result, flags, _DONE_CAP, ws.me,
                            ws.epoch, _comm_ctas(M, N, K, ws.n), m.status_device_ptr(), TRACE)
    from . import collective
    if collective._profiler is not None:
        collective._profiler.account("fused_gemm_all_reduce", 2 * (ws.n - 1) * M * N * a.element_size() // ws.n)
    return out


_GATHER_HALF = int(os.environ.get("CUBEWORK_B200_GATHER_MB", "384")) << 20      # per operand role and half
_RS_HALF = int(os.environ.get("CUBEWORK_B200_RS_STAGE_MB", "384")) << 20        # staging of partial tiles, per half
_PUSH_CTAS = int(os.environ.get("CUBEWORK_B200_PUSH_CTAS", "0"))     # 0: chosen per call by _push_ctas
_MAX_PANELS = 2048                                                              # (source, panel) flags per operand
_LOWP = (torch.bfloat16, torch.float16)


def _live(spec):
    return spec is not None and spec[0].world_size > 1


def _plan_gather(t, spec, mn_major):
    """(n, g, panel_rows) for a gathered stored shard ``t`` or None when the kernel's layout rules are not met."""
    mode, g = spec
    n = mode.world_size
    R, C = t.shape
    g = g % 2
    if n > 8 or C % 8 != 0 or n * R * C * 2 > _GATHER_HALF:
        return None
    if g == 1 and (C % 64 != 0 or (mn_major and R % 64 != 0)):
        return None
    panel_rows = 128
    while n * ((R + panel_rows - 1) // panel_rows) > _MAX_PANELS:
        panel_rows *= 2
    return n, g, panel_rows


def _push_ctas(push_bytes, M, N, K, n):
    """Communication CTAs for the operand gathers of one call.  One CTA moves about 40 GB/s (32 KB pieces, a dozen
    in flight), the links carry about 750 GB/s per direction, and every communication CTA is an SM the GEMM loses.
    Sixteen saturate a link between two GPUs (measured: 671 GB/s) and get a shard across before the tiles that
    need it first come up in every layout tried; fewer (sized to the product's duration) starved the layouts whose
    first tiles already read remote data (SUMMA ``ABT`` / ``ATB``: 2.09 / 2.76 ms against 1.84 / 2.38 ms).  With four
    or more sources all links are busy at once and twenty are used."""
    if push_bytes == 0 or n < 2:
        return 1          # nothing is gathered: the kernel launches no communication CTA
    if _PUSH_CTAS > 0:
        return _PUSH_CTAS
    return 16 if n < 4 else 20


def _aligned(t):
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


_ACT_CODE = {None: 0, "gelu": 1, "relu": 2}


def fused_gather_gemm_scatter(a, b, trans_a, trans_b, gather_a, gather_b, scatter, bias, out_dtype, keep_gathered,
                              act=None, pre_act_out=False):
    """One launch of ``ops/csrc/gather_gemm_scatter_sm100.cu``; None when the shapes are outside what it covers.

    ``keep_gathered``: False, True (the gathered operands are returned as tensors of their own) or ``"view"``
    (returned as views of the workspace, valid until the next fused call on the same group: for a consumer that
    runs next on the same stream).  With ``pre_act_out`` the value before ``act`` is returned after the output."""
    if a.dtype != b.dtype or a.dtype not in _LOWP or out_dtype not in (a.dtype, torch.float32):
        return None
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] % 8 != 0 or b.shape[1] % 8 != 0:
        return None
    ga = _plan_gather(a, gather_a, trans_a) if _live(gather_a) else None
    gb = _plan_gather(b, gather_b, not trans_b) if _live(gather_b) else None
    if (_live(gather_a) and ga is None) or (_live(gather_b) and gb is None):
        return None
    mul = lambda plan, dim: plan[0] if plan is not None and plan[1] == dim else 1
    a_rows, a_cols = a.shape[0] * mul(ga, 0), a.shape[1] * mul(ga, 1)
    b_rows, b_cols = b.shape[0] * mul(gb, 0), b.shape[1] * mul(gb, 1)
    M, K = (a_cols, a_rows) if trans_a else (a_rows, a_cols)
    N, Kb = (b_rows, b_cols) if trans_b else (b_cols, b_rows)
    assert K == Kb, (a.shape, b.shape, trans_a, trans_b)
    Ms, Ns, sc = M, N, None
    if _live(scatter):
        smode, sdim = scatter[0], scatter[1] % 2
        sn = smode.world_size
        if sn > 8:
            return None
        if sdim == 0:
            if M % sn != 0:
                return None
            Ms = M // sn
            if trans_a and (Ms % 8 != 0 or (ga is not None and ga[1] == 1 and Ms % 64 != 0)):
                return None
        else:
            if N % sn != 0 or (N // sn) % 8 != 0:
                return None
            Ns = N // sn
            if not trans_b and gb is not None and gb[1] == 1 and Ns % 64 != 0:
                return None
        owned = ((Ms + 127) // 128) * ((Ns + 255) // 256)
        if owned * sn * TILE_BYTES > _RS_HALF:
            return None
        sc = (smode, sdim, sn)
    from . import symm
    if not symm.prefer_fused_gather_scatter(M, N, K):
        return None
    m = ext.require()
    a, b = _aligned(a), _aligned(b)
    # one epoch step per distinct group that takes part in this call
    spaces = {}
    for spec in (gather_a if ga else None, gather_b if gb else None, scatter if sc else None):
        if spec is not None and spec[0].name not in spaces:
            ws = workspace(spec[0])
            ws.epoch += 1
            spaces[spec[0].name] = ws

    def gather_args(plan, spec, role):
        if plan is None:
            return [], [], []
        ws = spaces[spec[0].name]
        bufs = ws.halves(role, _GATHER_HALF)[ws.epoch & 1]
        flags = ws.region(role + "_flags", 4 * 8 * _MAX_PANELS, True)
        return [plan[0], ws.me, plan[1], plan[2], ws.epoch], bufs, flags

    ga_cfg, ga_bufs, ga_flags = gather_args(ga, gather_a, "ga")
    gb_cfg, gb_bufs, gb_flags = gather_args(gb, gather_b, "gb")
    sc_cfg, sc_stage, sc_flags = [], [], []
    if sc is not None:
        ws = spaces[sc[0].name]
        sc_stage = ws.halves("rs_stage", _RS_HALF)[ws.epoch & 1]
        sc_flags = ws.region("rs_flags", 4 * 8 * (_RS_HALF // TILE_BYTES), True)
        sc_cfg = [sc[1], sc[2], ws.me, ws.epoch]
    out = torch.empty((Ms, Ns), dtype=out_dtype, device=a.device)
    z = torch.empty((Ms, Ns), dtype=a.dtype, device=a.device) if pre_act_out else None
    push_bytes = sum((plan[0] - 1) * t.numel() * t.element_size() for plan, t in ((ga, a), (gb, b)) if plan is not None)
    comm_ctas = _push_ctas(push_bytes, M, N, K, max(plan[0] for plan in (ga, gb) if plan is not None) if (ga or gb) else 1)
    ext._count(1)
    STATS["gather_gemm_scatter"] += 1
    from . import collective
    prof = collective._profiler
    ev0 = ev1 = None
    if prof is not None:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    m.gather_gemm_scatter(a, b, bool(trans_a), bool(trans_b), bias, out, ga_cfg, ga_bufs, ga_flags, gb_cfg, gb_bufs,
                          gb_flags, sc_cfg, sc_stage, sc_flags, comm_ctas, m.status_device_ptr(), _ACT_CODE[act], z,
                          GGS_TRACE)
    if prof is not None:
        ev1.record()
        moved = 0
        for plan, t in ((ga, a), (gb, b)):
            if plan is not None:
                moved += (plan[0] - 1) * t.numel() * t.element_size()
        if sc is not None:
            moved += (sc[2] - 1) * Ms * Ns * a.element_size()
        prof.account("fused_gather_gemm_scatter", moved, ev0, ev1)
    res = (out, ) if not pre_act_out else (out, z)
    if not keep_gathered:
        return res if pre_act_out else out

    def gathered(plan, cfg, bufs, t):
        if plan is None:
            return t
        n, g = plan[0], plan[1]
        R, C = t.shape
        # the buffer holds the other ranks' shards (the own one only in some layouts): place the own one too
        full = m.as_tensor(bufs[cfg[1]], [n, R, C], t.dtype, t.device.index)
        if keep_gathered != "view":
            full = full.clone()
        full[cfg[1]].copy_(t)
        return full.reshape(n * R, C) if g == 0 else full.permute(1, 0, 2).reshape(R, n * C)

    return res + (gathered(ga, ga_cfg, ga_bufs, a), gathered(gb, gb_cfg, gb_bufs, b))


def dispatch(a, b, trans_a, trans_b, gather_a, gather_b, scatter, reduce, bias, out_dtype, keep_gathered, act=None,
             pre_act_out=False):
    live = lambda s: s is not None and s[0].world_size > 1
    if reduce is not None and reduce.world_size > 1 and not live(gather_a) and not live(gather_b) and not live(scatter):
        if act is not None or pre_act_out:
            return None
        out = fused_gemm_all_reduce(a, b, trans_a, trans_b, reduce, bias, out_dtype or a.dtype)
        if out is None:
            return None
        return (out, a, b) if keep_gathered else out
    if (reduce is None or reduce.world_size == 1) and (live(gather_a) or live(gather_b) or live(scatter)):
        return fused_gather_gemm_scatter(a, b, trans_a, trans_b, gather_a, gather_b, scatter, bias,
                                         out_dtype or a.dtype, keep_gathered, act, pre_act_out)
    return None
