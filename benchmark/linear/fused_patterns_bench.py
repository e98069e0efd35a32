"""Fused gather -> GEMM -> reduce-scatter kernel vs. the same product composed from NCCL collectives and the
plain tcgen05 GEMM, for the operand layouts of the 2D (SUMMA) and 3D linears.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmark/linear/fused_patterns_bench.py

All ranks form one 1D group that plays every role (gather group of A, of B, scatter group), which is what a
row / column / cube axis is to the kernel.  Times are CUDA-event times, max over ranks, median of ``--iters``
calls after warm-up; every call works on operands larger than a few MB and the calls of one pattern alternate
with an L2-sized scratch write.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import cubework_b200 as cube  # noqa: E402
from cubework_b200.distributed import ParallelManager as pm  # noqa: E402
from cubework_b200.ops import ext  # noqa: E402
from cubework_b200.parallel import fused, symm  # noqa: E402


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        flush.add_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    t = torch.tensor(sorted(ts)[len(ts) // 2], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--sizes", type=int, nargs="+", default=[4096, 8192])
    args = ap.parse_args()
    n = int(os.environ["WORLD_SIZE"])
    cube.initialize_distributed(argv=["--tp", "1d", "--tp_size", str(n)])
    mode = pm.PARALLEL_1D
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)
    M = args.rows
    rows = []
    for H in args.sizes:
        # name, stored A, stored B, trans_a, trans_b, gather_a, gather_b, scatter, out dtype
        pats = [
            ("2d_AB  gatherK(A) gatherK(B)", (M, H // n), (H // n, H), False, False, 1, 0, None, None),
            ("2d_ABT gatherN(B) scatterN", (M, H), (H // n, H), False, True, None, 0, 1, None),
            ("2d_ATB gatherM(A^T) scatterM", (M, H // n), (M, H), True, False, 1, None, 0, torch.float32),
            ("3d_fwd gatherM(X) gatherN(W) scatterM", (M // n, H), (H // n, H), False, True, 0, 0, 0, None),
            ("3d_dX  scatterM", (M, H), (H, H), False, False, None, None, 0, None),
        ]
        for name, sa, sb, ta, tb, ga, gb, sc, odt in pats:
            a = torch.randn(sa, device=dev).bfloat16()
            b = torch.randn(sb, device=dev).bfloat16()
            kw = dict(gather_a=None if ga is None else (mode, ga), gather_b=None if gb is None else (mode, gb),
                      scatter=None if sc is None else (mode, sc), out_dtype=odt)
            res = {}
            for label, pol in (("nccl+gemm", "0"), ("fused", "1")):
                symm._POLICY, symm._DISABLED = pol, pol == "0"
                res[label] = timed(lambda: fused.gather_gemm_reduce(a, b, ta, tb, **kw), args.iters, flush)
                ext.check_status()
            a_rows = sa[0] * (n if ga == 0 else 1)
            a_cols = sa[1] * (n if ga == 1 else 1)
            b_rows = sb[0] * (n if gb == 0 else 1)
            b_cols = sb[1] * (n if gb == 1 else 1)
            m_, k_ = (a_cols, a_rows) if ta else (a_rows, a_cols)
            n_ = b_rows if tb else b_cols
            flops = 2.0 * m_ * n_ * k_
            link = 0
            if ga is not None:
                link = max(link, (n - 1) * sa[0] * sa[1] * 2)
            if gb is not None:
                link = max(link, (n - 1) * sb[0] * sb[1] * 2)
            if sc is not None:
                link += (n - 1) * m_ * n_ * 2 // n
            roof_ms = max(flops / 1.6117e15, link / 770e9) * 1e3
            rows.append({"pattern": name, "M": m_, "N": n_, "K": k_, "ranks": n, "nccl_gemm_ms": round(res["nccl+gemm"], 4),
                         "fused_ms": round(res["fused"], 4), "roofline_ms": round(roof_ms, 4),
                         "fused_frac_of_roofline": round(roof_ms / res["fused"], 3)})
            if dist.get_rank() == 0:
                print(json.dumps(rows[-1]), flush=True)
    cube.destroy_distributed()


if __name__ == "__main__":
    main()
