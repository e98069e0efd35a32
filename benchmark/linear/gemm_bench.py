"""Single-GPU GEMM timing: the tcgen05 kernel of this package against torch.matmul (cuBLAS).

    python benchmark/linear/gemm_bench.py

Products of the GPT-2 XL benchmark (32768 tokens, hidden 1600, MLP 6400): the forward products (one with the fused
bias + GELU epilogue that also writes the pre-activation value), two data-gradient products (B operand MN-major),
two weight-gradient products (both operands MN-major, fp32 output, split-K), and 8192^3.  CUDA events around every
call, median of 10 after 3 warm-ups, a 256 MB scratch write between calls (larger than L2).  The cuBLAS column runs
the same contraction with a 16-bit output; for the GELU row it adds ``torch.nn.functional.gelu`` on the result.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from cubework_b200.ops import ext  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--only", default=None, help="run only the cases whose name contains this text (for profiler captures)")
ap.add_argument("--iters", type=int, default=10)
ap.add_argument("--no-library", action="store_true", help="skip the cuBLAS column")
cli = ap.parse_args()
ext.require()
BF = torch.bfloat16
T = 32768
# name, stored A, stored B, trans_a, trans_b, fused epilogue, fp32 output
CASES = [
    ("8192^3            A B^T", (8192, 8192), (8192, 8192), False, True, None, False),
    ("fwd proj  N=1600 K=1600", (T, 1600), (1600, 1600), False, True, None, False),
    ("fwd qkv   N=4800 K=1600", (T, 1600), (4800, 1600), False, True, None, False),
    ("fwd fc1 + bias + GELU  ", (T, 1600), (6400, 1600), False, True, "gelu", False),
    ("fwd fc2   N=1600 K=6400", (T, 6400), (1600, 6400), False, True, None, False),
    ("dgrad qkv N=1600 K=4800", (T, 4800), (4800, 1600), False, False, None, False),
    ("dgrad fc1 N=1600 K=6400", (T, 6400), (6400, 1600), False, False, None, False),
    ("wgrad fc1 6400x1600 fp32", (T, 6400), (T, 1600), True, False, None, True),
    ("wgrad fc2 1600x6400 fp32", (T, 1600), (T, 6400), True, False, None, True),
]
flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")


def timed(f):
    for _ in range(3):
        f()
    ts = []
    for _ in range(cli.iters):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


for name, sa, sb, ta, tb, act, f32 in CASES:
    if cli.only and cli.only not in name:
        continue
    a = torch.randn(*sa, device="cuda", dtype=BF)
    b = torch.randn(*sb, device="cuda", dtype=BF)
    M, K = (sa[1], sa[0]) if ta else sa
    N = sb[0] if tb else sb[1]
    bias = torch.randn(N, device="cuda") if act else None
    bias16 = bias.to(BF) if act else None

    def ours():
        return ext.gemm(a, b, ta, tb, bias, act, torch.float32 if f32 else BF, act is not None)

    def lib():
        A = a.t() if ta else a
        Bm = b.t() if tb else b
        if act:
            z = torch.addmm(bias16, A, Bm)
            return F.gelu(z), z
        return A @ Bm

    t_own = timed(ours)
    t_lib = t_own if cli.no_library else timed(lib)
    fl = 2.0 * M * N * K
    print(f"{name}: tcgen05 {t_own:.3f} ms {fl / t_own / 1e9:7.1f} TFLOP/s | cuBLAS {t_lib:.3f} ms {fl / t_lib / 1e9:7.1f} TFLOP/s"
          f" | ratio {t_lib / t_own:.3f}", flush=True)
ext.check_status()
