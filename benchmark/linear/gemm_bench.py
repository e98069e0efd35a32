"""Single-GPU GEMM timing: the tcgen05 kernel of this package against torch.matmul (cuBLAS) on the shapes of the
GPT-2 XL benchmark and on 8192^3.  CUDA events, 10 iterations after 3 warm-ups; prints ms and TFLOP/s."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402

from cubework_b200.ops import ext  # noqa: E402

ext.require()
SHAPES = [(8192, 8192, 8192), (32768, 1600, 1600), (32768, 6400, 1600), (32768, 4800, 1600), (32768, 1600, 6400),
          (16384, 4096, 2048)]
for (M, N, K) in SHAPES:
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    for name, f in (("tcgen05", lambda: ext.gemm(a, b, False, True, None, None, torch.bfloat16, False)),
                    ("cublas", lambda: a @ b.t())):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            f()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        print(f"{name:8s} {M}x{N}x{K}: {ms:.3f} ms  {2 * M * N * K / ms / 1e9:.1f} TFLOP/s", flush=True)
