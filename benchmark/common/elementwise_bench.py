"""Times the memory-bound kernels of the transformer block on the GPT-2 XL shapes (one B200).

    python benchmark/common/elementwise_bench.py

LayerNorm forward / backward fused with the residual add (32768 x 1600) and the GELU backward fused with the bias
gradient (32768 x 6400), bf16; CUDA events, median of 8 after 3 warm-ups, a 256 MB scratch write between calls.
The bandwidth figure counts every tensor the kernel has to read or write once.
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402

from cubework_b200.ops import ext  # noqa: E402

ext.require()
M, H, F = 32768, 1600, 6400
BF = torch.bfloat16
flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")


def timed(f, n=8):
    for _ in range(3):
        f()
    ts = []
    for _ in range(n):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        f()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


x = torch.randn(M, H, device="cuda", dtype=BF)
res = torch.randn(M, H, device="cuda", dtype=BF)
dy = torch.randn(M, H, device="cuda", dtype=BF)
g, b = torch.randn(H, device="cuda"), torch.randn(H, device="cuda")
_, mean, rstd = ext.layer_norm_fwd(x, g, b, 1e-5)[:3]
ms = timed(lambda: ext.layer_norm_fwd(x, g, b, 1e-5, residual=res))
print(f"layer_norm_fwd + residual   {M} x {H}: {ms * 1e3:7.1f} us  {4 * M * H * 2 / ms / 1e9:5.2f} TB/s")
ms = timed(lambda: ext.layer_norm_bwd(dy, x, mean, rstd, g, dres=res))
print(f"layer_norm_bwd + residual   {M} x {H}: {ms * 1e3:7.1f} us  {4 * M * H * 2 / ms / 1e9:5.2f} TB/s  (with the column sums)")
z = torch.randn(M, F, device="cuda", dtype=BF)
dz = torch.randn(M, F, device="cuda", dtype=BF)
ms = timed(lambda: ext.act_backward(dz, z, "gelu", True))
print(f"gelu backward + bias grad   {M} x {F}: {ms * 1e3:7.1f} us  {3 * M * F * 2 / ms / 1e9:5.2f} TB/s  (with the column sums)")
ext.check_status()
