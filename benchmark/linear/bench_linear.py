"""Parallel-Linear microbenchmark: forward + backward of one ``cube_nn.Linear`` per layout.

    torchrun --nproc_per_node N benchmark/linear/bench_linear.py --tp 1d --tp_size N [--kind col|row]
    torchrun --nproc_per_node 4 benchmark/linear/bench_linear.py --tp 2d --tp_size 4
    torchrun --nproc_per_node 8 benchmark/linear/bench_linear.py --tp 3d --tp_size 8

``X[M=16384, K] x W[K, N]`` with ``K = N`` in {4096, 8192, 12288}, bf16, X and W ~ N(0,1).  For each size the
script times fwd+bwd (CUDA events, max over ranks) three times: with the fused kernels, with this package's GEMM
followed by NCCL, and with cuBLAS + NCCL through the same layer code (``CUBEWORK_B200_KERNELS=0``).  It prints ms
and the achieved fraction of the roofline ``max(FLOPs / GEMM peak, NVLink bytes / link bandwidth)``.

``--impl reference`` times the unmodified reference instead (``cubework.module.Linear`` from ``baseline/_ref`` under
its fp16 autocast, i.e. its own NCCL + cuBLAS path: q rounds of broadcast + addmm in 2D, all-gather / matmul /
reduce-scatter in 3D, parallel_2d/_operation.py:15-239, parallel_3d/_operation.py:12-68) on the same shapes and
with the same timing, and prints the same JSON lines.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import cubework_b200 as cube  # noqa: E402
import cubework_b200.module as cube_nn  # noqa: E402
from cubework_b200 import ops  # noqa: E402
from cubework_b200.distributed import ParallelManager as pm  # noqa: E402
from cubework_b200.global_vars import env  # noqa: E402
from cubework_b200.parallel import symm  # noqa: E402
from cubework_b200.parallel.ops_1d import set_parallel_input  # noqa: E402

M = 16384
LINK_GBS = 770.0


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)["bf16_tflops"], "measured"
    except Exception:  # noqa: BLE001
        return 1590.0, "fallback"


def local_input(mode, kind, K, dev):
    tp = pm.TENSOR.world_size
    if mode == "1d":
        k_loc = K // tp if kind == "row" else K
        return torch.randn(M, k_loc, device=dev)
    if mode == "2d":
        q = env.summa_dim
        return torch.randn(M // q, K // q, device=dev)
    d = env.depth_3d
    return torch.randn(M // (d * d), K // d, device=dev)


def link_bytes(mode, kind, K, N):
    """Bytes each GPU must send over NVLink for forward + backward (bf16), the roofline numerator."""
    tp = pm.TENSOR.world_size
    e = 2
    if mode == "1d":
        ar = 2 * (tp - 1) / tp * M * (N if kind == "row" else K) * e   # one all-reduce: row fwd, or col bwd
        return ar
    if mode == "2d":
        q = env.summa_dim
        a, w, y = M / q * K / q * e, K / q * N / q * e, M / q * N / q * e
        fwd = (q - 1) * (a + w)                    # gather A over the row, W down the column
        bwd = (q - 1) * (w + y) + (q - 1) * (a + w)  # dX: gather W, reduce-scatter; dW: gather A, reduce-scatter
        return fwd + bwd
    d = env.depth_3d
    x, w, y = M / d**2 * K / d * e, K / d * N / d**2 * e, M / d**2 * N / d * e
    fwd = (d - 1) * (x + w + y)
    bwd = (d - 1) * (y + w + x)
    return fwd + bwd


def time_fb(layer, x, iters=10, warm=3):
    def once():
        xi = x.detach().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = layer(xi)
        y.backward(torch.ones_like(y))
        layer.zero_grad(set_to_none=True)
    for _ in range(warm):
        once()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        once()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=x.device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def run_reference(args):
    """The reference's ``cubework.module.Linear`` in the requested mode (flags are read from ``sys.argv`` by its own
    ``initialize_distributed``)."""
    import math
    import types
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "baseline", "_ref")
    six = types.ModuleType("torch._six")      # removed in torch 2.x; cubework/utils/clip_grad.py imports `inf` from it
    six.inf = math.inf
    sys.modules["torch._six"] = six
    sys.path.insert(0, root)
    import cubework
    import cubework.module as ref_nn
    from cubework.distributed import ParallelManager as rpm
    from cubework.global_vars import env as renv
    sys.argv = [sys.argv[0], "--tp", args.tensor_parallel, "--tp_size", str(args.tensor_parallel_size)]
    cubework.initialize_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    mode, tp = args.tensor_parallel, rpm.TENSOR.world_size
    peak, src = peaks()
    for K in args.sizes:
        N = K
        if mode == "1d":
            renv.parallel_input_1d = args.kind == "row"
        layer = ref_nn.Linear(K, N).to(dev)
        if mode == "1d":
            x = torch.randn(M, K // tp if args.kind == "row" else K, device=dev)
        elif mode == "2d":
            x = torch.randn(M // renv.summa_dim, K // renv.summa_dim, device=dev)
        else:
            x = torch.randn(M // renv.depth_3d**2, K // renv.depth_3d, device=dev)

        def once():
            xi = x.detach().requires_grad_(True)
            with torch.cuda.amp.autocast(enabled=True):
                y = layer(xi)
            y.backward(torch.ones_like(y))
            layer.zero_grad(set_to_none=True)

        for _ in range(3):
            once()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            once()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if dist.get_rank() == 0:
            print(json.dumps({"impl": "reference", "layout": mode + ("-" + args.kind if mode == "1d" else ""), "tp": tp,
                              "M": M, "K": K, "N": N, "ms": {"reference (fp16 autocast)": round(ms.item(), 4)}}), flush=True)
        del layer
    cubework.destroy_distributed()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", choices=["col", "row"], default="row")
    ap.add_argument("--sizes", type=int, nargs="*", default=[4096, 8192, 12288])
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    if "--impl" in sys.argv and sys.argv[sys.argv.index("--impl") + 1] == "reference":
        ap.add_argument("--tensor_parallel", "--tp", default="1d")
        ap.add_argument("--tensor_parallel_size", "--tp_size", type=int, default=1)
        ap.add_argument("--backend", default="nccl")
        ap.add_argument("--seed", type=int, default=None)
        return run_reference(ap.parse_args())
    args = cube.initialize_distributed(ap)
    dev = torch.device("cuda", torch.cuda.current_device())
    mode, tp = env.mode, pm.TENSOR.world_size
    peak, src = peaks()
    for K in args.sizes:
        N = K
        if mode == "1d":
            set_parallel_input(args.kind == "row")
        layer = cube_nn.Linear(K, N, weight_initializer=cube_nn.init.normal_()).to(dev)
        x = local_input(mode, args.kind, K, dev)
        res = {}
        for label, fused_on in (("fused", True), ("nccl+own-gemm", False)):
            symm._DISABLED = not fused_on
            symm._POLICY = "1" if fused_on else "0"
            res[label] = time_fb(layer, x)
        os.environ["CUBEWORK_B200_KERNELS"] = "0"
        res["nccl+cublas"] = time_fb(layer, x)
        os.environ["CUBEWORK_B200_KERNELS"] = "1"
        flops = 3 * 2.0 * M * K * N / tp
        t_roof = max(flops / (peak * 1e12), link_bytes(mode, args.kind, K, N) / (LINK_GBS * 1e9)) * 1e3
        if dist.get_rank() == 0:
            print(json.dumps({"layout": mode + ("-" + args.kind if mode == "1d" else ""), "tp": tp, "M": M, "K": K, "N": N,
                              "ms": {k: round(v, 4) for k, v in res.items()}, "roofline_ms": round(t_roof, 4),
                              "fraction_of_roofline": {k: round(t_roof / v, 3) for k, v in res.items()},
                              "peak_source": src}), flush=True)
        del layer
    cube.destroy_distributed()


if __name__ == "__main__":
    main()
