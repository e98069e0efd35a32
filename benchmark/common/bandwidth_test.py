"""All-reduce bandwidth probe: ``torchrun --nproc_per_node N benchmark/common/bandwidth_test.py``

Parity: benchmark/common/bandwidth_test.py:1-39 (20 global all-reduces of an fp32 [DIM, 4*DIM] tensor timed with
CUDA events, algorithm GB/s).  Reports the maximum time over ranks.
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import cubework_b200 as cube  # noqa: E402
from cubework_b200.distributed import ParallelManager as pm  # noqa: E402
from cubework_b200.distributed import all_reduce  # noqa: E402
from cubework_b200.utils import get_current_device, get_logger  # noqa: E402

DIM, REPS = 8192, 20

if __name__ == "__main__":
    cube.initialize_distributed()
    dev = get_current_device()
    x = torch.randn(DIM, 4 * DIM, device=dev)
    n = pm.GLOBAL.world_size
    for _ in range(3):
        all_reduce(x, pm.GLOBAL)
    if dev.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(REPS):
            all_reduce(x, pm.GLOBAL)
        e1.record()
        torch.cuda.synchronize()
        secs = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
        secs = secs.item()
    else:
        import time
        t0 = time.perf_counter()
        for _ in range(REPS):
            all_reduce(x, pm.GLOBAL)
        secs = time.perf_counter() - t0
    nbytes = x.numel() * 4
    algo = 2 * (n - 1) / n * nbytes * REPS / secs / 1e9 if n > 1 else 0.0
    get_logger().info(f"all-reduce {nbytes / 2**20:.0f} MiB x {REPS} on {n} ranks: {secs / REPS * 1e3:.3f} ms each, "
                      f"{algo:.1f} GB/s bus bandwidth")
    cube.destroy_distributed()
