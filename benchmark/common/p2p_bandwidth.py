"""Two ranks: bandwidth of the bulk-copy (cp.async.bulk) push / pull data path over NVLink peer memory, and NCCL all-reduce for comparison.
"""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import torch, torch.distributed as dist
import cubework_b200 as cube
from cubework_b200.distributed import ParallelManager as pm
from cubework_b200.ops import ext
from cubework_b200.parallel import symm_impl
cube.initialize_distributed(argv=["--tp", "1d", "--tp_size", "2"])
m = ext.require()
ws = symm_impl.workspace(pm.PARALLEL_1D)
me, peer = ws.me, 1 - ws.me
nbytes = 128 << 20
local = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
def run(name, dst, src, chunk, ctas):
    for _ in range(2): m.bulk_copy(dst, src, nbytes, chunk, ctas)
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5): m.bulk_copy(dst, src, nbytes, chunk, ctas)
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    if me == 0: print(f"{name:14s} chunk={chunk>>10:3d}K ctas={ctas:3d}: {ms:.3f} ms  {nbytes/ms/1e6:.0f} GB/s", flush=True)
for chunk in (8192, 16384, 32768):
    for ctas in (8, 16, 32, 64, 128):
        run("push(l->peer)", ws.ptrs["stage"][peer], local.data_ptr(), chunk, ctas)
        run("pull(peer->l)", local.data_ptr(), ws.ptrs["stage"][peer], chunk, ctas)
run("local", ws.ptrs["stage"][me], local.data_ptr(), 16384, 64)
x = torch.empty(nbytes // 2, dtype=torch.bfloat16, device="cuda")
for _ in range(3): dist.all_reduce(x)
torch.cuda.synchronize(); e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(5): dist.all_reduce(x)
e1.record(); torch.cuda.synchronize()
if me == 0: print(f"nccl all_reduce 128MB: {e0.elapsed_time(e1)/5:.3f} ms")
cube.destroy_distributed()
