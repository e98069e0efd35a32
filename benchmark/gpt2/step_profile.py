"""Per-kernel time table of one free-running GPT-2 XL-shape training step (1D tensor parallel over all ranks).

    python benchmark/gpt2/step_profile.py [--depth 8] [--ckpt] [--no-sp]
    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmark/gpt2/step_profile.py ...

A model with the benchmark's layer shapes (hidden 1600, 64 heads x 25, MLP 6400, vocab 50304, sequence 1024, global
batch 32) but ``--depth`` layers is trained for a few steps; the script prints the step time from CUDA events
(no profiler attached), the host time needed to enqueue a step, and then, from one step recorded with
``torch.profiler`` (CUPTI activity records, every rank runs freely), the time per kernel summed over its launches
on rank 0.  Kernel times taken this way are the real, overlapped ones; compare shares, and use the event-timed
step for absolute numbers.
"""
import argparse
import collections
import os
import re
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from torch.profiler import ProfilerActivity, profile  # noqa: E402

import cubework_b200 as cube  # noqa: E402
from cubework_b200.engine import Trainer  # noqa: E402
from cubework_b200.models import gpt2  # noqa: E402
from cubework_b200.optim import FusedAdamW  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=8)
    ap.add_argument("--ckpt", action="store_true", help="activation checkpointing per block")
    ap.add_argument("--no-sp", action="store_true", help="replicated activations between the linear pairs")
    ap.add_argument("--top", type=int, default=24)
    args = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ:
        from cubework_b200.utils import free_port
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_PORT=str(free_port()))
    n = int(os.environ["WORLD_SIZE"])
    cube.initialize_distributed(argv=["--tp", "1d", "--tp_size", str(n)])
    dev = torch.device("cuda", torch.cuda.current_device())
    model = gpt2.GPT2(vocab_size=50304, max_position_embeddings=1024, hidden_size=1600, num_heads=64,
                      intermediate_size=6400, depth=args.depth, dropout=0.0, embedding_dropout=0.0, init_std=0.02,
                      checkpoint=args.ckpt, sequence_parallel=not args.no_sp).to(dev)
    trainer = Trainer(model, gpt2.GPT2LMLoss(), FusedAdamW(model.parameters(), lr=1e-4), amp_dtype=torch.bfloat16, clip=1.0)
    ids = torch.randint(0, 50304, (32, 1024), device=dev)
    batch = dict(input_ids=ids, attention_mask=torch.ones(32, 1024, device=dev), labels=ids)
    for _ in range(3):
        trainer.step(batch)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        trainer.step(batch)
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / 3
    t0 = time.perf_counter()
    for _ in range(3):
        trainer.step(batch)
    host_ms = (time.perf_counter() - t0) / 3 * 1e3
    torch.cuda.synchronize()
    dist.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.step(batch)
        torch.cuda.synchronize()
    if dist.get_rank() == 0:
        agg, total = collections.defaultdict(lambda: [0, 0.0]), 0.0
        for ev in prof.events():
            if ev.device_type == torch.autograd.DeviceType.CUDA:
                name = re.sub(r"\(.*", "", ev.name)[:100]
                agg[name][0] += 1
                agg[name][1] += ev.device_time
                total += ev.device_time
        print(f"ranks {n}, depth {args.depth}, checkpointing {args.ckpt}, row-sharded activations {not args.no_sp}: "
              f"step {step_ms:.2f} ms (CUDA events), host enqueue {host_ms:.2f} ms per step, kernel time summed "
              f"{total / 1e3:.2f} ms")
        for name, (count, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:args.top]:
            print(f"{us / 1e3:9.3f} ms {100 * us / total:5.1f} %  x{count:4d}  avg {us / count:8.1f} us  {name}")
    cube.destroy_distributed()


if __name__ == "__main__":
    main()
