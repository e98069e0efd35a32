#!/usr/bin/env python
"""Headline benchmark: GPT-2 XL-shape training throughput (tokens/s) under 1D tensor parallelism.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...          # the unmodified reference from baseline/_ref

Config (both arms): 48 layers, hidden 1600, MLP 6400, vocab 50304, sequence 1024, global batch 32, 1D tensor
parallel over all N GPUs (strong scaling: the global batch is fixed), AdamW, gradient clipping 1.0, dropout 0,
synthetic token ids, random-init weights N(0, 0.02).  Heads: 64 x 25 (the reference's ``gpt2_xl`` preset; 25
heads would not divide 8-way tensor parallelism).  Activation checkpointing is ON in both arms
(``ACTIVATION_CHECKPOINTING``): the reference's default is off, but its materialised ``[batch, heads, T, T]``
attention scores of 48 layers do not fit one GPU at this batch without it, and both arms must run one
configuration.  This framework's step without checkpointing is timed too and reported under ``extra``.

This arm runs the 1D layers with row-sharded activations between the linear pairs (``sequence_parallel``):
all-gather -> GEMM and GEMM -> reduce-scatter inside one kernel each over NVLink peer memory; ``fused_per_step``
and ``nccl_per_step`` in the printed line count, inside the timed region, the fused launches and what still
went through NCCL (calls and payload bytes per kind).

One step = forward + backward + clip + optimizer step + zero_grad.  `value` is timed on the device with CUDA
events around exactly K steps whose inputs already sit on the device; `e2e` repeats the K steps through the
public Trainer API with a pinned-host -> device copy of every batch and a device -> host read of every loss.
Both are the max over ranks.  The working set (weights + activations, tens of GB) is far larger than L2, so no
explicit L2 flush is needed between steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(vocab_size=50304, max_position_embeddings=1024, hidden_size=1600, num_heads=64, intermediate_size=6400,
             depth=48)
SEQ, GLOBAL_BATCH = 1024, 32
ACTIVATION_CHECKPOINTING = True   # one value for both arms (see the module docstring)
BASELINE_PUBLISHED = None   # the reference publishes no number for this (or any) configuration


def _model_name():
    h = MODEL["num_heads"]
    return f"GPT-2 XL-shape (48L, hidden 1600, {h} heads x {MODEL['hidden_size'] // h}, MLP 6400, vocab 50304)"


def _env_defaults(n):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ:
        if n != 1:
            raise SystemExit("for --gpus > 1 launch with torch.distributed.run (one rank per GPU)")
        import socket
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_PORT=str(port))


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs (rank 0 only)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                power.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def _time_steps(torch, dist, step_fn, steps):
    """Barrier + sync, K steps between two CUDA events, sync + barrier; returns max-over-ranks milliseconds."""
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def _synthetic_batches(torch, n_distinct, micro_batch):
    g = torch.Generator().manual_seed(1234)
    out = []
    for _ in range(n_distinct):
        ids = torch.randint(0, MODEL["vocab_size"], (micro_batch, SEQ), generator=g)
        out.append(dict(input_ids=ids.pin_memory(), attention_mask=torch.ones(micro_batch, SEQ).pin_memory(),
                        labels=ids.clone().pin_memory()))
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    import cubework_b200 as cube
    from cubework_b200.engine import Trainer
    from cubework_b200.models import gpt2
    from cubework_b200.ops import ext
    from cubework_b200.optim import FusedAdamW
    from cubework_b200.parallel import collective, symm_impl
    n = args.gpus
    cube.initialize_distributed(argv=["--tp", "1d", "--tp_size", str(n)])
    dev = torch.device("cuda", torch.cuda.current_device())
    model = gpt2.GPT2(dropout=0.0, embedding_dropout=0.0, attention_dropout=0.0, checkpoint=ACTIVATION_CHECKPOINTING,
                      init_std=0.02, sequence_parallel=True, **MODEL).to(dev)
    opt = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    trainer = Trainer(model, gpt2.GPT2LMLoss(), opt, amp_dtype=torch.bfloat16, clip=1.0)
    host_batches = _synthetic_batches(torch, 4, GLOBAL_BATCH)
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches]

    # First step: every rank checks the kernels' status word; if any rank saw a bounded wait expire (a peer that
    # did not show up in a fused exchange) all ranks switch to the unfused composition (own GEMM + NCCL) together
    # and say so in the printed line, instead of measuring a broken run.
    from cubework_b200.parallel import symm
    fused_error = None
    trainer.step(dev_batches[0])
    torch.cuda.synchronize()
    try:
        ext.check_status()
        bad = 0
    except RuntimeError as e:
        bad, fused_error = 1, str(e)
    flag = torch.tensor([bad], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if flag.item():
        fused_error = fused_error or "a peer reported a device-side timeout"
        symm._DISABLED = True
        symm.invalidate_all()
    for i in range(args.warmup):
        trainer.step(dev_batches[i % len(dev_batches)])
    torch.cuda.synchronize()
    ext.check_status()

    sampler = ClockSampler(torch.cuda.current_device()) if dist.get_rank() == 0 else None
    if sampler:
        sampler.start()
    launches0 = ext.launch_count()
    fused0 = dict(symm_impl.STATS)
    nccl0 = collective.stats_snapshot()
    ms = _time_steps(torch, dist, lambda i: trainer.step(dev_batches[i % len(dev_batches)]), args.steps)
    launches = ext.launch_count() - launches0
    fused = {k: (v - fused0.get(k, 0)) / args.steps for k, v in symm_impl.STATS.items()}
    nccl = {k: {"calls": (v[0] - nccl0.get(k, (0, 0))[0]) / args.steps,
                "mbytes": round((v[1] - nccl0.get(k, (0, 0))[1]) / args.steps / 1e6, 3)}
            for k, v in collective.stats_snapshot().items()}
    clocks = sampler.stop() if sampler else None
    ext.check_status()

    # end to end through the public API: pinned host batch -> device every step, loss read back every step
    trainer.h2d_bytes = 0
    losses = []

    def e2e_step(i):
        losses.append(trainer.step(host_batches[i % len(host_batches)]).item())

    e2e_ms = _time_steps(torch, dist, e2e_step, args.steps)
    ext.check_status()
    # the same model without activation checkpointing (this framework does not need it at this size)
    for blk in model.blocks:
        blk.checkpoint = False
    for i in range(2):
        trainer.step(dev_batches[i % len(dev_batches)])
    nockpt_ms = _time_steps(torch, dist, lambda i: trainer.step(dev_batches[i % len(dev_batches)]), args.steps)
    ext.check_status()
    tokens = GLOBAL_BATCH * SEQ * args.steps
    if dist.get_rank() == 0:
        value = tokens / (ms / 1e3)
        line = {
            "metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None, "dtype": "bf16",
            "data": "synthetic token ids (uniform), random-init weights N(0,0.02)", "impl": "ours",
            "config": {"model": _model_name(),
                       "global_batch": GLOBAL_BATCH, "seq_len": SEQ, "parallelism": f"tp{n} (1D)",
                       "optimizer": "AdamW + clip 1.0", "activation_checkpointing": ACTIVATION_CHECKPOINTING,
                       "l2": "working set >> L2 (126 MB); no flush between steps"},
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": trainer.h2d_bytes // args.steps, "d2h_bytes_per_step": 4,
                    "last_loss": losses[-1]},
            "gpu_launches": launches,
            "sequence_parallel": n > 1,
            "fused_kernels": fused_error is None,
            **({"fused_error": fused_error} if fused_error else {}),
            "fused_per_step": fused,
            "nccl_per_step": nccl,
            "extra": {"activation_checkpointing_off": {"value": tokens / (nockpt_ms / 1e3), "unit": "tokens/s",
                                                       "ms_per_step": nockpt_ms / args.steps}},
        }
        print(json.dumps(line), flush=True)
    cube.destroy_distributed()


def run_reference(args):
    """The unmodified reference (baseline/_ref): its GPT2 model class, layers, loss, clip and its fp16 AMP loop."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(why):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        sys.exit(0)

    if not os.path.isdir(os.path.join(ref_root, "cubework")):
        unavailable("baseline/_ref/cubework is not installed")
    import math
    import types

    import torch
    if not torch.cuda.is_available():
        unavailable("the reference requires a CUDA device (ParallelMode.init reads the CUDA RNG state)")
    # the only shim: torch._six was removed in torch 2.x and cubework/utils/clip_grad.py imports `inf` from it
    six = types.ModuleType("torch._six")
    six.inf = math.inf
    sys.modules["torch._six"] = six
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "benchmark", "gpt2"))
    try:
        import cubework
        import cubework.module as cube_nn  # noqa: F401
        from cubework.utils import clip_grad_norm
        import gpt2 as ref_gpt2
    except Exception as e:  # noqa: BLE001
        unavailable(f"import of the reference failed: {type(e).__name__}: {str(e)[:160]}")
    import torch.distributed as dist
    n = args.gpus
    sys.argv = [sys.argv[0], "--tp", "1d", "--tp_size", str(n)]
    cubework.initialize_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    model = ref_gpt2.GPT2(dropout=0.0, embedding_dropout=0.0, attention_dropout=0.0,
                          checkpoint=ACTIVATION_CHECKPOINTING, **MODEL).to(dev)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    criterion = ref_gpt2.GPT2LMLoss()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    scaler = torch.cuda.amp.GradScaler()
    host_batches = _synthetic_batches(torch, 4, GLOBAL_BATCH)
    dev_batches = [{k: v.to(dev) for k, v in b.items()} for b in host_batches]
    h2d = [0]

    def step(batch, from_host):
        if from_host:
            h2d[0] += sum(v.numel() * v.element_size() for v in batch.values())
            batch = {k: v.to(dev, non_blocking=True) for k, v in batch.items()}
        labels = batch["labels"]
        with torch.cuda.amp.autocast(enabled=True):
            out = model(input_ids=batch["input_ids"], attention_mask=batch["attention_mask"])
            loss = criterion(out, labels)
        scaler.scale(loss).backward()
        scaler.unscale_(opt)
        clip_grad_norm(model.parameters(), 1.0)
        scaler.step(opt)
        scaler.update()
        opt.zero_grad()
        return loss

    model.train()
    for i in range(args.warmup):
        step(dev_batches[i % 4], False)
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device()) if dist.get_rank() == 0 else None
    if sampler:
        sampler.start()
    ms = _time_steps(torch, dist, lambda i: step(dev_batches[i % 4], False), args.steps)
    clocks = sampler.stop() if sampler else None
    losses = []
    e2e_ms = _time_steps(torch, dist, lambda i: losses.append(step(host_batches[i % 4], True).item()), args.steps)
    tokens = GLOBAL_BATCH * SEQ * args.steps
    if dist.get_rank() == 0:
        value = tokens / (ms / 1e3)
        print(json.dumps({
            "metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16 autocast + GradScaler (the reference's ops cast to fp16 themselves)",
            "data": "synthetic token ids (uniform), random-init weights N(0,0.02)", "impl": "reference",
            "config": {"model": _model_name(),
                       "global_batch": GLOBAL_BATCH, "seq_len": SEQ, "parallelism": f"tp{n} (1D)",
                       "optimizer": "AdamW + clip 1.0", "activation_checkpointing": ACTIVATION_CHECKPOINTING,
                       "l2": "working set >> L2 (126 MB); no flush between steps"},
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d[0] // args.steps, "d2h_bytes_per_step": 4, "last_loss": losses[-1]},
            "gpu_launches": 0,
        }), flush=True)
    cubework.destroy_distributed()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--heads", type=int, default=MODEL["num_heads"],
                    help="attention heads (default 64 x 25, the reference's gpt2_xl preset; 25 gives 25 x 64, which "
                         "only 1-GPU runs can use: 25 heads do not divide over 2, 4 or 8 ranks)")
    args = ap.parse_args()
    MODEL["num_heads"] = args.heads
    args.warmup = max(args.warmup, 3)
    _env_defaults(args.gpus)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
