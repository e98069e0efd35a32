"""Shared training driver behind ``benchmark/{gpt2,opt,vit}/train.py``.

Parity: benchmark/gpt2/train.py:44-376 (and the near-identical opt / vit drivers): framework + benchmark
flags on one parser, gradient accumulation (global batch / micro batch / DP size), mixed precision, gradient
clipping, LR schedule, per-phase timing, progress bar with running loss / lr / throughput / TFLOPS, epoch
summary (loss, step time, samples/s, tokens/s or images/s, model TFLOPS, peak / state / activation memory,
communication time / share / algorithm bandwidth), optional evaluation with the family's metric, per-rank log
files.  Added: sharded checkpoint save / resume (``--save_dir``, ``--resume_step``), synthetic data when no
dataset path is given (the default: these machines have no network), phase timers (data / fwd / bwd / opt) on CUDA
events instead of host clocks with device-wide synchronisation.  With ``--dataset_path`` the family's real-data
pipeline (:mod:`cubework_b200.utils.datasets`) feeds the loop, and ``--eval`` runs a separate pass over the held-out
split (the reference's ``_test``, train.py:187-270); with synthetic data the evaluation batches come from a second
generator that the training loop never sees.
"""
import argparse
import time

import torch
import torch.distributed as dist

import cubework_b200 as cube
from cubework_b200.distributed import ParallelManager as pm
from cubework_b200.engine import Trainer
from cubework_b200.parallel.collective import all_reduce
from cubework_b200.parallel.ddp import DataParallel
from cubework_b200.utils import (CommProfiler, calc_model_size, calc_tflops, checkpoint, get_current_device,
                                 get_logger, write_logger_to_file)


def get_parser(description, default_model, token_unit="tokens"):
    p = argparse.ArgumentParser(description=description)
    p.add_argument("-m", "--model_name", default=default_model)
    p.add_argument("--seq_length", type=int, default=512)
    p.add_argument("--dataset_path", default=None, help="omit for synthetic data")
    p.add_argument("--tokenizer_path", default=None)
    p.add_argument("--global_batch_size", "--bs", type=int, default=32)
    p.add_argument("--micro_batch_size", "--micro_bs", type=int, default=None)
    p.add_argument("--num_epochs", "--n_epoch", type=int, default=1)
    p.add_argument("--steps_per_epoch", "--n_step", type=int, default=20)
    p.add_argument("--warmup_steps", "--n_warm", type=int, default=0)
    p.add_argument("--learning_rate", "--lr", type=float, default=1e-4)
    p.add_argument("--weight_decay", type=float, default=1e-2)
    p.add_argument("--eval", dest="do_validation", action="store_true")
    p.add_argument("--n_eval", dest="validation_interval", type=int, default=1)
    p.add_argument("--ckpt", dest="use_activation_checkpoint", action="store_true")
    p.add_argument("--clip", dest="gradient_clipping", type=float, default=0.0)
    p.add_argument("--amp", dest="use_mixed_precision", action="store_true")
    p.add_argument("--amp_dtype", choices=["bf16", "fp16"], default="bf16")
    p.add_argument("--fp16_initial_scale", type=float, default=2**15)
    p.add_argument("--fp16_growth_factor", type=float, default=2.0)
    p.add_argument("--fp16_backoff_factor", type=float, default=0.5)
    p.add_argument("--fp16_growth_interval", type=int, default=1000)
    p.add_argument("--num_workers", type=int, default=0, help="data loader workers of the real-data pipelines")
    p.add_argument("--optimizer", choices=["adamw", "sgd"], default=None)
    p.add_argument("--prof_comm", dest="use_comm_profiler", action="store_true")
    p.add_argument("--log_file", default=None)
    p.add_argument("--save_dir", default=None, help="write a sharded checkpoint at the end of every epoch")
    p.add_argument("--resume_step", type=int, default=None)
    p.add_argument("--dropout", type=float, default=None)
    p.add_argument("--fsdp", action="store_true",
                   help="shard parameters, gradients and optimizer state over the data-parallel group (one unit per block)")
    p.set_defaults(token_unit=token_unit)
    return p


def _dp_mean(value):
    t = torch.tensor([float(value)], device=get_current_device())
    if pm.DATA.is_initialized() and pm.DATA.world_size > 1:
        t = all_reduce(t, pm.DATA) / pm.DATA.world_size
    return t.item()


class PhaseTimer:
    """Accumulates phase durations from CUDA events; one synchronisation per report, none per step.  A phase is the
    span between the device reaching its first and its last enqueued operation, so phases overlap nothing and add
    up to the step."""

    def __init__(self, use_cuda):
        self.use_cuda = use_cuda
        self.reset()

    def reset(self):
        self.open, self.spans = {}, {}

    def start(self, name):
        if self.use_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.open[name] = e
        else:
            self.open[name] = time.perf_counter()

    def stop(self, name):
        if self.use_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.spans.setdefault(name, []).append((self.open.pop(name), e))
        else:
            self.spans.setdefault(name, []).append(time.perf_counter() - self.open.pop(name))

    def totals(self):
        if self.use_cuda:
            torch.cuda.synchronize()
            return {k: sum(a.elapsed_time(b) for a, b in v) / 1e3 for k, v in self.spans.items()}
        return {k: sum(v) for k, v in self.spans.items()}


def _test(epoch, trainer, test_loader, metric, args, tokens_per_sample, use_cuda, logger):
    """One pass over the held-out data: mean loss, the family's metric, evaluation throughput (DATA-group totals)."""
    metric.reset()
    timer = PhaseTimer(use_cuda)
    losses, n_batches, samples = [], 0, 0
    limit = len(test_loader) if hasattr(test_loader, "__len__") else None
    it = iter(test_loader)
    timer.start("eval")
    while limit is None or n_batches < limit:
        try:
            batch = next(it)
        except StopIteration:
            break
        out, targets, loss = trainer.evaluate(batch)
        metric(out, targets, loss)
        losses.append(loss.detach().float())
        first = next(v for v in batch.values() if torch.is_tensor(v))
        samples += first.shape[0]
        n_batches += 1
    timer.stop("eval")
    secs = max(timer.totals().get("eval", 0.0), 1e-9)
    mean_loss = _dp_mean(torch.stack(losses).mean().item()) if losses else float("nan")
    total = samples * pm.DATA.world_size
    logger.info(f"[Epoch {epoch} / Test]: Loss = {mean_loss:.4f} | {metric.name} = {metric.to_str()} | "
                f"{n_batches} batches, {total / secs:.2f} samples/sec, {total * tokens_per_sample / secs:.1f} "
                f"{args.token_unit}/sec")
    return mean_loss


def run(args, family):
    """``family`` provides ``build(args) -> (model, criterion, metric, make_batch, tokens_per_sample)``."""
    logger = get_logger()
    if args.log_file:
        write_logger_to_file(args.log_file)
    dev = get_current_device()
    model, criterion, metric, make_batch, tokens_per_sample = family.build(args)
    model = model.to(dev)
    if getattr(args, "fsdp", False):
        from cubework_b200.models import gpt2 as _g, opt as _o, vit as _v
        from cubework_b200.parallel.fsdp import FullyShardedDataParallel
        model = FullyShardedDataParallel(model, unit_classes=(_g.GPT2Block, _o.OPTDecoderLayer, _v.ViTBlock))
    elif pm.DATA.world_size > 1:
        model = DataParallel(model)
    flop_tokens = getattr(model, "flop_tokens_per_sample", tokens_per_sample)   # ViT: tokens per image
    numel, numel_local = calc_model_size(model)
    logger.info(f"model {args.model_name}: {numel / 1e6:.1f} M parameters ({numel_local / 1e6:.1f} M on this rank)")

    from cubework_b200.optim import FusedAdamW, FusedSGD, cosine_warmup_schedule, linear_warmup_schedule
    opt_name = args.optimizer or family.DEFAULT_OPTIMIZER
    if opt_name == "sgd":
        optimizer = FusedSGD(model.parameters(), lr=args.learning_rate, weight_decay=args.weight_decay)
    else:
        optimizer = FusedAdamW(model.parameters(), lr=args.learning_rate, weight_decay=args.weight_decay)
    total_steps = args.steps_per_epoch * args.num_epochs
    sched_fn = cosine_warmup_schedule if family.SCHEDULE == "cosine" else linear_warmup_schedule
    scheduler = sched_fn(optimizer, min(args.warmup_steps, total_steps), total_steps)

    dp = pm.DATA.world_size
    micro = args.micro_batch_size or args.global_batch_size // dp
    accum = max(1, args.global_batch_size // (micro * dp))
    amp_dtype = None
    if args.use_mixed_precision and dev.type == "cuda":
        amp_dtype = torch.bfloat16 if args.amp_dtype == "bf16" else torch.float16
    timer = PhaseTimer(dev.type == "cuda")
    trainer = Trainer(model, criterion, optimizer, scheduler, amp_dtype=amp_dtype,
                      clip=args.gradient_clipping or None, accum_steps=accum, forward_fn=family.forward,
                      scaler_kwargs=dict(init_scale=args.fp16_initial_scale, growth_factor=args.fp16_growth_factor,
                                         backoff_factor=args.fp16_backoff_factor,
                                         growth_interval=args.fp16_growth_interval), timer=timer)
    start_step = 0
    if args.resume_step is not None and args.save_dir:
        start_step, _ = checkpoint.load_checkpoint(args.save_dir, args.resume_step, model, optimizer, scheduler,
                                                   trainer.scaler)
        logger.info(f"resumed from step {start_step}")

    if args.dataset_path:
        from cubework_b200.utils.datasets import Cycle
        train_loader, test_loader = family.build_data(args, micro, model)
        loader = Cycle(train_loader)
        logger.info(f"data: {args.dataset_path} ({len(train_loader)} training / {len(test_loader)} test batches "
                    f"of {micro} per data-parallel rank)")
    else:
        loader = cube.utils.SyntheticLoader(lambda g: make_batch(g, micro), n_distinct=4)
        n_eval = max(1, args.steps_per_epoch // 4)
        test_loader = cube.utils.SyntheticLoader(lambda g: make_batch(g, micro), n_distinct=min(4, n_eval), seed=4321,
                                                 length=n_eval)
    profiler = CommProfiler() if args.use_comm_profiler else None
    use_cuda = dev.type == "cuda"
    try:
        from tqdm import tqdm
    except Exception:  # noqa: BLE001
        tqdm = None

    step = start_step
    for epoch in range(args.num_epochs):
        if use_cuda:
            torch.cuda.reset_peak_memory_stats()
            mem_state = torch.cuda.memory_allocated()
        if profiler:
            profiler.reset()
            profiler.start()
        timer.reset()
        bar = tqdm(range(args.steps_per_epoch), desc=f"[Epoch {epoch}]") if (tqdm and pm.GLOBAL.rank == 0) else \
            range(args.steps_per_epoch)
        losses = []
        t_epoch = time.perf_counter()
        for _ in bar:
            timer.start("load")
            batches = [next(loader) for _ in range(accum)]
            timer.stop("load")
            timer.start("step")
            loss = trainer.step(batches)
            timer.stop("step")
            losses.append(loss)
            step += 1
            if tqdm and pm.GLOBAL.rank == 0 and step % 5 == 0:
                bar.set_postfix(loss=f"{losses[-1].item():.4f}", lr=f"{scheduler.get_last_lr()[0]:.3e}")
        tot = timer.totals()
        wall = time.perf_counter() - t_epoch
        step_time = tot["step"] / args.steps_per_epoch
        samples = args.global_batch_size * args.steps_per_epoch
        mean_loss = _dp_mean(torch.stack([x.float() for x in losses]).mean().item())
        phases = " / ".join(f"{k} {tot.get(k, 0.0) / args.steps_per_epoch * 1e3:.1f}" for k in ("data", "fwd", "bwd", "opt"))
        msg = (f"[Epoch {epoch} / Train]: Loss = {mean_loss:.4f} | Step time = {step_time:.3f} s "
               f"({phases} ms as enqueued) | "
               f"Throughput = {samples / tot['step']:.2f} samples/sec, "
               f"{samples * tokens_per_sample / tot['step']:.1f} {args.token_unit}/sec | TFLOPS = "
               f"{calc_tflops(numel, args.global_batch_size * flop_tokens, step_time, True, args.use_activation_checkpoint):.2f}"
               f" | wall = {wall:.1f} s")
        if use_cuda:
            peak = torch.cuda.max_memory_allocated()
            msg += (f" | Peak memory = {peak / 2**30:.2f} GB, state = {mem_state / 2**30:.2f} GB, activation = "
                    f"{(peak - mem_state) / 2**30:.2f} GB")
        if profiler:
            ops_, vol, secs = profiler.stop()
            msg += (f" | Comm: {ops_} ops, {secs:.3f} s ({100 * secs / max(tot['step'], 1e-9):.1f} % of the epoch), "
                    f"{vol / max(secs, 1e-9) / 1e9:.1f} GB/s algorithm bandwidth")
        logger.info(msg)
        if args.do_validation and (epoch + 1) % args.validation_interval == 0 and metric is not None:
            _test(epoch, trainer, test_loader, metric, args, tokens_per_sample, use_cuda, logger)
        if args.save_dir:
            d = checkpoint.save_checkpoint(args.save_dir, step, model, optimizer, scheduler, trainer.scaler)
            logger.info(f"checkpoint written to {d}")
    return trainer
