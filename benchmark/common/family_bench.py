"""ViT (2D SUMMA) and OPT (3D cube) training throughput, this framework against the unmodified reference.

    torchrun --nproc_per_node 4 benchmark/common/family_bench.py --family vit --model vit_base --tp 2d --tp_size 4 --bs 256
    torchrun --nproc_per_node 8 benchmark/common/family_bench.py --family opt --model opt_13b --tp 3d --tp_size 8 \\
        --bs 16 --seq 2048 --ckpt
    ... --impl reference          # the reference's own model class, layers, loss and fp16 AMP loop (baseline/_ref)

World size = tp_size x dp; the global batch is split over the data-parallel replicas.  Synthetic inputs of the named
shape (images ~ N(0,1), labels uniform; token ids uniform), random-init weights, AdamW (ViT) / SGD (OPT, the
reference's choice, benchmark/opt/opt.py:623).  One step = forward + backward + optimizer step + zero_grad; timed with
CUDA events around ``--steps`` steps after ``--warmup`` steps, maximum over ranks; every step works on tens of GB of
activations and weights, far more than L2.  Prints one JSON line per run.
"""
import argparse
import json
import math
import os
import sys
import types

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..")
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def timed_steps(step, steps, warmup):
    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def make_batch(args, micro, dev, vocab, classes, img):
    g = torch.Generator().manual_seed(1234)
    if args.family == "vit":
        return dict(pixel_values=torch.randn(micro, 3, img, img, generator=g).to(dev),
                    labels=torch.randint(0, classes, (micro, ), generator=g).to(dev))
    ids = torch.randint(2, vocab, (micro, args.seq), generator=g).to(dev)
    return dict(input_ids=ids, attention_mask=torch.ones(micro, args.seq, device=dev), labels=ids.clone())


def run_ours(args):
    import cubework_b200 as cube
    import cubework_b200.module as cube_nn
    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.engine import Trainer
    from cubework_b200.models import opt, vit
    from cubework_b200.ops import ext
    from cubework_b200.optim import FusedAdamW, FusedSGD
    from cubework_b200.parallel.ddp import DataParallel
    argv = ["--tp", args.tp, "--tp_size", str(args.tp_size)] if args.tp != "none" else []
    cube.initialize_distributed(argv=argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    if args.family == "vit":
        model = vit.build_model(args.model, checkpoint=args.ckpt, dropout=0.0).to(dev)
        crit, fwd = cube_nn.CrossEntropyLoss(), lambda m, b: (m(b["pixel_values"]), b["labels"])
        opt_ = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        vocab, classes, img = 0, 1000, model.img_size
    else:
        model = opt.build_model(args.model, max_position_embeddings=args.seq, checkpoint=args.ckpt, dropout=0.0,
                                init_std=0.02).to(dev)
        crit, fwd = opt.OPTLMLoss(), lambda m, b: (m(b["input_ids"], b["attention_mask"])[0], b["labels"])
        opt_ = FusedSGD(model.parameters(), lr=1e-4)
        vocab, classes, img = model.vocab_size, 0, 0
    if pm.DATA.world_size > 1:
        model = DataParallel(model)
    micro = args.bs // pm.DATA.world_size
    batch = make_batch(args, micro, dev, vocab, classes, img)
    trainer = Trainer(model, crit, opt_, amp_dtype=torch.bfloat16, forward_fn=fwd)
    losses = []
    ms = timed_steps(lambda: losses.append(trainer.step(batch)), args.steps, args.warmup)
    ext.check_status()
    report(args, ms, "ours", "bf16", losses[-1].item())
    cube.destroy_distributed()


def run_reference(args):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    six = types.ModuleType("torch._six")       # removed in torch 2.x; cubework/utils/clip_grad.py imports `inf` from it
    six.inf = math.inf
    sys.modules["torch._six"] = six
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "benchmark", args.family))
    import cubework
    import cubework.module as cube_nn
    from cubework.distributed import ParallelManager as pm
    sys.argv = [sys.argv[0]] + (["--tp", args.tp, "--tp_size", str(args.tp_size)] if args.tp != "none" else [])
    cubework.initialize_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    if args.family == "vit":
        import vit as ref_vit
        model = getattr(ref_vit, args.model)(checkpoint=args.ckpt).to(dev)
        crit = cube_nn.CrossEntropyLoss()
        opt_ = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        vocab, classes, img = 0, 1000, 224

        def loss_of(b):     # every rank feeds the full batch; the parallel patch embedding takes its slice itself
            return crit(model(b["pixel_values"]), b["labels"])
    else:
        import opt as ref_opt
        model = getattr(ref_opt, args.model)(max_position_embeddings=args.seq, checkpoint=args.ckpt).to(dev)
        crit = ref_opt.OPTLMLoss()
        opt_ = torch.optim.SGD(model.parameters(), lr=1e-4)
        vocab, classes, img = 50272, 0, 0

        def loss_of(b):
            out = model(input_ids=b["input_ids"], attention_mask=b["attention_mask"])
            return crit(out[0] if isinstance(out, (tuple, list)) else out, b["labels"])
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    if pm.DATA.world_size > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        model = DDP(model, process_group=pm.DATA.group)
    micro = args.bs // pm.DATA.world_size
    batch = make_batch(args, micro, dev, vocab, classes, img)
    scaler = torch.cuda.amp.GradScaler()
    losses = []
    model.train()

    def step():
        with torch.cuda.amp.autocast(enabled=True):
            loss = loss_of(batch)
        scaler.scale(loss).backward()
        scaler.step(opt_)
        scaler.update()
        opt_.zero_grad()
        losses.append(loss.detach())

    ms = timed_steps(step, args.steps, args.warmup)
    report(args, ms, "reference", "fp16 autocast + GradScaler", losses[-1].item())
    cubework.destroy_distributed()


def report(args, ms, impl, dtype, loss):
    if dist.get_rank() != 0:
        return
    per_sample = 1 if args.family == "vit" else args.seq
    unit = "images/s" if args.family == "vit" else "tokens/s"
    print(json.dumps({"impl": impl, "family": args.family, "model": args.model, "tp": args.tp, "tp_size": args.tp_size,
                      "world": dist.get_world_size(), "global_batch": args.bs, "seq": args.seq if args.family != "vit" else None,
                      "activation_checkpointing": args.ckpt, "dtype": dtype, "ms_per_step": round(ms, 3),
                      "value": round(args.bs * per_sample / (ms / 1e3), 1), "unit": unit, "steps": args.steps,
                      "warmup": args.warmup, "last_loss": round(loss, 4)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", choices=["vit", "opt"], required=True)
    ap.add_argument("--model", required=True)
    ap.add_argument("--tp", choices=["none", "1d", "2d", "3d"], default="none")
    ap.add_argument("--tp_size", type=int, default=1)
    ap.add_argument("--bs", type=int, default=256)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--ckpt", action="store_true")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    args = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_PORT="29577")
    (run_reference if args.impl == "reference" else run_ours)(args)


if __name__ == "__main__":
    main()
