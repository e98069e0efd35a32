"""Sharded checkpoints on CPU / gloo: save under one layout, consolidate offline, load under another; resume of
model + optimizer + RNG streams reproduces the uninterrupted run bit for bit; fully sharded data parallelism
writes and restores every DATA rank's own slice."""
import os
import tempfile

import torch

from dist_utils import run_dist


def _tiny(dropout=0.0):
    from cubework_b200.models import gpt2
    return gpt2.build_model("gpt2_tiny", 64, dropout=dropout, embedding_dropout=dropout), gpt2.GPT2LMLoss()


def _batch(seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1024, (4, 64), generator=g)
    return dict(input_ids=ids, attention_mask=torch.ones(4, 64), labels=ids)


def _trainer(model, crit):
    from cubework_b200.engine import Trainer
    from cubework_b200.optim import FusedAdamW, linear_warmup_schedule
    opt = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.01)
    sched = linear_warmup_schedule(opt, 2, 10)
    return Trainer(model, crit, opt, sched, amp_dtype=None, clip=1.0, device=torch.device("cpu"))


def _save_1d(root):
    from cubework_b200.utils import checkpoint as ck
    model, crit = _tiny()
    tr = _trainer(model, crit)
    tr.step(_batch(1))
    ck.save_checkpoint(root, 1, model, tr.optimizer, tr.lr_scheduler)
    full = ck.full_state_dict(model)
    import torch.distributed as dist
    if dist.get_rank() == 0:
        torch.save(full, os.path.join(root, "expected_full.pt"))


def _load_2d(root):
    from cubework_b200.utils import checkpoint as ck
    full, meta = ck.consolidate(root, 1)          # offline reconstruction from the 1D shard files
    expected = torch.load(os.path.join(root, "expected_full.pt"), weights_only=False)
    assert meta["mode"] == "1d" and meta["tp_size"] == 2 and not meta["fsdp"]
    assert set(full) == set(expected)
    for k in full:
        assert torch.equal(full[k], expected[k]), k
    model, _ = _tiny()                            # a 2D (2 x 2) model takes the same logical tensors
    ck.load_full_state_dict(model, full)
    again = ck.full_state_dict(model)
    for k in full:
        assert torch.equal(again[k], full[k]), k


def test_save_1d_consolidate_load_2d():
    with tempfile.TemporaryDirectory() as root:
        run_dist(_save_1d, 2, tp="1d", tp_size=2, args=(root, ))
        run_dist(_load_2d, 4, tp="2d", tp_size=4, args=(root, ))


def _resume(root):
    """Two steps, checkpoint, two more steps; then a fresh model resumes from the checkpoint and repeats the last
    two steps: losses and parameters must be identical (dropout is on, so the RNG streams matter too)."""
    from cubework_b200.utils import checkpoint as ck
    torch.manual_seed(5)
    model, crit = _tiny(dropout=0.1)
    tr = _trainer(model, crit)
    for s in range(2):
        tr.step(_batch(10 + s))
    ck.save_checkpoint(root, 2, model, tr.optimizer, tr.lr_scheduler, extra={"note": "two steps"})
    ref_losses = [tr.step(_batch(20 + s)).item() for s in range(2)]
    ref_params = {k: v.detach().clone() for k, v in model.named_parameters()}

    torch.manual_seed(999)                        # a different stream, to be overwritten by the restore
    model2, crit2 = _tiny(dropout=0.1)
    tr2 = _trainer(model2, crit2)
    step, extra = ck.load_checkpoint(root, 2, model2, tr2.optimizer, tr2.lr_scheduler)
    assert step == 2 and extra == {"note": "two steps"}
    assert tr2.lr_scheduler.last_epoch == 2
    losses = [tr2.step(_batch(20 + s)).item() for s in range(2)]
    assert losses == ref_losses, (losses, ref_losses)
    for k, v in model2.named_parameters():
        assert torch.equal(v.detach(), ref_params[k]), k


def test_resume_is_bit_identical_1d():
    with tempfile.TemporaryDirectory() as root:
        run_dist(_resume, 2, tp="1d", tp_size=2, args=(root, ))


def _resume_fsdp(root):
    import torch.distributed as dist

    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.models import gpt2
    from cubework_b200.parallel.fsdp import FullyShardedDataParallel
    from cubework_b200.utils import checkpoint as ck
    import pytest
    assert pm.DATA.world_size == 2
    rank = dist.get_rank()

    def build():
        torch.manual_seed(3)
        model, crit = _tiny()
        wrapped = FullyShardedDataParallel(model, unit_classes=(gpt2.GPT2Block, ))
        return wrapped, _trainer(wrapped, crit)

    fsdp, tr = build()
    for s in range(2):
        tr.step(_batch(30 + 2 * s + rank))        # each data-parallel rank has its own micro-batch
    ck.save_checkpoint(root, 2, fsdp, tr.optimizer, tr.lr_scheduler)
    assert os.path.exists(os.path.join(root, "step_2", f"tp0_dp{pm.DATA.local_rank}.pt"))
    ref_loss = tr.step(_batch(40 + rank)).item()
    ref_full = fsdp.full_state_dict()

    fsdp2, tr2 = build()
    ck.load_checkpoint(root, 2, fsdp2, tr2.optimizer, tr2.lr_scheduler)
    loss = tr2.step(_batch(40 + rank)).item()
    assert loss == ref_loss, (loss, ref_loss)
    full = fsdp2.full_state_dict()
    for k in ref_full:
        assert torch.equal(full[k], ref_full[k]), k
    # logical tensors through the generic entry point, too
    logical = ck.full_state_dict(fsdp2)
    assert set(logical) >= set(ref_full) and all(torch.equal(logical[k], ref_full[k]) for k in ref_full)   # + tied names
    # a plain (replicated) model must refuse the fully sharded checkpoint, and the offline path as well
    plain, _ = _tiny()
    with pytest.raises(ValueError):
        ck.load_checkpoint(root, 2, plain)
    with pytest.raises(ValueError):
        ck.consolidate(root, 2)


def test_fsdp_checkpoint_saves_every_data_rank_and_resumes():
    with tempfile.TemporaryDirectory() as root:
        run_dist(_resume_fsdp, 2, tp="1d", tp_size=1, args=(root, ))
