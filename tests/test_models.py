"""End-to-end parity of the model families with a single-process unsharded model.

The headline check is the tiny GPT-2 configuration: 2 layers, hidden 128, 4 heads, MLP 512, vocab 1024,
sequence 64, batch 4, fp32, weights N(0, 0.02), biases 0 — one forward + backward + AdamW step under 1D
tensor parallelism on 2 CPU/gloo ranks must match the unsharded model to 1e-5.  The same check runs for
2D (4 ranks) and 3D (8 ranks), and for tiny OPT and ViT models.
"""
import copy

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_dist


def _init_002(model):
    g = torch.Generator().manual_seed(1234)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
            if p.dim() >= 2 and "norm" not in name:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
            elif "norm" in name and name.endswith("weight"):
                p.fill_(1.0)
            else:
                p.zero_()


def _build(family):
    from cubework_b200.models import gpt2, opt, vit
    if family == "gpt2_sp":
        return (gpt2.build_model("gpt2_tiny", 64, dropout=0.0, embedding_dropout=0.0, sequence_parallel=True),
                gpt2.GPT2LMLoss())
    if family == "gpt2":
        return gpt2.build_model("gpt2_tiny", 64, dropout=0.0, embedding_dropout=0.0), gpt2.GPT2LMLoss()
    if family == "opt":
        return opt.build_model("opt_tiny", 64, dropout=0.0, vocab_size=512), opt.OPTLMLoss()
    if family == "vit":
        import cubework_b200.module as nn_
        return vit.build_model("vit_tiny", dropout=0.0), nn_.CrossEntropyLoss()
    raise ValueError(family)


def _batch(family):
    g = torch.Generator().manual_seed(7)
    if family in ("gpt2", "gpt2_sp"):
        ids = torch.randint(0, 1024, (4, 64), generator=g)
        return dict(input_ids=ids, attention_mask=torch.ones(4, 64), labels=ids)
    if family == "opt":
        ids = torch.randint(0, 512, (8, 64), generator=g)
        mask = torch.ones(8, 64)
        mask[1, 50:] = 0   # right padding on one sample exercises the key mask and the position ids
        return dict(input_ids=ids, attention_mask=mask, labels=ids)
    return dict(pixel_values=torch.randn(8, 3, 32, 32, generator=g), labels=torch.randint(0, 16, (8, ), generator=g))


def _one_step(model, crit, batch):
    """forward + backward + clip + AdamW; returns (loss, logical gradients before clipping)."""
    from cubework_b200.optim import FusedAdamW
    from cubework_b200.parallel.common import get_shard_spec
    from cubework_b200.utils import clip_grad_norm
    from cubework_b200.utils.checkpoint import gather_tensor
    opt_ = FusedAdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    model.train()
    labels = batch["labels"]
    out = model(**{k: v for k, v in batch.items() if k != "labels"})
    out = out[0] if isinstance(out, tuple) else out
    loss = crit(out, labels)
    loss.backward()
    from cubework_b200.parallel.ops_1d import reduce_partial_grads
    reduce_partial_grads(list(model.parameters()))
    grads = {}
    for name, p in model.named_parameters():
        g = gather_tensor(p.grad.detach().clone(), get_shard_spec(p))
        grads[name] = g.t().contiguous() if getattr(p, "STORED_IN_OUT", False) else g
    norm = clip_grad_norm(model.parameters(), 1.0)
    opt_.step()
    return loss.detach(), grads, float(norm)


def _check_family(family, tol):
    from cubework_b200.global_vars import env
    from cubework_b200.utils import checkpoint as ck
    saved = env.save()
    # --- oracle: the same model code with tensor parallelism switched off, on this rank alone ---
    env.load(mode=None)
    torch.manual_seed(0)
    master, mcrit = _build(family)
    _init_002(master)
    init_sd = {k: v.detach().clone() for k, v in master.state_dict().items()}
    mloss, mgrads, mnorm = _one_step(master, mcrit, _batch(family))
    master_sd = master.state_dict()
    env.load(**saved)
    # --- sharded model, loaded from the same initial values ---
    model, crit = _build(family)
    ck.load_full_state_dict(model, init_sd)
    loss, grads, norm = _one_step(model, crit, _batch(family))
    assert abs(loss.item() - mloss.item()) <= tol, f"{family}: loss {loss.item()} vs {mloss.item()}"
    for k in mgrads:
        scale = max(mgrads[k].abs().max().item(), 1e-6)
        err = (grads[k] - mgrads[k]).abs().max().item()
        assert err <= 2e-5 * scale + 1e-7, f"{family}: grad of {k} differs by {err:.3e} (scale {scale:.3e})"
    assert abs(norm - mnorm) <= 1e-4 * max(1.0, mnorm), f"{family}: grad norm {norm} vs {mnorm}"
    full = ck.full_state_dict(model)
    assert set(full) == set(master_sd), sorted(set(full) ^ set(master_sd))
    worst = max((full[k] - master_sd[k]).abs().max().item() for k in full)
    assert worst <= tol, f"{family}: parameters after one step differ by {worst:.3e}"
    # the gathered value must also be identical on every rank
    for k in sorted(full)[:4]:
        t = full[k].clone()
        dist.broadcast(t, src=0)
        assert torch.equal(t, full[k])


@pytest.mark.parametrize("tp,world", [("1d", 2), ("2d", 4), ("3d", 8)])
def test_gpt2_tiny_one_step_matches_unsharded(tp, world):
    run_dist(_check_family, world, tp=tp, tp_size=world, args=("gpt2", 1e-5))


@pytest.mark.parametrize("tp,world", [("1d", 2), ("2d", 4)])
def test_opt_tiny_one_step_matches_unsharded(tp, world):
    run_dist(_check_family, world, tp=tp, tp_size=world, args=("opt", 1e-5))


@pytest.mark.parametrize("tp,world", [("1d", 2), ("2d", 4), ("3d", 8)])
def test_vit_tiny_one_step_matches_unsharded(tp, world):
    run_dist(_check_family, world, tp=tp, tp_size=world, args=("vit", 1e-5))


@pytest.mark.parametrize("world", [2, 4])
def test_gpt2_tiny_sequence_parallel_matches_unsharded(world):
    """1D with row-sharded activations between the linear pairs (all-gather -> GEMM, GEMM -> reduce-scatter,
    layer norm / residual on batch/tp sequences) gives the unsharded model's step."""
    run_dist(_check_family, world, tp="1d", tp_size=world, args=("gpt2_sp", 1e-5))


def test_gpt2_tiny_tp_times_dp():
    """tp=2 x dp=2: replicas see the same batch here, so the result still equals the unsharded model."""
    run_dist(_check_family, 4, tp="1d", tp_size=2, args=("gpt2", 1e-5))


def _check_checkpointed(family, sp):
    """Activation checkpointing (with dropout, i.e. with random streams to rewind, and with the skipped last
    product of every re-run block) gives the gradients of the plain model."""
    import cubework_b200 as cube  # noqa: F401
    from cubework_b200.models import gpt2
    from cubework_b200.parallel.ops_1d import reduce_partial_grads
    from cubework_b200.utils import checkpoint as ck

    def build(ckpt):
        torch.manual_seed(11)
        return gpt2.build_model("gpt2_tiny", 64, dropout=0.1, embedding_dropout=0.1, checkpoint=ckpt, sequence_parallel=sp)

    ref, model = build(False), build(True)
    model.load_state_dict(ref.state_dict())
    crit = gpt2.GPT2LMLoss()
    batch = _batch("gpt2")
    grads = []
    for m in (ref, model):
        m.train()
        saved = ck._rng_states()
        torch.manual_seed(77)
        loss = crit(m(batch["input_ids"], batch["attention_mask"]), batch["labels"])
        loss.backward()
        reduce_partial_grads(list(m.parameters()))
        ck._set_rng_states(saved)            # both runs start from the same random streams
        grads.append((loss.item(), {k: p.grad.clone() for k, p in m.named_parameters()}))
    assert abs(grads[0][0] - grads[1][0]) < 1e-6
    for k in grads[0][1]:
        assert torch.allclose(grads[0][1][k], grads[1][1][k], rtol=1e-4, atol=1e-6), k


@pytest.mark.parametrize("sp", [False, True])
def test_gpt2_activation_checkpointing_matches_plain(sp):
    run_dist(_check_checkpointed, 2, tp="1d", tp_size=2, args=("gpt2", sp))
