"""Single-GPU end-to-end checks of the training engine on the kernel path: fp16 with a configured GradScaler,
activation checkpointing against the plain model, attention-probability dropout, and the smoke entry point."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny(**kw):
    from cubework_b200.global_vars import env
    from cubework_b200.models import gpt2
    env.load(mode=None)
    torch.manual_seed(0)
    return gpt2.GPT2(vocab_size=1024, max_position_embeddings=128, hidden_size=256, num_heads=4, intermediate_size=1024,
                     depth=2, init_std=0.02, **kw).cuda()


def _batch():
    ids = torch.randint(0, 1024, (4, 128), generator=torch.Generator().manual_seed(3))
    return dict(input_ids=ids, attention_mask=torch.ones(4, 128), labels=ids)


def test_fp16_with_grad_scaler_knobs():
    from cubework_b200.engine import Trainer
    from cubework_b200.models import gpt2
    from cubework_b200.ops import ext
    from cubework_b200.optim import FusedAdamW
    model = _tiny(dropout=0.0, embedding_dropout=0.0)
    tr = Trainer(model, gpt2.GPT2LMLoss(), FusedAdamW(model.parameters(), lr=1e-3), amp_dtype=torch.float16, clip=1.0,
                 scaler_kwargs=dict(init_scale=2.0**10, growth_factor=4.0, backoff_factor=0.25, growth_interval=2))
    assert tr.scaler is not None and tr.scaler.get_scale() == 2.0**10
    losses = [tr.step(_batch()).item() for _ in range(4)]
    torch.cuda.synchronize()
    ext.check_status()
    assert losses[-1] < losses[0] and all(l == l for l in losses)
    assert tr.scaler.get_scale() in (2.0**10 * 4, 2.0**10 * 16, 2.0**10, 2.0**8)    # grew (or backed off) by the given factors


def test_checkpointed_blocks_match_plain_on_the_kernel_path():
    """Same weights, same batch: losses and gradients with per-block recomputation (which skips each block's last
    product when it re-runs the forward) equal those of the plain model."""
    from cubework_b200.models import gpt2
    ref = _tiny(dropout=0.0, embedding_dropout=0.0, checkpoint=False)
    model = _tiny(dropout=0.0, embedding_dropout=0.0, checkpoint=True)
    model.load_state_dict(ref.state_dict())
    crit = gpt2.GPT2LMLoss()
    b = {k: v.cuda() for k, v in _batch().items()}
    out = []
    for m in (ref, model):
        m.train()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = crit(m(b["input_ids"], b["attention_mask"]), b["labels"])
        loss.backward()
        out.append((loss.item(), {k: p.grad.clone() for k, p in m.named_parameters()}))
    assert abs(out[0][0] - out[1][0]) < 1e-5
    for k in out[0][1]:
        assert torch.allclose(out[0][1][k], out[1][1][k], rtol=1e-3, atol=1e-6), k


def test_attention_dropout_trains_on_gpu():
    from cubework_b200.engine import Trainer
    from cubework_b200.models import gpt2
    from cubework_b200.optim import FusedAdamW
    model = _tiny(dropout=0.1, embedding_dropout=0.1, attention_dropout=0.1)
    tr = Trainer(model, gpt2.GPT2LMLoss(), FusedAdamW(model.parameters(), lr=1e-3), amp_dtype=torch.bfloat16, clip=1.0)
    losses = [tr.step(_batch()).item() for _ in range(4)]
    assert losses[-1] < losses[0]
    out, targets, loss = tr.evaluate(_batch())            # evaluation: fused kernel, no dropout
    assert torch.isfinite(loss).item()


def test_smoke_entry_point():
    import __graft_entry__ as g
    g.smoke()
