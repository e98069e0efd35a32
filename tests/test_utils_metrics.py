"""Communication profiler counts against hand-computed values, metrics over the DATA group, DropPath statistics,
the memory tracker thread and OPT's incremental decoding with a key/value cache (all on CPU / gloo)."""
import math

import torch

from dist_utils import run_dist


def _check_comm_profiler():
    import torch.distributed as dist

    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.parallel.collective import all_gather, all_reduce, broadcast, reduce, reduce_scatter
    from cubework_b200.utils import CommProfiler
    mode = pm.PARALLEL_1D
    n = mode.world_size
    assert n == 4
    prof = CommProfiler()
    prof.start()
    x = torch.ones(8, 16)                         # 512 bytes of fp32
    all_reduce(x.clone(), mode)                   # 2 (n-1)/n S          = 768
    g = all_gather(x, 0, mode)                    # (n-1)/n of the 2048-byte result = 1536
    reduce_scatter(g, 0, mode)                    # (n-1)/n of the 2048-byte input  = 1536
    broadcast(x.clone(), mode.rank_by_idx(0), mode)   # S = 512
    reduce(x.clone(), mode.rank_by_idx(1), mode)      # S = 512
    y, work = all_reduce(x.clone(), mode, async_op=True)
    work.wait()                                   # 768
    ops, volume, seconds = prof.stop()
    assert ops == 6, ops
    assert volume == 768 + 1536 + 1536 + 512 + 512 + 768, volume
    assert seconds > 0
    s = prof.summary()
    assert s["by_kind"]["all_reduce"] == (2, 1536) and s["by_kind"]["all_gather"] == (1, 1536)
    assert s["by_kind"]["reduce_scatter"] == (1, 1536) and s["by_kind"]["broadcast"] == (1, 512)
    assert torch.equal(y, torch.full((8, 16), float(n)))
    # fused launches report their link bytes (and, on a GPU, their kernel time) through account()
    prof.reset()
    prof.account("fused_gather_gemm_scatter", 4096)
    assert prof.ops == 1 and prof.fused_bytes == 4096 and prof.summary()["fused_seconds"] == 0.0
    # a stopped profiler sees nothing
    all_reduce(x.clone(), mode)
    assert prof.ops == 1
    dist.barrier()


def test_comm_profiler_counts():
    run_dist(_check_comm_profiler, 4, tp="1d", tp_size=4)


def _check_metrics():
    import torch.distributed as dist

    import cubework_b200.module as nn_
    from cubework_b200.distributed import ParallelManager as pm
    assert pm.DATA.world_size == 2 and pm.TENSOR.world_size == 1
    d = pm.DATA.local_rank
    acc = nn_.Accuracy()
    logits = torch.eye(4)                         # argmax of row i is i
    targets = torch.tensor([0, 1, 2, 3]) if d == 0 else torch.tensor([0, 0, 0, 0])
    frac = acc(logits, targets)
    assert abs(frac.item() - (1.0 if d == 0 else 0.25)) < 1e-6
    assert abs(acc.value().item() - 5.0 / 8.0) < 1e-6          # 4 + 1 correct out of 8 over both replicas
    assert acc.to_str() == "62.50 %"
    acc.reset()
    assert acc.total_samples.item() == 0
    ppl = nn_.Perplexity()
    ppl(None, None, torch.tensor(1.0 + d))        # losses 1 and 2 on the two replicas
    ppl(None, None, torch.tensor(3.0 + d))        # then 3 and 4
    assert abs(ppl.value().item() - math.exp(10.0 / 4.0)) < 1e-4
    dist.barrier()


def test_accuracy_and_perplexity_over_data_group():
    run_dist(_check_metrics, 2, tp="1d", tp_size=1)


def test_drop_path_statistics():
    import cubework_b200.module as nn_
    torch.manual_seed(0)
    dp = nn_.DropPath(0.25)
    x = torch.ones(4000, 3, 5)
    dp.train()
    y = dp(x)
    kept = (y[:, 0, 0] != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.03
    assert torch.all((y == 0) | (torch.abs(y - 1 / 0.75) < 1e-6))     # whole samples dropped, the rest rescaled
    assert torch.equal(y[:, 0, 0:1].expand(-1, 5), y[:, 2, :])
    dp.eval()
    assert torch.equal(dp(x), x)


def test_memory_tracker_thread(tmp_path):
    from cubework_b200.utils import MemoryTracker
    log = tmp_path / "mem.log"
    mt = MemoryTracker(log_file=str(log), interval=1e-3)
    mt.start()
    import time
    time.sleep(0.05)
    peak = mt.stop()
    assert peak >= 0 and len(mt.samples) >= 5
    assert len(log.read_text().strip().splitlines()) == len(mt.samples)


def test_opt_incremental_decoding_matches_full_forward():
    """Logits of position t computed from the key/value cache equal the logits of a full forward pass."""
    from cubework_b200.global_vars import env
    from cubework_b200.models import opt
    env.load(mode=None)
    torch.manual_seed(0)
    model = opt.build_model("opt_tiny", 64, dropout=0.0, vocab_size=512).eval()
    ids = torch.randint(0, 512, (2, 12))
    mask = torch.ones(2, 12)
    with torch.no_grad():
        full = model(ids, mask)[0]
        logits, cache = model(ids[:, :8], mask[:, :8], use_cache=True)
        assert torch.allclose(logits, full[:, :8], atol=1e-5)
        for t in range(8, 12):
            step_logits, cache = model(ids[:, t:t + 1], mask[:, :t + 1], past_key_values=cache, use_cache=True)
            assert torch.allclose(step_logits[:, 0], full[:, t], atol=1e-5), t
        assert cache[0][0].shape[2] == 12


def test_attention_probability_dropout():
    """``attention_dropout`` drops probabilities in training mode only; the expectation of the output is kept."""
    from cubework_b200 import ops
    from cubework_b200.global_vars import env
    from cubework_b200.models.common import SelfAttention
    env.load(mode=None)
    torch.manual_seed(0)
    attn = SelfAttention(64, 4, attention_dropout=0.5, dropout=0.0, causal=True)
    x = torch.randn(2, 16, 64)
    attn.eval()
    y_eval = attn(x)
    qkv = attn.query_key_value(x).view(2, 16, 4, 48)
    ref = attn.dense(ops.attention_packed(qkv, True, None))
    assert torch.allclose(y_eval, ref, atol=1e-6)             # evaluation: the plain (fused) attention
    attn.train()
    ys = torch.stack([attn(x) for _ in range(400)])
    assert not torch.allclose(ys[0], y_eval, atol=1e-3)       # training: masks differ from call to call
    assert not torch.allclose(ys[0], ys[1], atol=1e-3)
    # E[dropout(P)] = P, and everything after the dropout is linear
    assert (ys.mean(0) - y_eval).abs().max().item() < 0.15 * y_eval.abs().max().item()
    xg = x.clone().requires_grad_(True)
    attn(xg).sum().backward()
    assert xg.grad is not None and torch.isfinite(xg.grad).all()
    # with no dropped entry (p = 0) the materialised formulation equals the fused one
    y0 = ops.attention_with_prob_dropout(qkv, True, None, torch.nn.Identity())
    assert torch.allclose(y0, ops.attention_packed(qkv, True, None), atol=1e-5)
