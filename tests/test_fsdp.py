"""Fully sharded data parallelism against plain data parallelism on CPU / gloo: same losses, same parameters."""
import torch

from dist_utils import run_dist


def _check_fsdp(family):
    import torch.distributed as dist

    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.engine import Trainer
    from cubework_b200.models import gpt2, opt
    from cubework_b200.optim import FusedAdamW
    from cubework_b200.parallel.ddp import DataParallel
    from cubework_b200.parallel.fsdp import FullyShardedDataParallel
    import test_models as tm
    assert pm.DATA.world_size == 2
    rank = dist.get_rank()
    ref_model, crit = tm._build(family)
    tm._init_002(ref_model)
    init = {k: v.detach().clone() for k, v in ref_model.state_dict().items()}
    model, _ = tm._build(family)
    model.load_state_dict(init)
    ddp = DataParallel(ref_model)
    fsdp = FullyShardedDataParallel(model, unit_classes=(gpt2.GPT2Block, opt.OPTDecoderLayer))
    # every original parameter is empty between steps; the shards hold 1/2 of the elements (plus padding)
    assert all(p.numel() == 0 for p in model.parameters())
    n_full = sum(v.numel() for k, v in init.items())
    n_shard = sum(p.numel() for p in fsdp.parameters())
    assert n_shard * 2 >= len(set(id(p) for p in ref_model.parameters())) and n_shard <= n_full // 2 + 64
    tr_ref = Trainer(ddp, crit, FusedAdamW(ddp.parameters(), lr=1e-3), clip=1.0, amp_dtype=None, device=torch.device("cpu"))
    tr = Trainer(fsdp, crit, FusedAdamW(fsdp.parameters(), lr=1e-3), clip=1.0, amp_dtype=None, device=torch.device("cpu"))
    for step in range(3):
        torch.manual_seed(100 + step * 2 + rank)          # each data-parallel rank has its own micro-batch
        batch = tm._batch(family)
        for k in batch:
            if batch[k].dtype == torch.long and k != "attention_mask":
                batch[k] = torch.randint(0, 1000, batch[k].shape)
        a = tr_ref.step(batch).item()
        b = tr.step(batch).item()
        assert abs(a - b) < 1e-5, (step, a, b)
    full = fsdp.full_state_dict()
    ref = dict(ref_model.named_parameters())
    for n, v in full.items():
        assert torch.allclose(v, ref[n].detach(), rtol=1e-4, atol=1e-5), n
    assert all(p.numel() == 0 for p in model.parameters())


def test_fsdp_matches_ddp_gpt2():
    run_dist(_check_fsdp, 2, tp="1d", tp_size=1, args=("gpt2", ))


def test_fsdp_matches_ddp_opt():
    run_dist(_check_fsdp, 2, tp="1d", tp_size=1, args=("opt", ))


def test_fsdp_with_1d_tensor_parallel():
    run_dist(_check_fsdp, 4, tp="1d", tp_size=2, args=("opt", ))
