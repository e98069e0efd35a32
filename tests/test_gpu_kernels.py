"""Numerics of every sm_100a kernel against a plain PyTorch fp32 formulation of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from cubework_b200 import ops
    from cubework_b200.ops import ext
    ext.require()
    return ops, ext


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 512, 320), (1000, 328, 200), (128, 1608, 64),
                                   (4096, 1600, 1600)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_layouts(trans_a, trans_b, M, N, K, dtype):
    ops, ext = _ops()
    torch.manual_seed(0)
    a = torch.randn((K, M) if trans_a else (M, K), device=DEV, dtype=dtype)
    b = torch.randn((N, K) if trans_b else (K, N), device=DEV, dtype=dtype)
    ref = (a.float().t() if trans_a else a.float()) @ (b.float().t() if trans_b else b.float())
    out = ops.gemm(a, b, trans_a, trans_b)
    ext.check_status()
    assert out.dtype == dtype and out.shape == (M, N)
    assert _rel_err(out, ref) < 6e-3
    out32 = ops.gemm(a, b, trans_a, trans_b, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    assert _rel_err(out32, ref) < 1e-4 if dtype == torch.float16 else _rel_err(out32, ref) < 1e-4


@pytest.mark.parametrize("act", [None, "gelu", "relu"])
@pytest.mark.parametrize("N", [776, 1000, 60])
def test_gemm_epilogues(act, N):
    """Bias, activation and the pre-activation copy through both tile widths (N = 776 takes 128-wide tiles, N = 1000
    takes 256-wide ones) and through the direct-store path (N = 60: a row pitch that TMA cannot store)."""
    ops, ext = _ops()
    torch.manual_seed(1)
    M, K = 520, 264
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    z_ref = a.float() @ b.float().t() + bias
    y_ref = torch.nn.functional.gelu(z_ref) if act == "gelu" else torch.relu(z_ref) if act == "relu" else z_ref
    y, z = ext.gemm(a, b, False, True, bias, act, torch.bfloat16, True)
    ext.check_status()
    assert _rel_err(z, z_ref) < 6e-3 and _rel_err(y, y_ref) < 6e-3
    y32 = ext.gemm(a, b, False, True, bias, act, torch.float32, False)
    assert _rel_err(y32, y_ref) < 1e-4


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
def test_gemm_unaligned_extents_are_padded(trans_a, trans_b):
    """Extents that are not multiples of eight elements (TMA needs 16-byte row pitches) run on the same kernel
    after zero padding; no library GEMM is involved."""
    ops, ext = _ops()
    torch.manual_seed(5)
    M, N, K = 203, 61, 100
    a = torch.randn((K, M) if trans_a else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((N, K) if trans_b else (K, N), device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    ref = (a.float().t() if trans_a else a.float()) @ (b.float().t() if trans_b else b.float()) + bias
    before = ext.launch_count()
    y, z = ext.gemm(a, b, trans_a, trans_b, bias, "relu", torch.bfloat16, True)
    assert ext.launch_count() == before + 1
    ext.check_status()
    assert y.shape == (M, N) and z.shape == (M, N) and y.is_contiguous()
    assert _rel_err(z, ref) < 6e-3 and _rel_err(y, torch.relu(ref)) < 6e-3
    dz, db = ext.act_backward(y, z, "relu", True)
    assert dz.shape == (M, N) and _rel_err(db, (y.float() * (z.float() > 0)).sum(0)) < 5e-3
    assert _rel_err(ext.column_sum(y), y.float().sum(0)) < 5e-3
    with pytest.raises(ValueError):
        ops.layer_norm_fwd(torch.randn(4, 60, device=DEV, dtype=torch.bfloat16), torch.ones(60, device=DEV),
                           torch.zeros(60, device=DEV), 1e-5)


@pytest.mark.parametrize("tokens,out_f,in_f", [(4096, 200, 328), (8192, 1600, 1600), (2048, 72, 104)])
def test_gemm_split_k_weight_gradient_shape(tokens, out_f, in_f):
    """fp32 weight gradients: few tiles with a long K are split (8 ways / 3 ways for the first two shapes) and summed
    by TMA reduce-add; the last shape's row pitch (416 bytes) is fine for TMA, its 72 x 104 output a single tile."""
    ops, ext = _ops()
    torch.manual_seed(2)
    dy = torch.randn(tokens, out_f, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(tokens, in_f, device=DEV, dtype=torch.bfloat16)
    ref = dy.float().t() @ x.float()
    dw = ext.gemm(dy, x, True, False, None, None, torch.float32, False)
    ext.check_status()
    assert _rel_err(dw, ref) < 1e-4


@pytest.mark.parametrize("H", [64, 1600, 5120])
def test_layer_norm(H):
    ops, ext = _ops()
    torch.manual_seed(3)
    rows = 777
    x = (torch.randn(rows, H, device=DEV) * 2 + 0.5).bfloat16()
    g, b = torch.randn(H, device=DEV), torch.randn(H, device=DEV)
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    xr = x.float().requires_grad_(True)
    gr, br = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (H, ), gr, br, 1e-5)
    yr.backward(dy.float())
    y, mean, rstd = ops.layer_norm_fwd(x, g, b, 1e-5)
    dx, dg, db = ops.layer_norm_bwd(dy, x, mean, rstd, g)
    assert _rel_err(y, yr) < 5e-3 and _rel_err(dx, xr.grad) < 6e-3
    assert _rel_err(dg, gr.grad) < 1e-3 and _rel_err(db, br.grad) < 1e-3
    # the two-pass pieces used by the sharded layer norms reproduce the same numbers
    mom = ops.row_moments(x)
    mean2 = mom[:, 0] / H
    rstd2 = torch.rsqrt((mom[:, 1] / H - mean2 * mean2).clamp_min(0) + 1e-5)
    y2 = ops.norm_apply(x, mean2, rstd2, g, b)
    assert _rel_err(y2, yr) < 5e-3
    part, dg2, db2 = ops.norm_bwd_partials(dy, x, mean, rstd, g)
    dx2 = ops.norm_bwd_apply(dy, x, mean, rstd, g, part, H)
    assert _rel_err(dx2, xr.grad) < 6e-3 and _rel_err(dg2, gr.grad) < 1e-3 and _rel_err(db2, br.grad) < 1e-3


@pytest.mark.parametrize("H", [64, 1600, 2048, 5120])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_add_layer_norm_fused(H, dtype):
    """Residual add + layer norm in one kernel (forward: the sum and its normalised value; backward: the norm's input
    gradient plus the gradient that reaches the sum directly) against the fp32 formulation."""
    ops, ext = _ops()
    from cubework_b200.parallel.functional import add_layer_norm
    torch.manual_seed(6)
    rows = 391
    x = (torch.randn(rows, H, device=DEV) * 1.5).to(dtype).requires_grad_(True)
    r = (torch.randn(rows, H, device=DEV) * 0.5 + 0.3).to(dtype).requires_grad_(True)
    g = torch.randn(H, device=DEV).requires_grad_(True)
    b = torch.randn(H, device=DEV).requires_grad_(True)
    ds, dy = torch.randn(rows, H, device=DEV).to(dtype), torch.randn(rows, H, device=DEV).to(dtype)
    total, y = add_layer_norm(x, r, g, b, 1e-5)
    torch.autograd.backward([total, y], [ds, dy])
    xr, rr = x.detach().float().requires_grad_(True), r.detach().float().requires_grad_(True)
    gr, br = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    sr = xr + rr
    tr = sr + (sr.to(dtype).float() - sr).detach()       # the kernel normalises the rounded sum
    yr = torch.nn.functional.layer_norm(tr, (H, ), gr, br, 1e-5)
    torch.autograd.backward([tr, yr], [ds.float(), dy.float()])
    assert _rel_err(total, tr) < 1e-3 and _rel_err(y, yr) < 6e-3
    assert _rel_err(x.grad, xr.grad) < 8e-3 and torch.equal(x.grad, r.grad)
    assert _rel_err(g.grad, gr.grad) < 2e-3 and _rel_err(b.grad, br.grad) < 2e-3


@pytest.mark.parametrize("V,start", [(6288, 0), (1000, 3000), (50304, 0)])
def test_cross_entropy_pieces(V, start):
    ops, ext = _ops()
    from cubework_b200.parallel.loss import merge_ce_stats
    torch.manual_seed(4)
    rows = 513
    logits = (torch.randn(rows, V, device=DEV) * 3).bfloat16()
    targets = torch.randint(start, start + V, (rows, ), device=DEV)
    targets[::7] = start + V + 5     # not on this shard
    stats = ops.ce_local_stats(logits, targets, start)
    lf = logits.float()
    assert torch.allclose(stats[:, 0], lf.max(-1).values)
    assert _rel_err(stats[:, 1], torch.exp(lf - lf.max(-1, keepdim=True).values).sum(-1)) < 1e-4
    gmax, gsum, tl = merge_ce_stats(stats.unsqueeze(0))
    local = targets - start
    ok = (local >= 0) & (local < V)
    tl_ref = torch.where(ok, lf.gather(-1, local.clamp(0, V - 1)[:, None]).squeeze(-1), torch.zeros_like(tl))
    assert torch.allclose(tl, tl_ref)
    scale = torch.rand(rows, device=DEV)
    grad = ops.ce_grad(logits, targets, start, gmax, gsum, scale)
    p = torch.softmax(lf, -1)
    p[ok, local[ok]] -= 1
    assert _rel_err(grad, p * scale[:, None]) < 6e-3


@pytest.mark.parametrize("act", ["gelu", "relu"])
def test_act_backward_and_column_sum(act):
    ops, ext = _ops()
    torch.manual_seed(5)
    M, N = 1030, 6400
    z = torch.randn(M, N, device=DEV).bfloat16()
    dy = torch.randn(M, N, device=DEV).bfloat16()
    zr = z.float().requires_grad_(True)
    (torch.nn.functional.gelu(zr) if act == "gelu" else torch.relu(zr)).backward(dy.float())
    dz, db = ops.act_backward(dy, z, act, True)
    assert _rel_err(dz, zr.grad) < 6e-3
    assert _rel_err(db, zr.grad.sum(0)) < 5e-3
    assert _rel_err(ops.column_sum(dy), dy.float().sum(0)) < 1e-4


def test_embedding():
    ops, ext = _ops()
    torch.manual_seed(6)
    V, H, start = 500, 1600, 250
    w = torch.randn(V, H, device=DEV)
    ids = torch.randint(0, 1000, (4, 33), device=DEV)
    out = ops.embedding_fwd(ids, w, start, torch.bfloat16)
    local = ids - start
    ok = (local >= 0) & (local < V)
    ref = torch.nn.functional.embedding(local.clamp(0, V - 1), w) * ok[..., None]
    assert _rel_err(out, ref) < 5e-3
    dout = torch.randn(4, 33, H, device=DEV).bfloat16()
    dw = ops.embedding_bwd(dout, ids, start, V, torch.float32)
    ref_dw = torch.zeros(V, H, device=DEV)
    ref_dw.index_add_(0, local[ok], dout.float()[ok])
    assert _rel_err(dw, ref_dw) < 1e-5


def test_fused_adamw_and_clip_match_torch():
    ops, ext = _ops()
    from cubework_b200.optim import FusedAdamW, FusedSGD
    from cubework_b200.utils import clip_grad_norm
    torch.manual_seed(7)
    shapes = [(1600, 600), (600, ), (50, 7), (33000, )]
    ps = [torch.randn(s, device=DEV, requires_grad=True) for s in shapes]
    qs = [p.detach().clone().requires_grad_(True) for p in ps]
    # give two parameters a bf16 shadow, as the linears do under autocast
    sh = [ops.shadow(ps[0], torch.bfloat16), ops.shadow(ps[3], torch.bfloat16)]
    o1, o2 = FusedAdamW(ps, lr=1e-2, weight_decay=0.05), torch.optim.AdamW(qs, lr=1e-2, weight_decay=0.05)
    for step in range(3):
        for p, q in zip(ps, qs):
            g = torch.randn_like(p)
            p.grad = g.clone() if step != 1 else g.bfloat16().float().clone()
            q.grad = p.grad.clone()
        n1 = clip_grad_norm(ps, 1.0)
        n2 = torch.nn.utils.clip_grad_norm_(qs, 1.0)
        assert abs(n1.item() - n2.item()) < 1e-3 * n2.item()
        o1.step(), o2.step()
    for p, q in zip(ps, qs):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-6)
    assert torch.equal(sh[0], ps[0].detach().bfloat16()) and torch.equal(sh[1], ps[3].detach().bfloat16())
    assert ops.shadow(ps[0], torch.bfloat16) is sh[0]
    # SGD with momentum
    ps2 = [torch.randn(s, device=DEV, requires_grad=True) for s in shapes]
    qs2 = [p.detach().clone().requires_grad_(True) for p in ps2]
    s1, s2 = FusedSGD(ps2, lr=0.1, momentum=0.9, weight_decay=0.01), torch.optim.SGD(qs2, lr=0.1, momentum=0.9,
                                                                                     weight_decay=0.01)
    for step in range(3):
        for p, q in zip(ps2, qs2):
            p.grad = torch.randn_like(p)
            q.grad = p.grad.clone()
        s1.step(), s2.step()
    for p, q in zip(ps2, qs2):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dh,T", [(25, 256), (64, 197), (48, 130), (80, 384), (128, 256)])
def test_attention_matches_reference(causal, dh, T):
    ops, ext = _ops()
    torch.manual_seed(8)
    B, H = 2, 3
    qkv = (torch.randn(B, T, H, 3 * dh, device=DEV) * 0.7).bfloat16().requires_grad_(True)
    key_bias = None
    if not causal:
        key_bias = torch.zeros(B, T, device=DEV)
        key_bias[0, T - 9:] = -10000.0
    out = ops.attention_packed(qkv, causal, key_bias)
    dout = torch.randn_like(out)
    out.backward(dout)
    ext.check_status()
    q32 = qkv.detach().float().requires_grad_(True)
    q, k, v = q32.permute(0, 2, 1, 3).chunk(3, dim=-1)
    ref = ops.attention_reference(q, k, v, causal, key_bias).transpose(1, 2).reshape(B, T, H * dh)
    ref.backward(dout.float())
    assert _rel_err(out, ref) < 1e-2
    assert _rel_err(qkv.grad, q32.grad) < 2e-2


@pytest.mark.parametrize("dh,heads,batch", [(25, 64, 8), (64, 25, 8), (64, 16, 32)])
def test_attention_benchmark_regime_causal_with_key_bias(dh, heads, batch):
    """The benchmark's regime: sequence 1024, enough (batch x heads) tiles that every persistent CTA of the forward
    runs several tiles (512 / 200 / 512 (batch, head) pairs x 8 query tiles on 148 SMs), causal masking AND a
    non-zero key bias (padding) together, as GPT-2 passes them; forward and backward against the fp32 formulation."""
    ops, ext = _ops()
    torch.manual_seed(9)
    T = 1024
    qkv = (torch.randn(batch, T, heads, 3 * dh, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    key_bias = torch.zeros(batch, T, device=DEV)
    key_bias[0, T - 100:] = -10000.0            # right padding of different lengths
    key_bias[1, T - 1:] = -10000.0
    key_bias[batch - 1, 517:] = -10000.0
    out = ops.attention_packed(qkv, True, key_bias)
    dout = torch.randn_like(out)
    out.backward(dout)
    ext.check_status()
    # the fp32 oracle one batch entry at a time (its scores are [heads, T, T] floats)
    worst_o = worst_g = 0.0
    for b in (0, 1, batch // 2, batch - 1):
        q32 = qkv[b:b + 1].detach().float().requires_grad_(True)
        q, k, v = q32.permute(0, 2, 1, 3).chunk(3, dim=-1)
        ref = ops.attention_reference(q, k, v, True, key_bias[b:b + 1]).transpose(1, 2).reshape(1, T, heads * dh)
        ref.backward(dout[b:b + 1].float())
        # rows of padded queries attend to real keys only; compare everything
        worst_o = max(worst_o, _rel_err(out[b:b + 1], ref))
        worst_g = max(worst_g, _rel_err(qkv.grad[b:b + 1], q32.grad))
    assert worst_o < 1e-2 and worst_g < 2e-2, (worst_o, worst_g)


def test_gpt2_tiny_bf16_step_close_to_fp32_cpu():
    """The whole bf16 kernel path (GEMM epilogues, layer norm, attention, CE, AdamW) on a tiny GPT-2."""
    ops, ext = _ops()
    from cubework_b200.engine import Trainer
    from cubework_b200.global_vars import env
    from cubework_b200.models import gpt2
    from cubework_b200.optim import FusedAdamW
    env.load(mode=None)
    torch.manual_seed(0)
    ref = gpt2.build_model("gpt2_tiny", 64, dropout=0.0, embedding_dropout=0.0, init_std=0.02)
    model = gpt2.build_model("gpt2_tiny", 64, dropout=0.0, embedding_dropout=0.0, init_std=0.02)
    model.load_state_dict(ref.state_dict())
    model = model.to(DEV)
    ids = torch.randint(0, 1024, (4, 64))
    batch = dict(input_ids=ids, attention_mask=torch.ones(4, 64), labels=ids)
    crit = gpt2.GPT2LMLoss()
    l_ref = Trainer(ref, crit, FusedAdamW(ref.parameters(), lr=1e-3), amp_dtype=None,
                    device=torch.device("cpu")).step(batch)
    tr = Trainer(model, crit, FusedAdamW(model.parameters(), lr=1e-3), amp_dtype=torch.bfloat16, clip=1.0)
    l_gpu = tr.step(batch)
    ext.check_status()
    assert abs(l_gpu.item() - l_ref.item()) < 3e-2, (l_gpu.item(), l_ref.item())
    l2 = tr.step(batch)
    assert l2.item() < l_gpu.item()
