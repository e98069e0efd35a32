"""1D layers against an unsharded master on CPU/gloo ranks.

Same coverage as the reference's tests/test_1d/check_1d_modules.py (linear col/row, embedding,
vocab-parallel embedding, classifier own/tied weight, vocab-parallel classifier own/tied, vocab-parallel
loss) with the slicing recipes of that file, plus layer norm, dropout streams and gathered outputs.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from dist_utils import check_close, chunk, run_dist

B, S, H, V, C = 4, 6, 16, 32, 12


def _bcast(t):
    dist.broadcast(t, src=0)
    return t


def _check_1d():
    import cubework_b200.module as nn_
    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.global_vars import env
    from cubework_b200.parallel.ops_1d import set_parallel_input
    n, r = pm.PARALLEL_1D.world_size, pm.PARALLEL_1D.local_rank
    torch.manual_seed(0)

    # ---- column linear ------------------------------------------------------------------------
    set_parallel_input(False)
    layer = nn_.Linear1D(H, 2 * H)
    assert type(layer.linear).__name__ == "Linear1D_Col" and env.parallel_input_1d
    Wm, bm = _bcast(torch.randn(2 * H, H)), _bcast(torch.randn(2 * H))
    layer.weight.data.copy_(chunk(Wm, n, 0, r))
    layer.bias.data.copy_(chunk(bm, n, 0, r))
    xm = _bcast(torch.randn(B, S, H))
    x = xm.clone().requires_grad_(True)
    y = layer(x)
    Wm.requires_grad_(True), bm.requires_grad_(True)
    xr = xm.clone().requires_grad_(True)
    yr = F.linear(xr, Wm, bm)
    check_close(y, chunk(yr, n, -1, r), what="col fwd")
    g = _bcast(torch.randn_like(yr))
    y.backward(chunk(g, n, -1, r).contiguous())
    yr.backward(g)
    check_close(x.grad, xr.grad, what="col dx")
    check_close(layer.weight.grad, chunk(Wm.grad, n, 0, r), what="col dW")
    check_close(layer.bias.grad, chunk(bm.grad, n, 0, r), what="col db")

    # ---- row linear (constructed right after a column layer) -------------------------------------
    row = nn_.Linear1D(2 * H, H)
    assert type(row.linear).__name__ == "Linear1D_Row" and not env.parallel_input_1d
    W2, b2 = _bcast(torch.randn(H, 2 * H)), _bcast(torch.randn(H))
    row.weight.data.copy_(chunk(W2, n, -1, r))
    row.bias.data.copy_(b2)
    x2m = _bcast(torch.randn(B, S, 2 * H))
    x2 = chunk(x2m, n, -1, r).clone().requires_grad_(True)
    y2 = row(x2)
    W2.requires_grad_(True), b2.requires_grad_(True)
    x2r = x2m.clone().requires_grad_(True)
    y2r = F.linear(x2r, W2, b2)
    check_close(y2, y2r, what="row fwd")
    g2 = _bcast(torch.randn_like(y2r))
    y2.backward(g2)
    y2r.backward(g2)
    check_close(x2.grad, chunk(x2r.grad, n, -1, r), what="row dx")
    check_close(row.weight.grad, chunk(W2.grad, n, -1, r), what="row dW")
    check_close(row.bias.grad, b2.grad, what="row db")

    # ---- column linear with fused GELU and gathered output -----------------------------------------
    set_parallel_input(False)
    act = nn_.Linear(H, 2 * H, activation="gelu")
    act.weight.data.copy_(chunk(Wm.detach(), n, 0, r))
    act.bias.data.copy_(chunk(bm.detach(), n, 0, r))
    xa = xm.clone().requires_grad_(True)
    ya = act(xa)
    xar = xm.clone().requires_grad_(True)
    Wg, bg = Wm.detach().clone().requires_grad_(True), bm.detach().clone().requires_grad_(True)
    yar = F.gelu(F.linear(xar, Wg, bg))
    check_close(ya, chunk(yar, n, -1, r), what="col+gelu fwd")
    ya.backward(chunk(g, n, -1, r).contiguous())
    yar.backward(g)
    check_close(xa.grad, xar.grad, what="col+gelu dx")
    check_close(act.weight.grad, chunk(Wg.grad, n, 0, r), what="col+gelu dW")
    check_close(act.bias.grad, chunk(bg.grad, n, 0, r), what="col+gelu db")
    set_parallel_input(False)
    gat = nn_.Linear1D(H, 2 * H, gather_output=True)
    gat.weight.data.copy_(chunk(Wm.detach(), n, 0, r))
    gat.bias.data.copy_(chunk(bm.detach(), n, 0, r))
    check_close(gat(xm), F.linear(xm, Wm.detach(), bm.detach()), what="col gather fwd")
    set_parallel_input(False)

    # ---- layer norm --------------------------------------------------------------------------------
    ln = nn_.LayerNorm(H, eps=1e-5)
    gm, bem = _bcast(torch.randn(H)), _bcast(torch.randn(H))
    ln.weight.data.copy_(gm), ln.bias.data.copy_(bem)
    xl = xm.clone().requires_grad_(True)
    yl = ln(xl)
    xlr = xm.clone().requires_grad_(True)
    gmr, bemr = gm.clone().requires_grad_(True), bem.clone().requires_grad_(True)
    ylr = F.layer_norm(xlr, (H, ), gmr, bemr, 1e-5)
    check_close(yl, ylr, what="ln fwd")
    gl = _bcast(torch.randn_like(ylr))
    yl.backward(gl), ylr.backward(gl)
    check_close(xl.grad, xlr.grad, what="ln dx")
    check_close(ln.weight.grad, gmr.grad, what="ln dgamma")
    check_close(ln.bias.grad, bemr.grad, what="ln dbeta")

    # ---- embeddings ------------------------------------------------------------------------------------
    ids = _bcast(torch.randint(0, V, (B, S)))
    Em = _bcast(torch.randn(V, H))
    ge = _bcast(torch.randn(B, S, H))
    Er = Em.clone().requires_grad_(True)
    F.embedding(ids, Er).backward(ge)
    emb = nn_.Embedding(V, H)
    emb.weight.data.copy_(chunk(Em, n, -1, r))
    out = emb(ids)
    check_close(out, F.embedding(ids, Em), what="embed fwd")
    out.backward(ge)
    check_close(emb.weight.grad, chunk(Er.grad, n, -1, r), what="embed dW")
    vemb = nn_.Embedding(V, H, vocab_parallel=True)
    assert env.vocab_parallel
    vemb.weight.data.copy_(chunk(Em, n, 0, r))
    out = vemb(ids)
    check_close(out, F.embedding(ids, Em), what="vocab embed fwd")
    out.backward(ge)
    check_close(vemb.weight.grad, chunk(Er.grad, n, 0, r), what="vocab embed dW")

    # ---- vocab-parallel classifier: tied to the embedding, and with its own weight; + loss ----------------
    for tied in (True, False):
        env.vocab_parallel = True
        head = nn_.Classifier(H, V, weight=vemb.weight if tied else None, bias=not tied)
        assert type(head.linear).__name__ == "VocabParallelClassifier1D"
        Wc = Em if tied else _bcast(torch.randn(V, H))
        bc = None if tied else _bcast(torch.randn(V))
        if not tied:
            head.weight.data.copy_(chunk(Wc, n, 0, r))
            head.bias.data.copy_(chunk(bc, n, 0, r))
        vemb.weight.grad = None
        xh = xm.clone().requires_grad_(True)
        logits = head(xh)
        Wcr = Wc.clone().requires_grad_(True)
        bcr = bc.clone().requires_grad_(True) if bc is not None else None
        xhr = xm.clone().requires_grad_(True)
        logits_r = F.linear(xhr, Wcr, bcr)
        check_close(logits, chunk(logits_r, n, -1, r), what="vocab classifier fwd")
        tgt = _bcast(torch.randint(0, V, (B, S)))
        crit = nn_.CrossEntropyLoss()
        assert type(crit.loss).__name__ == "VocabParallelCrossEntropyLoss1D"
        loss = crit(logits.view(-1, logits.shape[-1]), tgt.view(-1))
        loss_r = F.cross_entropy(logits_r.view(-1, V), tgt.view(-1))
        check_close(loss, loss_r, what="vocab CE fwd")
        loss.backward(), loss_r.backward()
        check_close(xh.grad, xhr.grad, what="vocab classifier dx")
        check_close(head.weight.grad, chunk(Wcr.grad, n, 0, r), what="vocab classifier dW")
        if not tied:
            check_close(head.bias.grad, chunk(bcr.grad, n, 0, r), what="vocab classifier db")

    # ---- plain classifier (own / tied weight) ----------------------------------------------------------
    for tied in (False, True):
        env.vocab_parallel = False
        set_parallel_input(False)
        head = nn_.Classifier(H, C if not tied else V, weight=emb.weight if tied else None, bias=True)
        assert type(head.linear).__name__ == "Classifier1D"
        nc = V if tied else C
        Wc = Em if tied else _bcast(torch.randn(nc, H))
        bc = _bcast(torch.randn(nc))
        if not tied:
            head.weight.data.copy_(chunk(Wc, n, -1, r))
        head.bias.data.copy_(bc)
        emb.weight.grad = None
        xh = xm.clone().requires_grad_(True)
        logits = head(xh)
        Wcr, bcr, xhr = Wc.clone().requires_grad_(True), bc.clone().requires_grad_(True), xm.clone().requires_grad_(True)
        logits_r = F.linear(xhr, Wcr, bcr)
        check_close(logits, logits_r, what="classifier fwd")
        gc = _bcast(torch.randn_like(logits_r))
        logits.backward(gc), logits_r.backward(gc)
        check_close(xh.grad, xhr.grad, what="classifier dx")
        check_close(head.weight.grad, chunk(Wcr.grad, n, -1, r), what="classifier dW")
        check_close(head.bias.grad, bcr.grad, what="classifier db")
        crit = nn_.CrossEntropyLoss()
        tgt = _bcast(torch.randint(0, nc, (B, S)))
        check_close(crit(logits.detach().view(-1, nc), tgt.view(-1)),
                    F.cross_entropy(logits_r.detach().view(-1, nc), tgt.view(-1)), what="plain CE")

    # ---- dropout streams: replicated input -> same mask on every rank; sharded -> per-rank mask --------
    set_parallel_input(False)
    d_rep = nn_.Dropout(0.5)
    ones = torch.ones(64, 64)
    m = d_rep(ones)
    ms = [torch.empty_like(m) for _ in range(n)]
    dist.all_gather(ms, m)
    assert all(torch.equal(ms[0], t) for t in ms), "replicated dropout must agree across ranks"
    set_parallel_input(True)
    d_sh = nn_.Dropout(0.5)
    m = d_sh(ones)
    dist.all_gather(ms, m)
    assert not torch.equal(ms[0], ms[1]), "sharded dropout must differ across ranks"
    set_parallel_input(False)


def test_1d_world2():
    run_dist(_check_1d, 2, tp="1d", tp_size=2)


def test_1d_world4():
    run_dist(_check_1d, 4, tp="1d", tp_size=4)


if __name__ == "__main__":
    test_1d_world2()
