"""3D (cube) layers against an unsharded master on 8 CPU/gloo ranks (2x2x2 cube).

Coverage follows the reference's tests/test_3d/check_3d_modules.py: linear, layernorm, classifier,
vocab-parallel classifier (own / tied), embedding, vocab-parallel embedding, patch embedding, plain and
vocab-parallel loss, with that file's slicing recipes (j = input, i = weight, k = output group rank
before any swap).  One deliberate difference is asserted: the Classifier3D weight gradient is present
(and identical) on every rank holding that shard, not only on the cube diagonal.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from dist_utils import check_close, chunk, run_dist

B, S, H, V, C = 8, 3, 8, 16, 12
IMG, PATCH, CH = 8, 4, 3


def _bcast(t):
    dist.broadcast(t, src=0)
    return t


def _check_3d():
    import cubework_b200.module as nn_
    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.global_vars import env
    d = env.depth_3d
    j, i, k = pm.PARALLEL_3D_INPUT.local_rank, pm.PARALLEL_3D_WEIGHT.local_rank, pm.PARALLEL_3D_OUTPUT.local_rank
    torch.manual_seed(0)
    names0 = (env.input_group_3d, env.output_group_3d)

    def act_in(x):   # layer input: batch by (i outer, j inner), hidden by k
        return chunk(chunk(chunk(x, d, 0, i), d, -1, k), d, 0, j).contiguous()

    def act_out(x):  # linear output: batch by (i outer, k inner), hidden by j
        return chunk(chunk(chunk(x, d, 0, i), d, -1, j), d, 0, k).contiguous()

    # ---- linear (then a second one to come back to the input layout) ----------------------------------
    l1 = nn_.Linear(H, 2 * H)
    assert (env.input_group_3d, env.output_group_3d) == (names0[1], names0[0]), "Linear3D must swap in/out"
    Wm, bm = _bcast(torch.randn(H, 2 * H)), _bcast(torch.randn(2 * H))
    l1.weight.data.copy_(chunk(chunk(chunk(Wm, d, 0, k), d, -1, j), d, -1, i))
    l1.bias.data.copy_(chunk(bm, d, 0, j))
    xm = _bcast(torch.randn(B, S, H))
    x = act_in(xm).requires_grad_(True)
    y = l1(x)
    Wr, br, xr = (t.clone().requires_grad_(True) for t in (Wm, bm, xm))
    yr = xr @ Wr + br
    check_close(y, act_out(yr), what="linear3d fwd")
    g = _bcast(torch.randn_like(yr))
    y.backward(act_out(g)), yr.backward(g)
    check_close(x.grad, act_in(xr.grad), what="linear3d dx")
    check_close(l1.weight.grad, chunk(chunk(chunk(Wr.grad, d, 0, k), d, -1, j), d, -1, i), what="linear3d dW")
    check_close(l1.bias.grad, chunk(br.grad, d, 0, j), what="linear3d db")
    l2 = nn_.Linear(2 * H, H)   # built in the swapped state: its input layout is l1's output layout
    assert (env.input_group_3d, env.output_group_3d) == names0
    W2, b2 = _bcast(torch.randn(2 * H, H)), _bcast(torch.randn(H))
    l2.weight.data.copy_(chunk(chunk(chunk(W2, d, 0, j), d, -1, k), d, -1, i))
    l2.bias.data.copy_(chunk(b2, d, 0, k))
    zm = _bcast(torch.randn(B, S, 2 * H))
    check_close(l2(act_out(zm)), act_in(zm @ W2 + b2), what="linear3d (swapped) fwd")

    # ---- layer norm -------------------------------------------------------------------------------------
    ln = nn_.LayerNorm(H, eps=1e-5)
    gm, bem = _bcast(torch.randn(H)), _bcast(torch.randn(H))
    ln.weight.data.copy_(chunk(gm, d, 0, k)), ln.bias.data.copy_(chunk(bem, d, 0, k))
    xl = act_in(xm).requires_grad_(True)
    yl = ln(xl)
    xlr, gmr, bemr = (t.clone().requires_grad_(True) for t in (xm, gm, bem))
    ylr = F.layer_norm(xlr, (H, ), gmr, bemr, 1e-5)
    check_close(yl, act_in(ylr), what="ln3d fwd")
    gl = _bcast(torch.randn_like(ylr))
    yl.backward(act_in(gl)), ylr.backward(gl)
    check_close(xl.grad, act_in(xlr.grad), what="ln3d dx")
    check_close(ln.weight.grad, chunk(gmr.grad, d, 0, k), what="ln3d dgamma")
    check_close(ln.bias.grad, chunk(bemr.grad, d, 0, k), what="ln3d dbeta")

    # ---- embeddings -----------------------------------------------------------------------------------------
    ids = _bcast(torch.randint(0, V, (B, S)))
    Em = _bcast(torch.randn(V, H))
    ge = _bcast(torch.randn(B, S, H))
    Er = Em.clone().requires_grad_(True)
    F.embedding(ids, Er).backward(ge)
    emb = nn_.Embedding(V, H)
    emb.weight.data.copy_(chunk(Em, d, -1, k))
    out = emb(ids)
    check_close(out, act_in(F.embedding(ids, Em)), what="embed3d fwd")
    out.backward(act_in(ge))
    check_close(emb.weight.grad, chunk(Er.grad, d, -1, k), what="embed3d dW")
    vemb = nn_.Embedding(V, H, vocab_parallel=True)
    vslice = lambda t: chunk(chunk(chunk(t, d, 0, j), d, 0, i), d, -1, k)
    vemb.weight.data.copy_(vslice(Em))
    out = vemb(ids)
    check_close(out, act_in(F.embedding(ids, Em)), what="vocab embed3d fwd")
    out.backward(act_in(ge))
    check_close(vemb.weight.grad, vslice(Er.grad), what="vocab embed3d dW")

    # ---- patch embedding ------------------------------------------------------------------------------------------
    pe = nn_.PatchEmbedding(IMG, PATCH, CH, H)
    Wp, bp = _bcast(torch.randn(H, CH, PATCH, PATCH)), _bcast(torch.randn(H))
    cls, pos = _bcast(torch.randn(1, 1, H)), _bcast(torch.randn(1, (IMG // PATCH)**2 + 1, H))
    pe.weight.data.copy_(chunk(Wp, d, 0, k)), pe.bias.data.copy_(chunk(bp, d, 0, k))
    pe.cls_token.data.copy_(chunk(cls, d, -1, k)), pe.pos_embed.data.copy_(chunk(pos, d, -1, k))
    img = _bcast(torch.randn(B, CH, IMG, IMG))
    out = pe(img)
    refs = [t.clone().requires_grad_(True) for t in (Wp, bp, cls, pos)]
    o = F.conv2d(img, refs[0], refs[1], stride=PATCH).flatten(2).transpose(1, 2)
    o = torch.cat((refs[2].expand(B, -1, -1), o), dim=1) + refs[3]
    check_close(out, act_in(o), what="patch3d fwd")
    gp = _bcast(torch.randn_like(o))
    out.backward(act_in(gp)), o.backward(gp)
    check_close(pe.weight.grad, chunk(refs[0].grad, d, 0, k), what="patch3d dW")
    check_close(pe.bias.grad, chunk(refs[1].grad, d, 0, k), what="patch3d db")
    check_close(pe.cls_token.grad, chunk(refs[2].grad, d, -1, k), what="patch3d dcls")
    check_close(pe.pos_embed.grad, chunk(refs[3].grad, d, -1, k), what="patch3d dpos")

    # ---- plain classifier + loss + accuracy ---------------------------------------------------------------------------
    env.vocab_parallel = False
    head = nn_.Classifier(H, C, bias=True)
    assert type(head.linear).__name__ == "Classifier3D"
    Wc, bc = _bcast(torch.randn(C, H)), _bcast(torch.randn(C))
    head.weight.data.copy_(chunk(Wc, d, -1, k)), head.bias.data.copy_(bc)
    xh = act_in(xm).requires_grad_(True)
    logits = head(xh)
    Wcr, bcr, xhr = (t.clone().requires_grad_(True) for t in (Wc, bc, xm))
    logits_r = F.linear(xhr, Wcr, bcr)
    check_close(logits, chunk(chunk(logits_r, d, 0, i), d, 0, j), what="classifier3d fwd")
    tgt = _bcast(torch.randint(0, C, (B, S)))
    crit = nn_.CrossEntropyLoss()
    assert type(crit.loss).__name__ == "CrossEntropyLoss3D"
    loss = crit(logits.reshape(-1, C), tgt.view(-1))
    loss_r = F.cross_entropy(logits_r.view(-1, C), tgt.view(-1))
    check_close(loss, loss_r, what="CE3d")
    loss.backward(), loss_r.backward()
    check_close(xh.grad, act_in(xhr.grad), what="classifier3d dx")
    check_close(head.weight.grad, chunk(Wcr.grad, d, -1, k), what="classifier3d dW (every rank)")
    check_close(head.bias.grad, bcr.grad, what="classifier3d db")
    acc = nn_.Accuracy()
    check_close(acc(logits.detach(), tgt), ((logits_r.argmax(-1) == tgt).sum() / B).float(), what="accuracy3d")

    # ---- vocab-parallel classifier (own / tied) + vocab-parallel loss ---------------------------------------------------
    # tied first: the embedding table was laid out for the roles current before any further swap
    for tied in (True, False):
        env.vocab_parallel = True
        before = (env.input_group_3d, env.output_group_3d)
        head = nn_.Classifier(H, V, weight=vemb.weight if tied else None, bias=True)
        assert type(head.linear).__name__ == "VocabParallelClassifier3D"
        assert (env.input_group_3d, env.output_group_3d) == (before[1], before[0])
        Wc = Em if tied else _bcast(torch.randn(V, H))
        bc = _bcast(torch.randn(V))
        # the layer was built with the roles current at that time; recover them for the slicing
        jj = head.linear.input_parallel_mode.local_rank
        kk = head.linear.output_parallel_mode.local_rank
        wslice = lambda t: chunk(chunk(chunk(t, d, 0, jj), d, 0, i), d, -1, kk)
        if not tied:
            head.weight.data.copy_(wslice(Wc))
        head.bias.data.copy_(chunk(bc, d, 0, jj))
        a_in = lambda t: chunk(chunk(chunk(t, d, 0, i), d, -1, kk), d, 0, jj).contiguous()
        a_out = lambda t: chunk(chunk(chunk(t, d, 0, i), d, -1, jj), d, 0, kk).contiguous()
        vemb.weight.grad = None
        xh = a_in(xm).requires_grad_(True)
        logits = head(xh)
        Wcr, bcr, xhr = (t.clone().requires_grad_(True) for t in (Wc, bc, xm))
        logits_r = F.linear(xhr, Wcr, bcr)
        check_close(logits, a_out(logits_r), what=f"vocab classifier3d fwd tied={tied}")
        tgt = _bcast(torch.randint(0, V, (B, S)))
        crit = nn_.CrossEntropyLoss()
        assert type(crit.loss).__name__ == "VocabParallelCrossEntropyLoss3D"
        loss = crit(logits.reshape(-1, logits.shape[-1]), tgt.view(-1))
        loss_r = F.cross_entropy(logits_r.view(-1, V), tgt.view(-1))
        check_close(loss, loss_r, what="vocab CE3d")
        loss.backward(), loss_r.backward()
        check_close(xh.grad, a_in(xhr.grad), what=f"vocab classifier3d dx tied={tied}")
        if not tied or (jj, kk) == (j, k):
            check_close(head.weight.grad, wslice(Wcr.grad), what=f"vocab classifier3d dW tied={tied}")
        check_close(head.bias.grad, chunk(bcr.grad, d, 0, jj), what="vocab classifier3d db")


def test_3d_world8():
    run_dist(_check_3d, 8, tp="3d", tp_size=8)


if __name__ == "__main__":
    test_3d_world8()
