"""2D (SUMMA) layers against an unsharded master on 4 CPU/gloo ranks (2x2 grid).

Coverage follows the reference's tests/test_2d/check_2d_modules.py: linear, layernorm, embedding,
vocab-parallel embedding, patch embedding, classifier (own / tied), vocab-parallel classifier
(own / tied), plain and vocab-parallel loss — with that file's slicing recipes (i = grid row =
COL-group rank, j = grid column = ROW-group rank).
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from dist_utils import check_close, chunk, run_dist

B, S, H, V, C = 4, 3, 8, 16, 12
IMG, PATCH, CH = 8, 4, 3


def _bcast(t):
    dist.broadcast(t, src=0)
    return t


def _check_2d():
    import cubework_b200.module as nn_
    from cubework_b200.distributed import ParallelManager as pm
    from cubework_b200.global_vars import env
    from cubework_b200.parallel.ops_2d import summa_ABT, summa_ATB
    q = env.summa_dim
    i, j = pm.PARALLEL_2D_COL.local_rank, pm.PARALLEL_2D_ROW.local_rank
    torch.manual_seed(0)

    def act(x):  # [B,S,H] activation layout
        return chunk(chunk(x, q, 0, i), q, -1, j).contiguous()

    def vec2(x):  # parameters split q^2 ways on the last dim: j outer, i inner
        return chunk(chunk(x, q, -1, j), q, -1, i).contiguous()

    # ---- linear ---------------------------------------------------------------------------------------
    layer = nn_.Linear(H, 2 * H)
    Wm, bm = _bcast(torch.randn(H, 2 * H)), _bcast(torch.randn(2 * H))
    layer.weight.data.copy_(chunk(chunk(Wm, q, 0, i), q, -1, j))
    layer.bias.data.copy_(vec2(bm))
    xm = _bcast(torch.randn(B, S, H))
    x = act(xm).requires_grad_(True)
    y = layer(x)
    Wr, br, xr = Wm.clone().requires_grad_(True), bm.clone().requires_grad_(True), xm.clone().requires_grad_(True)
    yr = xr @ Wr + br
    check_close(y, act(yr), what="linear2d fwd")
    g = _bcast(torch.randn_like(yr))
    y.backward(act(g)), yr.backward(g)
    check_close(x.grad, act(xr.grad), what="linear2d dx")
    check_close(layer.weight.grad, chunk(chunk(Wr.grad, q, 0, i), q, -1, j), what="linear2d dW")
    check_close(layer.bias.grad, vec2(br.grad), what="linear2d db")

    # ---- the two other SUMMA products, directly ---------------------------------------------------------
    Am, Bm = _bcast(torch.randn(B * S, H)), _bcast(torch.randn(2 * H, H))
    a_loc, b_loc = chunk(chunk(Am, q, 0, i), q, -1, j).contiguous(), chunk(chunk(Bm, q, 0, i), q, -1, j).contiguous()
    c = summa_ABT(a_loc, b_loc, q, (B * S // q, 2 * H // q), pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL)
    check_close(c, chunk(chunk(Am @ Bm.t(), q, 0, i), q, -1, j), what="summa ABT")
    Dm = _bcast(torch.randn(B * S, 2 * H))
    d_loc = chunk(chunk(Dm, q, 0, i), q, -1, j).contiguous()
    c = summa_ATB(a_loc, d_loc, q, (H // q, 2 * H // q), pm.PARALLEL_2D_ROW, pm.PARALLEL_2D_COL)
    check_close(c, chunk(chunk(Am.t() @ Dm, q, 0, i), q, -1, j), what="summa ATB")

    # ---- layer norm ----------------------------------------------------------------------------------------
    ln = nn_.LayerNorm(H, eps=1e-5)
    gm, bem = _bcast(torch.randn(H)), _bcast(torch.randn(H))
    ln.weight.data.copy_(vec2(gm)), ln.bias.data.copy_(vec2(bem))
    xl = act(xm).requires_grad_(True)
    yl = ln(xl)
    xlr, gmr, bemr = xm.clone().requires_grad_(True), gm.clone().requires_grad_(True), bem.clone().requires_grad_(True)
    ylr = F.layer_norm(xlr, (H, ), gmr, bemr, 1e-5)
    check_close(yl, act(ylr), what="ln2d fwd")
    gl = _bcast(torch.randn_like(ylr))
    yl.backward(act(gl)), ylr.backward(gl)
    check_close(xl.grad, act(xlr.grad), what="ln2d dx")
    check_close(ln.weight.grad, vec2(gmr.grad), what="ln2d dgamma")
    check_close(ln.bias.grad, vec2(bemr.grad), what="ln2d dbeta")

    # ---- embeddings --------------------------------------------------------------------------------------------
    ids = _bcast(torch.randint(0, V, (B, S)))
    Em = _bcast(torch.randn(V, H))
    ge = _bcast(torch.randn(B, S, H))
    Er = Em.clone().requires_grad_(True)
    F.embedding(ids, Er).backward(ge)
    emb = nn_.Embedding(V, H)
    emb.weight.data.copy_(vec2(Em))
    out = emb(ids)
    check_close(out, act(F.embedding(ids, Em)), what="embed2d fwd")
    out.backward(act(ge))
    check_close(emb.weight.grad, vec2(Er.grad), what="embed2d dW")
    vemb = nn_.Embedding(V, H, vocab_parallel=True)
    vemb.weight.data.copy_(chunk(chunk(Em, q, -1, j), q, 0, i))
    out = vemb(ids)
    check_close(out, act(F.embedding(ids, Em)), what="vocab embed2d fwd")
    out.backward(act(ge))
    check_close(vemb.weight.grad, chunk(chunk(Er.grad, q, -1, j), q, 0, i), what="vocab embed2d dW")

    # ---- patch embedding -------------------------------------------------------------------------------------------
    pe = nn_.PatchEmbedding(IMG, PATCH, CH, H)
    Wp, bp = _bcast(torch.randn(H, CH, PATCH, PATCH)), _bcast(torch.randn(H))
    cls, pos = _bcast(torch.randn(1, 1, H)), _bcast(torch.randn(1, (IMG // PATCH)**2 + 1, H))
    pe.weight.data.copy_(chunk(chunk(Wp, q, 0, j), q, 0, i)), pe.bias.data.copy_(chunk(chunk(bp, q, 0, j), q, 0, i))
    pe.cls_token.data.copy_(vec2(cls)), pe.pos_embed.data.copy_(vec2(pos))
    img = _bcast(torch.randn(B, CH, IMG, IMG))
    out = pe(img)
    refs = [t.clone().requires_grad_(True) for t in (Wp, bp, cls, pos)]
    o = F.conv2d(img, refs[0], refs[1], stride=PATCH).flatten(2).transpose(1, 2)
    o = torch.cat((refs[2].expand(B, -1, -1), o), dim=1) + refs[3]
    check_close(out, act(o), what="patch2d fwd")
    gp = _bcast(torch.randn_like(o))
    out.backward(act(gp)), o.backward(gp)
    check_close(pe.weight.grad, chunk(chunk(refs[0].grad, q, 0, j), q, 0, i), what="patch2d dW")
    check_close(pe.bias.grad, chunk(chunk(refs[1].grad, q, 0, j), q, 0, i), what="patch2d db")
    check_close(pe.cls_token.grad, vec2(refs[2].grad), what="patch2d dcls")
    check_close(pe.pos_embed.grad, vec2(refs[3].grad), what="patch2d dpos")

    # ---- classifiers + losses --------------------------------------------------------------------------------------
    for vocab_parallel in (False, True):
        for tied in (False, True):
            env.vocab_parallel = vocab_parallel
            src = (vemb if vocab_parallel else emb)
            nc = V if tied else C
            head = nn_.Classifier(H, nc, weight=src.weight if tied else None, bias=True)
            Wc = Em if tied else _bcast(torch.randn(nc, H))
            bc = _bcast(torch.randn(nc))
            if vocab_parallel:
                assert type(head.linear).__name__ == "VocabParallelClassifier2D"
                w_slice = lambda t: chunk(chunk(t, q, 0, i), q, -1, j)
                head.bias.data.copy_(chunk(chunk(bc, q, 0, j), q, 0, i))
            else:
                assert type(head.linear).__name__ == "Classifier2D"
                w_slice = vec2
                head.bias.data.copy_(bc)
            if not tied:
                head.weight.data.copy_(w_slice(Wc))
            src.weight.grad = None
            xh = act(xm).requires_grad_(True)
            logits = head(xh)
            Wcr, bcr, xhr = (t.clone().requires_grad_(True) for t in (Wc, bc, xm))
            logits_r = F.linear(xhr, Wcr, bcr)
            exp = act(logits_r) if vocab_parallel else chunk(logits_r, q, 0, i)
            check_close(logits, exp, what=f"classifier2d fwd vp={vocab_parallel} tied={tied}")
            tgt = _bcast(torch.randint(0, nc, (B, S)))
            crit = nn_.CrossEntropyLoss()
            # the 2D losses take [N, classes] logits and split the *batch* of the targets themselves
            loss = crit(logits.reshape(-1, logits.shape[-1]), tgt.view(-1))
            loss_r = F.cross_entropy(logits_r.view(-1, nc), tgt.view(-1))
            check_close(loss, loss_r, what=f"CE2d vp={vocab_parallel}")
            loss.backward(), loss_r.backward()
            check_close(xh.grad, act(xhr.grad), what=f"classifier2d dx vp={vocab_parallel} tied={tied}")
            check_close(head.weight.grad, w_slice(Wcr.grad), what=f"classifier2d dW vp={vocab_parallel} tied={tied}")
            if vocab_parallel:
                check_close(head.bias.grad, chunk(chunk(bcr.grad, q, 0, j), q, 0, i), what="classifier2d db")
            else:
                check_close(head.bias.grad, bcr.grad, what="classifier2d db")
            acc = nn_.Accuracy() if not vocab_parallel else None
            if acc is not None:
                a = acc(logits.detach(), tgt)
                ar = (logits_r.argmax(-1) == tgt).sum() / B
                check_close(a, ar.float(), what="accuracy2d")


def test_2d_world4():
    run_dist(_check_2d, 4, tp="2d", tp_size=4)


def test_2d_with_data_parallel_world8():
    run_dist(_check_2d, 8, tp="2d", tp_size=4)


if __name__ == "__main__":
    test_2d_world4()
