"""Row kernels, loss, embedding, optimizer and utility kernels vs fp32 PyTorch references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _k():
    from frankentorch_b200.ops import kernels
    return kernels


def _bf(t, dev):
    return t.to(torch.bfloat16).to(dev)


@pytest.mark.parametrize("rows,cols", [(64, 768), (37, 1024), (16, 4096), (8, 264)])
def test_layernorm(cuda_device, rows, cols):
    k = _k()
    torch.manual_seed(0)
    x = _bf(torch.randn(rows, cols) * 2 + 0.5, cuda_device)
    g = _bf(torch.randn(cols) * 0.2 + 1, cuda_device)
    b = _bf(torch.randn(cols) * 0.1, cuda_device)
    y, mean, rstd, _ = k.layernorm_fwd(x, g, b, 1e-5)
    xf = x.float().requires_grad_(True)
    gf, bf = g.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = F.layer_norm(xf, (cols,), gf, bf, 1e-5)
    assert (y.float() - ref).abs().max().item() < 5e-2
    dy = _bf(torch.randn(rows, cols), cuda_device)
    dx, dg, db = k.layernorm_bwd(dy, x, g, mean, rstd)
    ref.backward(dy.float())
    assert (dx.float() - xf.grad).abs().max().item() < 5e-2 * max(1.0, xf.grad.abs().max().item())
    assert (dg - gf.grad).abs().max().item() < 2e-2 * max(1.0, gf.grad.abs().max().item())
    assert (db - bf.grad).abs().max().item() < 2e-2 * max(1.0, bf.grad.abs().max().item())
    k.check_status()


def test_layernorm_fused_residual(cuda_device):
    k = _k()
    torch.manual_seed(1)
    x = _bf(torch.randn(48, 768), cuda_device)
    r = _bf(torch.randn(48, 768), cuda_device)
    g = _bf(torch.ones(768), cuda_device)
    b = _bf(torch.zeros(768), cuda_device)
    y, mean, rstd, xs = k.layernorm_fwd(x, g, b, 1e-5, resid=r)
    s = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(xs, s)
    ref = F.layer_norm(s.float(), (768,), g.float(), b.float(), 1e-5)
    assert (y.float() - ref).abs().max().item() < 5e-2


def test_rmsnorm(cuda_device):
    k = _k()
    torch.manual_seed(2)
    rows, cols = 40, 1024
    x = _bf(torch.randn(rows, cols), cuda_device)
    g = _bf(torch.randn(cols) * 0.1 + 1, cuda_device)
    y, rstd = k.rmsnorm_fwd(x, g, 1e-6)
    xf, gf = x.float().requires_grad_(True), g.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * gf
    assert (y.float() - ref).abs().max().item() < 5e-2
    dy = _bf(torch.randn(rows, cols), cuda_device)
    dx, dg = k.rmsnorm_bwd(dy, x, g, rstd)
    ref.backward(dy.float())
    assert (dx.float() - xf.grad).abs().max().item() < 5e-2
    assert (dg - gf.grad).abs().max().item() < 5e-2 * max(1.0, gf.grad.abs().max().item())


def test_softmax(cuda_device):
    k = _k()
    torch.manual_seed(3)
    x = torch.randn(33, 517, device=cuda_device)
    assert (k.softmax_rows(x) - torch.softmax(x, -1)).abs().max().item() < 1e-5
    xb = _bf(torch.randn(16, 8), cuda_device)
    assert (k.softmax_rows(xb).float() - torch.softmax(xb.float(), -1)).abs().max().item() < 1e-2
    # guards: a row with a non-finite maximum gives zeros
    x[0, 3] = float("inf")
    assert k.softmax_rows(x)[0].abs().sum().item() == 0.0
    s = _bf(torch.randn(3, 64, 64), cuda_device)
    p = k.softmax_causal(s, 0.5)
    mask = torch.triu(torch.ones(64, 64, dtype=torch.bool, device=cuda_device), 1)
    ref = torch.softmax((s.float() * 0.5).masked_fill(mask, float("-inf")), -1)
    assert (p.float() - ref).abs().max().item() < 1e-2
    k.check_status()


@pytest.mark.parametrize("rows,vocab,ld", [(64, 50257, 50304), (17, 1000, 1000), (8, 120000, 120000)])
def test_cross_entropy(cuda_device, rows, vocab, ld):
    k = _k()
    torch.manual_seed(4)
    logits = _bf(torch.randn(rows, ld) * 3, cuda_device)
    tgt = torch.randint(0, vocab, (rows,), device=cuda_device)
    lf = logits.float()[:, :vocab].clone().requires_grad_(True)
    ref = F.cross_entropy(lf, tgt, reduction="none")
    ref.mean().backward()
    losses, dl = k.cross_entropy_fwd_bwd(logits, tgt, vocab, 1.0 / rows, inplace=False)
    k.check_status()
    assert (losses - ref).abs().max().item() < 2e-4          # fp32 statistics over bf16 logits
    # the gradient is rounded to bf16 once: 2^-9 relative, i.e. at most 2^-8 of the loss scale with margin
    err = (dl.float()[:, :vocab] - lf.grad).abs()
    assert (err <= lf.grad.abs() * 2.0 ** -8 + 1e-9).all(), err.max().item()
    assert dl[:, vocab:].abs().sum().item() == 0
    # rows whose target is out of range (the ignore convention) give no loss and no gradient
    tgt2 = tgt.clone()
    tgt2[0], tgt2[-1] = -100, vocab
    l2, d2 = k.cross_entropy_fwd_bwd(logits, tgt2, vocab, 1.0 / rows, inplace=False)
    assert l2[0].item() == 0 and l2[-1].item() == 0 and d2[0].abs().sum().item() == 0 and d2[-1].abs().sum().item() == 0
    assert torch.equal(d2[1:-1], dl[1:-1]) and torch.equal(l2[1:-1], losses[1:-1])
    m = k.reduce_mean(losses)
    assert abs(m.item() - losses.double().mean().item()) < 1e-4


def test_elementwise_and_colsum(cuda_device):
    k = _k()
    torch.manual_seed(5)
    x = _bf(torch.randn(4099) * 3, cuda_device)   # odd length: exercises the scalar tail
    x16 = _bf(torch.randn(4096) * 3, cuda_device)
    for tanh in (True, False):
        y = k.gelu_fwd(x16, tanh)
        ref = F.gelu(x16.float(), approximate="tanh" if tanh else "none")
        assert (y.float() - ref).abs().max().item() < 3e-2
        xf = x16.float().requires_grad_(True)
        F.gelu(xf, approximate="tanh" if tanh else "none").sum().backward()
        dy = torch.ones_like(x16)
        assert (k.gelu_bwd(x16, dy, tanh).float() - xf.grad).abs().max().item() < 2e-2
    a, b = _bf(torch.randn(1000, 16), cuda_device), _bf(torch.randn(1000, 16), cuda_device)
    assert torch.equal(k.add(a, b), (a.float() + b.float()).to(torch.bfloat16))
    f = torch.randn(777, device=cuda_device)
    assert torch.equal(k.cast_f32_to_bf16(f), f.to(torch.bfloat16))
    m = _bf(torch.randn(300, 770), cuda_device)
    cs = k.colsum(m)
    assert (cs - m.float().sum(0)).abs().max().item() < 1e-2
    # wide path (16-byte loads): ragged row counts, a strided view, accumulate mode, run-twice identity;
    # narrow path: an extent that is not a multiple of 8
    for rows, cols, ld in ((8192, 768, 768), (1000, 3072, 3072), (257, 264, 512), (33, 10, 16), (5, 8, 8)):
        base = (torch.randn(rows, ld) * 2).to(torch.bfloat16).to(cuda_device)
        v = base[:, :cols]
        want = v.float().sum(0)
        got = k.colsum(v)
        assert (got - want).abs().max().item() < 2e-2 * max(1.0, rows / 1000), (rows, cols)
        assert torch.equal(got, k.colsum(v))
        acc = got.clone()
        k.colsum(v, out=acc, accumulate=True)
        assert torch.allclose(acc, 2 * got)
    # dropout: replayable, right keep rate, right scale
    big = _bf(torch.ones(1 << 16), cuda_device)
    d1, d2 = k.dropout(big, 0.25, seed=7, offset=3), k.dropout(big, 0.25, seed=7, offset=3)
    assert torch.equal(d1, d2)
    keep = (d1 != 0).float().mean().item()
    assert abs(keep - 0.75) < 0.02
    assert abs(d1.float().max().item() - 1 / 0.75) < 1e-2
    sq = k.sumsq(torch.full((1 << 18,), 0.5, device=cuda_device))
    assert abs(sq.item() - (1 << 18) * 0.25) < 1.0
    k.check_status()


def test_embedding(cuda_device):
    k = _k()
    torch.manual_seed(6)
    V, S, B, d = 1000, 32, 4, 64
    wte = _bf(torch.randn(V, d), cuda_device)
    wpe = _bf(torch.randn(S, d), cuda_device)
    ids = torch.randint(0, 50, (B, S), device=cuda_device)   # many repeats
    out = k.embedding_fwd(ids, wte, wpe, S)
    pos = torch.arange(S, device=cuda_device).repeat(B)
    ref = (wte.float()[ids.reshape(-1)] + wpe.float()[pos]).to(torch.bfloat16)
    assert torch.equal(out, ref)
    dout = _bf(torch.randn(B * S, d), cuda_device)
    dwte = torch.zeros(V, d, device=cuda_device)
    dwpe = torch.zeros(S, d, device=cuda_device)
    k.embedding_bwd(ids, dout, dwte, dwpe, S)
    ref_wte = torch.zeros(V, d, device=cuda_device).index_add_(0, ids.reshape(-1), dout.float())
    ref_wpe = torch.zeros(S, d, device=cuda_device).index_add_(0, pos, dout.float())
    assert (dwte - ref_wte).abs().max().item() < 1e-3
    assert (dwpe - ref_wpe).abs().max().item() < 1e-3
    dwte2 = torch.zeros(V, d, device=cuda_device)
    k.embedding_bwd(ids, dout, dwte2, None, S)
    assert torch.equal(dwte, dwte2)
    # the sort-free form and the sorted form add each table row in the same order: same bits
    dwte3 = torch.zeros(V, d, device=cuda_device)
    k.embedding_bwd(ids, dout, dwte3, None, S, sorted_form=True)
    assert torch.equal(dwte, dwte3)
    # one token everywhere (a single CTA owns all rows), a wide table, a ragged number of positions
    for (rows, dd, hi) in ((300, 768, 1), (257, 1024, 7), (129, 64, 1000)):
        ids2 = torch.randint(0, hi, (1, rows), device=cuda_device)
        do2 = _bf(torch.randn(rows, dd), cuda_device)
        a, b = torch.zeros(V, dd, device=cuda_device), torch.zeros(V, dd, device=cuda_device)
        k.embedding_bwd(ids2, do2, a, None, rows)
        k.embedding_bwd(ids2, do2, b, None, rows, sorted_form=True)
        assert torch.equal(a, b)
        ref = torch.zeros(V, dd, device=cuda_device).index_add_(0, ids2.reshape(-1), do2.float())
        assert (a - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())
    k.check_status()


def test_embedding_reports_token_ids_outside_the_table(cuda_device):
    """A token id that is not a row of the table never becomes an address: the lookup reads row 0 in its place, the
    scatter-add skips it, the status word says BAD_INDEX, and the device keeps working."""
    k = _k()
    torch.manual_seed(7)
    V, S, d = 100, 4, 64
    wte = _bf(torch.randn(V, d), cuda_device)
    ids = torch.tensor([[1, 5, V, -3]], device=cuda_device)
    out = k.embedding_fwd(ids, wte, None, S)
    with pytest.raises(k.KernelError, match="BAD_INDEX"):
        k.check_status()
    assert torch.equal(out[0], wte[1]) and torch.equal(out[1], wte[5])
    assert torch.equal(out[2], wte[0]) and torch.equal(out[3], wte[0])
    k.check_status()                                   # the word was cleared; nothing else is wrong
    dout = _bf(torch.randn(S, d), cuda_device)
    dwte = torch.zeros(V, d, device=cuda_device)
    k.embedding_bwd(ids, dout, dwte, None, S)
    with pytest.raises(k.KernelError, match="BAD_INDEX"):
        k.check_status()
    assert torch.allclose(dwte[1], dout[0].float()) and torch.allclose(dwte[5], dout[1].float())
    assert float(dwte.abs().sum()) == pytest.approx(float(dout[:2].float().abs().sum()), rel=1e-5)
    assert torch.equal(k.embedding_fwd(ids[:, :2].contiguous(), wte, None, 2), wte[[1, 5]])
    k.check_status()


def test_adamw_matches_reference_formula(cuda_device):
    k = _k()
    torch.manual_seed(7)
    n = 10007
    p = torch.randn(n, device=cuda_device)
    g = torch.randn(n, device=cuda_device)
    m = torch.zeros(n, device=cuda_device)
    v = torch.zeros(n, device=cuda_device)
    sh = torch.empty(n, dtype=torch.bfloat16, device=cuda_device)
    pr, mr, vr = p.double().clone(), m.double().clone(), v.double().clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.01
    for step in (1, 2, 3):
        k.adamw(p, sh, g, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=step)
        gd = g.double()
        mr = b1 * mr + (1 - b1) * gd
        vr = b2 * vr + (1 - b2) * gd * gd
        mh, vh = mr / (1 - b1 ** step), vr / (1 - b2 ** step)
        pr = pr - (pr * lr * wd + lr * mh / (vh.sqrt() + eps))
    assert (p.double() - pr).abs().max().item() < 1e-5
    assert torch.equal(sh, p.to(torch.bfloat16))
    k.check_status()


def test_presenter_and_im2col(cuda_device):
    k = _k()
    w, h, rb = 13, 7, 64
    src = torch.randint(0, 256, (h, rb), dtype=torch.uint8, device=cuda_device)
    out = k.present_rgba8(src, w, h, rb)
    ref = src[:, : w * 4].reshape(h, w, 4).float() / 255.0
    assert (out - ref).abs().max().item() < 1e-6
    outh = k.present_rgba8(src, w, h, rb, half=True)
    assert (outh.float() - ref).abs().max().item() < 1e-3
    x = torch.randn(20, 3, device=cuda_device)
    y = k.im2col_1d(x, 3, stride=2, pad=1)
    xp = F.pad(x.t().unsqueeze(0), (1, 1))
    ref = xp.unfold(2, 3, 2).permute(0, 2, 1, 3).reshape(y.shape[0], -1)
    assert torch.equal(y, ref)
    k.check_status()
