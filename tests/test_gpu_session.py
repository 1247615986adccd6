"""``FrankenTorchSession(device="cuda")``: the operator entry point dispatches to the sm_100a kernels,
the ledger names the kernels that ran, and operators without a kernel follow the strict / hardened split."""
import math

import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def _session(mode="hardened"):
    from frankentorch_b200.session import FrankenTorchSession
    return FrankenTorchSession(mode, device="cuda")


def _leaf(s, t, rg=True):
    return s.tensor_variable_from_storage(t.to("cuda", torch.bfloat16).contiguous(), rg)


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))


def _dispatch_lines(s):
    return [e.summary for e in s.evidence() if e.kind.name == "Dispatch"]


def _check(s, out_id, ref_out, pairs, tol=3e-2):
    """Forward and gradients of a CUDA-session expression against the same expression in fp32 torch."""
    assert _rel(s.tensor(out_id), ref_out) < tol
    seed_w = torch.randn(ref_out.shape, generator=torch.Generator().manual_seed(1)).to(ref_out.device)
    loss_ref = (ref_out * seed_w).sum()
    grads_ref = torch.autograd.grad(loss_ref, [p for _, p in pairs], allow_unused=True)
    w = _leaf(s, seed_w.reshape(ref_out.shape), False)
    prod = s.tensor_mul(out_id, w) if ref_out.dim() else out_id
    root = s.tensor_sum(prod) if ref_out.dim() else out_id
    rep = s.tensor_backward(root)
    for (nid, _), g in zip(pairs, grads_ref):
        got = rep.gradient(nid)
        assert got is not None and _rel(got, g) < tol, (nid, _rel(got, g))


def test_hot_operators_run_on_ftk_kernels_and_match_fp32(cuda_device):
    from frankentorch_b200.ops import kernels as K
    torch.manual_seed(0)
    n0 = K.launch_count()
    s = _session("hardened")
    x = torch.randn(64, 128) * 0.5
    w = torch.randn(256, 128) * 0.1
    b = torch.randn(256) * 0.1
    xr, wr, br = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (x, w, b))
    xi, wi, bi = _leaf(s, x), _leaf(s, w), _leaf(s, b)
    _check(s, s.tensor_linear(xi, wi, bi), TF.linear(xr, wr, br), [(xi, xr), (wi, wr), (bi, br)])
    assert "kernel=ftk::gemm" in _dispatch_lines(s)[0] and "fallback_path=false" in _dispatch_lines(s)[0]

    s = _session("hardened")
    a2, b2 = torch.randn(64, 128) * 0.3, torch.randn(128, 96) * 0.3
    ar, b2r = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (a2, b2))
    ai, b2i = _leaf(s, a2), _leaf(s, b2)
    _check(s, s.tensor_matmul(ai, b2i), ar @ b2r, [(ai, ar), (b2i, b2r)])

    s = _session("hardened")
    a3, b3 = torch.randn(3, 64, 128) * 0.3, torch.randn(3, 128, 64) * 0.3
    a3r, b3r = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (a3, b3))
    a3i, b3i = _leaf(s, a3), _leaf(s, b3)
    _check(s, s.tensor_bmm(a3i, b3i), torch.bmm(a3r, b3r), [(a3i, a3r), (b3i, b3r)])

    s = _session("hardened")
    g, be = torch.rand(128) + 0.5, torch.randn(128) * 0.1
    xr, gr, ber = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (x, g, be))
    xi, gi, bei = _leaf(s, x), _leaf(s, g), _leaf(s, be)
    _check(s, s.tensor_layer_norm(xi, gi, bei, eps=1e-5), TF.layer_norm(xr, (128,), gr, ber, 1e-5),
           [(xi, xr), (gi, gr), (bei, ber)])
    assert "ftk::norm_fwd_kernel<layer_norm>" in _dispatch_lines(s)[0]

    s = _session("hardened")
    xr, gr = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (x, g))
    xi, gi = _leaf(s, x), _leaf(s, g)
    ref = xr * torch.rsqrt((xr * xr).mean(-1, keepdim=True) + 1e-6) * gr
    _check(s, s.tensor_rms_norm(xi, gi, eps=1e-6), ref, [(xi, xr), (gi, gr)])

    for op, fn in (("softmax", lambda t: torch.softmax(t, -1)), ("gelu", TF.gelu),
                   ("gelu_tanh", lambda t: TF.gelu(t, approximate="tanh"))):
        s = _session("hardened")
        xr = x.to(torch.bfloat16).float().cuda().requires_grad_(True)
        xi = _leaf(s, x)
        _check(s, getattr(s, "tensor_" + op)(xi), fn(xr), [(xi, xr)])
        assert "kernel=ftk::" in _dispatch_lines(s)[0], _dispatch_lines(s)[0]

    s = _session("hardened")
    y = torch.randn(64, 128)
    xr, yr = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (x, y))
    xi, yi = _leaf(s, x), _leaf(s, y)
    _check(s, s.tensor_add(xi, yi), xr + yr, [(xi, xr), (yi, yr)])

    s = _session("hardened")
    table = torch.randn(50, 64)
    ids = torch.randint(0, 50, (4, 16))
    tr = table.to(torch.bfloat16).float().cuda().requires_grad_(True)
    ti = _leaf(s, table)
    idn = s.tensor_variable_from_storage(ids.cuda(), False)
    _check(s, s.tensor_embedding(ti, idn), tr[ids.cuda()], [(ti, tr)])
    assert "ftk::embedding_fwd_kernel" in _dispatch_lines(s)[0]

    for causal in (True, False):
        s = _session("hardened")
        q, k, v = (torch.randn(2, 3, 128, 64) * 0.5 for _ in range(3))
        qr, kr, vr = (t.to(torch.bfloat16).float().cuda().requires_grad_(True) for t in (q, k, v))
        qi, ki, vi = _leaf(s, q), _leaf(s, k), _leaf(s, v)
        out = s.tensor_sdpa(qi, ki, vi, is_causal=causal)
        _check(s, out, TF.scaled_dot_product_attention(qr, kr, vr, is_causal=causal), [(qi, qr), (ki, kr), (vi, vr)])
        assert "ftk::attn_fwd2_kernel<hd=64>" in _dispatch_lines(s)[0]

    s = _session("hardened")
    logits = torch.randn(64, 512)
    tg = torch.randint(0, 512, (64,))
    lr = logits.to(torch.bfloat16).float().cuda().requires_grad_(True)
    li = _leaf(s, logits)
    tgi = s.tensor_variable_from_storage(tg.cuda(), False)
    loss = s.tensor_cross_entropy(li, tgi)
    ref = TF.cross_entropy(lr, tg.cuda())
    assert abs(s.tensor_item(loss) - float(ref)) < 2e-2
    rep = s.tensor_backward(loss)
    gref, = torch.autograd.grad(ref, [lr])
    assert _rel(rep.gradient(li), gref) < 3e-2
    assert "ftk::cross_entropy_kernel" in _dispatch_lines(s)[0]

    s = _session("hardened")
    xi = _leaf(s, torch.ones(64, 128))
    d1 = s.functional_dropout(xi, p=0.25, training=True)
    vals = s.tensor(d1).float()
    keep = float((vals > 0).float().mean())
    assert 0.65 < keep < 0.85 and abs(float(vals.max()) - 1 / 0.75) < 1e-2
    rep = s.tensor_backward(s.tensor_sum(d1))
    assert torch.equal(rep.gradient(xi).float() > 0, vals > 0)          # the backward regenerates the same mask
    assert "ftk::dropout_kernel" in _dispatch_lines(s)[0]
    K.check_status()
    assert K.launch_count() - n0 >= 25          # every operator above launched this package's kernels


def test_operator_without_kernel_strict_refuses_hardened_records_fallback(cuda_device):
    from frankentorch_b200.dispatch import sm100
    x = torch.randn(8, 16)
    s = _session("strict")
    xi = _leaf(s, x)
    with pytest.raises(sm100.NoKernelForBackend):
        s.tensor_sigmoid(xi)
    # operands that do not qualify (fp32) are refused the same way
    xf = s.tensor_variable_from_storage(x.cuda(), True)
    with pytest.raises(sm100.NoKernelForBackend):
        s.tensor_gelu(xf)
    # layout operators are not arithmetic: allowed, and recorded as such
    r = s.tensor_reshape(xi, shape=(16, 8))
    assert s.tensor_shape(r) == [16, 8] and "kernel=layout::reshape" in _dispatch_lines(s)[-1]

    h = _session("hardened")
    hi = _leaf(h, x)
    out = h.tensor_sigmoid(hi)
    assert _rel(h.tensor(out), torch.sigmoid(x.to(torch.bfloat16).float())) < 1e-2
    line = _dispatch_lines(h)[-1]
    assert "kernel=torch::sigmoid" in line and "fallback_path=true" in line and sm100.DEVIATION_ID in line
    ids = {d["id"] for d in sm100.load_allowlist()["deviations"]}
    assert sm100.DEVIATION_ID in ids and "dispatch.composite_backend_fallback" in ids


def test_typed_dispatch_families_on_the_gpu_name_the_launched_kernel(cuda_device):
    """``dispatch_tensor_*`` with CUDA operands goes through the sm_100a route table: routed operators report the
    kernel that ran, strict mode refuses an operator without one, hardened mode records the library fallback."""
    from frankentorch_b200.dispatch import families as F, sm100
    from frankentorch_b200.dispatch.keys import DispatchKey
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.runtime.ledger import ExecutionMode as M
    x = torch.randn(64, 128).to(torch.bfloat16).cuda()
    n0 = K.launch_count()
    out = F.dispatch_tensor_unary(F.UnaryOp.Gelu, M.Strict, x, requires_grad=True)
    assert _rel(out.values, torch.nn.functional.gelu(x.float())) < 2e-2
    d = out.decision
    assert d.kernel.startswith("ftk::") and d.backend_key is DispatchKey.SM100 and d.selected_key is DispatchKey.AutogradSM100
    assert not d.fallback_used and out.storage.dtype.value == "BF16" and out.storage.data.is_cuda
    mm = F.dispatch_tensor_binary(F.BinaryOp.MatMul, M.Strict, x, x.t().contiguous())
    assert "gemm" in mm.decision.kernel and _rel(mm.values, x.float() @ x.float().t()) < 2e-2
    sm = F.dispatch_tensor_normalize_dim(F.NormalizeOp.Softmax, M.Strict, x, 1)
    assert sm.decision.kernel.startswith("ftk::") and sm.decision.dim == 1 and _rel(sm.values, torch.softmax(x.float(), 1)) < 2e-2
    j = F.dispatch_tensor_join(F.JoinOp.Cat, M.Strict, [x, x], 0)
    assert j.decision.kernel == "layout::cat" and tuple(j.values.shape) == (128, 128)
    assert K.launch_count() - n0 >= 3
    with pytest.raises(sm100.NoKernelForBackend):
        F.dispatch_tensor_unary(F.UnaryOp.Sigmoid, M.Strict, x)
    h = F.dispatch_tensor_unary(F.UnaryOp.Sigmoid, M.Hardened, x)
    assert h.decision.kernel == "torch::sigmoid" and h.decision.fallback_used
    assert _rel(h.values, torch.sigmoid(x.float())) < 1e-2
    K.check_status()


def test_gpt_from_nn_modules_on_a_cuda_session_follows_the_fused_model(cuda_device):
    """A 2-layer GPT composed of ``ft.nn`` modules on a CUDA session against ``models/gpt.py`` with the
    same weights.  The two routes cut the computation into kernels at different places (the model
    fuses bias + GELU and the residual adds into GEMM epilogues and the loss into the LM head, the
    modules run them as separate kernels), so bf16 rounding happens at different points: losses and
    gradients agree to bf16 accuracy, not bit for bit.  Every hot operator of the module route must
    have run an ``ftk::`` kernel."""
    from frankentorch_b200 import nn
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.ops import kernels as K
    cfg = GPTConfig.preset("gpt-tiny")
    B, S, d, H = 2, 128, cfg.d_model, cfg.n_head
    tape = TensorTape(grad_dtype=None)
    tape.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
    ref = GPT(cfg, tape, device=cuda_device, seed=11)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).cuda()
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    loss_ref = ref.forward(ids, tgt)
    ref.reset_grads()
    tape.backward(loss_ref)
    P = lambda n: ref.arena.view(ref.arena.params, n)
    G = lambda n: ref.arena.view(ref.arena.grads, n)

    s = _session("strict")
    n0 = K.launch_count()

    def load(module_param, name, rows=None):
        t = P(name)
        s.tensor(module_param).copy_(t if rows is None else t[:rows])
    Vp = cfg.padded_vocab
    wte, wpe = nn.Embedding(s, Vp, d), nn.Embedding(s, cfg.max_seq, d)
    W = lambda mod: mod._parameters["weight"]
    load(W(wte), "wte.weight"), load(W(wpe), "wpe.weight")
    blocks = []
    for l in range(cfg.n_layer):
        p = f"blocks.{l}."
        m = dict(ln1=nn.LayerNorm(s, d), qkv=nn.Linear(s, d, 3 * d), proj=nn.Linear(s, d, d),
                 ln2=nn.LayerNorm(s, d), fc1=nn.Linear(s, d, cfg.d_ff), fc2=nn.Linear(s, cfg.d_ff, d))
        for mod, nm in ((m["ln1"], "ln1"), (m["qkv"], "attn.qkv_proj"), (m["proj"], "attn.out_proj"),
                        (m["ln2"], "ln2"), (m["fc1"], "mlp.fc1"), (m["fc2"], "mlp.fc2")):
            load(mod._parameters["weight"], p + nm + ".weight"), load(mod._parameters["bias"], p + nm + ".bias")
        blocks.append(m)
    ln_f = nn.LayerNorm(s, d)
    load(ln_f._parameters["weight"], "ln_f.weight"), load(ln_f._parameters["bias"], "ln_f.bias")

    idn = s.tensor_variable_from_storage(ids, False)
    pos = s.tensor_variable_from_storage(torch.arange(S, device="cuda").repeat(B, 1), False)
    x = s.tensor_add(wte.forward(s, idn), wpe.forward(s, pos))
    for m in blocks:
        h = m["ln1"].forward(s, x)
        qkv = m["qkv"].forward(s, h)                                           # [B, S, 3d]
        parts = []
        for i in range(3):
            t = s.tensor_narrow(qkv, dim=2, start=i * d, length=d)
            t = s.tensor_reshape(t, shape=(B, S, H, d // H))
            parts.append(s.tensor_contiguous(s.tensor_permute(t, dims=(0, 2, 1, 3))))   # [B, H, S, hd]
        a = s.tensor_sdpa(parts[0], parts[1], parts[2], is_causal=True)
        a = s.tensor_reshape(s.tensor_contiguous(s.tensor_permute(a, dims=(0, 2, 1, 3))), shape=(B, S, d))
        x = s.tensor_add(x, m["proj"].forward(s, a))
        h = m["ln2"].forward(s, x)
        x = s.tensor_add(x, m["fc2"].forward(s, s.tensor_gelu_tanh(m["fc1"].forward(s, h))))
    h = ln_f.forward(s, x)
    logits = s.tensor_linear(s.tensor_reshape(h, shape=(B * S, d)), W(wte))
    # the padded vocabulary columns are masked out of the loss by the fused model; slice them off here
    logits = s.tensor_contiguous(s.tensor_narrow(logits, dim=1, start=0, length=cfg.vocab_size))
    loss = s.tensor_cross_entropy(logits, s.tensor_variable_from_storage(tgt.reshape(-1), False))
    rep = s.tensor_backward(loss)
    K.check_status()
    assert abs(s.tensor_item(loss) - float(tape.value(loss_ref))) < 2e-2
    for mod_param, name in ((blocks[0]["qkv"].weight, "blocks.0.attn.qkv_proj.weight"),
                            (blocks[1]["fc2"].weight, "blocks.1.mlp.fc2.weight"),
                            (blocks[1]["ln2"]._parameters["weight"], "blocks.1.ln2.weight"),
                            (blocks[0]["fc1"].bias, "blocks.0.mlp.fc1.bias"),
                            (W(wpe), "wpe.weight")):
        got = rep.gradient(mod_param)
        assert got is not None and _rel(got.reshape(G(name).shape), G(name)) < 6e-2, (name, _rel(got.reshape(G(name).shape), G(name)))
    from frankentorch_b200.dispatch import sm100
    lines = _dispatch_lines(s)
    hot = [ln for ln in lines if any(f"op={op} " in ln for op in sm100.HOT_OPS)]
    assert len(hot) >= 2 + cfg.n_layer * 10 + 3
    assert all("kernel=ftk::" in ln and "fallback_path=false" in ln for ln in hot), [ln for ln in hot if "ftk::" not in ln][:3]
    assert all(("kernel=ftk::" in ln) or ("kernel=layout::" in ln) for ln in lines)
    assert K.launch_count() - n0 >= len(hot)           # at least one launcher call of this package per hot operator


@pytest.mark.gpu
def test_fused_session_operators_match_fp32_references():
    import math
    from frankentorch_b200.ops.fused_session import FusedSession, sgemm
    torch.manual_seed(0)
    fs = FusedSession("cuda:0")
    S, D, F, H = 256, 512, 1024, 8
    x, w, b = torch.randn(S, D), torch.randn(D, F) * 0.05, torch.randn(F) * 0.1
    xd, bd = fs.upload(x), fs.upload(b)
    xr, wr, br = xd.float().cpu(), w.bfloat16().float(), bd.float().cpu()
    y1 = fs.download(fs.matmul_bias(xd, fs.upload(w), bd))
    y2 = fs.download(fs.matmul_bias_w16(xd, fs.weight(w), bd))
    ref = xr @ wr + br
    assert torch.allclose(y1, ref, atol=0.05, rtol=0.02) and torch.equal(y1, y2)
    y3 = fs.download(fs.matmul_bias_w16(xd, fs.weight(w), bd, gelu=True))
    assert torch.allclose(y3, torch.nn.functional.gelu(ref, approximate="tanh"), atol=0.05, rtol=0.02)
    g, be = fs.upload(torch.rand(D) + 0.5), fs.upload(torch.randn(D) * 0.1)
    ln = fs.download(fs.layernorm(xd, g, be))
    assert torch.allclose(ln, torch.nn.functional.layer_norm(xr, (D,), g.float().cpu(), be.float().cpu()), atol=0.03, rtol=0.02)
    assert torch.allclose(fs.download(fs.gelu(xd)), torch.nn.functional.gelu(xr, approximate="tanh"), atol=0.02, rtol=0.02)
    assert torch.allclose(fs.download(fs.add(xd, xd)), 2 * xr, atol=0.02, rtol=0.01)
    assert torch.allclose(fs.download(fs.softmax(xd)), torch.softmax(xr, -1), atol=2e-3, rtol=0.02)
    q, k, v = (fs.upload(torch.randn(S, D)) for _ in range(3))
    o = fs.download(fs.mha(q, k, v, H))
    heads = lambda t: t.float().cpu().view(S, H, D // H).transpose(0, 1)     # noqa: E731
    want = torch.softmax(heads(q) @ heads(k).transpose(1, 2) / math.sqrt(D // H), -1) @ heads(v)
    assert torch.allclose(o, want.transpose(0, 1).reshape(S, D), atol=0.03, rtol=0.03)
    fs.finish()
    a, bb = torch.randn(128, 256), torch.randn(256, 128)
    c = sgemm(a.reshape(-1).tolist(), bb, 128, 256, 128)
    assert c.dtype == torch.float32 and torch.allclose(c, a.bfloat16().float() @ bb.bfloat16().float(), atol=0.05, rtol=0.02)
