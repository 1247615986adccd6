"""Module-level parity of the nn layer with the reference: recurrent stacks (bidirectional, batch-first,
packed states), masks of the transformer stack, embedding options, builder-style constructors."""
import pytest


@pytest.mark.parametrize("kind", ["rnn", "lstm", "gru"])
@pytest.mark.parametrize("batch_first", [False, True])
def test_bidirectional_recurrent_modules_match_pytorch_values_and_gradients(kind, batch_first):
    import torch
    from frankentorch_b200 import nn
    from frankentorch_b200.session import FrankenTorchSession
    torch.manual_seed(1)
    I, H, L, T, B = 3, 4, 2, 5, 2
    ref = {"rnn": torch.nn.RNN, "lstm": torch.nn.LSTM, "gru": torch.nn.GRU}[kind](
        I, H, L, bidirectional=True, batch_first=batch_first).double()
    s = FrankenTorchSession(ledger_dispatch=False)
    mod = {"rnn": nn.RNN, "lstm": nn.LSTM, "gru": nn.GRU}[kind](s, I, H, num_layers=L, bidirectional=True,
                                                                 batch_first=batch_first)
    assert mod.is_bidirectional() and len(mod.cells) == 2 * L
    for l in range(L):
        for k, suffix in enumerate(("", "_reverse")):
            cell = mod.cells[l * 2 + k]
            assert s.tensor_shape(cell._parameters["weight_ih"])[1] == (I if l == 0 else 2 * H)
            for n in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
                s.tensor_update_values(cell._parameters[n], getattr(ref, f"{n}_l{l}{suffix}").detach().to(torch.float64))
    x = torch.randn((B, T, I) if batch_first else (T, B, I), dtype=torch.float64, requires_grad=True)
    h0 = torch.randn(2 * L, B, H, dtype=torch.float64)
    c0 = torch.randn(2 * L, B, H, dtype=torch.float64)
    xv = s.tensor_variable(x.detach().reshape(-1).tolist(), list(x.shape), requires_grad=True)
    hv = s.tensor_variable(h0.reshape(-1).tolist(), list(h0.shape))
    cv = s.tensor_variable(c0.reshape(-1).tolist(), list(c0.shape))
    if kind == "lstm":
        r_out, (r_h, r_c) = ref(x, (h0, c0))
        got = mod.forward_lstm(s, xv, hv, cv)
        assert torch.allclose(s.tensor(got.c_n).double(), r_c, atol=1e-10)
    else:
        r_out, r_h = ref(x, h0)
        got = getattr(mod, "forward_" + kind)(s, xv, hv)
    assert torch.allclose(s.tensor(got.output).double(), r_out, atol=1e-10)
    assert torch.allclose(s.tensor(got.h_n).double(), r_h, atol=1e-10)
    r_out.square().sum().backward()
    rep = s.tensor_backward(s.tensor_sum(s.tensor_mul(got.output, got.output)))
    assert torch.allclose(rep.gradient(xv).double(), x.grad, atol=1e-9)
    w = mod.cells[3]._parameters["weight_hh"]
    assert torch.allclose(rep.gradient(w).double(), ref.weight_hh_l1_reverse.grad, atol=1e-9)
    # the list form: zero states when none are given, per-cell final states in torch's order
    out2, fin = mod(s, xv)
    with torch.no_grad():
        z_out, z_state = ref(x)
    assert torch.allclose(s.tensor(out2).double(), z_out, atol=1e-10)
    hs = fin[0] if kind == "lstm" else fin
    assert len(hs) == 2 * L and torch.allclose(s.tensor(hs[3]).double(), (z_state[0] if kind == "lstm" else z_state)[3], atol=1e-10)
    # one step of a cell under the reference's name
    cell = mod.cells[0]
    step = cell.forward_cell(s, s.tensor_variable([0.1] * (B * I), [B, I]),
                             (s.zeros([B, H]), s.zeros([B, H])) if kind == "lstm" else s.zeros([B, H]))
    assert s.tensor_shape(step[0] if kind == "lstm" else step) == [B, H]


def test_recurrent_constructor_refusals():
    from frankentorch_b200 import nn
    from frankentorch_b200.session import FrankenTorchSession
    s = FrankenTorchSession(ledger_dispatch=False)
    with pytest.raises(ValueError):
        nn.LSTM(s, 3, 4, num_layers=0)
    with pytest.raises(ValueError):
        nn.GRU(s, 3, 4, dropout=1.5)
    m = nn.LSTM(s, 3, 4)
    with pytest.raises(ValueError):
        m.forward_lstm(s, s.zeros([2, 5, 3]), s.zeros([1, 2, 4]), None)
    with pytest.raises(ValueError):
        m(s, s.zeros([5, 3]))
    cfg = nn.RNNConfig(3, 4, num_layers=2, bidirectional=True).build(s, "gru")
    assert cfg.is_bidirectional() and not cfg.batch_first and len(cfg.cells) == 4


def _copy_mha(ours_sd, prefix, tm):
    import torch
    with torch.no_grad():
        tm.in_proj_weight.copy_(torch.cat([ours_sd[prefix + n + ".weight"] for n in ("q_proj", "k_proj", "v_proj")]))
        tm.in_proj_bias.copy_(torch.cat([ours_sd[prefix + n + ".bias"] for n in ("q_proj", "k_proj", "v_proj")]))
        tm.out_proj.weight.copy_(ours_sd[prefix + "out_proj.weight"])
        tm.out_proj.bias.copy_(ours_sd[prefix + "out_proj.bias"])


def _copy_layer(ours_sd, prefix, tl, decoder=False):
    import torch
    _copy_mha(ours_sd, prefix + "self_attn.", tl.self_attn)
    if decoder:
        _copy_mha(ours_sd, prefix + "multihead_attn.", tl.multihead_attn)
    with torch.no_grad():
        for n in ("linear1", "linear2", "norm1", "norm2") + (("norm3",) if decoder else ()):
            getattr(tl, n).weight.copy_(ours_sd[f"{prefix}{n}.weight"])
            getattr(tl, n).bias.copy_(ours_sd[f"{prefix}{n}.bias"])


@pytest.mark.parametrize("norm_first", [False, True])
def test_transformer_key_padding_masks_match_pytorch(norm_first):
    import torch
    from frankentorch_b200 import nn
    from frankentorch_b200.session import FrankenTorchSession
    torch.manual_seed(2)
    E, Hh, F, N, S, T = 8, 2, 16, 2, 6, 4
    s = FrankenTorchSession(ledger_dispatch=False)
    ours = nn.Transformer(s, E, Hh, 2, 2, F, dropout=0.0, norm_first=norm_first)
    ref = torch.nn.Transformer(E, Hh, 2, 2, F, dropout=0.0, norm_first=norm_first, batch_first=True, dtype=torch.float64)
    ref.eval()
    sd = ours.state_dict(s)
    for i in range(2):
        _copy_layer(sd, f"encoder.layers.{i}.", ref.encoder.layers[i])
        _copy_layer(sd, f"decoder.layers.{i}.", ref.decoder.layers[i], decoder=True)
    with torch.no_grad():
        for part in ("encoder", "decoder"):
            getattr(ref, part).norm.weight.copy_(sd[part + ".norm.weight"])
            getattr(ref, part).norm.bias.copy_(sd[part + ".norm.bias"])
    src = torch.randn(N, S, E, dtype=torch.float64)
    tgt = torch.randn(N, T, E, dtype=torch.float64)
    src_pad = torch.zeros(N, S, dtype=torch.bool); src_pad[0, 4:] = True; src_pad[1, 5:] = True     # noqa: E702
    tgt_pad = torch.zeros(N, T, dtype=torch.bool); tgt_pad[1, 3:] = True                            # noqa: E702
    causal = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    leaf = lambda t: s.tensor_tape.leaf(t, False)      # noqa: E731
    sv = s.tensor_variable(src.reshape(-1).tolist(), list(src.shape), requires_grad=True)
    tv = s.tensor_variable(tgt.reshape(-1).tolist(), list(tgt.shape))
    got = ours.forward_transformer_masked(s, sv, tv, None, leaf(causal), None, leaf(src_pad), leaf(tgt_pad), leaf(src_pad))
    with torch.no_grad():
        want = ref(src, tgt, tgt_mask=causal, src_key_padding_mask=src_pad, tgt_key_padding_mask=tgt_pad,
                   memory_key_padding_mask=src_pad)
    assert torch.allclose(s.tensor(got), want, atol=1e-9)
    # a padded source position has no influence on the output: its gradient is exactly zero
    rep = s.tensor_backward(s.tensor_sum(s.tensor_mul(got, got)))
    g = rep.gradient(sv)
    assert float(g[0, 4:].abs().sum()) == 0.0 and float(g[0, :4].abs().sum()) > 0.0

    # the parts under the reference's names
    mem = ours.encoder.forward_masked(s, sv, None, leaf(src_pad), False)
    with torch.no_grad():
        mem_ref = ref.encoder(src, src_key_padding_mask=src_pad)
    # torch's fast path returns zeros at padded rows; compare the rows that carry data
    keep = ~src_pad
    assert torch.allclose(s.tensor(mem)[keep], mem_ref[keep], atol=1e-9)
    one = ours.encoder.layers[0].forward_layer_masked(s, sv, None, leaf(src_pad), False)
    assert torch.allclose(s.tensor(one), s.tensor(ours.encoder.layers[0](s, sv, None, False, leaf(src_pad))))
    dec = ours.decoder.forward_decoder_masked(s, tv, mem, leaf(causal), None, leaf(tgt_pad), leaf(src_pad), False, False)
    assert torch.allclose(s.tensor(dec), want, atol=1e-9)
    plain = ours.forward_transformer(s, sv, tv)
    assert torch.allclose(s.tensor(plain), s.tensor(ours(s, sv, tv)))
    assert s.tensor_shape(ours.decoder.forward_decoder(s, tv, mem)) == [N, T, E]
    assert s.tensor_shape(ours.decoder.layers[0].forward_layer(s, tv, mem)) == [N, T, E]
    assert s.tensor_shape(ours.encoder.layers[0].forward_layer(s, sv)) == [N, S, E]
    d1 = ours.decoder.layers[0].forward_layer_masked(s, tv, mem, None, None, None, leaf(src_pad), True, False)
    d2 = ours.decoder.layers[0](s, tv, mem, leaf(causal), None, False, None, leaf(src_pad))
    assert torch.allclose(s.tensor(d1), s.tensor(d2), atol=1e-12)


def test_builder_constructors_and_named_forwards():
    import math
    import torch
    from frankentorch_b200 import nn
    from frankentorch_b200.session import FrankenTorchSession
    s = FrankenTorchSession(ledger_dispatch=False)
    v = lambda t: s.tensor_variable(t.reshape(-1).tolist(), list(t.shape))   # noqa: E731
    torch.manual_seed(3)
    a, b = torch.randn(4, 6, dtype=torch.float64), torch.randn(4, 6, dtype=torch.float64)

    cs = nn.CosineSimilarity().with_eps(1e-6).with_dim(1)
    assert torch.allclose(s.tensor(cs.forward_pair(s, v(a), v(b))), torch.nn.functional.cosine_similarity(a, b, 1, 1e-6))
    pd = nn.PairwiseDistance().with_p(1.0).with_eps(1e-7).with_keepdim(True)
    got = s.tensor(pd.forward_pair(s, v(a), v(b)))
    assert got.shape == (4, 1) and torch.allclose(got, torch.nn.functional.pairwise_distance(a, b, 1.0, 1e-7, True))

    y = torch.tensor([1.0, -1.0, 1.0, -1.0], dtype=torch.float64)
    assert math.isclose(float(s.tensor(nn.CosineEmbeddingLoss(margin=0.1).forward_triplet(s, v(a), v(b), v(y)))),
                        float(torch.nn.functional.cosine_embedding_loss(a, b, y, margin=0.1)), rel_tol=1e-12)
    assert math.isclose(float(s.tensor(nn.MarginRankingLoss().forward_triplet(s, v(a[:, 0]), v(b[:, 0]), v(y)))),
                        float(torch.nn.functional.margin_ranking_loss(a[:, 0], b[:, 0], y)), rel_tol=1e-12)
    assert math.isclose(float(s.tensor(nn.HingeEmbeddingLoss().forward_hinge(s, v(a[:, 0]), v(y)))),
                        float(torch.nn.functional.hinge_embedding_loss(a[:, 0], y)), rel_tol=1e-12)
    with pytest.raises(ValueError):
        nn.HingeEmbeddingLoss(margin=float("inf")).forward_hinge(s, v(a[:, 0]), v(y))
    var = torch.rand(4, 6, dtype=torch.float64) + 0.1
    assert math.isclose(float(s.tensor(nn.GaussianNLLLoss().forward_with_var(s, v(a), v(b), v(var)))),
                        float(torch.nn.functional.gaussian_nll_loss(a, b, var)), rel_tol=1e-12)

    lp = torch.randn(7, 2, 5, dtype=torch.float64).log_softmax(-1)
    tg = torch.tensor([[1, 2, 3], [2, 2, 4]], dtype=torch.float64)
    il, tl = torch.tensor([7.0, 6.0], dtype=torch.float64), torch.tensor([3.0, 2.0], dtype=torch.float64)
    ctc = nn.CTCLoss(None).with_blank(0).with_reduction(nn.CTCReduction.Sum).with_zero_infinity(True)
    want = torch.nn.functional.ctc_loss(lp, tg.long(), il.long(), tl.long(), blank=0, reduction="sum", zero_infinity=True)
    assert math.isclose(float(s.tensor(ctc.forward_ctc(s, v(lp), v(tg), v(il), v(tl)))), float(want), rel_tol=1e-10)

    bl = nn.Bilinear(s, 6, 6, 3)
    assert s.tensor_shape(bl.forward_bilinear(s, v(a), v(b))) == [4, 3]
    lrn = nn.LocalResponseNorm.with_params(3, 1e-3, 0.5, 2.0)
    x4 = torch.randn(2, 5, 4, 4, dtype=torch.float64)
    assert torch.allclose(s.tensor(lrn(s, v(x4))), torch.nn.functional.local_response_norm(x4, 3, 1e-3, 0.5, 2.0))
    with pytest.raises(ValueError):
        nn.LocalResponseNorm.with_params(0, 1e-3, 0.5, 2.0)

    # embedding with max_norm: touched rows are rescaled in place, the others keep their norm
    emb = nn.Embedding.with_options(s, 6, 4, padding_idx=0, max_norm=0.5, norm_type=2.0, sparse=False)
    before = s.tensor(emb._parameters["weight"]).clone()
    ids = s.tensor_tape.leaf(torch.tensor([1, 3, 3]), False)
    out = emb(s, ids)
    w = s.tensor(emb._parameters["weight"])
    ref = torch.nn.functional.embedding(torch.tensor([1, 3, 3]), before.clone(), padding_idx=0, max_norm=0.5)
    assert torch.allclose(s.tensor(out), ref, atol=1e-6) and float(w[1].norm()) <= 0.5 + 1e-6
    assert torch.equal(w[2], before[2]) and torch.equal(w[5], before[5])
    for bad in (dict(num_embeddings=0, embedding_dim=4), dict(num_embeddings=4, embedding_dim=4, padding_idx=4),
                dict(num_embeddings=4, embedding_dim=4, max_norm=-1.0)):
        with pytest.raises(ValueError):
            nn.Embedding.with_options(s, **bad)

    bag = nn.EmbeddingBag(s, 10, 3, mode="sum")
    idx, off = torch.tensor([1, 2, 4, 5, 4, 3, 2, 9]), torch.tensor([0, 4])
    psw = torch.rand(8, dtype=torch.float64)
    pw = s.tensor_variable(psw.tolist(), [8], requires_grad=True)
    got = bag.forward_with_offsets(s, s.tensor_tape.leaf(idx, False), s.tensor_tape.leaf(off, False), pw)
    wt = s.tensor(bag._parameters["weight"]).detach().double()
    want = torch.nn.functional.embedding_bag(idx, wt, off, mode="sum", per_sample_weights=psw)
    assert torch.allclose(s.tensor(got).double(), want, atol=1e-10)
    rep = s.tensor_backward(s.tensor_sum(got))
    assert torch.allclose(rep.gradient(pw).double(), wt[idx].sum(1), atol=1e-10)
    plain = bag.forward_with_offsets(s, s.tensor_tape.leaf(idx, False), s.tensor_tape.leaf(off, False), None)
    assert torch.allclose(s.tensor(plain).double(), torch.nn.functional.embedding_bag(idx, wt, off, mode="sum"), atol=1e-10)
    with pytest.raises(ValueError):
        nn.EmbeddingBag(s, 10, 3, mode="mean").forward_with_offsets(s, s.tensor_tape.leaf(idx, False), s.tensor_tape.leaf(off, False), pw)

    conv = nn.Conv2d.new_grouped(s, 4, 6, 3, 1, 1, True, 2)
    assert s.tensor_shape(conv._parameters["weight"]) == [6, 2, 3, 3]
    assert s.tensor_shape(nn.Conv1d.new_grouped(s, 4, 4, 3, 1, 0, False, 4)._parameters["weight"]) == [4, 1, 3]
    with pytest.raises(ValueError):
        nn.Conv2d.new_grouped(s, 4, 6, 3, 1, 1, True, 4)
    x = torch.randn(1, 2, 5, 5, dtype=torch.float64)
    assert s.tensor_shape(nn.MaxPool2d(2).ceil_mode(True)(s, v(x))) == [1, 2, 3, 3]
    assert s.tensor_shape(nn.MaxPool2d(2)(s, v(x))) == [1, 2, 2, 2]

    pooled, where = torch.nn.functional.max_pool1d(x[0], 2, return_indices=True)         # [2, 5, 2]
    un = nn.MaxUnpool1d(2).forward_with_indices(s, v(pooled), where.reshape(-1).tolist(), 5)
    assert torch.allclose(s.tensor(un), torch.nn.functional.max_unpool1d(pooled, where, 2, output_size=[5]))
    with pytest.raises(ValueError):
        nn.MaxUnpool1d(2).forward_with_indices(s, v(pooled), [0, 1], 5)
    with pytest.raises(ValueError):
        nn.MaxUnpool1d(2).forward_with_indices(s, v(pooled), [9] * pooled.numel(), 5)

    up = nn.Upsample.with_uniform_scale_factor(2.0).with_mode(nn.UpsampleMode.Bilinear).with_align_corners(False)
    assert torch.allclose(s.tensor(up(s, v(x))), torch.nn.functional.interpolate(x, scale_factor=2.0, mode="bilinear", align_corners=False))
    assert s.tensor_shape(nn.Upsample.with_size([7, 9])(s, v(x))) == [1, 2, 7, 9]
    assert s.tensor_shape(nn.Upsample.with_uniform_size(8)(s, v(x))) == [1, 2, 8, 8]
    assert s.tensor_shape(nn.Upsample.with_scale_factor([2.0, 3.0])(s, v(x))) == [1, 2, 10, 15]
    assert s.tensor_shape(nn.Upsample.from_options([6, 6], None, nn.UpsampleMode.Nearest, None)(s, v(x))) == [1, 2, 6, 6]
    for args in (([6, 6], [2.0, 2.0]), (None, None)):
        with pytest.raises(ValueError):
            nn.Upsample.from_options(*args)
        with pytest.raises(ValueError):
            nn.UpsamplingBilinear2d.from_options(*args)
    assert s.tensor_shape(nn.UpsamplingNearest2d.with_scale_factors(2, 3)(s, v(x))) == [1, 2, 10, 15]
    assert s.tensor_shape(nn.UpsamplingBilinear2d.with_size(4, 6)(s, v(x))) == [1, 2, 4, 6]
    ub = nn.UpsamplingBilinear2d.with_scale_factor(2.0)
    assert torch.allclose(s.tensor(ub(s, v(x))), torch.nn.functional.interpolate(x, scale_factor=2.0, mode="bilinear", align_corners=True))
    assert s.tensor_shape(nn.UpsamplingBilinear2d.from_options(None, [2.0, 2.0])(s, v(x))) == [1, 2, 10, 10]

    obs = nn.MinMaxObserver()
    assert obs.compute_qparams() is None and not obs.initialized
    obs.observe(torch.tensor([0.5, 2.0]))
    qp = obs.compute_qparams()
    assert obs.initialized and qp.zero_point == -128 and math.isclose(qp.scale, 2.0 / 255)
    assert nn.qint8_range() == (-128, 127) and nn.quint8_range() == (0, 255)
