"""Session surface added on top of the rule tables: aliases, factorisations, FFT / complex layout,
quantisation, box and point-cloud utilities (CPU, f64, checked against torch)."""
import math

import pytest
import torch

from frankentorch_b200.session import FrankenTorchSession


def _s():
    return FrankenTorchSession()


def _var(s, t, rg=False):
    return s.tensor_variable(t.reshape(-1).tolist(), list(t.shape), rg)


def _val(s, nid):
    return s.tensor(nid).detach().to(torch.float64)


def test_aliases_bind_to_the_same_operator():
    s = _s()
    torch.manual_seed(0)
    a, b = torch.randn(4, 3, dtype=torch.float64), torch.randn(4, 3, dtype=torch.float64)
    x, y = _var(s, a, True), _var(s, b)
    l1, l2 = s.mse_loss(x, y), s.tensor_mse_loss(x, y)
    assert s.tensor_values(l1) == s.tensor_values(l2)
    logits, tgt = _var(s, torch.randn(5, 7, dtype=torch.float64), True), _var(s, torch.tensor([0., 3., 6., 1., 2.]))
    ce = s.functional_cross_entropy(logits, tgt, "mean")
    assert s.tensor_values(ce) == s.tensor_values(s.cross_entropy_loss(logits, tgt))
    assert s.tensor_tape.nodes[ce].rule == s.tensor_tape.nodes[s.tensor_cross_entropy(logits, tgt)].rule
    h = s.tensor_half(x)
    assert s.tensor(h).dtype == torch.float16 and s.tensor(s.tensor_double(h)).dtype == torch.float64
    assert s.tensor(s.tensor_float(x)).dtype == torch.float32


def test_svd_qr_eigh_factors_and_gradients():
    s = _s()
    torch.manual_seed(1)
    a = torch.randn(5, 3, dtype=torch.float64)
    x = _var(s, a, True)
    u, sv, vh = s.tensor_linalg_svd(x)
    rec = _val(s, u) @ torch.diag(_val(s, sv)) @ _val(s, vh)
    assert torch.allclose(rec, a, atol=1e-12)
    # gradient of sum of singular values = U Vh
    loss = s.tensor_sum(sv)
    rep = s.tensor_backward(loss)
    g = torch.tensor(s.tensor_gradient(rep, x), dtype=torch.float64).reshape(5, 3)
    assert torch.allclose(g, _val(s, u) @ _val(s, vh), atol=1e-10)
    q, r = s.tensor_linalg_qr(x)
    assert torch.allclose(_val(s, q) @ _val(s, r), a, atol=1e-12)
    sym = a.T @ a
    w, v = s.tensor_linalg_eigh(_var(s, sym))
    assert torch.allclose(_val(s, v) @ torch.diag(_val(s, w)) @ _val(s, v).T, sym, atol=1e-10)
    ev, _ = s.tensor_linalg_eig(_var(s, torch.tensor([[0., -1.], [1., 0.]], dtype=torch.float64)))
    vals = _val(s, ev)            # eigenvalues +-i in the [..., 2] layout
    assert vals.shape == (2, 2) and torch.allclose(vals[:, 0], torch.zeros(2, dtype=torch.float64), atol=1e-12)
    assert sorted(vals[:, 1].tolist()) == pytest.approx([-1.0, 1.0])
    sign, logabs = s.tensor_linalg_slogdet(_var(s, sym))
    assert float(_val(s, sign)) == 1.0 and float(_val(s, logabs)) == pytest.approx(float(torch.logdet(sym)))
    p, l, uu = s.tensor_linalg_lu(_var(s, sym))
    assert torch.allclose(_val(s, p) @ _val(s, l) @ _val(s, uu), sym, atol=1e-12)


def test_fft_family_round_trips_and_matches_torch():
    s = _s()
    torch.manual_seed(2)
    sig = torch.randn(3, 16, dtype=torch.float64)
    x = _var(s, sig, True)
    f = s.tensor_fft(x)
    assert torch.allclose(torch.view_as_complex(_val(s, f)), torch.fft.fft(sig), atol=1e-12)
    back = s.tensor_real(s.tensor_ifft(f))
    assert torch.allclose(_val(s, back), sig, atol=1e-12)
    # Parseval through the tape: d/dx sum |F|^2 = 2 N x
    e = s.tensor_sum(s.tensor_mul(s.tensor_complex_abs(f), s.tensor_complex_abs(f)))
    rep = s.tensor_backward(e)
    g = torch.tensor(s.tensor_gradient(rep, x), dtype=torch.float64).reshape(3, 16)
    assert torch.allclose(g, 2 * 16 * sig, atol=1e-9)
    rf = s.tensor_rfft(x)
    assert _val(s, rf).shape == (3, 9, 2)
    assert torch.allclose(_val(s, s.tensor_irfft(rf, 16)), sig, atol=1e-12)
    img = torch.randn(4, 6, dtype=torch.float64)
    f2 = s.tensor_fft2(_var(s, img))
    assert torch.allclose(torch.view_as_complex(_val(s, f2)), torch.fft.fft2(img), atol=1e-12)
    fn = s.tensor_fftn(_var(s, img))
    assert torch.allclose(_val(s, fn), _val(s, f2), atol=1e-12)
    assert torch.allclose(_val(s, s.tensor_real(s.tensor_ifft2(f2))), img, atol=1e-12)
    wave = torch.randn(64, dtype=torch.float64)
    win = torch.hann_window(16, periodic=True, dtype=torch.float64)
    z = s.tensor_stft(_var(s, wave), n_fft=16, hop_length=4, window=win)
    ref = torch.stft(wave, 16, 4, window=win, return_complex=True)
    assert torch.allclose(torch.view_as_complex(_val(s, z)), ref, atol=1e-12)
    inv = s.tensor_istft(z, n_fft=16, hop_length=4, window=win, length=64)
    assert torch.allclose(_val(s, inv), wave, atol=1e-10)


def test_complex_layout_helpers():
    s = _s()
    re, im = torch.tensor([1., 2.], dtype=torch.float64), torch.tensor([3., -1.], dtype=torch.float64)
    z = s.tensor_complex(_var(s, re, True), _var(s, im, True))
    assert _val(s, z).tolist() == [[1., 3.], [2., -1.]]
    assert _val(s, s.tensor_imag(z)).tolist() == [3., -1.]
    zz = s.tensor_complex_mul(z, s.tensor_complex_conj(z))
    assert torch.allclose(_val(s, zz), torch.tensor([[10., 0.], [5., 0.]], dtype=torch.float64))
    assert _val(s, s.tensor_view_as_real(s.tensor_view_as_complex(z))).shape == (2, 2)


def test_quantisation_codes_and_straight_through_gradient():
    s = _s()
    x = _var(s, torch.tensor([-2.0, -0.26, 0.0, 0.24, 0.5, 300.0], dtype=torch.float64), True)
    q = s.tensor_quantize_per_tensor(x, scale=0.5, zero_point=3, bits=8, signed=False)
    assert _val(s, q).tolist() == [0., 2., 3., 3., 4., 255.]
    dq = s.tensor_dequantize_per_tensor(q, scale=0.5, zero_point=3)
    assert _val(s, dq).tolist() == [-1.5, -0.5, 0., 0., 0.5, 126.]
    fq = s.tensor_fake_quantize_per_tensor(x, scale=0.5, zero_point=3, bits=8, signed=False)
    assert _val(s, fq).tolist() == _val(s, dq).tolist()
    rep = s.tensor_backward(s.tensor_sum(fq))
    assert s.tensor_gradient(rep, x) == [0., 1., 1., 1., 1., 0.]     # clipped ends get no gradient
    w = _var(s, torch.tensor([[1.0, -1.0], [10.0, 20.0]], dtype=torch.float64))
    sc, zp = _var(s, torch.tensor([0.5, 10.0])), _var(s, torch.tensor([0.0, 1.0]))
    qc = s.tensor_quantize_per_channel(w, sc, zp, axis=0)
    assert _val(s, qc).tolist() == [[2., -2.], [2., 3.]]
    assert _val(s, s.tensor_dequantize_per_channel(qc, sc, zp, axis=0)).tolist() == [[1., -1.], [10., 20.]]


def test_nms_keeps_best_non_overlapping_boxes_deterministically():
    s = _s()
    boxes = torch.tensor([[0, 0, 10, 10], [1, 1, 11, 11], [20, 20, 30, 30], [0, 0, 10, 10]], dtype=torch.float64)
    scores = torch.tensor([0.9, 0.8, 0.7, 0.9], dtype=torch.float64)
    keep = s.nms(_var(s, boxes), _var(s, scores), 0.5)
    assert s.tensor_values(keep) == [0.0, 2.0]        # the tie between 0 and 3 goes to the lower index
    cls = torch.tensor([0., 1., 0., 1.], dtype=torch.float64)
    keep2 = s.batched_nms(_var(s, boxes), _var(s, scores), _var(s, cls), 0.5)
    assert sorted(s.tensor_values(keep2)) == [0.0, 2.0, 3.0]
    iou = _val(s, s.tensor_box_iou(_var(s, boxes[:2]), _var(s, boxes[:2])))
    assert iou[0, 1] == pytest.approx(81.0 / 119.0)
    g = _val(s, s.tensor_generalized_box_iou(_var(s, boxes[:1]), _var(s, boxes[2:3])))
    assert float(g) == pytest.approx(0.0 - (900.0 - 200.0) / 900.0)


def test_box_losses_have_finite_difference_gradients():
    s = _s()
    p = torch.tensor([[0.1, 0.2, 2.0, 2.5], [1.0, 1.0, 3.0, 2.0]], dtype=torch.float64)
    t = torch.tensor([[0.0, 0.0, 2.0, 2.0], [1.5, 0.5, 3.5, 2.5]], dtype=torch.float64)
    for name in ("iou_loss", "giou_loss"):
        x = _var(s, p, True)
        rep = s.tensor_backward(getattr(s, name)(x, _var(s, t)))
        g = torch.tensor(s.tensor_gradient(rep, x), dtype=torch.float64).reshape(2, 4)
        h = 1e-6
        for i in range(2):
            for j in range(4):
                pp, pm = p.clone(), p.clone()
                pp[i, j] += h
                pm[i, j] -= h
                fp = float(_val(s, getattr(s, name)(_var(s, pp), _var(s, t))))
                fm = float(_val(s, getattr(s, name)(_var(s, pm), _var(s, t))))
                assert g[i, j] == pytest.approx((fp - fm) / (2 * h), abs=1e-6)


def test_roi_pool_ball_query_and_farthest_point_sampling():
    s = _s()
    feat = torch.arange(2 * 1 * 4 * 4, dtype=torch.float64).reshape(2, 1, 4, 4)
    rois = torch.tensor([[0, 0, 0, 3, 3], [1, 2, 2, 3, 3]], dtype=torch.float64)
    f = _var(s, feat, True)
    out = s.roi_pool(f, _var(s, rois), (2, 2), 1.0)
    assert _val(s, out)[0, 0].tolist() == [[5., 7.], [13., 15.]]
    assert _val(s, out)[1, 0].tolist() == [[26., 27.], [30., 31.]]
    rep = s.tensor_backward(s.tensor_sum(out))
    g = torch.tensor(s.tensor_gradient(rep, f), dtype=torch.float64).reshape(2, 1, 4, 4)
    assert g.sum() == 8 and g[0, 0, 1, 1] == 1 and g[1, 0, 3, 3] == 1
    xyz = torch.tensor([[[0., 0, 0], [1, 0, 0], [0, 2, 0], [5, 5, 5], [0.5, 0, 0]]], dtype=torch.float64)
    idx = s.ball_query(_var(s, xyz), _var(s, xyz[:, :1]), 1.1, 3)
    assert s.tensor_values(idx) == [0.0, 1.0, 4.0]
    far = s.ball_query(_var(s, xyz), _var(s, torch.tensor([[[100., 100, 100]]], dtype=torch.float64)), 1.0, 2)
    assert s.tensor_values(far) == [0.0, 0.0]
    fps = s.farthest_point_sampling(_var(s, xyz), 3)
    assert s.tensor_values(fps) == [0.0, 3.0, 2.0]


def test_functional_batch_norm_updates_running_statistics_like_torch():
    s = _s()
    torch.manual_seed(3)
    x = torch.randn(6, 3, 4, 4, dtype=torch.float64)
    w, b = torch.randn(3, dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    rm, rv = torch.zeros(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64)
    rm_t, rv_t = rm.clone(), rv.clone()
    ref = torch.nn.functional.batch_norm(x, rm_t, rv_t, w, b, True, 0.1, 1e-5)
    nrm, nrv = _var(s, rm), _var(s, rv)
    y = s.functional_batch_norm2d(_var(s, x, True), nrm, nrv, _var(s, w, True), _var(s, b, True), True, 0.1, 1e-5)
    assert torch.allclose(_val(s, y), ref, atol=1e-12)
    assert torch.allclose(_val(s, nrm), rm_t, atol=1e-12) and torch.allclose(_val(s, nrv), rv_t, atol=1e-12)
    ye = s.functional_batch_norm2d(_var(s, x), nrm, nrv, _var(s, w), _var(s, b), False)
    assert torch.allclose(_val(s, ye), torch.nn.functional.batch_norm(x, rm_t, rv_t, w, b, False), atol=1e-12)
    with pytest.raises(ValueError):
        s.functional_batch_norm3d(_var(s, x))


def test_multi_head_attention_forward_matches_torch():
    s = _s()
    torch.manual_seed(4)
    N, S, E, H = 2, 5, 8, 2
    x = torch.randn(N, S, E, dtype=torch.float64)
    ws = [torch.randn(E, E, dtype=torch.float64) * 0.3 for _ in range(4)]
    bs = [torch.randn(E, dtype=torch.float64) * 0.1 for _ in range(4)]
    xi = _var(s, x, True)
    out = s.multi_head_attention_forward(xi, xi, xi, H, *[_var(s, w, True) for w in ws],
                                         *[_var(s, b) for b in bs], is_causal=True)
    ref, _ = torch.nn.functional.multi_head_attention_forward(
        x.transpose(0, 1), x.transpose(0, 1), x.transpose(0, 1), E, H, None, torch.cat(bs[:3]), None, None, False, 0.0,
        ws[3], bs[3], use_separate_proj_weight=True, q_proj_weight=ws[0], k_proj_weight=ws[1], v_proj_weight=ws[2],
        attn_mask=torch.triu(torch.ones(S, S, dtype=torch.bool), 1), need_weights=False)
    assert torch.allclose(_val(s, out), ref.transpose(0, 1), atol=1e-10)
    rep = s.tensor_backward(s.tensor_sum(out))
    assert len(s.tensor_gradient(rep, xi)) == N * S * E


def test_fractional_max_pool_is_deterministic_with_given_samples():
    s = _s()
    x = torch.arange(36, dtype=torch.float64).reshape(1, 1, 6, 6)
    a = s.tensor_fractional_max_pool2d(_var(s, x), kernel_size=2, output_size=(3, 3))
    b = s.tensor_fractional_max_pool2d(_var(s, x), kernel_size=2, output_size=(3, 3))
    assert _val(s, a).shape == (1, 1, 3, 3) and s.tensor_values(a) == s.tensor_values(b)
