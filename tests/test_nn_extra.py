"""Lazy convolutions, fractional max pooling, max unpooling, adaptive softmax (CPU)."""
import pytest
import torch

import frankentorch_b200.nn as nn
from frankentorch_b200.session import FrankenTorchSession


def _var(s, t, rg=False):
    return s.tensor_variable(t.reshape(-1).tolist(), list(t.shape), rg)


def _val(s, nid):
    return s.tensor(nid).detach().to(torch.float64)


def test_lazy_modules_register_their_parameters_once():
    s = FrankenTorchSession()
    x = _var(s, torch.randn(2, 3, 8, 8, dtype=torch.float64))
    m = nn.LazyConv2d(s, 4, 3, padding=1)
    y = m.forward(s, x)
    assert s.tensor_shape(y) == [2, 4, 8, 8]
    assert [n for n, _ in nn.named_parameters(m)] == ["weight", "bias"]
    assert s.tensor_shape(m._parameters["weight"]) == [4, 3, 3, 3]
    ref = torch.nn.functional.conv2d(_val(s, x), _val(s, m._parameters["weight"]), _val(s, m._parameters["bias"]), padding=1)
    assert torch.allclose(_val(s, y), ref, atol=1e-12)
    lin = nn.LazyLinear(s, 5)
    lin.forward(s, _var(s, torch.ones(2, 3, dtype=torch.float64)))
    assert [n for n, _ in nn.named_parameters(lin)] == ["weight", "bias"]
    assert sorted(lin.state_dict(s)) == ["bias", "weight"]


def test_max_unpool_inverts_max_pool_positions():
    s = FrankenTorchSession()
    x = torch.arange(32, dtype=torch.float64).reshape(1, 2, 4, 4)
    xn = _var(s, x, True)
    pooled, idx = nn.MaxPool2dWithIndices(2).forward(s, xn)
    ref_p, ref_i = torch.nn.functional.max_pool2d(x, 2, return_indices=True)
    assert torch.equal(_val(s, pooled), ref_p) and torch.equal(_val(s, idx), ref_i.double())
    up = nn.MaxUnpool2d(2).forward(s, pooled, idx)
    assert torch.equal(_val(s, up), torch.nn.functional.max_unpool2d(ref_p, ref_i, 2))
    rep = s.tensor_backward(s.tensor_sum(up))
    g = torch.tensor(s.tensor_gradient(rep, xn), dtype=torch.float64).reshape(1, 2, 4, 4)
    assert g.sum() == 8 and g[0, 0, 1, 1] == 1 and g[0, 0, 0, 0] == 0


def test_fractional_max_pool_module_is_seeded():
    x = torch.arange(2 * 36, dtype=torch.float64).reshape(1, 2, 6, 6)
    outs = []
    for _ in range(2):
        s = FrankenTorchSession()
        m = nn.FractionalMaxPool2d(2, output_size=(3, 3))
        outs.append(s.tensor_values(m.forward(s, _var(s, x))))
    assert outs[0] == outs[1] and len(outs[0]) == 18
    s = FrankenTorchSession()
    m = nn.FractionalMaxPool2d(2, output_ratio=(0.5, 0.5))
    m.eval()
    assert s.tensor_shape(m.forward(s, _var(s, x))) == [1, 2, 3, 3]
    with pytest.raises(ValueError):
        nn.FractionalMaxPool2d(2)


def test_adaptive_log_softmax_is_a_distribution_and_trains():
    s = FrankenTorchSession()
    torch.manual_seed(0)
    m = nn.AdaptiveLogSoftmaxWithLoss(s, 16, 20, [4, 10], div_value=2.0)
    x = _var(s, torch.randn(6, 16, dtype=torch.float64), True)
    tgt = _var(s, torch.tensor([0., 3., 4., 9., 10., 19.]))
    lp = _val(s, m.log_prob(s, x))
    assert lp.shape == (6, 20)
    assert torch.allclose(lp.exp().sum(1), torch.ones(6, dtype=torch.float64), atol=1e-12)
    out, loss = m.forward(s, x, tgt)
    want = lp.gather(1, torch.tensor([[0], [3], [4], [9], [10], [19]]))[:, 0]
    assert torch.allclose(_val(s, out), want, atol=1e-12)
    assert float(_val(s, loss)) == pytest.approx(float(-want.mean()))
    names = [n for n, _ in nn.named_parameters(m)]
    assert names == ["head.weight", "tail.0.0.weight", "tail.0.1.weight", "tail.1.0.weight", "tail.1.1.weight"]
    assert s.tensor_shape(m.tail[0][0]._parameters["weight"]) == [8, 16] and s.tensor_shape(m.tail[1][1]._parameters["weight"]) == [10, 4]
    rep = s.tensor_backward(loss)
    assert all(s.tensor_gradient(rep, p) is not None for _, p in nn.named_parameters(m))
    assert len(s.tensor_values(m.predict(s, x))) == 6
    with pytest.raises(ValueError):
        nn.AdaptiveLogSoftmaxWithLoss(s, 16, 20, [10, 4])
