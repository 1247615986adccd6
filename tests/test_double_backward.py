"""Graph-building backward (``create_graph=True``) of the CPU session: second derivatives against
``torch.autograd`` and against the goldens of the reference's double-backward parity tests
(ft-api/tests/{cholesky,inverse_logdet,logsumexp,solve,triangular_solve}_double_backward_parity.rs)."""
import pytest
import torch

from frankentorch_b200.autograd.tape import AutogradError, BackwardOptions
from frankentorch_b200.session import FrankenTorchSession


def _hessian_torch(fn, x0):
    return torch.autograd.functional.hessian(fn, x0.clone().double()).reshape(x0.numel(), x0.numel())


def _hess(build, x0):
    s = FrankenTorchSession("strict")
    x = s.tensor_variable(x0.reshape(-1).tolist(), list(x0.shape), True)
    return s, x, s.tensor_functional_hessian(build(s, x), x)


def test_logsumexp_hessians_match_reference_goldens_and_torch():
    x0 = torch.tensor([0.5, 1.0, 1.5, 2.0], dtype=torch.float64)
    _, _, H = _hess(lambda s, x: s.tensor_logsumexp(x, dim=0), x0)
    diag = [0.091227, 0.139381, 0.199826, 0.24798]          # goldens of the reference test (torch, 6 decimals)
    assert all(abs(float(H[i, i]) - d) <= 1e-6 for i, d in enumerate(diag))
    assert abs(float(H[0, 1]) + 0.016998) <= 1e-6 and abs(float(H[0, 2]) + 0.028024) <= 1e-6
    assert (H - _hessian_torch(lambda t: torch.logsumexp(t, 0), x0)).abs().max() < 1e-10
    x1 = torch.tensor([[0.5, 1.0, 1.5], [2.0, -1.0, 0.3]], dtype=torch.float64)
    _, _, H = _hess(lambda s, x: s.tensor_sum(s.tensor_logsumexp(x, dim=1)), x1)
    diag = [0.151607, 0.212827, 0.249958, 0.153044, 0.038764, 0.126255]
    assert all(abs(float(H[i, i]) - d) <= 1e-6 for i, d in enumerate(diag))
    assert abs(float(H[0, 1]) + 0.057238) <= 1e-6 and abs(float(H[0, 3])) <= 1e-12


def test_cholesky_hessian_matches_reference_golden_and_torch():
    a0 = torch.tensor([[2.0, 0.5], [0.5, 1.5]], dtype=torch.float64)
    want = torch.tensor([-0.049353, -0.032665, -0.032665, -0.009691, -0.032665, -0.116291, -0.116291, 0.038764,
                         -0.032665, -0.116291, -0.116291, 0.038764, -0.009691, 0.038764, 0.038764, -0.155055],
                        dtype=torch.float64).reshape(4, 4)
    s, x, H = _hess(lambda s, x: s.tensor_sum(s.tensor_linalg_cholesky(x)), a0)
    assert (H - want).abs().max() <= 1e-6
    assert (H - _hessian_torch(lambda t: torch.linalg.cholesky(t).sum(), a0)).abs().max() < 1e-10


@pytest.mark.parametrize("name", ["inv", "logdet", "solve", "triangular_solve"])
def test_linalg_double_backward_matches_torch(name):
    a0 = torch.tensor([[2.0, 0.5, 0.1], [0.3, 1.5, -0.2], [0.0, 0.4, 1.8]], dtype=torch.float64)
    b0 = torch.tensor([[1.0, -0.5], [0.25, 2.0], [0.7, 0.1]], dtype=torch.float64)
    if name == "inv":
        build = lambda s, x: s.tensor_sum(s.tensor_mul(s.tensor_linalg_inv(x), s.tensor_linalg_inv(x)))
        ref = lambda t: (torch.linalg.inv(t) ** 2).sum()
    elif name == "logdet":
        build = lambda s, x: s.tensor_linalg_logdet(x)
        ref = lambda t: torch.logdet(t)
    elif name == "solve":
        build = lambda s, x: s.tensor_sum(s.tensor_square(s.tensor_linalg_solve(x, s.tensor_variable(b0.reshape(-1).tolist(), [3, 2], False))))
        ref = lambda t: (torch.linalg.solve(t, b0) ** 2).sum()
    else:
        a0 = torch.tril(a0) + torch.eye(3, dtype=torch.float64)
        build = lambda s, x: s.tensor_sum(s.tensor_square(s.tensor_linalg_triangular_solve(
            x, s.tensor_variable(b0.reshape(-1).tolist(), [3, 2], False), upper=False)))
        ref = lambda t: (torch.linalg.solve_triangular(t, b0, upper=False) ** 2).sum()
    _, _, H = _hess(build, a0)
    assert (H - _hessian_torch(ref, a0)).abs().max() < 1e-10


def test_mlp_loss_hessian_and_gradient_of_gradient_norm():
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(5, 4, generator=g, dtype=torch.float64) * 0.5
    w2 = torch.randn(3, 5, generator=g, dtype=torch.float64) * 0.5
    xs = torch.randn(6, 4, generator=g, dtype=torch.float64)
    ts = torch.randn(6, 3, generator=g, dtype=torch.float64)

    def build(s, w):
        x = s.tensor_variable(xs.reshape(-1).tolist(), [6, 4], False)
        t = s.tensor_variable(ts.reshape(-1).tolist(), [6, 3], False)
        v2 = s.tensor_variable(w2.reshape(-1).tolist(), [3, 5], False)
        h = s.tensor_tanh(s.tensor_linear(x, w))
        return s.tensor_mse_loss(s.tensor_linear(h, v2), t)
    ref = lambda w: torch.nn.functional.mse_loss(torch.tanh(xs @ w.t()) @ w2.t(), ts)
    s, w, H = _hess(build, w1)
    assert (H - _hessian_torch(ref, w1)).abs().max() < 1e-10
    # gradient penalty: d/dw |dL/dw|^2 through the graph-building backward
    s = FrankenTorchSession("strict")
    w = s.tensor_variable(w1.reshape(-1).tolist(), [5, 4], True)
    loss = build(s, w)
    (gid,) = s.tensor_autograd_grad(loss, [w], create_graph=True)
    pen = s.tensor_sum(s.tensor_mul(gid, gid))
    got = s.tensor_backward(pen).gradient(w)
    wt = w1.clone().requires_grad_(True)
    (g1,) = torch.autograd.grad(ref(wt), [wt], create_graph=True)
    (want,) = torch.autograd.grad((g1 * g1).sum(), [wt])
    assert (got - want).abs().max() < 1e-10


def test_first_order_gradients_are_bitwise_the_same_with_and_without_create_graph():
    vals = [0.3, -1.2, 2.5, 0.7, -0.4, 1.1]

    def run(create):
        s = FrankenTorchSession("strict")
        x = s.tensor_variable(vals, [2, 3], True)
        y = s.tensor_sum(s.tensor_mul(s.tensor_softmax(x, dim=-1), s.tensor_sigmoid(x)))
        rep = s.tensor_backward_with_options(y, BackwardOptions(create_graph=create))
        return rep.gradient(x), rep.telemetry.execution_order
    (g0, o0), (g1, o1) = run(False), run(True)
    assert torch.equal(g0, g1) and o0 == o1


def test_custom_function_needs_a_tape_building_backward_for_create_graph():
    s = FrankenTorchSession("strict")
    x = s.tensor_variable([0.5, -1.5], [2], True)
    y = s.tensor_apply_function([x], lambda ctx, ts: ts[0] ** 3, lambda ctx, g: [g * 3 * s.tensor(x) ** 2])
    with pytest.raises(AutogradError, match="graph-building"):
        s.tensor_backward_with_options(s.tensor_sum(y), BackwardOptions(create_graph=True))

    def fwd(ctx, ts):
        return ts[0] ** 3

    def bwd(sess, ctx, gid, ins):
        xx = sess.tensor_mul(ins[0], ins[0])
        three = sess.tensor_variable([3.0, 3.0], [2], False)
        return [sess.tensor_mul(gid, sess.tensor_mul(three, xx))]
    s = FrankenTorchSession("strict")
    x = s.tensor_variable([0.5, -1.5], [2], True)
    y = s.tensor_apply_function_with_create_graph([x], fwd, bwd)
    assert torch.allclose(s.tensor_backward_with_options(s.tensor_sum(y), BackwardOptions(retain_graph=True)).gradient(x),
                          torch.tensor([0.75, 6.75], dtype=torch.float64))
    H = s.tensor_functional_hessian(s.tensor_sum(y), x)
    assert torch.allclose(H, torch.diag(torch.tensor([3.0, -9.0], dtype=torch.float64)))


def test_complex_bridge_carries_interleaved_gradients():
    """A real -> complex -> real chain through two bridge nodes (FFT of a real signal, then |z|^2): the complex
    node's gradient travels as a real [..., 2] tensor and the result equals torch.autograd's."""
    import torch

    from frankentorch_b200.session import FrankenTorchSession
    s = FrankenTorchSession("strict", ledger_dispatch=False)
    x0 = torch.randn(16, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    x = s.tensor_variable_from_storage(x0.clone(), True)
    z_val = torch.fft.fft(s.tensor(x))

    def fft_bwd(ctx, g):                          # g: [16, 2] real view of the conjugate-Wirtinger gradient
        return [torch.fft.ifft(torch.view_as_complex(g.contiguous()), norm="forward").real]
    z = s.tensor_apply_complex_bridge([x], z_val, fft_bwd)
    assert s.tensor(z).is_complex()
    w_val = (s.tensor(z).abs() ** 2)

    def abs2_bwd(ctx, g):                         # d|z|^2 -> 2 g z, as [..., 2]
        return [torch.view_as_real(2.0 * g * s.tensor(z))]
    w = s.tensor_apply_complex_bridge([z], w_val, abs2_bwd)
    loss = s.tensor_sum(w)
    rep = s.tensor_backward(loss)
    xt = x0.clone().requires_grad_(True)
    (torch.fft.fft(xt).abs() ** 2).sum().backward()
    assert torch.allclose(rep.gradient(x), xt.grad, atol=1e-10)
    # a bridge whose inputs need no gradient is a plain leaf
    c = s.tensor_variable_from_storage(x0.clone(), False)
    leaf = s.tensor_apply_complex_bridge([c], torch.fft.fft(x0), fft_bwd)
    assert not s.tensor_tape.nodes[leaf].requires_grad
    # a backward that returns a complex gradient is refused
    bad = s.tensor_apply_complex_bridge([x], z_val, lambda ctx, g: [torch.view_as_complex(g.contiguous())])
    w2 = s.tensor_apply_complex_bridge([bad], w_val, abs2_bwd)
    import pytest
    with pytest.raises(Exception, match="must be real"):
        s.tensor_backward(s.tensor_sum(w2))
