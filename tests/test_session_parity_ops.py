"""Operators of the session that the reference's per-operator benches and probes call (ft-api/benches/ops_bench.rs,
special_bench.rs, ft-api/examples/*_h2h.rs): presence of every name, forward values against PyTorch, and every
closed-form backward rule against central differences of the forward (f64)."""
import math

import pytest
import torch

from frankentorch_b200.session import FrankenTorchSession

T = lambda *v, shape=None: torch.tensor(v, dtype=torch.float64).reshape(shape or [len(v)])   # noqa: E731


def _run(call, vals, weights=None):
    s = FrankenTorchSession(ledger_dispatch=False)
    ids = [s.tensor_variable(v.reshape(-1).tolist(), list(v.shape), rg) for v, rg in vals]
    out = call(s, ids)
    y = s.tensor(out)
    if weights is None:
        g = torch.Generator().manual_seed(7)
        weights = torch.rand(y.shape, generator=g, dtype=torch.float64) + 0.5
    w = s.tensor_variable(weights.reshape(-1).tolist(), list(y.shape))
    loss = s.tensor_sum(s.tensor_mul(out, w))
    return s, ids, out, loss, weights


def check_grad(call, vals, eps=1e-6, tol=2e-6):
    """Tape gradient of ``sum(w * call(inputs))`` vs central differences for every input with requires_grad."""
    s, ids, out, loss, w = _run(call, vals)
    rep = s.tensor_backward(loss)
    for k, (v, rg) in enumerate(vals):
        if not rg:
            continue
        g = rep.gradient(ids[k])
        assert g is not None, f"input {k} received no gradient"
        g = g.reshape(-1)
        for j in range(v.numel()):
            def f(delta):
                vv = [(x.clone(), r) for x, r in vals]
                vv[k][0].reshape(-1)[j] += delta
                s2, _, _, l2, _ = _run(call, vv, w)
                return s2.tensor_item(l2)
            fd = (f(eps) - f(-eps)) / (2 * eps)
            assert abs(fd - g[j].item()) <= tol * max(1.0, abs(fd)), (k, j, fd, g[j].item())


X = T(0.3, -1.2, 0.7, 1.5, 0.2, -0.4, shape=[2, 3])
P = T(0.3, 1.2, 0.7, 1.5, 0.25, 2.4, shape=[2, 3])          # positive
U = T(0.3, 0.12, 0.7, 0.55, 0.25, 0.84, shape=[2, 3])       # inside (0, 1)
Y = T(0.9, 0.4, -0.6, 1.1, -0.3, 0.8, shape=[2, 3])
IDX3 = T(2, 0, 1)

UNARY = [("acosh", P + 1.0), ("asinh", X), ("atanh", U), ("exp2", X), ("exp10", X), ("cbrt", P), ("deg2rad", X), ("rad2deg", X),
         ("absolute", X), ("entr", P), ("sinc", X), ("erfc", X), ("erfinv", U), ("erfcx", X), ("digamma", P), ("lgamma", P),
         ("gammaln", P), ("ndtr", X), ("log_ndtr", X), ("ndtri", U), ("special_ndtr", X), ("special_log_ndtr", X),
         ("special_ndtri", U), ("i0", X), ("i0e", X), ("i1", X), ("i1e", X), ("special_i0e", X), ("special_i1", X),
         ("special_i1e", X), ("special_bessel_j0", X), ("special_bessel_j1", X), ("special_bessel_y0", P),
         ("special_bessel_y1", P), ("special_modified_bessel_i0", X), ("special_modified_bessel_i1", X),
         ("special_modified_bessel_k0", P), ("special_modified_bessel_k1", P), ("special_scaled_modified_bessel_k0", P),
         ("special_scaled_modified_bessel_k1", P), ("special_spherical_bessel_j0", X), ("fliplr", X), ("flipud", X),
         ("matrix_transpose", X), ("ravel", X), ("squeeze_all", X), ("atleast_1d", X), ("atleast_3d", X), ("msort", X),
         ("nansum", X), ("nanmean", X), ("nanmedian", X), ("nanprod", X), ("nanmax", X), ("nanmin", X), ("inverse", T(2, 0.3, -0.4, 1.5, shape=[2, 2])),
         ("det", T(2, 0.3, -0.4, 1.5, shape=[2, 2])), ("logdet", T(2, 0.3, -0.4, 1.5, shape=[2, 2]))]


@pytest.mark.parametrize("name,x", UNARY, ids=[u[0] for u in UNARY])
def test_unary_rules_match_central_differences(name, x):
    check_grad(lambda s, i: getattr(s, "tensor_" + name)(i[0]), [(x, True)])


def test_unary_limits_at_zero():
    z = T(0.0, 0.5)
    for name, want in (("sinc", 0.0), ("i1", 0.5), ("special_bessel_j1", 0.5), ("special_spherical_bessel_j0", 0.0)):
        s = FrankenTorchSession(ledger_dispatch=False)
        x = s.tensor_variable(z.tolist(), [2], True)
        rep = s.tensor_backward(s.tensor_sum(getattr(s, "tensor_" + name)(x)))
        assert abs(rep.gradient(x)[0].item() - want) < 1e-12, name


BINARY = [("maximum", X, Y), ("minimum", X, Y), ("fmax", X, Y), ("fmin", X, Y), ("hypot", X, Y), ("logaddexp", X, Y),
          ("logaddexp2", X, Y), ("xlogy", X, P), ("xlog1py", X, P), ("copysign", X, Y), ("rel_entr", P, U), ("ldexp", X, Y),
          ("vdot", X.reshape(-1), Y.reshape(-1)), ("true_divide", X, P)]


@pytest.mark.parametrize("name,a,b", BINARY, ids=[b[0] for b in BINARY])
def test_binary_rules_match_central_differences(name, a, b):
    check_grad(lambda s, i: getattr(s, "tensor_" + name)(i[0], i[1]), [(a, True), (b, True)])


def test_binary_rules_broadcast_and_partial_derivatives():
    check_grad(lambda s, i: s.tensor_hypot(i[0], i[1]), [(X, True), (T(0.5, -0.7, 1.1), True)])
    check_grad(lambda s, i: s.tensor_zeta(i[0], i[1]), [(P + 1.5, False), (P, True)])
    check_grad(lambda s, i: s.tensor_igamma(i[0], i[1]), [(P, False), (P + 0.3, True)])
    check_grad(lambda s, i: s.tensor_igammac(i[0], i[1]), [(P, False), (P + 0.3, True)])
    check_grad(lambda s, i: s.tensor_special_gammainc(i[0], i[1]), [(P, False), (P + 0.3, True)])
    check_grad(lambda s, i: s.tensor_polar(i[0], i[1]), [(P, True), (X, True)])
    check_grad(lambda s, i: s.tensor_dist(i[0], i[1], 2.0), [(X, True), (Y, True)])
    check_grad(lambda s, i: s.tensor_dist(i[0], i[1], 3.0), [(X, True), (Y, True)])
    check_grad(lambda s, i: s.tensor_dist(i[0], i[1], 1.0), [(X, True), (Y, True)])


def test_fmax_sends_the_gradient_to_the_operand_that_is_a_number():
    s = FrankenTorchSession(ledger_dispatch=False)
    a = s.tensor_variable([float("nan"), 1.0, 2.0], [3], True)
    b = s.tensor_variable([0.5, float("nan"), 2.0], [3], True)
    rep = s.tensor_backward(s.tensor_sum(s.tensor_fmax(a, b)))
    assert rep.gradient(a).tolist() == [0.0, 1.0, 0.5] and rep.gradient(b).tolist() == [1.0, 0.0, 0.5]


PARAM = [
    ("logit", lambda s, i: s.tensor_logit(i[0], None), [(U, True)]),
    ("logit_eps", lambda s, i: s.tensor_logit(i[0], 0.2), [(U, True)]),
    ("nan_to_num", lambda s, i: s.tensor_nan_to_num(i[0], 0.0, None, None), [(X, True)]),
    ("clamp_min", lambda s, i: s.tensor_clamp_min(i[0], 0.25), [(X, True)]),
    ("clamp_max", lambda s, i: s.tensor_clamp_max(i[0], 0.25), [(X, True)]),
    ("clamp_tensor", lambda s, i: s.tensor_clamp_tensor(i[0], i[1], i[2]), [(X, True), (Y - 1.0, True), (Y + 0.1, True)]),
    ("float_power", lambda s, i: s.tensor_float_power(i[0], 2.5), [(P, True)]),
    ("polygamma", lambda s, i: s.tensor_polygamma(2, i[0]), [(P, True)]),
    ("mvlgamma", lambda s, i: s.tensor_mvlgamma(i[0], 3), [(P + 1.5, True)]),
    ("multigammaln", lambda s, i: s.tensor_multigammaln(i[0], 2), [(P + 1.5, True)]),
    ("cheb_t", lambda s, i: s.tensor_special_chebyshev_polynomial_t(i[0], 5), [(U, True)]),
    ("hermite_h", lambda s, i: s.tensor_special_hermite_polynomial_h(i[0], 5), [(U, True)]),
    ("hermite_he", lambda s, i: s.tensor_special_hermite_polynomial_he(i[0], 5), [(U, True)]),
    ("laguerre", lambda s, i: s.tensor_special_laguerre_polynomial_l(i[0], 5), [(U, True)]),
    ("legendre", lambda s, i: s.tensor_special_legendre_polynomial_p(i[0], 6), [(U, True)]),
    ("addcmul", lambda s, i: s.tensor_addcmul(i[0], i[1], i[2], 0.5), [(X, True), (Y, True), (P, True)]),
    ("addcdiv", lambda s, i: s.tensor_addcdiv(i[0], i[1], i[2], 0.7), [(X, True), (Y, True), (P, True)]),
    ("addr", lambda s, i: s.tensor_addr(i[0], i[1], i[2], 0.5, 2.0), [(X, True), (T(0.4, -0.9), True), (T(1.0, 0.2, -0.3), True)]),
    ("lerp_weighted", lambda s, i: s.tensor_lerp_weighted(i[0], i[1], i[2]), [(X, True), (Y, True), (U, True)]),
    ("renorm", lambda s, i: s.tensor_renorm(i[0], 2.0, 0, 1.0), [(X, True)]),
    ("renorm_p3", lambda s, i: s.tensor_renorm(i[0], 3.0, 1, 0.9), [(X, True)]),
    ("normalize", lambda s, i: s.tensor_normalize(i[0], 2.0, 1, 1e-12), [(X, True)]),
    ("amax_dim", lambda s, i: s.tensor_amax(i[0], 1), [(X, True)]),
    ("amin_all", lambda s, i: s.tensor_amin(i[0]), [(X, True)]),
    ("nanvar", lambda s, i: s.tensor_nanvar(i[0], 1), [(X, True)]),
    ("nanstd", lambda s, i: s.tensor_nanstd(i[0], 1), [(X, True)]),
    ("nanmean_dim", lambda s, i: s._apply("nanmean", [i[0]], dim=1), [(X, True)]),
    ("kthvalue", lambda s, i: s.tensor_kthvalue(i[0], 2)[0], [(X, True)]),
    ("quantile_dim", lambda s, i: s.tensor_quantile_dim(i[0], 0.4, 1, False, "linear"), [(X, True)]),
    ("quantile_multi", lambda s, i: s.tensor_quantile_multi(i[0], [0.25, 0.8], "linear"), [(X, True)]),
    ("quantile_dim_multi", lambda s, i: s.tensor_quantile_dim_multi(i[0], [0.25, 0.8], 0, True, "midpoint"), [(X, True)]),
    ("nanquantile", lambda s, i: s.tensor_nanquantile(i[0], 0.3), [(X, True)]),
    ("logcumsumexp", lambda s, i: s.tensor_logcumsumexp(i[0], 1), [(X, True)]),
    ("diff", lambda s, i: s.tensor_diff(i[0], 1), [(X, True)]),
    ("diff_full", lambda s, i: s.tensor_diff_full(i[0], 2, 1, i[1], i[2]), [(X, True), (Y[:, :1], True), (Y[:, 1:], True)]),
    ("diff_prepend", lambda s, i: s.tensor_diff_full(i[0], 1, 0, i[1], None), [(X, True), (Y[:1], True)]),
    ("trapezoid", lambda s, i: s.tensor_trapezoid(i[0], None, 1), [(X, True)]),
    ("trapezoid_x", lambda s, i: s.tensor_trapezoid(i[0], i[1], 1), [(X, True), (T(0.0, 0.4, 1.5), True)]),
    ("trapezoid_xfull", lambda s, i: s.tensor_trapezoid(i[0], i[1], 0), [(X, True), (P.cumsum(0), True)]),
    ("cumtrap", lambda s, i: s.tensor_cumulative_trapezoid(i[0], None, 1), [(X, True)]),
    ("cumtrap_x", lambda s, i: s.tensor_cumulative_trapezoid(i[0], i[1], 1), [(X, True), (T(0.0, 0.4, 1.5), True)]),
    ("gradient_eo1", lambda s, i: s.tensor_gradient_dim(i[0], 1, 0.5, 1), [(X, True)]),
    ("gradient_eo2", lambda s, i: s.tensor_gradient_dim(i[0], 0, 0.5, 2), [(torch.cat([X, Y, P]), True)]),
    ("select", lambda s, i: s.tensor_select(i[0], 1, 2), [(X, True)]),
    ("select_scatter", lambda s, i: s.tensor_select_scatter(i[0], i[1], 0, 1), [(X, True), (T(1.0, 2.0, 3.0), True)]),
    ("slice_scatter", lambda s, i: s.tensor_slice_scatter(i[0], i[1], 1, 0, 3, 2), [(X, True), (Y[:, :2], True)]),
    ("diagonal_scatter", lambda s, i: s.tensor_diagonal_scatter(i[0], i[1], 1), [(X, True), (T(5.0, 6.0), True)]),
    ("diag_1d", lambda s, i: s.tensor_diag(i[0], 1), [(T(1.0, 2.0, 3.0), True)]),
    ("diag_2d", lambda s, i: s.tensor_diag(i[0], 0), [(X, True)]),
    ("diag_embed", lambda s, i: s.tensor_diag_embed(i[0], 1), [(X, True)]),
    ("diagflat", lambda s, i: s.tensor_diagflat(i[0], 0), [(X, True)]),
    ("rot90", lambda s, i: s.tensor_rot90(i[0], 1, [0, 1]), [(X, True)]),
    ("repeat_interleave", lambda s, i: s.tensor_repeat_interleave(i[0], 3), [(X, True)]),
    ("repeat_interleave_dim", lambda s, i: s.tensor_repeat_interleave(i[0], 2, 1), [(X, True)]),
    ("repeat_interleave_tensor", lambda s, i: s.tensor_repeat_interleave_tensor(i[0], [1, 0, 2], 1), [(X, True)]),
    ("repeat_interleave_repeats", lambda s, i: s.tensor_repeat_interleave_repeats(i[0], i[1], 0), [(X, True), (T(2, 1), False)]),
    ("take", lambda s, i: s.tensor_take(i[0], i[1]), [(X, True), (T(5, 0, 0, 3), False)]),
    ("take_along_dim", lambda s, i: s.tensor_take_along_dim(i[0], i[1], 1), [(X, True), (T(2, 0, 1, 1, shape=[2, 2]), False)]),
    ("put", lambda s, i: s.tensor_put(i[0], i[1], i[2]), [(X, True), (T(4, 1), False), (T(9.0, 8.0), True)]),
    ("index_add", lambda s, i: s.tensor_index_add(i[0], 1, i[1], i[2]), [(X, True), (T(2, 0), False), (Y[:, :2], True)]),
    ("index_copy", lambda s, i: s.tensor_index_copy(i[0], 1, i[1], i[2]), [(X, True), (T(2, 0), False), (Y[:, :2], True)]),
    ("index_fill", lambda s, i: s.tensor_index_fill(i[0], 1, i[1], -3.0), [(X, True), (T(2, 0), False)]),
    ("masked_scatter", lambda s, i: s.tensor_masked_scatter(i[0], i[1], i[2]), [(X, True), (T(1, 0, 1, 0, 0, 1, shape=[2, 3]), False), (Y, True)]),
    ("block_diag", lambda s, i: s.tensor_block_diag([i[0], i[1]]), [(X, True), (T(1.0, 2.0), True)]),
    ("cartesian_prod", lambda s, i: s.tensor_cartesian_prod([i[0], i[1]]), [(T(1.0, 2.0, 3.0), True), (T(4.0, 5.0), True)]),
    ("column_stack", lambda s, i: s.tensor_column_stack([i[0], i[1]]), [(T(1.0, 2.0), True), (X[:, :2], True)]),
    ("combinations", lambda s, i: s.tensor_combinations(i[0], 2, False), [(T(1.0, 2.0, 3.0, 4.0), True)]),
    ("vander", lambda s, i: s.tensor_vander(i[0], 4, True), [(T(0.5, -1.5, 2.0), True)]),
    ("vander_dec", lambda s, i: s.tensor_vander(i[0], None, False), [(T(0.5, -1.5, 2.0), True)]),
    ("cholesky_inverse", lambda s, i: s.tensor_cholesky_inverse(i[0], False), [(T(1.5, 0.0, 0.4, 0.9, shape=[2, 2]), True)]),
    ("cross_entropy_full", lambda s, i: s.tensor_cross_entropy_full(i[0], i[1], i[2], 1, "mean"), [(X, True), (T(2, 1), False), (T(0.5, 1.0, 2.0), False)]),
    ("cross_entropy_smooth", lambda s, i: s.tensor_cross_entropy_full(i[0], i[1], None, None, "sum", 0.1), [(X, True), (T(2, 0), False)]),
    ("cross_entropy_smooth_w", lambda s, i: s.tensor_cross_entropy_full(i[0], i[1], i[2], None, "mean", 0.2), [(X, True), (T(2, 0), False), (T(0.5, 1.0, 2.0), False)]),
    ("nll_loss_full", lambda s, i: s.tensor_nll_loss_full(i[0], i[1], i[2], None, "mean"), [(X, True), (T(2, 1), False), (T(0.5, 1.0, 2.0), False)]),
    ("bce_pos_weight", lambda s, i: s.tensor_bce_with_logits_pos_weight(i[0], i[1], 2.5, "mean"), [(X, True), (U, True)]),
    ("binary_cross_entropy", lambda s, i: s.tensor_binary_cross_entropy(i[0], i[1], "none"), [(U, True), (U.flip(0), False)]),
    ("rfft2", lambda s, i: s.tensor_rfft2(i[0]), [(torch.cat([X, Y], 1), True)]),
    ("rfftn_odd", lambda s, i: s.tensor_rfftn(i[0], None, None), [(X, True)]),
    ("rfftn_ortho", lambda s, i: s.tensor_rfftn(i[0], None, [1], "ortho"), [(X, True)]),
    ("irfft2", lambda s, i: s.tensor_irfft2(i[0], None), [(torch.stack([X, Y], -1), True)]),
    ("sdpa_gqa", lambda s, i: s.tensor_scaled_dot_product_attention_gqa(i[0], i[1], i[2], None, False, None, True),
     [(torch.arange(32, dtype=torch.float64).reshape(1, 4, 2, 4).sin(), True), (torch.arange(16, dtype=torch.float64).reshape(1, 2, 2, 4).cos(), True),
      (torch.arange(16, dtype=torch.float64).reshape(1, 2, 2, 4).sin() * 0.5, True)]),
    ("lu_solve", lambda s, i: s.tensor_lu_solve(*s.tensor_lu_factor(i[0]), i[1]), [(T(2, 0.3, -0.4, 1.5, shape=[2, 2]), False), (T(1.0, 2.0, shape=[2, 1]), True)]),
    ("meshgrid", lambda s, i: s.tensor_add(*s.tensor_meshgrid([i[0], i[1]])), [(T(1.0, 2.0, 3.0), True), (T(4.0, 5.0), True)]),
    ("var_mean", lambda s, i: s.tensor_add(*s.tensor_var_mean(i[0], 1, 1)), [(X, True)]),
    ("std_mean", lambda s, i: s.tensor_add(*s.tensor_std_mean(i[0], 1, 1)), [(X, True)]),
    ("aminmax", lambda s, i: s.tensor_sub(*s.tensor_aminmax(i[0], 1)), [(X, True)]),
]


@pytest.mark.parametrize("name,call,vals", PARAM, ids=[p[0] for p in PARAM])
def test_parametrised_rules_match_central_differences(name, call, vals):
    check_grad(call, vals)


@pytest.mark.parametrize("mode", ["sum", "mean", "prod", "amax", "amin"])
@pytest.mark.parametrize("include_self", [True, False])
def test_scatter_and_index_reduce_rules(mode, include_self):
    idx = T(0, 2, 0, 1, 1, 0, shape=[2, 3])
    check_grad(lambda s, i: s.tensor_scatter_reduce(i[0], 1, i[1], i[2], mode, include_self), [(P, True), (idx, False), (P.flip(1) + 0.1, True)])
    if mode != "sum":
        src = torch.cat([Y.abs() + 0.2, P], 0)
        check_grad(lambda s, i: s.tensor_index_reduce(i[0], 0, i[1], i[2], mode, include_self), [(P, True), (T(1, 0, 1, 1), False), (src, True)])


def test_amax_ties_share_the_gradient_evenly():
    s = FrankenTorchSession(ledger_dispatch=False)
    x = s.tensor_variable([1.0, 3.0, 3.0, 2.0], [4], True)
    rep = s.tensor_backward(s.tensor_amax(x))
    assert rep.gradient(x).tolist() == [0.0, 0.5, 0.5, 0.0]


def test_forward_values_agree_with_pytorch():
    s = FrankenTorchSession(ledger_dispatch=False)
    v = lambda t: s.tensor_variable(t.reshape(-1).tolist(), list(t.shape))   # noqa: E731
    val = lambda i: s.tensor(i)                                               # noqa: E731
    x, y, p = v(X), v(Y), v(P)
    checks = [
        (s.tensor_heaviside(x, y), torch.heaviside(X, Y)), (s.tensor_floor_divide(x, p), torch.floor_divide(X, P)),
        (s.tensor_nextafter(x, y), torch.nextafter(X, Y)), (s.tensor_signbit(x), torch.signbit(X)),
        (s.tensor_logical_not(x), torch.logical_not(X)), (s.tensor_logical_and(x, y), torch.logical_and(X, Y)),
        (s.tensor_isinf(x), torch.isinf(X)), (s.tensor_isposinf(x), torch.isposinf(X)), (s.tensor_isneginf(x), torch.isneginf(X)),
        (s.tensor_count_nonzero(x), torch.count_nonzero(X)), (s.tensor_isclose(x, x, 1e-5, 1e-8, False), torch.isclose(X, X)),
        (s.tensor_gcd(v(T(12, 18)), v(T(8, 27))), T(4, 9)), (s.tensor_lcm(v(T(4, 6)), v(T(6, 15))), T(12, 30)),
        (s.tensor_bitwise_and(v(T(12, 10)), v(T(10, 6))), T(8, 2)), (s.tensor_bitwise_not(v(T(0, 5))), T(-1, -6)),
        (s.tensor_fix(x), torch.trunc(X)), (s.tensor_sgn(x), torch.sgn(X)), (s.tensor_angle(x), torch.angle(X)),
        (s.tensor_round_decimals(x, 1), torch.round(X, decimals=1)), (s.tensor_special_airy_ai(x), torch.special.airy_ai(X)),
        (s.tensor_where_scalar(v(T(1, 0, 1)), 2.0, -1.0), T(2.0, -1.0, 2.0)), (s.tensor_isin(x, v(T(0.3, 0.2))), torch.isin(X, T(0.3, 0.2))),
        (s.tensor_one_hot(v(T(0, 2, 1)), 4), torch.nn.functional.one_hot(torch.tensor([0, 2, 1]), 4)),
        (s.tensor_swapaxes(x, 0, 1), X.t()), (s.tensor_swapdims(x, 0, 1), X.t()), (s.tensor_broadcast_to(v(T(1.0, 2.0, 3.0)), [2, 3]), T(1.0, 2.0, 3.0).expand(2, 3)),
        (s.tensor_view_as(x, v(torch.zeros(3, 2, dtype=torch.float64))), X.reshape(3, 2)), (s.tensor_roll_dims(x, [1, 2], [0, 1]), torch.roll(X, (1, 2), (0, 1))),
        (s.tensor_cummax_dim(x, 1), torch.cummax(X, 1).values), (s.tensor_cummin_dim(x, 1), torch.cummin(X, 1).values),
        (s.tensor_cholesky(v(T(2, 0.5, 0.5, 1.5, shape=[2, 2])), True), torch.linalg.cholesky(T(2, 0.5, 0.5, 1.5, shape=[2, 2]), upper=True)),
        (s.tensor_matrix_power(v(T(2, 0.5, 0.5, 1.5, shape=[2, 2])), 3), torch.linalg.matrix_power(T(2, 0.5, 0.5, 1.5, shape=[2, 2]), 3)),
        (s.tensor_pinv(x), torch.linalg.pinv(X)), (s.tensor_matrix_exp(v(T(0.2, 0.5, 0.5, 0.1, shape=[2, 2]))), torch.linalg.matrix_exp(T(0.2, 0.5, 0.5, 0.1, shape=[2, 2]))),
        (s.tensor_eigvalsh(v(T(2, 0.5, 0.5, 1.5, shape=[2, 2]))), torch.linalg.eigvalsh(T(2, 0.5, 0.5, 1.5, shape=[2, 2]))),
        (s.tensor_fft_norm(v(T(1.0, 2.0, 0.5, -1.0)), None, "ortho"), torch.view_as_real(torch.fft.fft(T(1.0, 2.0, 0.5, -1.0), norm="ortho"))),
        (s.tensor_fft_fftfreq(4, 0.5), torch.fft.fftfreq(4, 0.5, dtype=torch.float64)), (s.tensor_fft_rfftfreq(4, 0.5), torch.fft.rfftfreq(4, 0.5, dtype=torch.float64)),
        (s.tensor_polar(p, x), torch.view_as_real(torch.polar(P, X))), (s.tensor_rel_entr(p, p), torch.zeros_like(P)),
        (s.tensor_entr(p), torch.special.entr(P)), (s.tensor_cbrt(x), torch.sign(X) * X.abs().pow(1 / 3)),
    ]
    for got, want in checks:
        g = val(got)
        assert tuple(g.shape) == tuple(want.shape), (g.shape, want.shape)
        assert torch.allclose(g.to(torch.float64), want.to(torch.float64), atol=1e-12, equal_nan=True)
    parts = s.tensor_split_with_sizes(x, [1, 2], 1)
    assert [tuple(val(q).shape) for q in parts] == [(2, 1), (2, 2)]
    assert len(s.tensor_unsafe_chunk(x, 3, 1)) == 3
    hist, edges = s.tensor_histogram(x, 4, 0.0, 0.0, None, False)
    ref = torch.histogram(X.reshape(-1), 4)
    assert torch.equal(val(hist), ref.hist) and torch.allclose(val(edges), ref.bin_edges)
    hd, ed = s.tensor_histogramdd(v(torch.cat([X, Y]).reshape(6, 2)), [2, 3], None, False)
    assert tuple(val(hd).shape) == (2, 3) and len(ed) == 2 and val(hd).sum() == 6
    u, inv, cnt = s.tensor_unique_consecutive(v(T(1, 1, 2, 3, 3, 1)), False, True)
    assert val(u).tolist() == [1, 2, 3, 1] and inv is None and val(cnt).tolist() == [2, 1, 2, 1]
    q, r = s.tensor_qr(x, True)
    assert torch.allclose(val(q) @ val(r), X)
    qc, rc = s.tensor_qr(v(X.t().contiguous()), False)
    assert tuple(val(qc).shape) == (3, 3) and torch.allclose(val(qc) @ val(rc), X.t())
    w, vec = s.tensor_eigh(v(T(2, 0.5, 0.5, 1.5, shape=[2, 2])))
    assert torch.allclose(val(vec) @ torch.diag(val(w)) @ val(vec).t(), T(2, 0.5, 0.5, 1.5, shape=[2, 2]))
    a = T(2, 0.3, -0.4, 1.5, shape=[2, 2])
    b = T(1.0, 2.0, shape=[2, 1])
    lu, piv = s.tensor_lu_factor(v(a))
    assert torch.allclose(a @ val(s.tensor_lu_solve(lu, piv, v(b))), b)
    assert torch.allclose(a @ val(s.tensor_solve(v(a), v(b))), b)
    assert torch.allclose(val(s.tensor_triangular_solve(v(torch.triu(a)), v(b), True)), torch.linalg.solve_triangular(torch.triu(a), b, upper=True))
    assert torch.allclose(val(s.tensor_multi_dot([v(a), v(a), v(b)])), a @ a @ b)
    assert torch.allclose(val(s.tensor_linalg_pinv_hermitian(v(a + a.t()))), torch.linalg.pinv(a + a.t()))
    assert torch.allclose(val(s.tensor_ormqr(v(a), v(T(1.2, 0.0)), v(a), True, False)), torch.ormqr(a, T(1.2, 0.0), a, True, False))


def test_inplace_variants_bump_the_version_and_write_through():
    s = FrankenTorchSession(ledger_dispatch=False)
    v = lambda t: s.tensor_variable(t.reshape(-1).tolist(), list(t.shape))   # noqa: E731
    cases = [("tensor_maximum_", torch.maximum), ("tensor_hypot_", torch.hypot), ("tensor_fmod_", torch.fmod),
             ("tensor_remainder_", torch.remainder), ("tensor_copysign_", torch.copysign), ("tensor_atan2_", torch.atan2),
             ("tensor_heaviside_", torch.heaviside), ("tensor_xlogy_", torch.xlogy)]
    for name, ref in cases:
        a, b = v(X), v(P)
        before = s.tensor_version(a)
        assert getattr(s, name)(a, b) == a and s.tensor_version(a) == before + 1
        assert torch.allclose(s.tensor(a), ref(X, P)), name
    a = v(X)
    s.tensor_where_(a, v(T(1, 0, 1, 0, 1, 0, shape=[2, 3])), v(Y))
    assert torch.equal(s.tensor(a), torch.where(T(1, 0, 1, 0, 1, 0, shape=[2, 3]).bool(), X, Y))
    a = v(X)
    s.tensor_masked_fill_(a, v(T(1, 0, 0, 0, 0, 1, shape=[2, 3])), -7.0)
    assert s.tensor(a)[0, 0] == -7.0 and s.tensor(a)[1, 2] == -7.0 and s.tensor(a)[0, 1] == X[0, 1]
    a = v(X)
    s.tensor_addcmul_(a, v(Y), v(P), 2.0)
    assert torch.allclose(s.tensor(a), X + 2.0 * Y * P)
    a = v(X)
    s.tensor_lerp_(a, v(Y), 0.25)
    assert torch.allclose(s.tensor(a), torch.lerp(X, Y, 0.25))
    a = v(X)
    s.tensor_sigmoid_(a)
    assert torch.allclose(s.tensor(a), torch.sigmoid(X))
    a = v(P + 1)
    s.tensor_acosh_(a)
    assert torch.allclose(s.tensor(a), torch.acosh(P + 1))
    a = v(X)
    s.tensor_ones_(a)
    assert torch.equal(s.tensor(a), torch.ones_like(X))
    leaf = s.tensor_variable([1.0, 2.0], [2], True)
    with pytest.raises(RuntimeError):
        s.tensor_hypot_(leaf, leaf)


def test_samplers_follow_the_session_stream_and_their_distributions():
    def draw(name, *args):
        s = FrankenTorchSession(ledger_dispatch=False)
        s.manual_seed(1234)
        return s.tensor(getattr(s, name)(*args, [20000], False))
    n = 20000
    tol = 6.0 / math.sqrt(n)
    assert abs(draw("tensor_normal", 1.0, 2.0).mean().item() - 1.0) < 2 * tol and abs(draw("tensor_normal", 1.0, 2.0).std().item() - 2.0) < 2 * tol
    assert abs(draw("tensor_exponential", 1.5).mean().item() - 1 / 1.5) < tol
    assert abs(draw("tensor_gamma", 2.5, 1.0).mean().item() - 2.5) < 2.5 * tol and abs(draw("tensor_gamma", 2.5, 1.0).var().item() - 2.5) < 0.2
    assert abs(draw("tensor_gamma", 0.5, 2.0).mean().item() - 0.25) < tol
    assert abs(draw("tensor_chi2", 4.0).mean().item() - 4.0) < 4 * tol
    assert abs(draw("tensor_beta", 2.0, 3.0).mean().item() - 0.4) < tol
    assert abs(draw("tensor_studentt", 5.0).mean().item()) < 2 * tol
    assert abs(draw("tensor_weibull", 1.0, 1.5).mean().item() - math.gamma(1 + 1 / 1.5)) < tol
    assert abs(draw("tensor_half_normal", 1.0).mean().item() - math.sqrt(2 / math.pi)) < tol
    assert abs(draw("tensor_log_normal", 0.0, 0.5).mean().item() - math.exp(0.125)) < tol
    assert abs(draw("tensor_cauchy", 0.0, 1.0).median().item()) < 3 * tol
    assert abs(draw("tensor_binomial", 20, 0.3).mean().item() - 6.0) < 3 * tol
    s = FrankenTorchSession(ledger_dispatch=False)
    d = s.tensor(s.tensor_dirichlet([1.5, 2.0, 0.7, 1.0], [5000], False))
    assert tuple(d.shape) == (5000, 4) and torch.allclose(d.sum(-1), torch.ones(5000, dtype=d.dtype))
    assert torch.allclose(d.mean(0), torch.tensor([1.5, 2.0, 0.7, 1.0], dtype=d.dtype) / 5.2, atol=0.03)
    # same seed, same draws; the in-place forms write through and bump the version
    a, b = draw("tensor_exponential", 1.5), draw("tensor_exponential", 1.5)
    assert torch.equal(a, b)
    t = s.zeros([4000])
    v0 = s.tensor_version(t)
    s.tensor_geometric_(t, 0.3)
    assert s.tensor_version(t) == v0 + 1 and s.tensor(t).min() >= 1 and abs(s.tensor(t).mean().item() - 1 / 0.3) < 0.2
    s.tensor_exponential_(t, 2.0)
    assert abs(s.tensor(t).mean().item() - 0.5) < 0.05
    s.tensor_cauchy_(t, 0.0, 1.0)
    s.tensor_log_normal_(t, 0.0, 0.25)
    assert (s.tensor(t) > 0).all()
    assert s.tensor_shape(s.tensor_randn([3, 2], False)) == [3, 2] and s.tensor_shape(s.tensor_rand([2], False)) == [2]
    assert s.tensor(s.tensor_zeros([3], False)).tolist() == [0.0, 0.0, 0.0] and s.tensor(s.tensor_1d([1.0, 2.0], False)).tolist() == [1.0, 2.0]
    assert s.tensor_shape(s.tensor_poisson(s.full([5], 3.0))) == [5]


@pytest.mark.parametrize("kind", ["rnn", "lstm", "gru"])
@pytest.mark.parametrize("bidirectional", [False, True])
def test_raw_recurrent_forwards_match_the_pytorch_modules(kind, bidirectional):
    torch.manual_seed(0)
    I, H, L, Tn, B = 3, 4, 2, 5, 2
    mod = {"rnn": torch.nn.RNN, "lstm": torch.nn.LSTM, "gru": torch.nn.GRU}[kind](I, H, L, bidirectional=bidirectional).double()
    x = torch.randn(Tn, B, I, dtype=torch.float64)
    s = FrankenTorchSession(ledger_dispatch=False)
    v = lambda t: s.tensor_variable(t.detach().reshape(-1).tolist(), list(t.shape))   # noqa: E731
    weights = []
    for l in range(L):
        for suffix in ([""] + (["_reverse"] if bidirectional else [])):
            weights.append(tuple(v(getattr(mod, f"{n}_l{l}{suffix}")) for n in ("weight_ih", "weight_hh", "bias_ih", "bias_hh")))
    with torch.no_grad():
        ref_out, ref_state = mod(x)
    if kind == "rnn":
        out, hn = s.tensor_rnn(v(x), None, weights, bidirectional, False, "tanh")
    elif kind == "gru":
        out, hn = s.tensor_gru(v(x), None, weights, bidirectional, False)
    else:
        out, (hn, cn) = s.tensor_lstm(v(x), None, weights, bidirectional, False)
        assert torch.allclose(s.tensor(cn), ref_state[1], atol=1e-12)
        ref_state = ref_state[0]
    assert torch.allclose(s.tensor(out), ref_out, atol=1e-12) and torch.allclose(s.tensor(hn), ref_state, atol=1e-12)
    assert not s.tensor_requires_grad(out)
    # batch-first input gives the transposed output
    outb = (s.tensor_rnn(v(x.transpose(0, 1).contiguous()), None, weights, bidirectional, True, "tanh") if kind == "rnn" else
            getattr(s, "tensor_" + kind)(v(x.transpose(0, 1).contiguous()), None, weights, bidirectional, True))[0]
    assert torch.allclose(s.tensor(outb), ref_out.transpose(0, 1), atol=1e-12)


def test_register_hook_alias_and_gradients_iter():
    s = FrankenTorchSession(ledger_dispatch=False)
    x = s.tensor_variable([1.0, 2.0], [2], True)
    y = s.tensor_mul(x, x)
    seen = []
    s.tensor_register_hook(y, lambda g: seen.append(g.clone()) or None)
    rep = s.tensor_backward(s.tensor_sum(y))
    assert len(seen) == 1 and seen[0].tolist() == [1.0, 1.0]
    got = dict(s.tensor_gradients_iter(rep))
    assert got[x] == [2.0, 4.0]


REFERENCE_NAMES = """
tensor_randn tensor_logit tensor_logaddexp tensor_amax tensor_xlogy tensor_logaddexp2 tensor_clamp_min tensor_rand tensor_nan_to_num
tensor_matrix_exp tensor_erfinv tensor_digamma tensor_cholesky tensor_xlog1py tensor_polygamma tensor_nextafter tensor_matrix_power
tensor_kthvalue tensor_inverse tensor_acosh tensor_triangular_solve tensor_special_ndtr tensor_special_log_ndtr tensor_maximum
tensor_heaviside tensor_exp2 tensor_entr tensor_diag tensor_cross_entropy_full tensor_copysign tensor_cholesky_solve tensor_angle
tensor_special_ndtri tensor_special_i1 tensor_repeat_interleave tensor_nanmedian tensor_hypot tensor_gradient_dim tensor_fmax tensor_dist
tensor_diff tensor_diag_embed tensor_count_nonzero tensor_combinations tensor_block_diag tensor_asinh tensor_amin tensor_vander tensor_sinc
tensor_select tensor_rot90 tensor_renorm tensor_nanmean tensor_minimum tensor_lgamma tensor_ldexp tensor_index_add tensor_deg2rad
tensor_cartesian_prod tensor_addcmul tensor_zeta tensor_round_decimals tensor_rfft2 tensor_repeat_interleave_repeats tensor_rad2deg
tensor_normalize tensor_ndtri tensor_ndtr tensor_nansum tensor_nanmin tensor_nanmax tensor_multigammaln tensor_lu_solve tensor_logdet
tensor_logcumsumexp tensor_index_fill tensor_index_copy tensor_igamma tensor_histogramdd tensor_histogram tensor_gcd tensor_floor_divide
tensor_diff_full tensor_diagonal_scatter tensor_det tensor_cummax_dim tensor_clamp_tensor tensor_cbrt tensor_split_with_sizes
tensor_special_spherical_bessel_j0 tensor_special_i1e tensor_special_i0e tensor_special_airy_ai tensor_rel_entr tensor_quantile_dim
tensor_polar tensor_pinv tensor_meshgrid tensor_maximum_ tensor_matrix_transpose tensor_masked_fill_ tensor_lu_factor tensor_logical_not
tensor_linalg_pinv_hermitian tensor_isin tensor_igammac tensor_i1 tensor_i0 tensor_float_power tensor_erfcx tensor_erfc tensor_diagflat
tensor_cummin_dim tensor_clamp_max tensor_cholesky_inverse tensor_addr tensor_addcmul_ tensor_addcdiv tensor_xlogy_ tensor_where_scalar
tensor_where_ tensor_vdot tensor_unique_consecutive tensor_take_along_dim tensor_take tensor_special_scaled_modified_bessel_k0
tensor_special_modified_bessel_k0 tensor_special_laguerre_polynomial_l tensor_special_hermite_polynomial_he
tensor_special_hermite_polynomial_h tensor_special_chebyshev_polynomial_t tensor_special_bessel_j0 tensor_slice_scatter tensor_signbit
tensor_sigmoid_ tensor_select_scatter tensor_scatter_reduce tensor_scaled_dot_product_attention_gqa tensor_repeat_interleave_tensor
tensor_remainder_ tensor_quantile_multi tensor_put tensor_ones_ tensor_one_hot tensor_nll_loss_full tensor_nanvar tensor_nanstd
tensor_nanquantile tensor_mvlgamma tensor_matrix_norm tensor_masked_scatter tensor_lstsq tensor_log_ndtr tensor_lerp_weighted tensor_lerp_
tensor_lcm tensor_isclose tensor_index_reduce tensor_hypot_ tensor_heaviside_ tensor_gammaln tensor_gamma tensor_fmod_ tensor_fmin
tensor_exponential tensor_eigvalsh tensor_copysign_ tensor_bitwise_not tensor_bitwise_and tensor_atleast_3d tensor_atleast_2d
tensor_atleast_1d tensor_atanh tensor_atan2_ tensor_aminmax tensor_zeros tensor_weibull tensor_view_as tensor_var_mean tensor_unsafe_chunk
tensor_trapezoid tensor_swapdims tensor_swapaxes tensor_studentt tensor_std_mean tensor_squeeze_all tensor_special_zeta
tensor_special_scaled_modified_bessel_k1 tensor_special_modified_bessel_k1 tensor_special_modified_bessel_i1
tensor_special_modified_bessel_i0 tensor_special_legendre_polynomial_p tensor_special_gammaincc tensor_special_gammainc
tensor_special_bessel_y1 tensor_special_bessel_y0 tensor_special_bessel_j1 tensor_solve tensor_roll_dims tensor_rnn tensor_rfftn
tensor_register_hook tensor_ravel tensor_quantile_dim_multi tensor_qr tensor_poisson tensor_ormqr tensor_normal tensor_nanprod
tensor_multi_dot tensor_msort tensor_lstm tensor_logical_and tensor_log_normal_ tensor_log_normal tensor_isposinf tensor_isneginf
tensor_isinf tensor_irfft2 tensor_i1e tensor_i0e tensor_householder_product tensor_half_normal tensor_gru tensor_gradients_iter
tensor_geometric_ tensor_flipud tensor_fliplr tensor_fix tensor_fft_rfftfreq tensor_fft_norm tensor_fft_fftfreq tensor_exponential_
tensor_exp10 tensor_eigh tensor_dirichlet tensor_cumulative_trapezoid tensor_column_stack tensor_chi2 tensor_cauchy_ tensor_cauchy
tensor_broadcast_to tensor_binomial tensor_binary_cross_entropy tensor_beta tensor_bce_with_logits_pos_weight tensor_acosh_
tensor_absolute tensor_1d
""".split()


PARITY_MATRIX_NAMES = """
tensor_cross_entropy_label_smoothing tensor_triplet_margin_loss_swap tensor_linalg_solve_triangular tensor_unflatten_dim
tensor_nanquantile_interpolation tensor_searchsorted_sorter tensor_movedim_multi tensor_flatten_dims tensor_var_dims tensor_unsqueeze_dim
tensor_searchsorted_side tensor_cross_entropy_soft tensor_quantile_interpolation tensor_linalg_inv_ex
tensor_special_shifted_chebyshev_polynomial_w tensor_special_shifted_chebyshev_polynomial_v tensor_special_shifted_chebyshev_polynomial_u
tensor_special_shifted_chebyshev_polynomial_t tensor_special_chebyshev_polynomial_w tensor_special_chebyshev_polynomial_v
tensor_special_chebyshev_polynomial_u tensor_cfloat tensor_ihfft tensor_conj tensor_any tensor_all tensor_trapezoid_dx tensor_squeeze_neg_dim
tensor_special_gammaln tensor_linalg_cholesky_ex tensor_vecdot tensor_trapz tensor_svdvals tensor_roll_flat tensor_linalg_solve_ex
tensor_linalg_lu_factor_ex tensor_irfftn_norm tensor_cumulative_trapezoid_dx tensor_linalg_tensorinv tensor_irfftn tensor_cdouble
tensor_linalg_cross tensor_ihfft_norm tensor_frobenius_norm tensor_linalg_ldl_factor tensor_std_dims tensor_rfftn_norm tensor_irfft_norm
tensor_ifftn_norm tensor_ifft2_norm tensor_fftn_norm tensor_clamp_min_tensor tensor_hfft_norm tensor_clamp_max_tensor tensor_slogdet
tensor_linalg_ldl_solve tensor_geqrf tensor_unique_dim tensor_addmm_scaled tensor_fft_along_dim
""".split()


def test_every_session_method_the_reference_benches_call_exists():
    missing = [n for n in REFERENCE_NAMES + PARITY_MATRIX_NAMES if not callable(getattr(FrankenTorchSession, n, None))]
    assert not missing, missing


# ------------------------------------------------------------------------------------ second batch
SQ = T(2, 0.3, -0.4, 1.5, shape=[2, 2])
BATCH2 = [
    ("ce_label_smoothing", lambda s, i: s.tensor_cross_entropy_label_smoothing(i[0], i[1], 0.15), [(X, True), (T(2, 0), False)]),
    ("ce_soft_mean", lambda s, i: s.tensor_cross_entropy_soft(i[0], i[1], "mean"), [(X, True), (U / U.sum(1, keepdim=True), True)]),
    ("ce_soft_none", lambda s, i: s.tensor_cross_entropy_soft(i[0], i[1], "none"), [(X, True), (U, True)]),
    ("triplet_swap", lambda s, i: s.tensor_triplet_margin_loss_swap(i[0], i[1], i[2], 1.0, 2.0, True, "mean"), [(X, True), (Y, True), (P, True)]),
    ("triplet_noswap_sum", lambda s, i: s.tensor_triplet_margin_loss_swap(i[0], i[1], i[2], 0.5, 1.0, False, "sum"), [(X, True), (Y, True), (P, True)]),
    ("var_dims", lambda s, i: s.tensor_var_dims(i[0], [0, 2], 1, False), [(torch.stack([X, Y, P]), True)]),
    ("std_dims_keep", lambda s, i: s.tensor_std_dims(i[0], [1, 2], 0, True), [(torch.stack([X, Y, P]), True)]),
    ("cheb_u", lambda s, i: s.tensor_special_chebyshev_polynomial_u(i[0], 4), [(U, True)]),
    ("cheb_v", lambda s, i: s.tensor_special_chebyshev_polynomial_v(i[0], 4), [(U, True)]),
    ("cheb_w", lambda s, i: s.tensor_special_chebyshev_polynomial_w(i[0], 3), [(U, True)]),
    ("shifted_t", lambda s, i: s.tensor_special_shifted_chebyshev_polynomial_t(i[0], 4), [(U, True)]),
    ("shifted_u", lambda s, i: s.tensor_special_shifted_chebyshev_polynomial_u(i[0], 3), [(U, True)]),
    ("shifted_v", lambda s, i: s.tensor_special_shifted_chebyshev_polynomial_v(i[0], 3), [(U, True)]),
    ("shifted_w", lambda s, i: s.tensor_special_shifted_chebyshev_polynomial_w(i[0], 4), [(U, True)]),
    ("clamp_min_tensor", lambda s, i: s.tensor_clamp_min_tensor(i[0], i[1]), [(X, True), (Y, True)]),
    ("clamp_max_tensor", lambda s, i: s.tensor_clamp_max_tensor(i[0], i[1]), [(X, True), (Y, True)]),
    ("vecdot", lambda s, i: s.tensor_vecdot(i[0], i[1], 1), [(X, True), (Y, True)]),
    ("roll_flat", lambda s, i: s.tensor_roll_flat(i[0], 2), [(X, True)]),
    ("frobenius_norm", lambda s, i: s.tensor_frobenius_norm(i[0]), [(X, True)]),
    ("tensorinv", lambda s, i: s.tensor_linalg_tensorinv(i[0], 2), [((torch.eye(4, dtype=torch.float64) * 2 + torch.arange(16, dtype=torch.float64).reshape(4, 4).sin() * 0.3).reshape(2, 2, 2, 2), True)]),
    ("irfftn", lambda s, i: s.tensor_irfftn(i[0], None, None), [(torch.stack([X, Y], -1), True)]),
    ("irfftn_ortho_odd", lambda s, i: s.tensor_irfftn_norm(i[0], [2, 5], None, "ortho"), [(torch.stack([X, Y], -1), True)]),
    ("irfft_norm", lambda s, i: s.tensor_irfft_norm(i[0], None, "forward"), [(torch.stack([X, Y], -1), True)]),
    ("ihfft", lambda s, i: s.tensor_ihfft(i[0], None, 1), [(torch.cat([X, Y], 1), True)]),
    ("ihfft_ortho", lambda s, i: s.tensor_ihfft_norm(i[0], None, "ortho", 0), [(torch.cat([X, Y, P], 0), True)]),
    ("hfft_norm", lambda s, i: s.tensor_hfft_norm(i[0], None, "ortho"), [(torch.stack([X, Y], -1), True)]),
    ("rfftn_norm", lambda s, i: s.tensor_rfftn_norm(i[0], None, None, "forward"), [(X, True)]),
    ("fftn_norm", lambda s, i: s.tensor_fftn_norm(i[0], "ortho"), [(X, True)]),
    ("fft_along_dim", lambda s, i: s.tensor_fft_along_dim(i[0], 0), [(X, True)]),
    ("trapezoid_dx", lambda s, i: s.tensor_trapezoid_dx(i[0], 0.5, 1), [(X, True)]),
    ("cumtrap_dx", lambda s, i: s.tensor_cumulative_trapezoid_dx(i[0], 0.25, 0), [(X, True)]),
    ("trapz", lambda s, i: s.tensor_trapz(i[0], i[1], 1), [(X, True), (T(0.0, 0.4, 1.5), True)]),
    ("unflatten_dim", lambda s, i: s.tensor_unflatten_dim(i[0], 1, [3, 1]), [(X, True)]),
    ("flatten_dims", lambda s, i: s.tensor_flatten_dims(i[0], 0, 1), [(X, True)]),
    ("movedim_multi", lambda s, i: s.tensor_movedim_multi(i[0], [0, 1], [1, 0]), [(X, True)]),
    ("cfloat_conj", lambda s, i: s.tensor_conj(s.tensor_cdouble(i[0])), [(X, True)]),
    ("slogdet", lambda s, i: s.tensor_slogdet(i[0])[1], [(SQ, True)]),
    ("svdvals", lambda s, i: s.tensor_svdvals(i[0]), [(X, True)]),
    ("linalg_cross", lambda s, i: s.tensor_linalg_cross(i[0], i[1]), [(X, True), (Y, True)]),
    ("solve_triangular", lambda s, i: s.tensor_linalg_solve_triangular(i[0], i[1], True), [(torch.triu(SQ), True), (T(1.0, 2.0, shape=[2, 1]), True)]),
    ("addmm_scaled", lambda s, i: s.tensor_addmm_scaled(i[0], i[1], i[2], 0.5, 2.0), [(SQ, True), (X, True), (X.t().contiguous(), True)]),
    ("inv_ex", lambda s, i: s.tensor_linalg_inv_ex(i[0])[0], [(SQ, True)]),
    ("solve_ex", lambda s, i: s.tensor_linalg_solve_ex(i[0], i[1])[0], [(SQ, True), (T(1.0, 2.0, shape=[2, 1]), True)]),
    ("cholesky_ex", lambda s, i: s.tensor_linalg_cholesky_ex(s.tensor_matmul(i[0], s.tensor_transpose(i[0], dim0=0, dim1=1)), False)[0], [(SQ, True)]),
]


@pytest.mark.parametrize("name,call,vals", BATCH2, ids=[p[0] for p in BATCH2])
def test_second_batch_rules_match_central_differences(name, call, vals):
    check_grad(call, vals)


def test_second_batch_values_and_non_differentiable_forms():
    s = FrankenTorchSession(ledger_dispatch=False)
    v = lambda t: s.tensor_variable(t.reshape(-1).tolist(), list(t.shape))   # noqa: E731
    val = lambda i: s.tensor(i)                                               # noqa: E731
    x, u = v(X), v(U)
    for name, fn in (("u", torch.special.chebyshev_polynomial_u), ("v", torch.special.chebyshev_polynomial_v), ("w", torch.special.chebyshev_polynomial_w)):
        assert torch.allclose(val(getattr(s, f"tensor_special_chebyshev_polynomial_{name}")(u, 5)), fn(U, 5))
        shifted = getattr(torch.special, f"shifted_chebyshev_polynomial_{name}")
        assert torch.allclose(val(getattr(s, f"tensor_special_shifted_chebyshev_polynomial_{name}")(u, 5)), shifted(U, 5))
    # the closed forms at the end points, where the generic formula divides by zero
    e = s.tensor_variable([1.0, -1.0], [2], True)
    rep = s.tensor_backward(s.tensor_sum(s.tensor_special_chebyshev_polynomial_u(e, 3)))
    assert rep.gradient(e).tolist() == [20.0, 20.0]                              # (+-1)^(n+1) * n(n+1)(n+2)/3
    assert val(s.tensor_any(x)).item() is True and val(s.tensor_all(v(T(1.0, 0.0)))).item() is False
    assert val(s.tensor_any(v(T(0.0, 0.0, 1.0, 0.0, shape=[2, 2])), 1)).tolist() == [False, True]
    assert val(s.tensor_searchsorted_side(v(T(1.0, 2.0, 2.0, 3.0)), v(T(2.0)), "right")).tolist() == [3.0]
    assert val(s.tensor_searchsorted_side(v(T(1.0, 2.0, 2.0, 3.0)), v(T(2.0)), "left")).tolist() == [1.0]
    assert val(s.tensor_searchsorted_sorter(v(T(3.0, 1.0, 2.0)), v(T(2.5)), v(T(1, 2, 0)))).tolist() == [2.0]
    with pytest.raises(ValueError):
        s.tensor_searchsorted_side(x, x, "middle")
    assert val(s.tensor_quantile_interpolation(x, 0.4, "nearest")).item() == torch.quantile(X, 0.4, interpolation="nearest").item()
    assert val(s.tensor_nanquantile_interpolation(v(T(1.0, float("nan"), 3.0)), 0.5, "higher")).item() == 3.0
    assert s.tensor_shape(s.tensor_unsqueeze_dim(x, 1)) == [2, 1, 3] and s.tensor_shape(s.tensor_squeeze_neg_dim(s.tensor_unsqueeze_dim(x, 2), -1)) == [2, 3]
    singular = v(T(1.0, 2.0, 2.0, 4.0, shape=[2, 2]))
    out, info = s.tensor_linalg_inv_ex(singular)
    assert out is None and info > 0
    out, info = s.tensor_linalg_cholesky_ex(v(T(1.0, 2.0, 2.0, 1.0, shape=[2, 2])))
    assert out is None and info == 2
    out, info = s.tensor_linalg_solve_ex(singular, v(T(1.0, 1.0, shape=[2, 1])))
    assert out is None and info > 0
    good, info = s.tensor_linalg_inv_ex(v(SQ))
    assert info == 0 and torch.allclose(val(good) @ SQ, torch.eye(2, dtype=torch.float64))
    lu, piv, info = s.tensor_linalg_lu_factor_ex(v(SQ))
    assert info == 0 and torch.allclose(SQ @ val(s.tensor_lu_solve(lu, piv, v(T(1.0, 2.0, shape=[2, 1])))), T(1.0, 2.0, shape=[2, 1]))
    sym = SQ + SQ.t()
    ld, lp = s.tensor_linalg_ldl_factor(v(sym))
    b = T(1.0, -2.0, shape=[2, 1])
    assert torch.allclose(sym @ val(s.tensor_linalg_ldl_solve(ld, lp, v(b))), b)
    qr, tau = s.tensor_geqrf(x)
    rq, rt = torch.geqrf(X)
    assert torch.allclose(val(qr), rq) and torch.allclose(val(tau), rt)
    uq, inv, cnt = s.tensor_unique_dim(v(T(1, 2, 1, 2, 3, 4, shape=[3, 2])), 0)
    assert val(uq).tolist() == [[1.0, 2.0], [3.0, 4.0]] and val(inv).tolist() == [0.0, 0.0, 1.0] and val(cnt).tolist() == [2.0, 1.0]
    assert tuple(val(s.tensor_cfloat(x)).shape) == (2, 3, 2) and val(s.tensor_cfloat(x)).dtype == torch.float32
    assert torch.allclose(val(s.tensor_special_gammaln(v(P))), torch.lgamma(P))
    assert torch.allclose(val(s.tensor_ihfft(x, None, 1)), torch.view_as_real(torch.fft.ihfft(X, dim=1).resolve_conj()))
    z = torch.stack([X, Y], -1)
    assert torch.allclose(val(s.tensor_irfftn(v(z), None, None)), torch.fft.irfftn(torch.view_as_complex(z.contiguous())))
    assert torch.allclose(val(s.tensor_hfft_norm(v(z), None, "forward")), torch.fft.hfft(torch.view_as_complex(z.contiguous()), norm="forward"))
    assert torch.allclose(val(s.tensor_ifft2_norm(v(z), "ortho")), torch.view_as_real(torch.fft.ifft2(torch.view_as_complex(z.contiguous()), norm="ortho")))
    assert torch.allclose(val(s.tensor_ifftn_norm(v(z), "forward")), torch.view_as_real(torch.fft.ifftn(torch.view_as_complex(z.contiguous()), norm="forward")))


# ------------------------------------------------------------------------------------ third batch
def test_metadata_splits_and_small_utilities():
    s = FrankenTorchSession(ledger_dispatch=False)
    v = lambda t, rg=False: s.tensor_variable(t.reshape(-1).tolist(), list(t.shape), rg)   # noqa: E731
    val = lambda i: s.tensor(i)                                                            # noqa: E731
    x = v(X)
    assert (s.tensor_dim(x), s.tensor_nelement(x), s.tensor_stride(x)) == (2, 6, [3, 1])
    assert s.tensor_stride(s.tensor_transpose(x, dim0=0, dim1=1)) in ([1, 3], [2, 1])       # a view or a fresh copy
    assert s.tensor_broadcast_shapes([2, 1, 3], [4, 1]) == [2, 4, 3]
    assert val(s.tensor_bool(x)).tolist() == [[1.0] * 3, [1.0] * 3] and val(s.tensor_bool(v(T(0.0, 2.0)))).tolist() == [0.0, 1.0]
    assert val(s.tensor_int_long(v(T(1.7, -2.9)))).tolist() == [1, -2] and val(s.tensor_int_long(x)).dtype == torch.int64
    parts = s.tensor_array_split(v(torch.arange(7, dtype=torch.float64)), 3)
    assert [val(p).tolist() for p in parts] == [[0.0, 1.0, 2.0], [3.0, 4.0], [5.0, 6.0]]
    nz = s.tensor_nonzero_as_tuple(v(T(0.0, 1.0, 2.0, 0.0, shape=[2, 2])))
    assert [val(t).tolist() for t in nz] == [[0.0, 1.0], [1.0, 0.0]]
    assert val(s.tensor_matrix_rank(v(T(1.0, 2.0, 2.0, 4.0, shape=[2, 2])))).item() == 1
    kv, ki = s.tensor_kthvalue_dim(x, 2, 1)
    assert val(kv).tolist() == [0.3, 0.2] and val(ki).tolist() == [0.0, 1.0]
    assert torch.equal(val(s.tensor_ger(v(T(1.0, 2.0)), v(T(3.0, 4.0, 5.0)))), torch.outer(T(1.0, 2.0), T(3.0, 4.0, 5.0)))
    assert torch.allclose(val(s.tensor_tensordot_dims(x, v(Y), [1], [1])), torch.tensordot(X, Y, dims=([1], [1])))
    assert torch.equal(val(s.tensor_fft_fftshift(x)), torch.fft.fftshift(X)) and torch.equal(val(s.tensor_fft_ifftshift(x)), torch.fft.ifftshift(X))
    assert torch.equal(val(s.tensor_scalbn(x, 3)), X * 8)
    fr, it = s.tensor_modf(x)
    assert torch.allclose(val(fr) + val(it), X) and torch.equal(val(it), torch.trunc(X))
    m, e = s.tensor_frexp(v(T(8.0, 0.3, -5.0)))
    rm, re_ = torch.frexp(T(8.0, 0.3, -5.0))
    assert torch.equal(val(m), rm) and val(e).tolist() == re_.tolist()
    # clone and frexp's mantissa stay in the graph
    check_grad(lambda s2, i: s2.tensor_clone(i[0]), [(X, True)])
    check_grad(lambda s2, i: s2.tensor_frexp(i[0])[0], [(P + 0.01, True)])       # away from the powers of two, where the mantissa jumps
    check_grad(lambda s2, i: s2.tensor_scalbn(i[0], -2), [(X, True)])


def test_lobpcg_finds_the_largest_eigenpairs():
    s = FrankenTorchSession(ledger_dispatch=False)
    g = torch.Generator().manual_seed(5)
    B = torch.randn(12, 12, generator=g, dtype=torch.float64)
    A = B @ B.t() + torch.diag(torch.arange(12, dtype=torch.float64))
    lam, V = s.tensor_lobpcg(s.tensor_variable(A.reshape(-1).tolist(), [12, 12]), 3, 500, 1e-11)
    ref = torch.linalg.eigvalsh(A).flip(0)[:3]
    assert torch.allclose(s.tensor(lam), ref, rtol=1e-8)
    Vt = s.tensor(V)
    assert torch.allclose(A @ Vt, Vt * s.tensor(lam), atol=1e-6) and torch.allclose(Vt.t() @ Vt, torch.eye(3, dtype=torch.float64), atol=1e-8)
    with pytest.raises(ValueError):
        s.tensor_lobpcg(s.tensor_variable([1.0, 2.0], [1, 2]), 1)


def test_in_place_families_match_their_out_of_place_forms():
    """Every generated ``tensor_<op>_`` writes what ``tensor_<op>`` returns, bumps the version and returns its
    argument (the reference's ``inplace_matches_out_of_place`` suite, ft-conformance/tests)."""
    unary = [("erf", X), ("erfc", X), ("logit", U), ("asin", U), ("acos", U), ("atan", X), ("sinh", X), ("cosh", X), ("tanh", X),
             ("asinh", X), ("atanh", U), ("sin", X), ("cos", X), ("tan", X), ("exp", X), ("exp2", X), ("expm1", X), ("log", P),
             ("log2", P), ("log10", P), ("log1p", P), ("sqrt", P), ("rsqrt", P), ("reciprocal", P), ("abs", X), ("sign", X),
             ("floor", X), ("ceil", X), ("round", X), ("trunc", X), ("frac", X), ("relu", X), ("relu6", X * 5), ("gelu", X), ("silu", X),
             ("mish", X), ("elu", X), ("selu", X), ("celu", X), ("leaky_relu", X), ("hardswish", X * 3), ("hardsigmoid", X * 3),
             ("hardtanh", X), ("hardshrink", X), ("softshrink", X), ("softplus", X), ("deg2rad", X), ("rad2deg", X), ("square", X),
             ("tril", X), ("triu", X), ("nan_to_num", T(float("nan"), 1.0, float("inf")))]
    for name, t in unary:
        s = FrankenTorchSession(ledger_dispatch=False)
        a = s.tensor_variable(t.reshape(-1).tolist(), list(t.shape))
        want = s.tensor(getattr(s, "tensor_" + name)(a)).clone()
        before = s.tensor_version(a)
        assert getattr(s, f"tensor_{name}_")(a) == a and s.tensor_version(a) == before + 1, name
        assert torch.equal(s.tensor(a), want.to(s.tensor(a).dtype)), name
    binary = [("logaddexp", X, Y), ("logaddexp2", X, Y), ("fmax", X, Y), ("fmin", X, Y), ("minimum", X, Y), ("ldexp", X, Y.round()),
              ("nextafter", X, Y), ("gcd", T(12.0, 18.0), T(8.0, 27.0)), ("lcm", T(4.0, 6.0), T(6.0, 15.0))]
    for name, t, u in binary:
        s = FrankenTorchSession(ledger_dispatch=False)
        a, b = s.tensor_variable(t.reshape(-1).tolist(), list(t.shape)), s.tensor_variable(u.reshape(-1).tolist(), list(u.shape))
        want = s.tensor(getattr(s, "tensor_" + name)(a, b)).clone()
        assert getattr(s, f"tensor_{name}_")(a, b) == a
        assert torch.equal(s.tensor(a), want.to(s.tensor(a).dtype)), name
    s = FrankenTorchSession(ledger_dispatch=False)
    a, b, c = (s.tensor_variable(t.reshape(-1).tolist(), [2, 3]) for t in (X, Y, P))
    s.tensor_addcdiv_(a, b, c, value=0.7)
    assert torch.allclose(s.tensor(a), torch.addcdiv(X, Y, P, value=0.7))
    p = s.tensor_variable(P.reshape(-1).tolist(), [2, 3])
    s.tensor_pow_(p, 2.0)
    assert torch.allclose(s.tensor(p), P ** 2)
    s.tensor_clamp_min_(p, 1.0)
    assert float(s.tensor(p).min()) == 1.0
    s.tensor_threshold_(p, threshold=2.0, value=-1.0)
    assert torch.equal(s.tensor(p), torch.nn.functional.threshold((P ** 2).clamp_min(1.0), 2.0, -1.0))
    z = s.zeros([4000])
    s.manual_seed(3)
    s.tensor_bernoulli_(z, 0.25)
    assert set(s.tensor(z).unique().tolist()) <= {0.0, 1.0} and abs(s.tensor(z).mean().item() - 0.25) < 0.03
    leaf = s.tensor_variable([0.5], [1], True)
    with pytest.raises(RuntimeError):
        s.tensor_erf_(leaf)


def test_third_batch_samplers():
    def draw(name, *args):
        s = FrankenTorchSession(ledger_dispatch=False)
        s.manual_seed(99)
        return s.tensor(getattr(s, name)(*args, [20000], False))
    vm = draw("tensor_von_mises", 0.5, 4.0)
    assert float(vm.min()) > -math.pi - 1e-9 and float(vm.max()) <= math.pi + 1e-9
    assert abs(torch.atan2(torch.sin(vm).mean(), torch.cos(vm).mean()).item() - 0.5) < 0.03          # circular mean
    r = torch.sqrt(torch.sin(vm).mean() ** 2 + torch.cos(vm).mean() ** 2).item()                      # = I1(k)/I0(k)
    assert abs(r - (torch.special.i1(torch.tensor(4.0)) / torch.i0(torch.tensor(4.0))).item()) < 0.02
    assert abs(draw("tensor_von_mises", 0.0, 0.0).mean().item()) < 0.06                               # uniform on the circle
    f = draw("tensor_fishersnedecor", 5.0, 8.0)
    assert abs(f.mean().item() - 8.0 / 6.0) < 0.06 and float(f.min()) > 0
    s = FrankenTorchSession(ledger_dispatch=False)
    nb = s.tensor(s.tensor_negative_binomial(5, 0.3, [4000], False))
    assert abs(nb.mean().item() - 5 * 0.3 / 0.7) < 0.12 and float(nb.min()) >= 0 and torch.equal(nb, nb.round())
