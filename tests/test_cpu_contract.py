"""CPU tests: golden conformance in both modes, the DAC acceptance checklist, ledger, dispatch."""
import pytest
import torch

from frankentorch_b200.autograd.tape import (BackwardOptions, BorrowedInputVersionMismatch, ReentrantDepthExceeded,
                                              ReentrantPolicy, TensorGraphConsumed, TensorRequiresGradNonFloating,
                                              TensorRootDoesNotRequireGrad, TensorGradientShapeMismatch)
from frankentorch_b200.conformance.runner_more import FAMILIES, run_family
from frankentorch_b200.dispatch.keys import (DispatchKey, DispatchKeyError, DispatchKeySet, dispatch_scalar_binary,
                                             resolve)
from frankentorch_b200.runtime.ledger import EvidenceKind, EvidenceLedger, ExecutionMode, RuntimeContext
from frankentorch_b200.session import FrankenTorchSession


@pytest.mark.parametrize("mode", ["strict", "hardened"])
@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_golden_family(family, mode):
    rep = run_family(family, mode)
    failed = [(r.name, r.detail) for r in rep.results if not r.passed]
    assert not failed, failed
    assert rep.cases_total > 0


def _golden_graph(s):
    a = s.tensor_variable([1.0, 2.0], [2], True)
    b = s.tensor_variable([3.0, 4.0], [2], True)
    return a, b, s.tensor_mul(s.tensor_add(a, b), s.tensor_mul(a, b))


def test_scheduler_golden_telemetry():
    s = FrankenTorchSession()
    a, b, e = _golden_graph(s)
    rep = s.tensor_backward(e)
    t = rep.telemetry
    assert t.execution_order == [4, 3, 2, 1, 0]
    assert t.dependency_snapshot == [2, 2, 1, 1, 0]
    assert (t.queue_pushes, t.queue_pops, t.max_queue_len) == (5, 5, 2)
    assert [st.rule for st in rep.steps] == ["d(a*b)/da=b; d(a*b)/db=a", "d(a*b)/da=b; d(a*b)/db=a",
                                            "d(a+b)/da=1; d(a+b)/db=1", "leaf", "leaf"]
    assert s.tensor_gradient(rep, a) == [15.0, 32.0]


def test_replay_is_bit_identical():
    outs = []
    for _ in range(2):
        s = FrankenTorchSession()
        x = s.randn([8, 16], requires_grad=True)
        w = s.randn([4, 16], requires_grad=True)
        y = s.tensor_sum(s.tensor_tanh(s.tensor_linear(x, w)))
        rep = s.tensor_backward(y)
        outs.append((s.tensor(x).clone(), rep.gradient(w).clone(), rep.telemetry.execution_order,
                     [e.summary for e in s.evidence()]))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert outs[0][2] == outs[1][2] and outs[0][3] == outs[1][3]   # ledger identical modulo timestamps


def test_graph_consumed_and_retain():
    s = FrankenTorchSession()
    a, b, e = _golden_graph(s)
    s.tensor_backward_with_options(e, BackwardOptions(retain_graph=True))
    s.tensor_backward(e)
    with pytest.raises(TensorGraphConsumed):
        s.tensor_backward(e)
    # leaf gradients accumulated across the two successful calls
    assert s.tensor_accumulated_gradient(a) == [30.0, 64.0]


def test_root_must_require_grad_and_float_leaves_only():
    s = FrankenTorchSession()
    x = s.tensor_variable([1.0], [1], False)
    with pytest.raises(TensorRootDoesNotRequireGrad):
        s.tensor_backward(s.tensor_neg(x))
    with pytest.raises(TensorRequiresGradNonFloating):
        s.tensor_tape.leaf(torch.tensor([1, 2]), True)


def test_reentrant_policy_strict_vs_hardened():
    s = FrankenTorchSession()
    _, _, e = _golden_graph(s)
    with pytest.raises(ReentrantDepthExceeded) as ei:
        s.tensor_backward_with_options(e, BackwardOptions(current_reentrant_depth=3, max_reentrant_depth=2))
    assert (ei.value.current, ei.value.max) == (3, 2)
    rep = s.tensor_backward_with_options(e, BackwardOptions(current_reentrant_depth=3, max_reentrant_depth=2,
                                                            policy=ReentrantPolicy.HardenedBoundedFallback))
    assert rep.telemetry.reentrant_guard_triggered and rep.telemetry.hardened_fallback_used
    assert rep.telemetry.reentrant_depth == 2


def test_hooks_run_in_registration_order_and_guard_shape():
    s = FrankenTorchSession()
    a, b, e = _golden_graph(s)
    seen = []
    s.register_tensor_hook(a, lambda g: seen.append("first") or None)
    h = s.register_tensor_hook(a, lambda g: (seen.append("second"), g * 2)[1])
    rep = s.tensor_backward_with_options(e, BackwardOptions(retain_graph=True))
    assert seen == ["first", "second"] and s.tensor_gradient(rep, a) == [30.0, 64.0]
    assert s.remove_tensor_hook(h)
    s.register_tensor_hook(b, lambda g: g[:1])
    with pytest.raises(TensorGradientShapeMismatch):
        s.tensor_backward(e)


def test_retain_grad_and_no_grad_and_truncate():
    s = FrankenTorchSession()
    a = s.tensor_variable([1.0, 2.0], [2], True)
    mid = s.tensor_mul_scalar(a, c=3.0)
    s.tensor_retain_grad(mid)
    s.tensor_backward(s.tensor_sum(s.tensor_square(mid)))
    assert s.tensor_accumulated_gradient(mid) == [6.0, 12.0]
    assert s.tensor_accumulated_gradient(a) == [18.0, 36.0]
    boundary = s.autograd_graph_len()
    with s.no_grad():
        z = s.tensor_exp(a)
    assert not s.tensor_requires_grad(z) and s.is_grad_enabled()
    s.truncate_autograd_graph(boundary)
    assert s.autograd_graph_len() == boundary


def test_custom_function_and_borrowed_version_guard():
    s = FrankenTorchSession()
    x = s.tensor_variable([1.0, 2.0, 3.0], [3], True)
    w = s.tensor_variable([2.0], [1], False)

    def fwd(ctx, ts):
        ctx.save_for_backward(ts[0])
        return ts[0] ** 3

    def bwd(ctx, g):
        return [g * 3 * ctx.saved_tensors[0] ** 2, None]

    y = s.tensor_apply_function([x, w], fwd, bwd, borrow_inputs=True)
    rep = s.tensor_backward_with_options(s.tensor_sum(y), BackwardOptions(retain_graph=True))
    assert s.tensor_gradient(rep, x) == [3.0, 12.0, 27.0]
    assert rep.steps[1].rule == "custom autograd function backward"
    s.tensor_fill_(w, 5.0)   # in-place mutation bumps the version of a borrowed input
    with pytest.raises(BorrowedInputVersionMismatch):
        s.tensor_backward(s.tensor_sum(y))


def test_checkpoint_recomputes_and_matches():
    def block(sess, h):
        return sess.tensor_tanh(sess.tensor_mul_scalar(h, c=2.0))
    g = []
    for use_ckpt in (False, True):
        s = FrankenTorchSession()
        x = s.tensor_variable([0.1, -0.2, 0.3], [3], True)
        y = s.checkpoint(block, [x]) if use_ckpt else block(s, x)
        s.tensor_backward(s.tensor_sum(y))
        g.append(s.tensor_accumulated_gradient(x))
    assert g[0] == g[1]


def test_sign_of_zero_preserved_in_first_accumulation():
    s = FrankenTorchSession()
    x = s.tensor_variable([1.0], [1], True)
    y = s.tensor_mul_scalar(x, c=-0.0)
    rep = s.tensor_backward(y)
    g = rep.gradient(x)
    assert torch.signbit(g).item() and g.item() == 0.0


def test_ledger_anchor_survives_trimming_and_mode_policy():
    rt = RuntimeContext(ExecutionMode.Strict, soft_cap=16)
    for i in range(100):
        rt.ledger.record(EvidenceKind.Dispatch, f"d{i}")
    ev = rt.evidence()
    assert ev[0].summary == "mode initialized to Strict" and len(ev) <= 16 and ev[-1].summary == "d99"
    rt.set_mode(ExecutionMode.Hardened)
    rt.record_checkpoint_decode_failure("bad json")
    kinds = [e.kind for e in rt.evidence()[-2:]]
    assert kinds == [EvidenceKind.Policy, EvidenceKind.Durability]


def test_dispatch_resolution_matrix():
    strict, hard = ExecutionMode.Strict, ExecutionMode.Hardened
    ks = DispatchKeySet.from_keys([DispatchKey.CompositeExplicitAutograd, DispatchKey.CPU, DispatchKey.BackendSelect])
    with pytest.raises(DispatchKeyError):
        resolve(strict, ks)
    sel, back, eff, fb = resolve(hard, ks)
    assert (sel, back, eff, fb) == (DispatchKey.CompositeExplicitAutograd, DispatchKey.CPU, DispatchKey.CPU, True)
    with pytest.raises(DispatchKeyError):
        resolve(hard, DispatchKeySet.from_keys([DispatchKey.AutogradCPU]))       # autograd key needs its backend
    with pytest.raises(DispatchKeyError):
        DispatchKeySet.from_bits_checked(1 << 40)
    sm = DispatchKeySet.from_keys([DispatchKey.SM100, DispatchKey.AutogradSM100, DispatchKey.BackendSelect])
    assert resolve(strict, sm)[:3] == (DispatchKey.AutogradSM100, DispatchKey.SM100, DispatchKey.AutogradSM100)
    v, d = dispatch_scalar_binary("mul", strict, 2.0, 4.0, True)
    assert v == 8.0 and d.kernel == "autograd_cpu::mul_scalar"


def test_finite_difference_gradient_audit():
    """Central differences vs the DAC gradient for a sample of operators (ft-api/tests/grad_fd_audit.rs)."""
    ops = [("tanh", {}), ("gelu", {}), ("softplus", {}), ("sigmoid", {}), ("exp", {}), ("softmax", {"dim": -1}),
           ("log_softmax", {"dim": -1}), ("cumsum", {"dim": 0}), ("layer_norm", {"eps": 1e-5}), ("rms_norm", {})]
    base = torch.tensor([[0.3, -1.2, 0.7], [1.5, 0.2, -0.4]], dtype=torch.float64)
    wts = torch.tensor([[0.5, -0.3, 0.8], [1.1, 0.4, -0.9]], dtype=torch.float64)
    for name, kw in ops:
        def loss_of(vals):
            s = FrankenTorchSession(ledger_dispatch=False)
            x = s.tensor_variable(vals.reshape(-1).tolist(), [2, 3], True)
            y = getattr(s, "tensor_" + name)(x, **kw)
            w = s.tensor_variable(wts.reshape(-1).tolist(), [2, 3])
            return s, x, s.tensor_sum(s.tensor_mul(y, w))
        s, x, l = loss_of(base)
        rep = s.tensor_backward(l)
        g = rep.gradient(x).reshape(-1)
        for i in range(6):
            e = torch.zeros(6, dtype=torch.float64)
            e[i] = 1e-6
            lp = loss_of(base.reshape(-1) + e)[0]
            fp = lp.tensor_item(lp.autograd_graph_len() - 1)
            lm = loss_of(base.reshape(-1) - e)[0]
            fm = lm.tensor_item(lm.autograd_graph_len() - 1)
            fd = (fp - fm) / 2e-6
            assert abs(fd - g[i].item()) < 1e-6, (name, i, fd, g[i].item())
