"""Public types that the reference's crates export next to their functions: serializer envelope / modes / error kinds
(ft-serialize/src/lib.rs:49-75, :166-175, :608), optimizer option enums (ft-optim/src/lib.rs:1818, :4381), ``nn`` option
enums, typed registration / state-dict errors and packed quantized linear weights (ft-nn/src/lib.rs:133, :177, :20192-20700)."""
import os

import pytest
import torch

from frankentorch_b200 import nn, serialize as S
from frankentorch_b200.optim import LBFGS, SGD, CyclicLR, CyclicLRMode, LBFGSLineSearch
from frankentorch_b200.session import FrankenTorchSession


def test_checkpoint_envelope_modes_and_snapshot_shorthands():
    entries = [S.SnapshotEntry(2, 1.5, None), S.SnapshotEntry(0, -2.0, 0.25)]
    env = S.encode_envelope(entries, S.CheckpointMode.Hardened)
    assert env.mode is S.CheckpointMode.Hardened and env.schema_version == 1 and [e.node_id for e in env.entries] == [0, 2]
    assert env.source_hash.startswith("det64:")
    assert S.decode_envelope(env.to_json(), S.DecodeMode.Hardened) == env
    assert env.to_json() == S.encode_checkpoint(entries, "hardened")
    assert S.decode_snapshot(S.encode_snapshot(entries)) == list(env.entries)
    with pytest.raises(S.SerializeError) as strict:
        S.decode_envelope("{", S.DecodeMode.Strict)
    with pytest.raises(S.SerializeError) as hard:
        S.decode_envelope("{", S.DecodeMode.Hardened)
    assert "invalid json" in str(strict.value) and "incompatible payload" in str(hard.value)
    side, _ = S.generate_repair_sidecar(b"frankentorch" * 400, 3)
    recs = side.symbol_records()
    assert len(recs) == side.repair_symbols and all(isinstance(r, S.RepairSymbolRecord) and r.bytes == side.symbol_size for r in recs)
    assert [r.esi for r in recs] == [m.esi for m in side.repair_manifest]


def test_tensor_io_error_kinds_and_byte_level_safetensors(tmp_path):
    sd = {"w": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.ones(2, dtype=torch.bfloat16)}
    blob = S.save_safetensors_to_bytes(sd, {"note": "x"})
    back = S.load_safetensors_from_bytes(blob)
    assert all(torch.equal(back[k], sd[k]) for k in sd)
    p = str(tmp_path / "a.safetensors")
    S.save_safetensors(sd, p, {"note": "x"})
    assert open(p, "rb").read() == blob and S.load_tensor_file(p).keys() == sd.keys()
    f = str(tmp_path / "a.ftsv")
    S.save_state_dict({"w": sd["w"]}, f)
    assert torch.equal(S.load_tensor_file(f)["w"], sd["w"])
    with pytest.raises(S.TensorIOError) as e:
        S.load_tensor_file(str(tmp_path / "missing"))
    assert e.value.kind == "Io" and e.value.fields["path"].endswith("missing")
    open(f, "wb").write(b"FTSV" + (99).to_bytes(4, "little") + b"\0" * 8)
    with pytest.raises(S.TensorIOError) as e:
        S.load_tensor_file(f)
    assert e.value.kind == "UnsupportedVersion"
    open(p, "wb").write(blob[:24])
    with pytest.raises(S.TensorIOError) as e:
        S.load_tensor_file(p)
    assert e.value.kind == "Corrupt" and "reason" in e.value.fields
    with pytest.raises(ValueError):
        S.TensorIOError("Nope", "x")
    n = S.save_linear_onnx(torch.ones(2, 3), torch.zeros(2), str(tmp_path / "l.onnx"))
    assert n == os.path.getsize(str(tmp_path / "l.onnx")) == len(S.export_linear_onnx_to_bytes(torch.ones(2, 3), torch.zeros(2)))


def _rosenbrock(s, w):
    x, y = s.tensor_select(w, 0, 0), s.tensor_select(w, 0, 1)
    one, hundred = s.tensor_variable([1.0], []), s.tensor_variable([100.0], [])
    return s.tensor_add(s.tensor_square(s.tensor_sub(one, x)), s.tensor_mul(hundred, s.tensor_square(s.tensor_sub(y, s.tensor_square(x)))))


def test_lbfgs_strong_wolfe_search_converges_on_rosenbrock_with_fewer_evaluations():
    def run(ls):
        s = FrankenTorchSession(ledger_dispatch=False)
        w = s.tensor_variable([-1.2, 1.0], [2], True)
        opt = LBFGS([w], lr=1.0, max_iter=60, line_search=ls)
        evals = [0]

        def closure():
            evals[0] += 1
            s.tensor_zero_grads([w])
            loss = _rosenbrock(s, w)
            s.tensor_backward(loss)
            return s.tensor_item(loss)
        for _ in range(3):
            loss = opt.step(s, closure)
        return loss, s.tensor(w).tolist(), evals[0]
    loss, w, n_wolfe = run(LBFGSLineSearch.StrongWolfe)
    assert loss < 1e-12 and abs(w[0] - 1) < 1e-5 and abs(w[1] - 1) < 1e-5
    loss_fixed, _, n_fixed = run(LBFGSLineSearch.NoSearch)
    assert loss_fixed < 1e-8 and n_wolfe < n_fixed
    assert LBFGSLineSearch.parse("strong_wolfe") is LBFGSLineSearch.StrongWolfe and LBFGSLineSearch.parse(None) is LBFGSLineSearch.NoSearch
    assert LBFGSLineSearch.parse("armijo") is LBFGSLineSearch.BacktrackingArmijo
    with pytest.raises(ValueError):
        LBFGSLineSearch.parse("golden")


def test_strong_wolfe_step_satisfies_both_conditions_on_a_quadratic():
    s = FrankenTorchSession(ledger_dispatch=False)
    w = s.tensor_variable([3.0, -2.0], [2], True)
    scale = s.tensor_variable([1.0, 10.0], [2])
    opt = LBFGS([w], line_search="strong_wolfe")

    def closure():
        s.tensor_zero_grads([w])
        loss = s.tensor_sum(s.tensor_mul(scale, s.tensor_square(w)))
        s.tensor_backward(loss)
        return s.tensor_item(loss)
    f0 = closure()
    g = opt._flat(s, True)
    d, x0 = -g, opt._flat(s, False)
    g0 = float(g @ d)
    t, f = opt._strong_wolfe(s, closure, x0, d, f0, g0, 1.0)
    gt = float(opt._flat(s, True) @ d)
    assert t > 0 and f <= f0 + 1e-4 * t * g0 and abs(gt) <= 0.9 * abs(g0)


def test_cyclic_lr_mode_objects_drive_the_schedule():
    def lrs(mode, gamma=1.0, n=9):
        s = FrankenTorchSession(ledger_dispatch=False)
        w = s.tensor_variable([0.0], [1], True)
        opt = SGD([w], lr=0.1)
        sched = CyclicLR(opt, 0.1, 1.0, step_size_up=2, mode=mode, gamma=gamma)
        out = []
        for _ in range(n):
            out.append(round(opt.get_lr(), 10))
            sched.step(opt)
        return out
    assert lrs(CyclicLRMode.Triangular) == lrs("triangular")
    assert lrs(CyclicLRMode.Triangular2) == lrs("triangular2") and lrs(CyclicLRMode.Triangular2)[6] < lrs(CyclicLRMode.Triangular)[6]
    assert lrs(CyclicLRMode.ExpRange(0.9)) == lrs("exp_range", 0.9)
    assert CyclicLRMode.ExpRange(0.9) == CyclicLRMode("exp_range", 0.9) and CyclicLRMode.Triangular != CyclicLRMode.Triangular2
    with pytest.raises(ValueError):
        CyclicLRMode("sawtooth")


def test_nn_option_enums_are_the_strings_the_modules_take():
    assert nn.Reduction.Mean == "mean" and nn.Reduction.parse("SUM") is nn.Reduction.Sum and str(nn.Reduction.NoReduction) == "none"
    assert nn.UpsampleMode.parse("nearest_exact") is nn.UpsampleMode.NearestExact and f"{nn.UpsampleMode.Bilinear}" == "bilinear"
    assert nn.PaddingMode.Zeros.pad_mode() == "constant" and nn.PaddingMode.Reflect.pad_mode() == "reflect"
    assert {m.value for m in nn.DistanceKind} == {"l2", "l1", "cosine"} and {m.value for m in nn.EmbeddingBagMode} == {"sum", "mean", "max"}
    assert [m.value for m in nn.CTCReduction] == ["none", "sum", "mean"] and [m.value for m in nn.TransformerActivation] == ["relu", "gelu"]
    with pytest.raises(ValueError):
        nn.Reduction.parse("median")
    s = FrankenTorchSession(ledger_dispatch=False)
    a, b = s.tensor_variable([1.0, 2.0], [2]), s.tensor_variable([0.0, 0.0], [2])
    assert s.tensor_item(nn.MSELoss(reduction=nn.Reduction.Sum)(s, a, b)) == 5.0
    assert s.tensor_item(nn.MSELoss(reduction=nn.Reduction.Mean)(s, a, b)) == 2.5
    x = s.tensor_variable(list(range(8)), [1, 1, 2, 4])
    up = nn.Upsample(scale_factor=2, mode=nn.UpsampleMode.Nearest)(s, x)
    assert s.tensor_shape(up) == [1, 1, 4, 8]


def test_registration_and_state_dict_errors_are_typed():
    s = FrankenTorchSession(ledger_dispatch=False)
    m = nn.Linear(s, 3, 2)
    with pytest.raises(nn.ModuleRegistrationError) as e:
        m.register_parameter("a.b", None)
    assert e.value.kind == "InvalidName" and e.value.fields == {"what": "parameter"} and isinstance(e.value, nn.ModuleError)
    with pytest.raises(nn.ModuleRegistrationError) as e:
        m.register_buffer("weight", None)
    assert e.value.kind == "NameConflict" and e.value.fields == {"name": "weight"}
    sd = m.state_dict(s)
    with pytest.raises(nn.StateDictError) as e:
        m.load_state_dict(s, {"weight": sd["weight"], "extra": sd["bias"]})
    assert e.value.kind == "StrictKeyMismatch" and e.value.fields == {"missing_keys": ["bias"], "unexpected_keys": ["extra"]}
    with pytest.raises(nn.StateDictError) as e:
        m.load_state_dict(s, {"weight": torch.zeros(2, 2, dtype=torch.float64), "bias": sd["bias"]})
    assert e.value.kind == "ShapeMismatch" and e.value.fields["expected"] == (2, 3) and e.value.fields["found"] == (2, 2)
    assert e.value.reason_code == "state_dict_shape_mismatch"


def test_packed_quantized_linear_per_tensor_and_per_channel():
    w = [0.5, -0.25, 1.0, 0.1, 0.2, -0.3]
    W = torch.tensor(w, dtype=torch.float64).reshape(2, 3)
    q = nn.QuantizedLinear.from_float_weights(w, [0.5, -0.5], 3, 2, nn.QuantizedStorageDType.QInt8, nn.QParams(0.01, 0, -128, 127))
    assert q.weight_storage().qint8_values() == [50, -25, 100, 10, 20, -30] and q.weight_storage().quint8_values() is None
    assert q.weight_qparams() == nn.QParams(0.01, 0, -128, 127) and q.weight_quantization_axis() is None
    assert (q.in_features(), q.out_features(), q.bias_values(), q.parameters()) == (3, 2, [0.5, -0.5], [])
    assert q.weight_tensor().dtype == torch.int8 and tuple(q.weight_tensor().shape) == (2, 3)
    s = FrankenTorchSession(ledger_dispatch=False)
    X = torch.tensor([[1.0, 2.0, 3.0], [-1.0, 0.5, 0.25]], dtype=torch.float64)
    x = s.tensor_variable(X.reshape(-1).tolist(), [2, 3], True)
    y = q(s, x)
    assert torch.allclose(s.tensor(y), X @ W.t() + torch.tensor([0.5, -0.5]), atol=1e-12)
    rep = s.tensor_backward(s.tensor_sum(y))
    assert torch.allclose(rep.gradient(x), W.sum(0).expand(2, 3))
    # clamping at the storage range and round-to-nearest-even
    c = nn.QuantizedLinear.from_float_weights([2.0, 0.005, 0.015], None, 3, 1, nn.QuantizedStorageDType.QInt8, nn.QParams(0.01, 0, -128, 127))
    assert c.weight_storage().qint8_values() == [127, 0, 2]
    pc = nn.QuantizedLinear.from_float_weights_per_channel(
        w, None, 3, 2, nn.QuantizedStorageDType.QUInt8, 0, [nn.QParams(0.01, 128, 0, 255), nn.QParams(0.005, 100, 0, 255)])
    assert pc.weight_storage().quint8_values() == [178, 103, 228, 120, 140, 40] and pc.weight_quantization_axis() == 0
    assert len(pc.weight_channel_qparams()) == 2 and pc.weight_qparams() is None
    assert torch.allclose(pc.weight_storage().dequantized(pc.weight_qparam_layout()), W, atol=1e-12)
    assert torch.allclose(s.tensor(pc(s, x)), X @ W.t(), atol=1e-12)
    for bad in (lambda: nn.QuantizedLinear.from_float_weights(w, None, 0, 2, nn.QuantizedStorageDType.QInt8, nn.QParams(0.01, 0)),
                lambda: nn.QuantizedLinear.from_float_weights(w[:5], None, 3, 2, nn.QuantizedStorageDType.QInt8, nn.QParams(0.01, 0)),
                lambda: nn.QuantizedLinear.from_float_weights(w, [0.0], 3, 2, nn.QuantizedStorageDType.QInt8, nn.QParams(0.01, 0)),
                lambda: nn.QuantizedLinear.from_float_weights(w, None, 3, 2, nn.QuantizedStorageDType.QInt8, nn.QParams(0.0, 0)),
                lambda: nn.QuantizedLinear.from_float_weights(w, None, 3, 2, nn.QuantizedStorageDType.QInt8, nn.QParams(0.01, 0, 0, 255)),
                lambda: nn.QuantizedLinear.from_float_weights(w, None, 3, 2, nn.QuantizedStorageDType.QUInt8, nn.QParams(0.01, 300, 0, 255)),
                lambda: nn.QuantizedLinear.from_float_weights_per_channel(w, None, 3, 2, nn.QuantizedStorageDType.QInt8, 0, [nn.QParams(0.01, 0)]),
                lambda: nn.QuantizedLinear.from_float_weights_per_channel(w, None, 3, 2, nn.QuantizedStorageDType.QInt8, 2, [nn.QParams(0.01, 0)] * 2)):
        with pytest.raises(ValueError):
            bad()
    assert nn.QuantizedStorageDType.QUInt8.qrange() == (0, 255)
    # the layer-derived form still works and reports that it has no packed weights
    lin = nn.QuantizedLinear(s, nn.Linear(s, 3, 2))
    assert s.tensor_shape(lin(s, x)) == [2, 2]
    with pytest.raises(ValueError):
        lin.weight_storage()


# ------------------------------------------------------------------------------------ optimizer / scheduler options
def _sgd(momentum=0.95):
    s = FrankenTorchSession(ledger_dispatch=False)
    x = s.tensor_variable([1.0], [1], True)
    return s, x, SGD([x], 1.0, momentum=momentum)


def _torch_sgd(momentum=0.95):
    p = torch.nn.Parameter(torch.zeros(1))
    return torch.optim.SGD([p], lr=1.0, momentum=momentum)


@pytest.mark.parametrize("three_phase,anneal", [(False, "cos"), (True, "linear"), (True, "cos")])
def test_one_cycle_lr_phases_and_momentum_match_pytorch(three_phase, anneal):
    from frankentorch_b200.optim import OneCycleLR
    o = _torch_sgd()
    ts = torch.optim.lr_scheduler.OneCycleLR(o, 2.0, total_steps=20, pct_start=0.25, three_phase=three_phase, anneal_strategy=anneal,
                                             div_factor=10.0, final_div_factor=100.0, base_momentum=0.8, max_momentum=0.95)
    _, _, opt = _sgd()
    sc = OneCycleLR(opt, 2.0, 20, pct_start=0.25, div_factor=10.0, final_div_factor=100.0, anneal=anneal, three_phase=three_phase,
                    cycle_momentum=True, base_momentum=0.8, max_momentum=0.95)
    for i in range(20):
        assert abs(opt.get_lr() - o.param_groups[0]["lr"]) < 1e-12 and abs(opt.get_momentum() - o.param_groups[0]["momentum"]) < 1e-12, i
        if i < 19:
            o.step()
            ts.step()
            sc.step(opt)
    assert sc.get_last_momentum() == opt.get_momentum()
    with pytest.raises(ValueError):
        sc.step(opt, epoch=21)
    # builder spelling, explicit epochs, state round trip
    _, _, opt2 = _sgd()
    b = OneCycleLR(opt2, 2.0, 30).three_phase(True).anneal_strategy_linear().cycle_momentum(True).base_momentum(0.8).max_momentum(0.95)
    b.step(opt2, epoch=11)
    st = b.state()
    c = OneCycleLR(opt2, 1.0, 5)
    c.load_state(st)
    assert c.state().extra == st.extra and c.last_epoch == 11
    s3 = FrankenTorchSession(ledger_dispatch=False)
    from frankentorch_b200.optim import Adagrad
    with pytest.raises(ValueError):
        OneCycleLR(Adagrad([s3.tensor_variable([1.0], [1], True)], lr=0.1), 1.0, 10, cycle_momentum=True)


def test_cyclic_lr_momentum_cycles_against_the_rate_as_in_pytorch():
    o = _torch_sgd(0.9)
    ts = torch.optim.lr_scheduler.CyclicLR(o, 0.1, 1.0, step_size_up=3, step_size_down=5, mode="triangular2", cycle_momentum=True,
                                           base_momentum=0.8, max_momentum=0.9)
    _, _, opt = _sgd(0.9)
    sc = CyclicLR(opt, 0.1, 1.0, step_size_up=3, step_size_down=5, mode=CyclicLRMode.Triangular2, cycle_momentum=True,
                  base_momentum=0.8, max_momentum=0.9)
    for i in range(20):
        assert abs(opt.get_lr() - o.param_groups[0]["lr"]) < 1e-12 and abs(opt.get_momentum() - o.param_groups[0]["momentum"]) < 1e-12, i
        o.step()
        ts.step()
        sc.step(opt)


def test_reduce_lr_on_plateau_threshold_modes_match_pytorch():
    from frankentorch_b200.optim import ReduceLROnPlateau
    metrics = [1.0, 0.99995, 0.9999, 0.9998, 0.9, 0.9, 0.9, 0.9, 0.85, 0.85, 0.85, 0.85, 0.85]
    for mode, tmode in (("min", "rel"), ("min", "abs"), ("max", "rel"), ("max", "abs")):
        o = _torch_sgd()
        ts = torch.optim.lr_scheduler.ReduceLROnPlateau(o, mode=mode, factor=0.5, patience=1, threshold=1e-3, threshold_mode=tmode)
        _, _, opt = _sgd()
        sc = ReduceLROnPlateau(opt, mode=mode, factor=0.5, patience=1, threshold=1e-3, threshold_mode=tmode)
        for m in metrics:
            v = m if mode == "min" else -m + 2
            ts.step(v)
            sc.step(opt, v)
            assert abs(opt.get_lr() - o.param_groups[0]["lr"]) < 1e-15, (mode, tmode, m)
    _, _, opt = _sgd()
    b = ReduceLROnPlateau(opt).mode_max().threshold_mode_abs()
    assert (b.mode, b.threshold_mode, b.best) == ("max", "abs", -float("inf"))
    assert ReduceLROnPlateau(opt).mode_min().threshold_mode_rel().threshold_mode == "rel"
    with pytest.raises(ValueError):
        ReduceLROnPlateau(opt, threshold_mode="pct")


def test_grad_scaler_switches_and_skip_flag():
    from frankentorch_b200.optim import GradScaler
    s, x, opt = _sgd(0.0)
    sc = GradScaler(init_scale=4.0)
    loss = s.tensor_sum(s.tensor_mul(x, x))
    s.tensor_backward(sc.scale_loss(s, loss))
    assert sc.step(s, opt) and not sc.last_step_was_skipped() and abs(s.tensor(x).item() - (1.0 - 2.0)) < 1e-12
    s.tensor_set_accumulated_gradient(x, [float("inf")])
    before = s.tensor(x).item()
    assert not sc.step(s, opt) and sc.last_step_was_skipped() and s.tensor(x).item() == before
    sc.update()
    assert sc.get_scale() == 2.0
    sc.disable()
    assert not sc.is_enabled() and sc.scale_loss(s, loss) == loss
    s.tensor_set_accumulated_gradient(x, [0.5])
    assert sc.step(s, opt) and not sc.last_step_was_skipped()
    sc.enable()
    assert sc.is_enabled()


@pytest.mark.parametrize("name", ["RAdam", "NAdam"])
def test_decoupled_weight_decay_of_radam_and_nadam_matches_pytorch(name):
    import frankentorch_b200.optim as O
    w0 = torch.tensor([0.5, -1.5, 2.0], dtype=torch.float64)
    for decoupled in (False, True):
        p = torch.nn.Parameter(w0.clone())
        to = getattr(torch.optim, name)([p], lr=0.05, weight_decay=0.1, decoupled_weight_decay=decoupled)
        s = FrankenTorchSession(ledger_dispatch=False)
        w = s.tensor_variable(w0.tolist(), [3], True)
        mine = getattr(O, name)([w], lr=0.05, weight_decay=0.1).decoupled_weight_decay(decoupled)
        for _ in range(8):
            to.zero_grad()
            (p ** 3).sum().backward()
            to.step()
            mine.zero_grad(s)
            s.tensor_backward(s.tensor_sum(s.tensor_pow(w, 3.0)))
            mine.step(s)
        assert torch.allclose(s.tensor(w), p.detach(), atol=1e-10), (name, decoupled)


def test_asgd_averaged_parameters_and_lbfgs_evaluation_budget():
    from frankentorch_b200.optim import ASGD
    s = FrankenTorchSession(ledger_dispatch=False)
    w = s.tensor_variable([1.0, -2.0], [2], True)
    opt = ASGD([w], lr=0.1, t0=2)
    assert opt.averaged_parameters() == [None]
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0], dtype=torch.float64))
    to = torch.optim.ASGD([p], lr=0.1, t0=2)
    for _ in range(6):
        opt.zero_grad(s)
        s.tensor_backward(s.tensor_sum(s.tensor_square(w)))
        opt.step(s)
        to.zero_grad()
        (p ** 2).sum().backward()
        to.step()
    (ax,) = opt.averaged_parameters()
    assert torch.allclose(ax, to.state[p]["ax"], atol=1e-12) and not torch.equal(ax, s.tensor(w))
    s2 = FrankenTorchSession(ledger_dispatch=False)
    v = s2.tensor_variable([-1.2, 1.0], [2], True)
    lb = LBFGS([v], max_iter=50, max_eval=7).line_search_fn("strong_wolfe")

    def closure():
        s2.tensor_zero_grads([v])
        loss = _rosenbrock(s2, v)
        s2.tensor_backward(loss)
        return s2.tensor_item(loss)
    lb.step_with_closure(s2, closure)
    assert 7 <= lb.n_evals <= 7 + 30          # the budget is checked between directions; one line search may overrun it
    assert LBFGS([v], max_iter=20).max_eval == 25


def test_tape_introspection_and_session_spellings():
    s = FrankenTorchSession(ledger_dispatch=False)
    x = s.tensor_variable([1.0, 2.0], [2], True)
    y = s.tensor_mul(x, x)
    w = s.tensor_variable([3.0, 4.0], [2], True)
    z = s.tensor_log_softmax(s.tensor_mul(y, w), dim=0)
    assert s.tensor_is_leaf(x) and not s.tensor_is_leaf(y) and s.tensor_grad_fn(x) is None
    assert s.tensor_grad_fn(y) == "MulBackward" and s.tensor_grad_fn(z) == "LogSoftmaxBackward"
    assert s.tensor_node_count() == s.autograd_graph_len() == 5
    assert not s.tensor_has_hooks(y)
    h = s.register_tensor_hook(y, lambda g: None)
    assert s.tensor_has_hooks(y) and s.remove_tensor_hook(h) and not s.tensor_has_hooks(y)
    assert not s.tensor_retains_grad(y)
    s.tensor_retain_grad(y)
    assert s.tensor_retains_grad(y) and not s.tensor_retains_grad(x)        # a leaf keeps its gradient without asking
    c = s.tensor_variable([1.0], [1], False)
    with pytest.raises(Exception):
        s.tensor_retain_grad(c)
    # detaching in place cuts the path to x; w still receives its gradient
    s.tensor_detach_(y)
    assert s.tensor_is_leaf(y) and not s.tensor_requires_grad(y)
    rep = s.tensor_backward(s.tensor_sum(z))
    assert rep.gradient(w) is not None and (rep.gradient(x) is None or float(rep.gradient(x).abs().sum()) == 0.0)
    # tape-level anomaly mode
    assert not s.is_detect_anomaly()
    s.set_detect_anomaly(True)
    a = s.tensor_variable([0.0], [1], True)
    from frankentorch_b200.autograd.tape import AnomalyDetected
    with pytest.raises(AnomalyDetected):
        s.tensor_backward(s.tensor_sum(s.tensor_log(a)))
    s.set_detect_anomaly(False)
    s.tensor_backward(s.tensor_sum(s.tensor_log(s.tensor_variable([0.0], [1], True))))
    # grad mode as a setter that returns the previous value
    assert s.set_grad_enabled(False) is True and not s.is_grad_enabled()
    n = s.tensor_mul(x, x)
    assert not s.tensor_requires_grad(n)
    assert s.set_grad_enabled(True) is False and s.is_grad_enabled()


def test_attention_weights_output_matches_pytorch_and_is_differentiable():
    s = FrankenTorchSession(ledger_dispatch=False)
    mha = nn.MultiheadAttention(s, 8, 2)
    x = s.randn([2, 5, 8], requires_grad=True)
    out, w = mha.forward_qkv_with_weights(s, x, x, x, None, True, True)
    assert torch.allclose(s.tensor(out), s.tensor(mha.forward_qkv(s, x, x, x, None, True)), atol=1e-12)
    assert s.tensor_shape(w) == [2, 5, 5] and torch.allclose(s.tensor(w).sum(-1), torch.ones(2, 5, dtype=torch.float64))
    assert float(s.tensor(w)[0, 0, 1:].abs().sum()) == 0.0                       # causal: the first query sees one key
    tm = torch.nn.MultiheadAttention(8, 2, batch_first=True, dtype=torch.float64)
    sd = mha.state_dict(s)
    with torch.no_grad():
        tm.in_proj_weight.copy_(torch.cat([sd["q_proj.weight"], sd["k_proj.weight"], sd["v_proj.weight"]]))
        tm.in_proj_bias.copy_(torch.cat([sd["q_proj.bias"], sd["k_proj.bias"], sd["v_proj.bias"]]))
        tm.out_proj.weight.copy_(sd["out_proj.weight"])
        tm.out_proj.bias.copy_(sd["out_proj.bias"])
    xt = s.tensor(x).detach()
    mask = torch.zeros(5, 5, dtype=torch.bool)
    mask[:, 3] = True
    o2, w2 = mha.forward_qkv_with_weights(s, x, x, x, s.tensor_tape.leaf(mask, False), False, False)
    to, tw = tm(xt, xt, xt, attn_mask=mask, need_weights=True, average_attn_weights=False)
    assert s.tensor_shape(w2) == [2, 2, 5, 5] and torch.allclose(to, s.tensor(o2), atol=1e-10) and torch.allclose(tw, s.tensor(w2), atol=1e-10)
    rep = s.tensor_backward(s.tensor_sum(s.tensor_square(w)))
    assert float(rep.gradient(x).abs().sum()) > 0


def test_weight_norm_functions_and_lazy_materialisation():
    s = FrankenTorchSession(ledger_dispatch=False)
    conv = nn.Conv2d(s, 3, 4, 3)
    for dim in (0, 1):
        cw = conv._parameters["weight"]
        g, v = nn.weight_norm_decompose(s, cw, dim)
        W = s.tensor(cw)
        assert s.tensor_shape(g) == [W.shape[dim]] and s.tensor_requires_grad(g) and s.tensor_requires_grad(v)
        others = [d for d in range(4) if d != dim]
        assert torch.allclose(s.tensor(g), W.pow(2).sum(others).sqrt())
        w = nn.weight_norm_reconstruct(s, g, v, dim)
        assert torch.allclose(s.tensor(w), W, atol=1e-12)
        rep = s.tensor_backward(s.tensor_sum(s.tensor_square(w)))
        # d/dg sum(w^2) = 2 g (the direction has unit norm); the direction's gradient is orthogonal to v per slice
        assert torch.allclose(rep.gradient(g), 2 * s.tensor(g), atol=1e-10)
        assert torch.allclose((rep.gradient(v) * s.tensor(v)).sum(others), torch.zeros(W.shape[dim], dtype=W.dtype), atol=1e-10)
    with pytest.raises(ValueError):
        nn.weight_norm_decompose(s, conv._parameters["weight"], 4)
    with pytest.raises(ValueError):
        nn.weight_norm_reconstruct(s, s.tensor_variable([1.0, 2.0], [2]), conv._parameters["weight"], 0)
    lazy = nn.LazyLinear(s, 3)
    assert not lazy.is_materialized() and lazy.parameters() == []
    lazy.materialize(s, 5)
    assert lazy.is_materialized() and s.tensor_shape(lazy.weight if hasattr(lazy, "weight") else lazy._parameters["weight"]) == [3, 5]
    lc = nn.LazyConv2d(s, 4, 3)
    assert not lc.is_materialized()
    y = lc.forward_lazy(s, s.randn([1, 2, 6, 6]))
    assert lc.is_materialized() and s.tensor_shape(y) == [1, 4, 4, 4] and s.tensor_shape(lc._parameters["weight"]) == [4, 2, 3, 3]
    with pytest.raises(ValueError):
        nn.LazyConv1d(s, 4, 3)(s, s.randn([1, 2, 6, 6]))


def test_quantized_metadata_typed_storage_constructors_and_sparse_accessors():
    from frankentorch_b200.core.dtype import DType
    from frankentorch_b200.core.meta import Device, QuantizationParams, TensorMeta, TensorMetaError
    from frankentorch_b200.core.storage import TensorStorage
    from frankentorch_b200.core.tensor import (DenseTensor, DenseTensorError, SparseCOOTensor, SparseCSRTensor, SparseTensorError,
                                                contiguous_bools, dense_bool_from_bools)
    q = QuantizationParams(0.5, 3)
    assert (q.scale, q.zero_point, q.axis, len(q), q.is_per_channel()) == (0.5, 3, None, 1, False)
    assert q == QuantizationParams(0.5, 3) and hash(q) == hash(QuantizationParams(0.5, 3)) and q != QuantizationParams(0.5, 4)
    pc = QuantizationParams.per_channel([0.5, 0.25], [0, 10], 0)
    assert pc.scales() == [0.5, 0.25] and pc.zero_points() == [0, 10] and pc.axis == 0 and pc.is_per_channel()
    for bad in (lambda: QuantizationParams(0.0, 0), lambda: QuantizationParams(float("nan"), 0), lambda: QuantizationParams(-1.0, 0),
                lambda: QuantizationParams.per_channel([], [], 0), lambda: QuantizationParams.per_channel([1.0], [0, 1], 0)):
        with pytest.raises(TensorMetaError):
            bad()
    m = TensorMeta.quantized_per_channel_from_shape([2, 3], DType.QInt8, Device.Cpu, [0.5, 0.25], [0, 10], 0)
    t = DenseTensor.from_storage(m, [2, 4, 6, 14, 18, 10])
    assert t.dequantized_values_as_f64() == [1.0, 2.0, 3.0, 1.0, 2.0, 0.0] == t.contiguous_values_as_f64()
    assert t.meta.dtype is DType.QInt8 and t.meta.quantization == pc
    pt = TensorMeta.quantized_from_shape([3], DType.QUInt8, Device.Cpu, 0.1, 128)
    assert pt.fingerprint64() != TensorMeta.quantized_from_shape([3], DType.QUInt8, Device.Cpu, 0.2, 128).fingerprint64()
    assert m.fingerprint64() != TensorMeta.quantized_per_channel_from_shape([2, 3], DType.QInt8, Device.Cpu, [0.5, 0.25], [0, 11], 0).fingerprint64()
    assert DenseTensor.from_contiguous_values_quantized([0, 128, 255], [3], DType.QUInt8, 0.1, 128).contiguous_values_as_f64()[1] == 0.0
    with pytest.raises(TensorMetaError):
        TensorMeta.quantized_per_channel_from_shape([2, 3], DType.QInt8, Device.Cpu, [0.5], [0], 0)       # 1 channel for extent 2
    with pytest.raises(TensorMetaError):
        TensorMeta.quantized_per_channel_from_shape([2, 3], DType.QInt8, Device.Cpu, [0.5, 0.25], [0, 0], 2)
    with pytest.raises(TensorMetaError):
        TensorMeta.from_shape([2], DType.QInt8).validate()
    with pytest.raises(TensorMetaError):
        TensorMeta.from_shape([2], DType.F32).with_quantization(q).validate()
    assert m.with_dtype(DType.F32).quantization is None and m.with_dtype(DType.QUInt8).quantization == pc
    sm = TensorMeta.quantized_from_shape_and_strides([2, 2], [1, 2], 0, DType.QInt8, Device.Cpu, 1.0, 0)
    assert sm.strides == (1, 2) and sm.quantization.scale == 1.0
    st = TensorStorage.from_values([1., 2., 3., 4., 5., 6.], DType.F32)
    v = DenseTensor.from_typed_storage(TensorMeta.from_shape_and_strides([2, 2], [2, 1], 2, DType.F32), st)
    assert v.data.tolist() == [[3.0, 4.0], [5.0, 6.0]] and len(v.typed_storage()) == 6 and v.typed_storage().dtype is DType.F32
    with pytest.raises(DenseTensorError):
        DenseTensor.from_typed_storage(TensorMeta.from_shape([7], DType.F32), st)
    with pytest.raises(DenseTensorError):
        DenseTensor.from_typed_storage(TensorMeta.from_shape([6], DType.F64), st)
    assert DenseTensor.from_contiguous_values([1.0, 2.0], [2], dtype=DType.BF16).data.dtype == torch.bfloat16
    a = DenseTensor.from_values([1., 2., 3., 4.], [4])
    assert a.shares_storage_with(a.view([2, 2])) and not a.shares_storage_with(t)
    b = dense_bool_from_bools([True, False, True, True], [2, 2])
    assert contiguous_bools(b) == [True, False, True, True] and b.data.dtype == torch.bool
    with pytest.raises(DenseTensorError):
        dense_bool_from_bools([True], [2])
    s = SparseCOOTensor.from_coords([[0, 1], [1, 0], [0, 1]], [1., 2., 3.], [2, 2])
    assert not s.is_coalesced() and s.coalesce().is_coalesced() and s.dense_shape() == [2, 2] and s.sparse_dim == 2
    assert s.to_dense().tolist() == [[0.0, 4.0], [2.0, 0.0]]
    e = SparseCOOTensor.from_coords([], [], [2, 3])
    assert e.nnz == 0 and e.sparse_dim == 2 and float(e.to_dense().abs().sum()) == 0.0 and e.is_coalesced()
    with pytest.raises(SparseTensorError):
        SparseCOOTensor.from_coords([[0, 1], [1]], [1., 2.], [2, 2])
    c = SparseCSRTensor([0, 1, 2], [1, 0], [5., 6.], [2, 2])
    assert (c.nrows(), c.ncols(), c.nnz) == (2, 2, 2)


def test_runtime_durability_envelope_updates_and_integration_hooks():
    from frankentorch_b200.runtime.integrations import (Budget, Style, asupersync_infinite_budget, frankentui_default_style,
                                                        render_ledger_panel)
    from frankentorch_b200.runtime.ledger import DurabilityEnvelope, EvidenceKind, RuntimeContext, ScrubStatus
    env = DurabilityEnvelope("ckpt-1", "checkpoint", "det64:00")
    env.mark_scrub_status(ScrubStatus.Failed)
    assert env.scrub_status is ScrubStatus.Failed and env.last_ok_unix_ms is None
    env.mark_scrub_status(ScrubStatus.Ok)
    assert env.last_ok_unix_ms is not None
    env.add_decode_proof("two source symbols dropped", "det64:ab", 2)
    assert len(env.decode_proofs) == 1 and env.decode_proofs[0].proof_hash == "det64:ab" and env.decode_proofs[0].recovered_blocks == 2
    rt = RuntimeContext("hardened")
    rt.ledger_mut().record(EvidenceKind.Durability, "scrub ok artifact=ckpt-1")
    assert rt.ledger_mut() is rt.ledger and rt.evidence()[-1].summary == "scrub ok artifact=ckpt-1"
    b = asupersync_infinite_budget()
    assert b is Budget.INFINITE and b.is_infinite() and not b.exhausted(10 ** 15, 10 ** 9, 10 ** 9)
    tight = b.meet(Budget(deadline_unix_ms=1000, poll_quota=5)).meet(Budget(deadline_unix_ms=2000, cost_quota=7, priority=3))
    assert (tight.deadline_unix_ms, tight.poll_quota, tight.cost_quota, tight.priority) == (1000, 5, 7, 3) and not tight.is_infinite()
    assert tight.exhausted(1000) and tight.exhausted(0, polls=5) and tight.exhausted(0, cost=7) and not tight.exhausted(999, 4, 6)
    st = frankentui_default_style()
    assert st == Style() and st.border == "plain" and st.width == 100
    panel = render_ledger_panel(rt.ledger, st, last=1)
    lines = panel.split("\n")
    assert lines[0] == "+" + "-" * 98 + "+" == lines[-1] and all(len(l) == 100 for l in lines)
    assert "Durability=1" in lines[1] and "Policy=1" in lines[1] and "scrub ok artifact=ckpt-1" in lines[2]
    bare = render_ledger_panel(rt.ledger, Style(border="none", width=40), last=5)
    assert not bare.startswith("+") and all(len(l) <= 40 for l in bare.split("\n"))


def test_dataset_constructors_from_items_and_input_target_pairs():
    from frankentorch_b200.data import DataError, DataItem, TensorDataset
    ds = TensorDataset.from_inputs_targets([([1., 2.], [2]), ([3., 4.], [2]), ([5., 6.], [2])], [([0.], [1]), ([1.], [1]), ([0.], [1])])
    assert len(ds) == 3 and ds.get(1).tensors == {"input": ([3.0, 4.0], (2,)), "target": ([1.0], (1,))}
    got = ds.collate_indices([2, 0])
    assert got["input"].tolist() == [[5.0, 6.0], [1.0, 2.0]] and got["target"].tolist() == [[0.0], [0.0]]
    it = DataItem.input_target([1., 2., 3., 4.], [2, 2], [7.], [1])
    assert list(it.tensors) == ["input", "target"] and it.tensors["input"][1] == (2, 2)
    assert DataItem.single("x", [1., 2.], [2]).tensors == {"x": ([1.0, 2.0], (2,))}
    with pytest.raises(DataError):
        TensorDataset.from_inputs_targets([([1.], [1])], [])
    with pytest.raises(DataError):
        TensorDataset.from_items([DataItem.single("x", [1.], [1]), DataItem.single("x", [1., 2.], [2])])
    with pytest.raises(DataError):
        DataItem.input_target([1., 2.], [3], [0.], [1])


def test_backward_option_builders_and_gradient_values():
    from frankentorch_b200.autograd.tape import BackwardOptions, GradientValue
    o = BackwardOptions.strict_default()
    o2 = o.with_create_graph(True)
    assert o2.create_graph and o2.retain_graph and not o.create_graph and not o.retain_graph      # copies, not mutation
    assert o.with_retain_graph().retain_graph and o.with_detect_anomaly().detect_anomaly
    s = FrankenTorchSession(ledger_dispatch=False)
    table = s.tensor_variable([float(i) for i in range(12)], [4, 3], True)
    idx = s.tensor_variable([2.0, 0.0, 2.0], [3])
    w = s.tensor_variable([1.0, 2.0, 3.0], [3], True)
    picked = s.tensor_index_select_sparse(table, idx)
    loss = s.tensor_sum(s.tensor_mul(picked, w))
    rep = s.tensor_backward_with_options(loss, BackwardOptions.strict_default().with_retain_graph())
    gv = rep.gradient_value(table)
    assert gv.is_sparse() and gv.as_dense() is None
    coo = gv.as_sparse()
    assert coo.indices.tolist() == [[0, 2]] and coo.values.tolist() == [[1.0, 2.0, 3.0], [2.0, 4.0, 6.0]]
    assert gv.to_dense().tolist() == [[1.0, 2.0, 3.0], [0.0, 0.0, 0.0], [2.0, 4.0, 6.0], [0.0, 0.0, 0.0]]
    assert gv.to_dense(5).tolist() == [1.0, 2.0, 3.0, 0.0, 0.0] and gv.to_dense(14).numel() == 14
    half = gv.scaled_clone(0.5)
    assert half.is_sparse() and half.as_sparse().values.tolist() == [[0.5, 1.0, 1.5], [1.0, 2.0, 3.0]]
    gw = rep.gradient_value(w)
    assert not gw.is_sparse() and gw.as_sparse() is None and gw.as_dense().tolist() == [12.0, 15.0, 18.0]
    assert gw.scaled_clone(2.0).as_dense().tolist() == [24.0, 30.0, 36.0] and rep.gradient_value(idx) is None
    with pytest.raises(ValueError):
        GradientValue()


def test_ftsv_rejects_an_extent_beyond_the_index_range_even_next_to_a_zero_extent():
    """A corrupted shape such as [0, 2^63] has volume 0, so the volume check alone lets it through to reshape."""
    import struct
    blob = bytearray(S.state_dict_to_bytes({"w": torch.zeros(0, 3)}))
    needle = struct.pack("<QQ", 0, 3)
    at = bytes(blob).index(needle)
    blob[at + 8: at + 16] = struct.pack("<Q", 1 << 63)
    with pytest.raises(S.SerializeError) as e:
        S.load_state_dict_from_bytes(bytes(blob))
    assert e.value.kind == "ShapeOverflow"
    # no single extent is out of range, but the strides of [0, 2^40, 2^40] are
    blob3 = bytearray(S.state_dict_to_bytes({"w": torch.zeros(0, 2, 3)}))
    at = bytes(blob3).index(struct.pack("<QQQ", 0, 2, 3))
    blob3[at + 8: at + 24] = struct.pack("<QQ", 1 << 40, 1 << 40)
    with pytest.raises(S.SerializeError) as e:
        S.load_state_dict_from_bytes(bytes(blob3))
    assert e.value.kind == "ShapeOverflow"


# ----------------------------------------------------------------------------- per-dtype tensor forms, value-level tape
def test_dense_tensor_per_dtype_constructors_and_accessors():
    import torch
    from frankentorch_b200.core.dtype import DType
    from frankentorch_b200.core.meta import Device, TensorMeta
    from frankentorch_b200.core.tensor import DenseTensor, DenseTensorError

    t = DenseTensor.from_contiguous_values_f32([1, 2, 3, 4, 5, 6], [2, 3])
    assert t.meta.dtype is DType.F32 and t.contiguous_values_f32().tolist() == [1, 2, 3, 4, 5, 6] and t.version == 0
    t.update_contiguous_values_f32([0.0] * 6)
    assert t.version == 1
    t.contiguous_values_f32_mut().add_(2.0)
    assert t.version == 2 and t.contiguous_values_f32().tolist() == [2.0] * 6
    with pytest.raises(DenseTensorError):
        t.update_contiguous_values_f32([1.0])
    with pytest.raises(DenseTensorError):
        t.contiguous_values_qint8()
    with pytest.raises(DenseTensorError):
        t.dispatch_values()                                    # f64 only
    for ctor, dt in ((DenseTensor.from_contiguous_values_f16, DType.F16), (DenseTensor.from_contiguous_values_bf16, DType.BF16)):
        assert ctor([1.5, 2.5], [2]).meta.dtype is dt
    q = DenseTensor.from_contiguous_values_quint8([1, 2, 3, 4], [4], 0.5, 2)
    assert q.meta.dtype is DType.QUInt8 and q.contiguous_values_quint8().tolist() == [1, 2, 3, 4]
    assert DenseTensor.from_contiguous_values_qint8([-1, 2], [2], 0.25, 0).dequantized_values_as_f64() == [-0.25, 0.5]
    qc = DenseTensor.from_contiguous_values_qint8_per_channel([1, 2, 3, 4], [2, 2], [0.5, 1.0], [0, 0], 0)
    assert qc.dequantized_values_as_f64() == [0.5, 1.0, 3.0, 4.0]
    assert DenseTensor.from_contiguous_values_quint8_per_channel([1, 2, 3, 4], [2, 2], [1.0, 2.0], [1, 0], 1) \
        .dequantized_values_as_f64() == [0.0, 4.0, 2.0, 8.0]

    m = TensorMeta.from_shape([2, 2], DType.F64, Device.Cpu)
    assert DenseTensor.from_storage_f64_inline4(m, [1, 2, 3, 4]).dispatch_values().tolist() == [1, 2, 3, 4]
    with pytest.raises(DenseTensorError):
        DenseTensor.from_storage_f64_inline4(m, [1, 2, 3])
    for ctor in (DenseTensor.from_storage_f32, DenseTensor.from_storage_f16, DenseTensor.from_storage_bf16,
                 DenseTensor.from_storage_qint8, DenseTensor.from_storage_quint8):
        with pytest.raises(DenseTensorError):
            ctor(m, [1, 2, 3, 4])                              # the meta says f64
    assert DenseTensor.from_storage_f64(m, [1, 2, 3, 4]).contiguous_values() == [1, 2, 3, 4]
    view = DenseTensor(torch.arange(12, dtype=torch.float64).reshape(3, 4)[:, 1:3])
    assert view.dispatch_values().tolist() == list(range(1, 11))      # offset .. last element, strides not applied


def test_tape_value_level_entry_points():
    import torch
    from frankentorch_b200.autograd.tape import AutogradError, TensorGradientShapeMismatch, TensorRequiresGradNonLeaf, TensorTape
    from frankentorch_b200.core.tensor import DenseTensor

    tape = TensorTape()
    w = tape.leaf_tensor(DenseTensor.from_contiguous_values_f32([1, 2, 3], [3]), True)
    x = tape.leaf_f32([4, 5, 6], [3])
    assert tape.values(w) == [1, 2, 3] and tape.values_f32(x).dtype == torch.float32
    with pytest.raises(AutogradError):
        tape.leaf_f32([1, 2], [3])
    tape.set_tensor_requires_grad(x, True)
    assert tape.nodes[x].requires_grad
    h = tape.to_bf16(w)
    assert tape.value(h).dtype == torch.bfloat16 and tape.to_bf16(h) == h and tape.to_f16(h) != h
    with pytest.raises(TensorRequiresGradNonLeaf):
        tape.set_tensor_requires_grad(h, False)
    with pytest.raises(AutogradError):
        tape.to_dtype(w, torch.int32)
    y = tape.record("mul", [h, x], tape.value(h).float() * tape.value(x),
                    lambda g, targets: [g * tape.value(x).to(g.dtype), g * tape.value(h).to(g.dtype)], "product")
    s = tape.record("sum", [y], tape.value(y).sum(), lambda g, targets: [g.expand(3)], "sum")
    rep = tape.backward(s)
    assert rep.gradient(w).tolist() == [4, 5, 6] and not rep.is_sparse_gradient(w)
    assert tape.tensor_accumulated_gradient_values(w) == [4, 5, 6] and tape.tensor_accumulated_gradient_len(w) == 3

    # an SGD step through the no-copy form, then the gradient slot is cleared but stays allocated
    v0 = tape.version(w)
    assert tape.update_tensor_values_with_accumulated_gradient(w, lambda g, p: p.sub_(0.5 * g.to(p.dtype)))
    assert tape.values(w) == [-1.0, -0.5, 0.0] and tape.version(w) == v0 + 1
    tape.zero_tensor_accumulated_gradient(w)
    assert tape.tensor_accumulated_gradient_values(w) == [0, 0, 0]
    fresh = tape.leaf_f32([1.0], [1], True)
    assert not tape.update_tensor_values_with_accumulated_gradient(fresh, lambda g, p: p.zero_())
    tape.zero_tensor_accumulated_gradient(fresh)
    assert tape.tensor_accumulated_gradient_values(fresh) is None

    tape.set_tensor_accumulated_gradient(w, [1, 1, 1])
    with pytest.raises(TensorGradientShapeMismatch):
        tape.set_tensor_accumulated_gradient(w, [1, 1])
    tape.update_tensor_values(w, [7, 8, 9])
    tape.update_tensor_values_f32(w, [1, 1, 1])
    tape.update_tensor_values_with(w, lambda p: p.mul_(3))
    assert tape.values(w) == [3, 3, 3] and tape.version(w) == v0 + 4
    with pytest.raises(AutogradError):
        tape.update_tensor_values(w, [1])
    d = tape.leaf_f64([1.0, 2.0], [2], True)
    with pytest.raises(AutogradError):
        tape.update_tensor_values_f32(d, [1, 2])

    tape.detach_tensor_in_place(w)
    assert not tape.nodes[w].requires_grad and tape.tensor_accumulated_gradient(w) is None
    tape.set_grad_enabled(False)
    assert not tape.nodes[tape.leaf_tensor(torch.ones(2), True)].requires_grad


def test_session_custom_functions_over_live_inputs():
    import torch
    from frankentorch_b200.autograd.tape import AutogradError, BorrowedInputVersionMismatch
    from frankentorch_b200.core.dtype import DType
    from frankentorch_b200.session import FrankenTorchSession

    s = FrankenTorchSession(mode="strict")
    x = s.tensor_variable([1.0, 2.0, 3.0], [3], requires_grad=True)

    def fwd(ctx, ts):
        return ts[0] ** 2

    out = s.tensor_apply_function_f64_borrowed_inputs([x], fwd, lambda ctx, g, ts: [2.0 * ts[0] * g])
    loss = s.tensor_sum(out)
    assert s.tensor_backward(loss).gradient(x).tolist() == [2.0, 4.0, 6.0]

    # a mutated input is caught at backward
    out = s.tensor_apply_function_f64_borrowed_inputs([x], fwd, lambda ctx, g, ts: [2.0 * ts[0] * g])
    loss = s.tensor_sum(out)
    s.tensor_update_values(x, [0.0, 0.0, 0.0])
    with pytest.raises(BorrowedInputVersionMismatch):
        s.tensor_backward(loss)
    s.tensor_update_values(x, [1.0, 2.0, 3.0])

    def fwd_saving(ctx, ts):
        ctx.save_for_backward(ts[0].cos())
        return ts[0].sin()

    out = s.tensor_apply_function_f64_borrowed_forward([x], fwd_saving, lambda ctx, g: [ctx.saved_tensors[0] * g])
    g = s.tensor_backward(s.tensor_sum(out)).gradient(x)
    assert torch.allclose(g, torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64).cos())

    cached = torch.tensor(14.0, dtype=torch.float64)           # sum of squares, computed by the producer
    out = s.tensor_apply_function_f64_saved_forward([x], lambda ctx: cached, lambda ctx, g: [2.0 * s.tensor(x) * g])
    assert s.tensor_values(out) == [14.0]
    assert s.tensor_backward(out).gradient(x).tolist() == [2.0, 4.0, 6.0]

    with pytest.raises(AutogradError):                          # f32 entry point, f64 input
        s.tensor_apply_function_f32_output_borrowed_inputs([x], fwd, lambda ctx, g, ts: [g])
    xf = s.tensor_leaf_f32([1.0, 2.0], [2], True)
    out = s.tensor_apply_function_f32_output_borrowed_inputs([xf], lambda ctx, ts: ts[0] * 3.0,
                                                             lambda ctx, g, ts: [3.0 * g])
    assert s.tensor(out).dtype == torch.float32
    assert s.tensor_backward(s.tensor_sum(out)).gradient(xf).tolist() == [3.0, 3.0]
    with pytest.raises(AutogradError):                          # the forward must give the promised dtype
        s.tensor_apply_function_f32_output_borrowed_inputs([xf], lambda ctx, ts: ts[0].double(), lambda ctx, g, ts: [g])

    # twice differentiable: d/dx sum(x^3) = 3x^2, d/dx of that summed = 6x
    def bwd_cg(sess, ctx, gid, ids):
        sq = sess.tensor_mul(ids[0], ids[0])
        return [sess.tensor_mul(sess.tensor_mul_scalar(sq, 3.0), gid)]

    out = s.tensor_apply_function_with_create_graph_borrowed_inputs([x], lambda ctx, ts: ts[0] ** 3, bwd_cg)
    (g1,) = s.tensor_autograd_grad(s.tensor_sum(out), [x], create_graph=True)
    assert s.tensor_values(g1) == [3.0, 12.0, 27.0]
    (g2,) = s.tensor_autograd_grad(s.tensor_sum(g1), [x])
    assert g2.tolist() == [6.0, 12.0, 18.0]

    # constant inputs: the result is a plain leaf
    c = s.tensor_variable([1.0], [1])
    k = s.tensor_apply_function_f64_borrowed_inputs([c], fwd, lambda ctx, g, ts: [g])
    assert s.tensor_is_leaf(k) and not s.tensor_requires_grad(k)

    h = s.tensor_to_bf16(x)
    assert s.tensor(h).dtype == torch.bfloat16 and s.tensor(s.tensor_to_f16(x)).dtype == torch.float16
    s.tensor_set_requires_grad(c, True)
    assert s.tensor_requires_grad(c)
    assert s.tensor_leaf_tensor(torch.ones(2, dtype=torch.float64), False) >= 0
