"""GPT on the DAC tape: gradients vs a PyTorch autograd reference of the same model, replay
determinism, and loss decrease through the CUDA-graph engine."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _build(dev, seed=3):
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.ops import kernels as K
    cfg = GPTConfig.preset("gpt-tiny")
    tape = TensorTape(grad_dtype=None)
    tape.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
    return cfg, tape, GPT(cfg, tape, device=dev, seed=seed)


def _torch_reference(cfg, params, ids, targets):
    """The same pre-LN GPT-2 in fp32 PyTorch (parameters rounded to bf16 like the compute copy)."""
    P = {k: v.float().to(torch.bfloat16).float().requires_grad_(True) for k, v in params.items()}
    B, S = ids.shape
    d, H = cfg.d_model, cfg.n_head
    x = P["wte.weight"][ids] + P["wpe.weight"][:S]
    for l in range(cfg.n_layer):
        p = f"blocks.{l}."
        h = F.layer_norm(x, (d,), P[p + "ln1.weight"], P[p + "ln1.bias"], cfg.ln_eps)
        qkv = h @ P[p + "attn.qkv_proj.weight"].t() + P[p + "attn.qkv_proj.bias"]
        q, k, v = (t.view(B, S, H, d // H).transpose(1, 2) for t in qkv.split(d, dim=-1))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, d)
        x = x + a @ P[p + "attn.out_proj.weight"].t() + P[p + "attn.out_proj.bias"]
        h = F.layer_norm(x, (d,), P[p + "ln2.weight"], P[p + "ln2.bias"], cfg.ln_eps)
        u = F.gelu(h @ P[p + "mlp.fc1.weight"].t() + P[p + "mlp.fc1.bias"], approximate="tanh")
        x = x + u @ P[p + "mlp.fc2.weight"].t() + P[p + "mlp.fc2.bias"]
    h = F.layer_norm(x, (d,), P["ln_f.weight"], P["ln_f.bias"], cfg.ln_eps)
    logits = h @ P["wte.weight"][: cfg.vocab_size].t()
    loss = F.cross_entropy(logits.view(-1, cfg.vocab_size), targets.view(-1))
    loss.backward()
    return loss.item(), {k: v.grad for k, v in P.items()}


def test_gpt_gradients_match_torch(cuda_device):
    from frankentorch_b200.ops import kernels as K
    cfg, tape, model = _build(cuda_device)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(cuda_device)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    loss_id = model.forward(ids, tgt)
    report = tape.backward(loss_id)
    K.check_status()
    loss = tape.value(loss_id).item()
    params = {n: t[: cfg.vocab_size] if n == "wte.weight" else t for n, t in model.named_parameters()}
    ref_loss, ref_grads = _torch_reference(cfg, params, ids, tgt)
    assert abs(loss - ref_loss) < 2e-2, (loss, ref_loss)
    worst = 0.0
    for name, _ in model.arena.specs:
        got = model.arena.view(model.arena.grads, name)
        if name == "wte.weight":
            got = got[: cfg.vocab_size]
        want = ref_grads[name]
        rel = (got - want).norm().item() / (want.norm().item() + 1e-8)
        worst = max(worst, rel)
        assert rel < 6e-2, f"{name}: relative gradient error {rel:.3g}"
    # scheduler contract: highest node id first, every node exactly once
    order = report.telemetry.execution_order
    assert order[0] == loss_id and order == sorted(order, reverse=True)
    assert report.telemetry.queue_pushes == report.telemetry.queue_pops == len(order)


def test_gpt_backward_replays_bit_identically(cuda_device):
    outs = []
    for _ in range(2):
        cfg, tape, model = _build(cuda_device, seed=11)
        g = torch.Generator().manual_seed(5)
        tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(cuda_device)
        loss_id = model.forward(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
        rep = tape.backward(loss_id)
        outs.append((tape.value(loss_id).clone(), model.arena.grads.clone(), rep.telemetry.execution_order,
                     [s.rule for s in rep.steps]))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])
    assert outs[0][2] == outs[1][2] and outs[0][3] == outs[1][3]


@pytest.mark.parametrize("graph", [False, True])
def test_engine_trains(cuda_device, graph):
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg, tape, model = _build(cuda_device, seed=5)
    eng = TrainEngine(model, 2, 128, OptimConfig(lr=1e-3, grad_clip=1.0), use_cuda_graph=graph)
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
    ids, tgt = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    losses = [eng.step(ids, tgt) for _ in range(8)]
    K.check_status()
    assert abs(losses[0] - math.log(cfg.vocab_size)) < 0.5
    assert losses[-1] < losses[0] - 0.3, losses
    assert int(eng.step_dev.item()) == 8


def test_grouped_weight_gradients_match_the_direct_path(cuda_device, monkeypatch):
    """The queue that launches a block's weight gradients together changes the schedule, not the gradients:
    against the direct path (one GEMM per weight gradient, split-K where the planner wants it) every parameter
    gradient agrees to fp32 summation-order accuracy, and the queue really was used."""
    from frankentorch_b200.autograd.tape import BackwardOptions
    from frankentorch_b200.ops import fused
    grads, launches = [], []
    for on in (True, False):
        monkeypatch.setattr(fused.WgradQueue, "enabled", on)
        cfg, tape, model = _build(cuda_device, seed=9)
        assert (getattr(tape, "wgrad_queue", None) is not None) == on
        g = torch.Generator().manual_seed(4)
        tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(cuda_device)
        model.reset_grads()
        loss = model.forward(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
        tape.backward(loss, BackwardOptions())
        torch.cuda.synchronize()
        grads.append(model.arena.grads.clone())
        launches.append(tape.wgrad_queue.launches if on else 0)
    assert launches[0] >= 1
    scale = float(grads[1].abs().max())
    assert float((grads[0] - grads[1]).abs().max()) <= 2e-4 * scale
    for name, _ in model.arena.specs:
        a, b = model.arena.view(grads[0], name), model.arena.view(grads[1], name)
        assert float((a - b).abs().max()) <= 1e-3 * float(b.abs().max()) + 1e-7, name


@pytest.mark.parametrize("graph", [False, True])
def test_training_step_is_on_the_evidence_ledger(cuda_device, graph):
    """The GPU training path writes what it dispatches to an EvidenceLedger: once (the eager step before the
    capture), one interned entry per (phase, operator, shape, kernels) naming launcher calls that were really
    made, plus the backward telemetry; replays add nothing."""
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.runtime.ledger import EvidenceKind, EvidenceLedger
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg, tape, model = _build(cuda_device, seed=6)
    ledger = EvidenceLedger()
    eng = TrainEngine(model, 2, 128, OptimConfig(lr=1e-3, grad_clip=1.0), use_cuda_graph=graph, ledger=ledger)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
    ids, tgt = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    eng.step(ids, tgt)
    n = len(ledger)
    assert n > 10
    for _ in range(3):
        eng.step(ids, tgt)
    K.check_status()
    assert len(ledger) == n, "replayed steps must not grow the ledger"
    entries = ledger.entries()
    disp = [e.summary for e in entries if e.kind == EvidenceKind.Dispatch]
    back = [e.summary for e in entries if e.kind == EvidenceKind.Backward]
    assert len(back) == 1 and "order_fnv1a=" in back[0] and "nodes=" in back[0]
    fwd = [s for s in disp if "phase=fwd" in s]
    bwd = [s for s in disp if "phase=bwd" in s]
    opt = [s for s in disp if "phase=optimizer" in s]
    assert fwd and bwd and len(opt) == 1
    assert all("backend=sm100" in s and "mode=strict" in s for s in disp)
    # every forward GEMM-bearing operator names the tcgen05 kernel and the tile the planner chose
    lin = [s for s in fwd if s.startswith("op=linear")]
    assert lin and all("ftk::gemm" in s and "splitK=" in s for s in lin)
    assert any("ftk_attn_fwd" in s for s in fwd) and any("ftk_attn_bwd" in s for s in bwd)
    assert "ftk_adamw_dev" in opt[0]
    # the counts add up to the nodes of the step: 2 layers x the operators of a block, not one entry per node
    total = sum(int(s.rsplit("count=", 1)[1]) for s in fwd)
    assert total >= 2 * 6 and len(fwd) < total
    # nothing on the ledger names a kernel that was not launched: the trace saw exactly launches_per_step calls
    launched = sum(int(s.rsplit("count=", 1)[1]) * len(s.split("kernel=[", 1)[1].split("] out=", 1)[0].split(", "))
                   for s in disp if "kernel=[-]" not in s)
    assert launched <= eng.launches_per_step


def _tile_rel_err(got, want, tile=128):
    """Max over ``tile x tile`` tiles of (max abs error in the tile) / (max abs reference in the tile):
    a wrong low-magnitude tile cannot hide behind large values elsewhere in the matrix."""
    g, w = got.float(), want.float()
    if g.dim() == 1:
        g, w = g[None], w[None]
    R, Cc = g.shape
    pr, pc = (-R) % tile, (-Cc) % tile
    g, w = F.pad(g, (0, pc, 0, pr)), F.pad(w, (0, pc, 0, pr))
    e = (g - w).abs().view((R + pr) // tile, tile, (Cc + pc) // tile, tile).amax((1, 3))
    m = w.abs().view((R + pr) // tile, tile, (Cc + pc) // tile, tile).amax((1, 3))
    floor = w.abs().max() * 1e-3                       # tiles that are all (near) zero in the reference
    return float((e / m.clamp_min(floor)).max())


def test_full_shape_gpt2_small_step_against_fp32_torch(cuda_device):
    """One forward + backward of the real GPT-2 small shape (12 layers, d = 768, vocab 50257 padded to
    50304, S = 1024: pair tiles, split-K weight gradients, eight key blocks of attention) against the
    same model in fp32 PyTorch: loss, every parameter's gradient (norm-relative), and a per-tile check
    of the big matrices."""
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.ops import kernels as K
    cfg = GPTConfig.preset("gpt2-small")
    tape = TensorTape(grad_dtype=None)
    tape.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
    model = GPT(cfg, tape, device=cuda_device, seed=21)
    g = torch.Generator().manual_seed(8)
    tok = torch.randint(0, cfg.vocab_size, (2, 1025), generator=g).to(cuda_device)
    ids, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    loss_id = model.forward(ids, tgt)
    tape.backward(loss_id)
    K.check_status()
    params = {n: t[: cfg.vocab_size] if n == "wte.weight" else t for n, t in model.named_parameters()}
    ref_loss, ref_grads = _torch_reference(cfg, params, ids, tgt)
    assert abs(tape.value(loss_id).item() - ref_loss) < 2e-2
    worst = ("", 0.0)
    for name, _ in model.arena.specs:
        got = model.arena.view(model.arena.grads, name)
        if name == "wte.weight":
            assert float(got[cfg.vocab_size:].abs().max()) == 0.0          # padding rows get no gradient
            got = got[: cfg.vocab_size]
        want = ref_grads[name]
        rel = (got - want).norm().item() / (want.norm().item() + 1e-12)
        if rel > worst[1]:
            worst = (name, rel)
        assert rel < 3e-2, f"{name}: relative gradient error {rel:.3g}"
    for name in ("blocks.0.attn.qkv_proj.weight", "blocks.6.mlp.fc1.weight", "blocks.11.mlp.fc2.weight",
                 "blocks.11.attn.out_proj.weight", "wpe.weight"):
        t = _tile_rel_err(model.arena.view(model.arena.grads, name), ref_grads[name])
        assert t < 0.15, f"{name}: worst 128x128 tile is off by {t:.3g} of its own magnitude"
    print("worst parameter", worst)
