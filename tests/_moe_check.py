"""MoE layer check shared by the single-GPU test and the multi-GPU worker.

Every rank regenerates all ranks' tokens and all experts' weights from seeds; the reference is a
differentiable fp32 PyTorch model of the same routing rule, evaluated for this rank's tokens.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rnd(shape, seed, scale):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def run(group, rank, world, dev, T=512, d=128, ff=256, E=8):
    from frankentorch_b200.autograd.tape import BackwardOptions, TensorTape
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.moe import ROUTER_ROWS, ExpertParallel, moe_ffn

    ep = ExpertParallel(group, dev, tokens=T, d_model=d, n_experts=E, capacity_factor=1.25)
    bufs = ep.new_layer_buffers()
    el = ep.e_local
    bf = lambda t: t.to(torch.bfloat16).to(dev)
    wr_full = torch.zeros(ROUTER_ROWS, d)
    wr_full[:E] = rnd((E, d), 1, 0.5)
    w1_all, b1_all = rnd((E, ff, d), 2, 0.08), rnd((E, ff), 3, 0.1)
    w2_all, b2_all = rnd((E, d, ff), 4, 0.08), rnd((E, d), 5, 0.1)
    x_all = [rnd((T, d), 10 + r, 1.0) for r in range(world)]
    gy_all = [rnd((T, d), 20 + r, 1.0) for r in range(world)]
    mine = slice(rank * el, (rank + 1) * el)

    for rep in range(2):                       # second pass reuses flags and buffers (epochs 5..8)
        tape = TensorTape(grad_dtype=None)
        tape.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
        ids = {}
        for name, t in (("x", x_all[rank]), ("wr", wr_full), ("w1", w1_all[mine]), ("b1", b1_all[mine]),
                        ("w2", w2_all[mine]), ("b2", b2_all[mine])):
            ids[name] = tape.leaf(bf(t).contiguous(), requires_grad=True, name=name)
        out = moe_ffn(tape, ids["x"], ids["wr"], ids["w1"], ids["b1"], ids["w2"], ids["b2"], ep, bufs)
        K.check_status()
        report = tape.backward(out, BackwardOptions(), seed=bf(gy_all[rank]))
        K.check_status()
        got = {n: report.gradient(i) for n, i in ids.items()}
        y = tape.value(out).float().cpu()

        # ---- reference: every rank's tokens through every expert, fp32 autograd
        P = {n: t.to(torch.bfloat16).float().requires_grad_(True) for n, t in
             (("wr", wr_full), ("w1", w1_all), ("b1", b1_all), ("w2", w2_all), ("b2", b2_all))}
        xs = [x.to(torch.bfloat16).float().requires_grad_(True) for x in x_all]
        outs = []
        for r in range(world):
            p = torch.softmax(xs[r] @ P["wr"][:E].t(), dim=-1)
            top = torch.topk(p, 2, dim=-1)
            gate = top.values / top.values.sum(-1, keepdim=True)
            flat = top.indices.reshape(-1).tolist()
            seen, keep = [0] * E, []
            for e in flat:
                keep.append(seen[e] < ep.capacity)
                seen[e] += 1
            keep = torch.tensor(keep).reshape(T, 2)
            o = torch.zeros(T, d)
            for k in range(2):
                for e in range(E):
                    sel = (top.indices[:, k] == e) & keep[:, k]
                    if sel.any():
                        hh = torch.nn.functional.gelu(xs[r][sel] @ P["w1"][e].t() + P["b1"][e], approximate="tanh")
                        o = o.index_put((sel.nonzero().squeeze(1),),
                                        gate[sel, k:k + 1] * (hh @ P["w2"][e].t() + P["b2"][e]), accumulate=True)
            outs.append(o)
        loss = sum((o * g.to(torch.bfloat16).float()).sum() for o, g in zip(outs, gy_all))
        loss.backward()

        def close(a, b, what, tol):
            a, b = a.float().cpu(), b.float().cpu()
            err = (a - b).abs().max().item()
            lim = tol * max(1.0, b.abs().max().item())
            assert err <= lim, f"rank {rank} rep {rep} {what}: max err {err} > {lim}"

        close(y, outs[rank].detach(), "forward", 3e-2)
        close(got["x"], xs[rank].grad, "dx", 4e-2)
        close(got["w1"], P["w1"].grad[mine], "dw1", 4e-2)
        close(got["b1"], P["b1"].grad[mine], "db1", 4e-2)
        close(got["w2"], P["w2"].grad[mine], "dw2", 4e-2)
        close(got["b2"], P["b2"].grad[mine], "db2", 4e-2)
        if world == 1:                          # the router weight gradient is a sum over ranks
            close(got["wr"][:E], P["wr"].grad[:E], "dwr", 5e-2)
    return True
