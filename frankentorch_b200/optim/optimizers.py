"""Optimizers (reference: ft-optim/src/lib.rs).

``Optimizer`` trait :226 - ``step(session, report)``, ``zero_grad``, ``get_lr/set_lr``,
``get_momentum/set_momentum``.  Optimizers read the tape's persistent accumulated gradients
(not the report, :919-931), so gradients accumulate across backward calls until ``zero_grad``.
Builder-style setters mirror the reference (``AdamW(params, lr).betas(..).weight_decay(..)``).
Math per optimizer: SGD :277 (momentum buffer seeded with the first gradient, dampening,
nesterov, L2 decay, maximize), Adam :518, AdamW :800-1085 (decoupled decay
``p -= p*lr*wd + lr*m_hat/(sqrt(v_hat)+eps)`` :1040-1054), RMSprop :1094, Adagrad :1377,
RAdam :1570, LBFGS :1829, Adamax :4541, Adadelta :4722, NAdam :4894, ASGD :5117, Rprop :5327,
SparseAdam :5519, Muon :5843 (Newton-Schulz orthogonalisation).

State tensors share the parameter's device; on CUDA parameters of bf16/fp32 dtype the AdamW
step is the fused sm_100a kernel (``ftk_adamw``), everything else is tensor arithmetic on the
session's storage layer.
"""
from __future__ import annotations

import enum
import math
from typing import Callable, Dict, List, Optional, Sequence

import torch


class Optimizer:
    def __init__(self, params: Sequence[int], lr: float):
        self.params = list(params)
        self.lr = float(lr)
        self.state: Dict[int, Dict[str, torch.Tensor]] = {p: {} for p in self.params}
        self.steps: Dict[int, int] = {p: 0 for p in self.params}
        self._maximize = False

    # builder-style configuration
    def maximize(self, flag: bool = True):
        self._maximize = flag
        return self

    def get_lr(self) -> float:
        return self.lr

    def set_lr(self, lr: float) -> None:
        self.lr = float(lr)

    def get_momentum(self) -> Optional[float]:
        return getattr(self, "_momentum", None)

    def set_momentum(self, momentum: float) -> None:
        if hasattr(self, "_momentum"):
            self._momentum = float(momentum)

    def zero_grad(self, session) -> None:
        session.tensor_zero_grads(self.params)

    def _grad(self, session, p: int) -> Optional[torch.Tensor]:
        g = session.tensor_tape.accumulated_gradient(p)
        if g is None:
            return None
        return -g if self._maximize else g

    def step(self, session, report=None) -> None:
        for p in self.params:
            g = self._grad(session, p)
            if g is None:
                continue
            self.steps[p] += 1
            w = session.tensor(p)
            self._update(p, w, g.to(torch.float64) if not w.is_cuda else g.to(torch.float32), self.steps[p])
            session.tensor_tape.bump_version(p)

    def _update(self, p: int, w: torch.Tensor, g: torch.Tensor, t: int) -> None:
        raise NotImplementedError

    def _st(self, p: int, key: str, like: torch.Tensor, init: float = 0.0) -> torch.Tensor:
        s = self.state[p]
        if key not in s:
            s[key] = torch.full_like(like, init)
        return s[key]

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self) -> Dict:
        return {"lr": self.lr, "steps": [self.steps[p] for p in self.params],
                "state": [{k: v.clone() for k, v in self.state[p].items()} for p in self.params],
                "hyper": {k: v for k, v in self.__dict__.items()
                          if k.startswith("_") and isinstance(v, (int, float, bool, tuple))}}

    def load_state_dict(self, sd: Dict) -> None:
        if len(sd["steps"]) != len(self.params):
            raise ValueError("optimizer state has a different number of parameters")
        self.lr = float(sd["lr"])
        for p, t, st in zip(self.params, sd["steps"], sd["state"]):
            self.steps[p] = max(0, int(t))     # saturating decode of the step counter
            self.state[p] = {k: v.clone() for k, v in st.items()}
        for k, v in sd.get("hyper", {}).items():
            setattr(self, k, v)


def _apply(w: torch.Tensor, new: torch.Tensor) -> None:
    w.copy_(new.to(w.dtype))


class SGD(Optimizer):
    def __init__(self, params, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False):
        super().__init__(params, lr)
        self._momentum, self._dampening, self._wd, self._nesterov = momentum, dampening, weight_decay, nesterov

    def momentum(self, v):
        self._momentum = v
        return self

    def dampening(self, v):
        self._dampening = v
        return self

    def weight_decay(self, v):
        self._wd = v
        return self

    def nesterov(self, flag=True):
        if flag and self._dampening != 0.0:
            raise ValueError("nesterov momentum requires zero dampening")
        self._nesterov = flag
        return self

    def _update(self, p, w, g, t):
        wf = w.to(g.dtype)
        if self._wd:
            g = g + self._wd * wf
        if self._momentum:
            if "buf" not in self.state[p]:
                self.state[p]["buf"] = g.clone()             # first step seeds the buffer with the raw gradient
            else:
                self.state[p]["buf"].mul_(self._momentum).add_(g, alpha=1 - self._dampening)
            buf = self.state[p]["buf"]
            g = g + self._momentum * buf if self._nesterov else buf
        _apply(w, wf - self.lr * g)


class Adam(Optimizer):
    decoupled = False

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False):
        super().__init__(params, lr)
        self._betas, self._eps, self._wd, self._amsgrad = tuple(betas), eps, weight_decay, amsgrad

    def betas(self, b1, b2=None):
        self._betas = (b1, b2) if b2 is not None else tuple(b1)
        return self

    def eps(self, v):
        self._eps = v
        return self

    def weight_decay(self, v):
        self._wd = v
        return self

    def amsgrad(self, flag=True):
        self._amsgrad = flag
        return self

    def _update(self, p, w, g, t):
        b1, b2 = self._betas
        if w.is_cuda and self.decoupled and not self._amsgrad and w.dtype in (torch.float32, torch.bfloat16):
            return self._update_fused(p, w, g, t)
        wf = w.to(g.dtype)
        if self._wd and not self.decoupled:
            g = g + self._wd * wf                              # L2 decay folded into the gradient
        m, v = self._st(p, "m", g), self._st(p, "v", g)
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = m / (1 - b1 ** t)
        if self._amsgrad:
            vmax = self._st(p, "vmax", g)
            torch.maximum(vmax, v, out=vmax)
            vh = vmax / (1 - b2 ** t)
        else:
            vh = v / (1 - b2 ** t)
        if self.decoupled:
            wf = wf - wf * self.lr * self._wd
        _apply(w, wf - self.lr * mh / (vh.sqrt() + self._eps))

    def _update_fused(self, p, w, g, t):
        from ..ops import kernels as K
        b1, b2 = self._betas
        st = self.state[p]
        if "master" not in st:
            st["master"] = w.detach().float().clone()
            st["m"] = torch.zeros_like(st["master"])
            st["v"] = torch.zeros_like(st["master"])
        K.adamw(st["master"].view(-1), w.view(-1) if w.dtype == torch.bfloat16 else None, g.contiguous().view(-1),
                st["m"].view(-1), st["v"].view(-1), lr=self.lr, beta1=b1, beta2=b2, eps=self._eps,
                weight_decay=self._wd, step=t)
        if w.dtype != torch.bfloat16:
            w.copy_(st["master"])


class AdamW(Adam):
    """Decoupled weight decay; defaults beta=(0.9, 0.999), eps=1e-8, wd=0.01 (ft-optim :800)."""

    decoupled = True

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=False):
        super().__init__(params, lr, betas, eps, weight_decay, amsgrad)


class RMSprop(Optimizer):
    def __init__(self, params, lr=1e-2, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False):
        super().__init__(params, lr)
        self._alpha, self._eps, self._wd, self._momentum, self._centered = alpha, eps, weight_decay, momentum, centered

    def _update(self, p, w, g, t):
        wf = w.to(g.dtype)
        if self._wd:
            g = g + self._wd * wf
        sq = self._st(p, "sq", g)
        sq.mul_(self._alpha).addcmul_(g, g, value=1 - self._alpha)
        if self._centered:
            ga = self._st(p, "gavg", g)
            ga.mul_(self._alpha).add_(g, alpha=1 - self._alpha)
            avg = (sq - ga * ga).sqrt() + self._eps
        else:
            avg = sq.sqrt() + self._eps
        if self._momentum:
            buf = self._st(p, "buf", g)
            buf.mul_(self._momentum).add_(g / avg)
            _apply(w, wf - self.lr * buf)
        else:
            _apply(w, wf - self.lr * g / avg)


class Adagrad(Optimizer):
    def __init__(self, params, lr=1e-2, lr_decay=0.0, weight_decay=0.0, initial_accumulator_value=0.0, eps=1e-10):
        super().__init__(params, lr)
        self._lr_decay, self._wd, self._init, self._eps = lr_decay, weight_decay, initial_accumulator_value, eps

    def _update(self, p, w, g, t):
        wf = w.to(g.dtype)
        if self._wd:
            g = g + self._wd * wf
        acc = self._st(p, "sum", g, self._init)
        acc.addcmul_(g, g)
        clr = self.lr / (1 + (t - 1) * self._lr_decay)
        _apply(w, wf - clr * g / (acc.sqrt() + self._eps))


class RAdam(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled_weight_decay=False):
        super().__init__(params, lr)
        self._betas, self._eps, self._wd, self._decoupled = tuple(betas), eps, weight_decay, bool(decoupled_weight_decay)

    def decoupled_weight_decay(self, flag: bool = True):
        """Decay the parameter directly (``w *= 1 - lr * wd``) instead of adding ``wd * w`` to the gradient."""
        self._decoupled = bool(flag)
        return self

    def _update(self, p, w, g, t):
        b1, b2 = self._betas
        wf = w.to(g.dtype)
        if self._wd:
            if self._decoupled:
                wf = wf * (1 - self.lr * self._wd)
            else:
                g = g + self._wd * wf
        m, v = self._st(p, "m", g), self._st(p, "v", g)
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = m / (1 - b1 ** t)
        rho_inf = 2 / (1 - b2) - 1
        rho = rho_inf - 2 * t * b2 ** t / (1 - b2 ** t)
        if rho > 5:
            vh = (v / (1 - b2 ** t)).sqrt()
            r = math.sqrt((rho - 4) * (rho - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho))
            _apply(w, wf - self.lr * mh * r / (vh + self._eps))
        else:
            _apply(w, wf - self.lr * mh)


class Adamax(Optimizer):
    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr)
        self._betas, self._eps, self._wd = tuple(betas), eps, weight_decay

    def _update(self, p, w, g, t):
        b1, b2 = self._betas
        wf = w.to(g.dtype)
        if self._wd:
            g = g + self._wd * wf
        m, u = self._st(p, "m", g), self._st(p, "u", g)
        m.mul_(b1).add_(g, alpha=1 - b1)
        torch.maximum(u * b2, g.abs() + self._eps, out=u)
        _apply(w, wf - (self.lr / (1 - b1 ** t)) * m / u)


class Adadelta(Optimizer):
    def __init__(self, params, lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0):
        super().__init__(params, lr)
        self._rho, self._eps, self._wd = rho, eps, weight_decay

    def _update(self, p, w, g, t):
        wf = w.to(g.dtype)
        if self._wd:
            g = g + self._wd * wf
        sq, acc = self._st(p, "sq", g), self._st(p, "acc", g)
        sq.mul_(self._rho).addcmul_(g, g, value=1 - self._rho)
        delta = (acc + self._eps).sqrt() / (sq + self._eps).sqrt() * g
        acc.mul_(self._rho).addcmul_(delta, delta, value=1 - self._rho)
        _apply(w, wf - self.lr * delta)


class NAdam(Optimizer):
    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, momentum_decay=4e-3,
                 decoupled_weight_decay=False):
        super().__init__(params, lr)
        self._betas, self._eps, self._wd, self._md = tuple(betas), eps, weight_decay, momentum_decay
        self._decoupled = bool(decoupled_weight_decay)
        self._mu_prod: Dict[int, float] = {}

    def decoupled_weight_decay(self, flag: bool = True):
        self._decoupled = bool(flag)
        return self

    def _update(self, p, w, g, t):
        b1, b2 = self._betas
        wf = w.to(g.dtype)
        if self._wd:
            if self._decoupled:
                wf = wf * (1 - self.lr * self._wd)
            else:
                g = g + self._wd * wf
        m, v = self._st(p, "m", g), self._st(p, "v", g)
        mu = b1 * (1 - 0.5 * 0.96 ** (t * self._md))
        mu_next = b1 * (1 - 0.5 * 0.96 ** ((t + 1) * self._md))
        prod = self._mu_prod.get(p, 1.0) * mu
        self._mu_prod[p] = prod
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        denom = (v / (1 - b2 ** t)).sqrt() + self._eps
        _apply(w, wf - self.lr * (1 - mu) / (1 - prod) * g / denom - self.lr * mu_next / (1 - prod * mu_next) * m / denom)


class ASGD(Optimizer):
    def __init__(self, params, lr=1e-2, lambd=1e-4, alpha=0.75, t0=1e6, weight_decay=0.0):
        super().__init__(params, lr)
        self._lambd, self._alpha, self._t0, self._wd = lambd, alpha, t0, weight_decay

    def _update(self, p, w, g, t):
        wf = w.to(g.dtype)
        st = self.state[p]
        eta = st.get("eta_f", self.lr)
        mu = st.get("mu_f", 1.0)
        if self._wd:
            g = g + self._wd * wf
        wf = wf * (1 - self._lambd * eta) - eta * g
        ax = self._st(p, "ax", g)
        if mu != 1.0:
            ax.add_((wf - ax) * mu)
        else:
            ax.copy_(wf)
        st["eta_f"] = self.lr / ((1 + self._lambd * self.lr * t) ** self._alpha)
        st["mu_f"] = 1.0 / max(1.0, t - self._t0)
        _apply(w, wf)

    def averaged_parameters(self) -> List[Optional[torch.Tensor]]:
        """The running averages ``ax`` of the parameters, in parameter order (``None`` before a parameter's first
        step); use them in place of the raw iterates once training is over."""
        return [self.state[p]["ax"].clone() if "ax" in self.state[p] else None for p in self.params]

    def state_dict(self):
        sd = super().state_dict()
        sd["state"] = [{k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in self.state[p].items()}
                       for p in self.params]
        return sd


class Rprop(Optimizer):
    def __init__(self, params, lr=1e-2, etas=(0.5, 1.2), step_sizes=(1e-6, 50.0)):
        super().__init__(params, lr)
        self._etas, self._sizes = tuple(etas), tuple(step_sizes)

    def _update(self, p, w, g, t):
        prev = self._st(p, "prev", g)
        step = self._st(p, "step", g, self.lr)
        sign = (g * prev).sign()
        step.mul_(torch.where(sign > 0, self._etas[1], torch.where(sign < 0, self._etas[0], 1.0)).to(step.dtype))
        step.clamp_(self._sizes[0], self._sizes[1])
        g = torch.where(sign < 0, torch.zeros_like(g), g)
        _apply(w, w.to(g.dtype) - g.sign() * step)
        prev.copy_(g)


class SparseAdam(Optimizer):
    """Adam that only touches the rows that received gradient (row-sparse embedding gradients)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8):
        super().__init__(params, lr)
        self._betas, self._eps = tuple(betas), eps

    def step(self, session, report=None) -> None:
        """Rows come from the tape's row-sparse accumulated gradient when the parameter was read
        through ``index_select_sparse`` / ``Embedding(sparse=True)`` (no dense gradient is ever
        formed, ft-optim/src/lib.rs:5519); a dense gradient is scanned for its non-zero rows."""
        tape = session.tensor_tape
        for p in self.params:
            sg = tape.accumulated_sparse_gradient(p)
            if sg is None:
                g = self._grad(session, p)
                if g is None:
                    continue
                g = g.to(torch.float64) if not g.is_cuda else g.to(torch.float32)
                rows = torch.nonzero(g.reshape(g.shape[0], -1).abs().sum(1) != 0).reshape(-1)
                vals = g[rows]
            else:
                rows = sg.rows
                vals = sg.values.to(torch.float64) if not sg.values.is_cuda else sg.values.to(torch.float32)
                if self._maximize:
                    vals = -vals
            self.steps[p] += 1
            self._update_rows(p, session.tensor(p), rows, vals, self.steps[p])
            tape.bump_version(p)

    def _update_rows(self, p, w, rows, gm, t):
        b1, b2 = self._betas
        if rows.numel() == 0:
            return
        st = self.state[p]
        if "m" not in st:
            st["m"] = torch.zeros(w.shape, dtype=gm.dtype, device=w.device)
            st["v"] = torch.zeros(w.shape, dtype=gm.dtype, device=w.device)
        m, v = st["m"], st["v"]
        m[rows] = b1 * m[rows] + (1 - b1) * gm
        v[rows] = b2 * v[rows] + (1 - b2) * gm * gm
        upd = (m[rows] / (1 - b1 ** t)) / ((v[rows] / (1 - b2 ** t)).sqrt() + self._eps)
        w[rows] = (w[rows].to(gm.dtype) - self.lr * upd).to(w.dtype)      # only the touched rows are rewritten


class Muon(Optimizer):
    """Momentum + Newton-Schulz orthogonalisation of 2-D updates (ft-optim :5843)."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0):
        super().__init__(params, lr)
        self._momentum, self._nesterov, self._ns, self._wd = momentum, nesterov, ns_steps, weight_decay

    @staticmethod
    def newton_schulz(g: torch.Tensor, steps: int) -> torch.Tensor:
        a, b, c = 3.4445, -4.7750, 2.0315
        x = g / (g.norm() + 1e-7)
        tr = x.shape[0] > x.shape[1]
        if tr:
            x = x.t()
        for _ in range(steps):
            A = x @ x.t()
            x = a * x + (b * A + c * A @ A) @ x
        return x.t() if tr else x

    def _update(self, p, w, g, t):
        buf = self._st(p, "buf", g)
        buf.mul_(self._momentum).add_(g)
        u = g + self._momentum * buf if self._nesterov else buf
        wf = w.to(g.dtype)
        if u.dim() == 2:
            u = self.newton_schulz(u, self._ns) * max(1.0, u.shape[0] / u.shape[1]) ** 0.5
        if self._wd:
            wf = wf * (1 - self.lr * self._wd)
        _apply(w, wf - self.lr * u)


class LBFGSLineSearch(enum.Enum):
    """Step-length rule of :class:`LBFGS` (ft-optim/src/lib.rs:1818)."""
    NoSearch = "none"                       # the reference's ``None`` variant: a fixed step of ``lr``
    BacktrackingArmijo = "backtracking_armijo"
    StrongWolfe = "strong_wolfe"

    @staticmethod
    def parse(v) -> "LBFGSLineSearch":
        if isinstance(v, LBFGSLineSearch):
            return v
        if v is None:
            return LBFGSLineSearch.NoSearch
        key = str(v).lower()
        alias = {"none": "none", "backtracking": "backtracking_armijo", "armijo": "backtracking_armijo",
                 "backtracking_armijo": "backtracking_armijo", "strong_wolfe": "strong_wolfe"}
        if key not in alias:
            raise ValueError(f"unknown LBFGS line search {v!r}")
        return LBFGSLineSearch(alias[key])


class LBFGS(Optimizer):
    """Limited-memory BFGS (ft-optim :1829) with a fixed step, a backtracking Armijo search, or a strong-Wolfe
    search (bracketing, then a zoom phase with safeguarded cubic interpolation; c1 = 1e-4, c2 = 0.9)."""

    def __init__(self, params, lr=1.0, max_iter=20, history_size=100, tolerance_grad=1e-7, tolerance_change=1e-9,
                 line_search: Optional[str] = None, max_eval: Optional[int] = None):
        super().__init__(params, lr)
        self.max_iter, self.history, self.tol_g, self.tol_c, self.line_search = max_iter, history_size, tolerance_grad, tolerance_change, line_search
        self.max_eval = max_eval if max_eval is not None else max_iter * 5 // 4      # closure evaluations per step()
        self.n_evals = 0
        self._s: List[torch.Tensor] = []
        self._y: List[torch.Tensor] = []

    def _flat(self, session, grads: bool):
        out = []
        for p in self.params:
            t = session.tensor_tape.accumulated_gradient(p) if grads else session.tensor(p)
            out.append(torch.zeros(session.tensor_numel(p), dtype=torch.float64) if t is None else t.detach().reshape(-1).to(torch.float64))
        return torch.cat(out)

    def _set(self, session, flat):
        off = 0
        for p in self.params:
            n = session.tensor_numel(p)
            session.tensor_update_param_values(p, flat[off: off + n])
            off += n

    def _phi(self, session, closure, x0, d, t):
        """Loss and directional derivative at ``x0 + t d`` (leaves the parameters there)."""
        self._set(session, x0 + t * d)
        f = float(closure())
        return f, float(self._flat(session, True) @ d)

    @staticmethod
    def _cubic_min(a, fa, ga, b, fb, gb):
        """Minimiser of the cubic through (a, fa, ga), (b, fb, gb), kept inside the middle 80 % of the interval."""
        lo, hi = (a, b) if a <= b else (b, a)
        d1 = ga + gb - 3 * (fa - fb) / (a - b)
        sq = d1 * d1 - ga * gb
        if sq >= 0:
            d2 = math.sqrt(sq)
            t = b - (b - a) * ((gb + d2 - d1) / (gb - ga + 2 * d2)) if a <= b else a - (a - b) * ((ga + d2 - d1) / (ga - gb + 2 * d2))
        else:
            t = 0.5 * (lo + hi)
        return min(max(t, lo + 0.1 * (hi - lo)), hi - 0.1 * (hi - lo))

    def _strong_wolfe(self, session, closure, x0, d, f0, g0, t, c1=1e-4, c2=0.9, max_ls=25):
        """Step ``t`` with ``f(t) <= f0 + c1 t g0`` and ``|g(t)| <= c2 |g0|``; returns ``(t, f(t))`` with the
        parameters (and their gradients) left at that point."""
        if g0 >= 0:                       # not a descent direction: take no step
            self._set(session, x0)
            return 0.0, float(closure())
        t_prev, f_prev, g_prev = 0.0, f0, g0
        bracket = None
        for it in range(max_ls):
            f, gt = self._phi(session, closure, x0, d, t)
            if f > f0 + c1 * t * g0 or (it > 0 and f >= f_prev):
                bracket = (t_prev, f_prev, g_prev, t, f, gt)
                break
            if abs(gt) <= -c2 * g0:
                return t, f
            if gt >= 0:
                bracket = (t, f, gt, t_prev, f_prev, g_prev)
                break
            t_prev, f_prev, g_prev, t = t, f, gt, t * 2.0
        if bracket is None:
            return t_prev, self._phi(session, closure, x0, d, t_prev)[0]
        lo, f_lo, g_lo, hi, f_hi, g_hi = bracket
        for _ in range(max_ls):
            if abs(hi - lo) < 1e-12:
                break
            t = self._cubic_min(lo, f_lo, g_lo, hi, f_hi, g_hi)
            f, gt = self._phi(session, closure, x0, d, t)
            if f > f0 + c1 * t * g0 or f >= f_lo:
                hi, f_hi, g_hi = t, f, gt
            else:
                if abs(gt) <= -c2 * g0:
                    return t, f
                if gt * (hi - lo) >= 0:
                    hi, f_hi, g_hi = lo, f_lo, g_lo
                lo, f_lo, g_lo = t, f, gt
        return lo, self._phi(session, closure, x0, d, lo)[0]

    def line_search_fn(self, ls):
        self.line_search = ls
        return self

    def step_with_closure(self, session, closure: Callable[[], float]) -> float:
        return self.step(session, closure)

    def step(self, session, closure: Callable[[], float]) -> float:
        """``closure`` zeroes the gradients, runs forward + backward and returns the loss value.  Iterates until
        ``max_iter`` directions were taken, ``max_eval`` closure evaluations were spent, or a tolerance is met."""
        evals = [0]
        inner = closure

        def closure():                                   # noqa: F811  (counts evaluations of the user's closure)
            evals[0] += 1
            self.n_evals += 1
            return inner()
        loss = float(closure())
        g = self._flat(session, True)
        for _ in range(self.max_iter):
            if float(g.abs().max()) <= self.tol_g or evals[0] >= self.max_eval:
                break
            q, alphas = g.clone(), []
            for s, y in zip(reversed(self._s), reversed(self._y)):
                a = float(s @ q) / float(y @ s)
                alphas.append(a)
                q -= a * y
            if self._s:
                q *= float(self._s[-1] @ self._y[-1]) / float(self._y[-1] @ self._y[-1])
            for (s, y), a in zip(zip(self._s, self._y), reversed(alphas)):
                q += (a - float(y @ q) / float(y @ s)) * s
            d = -q
            x0, t = self._flat(session, False), self.lr
            ls = LBFGSLineSearch.parse(self.line_search)
            if ls is LBFGSLineSearch.BacktrackingArmijo:
                gd = float(g @ d)
                for _ls in range(20):
                    self._set(session, x0 + t * d)
                    new_loss = float(closure())
                    if new_loss <= loss + 1e-4 * t * gd:
                        break
                    t *= 0.5
            elif ls is LBFGSLineSearch.StrongWolfe:
                t, new_loss = self._strong_wolfe(session, closure, x0, d, loss, float(g @ d), t)
            else:
                self._set(session, x0 + t * d)
                new_loss = float(closure())
            g_new = self._flat(session, True)
            s, y = t * d, g_new - g
            if float(y @ s) > 1e-10:
                self._s.append(s)
                self._y.append(y)
                if len(self._s) > self.history:
                    self._s.pop(0)
                    self._y.pop(0)
            if abs(new_loss - loss) < self.tol_c:
                loss, g = new_loss, g_new
                break
            loss, g = new_loss, g_new
        return loss
