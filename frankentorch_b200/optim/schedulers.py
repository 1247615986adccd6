"""Learning-rate schedulers and the AMP gradient scaler.

Reference: ft-optim/src/lib.rs - ``LRScheduler`` trait :2315-2342 (``step(optimizer, metric)``,
``get_last_lr``, ``state``/``load_state``), ``SchedulerState{last_epoch,last_lrs,extra}`` :2301,
the fifteen schedulers :2351-4471, ``GradScaler`` :6093-6264 (init scale 65536, growth 2.0,
backoff 0.5, growth interval 2000; inf/nan check over the accumulated gradients -> skip the
step and back off, else unscale in place and step).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch


@dataclass
class SchedulerState:
    last_epoch: int = 0
    last_lrs: List[float] = field(default_factory=list)
    extra: Dict[str, float] = field(default_factory=dict)


class LRScheduler:
    def __init__(self, optimizer):
        self.base_lr = optimizer.get_lr()
        self.last_epoch = 0
        self.last_lr = self.base_lr

    def _lr_at(self, epoch: int) -> float:
        raise NotImplementedError

    def step(self, optimizer, metric: Optional[float] = None) -> float:
        self.last_epoch += 1
        self.last_lr = self._lr_at(self.last_epoch)
        optimizer.set_lr(self.last_lr)
        return self.last_lr

    def get_last_lr(self) -> List[float]:
        return [self.last_lr]

    def state(self) -> SchedulerState:
        return SchedulerState(self.last_epoch, [self.last_lr], {"base_lr": self.base_lr})

    def load_state(self, st: SchedulerState) -> None:
        self.last_epoch = int(st.last_epoch)
        self.last_lr = st.last_lrs[0] if st.last_lrs else self.base_lr
        self.base_lr = st.extra.get("base_lr", self.base_lr)


class StepLR(LRScheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1):
        super().__init__(optimizer)
        if step_size <= 0:
            raise ValueError("step_size must be positive")
        self.step_size, self.gamma = step_size, gamma

    def _lr_at(self, e):
        return self.base_lr * self.gamma ** (e // self.step_size)


class MultiStepLR(LRScheduler):
    def __init__(self, optimizer, milestones: Sequence[int], gamma: float = 0.1):
        super().__init__(optimizer)
        self.milestones, self.gamma = sorted(milestones), gamma

    def _lr_at(self, e):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if m <= e)


class ConstantLR(LRScheduler):
    def __init__(self, optimizer, factor: float = 1.0 / 3, total_iters: int = 5):
        super().__init__(optimizer)
        self.factor, self.total = factor, total_iters
        optimizer.set_lr(self.base_lr * factor)
        self.last_lr = self.base_lr * factor

    def _lr_at(self, e):
        return self.base_lr * (self.factor if e < self.total else 1.0)


class LinearLR(LRScheduler):
    def __init__(self, optimizer, start_factor: float = 1.0 / 3, end_factor: float = 1.0, total_iters: int = 5):
        super().__init__(optimizer)
        self.sf, self.ef, self.total = start_factor, end_factor, total_iters
        optimizer.set_lr(self.base_lr * start_factor)
        self.last_lr = self.base_lr * start_factor

    def _lr_at(self, e):
        f = self.sf + (self.ef - self.sf) * min(e, self.total) / self.total
        return self.base_lr * f


class ExponentialLR(LRScheduler):
    def __init__(self, optimizer, gamma: float):
        super().__init__(optimizer)
        self.gamma = gamma

    def _lr_at(self, e):
        return self.base_lr * self.gamma ** e


class PolynomialLR(LRScheduler):
    def __init__(self, optimizer, total_iters: int = 5, power: float = 1.0):
        super().__init__(optimizer)
        self.total, self.power = total_iters, power

    def _lr_at(self, e):
        return self.base_lr * (1 - min(e, self.total) / self.total) ** self.power


class CosineAnnealingLR(LRScheduler):
    def __init__(self, optimizer, T_max: int, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.T_max, self.eta_min = T_max, eta_min

    def _lr_at(self, e):
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * e / self.T_max)) / 2


class CosineAnnealingWarmRestarts(LRScheduler):
    def __init__(self, optimizer, T_0: int, T_mult: int = 1, eta_min: float = 0.0):
        super().__init__(optimizer)
        if T_0 <= 0 or T_mult < 1:
            raise ValueError("T_0 must be positive and T_mult >= 1")
        self.T_0, self.T_mult, self.eta_min = T_0, T_mult, eta_min

    def t_mult(self, t_mult: int) -> "CosineAnnealingWarmRestarts":
        """Builder form (ft-optim/src/lib.rs:2802): growth factor of the cycle length, at least 1."""
        self.T_mult = max(int(t_mult), 1)
        return self

    def with_eta_min(self, eta_min: float) -> "CosineAnnealingWarmRestarts":
        """Builder form (ft-optim/src/lib.rs:2809): the floor of the schedule; a negative or non-finite value
        is taken as 0."""
        self.eta_min = float(eta_min) if math.isfinite(eta_min) and eta_min >= 0.0 else 0.0
        return self

    def _lr_at(self, e):
        t_i, t_cur = self.T_0, e
        while t_cur >= t_i:
            t_cur -= t_i
            t_i *= self.T_mult
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * t_cur / t_i)) / 2


class LambdaLR(LRScheduler):
    def __init__(self, optimizer, lr_lambda: Callable[[int], float]):
        super().__init__(optimizer)
        self.fn = lr_lambda

    def _lr_at(self, e):
        return self.base_lr * self.fn(e)


class MultiplicativeLR(LRScheduler):
    def __init__(self, optimizer, lr_lambda: Callable[[int], float]):
        super().__init__(optimizer)
        self.fn = lr_lambda

    def step(self, optimizer, metric=None):
        self.last_epoch += 1
        self.last_lr = self.last_lr * self.fn(self.last_epoch)
        optimizer.set_lr(self.last_lr)
        return self.last_lr


class OneCycleLR(LRScheduler):
    """One-cycle policy (ft-optim/src/lib.rs:3798-4030).  Two phases (warm-up to ``max_lr``, anneal to the final
    rate) or, with ``three_phase``, three (up, back down to the initial rate, then down to the final rate).  The
    phase boundaries are the real numbers ``pct_start * total - 1`` and ``2 * pct_start * total - 2`` over steps
    ``0 .. total - 1``.  With ``cycle_momentum`` the optimizer's momentum moves against the rate between
    ``max_momentum`` and ``base_momentum``.  ``step(optimizer, epoch=k)`` jumps to step ``k``."""

    def __init__(self, optimizer, max_lr: float, total_steps: int, pct_start: float = 0.3, div_factor: float = 25.0,
                 final_div_factor: float = 1e4, anneal: str = "cos", three_phase: bool = False,
                 cycle_momentum: bool = False, base_momentum: float = 0.85, max_momentum: float = 0.95):
        super().__init__(optimizer)
        if total_steps <= 0:
            raise ValueError("total_steps must be positive")
        if not 0.0 <= pct_start <= 1.0:
            raise ValueError("pct_start must lie in [0, 1]")
        if anneal not in ("cos", "linear"):
            raise ValueError("anneal must be 'cos' or 'linear'")
        self.max_lr, self.total, self.pct = max_lr, total_steps, pct_start
        self.div_factor, self.final_div_factor = div_factor, final_div_factor
        self.anneal = anneal
        self._three_phase, self._cycle_momentum = bool(three_phase), bool(cycle_momentum)
        self._base_momentum, self._max_momentum = float(base_momentum), float(max_momentum)
        self.last_momentum: Optional[float] = None
        optimizer.set_lr(self.initial)
        self.last_lr = self.initial
        if self._cycle_momentum:
            self._apply_momentum(optimizer, self._max_momentum)

    initial = property(lambda self: self.max_lr / self.div_factor)
    min_lr = property(lambda self: self.max_lr / self.div_factor / self.final_div_factor)

    # builder-style options
    def three_phase(self, flag: bool = True):
        self._three_phase = bool(flag)
        return self

    def cycle_momentum(self, flag: bool = True):
        self._cycle_momentum = bool(flag)
        return self

    def base_momentum(self, v: float):
        self._base_momentum = float(v)
        return self

    def max_momentum(self, v: float):
        self._max_momentum = float(v)
        return self

    def anneal_strategy_cos(self):
        self.anneal = "cos"
        return self

    def anneal_strategy_linear(self):
        self.anneal = "linear"
        return self

    def get_last_momentum(self) -> Optional[float]:
        return self.last_momentum

    def _apply_momentum(self, optimizer, m: float) -> None:
        if optimizer.get_momentum() is None:
            raise ValueError("cycle_momentum needs an optimizer with a momentum (SGD momentum, Adam-family beta1)")
        optimizer.set_momentum(m)
        self.last_momentum = m

    def _interp(self, a, b, pct):
        pct = min(max(pct, 0.0), 1.0)
        if self.anneal == "cos":
            return b + (a - b) * (1 + math.cos(math.pi * pct)) / 2
        return a + (b - a) * pct

    def _phases(self):
        """``(end_step, start_lr, end_lr, start_momentum, end_momentum)`` per phase."""
        t, hi_m, lo_m = float(self.total), self._max_momentum, self._base_momentum
        if self._three_phase:
            return [(self.pct * t - 1, self.initial, self.max_lr, hi_m, lo_m),
                    (2 * self.pct * t - 2, self.max_lr, self.initial, lo_m, hi_m),
                    (t - 1, self.initial, self.min_lr, hi_m, hi_m)]
        return [(self.pct * t - 1, self.initial, self.max_lr, hi_m, lo_m), (t - 1, self.max_lr, self.min_lr, lo_m, hi_m)]

    def _values_at(self, e: int):
        phases, start = self._phases(), 0.0
        for k, (end, lr_a, lr_b, m_a, m_b) in enumerate(phases):
            if e <= end or k == len(phases) - 1:
                pct = 0.0 if end == start else (e - start) / (end - start)      # a zero-width phase pins to its start
                return self._interp(lr_a, lr_b, pct), (self._interp(m_a, m_b, pct) if self._cycle_momentum else None)
            start = end
        return self.initial, None

    def _lr_at(self, e):
        if e > self.total:
            raise ValueError("OneCycleLR stepped past total_steps")
        return self._values_at(e)[0]

    def step(self, optimizer, metric=None, epoch: Optional[int] = None) -> float:
        self.last_epoch = self.last_epoch + 1 if epoch is None else int(epoch)
        if self.last_epoch > self.total:
            raise ValueError("OneCycleLR stepped past total_steps")
        self.last_lr, m = self._values_at(max(self.last_epoch, 0))
        optimizer.set_lr(self.last_lr)
        if m is not None:
            self._apply_momentum(optimizer, m)
        return self.last_lr

    def state(self):
        st = super().state()
        st.extra.update(max_lr=self.max_lr, total=self.total, pct=self.pct, div_factor=self.div_factor,
                        final_div_factor=self.final_div_factor, anneal=self.anneal, three_phase=self._three_phase,
                        cycle_momentum=self._cycle_momentum, base_momentum=self._base_momentum,
                        max_momentum=self._max_momentum, last_momentum=self.last_momentum)
        return st

    def load_state(self, st):
        super().load_state(st)
        x = st.extra
        self.max_lr, self.total, self.pct = x.get("max_lr", self.max_lr), int(x.get("total", self.total)), x.get("pct", self.pct)
        self.div_factor, self.final_div_factor = x.get("div_factor", self.div_factor), x.get("final_div_factor", self.final_div_factor)
        self.anneal = x.get("anneal", self.anneal)
        self._three_phase, self._cycle_momentum = bool(x.get("three_phase", self._three_phase)), bool(x.get("cycle_momentum", self._cycle_momentum))
        self._base_momentum, self._max_momentum = x.get("base_momentum", self._base_momentum), x.get("max_momentum", self._max_momentum)
        self.last_momentum = x.get("last_momentum", self.last_momentum)


class CyclicLRMode:
    """Amplitude policy of :class:`CyclicLR` (ft-optim/src/lib.rs:4381): ``Triangular`` (constant), ``Triangular2``
    (halved every cycle) or ``ExpRange(gamma)`` (scaled by ``gamma ** iteration``)."""

    def __init__(self, name: str, gamma: float = 1.0):
        if name not in ("triangular", "triangular2", "exp_range"):
            raise ValueError(f"unknown CyclicLR mode {name!r}")
        self.name, self.gamma = name, float(gamma)

    @staticmethod
    def ExpRange(gamma: float) -> "CyclicLRMode":
        return CyclicLRMode("exp_range", gamma)

    def scale(self, cycle: int, iteration: int) -> float:
        return {"triangular": 1.0, "triangular2": 1.0 / (2 ** (cycle - 1)), "exp_range": self.gamma ** iteration}[self.name]

    def __eq__(self, other):
        return isinstance(other, CyclicLRMode) and (other.name, other.gamma) == (self.name, self.gamma)

    def __repr__(self):
        return f"CyclicLRMode.ExpRange(gamma={self.gamma})" if self.name == "exp_range" else f"CyclicLRMode.{self.name.title()}"


CyclicLRMode.Triangular = CyclicLRMode("triangular")
CyclicLRMode.Triangular2 = CyclicLRMode("triangular2")


class CyclicLR(LRScheduler):
    def __init__(self, optimizer, base_lr: float, max_lr: float, step_size_up: int = 2000,
                 step_size_down: Optional[int] = None, mode="triangular", gamma: float = 1.0,
                 cycle_momentum: bool = False, base_momentum: float = 0.8, max_momentum: float = 0.9):
        super().__init__(optimizer)
        self.lo, self.hi, self.up, self.down = base_lr, max_lr, step_size_up, step_size_down or step_size_up
        self.policy = mode if isinstance(mode, CyclicLRMode) else CyclicLRMode(mode, gamma)
        self.mode, self.gamma = self.policy.name, self.policy.gamma
        self._cycle_momentum, self._base_momentum, self._max_momentum = bool(cycle_momentum), float(base_momentum), float(max_momentum)
        self.last_momentum: Optional[float] = None
        optimizer.set_lr(base_lr)
        self.last_lr = base_lr
        if self._cycle_momentum:
            if optimizer.get_momentum() is None:
                raise ValueError("cycle_momentum needs an optimizer with a momentum")
            optimizer.set_momentum(self._max_momentum)
            self.last_momentum = self._max_momentum

    def cycle_momentum(self, flag: bool = True):
        self._cycle_momentum = bool(flag)
        return self

    def base_momentum(self, v: float):
        self._base_momentum = float(v)
        return self

    def max_momentum(self, v: float):
        self._max_momentum = float(v)
        return self

    def get_last_momentum(self) -> Optional[float]:
        return self.last_momentum

    def _position(self, e):
        total = self.up + self.down
        cycle = math.floor(1 + e / total)
        x = 1 + e / total - cycle
        pos = x / (self.up / total) if x <= self.up / total else (x - 1) / (self.up / total - 1)
        return pos * self.policy.scale(cycle, e)

    def _lr_at(self, e):
        return self.lo + (self.hi - self.lo) * self._position(e)

    def step(self, optimizer, metric=None) -> float:
        lr = super().step(optimizer, metric)
        if self._cycle_momentum:      # the momentum runs against the rate: highest where the rate is lowest
            self.last_momentum = self._max_momentum - (self._max_momentum - self._base_momentum) * self._position(self.last_epoch)
            optimizer.set_momentum(self.last_momentum)
        return lr


class ReduceLROnPlateau(LRScheduler):
    def __init__(self, optimizer, mode: str = "min", factor: float = 0.1, patience: int = 10, threshold: float = 1e-4,
                 cooldown: int = 0, min_lr: float = 0.0, threshold_mode: str = "rel"):
        super().__init__(optimizer)
        if mode not in ("min", "max") or threshold_mode not in ("rel", "abs"):
            raise ValueError("mode must be 'min' or 'max' and threshold_mode 'rel' or 'abs'")
        if factor >= 1.0:
            raise ValueError("factor must be below 1")
        self.mode, self.factor, self.patience, self.threshold, self.cooldown, self.min_lr = mode, factor, patience, threshold, cooldown, min_lr
        self.threshold_mode = threshold_mode
        self.best = math.inf if mode == "min" else -math.inf
        self.bad, self.cool = 0, 0

    # builder-style options (ft-optim/src/lib.rs ReduceLROnPlateau)
    def mode_min(self):
        self.mode, self.best = "min", math.inf
        return self

    def mode_max(self):
        self.mode, self.best = "max", -math.inf
        return self

    def threshold_mode_rel(self):
        self.threshold_mode = "rel"
        return self

    def threshold_mode_abs(self):
        self.threshold_mode = "abs"
        return self

    def _is_better(self, metric: float) -> bool:
        if self.threshold_mode == "rel":
            return metric < self.best * (1 - self.threshold) if self.mode == "min" else metric > self.best * (1 + self.threshold)
        return metric < self.best - self.threshold if self.mode == "min" else metric > self.best + self.threshold

    def step(self, optimizer, metric: Optional[float] = None) -> float:
        if metric is None:
            raise ValueError("ReduceLROnPlateau.step needs the monitored metric")
        self.last_epoch += 1
        if self._is_better(metric):
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
        if self.cool > 0:
            self.cool -= 1
            self.bad = 0
        if self.bad > self.patience:
            self.last_lr = max(self.last_lr * self.factor, self.min_lr)
            optimizer.set_lr(self.last_lr)
            self.cool, self.bad = self.cooldown, 0
        return self.last_lr

    def state(self):
        st = super().state()
        st.extra.update(best=self.best, bad=self.bad, cool=self.cool)
        return st

    def load_state(self, st):
        super().load_state(st)
        self.best, self.bad, self.cool = st.extra.get("best", self.best), int(st.extra.get("bad", 0)), int(st.extra.get("cool", 0))


class SequentialLR(LRScheduler):
    def __init__(self, optimizer, schedulers: Sequence[LRScheduler], milestones: Sequence[int]):
        super().__init__(optimizer)
        if len(milestones) != len(schedulers) - 1:
            raise ValueError("SequentialLR needs len(schedulers) - 1 milestones")
        self.scheds, self.milestones = list(schedulers), list(milestones)

    def step(self, optimizer, metric=None):
        self.last_epoch += 1
        idx = sum(1 for m in self.milestones if m <= self.last_epoch)
        s = self.scheds[idx]
        if idx > 0 and self.last_epoch == self.milestones[idx - 1]:
            s.last_epoch = 0
            self.last_lr = s._lr_at(0) if not isinstance(s, (MultiplicativeLR, ReduceLROnPlateau)) else s.last_lr
            optimizer.set_lr(self.last_lr)
        else:
            self.last_lr = s.step(optimizer, metric)
        return self.last_lr


class ChainedScheduler(LRScheduler):
    """Applies every scheduler's multiplicative change in turn."""

    def __init__(self, optimizer, schedulers: Sequence[LRScheduler]):
        super().__init__(optimizer)
        self.scheds = list(schedulers)

    def step(self, optimizer, metric=None):
        self.last_epoch += 1
        lr = optimizer.get_lr()
        for s in self.scheds:
            prev = s.last_lr
            new = s.step(optimizer, metric)
            lr = lr * (new / prev if prev else 1.0)
        self.last_lr = lr
        optimizer.set_lr(lr)
        return lr


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self.scale, self.growth, self.backoff, self.interval, self.enabled = init_scale, growth_factor, backoff_factor, growth_interval, enabled
        self._good_steps = 0
        self._found_inf = False
        self._last_skipped = False

    @staticmethod
    def with_config(init_scale: float, growth_factor: float, backoff_factor: float, growth_interval: int) -> "GradScaler":
        """Explicit parameters (ft-optim/src/lib.rs:6128); the scaler starts enabled."""
        return GradScaler(init_scale, growth_factor, backoff_factor, growth_interval, True)

    def enable(self) -> None:
        self.enabled = True

    def disable(self) -> None:
        """Scaling off: ``scale_loss`` returns the loss itself and ``step`` always steps."""
        self.enabled = False

    def is_enabled(self) -> bool:
        return self.enabled

    def last_step_was_skipped(self) -> bool:
        """Whether the latest ``step`` found a non-finite gradient and left the parameters untouched."""
        return self._last_skipped

    def get_scale(self) -> float:
        return self.scale

    def scale_loss(self, session, loss: int) -> int:
        return session.tensor_mul_scalar(loss, c=self.scale) if self.enabled else loss

    def unscale_(self, session, optimizer) -> bool:
        """Divide the accumulated gradients by the scale in place; returns True if all are finite."""
        self._found_inf = False
        for p in optimizer.params:
            g = session.tensor_tape.accumulated_gradient(p)
            if g is None:
                continue
            if not bool(torch.isfinite(g).all()):
                self._found_inf = True
        if not self._found_inf:
            for p in optimizer.params:
                g = session.tensor_tape.accumulated_gradient(p)
                if g is not None:
                    g.div_(self.scale)
        return not self._found_inf

    def step(self, session, optimizer, report=None) -> bool:
        """Unscale and step; skips the step (returns False) when an inf/nan gradient was found."""
        if not self.enabled:
            optimizer.step(session, report)
            self._last_skipped = False
            return True
        if self.unscale_(session, optimizer):
            optimizer.step(session, report)
            self._last_skipped = False
            return True
        self._last_skipped = True
        return False

    def update(self) -> None:
        if not self.enabled:
            return
        if self._found_inf:
            self.scale *= self.backoff
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self._good_steps >= self.interval:
                self.scale *= self.growth
                self._good_steps = 0
        self._found_inf = False

    def state_dict(self):
        return {"scale": self.scale, "good_steps": self._good_steps}

    def load_state_dict(self, sd):
        self.scale, self._good_steps = float(sd["scale"]), int(sd["good_steps"])
