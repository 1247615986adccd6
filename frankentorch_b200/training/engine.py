"""Training engine: one optimizer step of a tape-recorded model, captured in a CUDA graph.

Per step the engine (1) copies the step's token ids / targets from pinned host memory
into static device buffers, (2) replays the captured graph (forward through the DAC
tape, deterministic backward in scheduler order, gradient clipping, fused AdamW on the
flat parameter arena) and (3) reads the loss back to the host.  The tape is recorded
once, at capture time; replaying the graph re-executes exactly the recorded kernel
sequence, which is what makes the step replayable bit for bit.

With more than one rank the gradient reduction + sharded AdamW + parameter all-gather
are delegated to :mod:`frankentorch_b200.parallel` (in-kernel peer loads/stores over
NVLink); the single-GPU path uses the plain fused AdamW kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..autograd.tape import BackwardOptions
from ..ops import kernels as K
from ..utils.profiling import install_tape_ranges


@dataclass
class OptimConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01      # AdamW defaults of the reference, ft-optim/src/lib.rs:800
    grad_clip: Optional[float] = 1.0


class TrainEngine:
    def __init__(self, model, micro_batch: int, seq_len: int, optim: Optional[OptimConfig] = None, *,
                 use_cuda_graph: bool = True, dp=None, ledger=None):
        self.model = model
        self.tape = model.tape
        install_tape_ranges(self.tape)       # NVTX range per backward rule when FT_NVTX=1
        self.B, self.S = micro_batch, seq_len
        self.opt = optim or OptimConfig()
        self.dp = dp
        if dp is not None and hasattr(dp, "attach"):
            dp.attach(self.tape, getattr(model, "leaf", {}))
        self._wire_param_gates()
        dev = model.device
        self.ids = torch.zeros((micro_batch, seq_len), dtype=torch.int64, device=dev)
        self.targets = torch.zeros((micro_batch, seq_len), dtype=torch.int64, device=dev)
        self.loss_dev = torch.zeros((), dtype=torch.float32, device=dev)
        self.loss_host = torch.zeros((), dtype=torch.float32).pin_memory()
        self.hyper = torch.tensor([self.opt.lr, 1.0, 1.0, 1.0], dtype=torch.float32, device=dev)
        self.lr_host = torch.tensor([self.opt.lr], dtype=torch.float32).pin_memory()
        self.step_dev = torch.zeros((), dtype=torch.int64, device=dev)
        # rank-local parameter shards (tensor / expert parallel models) use their own hyper vector:
        # the same step and clip factor with the model's gradient scale folded in
        self.local_arenas = list(getattr(model, "local_arenas", []))
        self.local_grad_scale = float(getattr(model, "local_grad_scale", 1.0))
        self.hyper_local = self.hyper.clone()
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.local_sumsq = torch.zeros(1, dtype=torch.float32, device=dev)   # squared norm of rank-local gradients
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        # library collectives (the NCCL baseline path) stay out of graph capture
        self._graph_requested = use_cuda_graph
        self.use_graph = use_cuda_graph and not getattr(dp, "eager_only", False)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0
        self.last_report = None
        self.steps_done = 0
        # evidence ledger of the GPU path: the first step that runs eagerly (the one before graph capture, or
        # the first step of an eager engine) is observed and written down once, see training/step_ledger.py
        self.ledger = ledger
        self._ledger_done = ledger is None

    def _wire_param_gates(self) -> None:
        """A model with a ``param_gate`` slot tells the data-parallel object which parameters its
        forward pass is about to read, so a deferred all-gather can run under the forward pass."""
        dp = self.dp
        if hasattr(self.model, "param_gate"):
            gated = dp is not None and hasattr(dp, "gate_param")
            self.model.param_gate = dp.gate_param if gated else None
            if gated:
                dp.uses_gates = True

    def sync_parameters(self) -> None:
        """Make the parameter arena current on every rank (applies a deferred optimizer update).
        Call before reading weights: evaluation, export, checkpoints, the end of training."""
        if self.dp is not None and hasattr(self.dp, "flush"):
            self.dp.flush()
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ one step, eager
    def _optimizer(self) -> None:
        o, a = self.opt, self.model.arena
        K.adamw_tick(self.step_dev, self.hyper, o.beta1, o.beta2)
        # The clip factor comes from the norm of every gradient of the job: the replicated arena's
        # (reduced over the ranks) and the rank-local arenas' (tensor-parallel / ZeRO-3 shards, local
        # experts), the latter with the model's gradient scale, summed over the ranks.
        extra = None
        if self.local_arenas and o.grad_clip is not None:
            for i, la in enumerate(self.local_arenas):
                K.sumsq(la.grads, out=self.local_sumsq, accumulate=i > 0)
            if self.local_grad_scale != 1.0:
                self.local_sumsq.mul_(self.local_grad_scale ** 2)
            extra = self.local_sumsq
        if self.dp is not None:
            if extra is not None:
                self.dp.reduce_and_update(a, self.hyper, o, self.sumsq, self.grad_norm, self.step_dev,
                                          extra_sumsq=extra)
            else:
                self.dp.reduce_and_update(a, self.hyper, o, self.sumsq, self.grad_norm, self.step_dev)
        else:
            if o.grad_clip is not None:
                K.sumsq(a.grads, out=self.sumsq)
                if extra is not None:
                    self.sumsq.add_(extra)
                K.clip_scale(self.sumsq, o.grad_clip, self.hyper, self.grad_norm)
            K.adamw_dev(a.master, a.params, a.grads, a.m, a.v, self.hyper,
                        beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay)
        if self.local_arenas:
            self.hyper_local.copy_(self.hyper)
            if self.local_grad_scale != 1.0:
                self.hyper_local[3:4].mul_(self.local_grad_scale)
            for la in self.local_arenas:
                K.adamw_dev(la.master, la.params, la.grads, la.m, la.v, self.hyper_local,
                            beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay)

    def _step_body(self) -> None:
        if not self._ledger_done and not torch.cuda.is_current_stream_capturing():
            self._ledger_done = True
            from .step_ledger import StepLedger
            with StepLedger(self.tape, self.ledger) as sl:
                self._step_body_inner(sl)
            sl.record_backward(self.last_report)
            return
        self._step_body_inner(None)

    def _step_body_inner(self, sl) -> None:
        n0 = K.launch_count()
        if self.dp is not None and hasattr(self.dp, "begin_step"):
            self.dp.begin_step()
        if hasattr(self.model, "begin_step"):
            self.model.begin_step()
        self.model.reset_grads()
        loss_id = self.model.forward(self.ids, self.targets)
        self.last_report = self.tape.backward(loss_id, BackwardOptions())
        self.loss_dev.copy_(self.tape.value(loss_id))
        if sl is not None:
            K.trace_take()          # accumulation kernels after the last rule belong to no operator
        self._optimizer()
        self.tape.truncate_graph_to(self.model.param_boundary)
        self.launches_per_step = K.launch_count() - n0

    def _ensure_graph(self) -> None:
        if self.graph is not None or not self.use_graph:
            return
        # one eager step on a side stream initialises lazy state (function attributes, status
        # word, driver entry points) outside of capture; its weight update is undone below
        a = self.model.arena
        own = self.dp if (self.dp is not None and a.master is None) else a   # who holds master/m/v
        snap = (own.master.clone(), own.m.clone(), own.v.clone(), self.step_dev.clone(), self.hyper.clone(),
                a.params.clone())
        snap_local = [(la.master.clone(), la.m.clone(), la.v.clone(), la.params.clone()) for la in self.local_arenas]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._step_body()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        K.check_status()
        own.master.copy_(snap[0]); own.m.copy_(snap[1]); own.v.copy_(snap[2])
        self.hyper.copy_(snap[4])
        a.params.copy_(snap[5])
        for la, sl in zip(self.local_arenas, snap_local):
            la.master.copy_(sl[0]); la.m.copy_(sl[1]); la.v.copy_(sl[2]); la.params.copy_(sl[3])
        self.step_dev.copy_(snap[3])   # (the multi-GPU path keeps its own, never-rewinding sequence)
        if self.dp is not None and hasattr(self.dp, "discard_pending"):
            self.dp.discard_pending()  # the warm-up step's reduced gradients must not be applied
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step_body()

    def switch_data_parallel(self, factory) -> None:
        """Replace the data-parallel object between steps (the hardened-mode fallback).

        A sharded optimizer (fp32 master / moments held per rank) is first gathered back into
        the arena, so that the replacement - built by ``factory()`` afterwards - finds the full
        state a replicated optimizer needs; the captured graph is dropped and rebuilt (or not
        used at all when the replacement runs library collectives)."""
        torch.cuda.synchronize()
        a, old = self.model.arena, self.dp
        if old is not None and a.master is None and hasattr(old, "gather_optimizer_state"):
            a.master, a.m, a.v = old.gather_optimizer_state()
        self.tape.leaf_grad_written_fn = None
        self.dp = factory()
        if self.dp is not None and hasattr(self.dp, "attach"):
            self.dp.attach(self.tape, getattr(self.model, "leaf", {}))
        self._wire_param_gates()
        self.use_graph = self._graph_requested and not getattr(self.dp, "eager_only", False)
        self.graph = None

    # ------------------------------------------------------------------ public API
    def set_lr(self, lr: float) -> None:
        self.lr_host[0] = lr
        self.hyper[0:1].copy_(self.lr_host, non_blocking=True)

    def step(self, ids_host: torch.Tensor, targets_host: torch.Tensor, *, read_loss: bool = True):
        """One optimizer step on a batch given in (pinned) host memory; returns the loss."""
        self.ids.copy_(ids_host, non_blocking=True)
        self.targets.copy_(targets_host, non_blocking=True)
        return self.step_device(read_loss=read_loss)

    def step_device(self, *, read_loss: bool = False):
        """One step on whatever is already in ``self.ids`` / ``self.targets``."""
        if self.use_graph:
            self._ensure_graph()
            self.graph.replay()
        else:
            self._step_body()
        self.steps_done += 1
        if read_loss:
            self.loss_host.copy_(self.loss_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(self.loss_host)
        return None
