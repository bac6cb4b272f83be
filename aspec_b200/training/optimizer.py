"""bf16 parameters + fp32 master weights, in flat buffers, with one fused AdamW kernel.

Semantics of the reference ``BF16Optimizer`` (aspec/training/optimizer.py:40-182): gradients are
taken in fp32, a global L2 norm gives the clip coefficient ``min(1, max_norm / (norm + 1e-6))``, a
non-finite norm skips the whole update on every rank (MAX all-reduce of a device flag, no host
sync), AdamW runs on the fp32 masters, the scheduler steps, masters are copied back to bf16.

Layout here: every trainable parameter is re-homed as a view of ONE bf16 buffer (module order, so
adjacent fused weights stay adjacent), with matching flat fp32 buffers for masters, gradients and
the two moments.  ``param.main_grad`` is the parameter's fp32 gradient view: the GEMM kernels
accumulate weight gradients straight into it, so "copy bf16 grads to fp32" disappears and gradient
accumulation over micro-batches is exact.  Norm, clip, the loss-denominator rescale
(``set_grad_scale``), the update and the bf16 write-back are two kernel launches over the flat
buffers, independent of the number of parameters.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from aspec_b200.training.lr_scheduler import LRSchedulerWithWarmup


def _align(n: int, a: int = 8) -> int:
    return -(-n // a) * a


class _AppliedSteps:
    """Adam's step counter lives on the device and advances only when an update is applied: an update skipped for
    non-finite gradients changes neither parameters, moments nor the bias-correction step, as with a fused AdamW
    driven by ``found_inf`` (reference: aspec/training/optimizer.py:123-135).  Reading ``step_count`` or
    ``skipped_steps`` on the host is a device-to-host read, done at checkpoint / metrics time only."""

    def _init_steps(self, device) -> None:
        self._applied = torch.zeros((), dtype=torch.float32, device=device)
        self.attempted_steps = 0

    def _advance_steps(self, ctrl: torch.Tensor) -> None:
        """``ctrl[0:2]`` hold the agreed norm / non-finite flag; writes this update's step index to ``ctrl[4]``."""
        self.attempted_steps += 1
        ok = ((ctrl[1] <= 0) & torch.isfinite(ctrl[0])).to(torch.float32)
        self._applied += ok
        ctrl[4] = self._applied

    @property
    def step_count(self) -> int:
        return int(round(float(self._applied)))

    @step_count.setter
    def step_count(self, value: int) -> None:
        self._applied.fill_(float(value))
        self.attempted_steps = max(self.attempted_steps, int(value))

    @property
    def skipped_steps(self) -> int:
        return self.attempted_steps - self.step_count


class BF16Optimizer(_AppliedSteps):
    def __init__(self, model: torch.nn.Module, lr: float, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.5, total_steps: int = 800_000, warmup_ratio: float = 0.015,
                 decay_style: str = "cosine", min_lr: float = 0.0, wsd_decay_steps=None,
                 wsd_decay_style=None, betas=(0.9, 0.999), eps: float = 1e-8,
                 norm_group: Optional[dist.ProcessGroup] = None, shard_group: Optional[dist.ProcessGroup] = None):
        self.model = model
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        # expert-parallel shards go last: the flat buffers are then a replicated region followed by a region that
        # differs from rank to rank, and each is reduced over its own set of ranks
        named.sort(key=lambda item: bool(getattr(item[1], "expert_parallel", False)))
        self.param_names = [n for n, _ in named]
        self.model_params = [p for _, p in named]
        if not self.model_params:
            raise ValueError("BF16Optimizer needs at least one trainable parameter")
        self.expert_group = None        # ranks that together hold all experts: their expert norms add up
        self.expert_names: Dict[str, tuple] = {}   # name -> (ep_rank, ep_size): state dicts carry whole banks
        self.max_grad_norm = float(max_grad_norm)
        self.weight_decay, self.betas, self.eps = float(weight_decay), betas, float(eps)
        self.lr = float(lr)
        self.norm_group = norm_group      # ranks whose gradient shards together form the full gradient
        self.shard_group = shard_group
        dev = self.model_params[0].device
        dtype = self.model_params[0].dtype
        self.offsets: List[int] = []
        off = 0
        for p in self.model_params:
            off = _align(off)
            self.offsets.append(off)
            off += p.numel()
        self.numel = _align(off)
        # first element of the expert-parallel region (== numel when there is none)
        self.dense_numel = next((o for p, o in zip(self.model_params, self.offsets) if getattr(p, "expert_parallel", False)),
                                self.numel)
        self.flat_param = torch.zeros(self.numel, dtype=dtype, device=dev)
        self.flat_master = torch.zeros(self.numel, dtype=torch.float32, device=dev)
        self.flat_grad = torch.zeros(self.numel, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(self.numel, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.numel, dtype=torch.float32, device=dev)
        with torch.no_grad():
            for p, o in zip(self.model_params, self.offsets):
                n = p.numel()
                self.flat_param[o:o + n].copy_(p.detach().reshape(-1))
                self.flat_master[o:o + n].copy_(p.detach().reshape(-1).float())
                p.data = self.flat_param[o:o + n].view(p.shape)
                p.main_grad = self.flat_grad[o:o + n].view(p.shape)
                p.main_grad_touched = False
                p.grad = None
        self._init_steps(dev)
        self._ctrl = torch.zeros(8, dtype=torch.float32, device=dev)
        self._grad_scale = torch.ones((), dtype=torch.float32, device=dev)
        self.use_kernel = dev.type == "cuda" and dtype == torch.bfloat16
        self.scheduler = LRSchedulerWithWarmup(
            self, max_lr=lr, total_steps=total_steps, warmup_steps=int(warmup_ratio * total_steps),
            decay_style=decay_style, min_lr=min_lr, wsd_decay_steps=wsd_decay_steps,
            wsd_decay_style=wsd_decay_style)

    # -- gradient plumbing --------------------------------------------------------
    def fold_autograd_grads(self) -> None:
        """Add ``p.grad`` left by ops that do not write ``main_grad`` themselves, then drop it."""
        with torch.no_grad():
            for p in self.model_params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(torch.float32))
                    p.grad = None

    def set_grad_scale(self, scale) -> None:
        """Multiply all gradients by ``scale`` (float or 0-d device tensor) inside the next step."""
        if torch.is_tensor(scale):
            self._grad_scale = scale.detach().to(self.flat_grad.device, torch.float32).reshape(())
        else:
            self._grad_scale = torch.full((), float(scale), dtype=torch.float32, device=self.flat_grad.device)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat_grad.zero_()
        for p in self.model_params:
            p.grad = None
            p.main_grad_touched = False

    # -- the update ---------------------------------------------------------------
    def step(self, closure=None) -> torch.Tensor:
        """One update; returns the global gradient norm before clipping (0-d device tensor)."""
        self.fold_autograd_grads()
        ctrl = self._ctrl
        ctrl.zero_()
        self._sumsq(self.flat_grad[: self.dense_numel], ctrl)
        if self.dense_numel < self.numel:
            # the expert region differs per rank of the expert-parallel group: its squares add up over that group
            part = torch.zeros_like(ctrl)
            self._sumsq(self.flat_grad[self.dense_numel:], part)
            if self.expert_group is not None and dist.get_world_size(self.expert_group) > 1:
                dist.all_reduce(part[0:2], group=self.expert_group)
            ctrl[0:2] += part[0:2]
        if self.norm_group is not None and dist.get_world_size(self.norm_group) > 1:
            dist.all_reduce(ctrl[0:1], group=self.norm_group)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            # one rank may be the only one that saw a non-finite value; all must agree on skipping
            flag = ((ctrl[1] > 0) | ~torch.isfinite(ctrl[0])).float().reshape(1)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            ctrl[1] = flag[0]
        ctrl[2] = self._grad_scale
        self._advance_steps(ctrl)
        b1, b2 = self.betas
        if self.use_kernel:
            from aspec_b200.ops import elementwise_sm100 as E
            E.adamw(self.flat_master, self.flat_grad, self.exp_avg, self.exp_avg_sq, self.flat_param, ctrl,
                    lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, wd=self.weight_decay,
                    step=None, max_norm=self.max_grad_norm)
        else:
            self._step_reference(ctrl, b1, b2)
        grad_norm = ctrl[2] * torch.sqrt(ctrl[0])
        self.flat_grad.zero_()
        for p in self.model_params:
            p.main_grad_touched = False
        self._grad_scale = torch.ones_like(self._grad_scale)
        self.scheduler.step()
        return grad_norm.clone()

    def _sumsq(self, grad: torch.Tensor, ctrl: torch.Tensor) -> None:
        """``ctrl[0] += sum(grad^2)``, ``ctrl[1] += non-finite``."""
        if grad.numel() == 0:
            return
        if self.use_kernel:
            from aspec_b200.ops import elementwise_sm100 as E
            E.sumsq(grad, ctrl)
        else:
            ctrl[0] += grad.double().pow(2).sum().float()
            ctrl[1] += (~torch.isfinite(grad)).any().float()

    def set_expert_parallel(self, group, ep_rank: int, ep_size: int) -> None:
        """Declare the expert-parallel layout of the parameters marked ``expert_parallel``."""
        self.expert_group = group
        self.expert_names = {n: (ep_rank, ep_size) for n, p in zip(self.param_names, self.model_params)
                             if getattr(p, "expert_parallel", False)}

    def _whole_bank(self, name: str, local: torch.Tensor) -> torch.Tensor:
        if name not in self.expert_names or self.expert_group is None:
            return local
        _, ep = self.expert_names[name]
        pieces = [torch.empty_like(local) for _ in range(ep)]
        dist.all_gather(pieces, local.contiguous(), group=self.expert_group)
        return torch.cat(pieces, 0)

    def _local_bank(self, name: str, saved: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
        if name in self.expert_names and saved.shape[0] != like.shape[0]:
            rank, ep = self.expert_names[name]
            n = saved.shape[0] // ep
            return saved[rank * n:(rank + 1) * n]
        return saved

    def _step_reference(self, ctrl, b1, b2) -> None:
        bad = bool(ctrl[1] > 0) or not bool(torch.isfinite(ctrl[0]))
        if bad:
            return
        pre = ctrl[2]
        norm = pre * torch.sqrt(ctrl[0])
        coef = pre
        if self.max_grad_norm > 0:
            coef = coef * torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
        g = self.flat_grad * coef
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        step = self.step_count
        bc1 = 1 - b1 ** step
        bc2 = 1 - b2 ** step
        self.flat_master.mul_(1 - self.lr * self.weight_decay)
        self.flat_master.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt() + self.eps, value=-self.lr)
        self.flat_param.copy_(self.flat_master)

    # -- state ---------------------------------------------------------------------
    def sync_fp32_params_from_model(self) -> None:
        """Re-derive the masters from the (just loaded) model weights."""
        with torch.no_grad():
            self.flat_master.copy_(self.flat_param.float())

    def _views(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: flat[o:o + p.numel()].view(p.shape)
                for n, p, o in zip(self.param_names, self.model_params, self.offsets)}

    def state_dict(self) -> dict:
        """AdamW state and fp32 masters keyed by parameter name."""
        whole = lambda flat: {n: self._whole_bank(n, t) for n, t in self._views(flat).items()}
        return {"step": self.step_count, "master": whole(self.flat_master),
                "exp_avg": whole(self.exp_avg), "exp_avg_sq": whole(self.exp_avg_sq),
                "hyper": {"lr": self.lr, "betas": list(self.betas), "eps": self.eps,
                          "weight_decay": self.weight_decay, "max_grad_norm": self.max_grad_norm}}

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(state["step"])
        with torch.no_grad():
            for key, flat in (("master", self.flat_master), ("exp_avg", self.exp_avg),
                              ("exp_avg_sq", self.exp_avg_sq)):
                views = self._views(flat)
                missing = set(views) - set(state[key])
                if missing:
                    raise KeyError(f"optimizer state lacks {sorted(missing)[:3]}...")
                for name, dst in views.items():
                    dst.copy_(self._local_bank(name, state[key][name], dst).to(dst))
            self.flat_param.copy_(self.flat_master)

    def get_learning_rate(self) -> float:
        return self.lr

    @property
    def lr_scheduler(self):
        return self.scheduler

    @property
    def param_groups(self):
        return [{"lr": self.lr, "params": self.model_params}]
