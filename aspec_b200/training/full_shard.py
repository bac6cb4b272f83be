"""FULL_SHARD: parameters, gradients, fp32 masters and Adam moments all sharded over the data-parallel ranks.

What the reference gets from FSDP2 ``fully_shard`` per decoder layer plus a sharded ``BF16Optimizer``
(aspec/training/fsdp.py:200-231, aspec/training/optimizer.py:88-147, aspec/training/dflash_trainer.py:494-533), built
on peer memory and flags instead of library collectives:

* **At rest** a rank holds ``1 / p`` of every unit (a unit = one decoder layer; everything else forms the root unit):
  the bf16 shard (peer-visible), its fp32 master, both moments and an fp32 gradient shard.
* **Forward / backward of a layer** run on a full copy of the layer in one of TWO rotating buffers.  The copy is made by
  ``peer_gather`` (plain loads from the peers' shards over NVLink) on a side stream, one layer ahead of the compute
  stream, and made again before the layer's backward; the parameters' storage never moves, so tensors saved by autograd
  stay valid.  The root unit stays gathered for the whole update.
* **Gradients** of a layer are accumulated in one of two rotating fp32 buffers (peer-visible).  When the layer's
  backward has finished, the rank raises a flag on every peer; the side stream waits for all peers' flags and
  ``shard_reduce_accum`` adds the ``p`` replicas of the rank's own range into its gradient shard - the reduce-scatter,
  running under the backward of the layers below.  A second flag tells the peers that the buffer has been read and may
  be reused.
* **The update** is AdamW on the shards (the only cross-rank traffic: two scalars for the global norm).  A parameter
  flag orders the next gathers after every rank's update.

Every wait on a flag is bounded (``comm.flags_wait_all``); a wait that runs out leaves the peer-timeout code in the
status word that ``step`` checks, and the context stays usable.  On CPU (``gloo``) the same hooks run the protocol with
``all_gather`` / ``all_reduce`` so that it is testable without GPUs.

Micro-batches of the ranks move in lock-step at layer granularity (that is what sharding the gradient buys and costs);
the optimizer-state-only variant (``sharded_optimizer.ShardedBF16Optimizer``, strategy ``SHARD_OPTIMIZER``) keeps
whole replicas and synchronises once per update.
"""
from __future__ import annotations

import contextlib
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from aspec_b200.parallel.symmetric_memory import SymmetricBuffer
from aspec_b200.training.lr_scheduler import LRSchedulerWithWarmup
from aspec_b200.training.optimizer import _AppliedSteps, _align

F_PARAM, F_GRAD, F_READ = 0, 1, 4          # flag slots: parameters published; gradient buffer s complete; buffer s read
N_FLAG_SLOTS = 7
ROOT_SLOT = 2                              # buffers 0 / 1 rotate over the layers, buffer 2 belongs to the root unit


class _Enter(torch.autograd.Function):
    """Identity on a unit's differentiable inputs; its backward runs when the unit's backward has produced them all."""

    @staticmethod
    def forward(ctx, engine, unit, *tensors):
        ctx.engine, ctx.unit = engine, unit
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        ctx.engine._post_backward(ctx.unit)
        return (None, None, *grads)


class _Exit(torch.autograd.Function):
    """Identity on a unit's outputs; its backward runs right before the unit's own backward starts."""

    @staticmethod
    def forward(ctx, engine, unit, *tensors):
        ctx.engine, ctx.unit = engine, unit
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        ctx.engine._pre_backward(ctx.unit)
        return (None, None, *grads)


class _Unit:
    def __init__(self, index: int, names: List[str], params: List[torch.nn.Parameter], world: int):
        self.index, self.names, self.params = index, names, params
        self.offsets: List[int] = []
        off = 0
        for p in params:
            off = _align(off)
            self.offsets.append(off)
            off += p.numel()
        self.numel = _align(max(off, 8 * world), 8 * world)          # full (padded) element count
        self.per = self.numel // world                                # elements every rank owns
        self.shard_offset = 0                                         # start of this unit in the flat shard arrays


class FullShardOptimizer(_AppliedSteps):
    def __init__(self, model: torch.nn.Module, layers: Sequence[torch.nn.Module], lr: float, weight_decay: float = 0.0,
                 max_grad_norm: float = 0.5, total_steps: int = 800_000, warmup_ratio: float = 0.015,
                 decay_style: str = "cosine", min_lr: float = 0.0, wsd_decay_steps=None, wsd_decay_style=None,
                 betas=(0.9, 0.999), eps: float = 1e-8, group: Optional[dist.ProcessGroup] = None,
                 wait_limit_ms: float = 8000.0):
        self.model, self.group = model, group
        on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        self.max_grad_norm, self.weight_decay, self.betas, self.eps, self.lr = float(max_grad_norm), float(weight_decay), betas, float(eps), float(lr)
        self.wait_limit_ms = float(wait_limit_ms)
        # ---- units: one per layer, the rest of the trainable parameters is the root ---------------------------
        in_layer: Dict[int, int] = {}
        self.layers = list(layers)
        for li, layer in enumerate(self.layers):
            for p in layer.parameters():
                in_layer[id(p)] = li
        grouped: List[List] = [[] for _ in range(len(self.layers) + 1)]
        for name, p in model.named_parameters():
            if p.requires_grad:
                if getattr(p, "expert_parallel", False):
                    raise ValueError("FULL_SHARD does not combine with expert parallelism")
                grouped[in_layer.get(id(p), len(self.layers))].append((name, p))
        self.units = [_Unit(i, [n for n, _ in g], [p for _, p in g], self.world) for i, g in enumerate(grouped)]
        self.root = self.units[-1]
        self.n_layers = len(self.layers)
        first = next(p for u in self.units for p in u.params)
        dev, dtype = first.device, first.dtype
        self.device, self.dtype = dev, dtype
        self.use_kernel = dev.type == "cuda" and dtype == torch.bfloat16
        elem = torch.empty(0, dtype=dtype).element_size()
        off = 0
        for u in self.units:
            u.shard_offset = off
            off += u.per
        self.shard_numel = off
        self.param_names = [n for u in self.units for n in u.names]
        self.model_params = [p for u in self.units for p in u.params]
        # ---- at rest: 1 / world of everything ------------------------------------------------------------
        self._shard_mem = SymmetricBuffer.allocate(max(self.shard_numel * elem, 16), dev)
        self.shard_param = self._shard_mem.tensor[: self.shard_numel * elem].view(dtype)
        self.shard_grad = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
        self.shard_master = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
        # ---- working copies: two rotating layer buffers and the root's own ----------------------------------------
        layer_max = max([u.numel for u in self.units[:-1]], default=0)
        self._slot_numel = [layer_max, layer_max, self.root.numel]
        self.param_buf = [torch.zeros(n, dtype=dtype, device=dev) for n in self._slot_numel]
        self._grad_mem = [SymmetricBuffer.allocate(max(n * 4, 16), dev) for n in self._slot_numel]
        self.grad_buf = [m.tensor[: n * 4].view(torch.float32) for m, n in zip(self._grad_mem, self._slot_numel)]
        for g in self.grad_buf:
            g.zero_()
        self._flag_mem = SymmetricBuffer.allocate(N_FLAG_SLOTS * self.world * 8, dev)
        self.flags = self._flag_mem.tensor[: N_FLAG_SLOTS * self.world * 8].view(torch.int64)
        self.flags.zero_()
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        with torch.no_grad():
            for u in self.units:
                slot = self._slot(u)
                buf, gbuf = self.param_buf[slot], self.grad_buf[slot]
                full = torch.zeros(u.numel, dtype=dtype, device=dev)
                for p, o in zip(u.params, u.offsets):
                    full[o:o + p.numel()].copy_(p.detach().reshape(-1))
                lo = self.rank * u.per
                self._shard_of(self.shard_param, u).copy_(full[lo:lo + u.per])
                self._shard_of(self.shard_master, u).copy_(full[lo:lo + u.per].float())
                for p, o in zip(u.params, u.offsets):
                    p.data = buf[o:o + p.numel()].view(p.shape)
                    p.main_grad = gbuf[o:o + p.numel()].view(p.shape)
                    p.main_grad_touched = False
                    p.grad = None
                del full
        # ---- peers --------------------------------------------------------------------------------------------
        self._peer_shards: List[torch.Tensor] = [self.shard_param]
        self._peer_grads: List[List[torch.Tensor]] = [[g] for g in self.grad_buf]
        self._peer_flags: List[torch.Tensor] = [self.flags]
        self._opened: List[SymmetricBuffer] = []
        if self.world > 1 and self.use_kernel:
            torch.cuda.synchronize(dev)       # shards and zeroed flags are in memory before any peer can map them
            self._exchange_handles()
        self._comm = torch.cuda.Stream(dev) if self.use_kernel else None
        self._holds: List[Optional[int]] = [None, None, None]
        self._gathered_event = [None, None, None]
        self._free_event = [None, None, None]
        self._reduced_event = [None, None, None]
        self._uses = [0, 0, 0]                       # how often each gradient buffer has been filled
        self._in_backward = [False] * len(self.units)
        self._touched: set = set()                   # units whose forward ran with gradients in this micro-batch
        self._root_open = False
        self._version = 0
        self._init_steps(dev)
        self._ctrl = torch.zeros(8, dtype=torch.float32, device=dev)
        self._grad_scale = torch.ones((), dtype=torch.float32, device=dev)
        self.scheduler = LRSchedulerWithWarmup(self, max_lr=lr, total_steps=total_steps, warmup_steps=int(warmup_ratio * total_steps),
                                               decay_style=decay_style, min_lr=min_lr, wsd_decay_steps=wsd_decay_steps,
                                               wsd_decay_style=wsd_decay_style)
        for u in self.units[:-1]:
            self._wrap(u, self.layers[u.index])
        self._gather_root()

    # ---- layout helpers ---------------------------------------------------------------------------------------
    def _slot(self, u: _Unit) -> int:
        return ROOT_SLOT if u is self.root else u.index % 2

    def _shard_of(self, flat: torch.Tensor, u: _Unit) -> torch.Tensor:
        return flat[u.shard_offset:u.shard_offset + u.per]

    def _exchange_handles(self) -> None:
        mine = [{"shard": self._shard_mem.export(), "flags": self._flag_mem.export(),
                 "grads": [m.export() for m in self._grad_mem]} for _ in range(self.world)]
        gathered: List = [None] * self.world
        dist.all_gather_object(gathered, mine, group=self.group)
        elem = self.shard_param.element_size()
        shards, flags = [], []
        grads: List[List[torch.Tensor]] = [[] for _ in self.grad_buf]
        for r in range(self.world):
            if r == self.rank:
                shards.append(self.shard_param)
                flags.append(self.flags)
                for s, g in enumerate(self.grad_buf):
                    grads[s].append(g)
                continue
            meta = gathered[r][self.rank]
            sb, fb = SymmetricBuffer.open(meta["shard"]), SymmetricBuffer.open(meta["flags"])
            self._opened += [sb, fb]
            shards.append(sb.tensor[: self.shard_numel * elem].view(self.dtype))
            flags.append(fb.tensor[: N_FLAG_SLOTS * self.world * 8].view(torch.int64))
            for s, gm in enumerate(meta["grads"]):
                gb = SymmetricBuffer.open(gm)
                self._opened.append(gb)
                grads[s].append(gb.tensor[: self._slot_numel[s] * 4].view(torch.float32))
        self._peer_shards, self._peer_flags, self._peer_grads = shards, flags, grads

    def memory_report(self) -> dict:
        """Bytes this rank holds for weights, gradients and optimizer state, against one full replica."""
        elem = self.shard_param.element_size()
        total = sum(u.numel for u in self.units)
        at_rest = self.shard_numel * (elem + 16)
        working = sum(self._slot_numel) * (elem + 4)
        return {"world": self.world, "parameters": total, "at_rest_bytes": at_rest, "working_bytes": working,
                "replicated_bytes": total * (elem + 16), "largest_layer": self._slot_numel[0], "root": self.root.numel}

    # ---- gathers ----------------------------------------------------------------------------------------------
    def _issue_gather(self, u: _Unit) -> None:
        slot = self._slot(u)
        buf = self.param_buf[slot][: u.numel]
        if self.use_kernel:
            from aspec_b200.ops import comm
            cur = torch.cuda.current_stream(self.device)
            if self._free_event[slot] is not None:
                self._comm.wait_event(self._free_event[slot])
            else:
                self._comm.wait_stream(cur)
            if self.world > 1:
                comm.flags_wait_all(self.flags, F_PARAM * self.world, self.world, self._version, self.status,
                                    self.wait_limit_ms, stream=self._comm)
            shards = [self._shard_of(t, u) for t in self._peer_shards]
            comm.peer_gather(shards, buf, stream=self._comm)
            ev = torch.cuda.Event()
            ev.record(self._comm)
            self._gathered_event[slot] = ev
        else:
            mine = self._shard_of(self.shard_param, u)
            with torch.no_grad():
                if self.world > 1:
                    parts = [torch.empty_like(mine) for _ in range(self.world)]
                    dist.all_gather(parts, mine.contiguous(), group=self.group)
                    torch.cat(parts, out=buf)
                else:
                    buf.copy_(mine)
        self._holds[slot] = u.index

    def _ensure_gathered(self, u: _Unit) -> None:
        slot = self._slot(u)
        if self._holds[slot] != u.index:
            self._issue_gather(u)
        if self.use_kernel and self._gathered_event[slot] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._gathered_event[slot])

    def _prefetch(self, index: int) -> None:
        if 0 <= index < self.n_layers and self.use_kernel:      # collectives on CPU are synchronous: nothing to hide
            u = self.units[index]
            if self._holds[self._slot(u)] != index:
                self._issue_gather(u)

    def _release(self, u: _Unit) -> None:
        if self.use_kernel:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._free_event[self._slot(u)] = ev

    def _gather_root(self) -> None:
        self._holds[ROOT_SLOT] = None
        self._free_event[ROOT_SLOT] = None
        self._ensure_gathered(self.root)

    # ---- hooks around a layer ---------------------------------------------------------------------------------
    def _wrap(self, u: _Unit, module: torch.nn.Module) -> None:
        inner = module.forward
        engine = self

        def forward(*args, **kwargs):
            if engine._in_backward[u.index]:                 # activation recomputation inside this layer's backward
                return inner(*args, **kwargs)
            engine._ensure_gathered(u)
            track = torch.is_grad_enabled()
            engine._prefetch(u.index + 1)
            if track:
                engine._begin_micro_batch()
                idx = [i for i, a in enumerate(args) if torch.is_tensor(a) and a.requires_grad]
                if idx:
                    fresh = _Enter.apply(engine, u.index, *[args[i] for i in idx])
                    args = list(args)
                    for i, t in zip(idx, fresh):
                        args[i] = t
            out = inner(*args, **kwargs)
            if track:
                engine._touched.add(u.index)
                out = engine._guard_outputs(u, out)
            engine._release(u)
            return out

        module.forward = forward

    def _guard_outputs(self, u: _Unit, out):
        if torch.is_tensor(out):
            return _Exit.apply(self, u.index, out)[0] if out.requires_grad else out
        if isinstance(out, (tuple, list)):
            idx = [i for i, t in enumerate(out) if torch.is_tensor(t) and t.requires_grad]
            if idx:
                fresh = _Exit.apply(self, u.index, *[out[i] for i in idx])
                items = list(out)
                for i, t in zip(idx, fresh):
                    items[i] = t
                return type(out)(items) if isinstance(out, tuple) else items
        return out

    def _begin_micro_batch(self) -> None:
        """The root's gradient buffer is opened once per micro-batch, before anything can write into it."""
        if not self._root_open:
            self._open_grad_buffer(self.root)
            self._root_open = True

    def _open_grad_buffer(self, u: _Unit) -> None:
        slot = self._slot(u)
        if self.use_kernel:
            from aspec_b200.ops import comm
            cur = torch.cuda.current_stream(self.device)
            if self._reduced_event[slot] is not None:
                cur.wait_event(self._reduced_event[slot])
            if self.world > 1 and self._uses[slot] > 0:           # every peer has read the previous contents
                comm.flags_wait_all(self.flags, (F_READ + slot) * self.world, self.world, self._uses[slot], self.status,
                                    self.wait_limit_ms, stream=cur)
        self.grad_buf[slot][: u.numel].zero_()
        self._uses[slot] += 1

    def _pre_backward(self, index: int) -> None:
        u = self.units[index]
        self._in_backward[index] = True
        self._ensure_gathered(u)
        self._prefetch(index - 1)
        self._open_grad_buffer(u)

    def _fold(self, u: _Unit) -> None:
        with torch.no_grad():
            for p in u.params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(torch.float32))
                    p.grad = None

    def _post_backward(self, index: int) -> None:
        u = self.units[index]
        if index in self._touched:
            self._touched.discard(index)
        self._fold(u)
        self._in_backward[index] = False
        if u is not self.root:
            self._release(u)
        self._reduce(u)

    def _reduce(self, u: _Unit) -> None:
        """Reduce-scatter of the unit's gradient buffer into this rank's shard (accumulating over micro-batches)."""
        slot = self._slot(u)
        lo = self.rank * u.per
        mine = self._shard_of(self.shard_grad, u)
        if self.use_kernel:
            from aspec_b200.ops import comm
            cur = torch.cuda.current_stream(self.device)
            k = self._uses[slot]
            if self.world > 1:
                comm.flags_signal(self._peer_flags, (F_GRAD + slot) * self.world + self.rank, k, stream=cur)
            done = torch.cuda.Event()
            done.record(cur)
            self._comm.wait_event(done)
            if self.world > 1:
                comm.flags_wait_all(self.flags, (F_GRAD + slot) * self.world, self.world, k, self.status,
                                    self.wait_limit_ms, stream=self._comm)
            comm.shard_reduce_accum([g[: u.numel] for g in self._peer_grads[slot]], lo, mine, stream=self._comm)
            if self.world > 1:
                comm.flags_signal(self._peer_flags, (F_READ + slot) * self.world + self.rank, k, stream=self._comm)
            ev = torch.cuda.Event()
            ev.record(self._comm)
            self._reduced_event[slot] = ev
        else:
            g = self.grad_buf[slot][: u.numel]
            with torch.no_grad():
                if self.world > 1:
                    dist.all_reduce(g, group=self.group)
                mine.add_(g[lo:lo + u.per])

    def finish_micro_batch(self) -> None:
        """After a micro-batch's ``backward`` has returned: close whatever no hook closed (a layer whose inputs need no
        gradient has no ``_Enter``; the root has no boundaries at all)."""
        for index in sorted(self._touched, reverse=True):
            u = self.units[index]
            if not self._in_backward[index]:                 # the layer received no gradient: still take part
                self._open_grad_buffer(u)
            self._post_backward(index)
        self._touched.clear()
        for u in self.units[:-1]:
            if any(p.grad is not None for p in u.params):
                raise RuntimeError(f"layer {u.index} received a gradient after its reduce-scatter had started")
        # the root takes part in every micro-batch, also when no wrapped layer ran before it (a Draft whose decoder is not
        # a ``layers`` list lives in the root whole): its buffer is cleared here, before its gradients are folded in
        if not self._root_open:
            self._open_grad_buffer(self.root)
        self._fold(self.root)
        self._reduce(self.root)
        self._root_open = False

    # ---- the optimizer contract -----------------------------------------------------------------------------------
    def fold_autograd_grads(self) -> None:
        if self._root_open or self._touched or any(p.grad is not None for p in self.root.params):
            self.finish_micro_batch()

    def set_grad_scale(self, scale) -> None:
        self._grad_scale = (scale.detach().to(self.device, torch.float32).reshape(()) if torch.is_tensor(scale)
                            else torch.full((), float(scale), dtype=torch.float32, device=self.device))

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.shard_grad.zero_()
        for p in self.model_params:
            p.grad = None
            p.main_grad_touched = False

    def step(self, closure=None) -> torch.Tensor:
        self.fold_autograd_grads()
        ctrl = self._ctrl
        b1, b2 = self.betas
        if self.use_kernel:
            cur = torch.cuda.current_stream(self.device)
            for ev in self._reduced_event:
                if ev is not None:
                    cur.wait_event(ev)
        ctrl.zero_()
        g = self.shard_grad
        ctrl[0] = g.double().pow(2).sum().float()
        ctrl[1] = (~torch.isfinite(g)).any().float()
        if self.world > 1:
            dist.all_reduce(ctrl[0:2], group=self.group)
        ctrl[2] = self._grad_scale
        self._advance_steps(ctrl)
        if self.use_kernel:
            from aspec_b200.ops import comm
            comm.shard_adamw_scatter(self.shard_master, g, self.exp_avg, self.exp_avg_sq, [self.shard_param], 0, ctrl,
                                     lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, wd=self.weight_decay, step=None,
                                     max_norm=self.max_grad_norm)
        else:
            self._adamw_reference(ctrl, b1, b2)
        g.zero_()
        self._publish()
        grad_norm = ctrl[2] * torch.sqrt(ctrl[0])
        for p in self.model_params:
            p.main_grad_touched = False
        self._grad_scale = torch.ones_like(self._grad_scale)
        self.scheduler.step()
        self.check_status()
        return grad_norm.clone()

    def _adamw_reference(self, ctrl, b1, b2) -> None:
        if bool(ctrl[1] > 0) or not bool(torch.isfinite(ctrl[0])):
            return
        coef = ctrl[2]
        if self.max_grad_norm > 0:
            coef = coef * torch.clamp(self.max_grad_norm / (ctrl[2] * torch.sqrt(ctrl[0]) + 1e-6), max=1.0)
        g = self.shard_grad * coef
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        step = self.step_count
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        self.shard_master.mul_(1 - self.lr * self.weight_decay)
        self.shard_master.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt() + self.eps, value=-self.lr)
        self.shard_param.copy_(self.shard_master.to(self.shard_param.dtype))

    def _publish(self) -> None:
        """New shards are in place: tell the peers, forget the layer copies, refresh the root."""
        self._version += 1
        if self.use_kernel and self.world > 1:
            from aspec_b200.ops import comm
            comm.flags_signal(self._peer_flags, F_PARAM * self.world + self.rank, self._version,
                              stream=torch.cuda.current_stream(self.device))
        self._holds = [None, None, None]
        self._gather_root()

    def check_status(self) -> None:
        """One host read: a peer that never raised a flag shows up here instead of hanging the stream."""
        if self.use_kernel and self.world > 1:
            code = int(self.status.item())
            if code:
                self.status.zero_()
                raise RuntimeError(f"FULL_SHARD: a wait on a peer's flag ran out (status {code}); a rank is missing or late "
                                   f"by more than {self.wait_limit_ms:.0f} ms")

    # ---- whole parameters for checkpoints, exports and loads ------------------------------------------------------
    @contextlib.contextmanager
    def full_parameters(self, writeback: bool = False):
        """Inside the block every layer's parameters are whole at the same time (in temporary memory).  With
        ``writeback`` the block's changes (a loaded checkpoint) become the new shards and fp32 masters."""
        saved = []
        with torch.no_grad():
            for u in self.units[:-1]:
                self._ensure_gathered(u)
                if self.use_kernel:
                    torch.cuda.current_stream(self.device).synchronize()
                tmp = self.param_buf[self._slot(u)][: u.numel].clone()
                for p, o in zip(u.params, u.offsets):
                    saved.append((p, p.data))
                    p.data = tmp[o:o + p.numel()].view(p.shape)
                u._tmp = tmp
            self._ensure_gathered(self.root)
        try:
            yield self
        finally:
            with torch.no_grad():
                if writeback:
                    for u in self.units:
                        full = u._tmp if u is not self.root else self.param_buf[ROOT_SLOT][: u.numel]
                        lo = self.rank * u.per
                        self._shard_of(self.shard_param, u).copy_(full[lo:lo + u.per])
                        self._shard_of(self.shard_master, u).copy_(full[lo:lo + u.per].float())
                for p, data in saved:
                    p.data = data
                for u in self.units[:-1]:
                    u._tmp = None
                if writeback:
                    self._host_fence()
                    self._publish()
                else:
                    self._holds[0] = self._holds[1] = None

    def sync_fp32_params_from_model(self) -> None:
        """Masters from the bf16 shards (after weights were written through ``full_parameters(writeback=True)``)."""
        with torch.no_grad():
            self.shard_master.copy_(self.shard_param.float())

    def _full_flat(self, shard: torch.Tensor, u: _Unit) -> torch.Tensor:
        mine = self._shard_of(shard, u)
        if self.world == 1:
            return mine.clone()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine.contiguous(), group=self.group)
        return torch.cat(parts)

    def state_dict(self) -> dict:
        """Collective.  Same keys as the replicated optimizer: a checkpoint does not depend on the shard count."""
        out = {"step": self.step_count, "master": {}, "exp_avg": {}, "exp_avg_sq": {},
               "hyper": {"lr": self.lr, "betas": list(self.betas), "eps": self.eps, "weight_decay": self.weight_decay,
                         "max_grad_norm": self.max_grad_norm}}
        for key, shard in (("master", self.shard_master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            for u in self.units:
                full = self._full_flat(shard, u)
                for n, p, o in zip(u.names, u.params, u.offsets):
                    out[key][n] = full[o:o + p.numel()].view(p.shape)
        return out

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(state["step"])
        with torch.no_grad():
            for key, shard in (("master", self.shard_master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                for u in self.units:
                    full = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
                    for n, p, o in zip(u.names, u.params, u.offsets):
                        if n not in state[key]:
                            raise KeyError(f"optimizer state lacks {n}")
                        full[o:o + p.numel()].copy_(state[key][n].reshape(-1).to(full))
                    lo = self.rank * u.per
                    self._shard_of(shard, u).copy_(full[lo:lo + u.per])
            self.shard_param.copy_(self.shard_master.to(self.shard_param.dtype))
        self._host_fence()
        self._publish()

    def _host_fence(self) -> None:
        """Outside the training protocol (loads): every rank's writes are in memory and every rank's outstanding reads
        are finished before anyone continues."""
        if self.use_kernel:
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def get_learning_rate(self) -> float:
        return self.lr

    @property
    def lr_scheduler(self):
        return self.scheduler

    @property
    def param_groups(self):
        return [{"lr": self.lr, "params": self.model_params}]

    def close(self) -> None:
        for b in self._opened:
            b.close()
        self._opened = []
