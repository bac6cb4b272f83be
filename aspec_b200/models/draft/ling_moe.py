"""Ling-MoE FFN: fp32 sigmoid routing with a balancing bias, group-limited top-k, clamped SwiGLU experts,
a shared expert, router z-loss and the once-per-optimizer-step bias update
(reference: aspec/models/draft/ling_moe.py:34-172, aspec/training/dflash_trainer.py:829-845)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from aspec_b200.models.draft.dflash import DFlashMLP
from aspec_b200.models.draft.moe import ExpertBank, route_and_run


class LingGate(nn.Module):
    """Sigmoid router.  ``weight [E, D]`` trains; ``expert_bias [E]`` is fp32 control state that only the balancing rule
    moves (never the optimizer) and that only steers the *selection*: mixing weights come from the raw scores."""

    def __init__(self, config):
        super().__init__()
        E = config.num_experts
        self.top_k = config.num_experts_per_tok
        self.groups, self.group_topk = config.n_group, config.topk_group
        self.scale = config.routed_scaling_factor
        self.bias_enabled = bool(config.moe_router_enable_expert_bias)
        self.weight = nn.Parameter(torch.empty(E, config.hidden_size))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32))

    def _apply(self, fn, recurse=True):
        # ``module.to(torch.bfloat16)`` must not round the bias: take it out of the way of the cast and put it back in
        # fp32 on whatever device the weight ended up on
        held = self._buffers.pop("expert_bias")
        try:
            super()._apply(fn, recurse=recurse)
        finally:
            where = self.weight.device
            self._buffers["expert_bias"] = (torch.zeros_like(held, dtype=torch.float32, device=where) if held.is_meta and where.type != "meta"
                                            else held.to(device=where, dtype=torch.float32))
        return self

    def forward(self, hidden: torch.Tensor):
        """``(selected [N, k], mixing weights [N, k], router logits [N, E])`` in fp32."""
        from aspec_b200.models.draft.eagle4_moe import select_experts
        tokens = hidden.reshape(-1, hidden.shape[-1]).float()
        logits = tokens @ self.weight.float().t()
        scores = torch.sigmoid(logits)
        steer = self.expert_bias if self.bias_enabled else torch.zeros_like(self.expert_bias)
        selected = select_experts(scores, steer, self.top_k, self.groups, self.group_topk)
        mix = torch.gather(scores, 1, selected)
        if self.top_k > 1:                       # with one expert per token the raw sigmoid score is kept as is
            mix = mix / (mix.sum(-1, keepdim=True) + 1e-20)
        return selected, mix * self.scale, logits


class LingMoE(nn.Module):
    wants_aux = True

    def __init__(self, config, layer_idx: int = 0, ep_rank: int = 0, ep_size: int = 1, ep_group=None):
        super().__init__()
        self.num_experts, self.top_k = config.num_experts, config.num_experts_per_tok
        self.gate = LingGate(config)
        self.experts = ExpertBank(config.num_experts, config.hidden_size, config.moe_intermediate_size,
                                  clamp=config.expert_swiglu_limit_list[layer_idx], ep_rank=ep_rank, ep_size=ep_size)
        self.shared_experts = (DFlashMLP(config.hidden_size,
                                         config.num_shared_experts * config.moe_shared_expert_intermediate_size,
                                         clamp=config.share_expert_swiglu_limit_list[layer_idx])
                               if config.num_shared_experts else None)
        self.ep_group = ep_group

    def forward(self, x: torch.Tensor, aux: Optional[dict] = None) -> torch.Tensor:
        shape = x.shape
        h = x.reshape(-1, shape[-1])
        selected, w, logits = self.gate(h)
        out = route_and_run(self.experts, h, selected, w, self.ep_group, fp32_accumulate=True).reshape(shape)
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        if aux is not None:
            aux.setdefault("router_logits", []).append((logits, selected))
        return out


def _layer_router_statistics(logits: torch.Tensor, selected: torch.Tensor, live: torch.Tensor):
    """One layer: how often each expert was chosen by a supervised slot, and the summed squared log-partition."""
    E = logits.shape[-1]
    hits = torch.zeros(E, dtype=torch.float32, device=logits.device)
    hits.scatter_add_(0, selected.reshape(-1), live[:, None].expand_as(selected).reshape(-1))
    z = torch.logsumexp(logits.float(), dim=-1)
    return hits, (z * z * live).sum()


def ling_router_terms(observations, objective_weights, denominator, z_coefficient, cp_group=None):
    """Router z-loss numerator and balancing statistics of one forward.

    ``observations``: per MoE layer ``(router logits [N, E], selected [N, k])``.  Only slots with a positive objective
    weight count.  The z-loss of a forward is the sum over layers of the mean squared log-partition; it is returned
    multiplied by the forward's loss denominator so that it pools over micro-batches and ranks like every other term.
    The per-expert hit counts (``_ling_router_counts``, ``[layers, E]``) stay local: the trainer sums them over the
    accumulation window and the data-parallel ranks before the bias rule reads them.
    """
    live = (objective_weights.reshape(-1) > 0).to(torch.float32)
    per_layer = [_layer_router_statistics(lg, sel, live) for lg, sel in observations]
    hits = torch.stack([h for h, _ in per_layer])                    # [layers, E]
    z_total = torch.stack([z for _, z in per_layer]).sum()
    slots = live.sum()
    seen = hits.detach().clone()
    if cp_group is not None:
        # a context-parallel group shares one row: its slots and hits are one population
        import torch.distributed as dist
        from torch.distributed.nn.functional import all_reduce as differentiable_all_reduce
        z_total = differentiable_all_reduce(z_total, group=cp_group)
        slots = slots.clone()
        dist.all_reduce(slots, group=cp_group)
        dist.all_reduce(seen, group=cp_group)
    slots = slots.clamp_min(1)
    z_numerator = z_total / slots * denominator
    k = observations[0][1].shape[-1]
    den = denominator.detach()
    busiest = (seen / (slots * k)).max()
    used = (seen > 0).sum(-1).float().mean()
    stats = {"router_z_loss": (z_numerator.detach(), den),
             "router_max_load": ((busiest * denominator).detach(), den),
             "router_used_experts": ((used * denominator).detach(), den),
             "_ling_router_counts": hits.detach()}
    return z_coefficient * z_numerator, stats


@torch.no_grad()
def update_ling_bias(layers, counts, update_rate: float, zero_mean: bool = True, group=None, apply_update=True) -> None:
    """Balancing rule, once per committed optimizer step: experts chosen less often than their layer's average get
    ``+rate``, busier ones ``-rate`` (optionally re-centred to zero mean).  A layer that saw no supervised slot, or a
    step that was not applied, leaves the bias where it was."""
    if group is not None:
        import torch.distributed as dist
        dist.all_reduce(counts, group=group)
    applied = torch.as_tensor(apply_update, device=counts.device).bool()
    for layer, hits in zip(layers, counts):
        if not layer.gate.bias_enabled:
            continue
        direction = torch.sign(hits.mean() - hits)
        if zero_mean:
            direction = direction - direction.mean()
        move = applied & (hits.sum() > 0)
        layer.gate.expert_bias += torch.where(move, direction * update_rate, torch.zeros_like(direction))
