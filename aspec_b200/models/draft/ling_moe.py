"""Ling-MoE FFN: fp32 sigmoid routing with a balancing bias, group-limited top-k, clamped SwiGLU experts,
a shared expert, router z-loss and the once-per-optimizer-step bias update
(reference: aspec/models/draft/ling_moe.py:34-172, aspec/training/dflash_trainer.py:829-845)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.models.draft.dflash import DFlashMLP
from aspec_b200.models.draft.moe import ExpertBank, route_and_run


class LingGate(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(config.num_experts, config.hidden_size))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        self.register_buffer("expert_bias", torch.zeros(config.num_experts, dtype=torch.float32))
        self.top_k, self.groups, self.group_topk = config.num_experts_per_tok, config.n_group, config.topk_group
        self.scale = config.routed_scaling_factor
        self.bias_enabled = config.moe_router_enable_expert_bias

    def _apply(self, fn, recurse=True):
        # the bias is fp32 control state: it must survive ``module.to(torch.bfloat16)`` unrounded
        bias = self.expert_bias
        super()._apply(fn, recurse=recurse)
        self.expert_bias = bias.to(device=self.expert_bias.device, dtype=torch.float32)
        return self

    def forward(self, hidden: torch.Tensor):
        """``(selected [N, k], mixing weights [N, k], router logits [N, E])`` in fp32."""
        from aspec_b200.models.draft.eagle4_moe import select_experts
        logits = hidden.reshape(-1, hidden.shape[-1]).float() @ self.weight.float().t()
        scores = torch.sigmoid(logits)
        bias = self.expert_bias if self.bias_enabled else torch.zeros_like(self.expert_bias)
        selected = select_experts(scores, bias, self.top_k, self.groups, self.group_topk)
        mix = torch.gather(scores, 1, selected)
        if self.top_k > 1:                       # a single expert keeps its raw sigmoid score
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


def ling_router_terms(observations, objective_weights, denominator, z_coefficient, cp_group=None):
    mask = (objective_weights.reshape(-1) > 0).float()
    counts = torch.stack([(F.one_hot(sel, lg.shape[-1]).sum(1).float() * mask[:, None]).sum(0) for lg, sel in observations])
    z_sums = torch.stack([(lg.float().logsumexp(-1).square() * mask).sum() for lg, _ in observations])
    count = mask.sum()
    metric_counts = counts.detach().clone()
    if cp_group is not None:
        import torch.distributed as dist
        from torch.distributed.nn.functional import all_reduce
        z_sums = all_reduce(z_sums, group=cp_group)
        count = count.clone()
        dist.all_reduce(count, group=cp_group)
        dist.all_reduce(metric_counts, group=cp_group)
    num = z_sums.sum() / count.clamp_min(1) * denominator
    top_k = observations[0][1].shape[-1]
    load = metric_counts / (count.clamp_min(1) * top_k)
    d = denominator.detach()
    return z_coefficient * num, {
        "router_z_loss": (num.detach(), d), "router_max_load": ((load.max() * denominator).detach(), d),
        "router_used_experts": (((metric_counts > 0).sum(-1).float().mean() * denominator).detach(), d),
        "_ling_router_counts": counts.detach()}


@torch.no_grad()
def update_ling_bias(layers, counts, update_rate: float, zero_mean: bool = True, group=None, apply_update=True) -> None:
    """After each committed optimizer step: ``bias += rate * (sign(mean - count) [- its mean])`` per layer."""
    if group is not None:
        import torch.distributed as dist
        dist.all_reduce(counts, group=group)
    sign = (counts.mean(-1, keepdim=True) - counts).sign()
    if zero_mean:
        sign = sign - sign.mean(-1, keepdim=True)
    active = (counts.sum(-1, keepdim=True) > 0) & torch.as_tensor(apply_update, device=counts.device)
    delta = torch.where(active, sign * update_rate, torch.zeros_like(sign))
    for layer, change in zip(layers, delta):
        if layer.gate.bias_enabled:
            layer.gate.expert_bias.add_(change)
