"""Mixture-of-experts feed-forward of the EAGLE4 Draft.

Two expert layouts share one module (parameter names follow the reference's checkpoints,
aspec/models/draft/eagle4_moe.py:38-213, so its weights load unchanged):

* ``sparse_swiglu``: ``experts.w13_weight [E, 2I, D]`` (gate rows, then up rows) and ``experts.w2_weight [E, D, I]``;
  on CUDA in bf16 the whole bank runs as grouped tcgen05 launches (``ops/grouped_gemm.py``);
* ``nemotron_latent_relu2``: the tokens are projected to a latent width, every expert is ``down(relu(up(x))^2)`` in
  that width, and the sum is projected back.

Routing is sigmoid scoring with a selection-only bias: ``sigmoid(W x) + bias`` picks the experts (optionally only
inside the ``topk_group`` groups whose two best biased scores sum highest), the unbiased scores of the picked experts
are the mixing weights (renormalised, then scaled).  The bias is the loss-free balancer: once per optimizer step it
moves by ``rate * sign(mean load - load)`` with the load counted on valid query rows.  ``down`` projections start at
zero, so a freshly initialised routed bank adds nothing to the residual stream.
"""
from __future__ import annotations

import re
from collections import defaultdict
from typing import Callable, Dict, List, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.ops.linear import Linear, linear

LATENT_MOE = "nemotron_latent_relu2"

_ACTIVATIONS: Dict[str, Callable[[torch.Tensor], torch.Tensor]] = {
    "silu": F.silu, "gelu": F.gelu, "relu": F.relu, "relu2": lambda t: F.relu(t).square()}


def select_experts(scores: torch.Tensor, bias: torch.Tensor, top_k: int, n_group: int, topk_group: int) -> torch.Tensor:
    """Indices ``[N, top_k]`` of the experts with the highest biased scores, restricted to the best groups."""
    ranked = scores + bias
    if n_group > 1:
        per_group = ranked.view(ranked.shape[0], n_group, -1)
        group_value = per_group.topk(min(2, per_group.shape[-1]), dim=-1).values.sum(-1)   # two best members speak for a group
        chosen = group_value.topk(topk_group, dim=-1).indices
        allowed = torch.zeros_like(group_value, dtype=torch.bool).scatter_(1, chosen, True)
        ranked = per_group.masked_fill(~allowed[..., None], float("-inf")).flatten(1)
    return ranked.topk(top_k, dim=-1).indices


class Eagle4Router(nn.Module):
    """Scoring matrix, the balancing bias (kept in fp32 whatever the module is cast to) and the load counter."""

    def __init__(self, config):
        super().__init__()
        experts = int(config.n_routed_experts)
        std = getattr(config, "initializer_range", 0.02)
        self.weight = nn.Parameter(torch.randn(experts, config.hidden_size) * std)
        self.register_buffer("e_score_correction_bias", torch.zeros(experts))
        self.register_buffer("load", torch.zeros(experts, dtype=torch.long), persistent=False)
        rate = getattr(config, "expert_bias_update_rate", None)
        self.update_rate = rate if rate is not None else getattr(config, "moe_router_bias_update_rate", 1e-3)

    def _apply(self, fn, recurse=True):
        # steps of 1e-3 vanish in bf16 once the bias is a few tenths: carry the fp32 values across any cast
        exact = self.e_score_correction_bias.detach().float().clone()
        super()._apply(fn, recurse)
        self.e_score_correction_bias = exact.to(self.e_score_correction_bias.device)
        return self

    def scores(self, x: torch.Tensor) -> torch.Tensor:
        return torch.sigmoid(x.float() @ self.weight.float().t())

    @torch.no_grad()
    def update_bias(self, *, apply_update: bool = True, group=None) -> torch.Tensor:
        """Fold the committed load into the bias (once per optimizer step).  Returns max load / mean load."""
        counts = self.load.to(torch.float32)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(counts, group=group)
        self.load.zero_()
        mean = counts.mean()
        if apply_update and counts.sum().item() > 0:
            self.e_score_correction_bias += self.update_rate * torch.sign(mean - counts)
        return counts.max() / mean.clamp_min(1.0)


class SharedExpert(nn.Module):
    """Always-on expert: gated (``act(gate) * up``) for the SwiGLU layout, plain ``act(up)`` for the latent layout."""

    def __init__(self, hidden_size: int, intermediate_size: int, act, gated: bool):
        super().__init__()
        self.act = act
        self.up_proj = Linear(hidden_size, intermediate_size)
        self.down_proj = Linear(intermediate_size, hidden_size)
        if gated:
            self.gate_proj = Linear(hidden_size, intermediate_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        inner = self.up_proj(x)
        inner = self.act(self.gate_proj(x)) * inner if hasattr(self, "gate_proj") else self.act(inner)
        return self.down_proj(inner)


class Eagle4MoE(nn.Module):
    def __init__(self, config):
        super().__init__()
        hidden, inter, experts = config.hidden_size, config.moe_intermediate_size, int(config.n_routed_experts)
        std = getattr(config, "initializer_range", 0.02)
        self.latent = getattr(config, "moe_architecture", "sparse_swiglu") == LATENT_MOE
        self.hidden_act = config.hidden_act
        self.act = _ACTIVATIONS[config.hidden_act]
        self.top_k = int(config.num_experts_per_tok)
        self.n_group = getattr(config, "n_group", None) or 1
        self.topk_group = getattr(config, "topk_group", None) or self.n_group
        self.norm_topk_prob = getattr(config, "norm_topk_prob", True)
        self.routed_scaling_factor = getattr(config, "routed_scaling_factor", 1.0)
        self.gate = Eagle4Router(config)
        expert_width = config.moe_latent_size if self.latent else hidden
        first_rows = inter if self.latent else 2 * inter
        self.expert_names = ("up_proj", "down_proj") if self.latent else ("w13_weight", "w2_weight")
        self.experts = nn.ParameterDict({
            self.expert_names[0]: nn.Parameter(torch.randn(experts, first_rows, expert_width) * std),
            self.expert_names[1]: nn.Parameter(torch.zeros(experts, expert_width, inter))})
        if self.latent:
            self.fc1_latent_proj = Linear(hidden, expert_width)
            self.fc2_latent_proj = Linear(expert_width, hidden)
        shared = getattr(config, "n_shared_experts", None) or 0
        self.shared_experts = None
        if shared:
            shared_inter = (config.moe_shared_expert_intermediate_size if self.latent else inter) * shared
            self.shared_experts = SharedExpert(hidden, shared_inter, self.act, gated=not self.latent)
        self.query_mask = None          # set by the training wrapper: rows that count for the load statistics
        self.last_load = None

    # -- routing ----------------------------------------------------------------------------------------------------
    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        scores = self.gate.scores(x)
        picked = select_experts(scores, self.gate.e_score_correction_bias, self.top_k, self.n_group, self.topk_group)
        mix = torch.gather(scores, 1, picked)
        if self.norm_topk_prob:
            mix = mix / mix.sum(-1, keepdim=True)
        return picked, mix * self.routed_scaling_factor

    def _record_load(self, picked: torch.Tensor) -> None:
        if not (self.training and any(p.requires_grad for p in self.parameters())):
            return
        per_row = torch.ones_like(picked)
        if self.query_mask is not None:
            per_row = self.query_mask.reshape(-1, 1).to(picked.dtype).expand_as(picked)
        self.last_load = picked.new_zeros(self.gate.weight.shape[0]).scatter_add_(0, picked.reshape(-1), per_row.reshape(-1))

    # -- experts ----------------------------------------------------------------------------------------------------
    def _bank(self, rows: torch.Tensor, counts: List[int]) -> torch.Tensor:
        """``rows`` sorted by expert (``counts[e]`` each) -> expert outputs in the same order."""
        first, second = (self.experts[name] for name in self.expert_names)
        swiglu_kernel = (not self.latent and self.hidden_act == "silu" and rows.is_cuda and rows.dtype == torch.bfloat16
                         and first.dtype == torch.bfloat16 and rows.shape[0] > 0 and rows.shape[1] % 64 == 0
                         and second.shape[2] % 64 == 0)
        if swiglu_kernel:
            from aspec_b200.ops.grouped_gemm import grouped_experts
            return grouped_experts(rows, first, second, counts)
        pieces, start = [], 0
        for e, n in enumerate(counts):
            if n:
                inner = linear(rows[start:start + n], first[e].to(rows.dtype))
                if self.latent:
                    inner = self.act(inner)
                else:
                    gate, value = inner.chunk(2, dim=-1)
                    inner = self.act(gate) * value
                pieces.append(linear(inner.contiguous(), second[e].to(rows.dtype)))
            start += n
        anchor = (first.sum() + second.sum()).to(rows.dtype) * 0.0          # experts without rows still get (zero) grads
        return (torch.cat(pieces, 0) if pieces else rows.new_zeros(0, second.shape[1])) + anchor

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        picked, mix = self.route(x)
        self._record_load(picked)
        flat = picked.reshape(-1)
        by_expert = torch.argsort(flat)
        token_of = by_expert // self.top_k
        counts = torch.bincount(flat, minlength=self.gate.weight.shape[0]).tolist()
        inner_x = self.fc1_latent_proj(x) if self.latent else x
        produced = self._bank(inner_x[token_of], counts)
        produced = produced * mix.reshape(-1)[by_expert].unsqueeze(-1).to(produced.dtype)
        routed = torch.zeros_like(inner_x).index_add_(0, token_of, produced)
        out = self.fc2_latent_proj(routed) if self.latent else routed
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        return out.reshape(hidden_states.shape)


# -- checkpoint layouts of the latent experts --------------------------------------------------------------------------
_STACKED = re.compile(r"(?P<bank>.*\.experts)\.(?P<proj>up_proj|down_proj)")
_SINGLE = re.compile(r"(?P<bank>.*\.experts)\.(?P<index>\d+)\.(?P<proj>up_proj|down_proj)\.weight")


def split_latent_experts(tensors: dict) -> dict:
    """``...experts.up_proj [E, ...]`` -> ``...experts.<e>.up_proj.weight`` (one tensor per expert, as serving loaders read them)."""
    result = {}
    for name, tensor in tensors.items():
        hit = _STACKED.fullmatch(name)
        if hit is None:
            result[name] = tensor
            continue
        for index, one in enumerate(tensor.unbind(0)):
            result[f"{hit['bank']}.{index}.{hit['proj']}.weight"] = one.clone()
    return result


def stack_latent_experts(tensors: dict) -> dict:
    """Inverse of ``split_latent_experts``."""
    result, banks = {}, defaultdict(dict)
    for name, tensor in tensors.items():
        hit = _SINGLE.fullmatch(name)
        if hit is None:
            result[name] = tensor
        else:
            banks[f"{hit['bank']}.{hit['proj']}"][int(hit["index"])] = tensor
    for name, members in banks.items():
        result[name] = torch.stack([members[i] for i in sorted(members)])
    return result
