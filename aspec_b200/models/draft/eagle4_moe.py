"""EAGLE4 MoE feed-forward: sigmoid router with a loss-free load-balancing bias, packed routed experts
(``sparse_swiglu`` as ``w13 | w2``, or ``nemotron_latent_relu2`` running ReLU^2 experts in a latent width between two
dense projections) and optional shared experts (reference: aspec/models/draft/eagle4_moe.py:38-213).

Routing: ``scores = sigmoid(W x)`` in fp32; the bias only selects (optionally group-limited by the sum of each
group's top-2), the un-biased scores weight the selected experts, renormalised and scaled.  ``down`` projections
start at zero so that a freshly added routed bank is a no-op.  The load observed on valid query rows is committed
to the router once per optimizer step and moves the bias by ``rate * sign(mean - load)``.
"""
from __future__ import annotations

import re
from collections import defaultdict

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.ops.linear import Linear, linear

LATENT_MOE = "nemotron_latent_relu2"
_PACKED = re.compile(r"(.*\.experts)\.(up_proj|down_proj)")
_PER_EXPERT = re.compile(r"(.*\.experts)\.(\d+)\.(up_proj|down_proj)\.weight")


def _activation(name: str):
    if name == "relu2":
        return lambda x: F.relu(x).square()
    return {"silu": F.silu, "gelu": F.gelu, "relu": F.relu}[name]


class Eagle4Router(nn.Module):
    def __init__(self, config):
        super().__init__()
        n = config.n_routed_experts
        self.weight = nn.Parameter(torch.empty(n, config.hidden_size).normal_(std=getattr(config, "initializer_range", 0.02)))
        self.register_buffer("e_score_correction_bias", torch.zeros(n))
        self.register_buffer("load", torch.zeros(n, dtype=torch.long), persistent=False)
        self.update_rate = getattr(config, "expert_bias_update_rate", getattr(config, "moe_router_bias_update_rate", 1e-3))

    def _apply(self, fn, recurse=True):
        bias = self.e_score_correction_bias
        super()._apply(fn, recurse)
        # bf16 cannot represent 1e-3 steps once |bias| passes 0.25, so the bias keeps fp32 through casts
        self.e_score_correction_bias = bias.to(device=self.e_score_correction_bias.device, dtype=torch.float32)
        return self

    @torch.no_grad()
    def update_bias(self, *, apply_update: bool = True, group=None) -> torch.Tensor:
        """Once per optimizer step; returns max / mean expert load."""
        load = self.load.float()
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(load, group=group)
        self.load.zero_()
        if apply_update and float(load.sum()) > 0:
            self.e_score_correction_bias.add_(self.update_rate * (load.mean() - load).sign())
        return load.max() / load.mean().clamp_min(1.0)


class SharedExpert(nn.Module):
    def __init__(self, hidden_size, intermediate_size, act, gated):
        super().__init__()
        if gated:
            self.gate_proj = Linear(hidden_size, intermediate_size)
        self.up_proj = Linear(hidden_size, intermediate_size)
        self.down_proj = Linear(intermediate_size, hidden_size)
        self.act = act

    def forward(self, x):
        h = self.up_proj(x)
        return self.down_proj(self.act(self.gate_proj(x)) * h if hasattr(self, "gate_proj") else self.act(h))


class Eagle4MoE(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.latent = getattr(config, "moe_architecture", "sparse_swiglu") == LATENT_MOE
        self.top_k = config.num_experts_per_tok
        self.n_group = getattr(config, "n_group", None) or 1
        self.topk_group = getattr(config, "topk_group", None) or self.n_group
        self.norm_topk_prob = getattr(config, "norm_topk_prob", True)
        self.routed_scaling_factor = getattr(config, "routed_scaling_factor", 1.0)
        self.act = _activation(config.hidden_act)
        n, D, inter = config.n_routed_experts, config.hidden_size, config.moe_intermediate_size
        width = config.moe_latent_size if self.latent else D
        self.gate = Eagle4Router(config)
        up = torch.empty(n, inter if self.latent else 2 * inter, width).normal_(std=getattr(config, "initializer_range", 0.02))
        self.expert_names = ("up_proj", "down_proj") if self.latent else ("w13_weight", "w2_weight")
        self.experts = nn.ParameterDict({self.expert_names[0]: nn.Parameter(up),
                                         self.expert_names[1]: nn.Parameter(torch.zeros(n, width, inter))})
        if self.latent:
            self.fc1_latent_proj = Linear(D, width)
            self.fc2_latent_proj = Linear(width, D)
        n_shared = getattr(config, "n_shared_experts", None) or 0
        shared_inter = config.moe_shared_expert_intermediate_size if self.latent else inter
        self.shared_experts = SharedExpert(D, shared_inter * n_shared, self.act, gated=not self.latent) if n_shared else None
        self.query_mask = None
        self.last_load = None

    def route(self, x):
        scores = F.linear(x.float(), self.gate.weight.float()).sigmoid()
        biased = scores + self.gate.e_score_correction_bias
        if self.n_group > 1:
            groups = biased.unflatten(-1, (self.n_group, -1))
            best = groups.topk(2, -1).values.sum(-1).topk(self.topk_group, -1).indices
            dropped = torch.ones_like(groups[..., 0], dtype=torch.bool).scatter_(1, best, False)
            biased = groups.masked_fill(dropped[..., None], float("-inf")).flatten(1)
        idx = biased.topk(self.top_k, -1).indices
        w = scores.gather(1, idx)
        if self.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        return idx, w * self.routed_scaling_factor

    def forward(self, hidden_states):
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        idx, weights = self.route(x)
        n_exp = self.gate.weight.shape[0]
        if self.training and any(p.requires_grad for p in self.parameters()):
            mask = self.query_mask
            lw = torch.ones_like(idx) if mask is None else mask.reshape(-1, 1).expand_as(idx).to(idx.dtype)
            self.last_load = idx.new_zeros(n_exp).scatter_add_(0, idx.flatten(), lw.flatten())
        order = idx.flatten().argsort()
        tokens = order // self.top_k
        counts = torch.bincount(idx.flatten(), minlength=n_exp).tolist()
        h = self.fc1_latent_proj(x) if self.latent else x
        up, down = (self.experts[name] for name in self.expert_names)
        rows = h[tokens]
        outs, off = [], 0
        for e, c in enumerate(counts):
            if c == 0:
                continue
            inner = linear(rows[off:off + c], up[e].to(rows.dtype))
            if self.latent:
                inner = self.act(inner)
            else:
                g, v = inner.chunk(2, -1)
                inner = self.act(g) * v
            outs.append(linear(inner.contiguous(), down[e].to(rows.dtype)))
            off += c
        out = torch.cat(outs, 0) * weights.flatten()[order, None].to(rows.dtype)
        out = h.new_zeros(h.shape).index_add_(0, tokens, out) + 0.0 * (up.sum() + down.sum()).to(h.dtype)
        if self.latent:
            out = self.fc2_latent_proj(out)
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        return out.view_as(hidden_states)


def split_latent_experts(tensors: dict) -> dict:
    """Packed latent experts -> one key per expert (the layout the serving loader reads)."""
    out = {}
    for key, value in tensors.items():
        m = _PACKED.fullmatch(key)
        if m:
            out.update({f"{m[1]}.{i}.{m[2]}.weight": w.clone() for i, w in enumerate(value)})
        else:
            out[key] = value
    return out


def stack_latent_experts(tensors: dict) -> dict:
    out, groups = {}, defaultdict(dict)
    for key, value in tensors.items():
        m = _PER_EXPERT.fullmatch(key)
        if m:
            groups[f"{m[1]}.{m[3]}"][int(m[2])] = value
        else:
            out[key] = value
    out.update({k: torch.stack([g[i] for i in sorted(g)]) for k, g in groups.items()})
    return out
