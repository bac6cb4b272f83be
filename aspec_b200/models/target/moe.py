"""Mixture-of-experts feed-forward of a Ling / DeepSeek-style Target, inference only (the reference serves such
Targets through its serving engine's ``bailing_moe`` models: compat/patches/sglang-v0.5.21.patch:389-689).

Routing: fp32 ``sigmoid(W_g x)``; the selection score adds ``expert_bias``; groups are ranked by the sum of their
top-2 scores and ``topk_group`` groups stay; top-k inside; combine weights are the un-biased scores, renormalised
and scaled by ``routed_scaling_factor``.  Tokens are sorted by expert once, every expert runs two GEMMs on its
contiguous slice (on CUDA all experts of a layer share two grouped tcgen05 launches), results are scattered back with
``index_add``; the shared expert is a dense SwiGLU on all tokens.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class TargetMoE(nn.Module):
    """``tp_size > 1``: this rank holds ``E / tp_size`` whole experts and ``1 / tp_size`` of the shared expert's width; every
    rank routes all tokens (the router is replicated), runs the rows that chose its experts, and returns a PARTIAL sum
    that the caller adds up over the group."""

    def __init__(self, cfg, tp_rank: int = 0, tp_size: int = 1):
        super().__init__()
        D, E, I = cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size
        self.cfg = cfg
        self.num_experts, self.local_experts, self.first_expert = E, E // tp_size, tp_rank * (E // tp_size)
        self.top_k = cfg.num_experts_per_tok
        self.n_group, self.topk_group = max(cfg.n_group, 1), max(cfg.topk_group, 1)
        self.scale = cfg.routed_scaling_factor
        self.gate = nn.Parameter(torch.empty(E, D))
        self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32))
        self.gate_up_proj = nn.Parameter(torch.empty(self.local_experts, 2 * I, D))      # rows [gate | up] per expert
        self.down_proj = nn.Parameter(torch.empty(self.local_experts, D, I))
        if cfg.num_shared_experts:
            Is = (cfg.moe_shared_expert_intermediate_size or I) * cfg.num_shared_experts
            if Is % tp_size:
                raise ValueError(f"tensor parallel size {tp_size} must divide the shared expert width ({Is})")
            Is //= tp_size
            self.shared_gate_up = nn.Parameter(torch.empty(2 * Is, D))
            self.shared_down = nn.Parameter(torch.empty(D, Is))
        else:
            self.shared_gate_up = self.shared_down = None

    def _apply(self, fn, recurse=True):
        bias = self.expert_bias
        super()._apply(fn, recurse)
        self.expert_bias = bias.to(device=self.expert_bias.device, dtype=torch.float32)
        return self

    def route(self, x: torch.Tensor):
        scores = torch.sigmoid(F.linear(x.float(), self.gate.float()))
        biased = scores + self.expert_bias
        if self.n_group > 1:
            g = biased.unflatten(-1, (self.n_group, -1))
            keep = g.topk(min(2, g.shape[-1]), -1).values.sum(-1).topk(self.topk_group, -1).indices
            drop = torch.ones_like(g[..., 0], dtype=torch.bool).scatter_(1, keep, False)
            biased = g.masked_fill(drop[..., None], float("-inf")).flatten(1)
        idx = biased.topk(self.top_k, -1).indices
        w = scores.gather(1, idx)
        if self.top_k > 1:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        return idx, w * self.scale

    @staticmethod
    def _swiglu_mlp(x, gate_up, down):
        if x.is_cuda and x.dtype == torch.bfloat16:
            from aspec_b200.ops import gemm as G
            from aspec_b200.ops.activation import swiglu
            return G.gemm(swiglu(G.gemm(x, gate_up)), down)
        g, u = F.linear(x, gate_up).chunk(2, -1)
        return F.linear(F.silu(g) * u, down)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T, D = x.shape
        idx, w = self.route(x)
        flat = idx.flatten()
        order = flat.argsort(stable=True)
        tokens = order // self.top_k
        counts = torch.bincount(flat, minlength=self.gate.shape[0]).tolist()      # one host read per MoE layer
        if self.local_experts != self.num_experts:
            # the sorted rows of this rank's experts are one contiguous run
            lo = sum(counts[: self.first_expert])
            counts = counts[self.first_expert: self.first_expert + self.local_experts]
            order = order[lo: lo + sum(counts)]
            tokens = tokens[lo: lo + sum(counts)]
        rows = x[tokens].contiguous()
        out = torch.zeros(T, D, device=x.device, dtype=torch.float32)
        I = self.gate_up_proj.shape[1] // 2
        if x.is_cuda and x.dtype == torch.bfloat16 and D % 64 == 0 and I % 64 == 0 and rows.shape[0]:
            # all experts in two grouped tcgen05 launches (gate/up with the SwiGLU between, then down)
            from aspec_b200.ops.grouped_gemm import grouped_experts
            y = grouped_experts(rows, self.gate_up_proj, self.down_proj, counts, 0.0)
            out.index_add_(0, tokens, y.float() * w.flatten()[order, None])
            counts = []
        off = 0
        for e, n in enumerate(counts):
            if n:
                y = self._swiglu_mlp(rows[off:off + n], self.gate_up_proj[e], self.down_proj[e])
                out.index_add_(0, tokens[off:off + n], y.float() * w.flatten()[order[off:off + n], None])
                off += n
        out = out.to(x.dtype)
        if self.shared_gate_up is not None:
            out = out + self._swiglu_mlp(x, self.shared_gate_up, self.shared_down)
        return out
