"""Mixture-of-experts FFNs for Draft layers: Qwen3-MoE and the shared expert bank.

Routing semantics follow the reference (aspec/models/draft/moe.py:25-93): softmax over experts in fp32, top-k,
optional renormalisation, weighted sum of SwiGLU experts, and a load-balancing auxiliary loss over the
supervised draft slots.  Storage and execution are different: the experts live in two stacked tensors
(``gate_up_proj [E, 2I, D]``, ``down_proj [E, D, I]``); tokens are sorted by expert once and every expert runs
one GEMM over its contiguous slice (tcgen05 GEMM on CUDA).  With expert parallelism each rank holds
``E / ep`` experts and the sorted token slices are exchanged with an all-to-all before and after
(``parallel.expert_parallel``).  Checkpoints written with one module per expert
(``experts.<i>.gate_proj.weight`` ...) are accepted on load.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from aspec_b200.ops.activation import swiglu
from aspec_b200.ops.linear import Linear, linear


class ExpertBank(nn.Module):
    """``E`` SwiGLU experts in stacked storage; ``forward`` takes tokens already sorted by expert."""

    def __init__(self, num_experts: int, hidden_size: int, intermediate_size: int, clamp: float = 0.0,
                 ep_rank: int = 0, ep_size: int = 1):
        super().__init__()
        if num_experts % ep_size:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.num_experts, self.ep_rank, self.ep_size = num_experts, ep_rank, ep_size
        self.local_experts = num_experts // ep_size
        self.first_expert = ep_rank * self.local_experts
        self.intermediate_size, self.clamp = intermediate_size, clamp
        self.gate_up_proj = nn.Parameter(torch.empty(self.local_experts, 2 * intermediate_size, hidden_size))
        self.down_proj = nn.Parameter(torch.empty(self.local_experts, hidden_size, intermediate_size))
        nn.init.normal_(self.gate_up_proj, std=0.02)
        nn.init.normal_(self.down_proj, std=0.02)
        self.ep_group = None          # process group of the ranks that together hold all experts
        self.fused_ep = None          # parallel.expert_parallel.FusedExpertParallel when peer memory is set up
        self._register_state_dict_hook(ExpertBank._full_bank_state)

    # -- expert parallelism: each rank keeps ``E / ep`` experts; state dicts always show the whole bank ------------
    @torch.no_grad()
    def shard_(self, ep_rank: int, ep_size: int, group=None) -> "ExpertBank":
        """Keep only this rank's experts of a bank that was built whole (every rank built it from the same seed or
        loaded the same weights).  Checkpoints stay topology-independent: ``state_dict`` gathers the bank over
        ``group`` and ``load_state_dict`` slices a whole bank down to the local experts."""
        if self.ep_size != 1:
            raise ValueError("the bank is already sharded")
        if self.num_experts % ep_size:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        local = self.num_experts // ep_size
        first = ep_rank * local
        for name in ("gate_up_proj", "down_proj"):
            full = getattr(self, name)
            part = nn.Parameter(full.detach()[first:first + local].clone(), requires_grad=full.requires_grad)
            part.expert_parallel = True          # the optimizer reduces these over expert replicas only
            setattr(self, name, part)
        self.ep_rank, self.ep_size, self.local_experts, self.first_expert, self.ep_group = ep_rank, ep_size, local, first, group
        return self

    @staticmethod
    def _full_bank_state(module, state_dict, prefix, local_metadata):
        if module.ep_size > 1 and module.ep_group is not None:
            import torch.distributed as dist
            for name in ("gate_up_proj", "down_proj"):
                part = state_dict[prefix + name]
                pieces = [torch.empty_like(part) for _ in range(module.ep_size)]
                dist.all_gather(pieces, part.contiguous(), group=module.ep_group)
                state_dict[prefix + name] = torch.cat(pieces, 0)
        return state_dict

    def forward(self, x_sorted: torch.Tensor, counts: List[int]) -> torch.Tensor:
        """``x_sorted [N, D]`` grouped by local expert, ``counts[e]`` rows each -> ``[N, D]``."""
        if (x_sorted.is_cuda and x_sorted.dtype == torch.bfloat16 and self.gate_up_proj.dtype == torch.bfloat16 and x_sorted.shape[0]
                and x_sorted.shape[1] % 64 == 0 and self.intermediate_size % 64 == 0):
            from aspec_b200.ops.grouped_gemm import grouped_experts
            return grouped_experts(x_sorted, self.gate_up_proj, self.down_proj, counts, self.clamp)
        outs = []
        off = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            xe = x_sorted[off:off + n]
            act = swiglu(linear(xe, self.gate_up_proj[e]), self.clamp)
            outs.append(linear(act, self.down_proj[e]))
            off += n
        if not outs:
            return x_sorted.new_zeros(0, x_sorted.shape[-1]) + 0.0 * (self.gate_up_proj.sum() + self.down_proj.sum())
        return torch.cat(outs, 0)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # accept one-module-per-expert checkpoints
        key = f"{prefix}0.gate_proj.weight"
        if key in state_dict and f"{prefix}gate_up_proj" not in state_dict:
            gu, dn = [], []
            for e in range(self.first_expert, self.first_expert + self.local_experts):
                g = state_dict.pop(f"{prefix}{e}.gate_proj.weight")
                u = state_dict.pop(f"{prefix}{e}.up_proj.weight")
                gu.append(torch.cat([g, u], 0))
                dn.append(state_dict.pop(f"{prefix}{e}.down_proj.weight"))
            for k in [k for k in state_dict if k.startswith(prefix) and k[len(prefix):].split(".")[0].isdigit()]:
                state_dict.pop(k)
            state_dict[f"{prefix}gate_up_proj"] = torch.stack(gu)
            state_dict[f"{prefix}down_proj"] = torch.stack(dn)
        if self.ep_size > 1:
            # a whole bank (any checkpoint) is cut down to this rank's experts
            for name in ("gate_up_proj", "down_proj"):
                t = state_dict.get(prefix + name)
                if t is not None and t.shape[0] == self.num_experts:
                    state_dict[prefix + name] = t[self.first_expert:self.first_expert + self.local_experts]
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


def route_and_run(bank: ExpertBank, hidden: torch.Tensor, selected: torch.Tensor, weights: torch.Tensor,
                  ep_group=None, fp32_accumulate: bool = False) -> torch.Tensor:
    """Dispatch ``hidden [N, D]`` to its ``selected [N, k]`` experts, run them, combine with ``weights [N, k]``."""
    N, k = selected.shape
    flat_expert = selected.reshape(-1)
    order = torch.argsort(flat_expert, stable=True)
    token_of = order // k
    sorted_expert = flat_expert[order]
    x_sorted = hidden.index_select(0, token_of)        # backward: atomic index_add_ (every token repeats top-k times)
    if bank.ep_size > 1:
        group = ep_group if ep_group is not None else bank.ep_group
        if bank.fused_ep is not None and x_sorted.is_cuda:
            # dispatch and combine are the grouped expert GEMMs' own loads and stores over peer memory
            from aspec_b200.parallel.expert_parallel import fused_dispatch_combine
            y_sorted = fused_dispatch_combine(bank.fused_ep, bank, x_sorted, sorted_expert, group)
        else:
            from aspec_b200.parallel.expert_parallel import dispatch_combine
            y_sorted = dispatch_combine(bank, x_sorted, sorted_expert, group)
    else:
        counts = torch.bincount(sorted_expert, minlength=bank.num_experts).tolist()
        y_sorted = bank(x_sorted, counts)
    w_sorted = weights.reshape(-1)[order]
    acc_dtype = torch.float32 if fp32_accumulate else hidden.dtype
    out = torch.zeros(N, hidden.shape[-1], device=hidden.device, dtype=acc_dtype)
    out.index_add_(0, token_of, (y_sorted.to(acc_dtype) * w_sorted[:, None].to(acc_dtype)))
    return out.to(hidden.dtype)


class QwenMoE(nn.Module):
    wants_aux = True

    def __init__(self, config, ep_rank: int = 0, ep_size: int = 1, ep_group=None):
        super().__init__()
        self.num_experts, self.top_k = config.num_experts, config.num_experts_per_tok
        self.norm_topk_prob = config.norm_topk_prob
        self.gate = Linear(config.hidden_size, self.num_experts)
        self.experts = ExpertBank(self.num_experts, config.hidden_size, config.moe_intermediate_size,
                                  ep_rank=ep_rank, ep_size=ep_size)
        self.ep_group = ep_group

    def forward(self, x: torch.Tensor, aux: Optional[dict] = None) -> torch.Tensor:
        shape = x.shape
        h = x.reshape(-1, shape[-1])
        logits = F.linear(h.float(), self.gate.weight.float())
        probs = torch.softmax(logits, -1)
        w, selected = probs.topk(self.top_k, -1)
        if self.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        out = route_and_run(self.experts, h, selected, w.to(h.dtype), self.ep_group)
        if aux is not None:
            aux.setdefault("router_logits", []).append(logits)
        return out.reshape(shape)


def router_loss_terms(router_logits, objective_weights, denominator, top_k, cp_group=None):
    """Load-balancing loss ``E * sum_e load_e * importance_e`` over supervised slots, all MoE layers pooled."""
    logits = torch.cat(router_logits, 0)
    mask = (objective_weights.reshape(-1) > 0).float().repeat(len(router_logits))
    probs = torch.softmax(logits.float(), -1)
    sel = probs.topk(top_k, -1).indices
    expert_mask = F.one_hot(sel, logits.shape[-1]).sum(1).float()
    count = mask.sum()
    load_sum = (expert_mask * mask[:, None]).sum(0)
    importance_sum = (probs * mask[:, None]).sum(0)
    if cp_group is not None:
        import torch.distributed as dist
        from torch.distributed.nn.functional import all_reduce
        totals = torch.cat([count.reshape(1), load_sum])
        dist.all_reduce(totals, group=cp_group)
        count, load_sum = totals[0], totals[1:]
        importance_sum = all_reduce(importance_sum, group=cp_group)
    safe = count.clamp_min(1)
    load, importance = load_sum / safe, importance_sum / safe
    aux = logits.shape[-1] * (load * importance).sum()
    num = aux * denominator
    d = denominator.detach()
    return num, {"router_aux_loss": (num.detach(), d), "router_max_load": ((load.max() / top_k * denominator).detach(), d),
                 "router_used_experts": (((load > 0).sum() * denominator).detach(), d)}
