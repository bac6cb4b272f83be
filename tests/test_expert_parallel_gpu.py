"""Fused expert-parallel dispatch / combine over peer memory: two ranks emulated on one GPU against the replicated
expert bank (every expert on one rank)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_emulated_ranks_match_the_replicated_bank():
    from aspec_b200.models.draft.moe import ExpertBank
    from aspec_b200.parallel.expert_parallel import EPWorkspace, FusedExpertParallel
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    world, E, D, I, N, k = 2, 4, 256, 128, 300, 2
    bf = torch.bfloat16
    full = ExpertBank(E, D, I).to(dev, bf)
    banks = [ExpertBank(E, D, I, ep_rank=r, ep_size=world).to(dev, bf) for r in range(world)]
    for r, b in enumerate(banks):
        b.gate_up_proj.data.copy_(full.gate_up_proj.data[r * 2:(r + 1) * 2])
        b.down_proj.data.copy_(full.down_proj.data[r * 2:(r + 1) * 2])
    xs, experts, refs, dys = [], [], [], []
    for r in range(world):
        x = (torch.randn(N, D, device=dev) * 0.5).to(bf)
        sel = torch.randint(0, E, (N * k,), device=dev)
        order = torch.argsort(sel, stable=True)
        x_sorted = x.repeat_interleave(k, 0)[order].contiguous().requires_grad_(True)
        sorted_e = sel[order]
        y = full(x_sorted, torch.bincount(sorted_e, minlength=E).tolist())
        dy = (torch.randn_like(y) * 0.1)
        y.backward(dy)
        xs.append(x_sorted)
        experts.append(sorted_e)
        refs.append((y.detach(), x_sorted.grad.clone()))
        dys.append(dy)
    ref_dgu, ref_ddn = full.gate_up_proj.grad.float(), full.down_proj.grad.float()
    counts = [torch.bincount(e, minlength=E).tolist() for e in experts]
    ws = [EPWorkspace(N * k, D, device=dev) for _ in range(world)]
    eps = [FusedExpertParallel(r, world, E, ws) for r in range(world)]
    for r in range(world):
        eps[r].publish(xs[r].detach())
    for r in range(world):
        eps[r].run_experts(counts, banks[r].gate_up_proj.detach(), banks[r].down_proj.detach())
    for r in range(world):
        assert torch.allclose(eps[r].collect().float(), refs[r][0].float(), rtol=3e-2, atol=3e-2)
    for r in range(world):
        eps[r].publish_grad(dys[r])
    grads = [eps[r].run_experts_backward(banks[r].gate_up_proj.detach(), banks[r].down_proj.detach()) for r in range(world)]
    for r in range(world):
        gx = eps[r].collect_grad().float()
        assert torch.allclose(gx, refs[r][1].float(), rtol=5e-2, atol=2e-2 * refs[r][1].float().abs().max().item())
        d_gu, d_dn = grads[r]
        want_gu, want_dn = ref_dgu[r * 2:(r + 1) * 2], ref_ddn[r * 2:(r + 1) * 2]
        assert torch.allclose(d_gu, want_gu, rtol=5e-2, atol=3e-2 * want_gu.abs().max().item())
        assert torch.allclose(d_dn, want_dn, rtol=5e-2, atol=3e-2 * want_dn.abs().max().item())


def test_a_rank_whose_experts_receive_no_rows_returns_zero_gradients():
    """Group-limited routing can send every token of a micro-batch to the experts of other ranks."""
    from aspec_b200.models.draft.moe import ExpertBank
    from aspec_b200.parallel.expert_parallel import EPWorkspace, FusedExpertParallel
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    world, E, D, I, N = 2, 4, 256, 128, 96
    bf = torch.bfloat16
    full = ExpertBank(E, D, I).to(dev, bf)
    banks = [ExpertBank(E, D, I, ep_rank=r, ep_size=world).to(dev, bf) for r in range(world)]
    for r, b in enumerate(banks):
        b.gate_up_proj.data.copy_(full.gate_up_proj.data[r * 2:(r + 1) * 2])
        b.down_proj.data.copy_(full.down_proj.data[r * 2:(r + 1) * 2])
    xs, experts, refs, dys = [], [], [], []
    for r in range(world):
        sel = torch.randint(0, 2, (N,), device=dev)                  # experts 0 and 1 only: all on rank 0
        order = torch.argsort(sel, stable=True)
        x_sorted = (torch.randn(N, D, device=dev) * 0.5).to(bf)[order].contiguous().requires_grad_(True)
        y = full(x_sorted, torch.bincount(sel[order], minlength=E).tolist())
        dy = torch.randn_like(y) * 0.1
        y.backward(dy)
        xs.append(x_sorted)
        experts.append(sel[order])
        refs.append((y.detach(), x_sorted.grad.clone()))
        dys.append(dy)
    counts = [torch.bincount(e, minlength=E).tolist() for e in experts]
    ws = [EPWorkspace(N, D, device=dev) for _ in range(world)]
    eps = [FusedExpertParallel(r, world, E, ws) for r in range(world)]
    for r in range(world):
        eps[r].publish(xs[r].detach())
    for r in range(world):
        eps[r].run_experts(counts, banks[r].gate_up_proj.detach(), banks[r].down_proj.detach())
    for r in range(world):
        assert torch.allclose(eps[r].collect().float(), refs[r][0].float(), rtol=3e-2, atol=3e-2)
        eps[r].publish_grad(dys[r])
    grads = [eps[r].run_experts_backward(banks[r].gate_up_proj.detach(), banks[r].down_proj.detach()) for r in range(world)]
    assert float(grads[1][0].abs().max()) == 0.0 and float(grads[1][1].abs().max()) == 0.0
    assert float(grads[0][0].abs().max()) > 0.0
    for r in range(world):
        gx = eps[r].collect_grad().float()
        assert torch.allclose(gx, refs[r][1].float(), rtol=5e-2, atol=2e-2 * refs[r][1].float().abs().max().item())
