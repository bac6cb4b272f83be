"""Memory-bound sm_100a kernels against fp32 PyTorch statements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_rmsnorm_fwd_bwd():
    from aspec_b200.ops.norm import rmsnorm, rmsnorm_reference
    torch.manual_seed(0)
    for rows, H in [(37, 256), (300, 4096), (5, 8192)]:
        x = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_()
        w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
        y = rmsnorm(x, w, 1e-6)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr = x.detach().float().requires_grad_()
        wr = w.detach().float().requires_grad_()
        yr = rmsnorm_reference(xr, wr, 1e-6)
        yr.backward(dy.float())
        assert (y.float() - yr).abs().max() < 3e-2
        assert (x.grad.float() - xr.grad).abs().max() < 3e-2
        rel = (w.grad.float() - wr.grad).abs().max() / wr.grad.abs().max()
        assert rel < 2e-2


def test_qk_norm_rope_fwd_bwd():
    from aspec_b200.ops.rope import qk_norm_rope, qk_norm_rope_reference
    torch.manual_seed(1)
    for N, H, D in [(50, 4, 128), (333, 8, 128), (40, 2, 64)]:
        x = torch.randn(N, H, D, device="cuda").bfloat16().requires_grad_()
        w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_()
        pos = torch.randint(0, 4096, (N,), device="cuda", dtype=torch.int32)
        inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
        y = qk_norm_rope(x, w, pos, inv, 1e-6)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr = x.detach().float().requires_grad_()
        wr = w.detach().float().requires_grad_()
        yr = qk_norm_rope_reference(xr, wr, pos, inv, 1e-6)
        yr.backward(dy.float())
        assert (y.float() - yr).abs().max() < 4e-2
        assert (x.grad.float() - xr.grad).abs().max() < 4e-2
        rel = (w.grad.float() - wr.grad).abs().max() / wr.grad.abs().max()
        assert rel < 2e-2


def test_swiglu_fwd_bwd():
    from aspec_b200.ops.activation import swiglu, swiglu_reference
    torch.manual_seed(2)
    for clamp in (0.0, 1.5):
        gu = (2 * torch.randn(77, 512, device="cuda")).bfloat16().requires_grad_()
        y = swiglu(gu, clamp)
        dy = torch.randn_like(y)
        y.backward(dy)
        gr = gu.detach().float().requires_grad_()
        yr = swiglu_reference(gr, clamp)
        yr.backward(dy.float())
        assert ((y.float() - yr).abs() / (1 + yr.abs())).max() < 2e-2
        assert ((gu.grad.float() - gr.grad).abs() / (1 + gr.grad.abs())).max() < 3e-2


def test_linear_and_fused_linear_grads():
    from aspec_b200.ops.fused_params import allocate_adjacent, fused_linear
    from aspec_b200.ops.linear import linear
    torch.manual_seed(3)
    x = (torch.randn(200, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.1).bfloat16().requires_grad_()
    y = linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(dy.float())
    assert (y.float() - xr @ wr.t()).abs().max() < 5e-2
    assert (x.grad.float() - xr.grad).abs().max() < 1e-1
    assert (w.grad.float() - wr.grad).abs().max() < 3e-1
    a, b = allocate_adjacent([(128, 256), (128, 256)], device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        a.normal_(std=0.1)
        b.normal_(std=0.1)
    a.main_grad = torch.zeros(128, 256, device="cuda")
    x2 = x.detach().clone().requires_grad_()
    y2 = fused_linear(x2, [a, b])
    ref = torch.cat([x2.detach().float() @ a.float().t(), x2.detach().float() @ b.float().t()], 1)
    assert (y2.float() - ref).abs().max() < 5e-2
    dy2 = torch.randn_like(y2)
    y2.backward(dy2)
    assert (a.main_grad - dy2[:, :128].float().t() @ x2.detach().float()).abs().max() < 3e-1
    assert (b.grad.float() - dy2[:, 128:].float().t() @ x2.detach().float()).abs().max() < 3e-1


@pytest.mark.parametrize("with_teacher,markov", [(True, True), (False, False), (True, False)])
def test_head_loss_matches_reference(with_teacher, markov):
    from aspec_b200.ops.vocab_head import head_loss, head_loss_reference
    torch.manual_seed(4)
    R, D, V, r, Tt = 150, 128, 1000, 32, 90
    hidden = (torch.randn(R, D, device="cuda")).bfloat16().requires_grad_()
    lm_w = (torch.randn(V, D, device="cuda") * 0.2).bfloat16()
    labels = torch.randint(0, V, (R,), device="cuda")
    weight = torch.rand(R, device="cuda") * (torch.rand(R, device="cuda") > 0.2)
    kw = {}
    if markov:
        kw["prev_emb"] = (torch.randn(R, r, device="cuda")).bfloat16().requires_grad_()
        kw["markov_w2"] = (torch.randn(V, r, device="cuda") * 0.2).bfloat16().requires_grad_()
    if with_teacher:
        kw["teacher_hidden"] = torch.randn(Tt, D, device="cuda").bfloat16()
        kw["t_index"] = torch.randint(0, Tt, (R,), device="cuda", dtype=torch.int32)
    num, ce, l1, correct = head_loss(hidden, lm_w, labels, weight, a_ce=0.1, a_l1=0.9 if with_teacher else 0.0, **kw)
    (num * 0.5).backward()
    kw_ref = {k: (v.detach().float().requires_grad_() if v.dtype == torch.bfloat16 and k != "teacher_hidden" else v)
              for k, v in kw.items()}
    hr = hidden.detach().float().requires_grad_()
    num_r, ce_r, l1_r, cor_r = head_loss_reference(hr, lm_w, labels, weight, a_ce=0.1,
                                                   a_l1=0.9 if with_teacher else 0.0, **kw_ref)
    (num_r * 0.5).backward()
    assert abs(num.item() - num_r.item()) / abs(num_r.item()) < 2e-2
    assert (ce - ce_r).abs().max() < 0.15
    assert (l1 - l1_r).abs().max() < 5e-2
    assert (correct - cor_r).abs().mean() < 0.03
    g, gr = hidden.grad.float(), hr.grad
    assert (g - gr).abs().max() / gr.abs().max() < 5e-2
    if markov:
        g2, g2r = kw["markov_w2"].grad.float(), kw_ref["markov_w2"].grad
        assert (g2 - g2r).abs().max() / g2r.abs().max() < 5e-2
        g3, g3r = kw["prev_emb"].grad.float(), kw_ref["prev_emb"].grad
        assert (g3 - g3r).abs().max() / g3r.abs().max() < 5e-2


def test_chunked_head_loss_on_the_kernel_path_matches_the_whole_head():
    """Row chunks under activation checkpointing (bounded vocabulary-sized memory) against one call over all rows."""
    from aspec_b200.ops.vocab_head import head_loss
    torch.manual_seed(6)
    R, D, V, r, Tt = 300, 128, 1000, 32, 170
    lm_w = (torch.randn(V, D, device="cuda") * 0.2).bfloat16()
    labels = torch.randint(0, V, (R,), device="cuda")
    weight = torch.rand(R, device="cuda")
    teacher = torch.randn(Tt, D, device="cuda").bfloat16()
    t_index = torch.randint(0, Tt, (R,), device="cuda", dtype=torch.int32)
    h0, p0 = torch.randn(R, D, device="cuda").bfloat16(), torch.randn(R, r, device="cuda").bfloat16()
    w20 = (torch.randn(V, r, device="cuda") * 0.2).bfloat16()
    outs = []
    for chunk in (0, 128):
        h, p, w2 = h0.clone().requires_grad_(), p0.clone().requires_grad_(), w20.clone().requires_grad_()
        num, ce, l1, ok = head_loss(h, lm_w, labels, weight, prev_emb=p, markov_w2=w2, teacher_hidden=teacher, t_index=t_index,
                                    a_ce=0.1, a_l1=0.9, chunk_rows=chunk)
        num.backward()
        outs.append((num.detach().float().reshape(1), ce.float(), l1.float(), ok.float(), h.grad.float(), p.grad.float(), w2.grad.float()))
    for a, b in zip(*outs):
        assert (a - b).abs().max() <= 2e-2 * max(1.0, b.abs().max().item())


def test_flat_adamw_matches_torch():
    from aspec_b200.ops import elementwise_sm100 as E
    torch.manual_seed(5)
    n = 10007
    master = torch.randn(n, device="cuda")
    grad = torch.randn(n, device="cuda") * 3
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    param = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        ctrl = torch.zeros(4, device="cuda")
        E.sumsq(grad, ctrl)
        ctrl[2] = 1.0
        norm = grad.norm()
        assert abs(ctrl[0].sqrt().item() - norm.item()) / norm.item() < 1e-4
        E.adamw(master, grad, m, v, param, ctrl, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1,
                step=step, max_norm=1.0)
        ref.grad = grad * min(1.0, 1.0 / (norm.item() + 1e-6))
        opt.step()
        assert (master - ref.detach()).abs().max() < 1e-5
        assert (param.float() - master).abs().max() < 2e-2
