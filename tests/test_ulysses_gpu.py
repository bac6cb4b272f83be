"""Ulysses exchange fused into the QKV / output projections: two ranks emulated on one GPU against plain matmuls."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_projection_scatter_and_multi_source_output_projection(world):
    from aspec_b200.parallel.ulysses import UlyssesExchange, UlyssesWorkspace, group_qkv_rows
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    T_loc, D, hq, hk, d = 192, 256, 8, 4, 64        # four ranks reduce over four sources in one grouped launch
    bf = torch.bfloat16
    wq, wk, wv = [(torch.randn(n * d, D, device=dev) * 0.05).to(bf) for n in (hq, hk, hk)]
    wo = (torch.randn(D, hq * d, device=dev) * 0.05).to(bf)
    wg = group_qkv_rows(wq, wk, wv, world, d)
    qkv_cols, out_cols = (hq + 2 * hk) * d // world, hq * d // world
    xs = [(torch.randn(T_loc, D, device=dev) * 0.5).to(bf) for _ in range(world)]
    ws = [UlyssesWorkspace(world, T_loc, qkv_cols, out_cols, device=dev) for _ in range(world)]
    ex = [UlyssesExchange(r, world, ws) for r in range(world)]
    for r in range(world):
        ex[r].project_scatter(xs[r], wg)
    x_all = torch.cat(xs).float()
    for g in range(world):
        want = x_all @ wg[g * qkv_cols:(g + 1) * qkv_cols].float().T
        assert torch.allclose(ex[g].received_qkv().float(), want, rtol=2e-2, atol=2e-2)
    # stand-in for attention: any function of (all rows, my heads)
    attn = [(torch.randn(world * T_loc, out_cols, device=dev) * 0.5).to(bf) for _ in range(world)]
    for g in range(world):
        ex[g].publish_attention(attn[g])
    full = torch.cat(attn, 1).float()                       # [T_tot, Hq*d], columns grouped by rank
    for r in range(world):
        out = ex[r].output_projection(wo)
        want = full[r * T_loc:(r + 1) * T_loc] @ wo.float().T
        assert torch.allclose(out.float(), want, rtol=2e-2, atol=3e-2)
    # backward primitives
    douts = [(torch.randn(T_loc, D, device=dev) * 0.5).to(bf) for _ in range(world)]
    dwo = [ex[r].output_projection_backward(douts[r], wo) for r in range(world)]
    d_all = torch.cat(douts).float()
    for g in range(world):
        want = d_all @ wo.float()[:, g * out_cols:(g + 1) * out_cols]
        assert torch.allclose(ex[g].received_dattn().float(), want, rtol=2e-2, atol=3e-2)
    want_dwo = sum(douts[r].float().T @ full[r * T_loc:(r + 1) * T_loc] for r in range(world))
    assert torch.allclose(sum(dwo), want_dwo, rtol=2e-2, atol=5e-2)
    dqkv = [(torch.randn(world * T_loc, qkv_cols, device=dev) * 0.5).to(bf) for _ in range(world)]
    for g in range(world):
        ex[g].publish_dqkv(dqkv[g])
    dfull = torch.cat(dqkv, 1).float()
    for r in range(world):
        dx, dw = ex[r].projection_backward(xs[r], wg)
        rows = dfull[r * T_loc:(r + 1) * T_loc]
        assert torch.allclose(dx.float(), rows @ wg.float(), rtol=2e-2, atol=3e-2)
        assert torch.allclose(dw, rows.T @ xs[r].float(), rtol=2e-2, atol=5e-2)
