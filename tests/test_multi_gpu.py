"""Real two-GPU runs of the peer-memory layers (one process per GPU, NCCL for the barriers only): FULL_SHARD
optimizer, vocabulary-parallel head, direct context-parallel attention, Ulysses projections.  Skipped when fewer
than two GPUs are visible.  NVLS is off and the kernels use plain peer loads / stores."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _close(a, b, rtol, atol):
    return bool(torch.allclose(a.float(), b.float(), rtol=rtol, atol=atol))


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    from aspec_b200.parallel.group import exchange_workspaces, make_barrier
    barrier = make_barrier(dev)
    bf = torch.bfloat16
    try:
        # ---- FULL_SHARD optimizer against the replicated one -------------------------------------------------
        from aspec_b200.training.optimizer import BF16Optimizer
        from aspec_b200.training.sharded_optimizer import ShardedBF16Optimizer
        torch.manual_seed(0)
        make = lambda: torch.nn.Sequential(torch.nn.Linear(256, 512, bias=False), torch.nn.Linear(512, 128, bias=False)).to(dev, bf)
        m_s, m_r = make(), make()
        m_r.load_state_dict(m_s.state_dict())
        opt_s = ShardedBF16Optimizer(m_s, lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
        opt_r = BF16Optimizer(m_r, lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
        for step in range(3):
            for ps, pr in zip(m_s.parameters(), m_r.parameters()):
                g = torch.Generator(device=dev).manual_seed(1000 * step + 10 * rank + ps.numel() % 7)
                grad = torch.randn(ps.shape, device=dev, generator=g)
                ps.main_grad.add_(grad)
                pr.main_grad.add_(grad)
            dist.all_reduce(opt_r.flat_grad)
            n_s, n_r = opt_s.step(), opt_r.step()
        res["fsdp_params"] = all(_close(a, b, 0, 1e-2) for a, b in zip(m_s.parameters(), m_r.parameters()))
        res["fsdp_norm"] = _close(n_s, n_r, 1e-4, 1e-6)
        res["fsdp_state_bytes"] = int(opt_s.shard_master.numel() * 12)
        res["repl_state_bytes"] = int(opt_r.flat_master.numel() * 12)
        opt_s.close()

        # ---- vocabulary-parallel head ------------------------------------------------------------------------
        from aspec_b200.ops.vocab_head import head_loss
        from aspec_b200.parallel.vocab_parallel import VocabParallelHead, VocabShardWorkspace, vocab_parallel_head_loss
        torch.manual_seed(1)
        R, Tt, D, V, rk = 384, 128, 256, 8192, 32
        hidden = (torch.randn(R, D, device=dev) * 0.5).to(bf)
        W = (torch.randn(V, D, device=dev) * 0.05).to(bf)
        W2 = torch.nn.Parameter((torch.randn(V, rk, device=dev) * 0.05).to(bf))
        prev = (torch.randn(R, rk, device=dev) * 0.5).to(bf)
        teacher = (torch.randn(Tt, D, device=dev) * 0.5).to(bf)
        t_index = torch.randint(0, Tt, (R,), device=dev, dtype=torch.int32)
        labels = torch.randint(0, V, (R,), device=dev)
        weight = torch.rand(R, device=dev)
        for t in (hidden, W, W2.data, prev, teacher, t_index, labels, weight):
            dist.broadcast(t, 0)
        h1, p1 = hidden.clone().requires_grad_(True), prev.clone().requires_grad_(True)
        w2_ref = W2.detach().clone().requires_grad_(True)
        num1, ce1, l11, _ = head_loss(h1, W, labels, weight, prev_emb=p1, markov_w2=w2_ref, teacher_hidden=teacher,
                                      t_index=t_index, a_ce=0.1, a_l1=0.9)
        num1.backward()
        ws = exchange_workspaces(VocabShardWorkspace(R, Tt, D, rk, world, device=dev), VocabShardWorkspace.open)
        head = VocabParallelHead(rank, world, V, ws, barrier)
        h2, p2 = hidden.clone().requires_grad_(True), prev.clone().requires_grad_(True)
        num2, ce2, l12, _ = vocab_parallel_head_loss(head, h2, head.shard_rows(W).contiguous(), labels, weight, prev_emb=p2,
                                                     markov_w2=W2, teacher_hidden=teacher, t_index=t_index, a_ce=0.1, a_l1=0.9)
        num2.backward()
        gmax = h1.grad.float().abs().max().item()
        res["vp_loss"] = _close(num2, num1, 2e-3, 1e-3) and _close(ce2, ce1, 2e-3, 2e-3) and _close(l12, l11, 2e-3, 2e-3)
        res["vp_dhidden"] = _close(h2.grad, h1.grad, 5e-2, 4e-3 * gmax)
        res["vp_dprev"] = _close(p2.grad, p1.grad, 5e-2, 4e-3 * p1.grad.float().abs().max().item())
        sl = slice(head.offset, head.offset + head.shard)
        # shard-only gradients carry the group size (the data-parallel sum then treats them like replicated ones)
        res["vp_dw2"] = _close(W2.grad[sl].float() / world, w2_ref.grad[sl], 5e-2, 4e-3 * w2_ref.grad.float().abs().max().item())

        # ---- direct context-parallel attention ----------------------------------------------------------------
        from aspec_b200.ops import attention_sm100 as K
        from aspec_b200.ops.attention import build_block_intervals
        from aspec_b200.parallel.context import context_shard_bounds
        from aspec_b200.parallel.context_parallel import CPWorkspace, DirectCPAttention, direct_cp_attention, local_intervals
        torch.manual_seed(2)
        T, A, bs, H, Hk, d = 1024, 64, 4, 8, 2, 128
        Q = A * bs
        anchors = torch.sort(torch.randint(8, T - bs, (A,), device=dev)).values
        q = (torch.randn(Q, H, d, device=dev) * 0.5).to(bf)
        k = (torch.randn(T + Q, Hk, d, device=dev) * 0.5).to(bf)
        v = (torch.randn(T + Q, Hk, d, device=dev) * 0.5).to(bf)
        dout = (torch.randn(Q, H, d, device=dev) * 0.5).to(bf)
        for t in (anchors, q, k, v, dout):
            dist.broadcast(t, 0)
        iv = build_block_intervals(anchors, torch.ones(A, dtype=torch.bool, device=dev), ctx_len=T, block_size=bs)
        scale = d ** -0.5
        o_ref, l_ref = K.forward(q, k, v, iv, scale)
        dq_ref, dk_ref, dv_ref = K.backward(q, k, v, iv, o_ref, l_ref, dout, scale)
        ql = Q // world
        s, e = context_shard_bounds(T, rank, world, 1)
        cws = exchange_workspaces(CPWorkspace(world, ql, H, d, device=dev), CPWorkspace.open)
        cp = DirectCPAttention(rank, world, cws, barrier)
        k_loc = torch.cat([k[s:e], k[T + rank * ql: T + (rank + 1) * ql]]).clone().requires_grad_(True)
        v_loc = torch.cat([v[s:e], v[T + rank * ql: T + (rank + 1) * ql]]).clone().requires_grad_(True)
        q_loc = q[rank * ql:(rank + 1) * ql].clone().requires_grad_(True)
        tables = [local_intervals(iv[o * ql:(o + 1) * ql], s, e, T, own=(o == rank), query_start=rank * ql) for o in range(world)]
        out, lse = direct_cp_attention(cp, q_loc, k_loc, v_loc, tables, [ql] * world, scale)
        out.backward(dout[rank * ql:(rank + 1) * ql])
        tol = dict(rtol=5e-2, atol=3e-2)
        res["cp_out"] = _close(out, o_ref[rank * ql:(rank + 1) * ql], 2e-2, 2e-2)
        res["cp_dq"] = _close(q_loc.grad, dq_ref[rank * ql:(rank + 1) * ql], **tol)
        res["cp_dk"] = _close(k_loc.grad[: e - s], dk_ref[s:e], **tol) and _close(v_loc.grad[: e - s], dv_ref[s:e], **tol)

        # ---- Ulysses projections ----------------------------------------------------------------------------------
        from aspec_b200.parallel.ulysses import UlyssesExchange, UlyssesWorkspace, group_qkv_rows
        torch.manual_seed(3)
        T_loc, D2, hq, hk, d2 = 256, 512, 8, 2, 64
        wq, wk, wv = [(torch.randn(n * d2, D2, device=dev) * 0.05).to(bf) for n in (hq, hk, hk)]
        wo = (torch.randn(D2, hq * d2, device=dev) * 0.05).to(bf)
        xs = [(torch.randn(T_loc, D2, device=dev) * 0.5).to(bf) for _ in range(world)]
        for t in [wq, wk, wv, wo] + xs:
            dist.broadcast(t, 0)
        wg = group_qkv_rows(wq, wk, wv, world, d2)
        qc, oc = (hq + 2 * hk) * d2 // world, hq * d2 // world
        uws = exchange_workspaces(UlyssesWorkspace(world, T_loc, qc, oc, device=dev), UlyssesWorkspace.open)
        ex = UlyssesExchange(rank, world, uws, barrier)
        ex.project_scatter(xs[rank], wg)
        barrier()
        want = torch.cat(xs).float() @ wg[rank * qc:(rank + 1) * qc].float().T
        res["ulysses_scatter"] = _close(ex.received_qkv(), want, 2e-2, 3e-2)
        attn_all = [(torch.sin(torch.arange(world * T_loc * oc, device=dev).float() * (g + 1) * 0.37).view(world * T_loc, oc) * 0.5).to(bf)
                    for g in range(world)]
        ex.publish_attention(attn_all[rank])
        barrier()
        got = ex.output_projection(wo)
        want = torch.cat(attn_all, 1).float()[rank * T_loc:(rank + 1) * T_loc] @ wo.float().T
        res["ulysses_oproj"] = _close(got, want, 2e-2, 5e-2)
        barrier()

        # ---- Ulysses self-attention block (autograd) against the same module on one GPU over the whole sequence ----
        from aspec_b200.models.target.dense import DenseTarget
        from aspec_b200.parallel.ulysses_attention import UlyssesSelfAttention
        torch.manual_seed(5)
        T5, D5, hq5, hk5, d5 = 256, 512, 8, 2, 128
        ref_attn = UlyssesSelfAttention(D5, hq5, hk5, d5).to(dev, bf)
        for prm in ref_attn.parameters():
            dist.broadcast(prm.data, 0)
        x_all = (torch.randn(world * T5, D5, device=dev) * 0.5).to(bf)
        dy_all = (torch.randn(world * T5, D5, device=dev) * 0.1).to(bf)
        dist.broadcast(x_all, 0)
        dist.broadcast(dy_all, 0)
        iv5 = DenseTarget.causal_intervals([300, world * T5 - 300], dev)
        xr = x_all.clone().requires_grad_(True)
        ref_attn(xr, iv5).backward(dy_all)
        qc5, oc5 = (hq5 + 2 * hk5) * d5 // world, hq5 * d5 // world
        uws5 = exchange_workspaces(UlyssesWorkspace(world, T5, qc5, oc5, device=dev), UlyssesWorkspace.open)
        par = UlyssesSelfAttention(D5, hq5, hk5, d5, exchange=UlyssesExchange(rank, world, uws5, barrier)).to(dev, bf)
        par.load_state_dict(ref_attn.state_dict())
        rows = slice(rank * T5, (rank + 1) * T5)
        xp = x_all[rows].clone().requires_grad_(True)
        yp = par(xp, iv5)
        yp.backward(dy_all[rows])
        with torch.no_grad():
            yr = ref_attn(x_all, iv5)[rows]
        res["ulysses_block_forward"] = _close(yp, yr, 3e-2, 2e-2)
        res["ulysses_block_dx"] = _close(xp.grad, xr.grad[rows], 5e-2, 2e-2)
        ok = True
        for (n, pp), (_, pr) in zip(par.named_parameters(), ref_attn.named_parameters()):
            g = pp.grad.float().clone()
            dist.all_reduce(g)                      # every rank contributed its own rows
            ok = ok and _close(g, pr.grad, 5e-2, 3e-2 * max(pr.grad.abs().max().item(), 1e-3))
        res["ulysses_block_dw"] = ok
        barrier()

        # ---- EAGLE3 training wrapper, sequence parallel over the Ulysses block, against one GPU over the whole row ----
        from aspec_b200.config.draft_config import AutoDraftModelConfig
        from aspec_b200.training.factory import build_training_model
        raw6 = dict(architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=256, intermediate_size=512,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=128, vocab_size=512, draft_vocab_size=512,
                    target_hidden_size=256, num_aux_hidden_states=3, rope_theta=10000.0, max_position_embeddings=2048)
        args6 = dict(ttt_length=3, seed=0)
        torch.manual_seed(6)
        ref6 = build_training_model(AutoDraftModelConfig.from_dict(raw6), args6, dev, bf)
        par6 = build_training_model(AutoDraftModelConfig.from_dict(raw6), args6, dev, bf)
        for prm in ref6.parameters():
            dist.broadcast(prm.data, 0)
        par6.load_state_dict(ref6.state_dict())
        T6 = 301                                                        # odd on purpose: the row is padded to the group size
        g6 = torch.Generator(device="cpu").manual_seed(66)
        batch6 = dict(input_ids=torch.randint(0, 500, (1, T6), generator=g6).to(dev),
                      hidden_states_list=(torch.randn(1, T6, 768, generator=g6) * 0.5).to(dev, bf),
                      loss_mask=torch.cat([torch.zeros(1, 40), torch.ones(1, T6 - 40)], 1).to(dev),
                      lm_head_weight=(torch.randn(512, 256, generator=g6) * 0.05).to(dev, bf),
                      last_hidden_states=(torch.randn(1, T6, 256, generator=g6) * 0.5).to(dev, bf),
                      ctx_doc_ids=torch.cat([torch.zeros(1, 120), torch.ones(1, T6 - 120)], 1).long().to(dev))
        ref6.train()
        par6.train()
        out_r = ref6(**batch6)
        out_r[6][0].backward()
        d6 = par6.draft_model
        sa6 = d6.midlayer.self_attn
        rows6 = -(-T6 // world)
        qc6 = (sa6.num_heads + 2 * sa6.num_kv_heads) * sa6.head_dim // world
        oc6 = sa6.num_heads * sa6.head_dim // world
        uws6 = exchange_workspaces(UlyssesWorkspace(world, rows6 + 8, qc6, oc6, device=dev), UlyssesWorkspace.open)
        d6.ulysses = UlyssesExchange(rank, world, uws6, barrier)
        par6.sequence_parallel = (rank, world, None)
        out_p = par6(**batch6)
        out_p[6][0].backward()
        num6 = out_p[6][0].detach().float().clone()
        den6 = out_p[6][1].detach().float().clone()
        dist.all_reduce(num6)
        dist.all_reduce(den6)
        res["sp_eagle_loss"] = _close(num6 / den6, out_r[6][0].detach().float() / out_r[6][1].float(), 2e-2, 2e-2)
        res["sp_eagle_counts"] = bool(torch.equal(out_p[4], out_r[4]))
        ok6, worst6 = True, ""
        for (n, pp), (_, pr) in zip(par6.draft_model.named_parameters(), ref6.draft_model.named_parameters()):
            if pr.grad is None:
                continue
            g = (pp.grad if pp.grad is not None else torch.zeros_like(pr)).float().clone()
            dist.all_reduce(g)
            if not _close(g, pr.grad, 8e-2, 4e-2 * max(pr.grad.float().abs().max().item(), 1e-3)):
                ok6, worst6 = False, n
        res["sp_eagle_grads"] = ok6
        if not ok6:
            res["sp_eagle_worst"] = worst6
        barrier()

        # ---- expert parallelism: fused peer-memory dispatch / combine against the NCCL all-to-all path ------------
        from aspec_b200.models.draft.moe import ExpertBank
        from aspec_b200.parallel.expert_parallel import (EPWorkspace, FusedExpertParallel, dispatch_combine,
                                                         fused_dispatch_combine)
        torch.manual_seed(4)
        E, D3, I3, N3, k3 = 8, 256, 128, 512, 2
        full_gu = (torch.randn(E, 2 * I3, D3, device=dev) * 0.05).to(bf)
        full_dn = (torch.randn(E, D3, I3, device=dev) * 0.05).to(bf)
        dist.broadcast(full_gu, 0)
        dist.broadcast(full_dn, 0)
        loc = E // world
        outs = {}
        torch.manual_seed(100 + rank)
        x3 = (torch.randn(N3, D3, device=dev) * 0.5).to(bf)
        sel = torch.randint(0, E, (N3 * k3,), device=dev)
        order = torch.argsort(sel, stable=True)
        dy3 = (torch.randn(N3 * k3, D3, device=dev) * 0.1).to(bf)
        ews = exchange_workspaces(EPWorkspace(N3 * k3, D3, device=dev), EPWorkspace.open)
        ep = FusedExpertParallel(rank, world, E, ews, barrier)
        for name in ("nccl", "fused"):
            bank = ExpertBank(E, D3, I3, ep_rank=rank, ep_size=world).to(dev, bf)
            bank.gate_up_proj.data.copy_(full_gu[rank * loc:(rank + 1) * loc])
            bank.down_proj.data.copy_(full_dn[rank * loc:(rank + 1) * loc])
            xs3 = x3.repeat_interleave(k3, 0)[order].contiguous().requires_grad_(True)
            y3 = (dispatch_combine(bank, xs3, sel[order]) if name == "nccl" else fused_dispatch_combine(ep, bank, xs3, sel[order]))
            y3.backward(dy3)
            outs[name] = (y3.detach().float(), xs3.grad.float(), bank.gate_up_proj.grad.float(), bank.down_proj.grad.float())
        tolf = lambda a, b: _close(a, b, 5e-2, 3e-2 * max(b.abs().max().item(), 1e-3))
        res["ep_forward"] = tolf(outs["fused"][0], outs["nccl"][0])
        res["ep_dx"] = tolf(outs["fused"][1], outs["nccl"][1])
        res["ep_dw"] = tolf(outs["fused"][2], outs["nccl"][2]) and tolf(outs["fused"][3], outs["nccl"][3])
        barrier()
        torch.cuda.synchronize()
    except Exception as exc:                                     # noqa: BLE001 - reported to the parent
        import traceback
        res["error"] = f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-1500:]}"
    torch.save(res, f"{out_path}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(900)
def test_peer_memory_layers_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, 29700 + os.getpid() % 500, out), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(f"{out}.{rank}")
        assert "error" not in res, res.get("error")
        bad = [k for k, v in res.items() if isinstance(v, bool) and not v]
        assert not bad, (rank, bad, res)
        assert res["fsdp_state_bytes"] * 2 <= res["repl_state_bytes"] + 12 * 16


def _eagle_recipe(tmp_path, name, gpus, extra=""):
    import json
    draft = tmp_path / "eagle3_small.json"
    draft.write_text(json.dumps(dict(
        architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=256, intermediate_size=512,
        num_attention_heads=4, num_key_value_heads=2, head_dim=128, vocab_size=512, draft_vocab_size=512, target_hidden_size=256,
        target_num_hidden_layers=8, num_aux_hidden_states=3, rope_theta=10000.0, max_position_embeddings=2048)))
    recipe = tmp_path / f"{name}.yaml"
    recipe.write_text(f"""
model:
  draft_model_config: {draft}
dataset:
  train_data_path: synthetic
  synthetic_num_documents: 32
  synthetic_min_length: 200
  synthetic_max_length: 420
  shuffle_dataset: false
inference:
  inference_engine_type: synthetic
training:
  training_num_gpus_per_node: {gpus}
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 512
  num_train_steps: 3
  learning_rate: 1e-3
  ttt_length: 3
  save_interval: 0
  save_final_checkpoint: false
  seed: 11
{extra}
transport:
  destination_ring_slots: 4
output_dir: {tmp_path / name}
""")
    from aspec_b200.config.train_config import load_config
    from aspec_b200.planning import compile_execution_plan
    return compile_execution_plan(load_config(str(recipe), []))


@pytest.mark.timeout(900)
def test_sequence_parallel_eagle3_pipeline_matches_one_gpu(tmp_path):
    """The whole pipeline (driver, synthetic engine, trainer processes): EAGLE3 with ``sp_ulysses_size: 2`` on two GPUs
    trains on the same rows as one GPU and reports the same losses."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from aspec_b200.train_entry import train_async_no_generation
    losses = {}
    for name, gpus, extra in (("one", 1, ""), ("sp2", 2, "  sp_ulysses_size: 2")):
        plan = _eagle_recipe(tmp_path, name, gpus, extra)
        flat = plan.to_runtime_args()
        flat.update(synthetic_vocab_size=500)
        os.makedirs(flat["output_dir"], exist_ok=True)
        logs = []
        summary = train_async_no_generation(flat, plan.draft_config, log=logs.append)
        assert summary["completed_steps"] == 3 and summary["ledger"]["validated"]
        losses[name] = [l["train/avg_loss"] for l in logs]
    assert losses["one"][0] == pytest.approx(losses["sp2"][0], rel=3e-2)
    assert losses["one"][-1] == pytest.approx(losses["sp2"][-1], rel=6e-2)


def _full_shard_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    try:
        from aspec_b200.training.full_shard import FullShardOptimizer
        from aspec_b200.training.optimizer import BF16Optimizer

        class Layer(torch.nn.Module):
            def __init__(self, d):
                super().__init__()
                self.a, self.b = torch.nn.Linear(d, d, bias=False), torch.nn.Linear(d, d, bias=False)

            def forward(self, x, ctx):
                return x + torch.tanh(self.a(x) + self.b(ctx)) * 0.5

        class Net(torch.nn.Module):
            def __init__(self, d=256, n=4):
                super().__init__()
                self.inp = torch.nn.Linear(64, d, bias=False)
                self.layers = torch.nn.ModuleList([Layer(d) for _ in range(n)])
                self.out = torch.nn.Linear(d, 32, bias=False)

            def forward(self, x, feats):
                ctx = self.inp(feats)
                for layer in self.layers:
                    x = layer(x, ctx)
                return self.out(x).float().pow(2).mean()

        torch.manual_seed(0)
        a = Net().to(dev, torch.bfloat16)
        b = Net().to(dev, torch.bfloat16)
        b.load_state_dict(a.state_dict())
        opt_a = FullShardOptimizer(a, list(a.layers), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100,
                                   wait_limit_ms=4000.0)
        opt_b = BF16Optimizer(b, lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, total_steps=100)
        norms = []
        for step in range(3):
            for mb in range(2):
                g = torch.Generator(device=dev).manual_seed(1000 * step + 10 * rank + mb)
                x = torch.randn(48, 256, device=dev, generator=g).bfloat16()       # no gradient into layer 0 through x
                feats = torch.randn(48, 64, device=dev, generator=g).bfloat16()
                a(x, feats).backward()
                opt_a.finish_micro_batch()
                b(x, feats).backward()
            opt_b.fold_autograd_grads()
            dist.all_reduce(opt_b.flat_grad)
            opt_a.set_grad_scale(0.25)
            opt_b.set_grad_scale(0.25)
            norms.append((opt_a.step(), opt_b.step()))
        res["norms"] = all(_close(x, y, 2e-2, 1e-4) for x, y in norms)
        with opt_a.full_parameters():
            res["params"] = all(_close(p, q, 0, 2e-2) for p, q in zip(a.parameters(), b.parameters()))
        sd = opt_a.state_dict()
        ref_master = opt_b.state_dict()["master"]
        res["masters"] = all(_close(sd["master"][n], ref_master[n], 0, 2e-2) for n in ref_master)
        rep = opt_a.memory_report()
        res["at_rest_half"] = rep["at_rest_bytes"] * 2 <= rep["replicated_bytes"] * 1.05 + 4096
        res["status_clean"] = int(opt_a.status.item()) == 0
        dist.barrier()
        opt_a.close()
    except Exception as exc:  # noqa: BLE001
        import traceback
        res["error"] = f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-1500:]}"
    torch.save(res, f"{out_path}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_full_shard_trains_like_the_replicated_optimizer_on_two_gpus(tmp_path):
    """Parameters, gradients and optimizer state sharded per layer over two real GPUs: gathers by peer loads, the
    reduce-scatter by peer loads, ordering by flags in peer memory (no library collective but the two-scalar norm)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "res")
    mp.spawn(_full_shard_worker, args=(2, 29300 + os.getpid() % 500, out), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(f"{out}.{rank}")
        assert "error" not in res, res.get("error")
        bad = [k for k, v in res.items() if v is not True]
        assert not bad, (rank, bad, res)


def _ring_problem(world, S, E, HQ, HKV, D):
    g = torch.Generator().manual_seed(world)
    T = world * S
    q = torch.randn(world, S, HQ, D, generator=g) * 0.5
    k = torch.randn(T, HKV, D, generator=g) * 0.5
    v = torch.randn(T, HKV, D, generator=g) * 0.5
    ke = torch.randn(world, E, HKV, D, generator=g) * 0.5
    ve = torch.randn(world, E, HKV, D, generator=g) * 0.5
    iv = []
    for r in range(world):
        pos = r * S + torch.arange(S)
        lo = torch.randint(0, T // 2, (S,), generator=g).clamp(max=pos)
        n_extra = torch.randint(0, E + 1, (S,), generator=g)
        iv.append(torch.stack([lo, pos + 1, torch.full((S,), S), S + n_extra], -1).to(torch.int32))
    dout = torch.randn(world, S, HQ, D, generator=g) * 0.5
    return q, k, v, ke, ve, iv, dout


def _ring_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    try:
        from aspec_b200.ops.attention import interval_attention_reference
        from aspec_b200.ops.gemm import check_status
        from aspec_b200.parallel.ring_attention import ring_attention
        S, E, HQ, HKV, D = 384, 16, 8, 2, 128
        bf = torch.bfloat16
        q, k, v, ke, ve, iv, dout = _ring_problem(world, S, E, HQ, HKV, D)
        ql = q[rank].to(dev, bf).requires_grad_()
        kl = torch.cat([k[rank * S:(rank + 1) * S], ke[rank]]).to(dev, bf).requires_grad_()
        vl = torch.cat([v[rank * S:(rank + 1) * S], ve[rank]]).to(dev, bf).requires_grad_()
        o, lse = ring_attention(ql, kl, vl, iv[rank].to(dev), S, D ** -0.5)
        o.backward(dout[rank].to(dev, bf))
        check_status(dev)
        # fp32 statement of the unsharded problem on this rank's queries (keys: the whole sequence, then own extra rows)
        T = world * S
        qr = q[rank].to(bf).float().requires_grad_()
        kr = torch.cat([k, ke[rank]]).to(bf).float().requires_grad_()
        vr = torch.cat([v, ve[rank]]).to(bf).float().requires_grad_()
        table = iv[rank].clone()
        table[:, 2:] += T - S
        ref, ref_lse = interval_attention_reference(qr, kr, vr, table, D ** -0.5)
        ref.backward(dout[rank].to(bf).float())
        fin = torch.isfinite(ref_lse)
        res["out"] = _close(o.cpu(), ref.detach(), 3e-2, 3e-2)
        res["lse"] = _close(lse.cpu()[fin], ref_lse.detach()[fin], 2e-2, 2e-2)
        res["dq"] = _close(ql.grad.cpu(), qr.grad, 5e-2, 3e-2 * qr.grad.abs().max().item())
        # this shard's own keys collect gradient from every rank's queries: compare the sum over ranks through rank 0
        mine = torch.zeros(T, HKV, D)
        mine[rank * S:(rank + 1) * S] = kl.grad[:S].float().cpu()
        total = mine.to(dev)
        dist.all_reduce(total)
        want = kr.grad[:T].to(dev)
        dist.all_reduce(want)                        # every rank's reference holds only its own queries' share
        res["dk"] = _close(total.cpu(), want.cpu(), 5e-2, 3e-2 * want.abs().max().item())
        res["dk_extra"] = _close(kl.grad[S:].cpu(), kr.grad[T:], 5e-2, 3e-2 * max(kr.grad[T:].abs().max().item(), 1e-3))
    except Exception as exc:  # noqa: BLE001
        import traceback
        res["error"] = f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-1500:]}"
    torch.save(res, f"{out_path}.{rank}")
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_ring_attention_on_two_gpus_matches_the_unsharded_statement(tmp_path):
    """Key / value blocks travel the ring over NCCL point-to-point while each stop runs the interval attention kernels;
    output, log-sum-exp and all gradients against fp32 attention over the whole sequence."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "ring")
    mp.spawn(_ring_worker, args=(2, 29100 + os.getpid() % 500, out), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(f"{out}.{rank}")
        assert "error" not in res, res.get("error")
        bad = [k for k, v in res.items() if v is not True]
        assert not bad, (rank, bad, res)
