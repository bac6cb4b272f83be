"""One whole DSpark update on the kernel path against the same update of the fp32 CPU model: loss terms, gradient norm
and the updated weights (two micro-batches, so accumulation and the pooled denominators are covered too)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _batches(cfg_vocab, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for T, sup0 in ((300, 100), (220, 40)):
        out.append({"input_ids": torch.randint(0, cfg_vocab - 48, (1, T), generator=g),
                    "loss_mask": torch.cat([torch.zeros(1, sup0), torch.ones(1, T - sup0)], 1),
                    "hidden_states": (torch.randn(1, T, 768, generator=g)).bfloat16(),
                    "last_hidden_states": (torch.randn(1, T, 256, generator=g)).bfloat16()})
    return out


def test_one_update_matches_the_cpu_fp32_model():
    from aspec_b200.config.draft_config import DSparkConfig
    from aspec_b200.models.draft.dspark import DSparkDraftModel
    from aspec_b200.models.dspark import DSparkModel
    from aspec_b200.ops.anchors import sample_anchor_positions
    from aspec_b200.ops.gemm import check_status
    from aspec_b200.training.draft_trainer import DraftTrainer
    torch.manual_seed(0)
    cfg = DSparkConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=128, vocab_size=2048, num_target_layers=3,
                       target_hidden_size=256, target_num_hidden_layers=8, markov_rank=32, mask_token_id=2047)
    seed_model = DSparkDraftModel(cfg).to(torch.bfloat16)                 # weights both sides share, already bf16-exact
    head = (torch.randn(2048, 256) * 0.05).bfloat16()
    batches = _batches(2048, 1)
    rng = torch.Generator().manual_seed(5)
    for b in batches:
        anchors, keep = sample_anchor_positions(b["input_ids"].shape[1], b["loss_mask"], 32, 7, generator=rng)
        b["injected_anchors"], b["injected_keep_mask"] = anchors, keep

    def run(device, dtype):
        draft = copy.deepcopy(seed_model).to(device, dtype)
        model = DSparkModel(draft, block_size=7, num_anchors=32)
        trainer = DraftTrainer(model, head.to(device, dtype), lr=1e-3, total_steps=10, warmup_ratio=0.0, accumulation=2,
                               device=torch.device(device))
        mine = [{k: (v.to(dtype) if v.is_floating_point() and k not in ("loss_mask",) else v) for k, v in b.items()} for b in batches]
        trainer.train_update(mine)
        metrics = trainer.metrics()
        weights = {k: v.detach().float().cpu() for k, v in draft.state_dict().items() if v.is_floating_point()}
        return metrics, weights

    want_m, want_w = run("cpu", torch.float32)
    got_m, got_w = run("cuda", torch.bfloat16)
    check_status("cuda")
    for key in ("train/avg_loss", "train/l1_loss", "train/ce_loss", "train/grad_norm"):
        if key in want_m:
            assert got_m[key] == pytest.approx(want_m[key], rel=0.03, abs=2e-3), (key, got_m[key], want_m[key])
    assert got_m["train/avg_acc"] == pytest.approx(want_m["train/avg_acc"], abs=0.02)
    # the update itself: lr 1e-3 AdamW moves every weight by about lr; the bf16 weights must have moved the same way
    moved = agree = 0
    for name, w0 in seed_model.state_dict().items():
        if not w0.is_floating_point():
            continue
        dw_want, dw_got = want_w[name] - w0.float(), got_w[name] - w0.float()
        big = dw_want.abs() > 5e-4
        moved += int(big.sum())
        agree += int((torch.sign(dw_want[big]) == torch.sign(dw_got[big])).sum())
        assert (got_w[name] - want_w[name]).abs().max() < 2.5e-3 + 0.01 * w0.float().abs().max(), name
    assert moved > 1000 and agree / moved > 0.97, (moved, agree)
