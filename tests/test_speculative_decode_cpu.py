"""Speculative decoding loop on CPU: whatever the Draft proposes, the text is the Target's greedy continuation, one
Target pass per round, and the acceptance statistics add up (reference: tests/test_sgl_engine_decode.py for the
serving-engine loop this replaces)."""
import json

import pytest
import torch

from aspec_b200.config.draft_config import AutoDraftModelConfig
from aspec_b200.draft_artifact import BlockDraftConsumer
from aspec_b200.inference.speculative_decode import greedy_generate, speculative_generate
from aspec_b200.models.draft.auto import AutoEagle3DraftModel
from aspec_b200.models.target.dense import DenseTarget, TargetConfig

LAYERS = {"dspark": [0, 1, 3], "dflash": [1, 2]}


def _target():
    torch.manual_seed(0)
    cfg = TargetConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, vocab_size=512)
    return DenseTarget(cfg).init_random(0, std=0.3).eval()


def _consumer(kind):
    import os
    import aspec_b200
    root = os.path.join(os.path.dirname(aspec_b200.__file__), "config", "drafts")
    raw = json.load(open(os.path.join(root, f"{kind}_tiny.json")))
    torch.manual_seed(1)
    draft = AutoEagle3DraftModel.from_config(AutoDraftModelConfig.from_dict(raw))
    return BlockDraftConsumer(draft, block_size=4)


@pytest.mark.parametrize("kind", ["dspark", "dflash"])
def test_text_is_the_targets_greedy_continuation(kind):
    target, consumer = _target(), _consumer(kind)
    prompt = torch.randint(0, 500, (11,), generator=torch.Generator().manual_seed(3))
    want = greedy_generate(target, prompt, 14)
    got = speculative_generate(target, consumer, prompt, LAYERS[kind], max_new_tokens=14)
    assert got["tokens"] == want
    rounds = got["accepted_per_round"]
    assert got["target_passes"] == len(rounds) + 1
    assert 1 + sum(n + 1 for n in rounds) >= len(want) >= 1 + len(rounds)         # every round yields at least its bonus token
    assert all(0 <= n <= consumer.block_size - 1 for n in rounds)


def test_a_draft_that_knows_the_answer_is_accepted_whole_and_eos_stops():
    target, consumer = _target(), _consumer("dspark")
    prompt = torch.randint(0, 500, (9,), generator=torch.Generator().manual_seed(4))
    want = greedy_generate(target, prompt, 13)

    class Oracle:
        block_size = 4

        def propose(self, ids, feats, *, lm_head_weight):
            assert feats.shape[1] == ids.shape[1] and float(feats[0, -1].abs().sum()) == 0.0     # the anchor has no features
            done = ids.shape[1] - prompt.numel()
            return {"token_ids": torch.tensor([want[done:done + 3] + [0] * max(0, 3 - len(want[done:done + 3]))])}
    got = speculative_generate(target, Oracle(), prompt, [0, 1, 3], max_new_tokens=13)
    assert got["tokens"] == want and got["accepted_per_round"] == [3, 3, 3] and got["target_passes"] == 4
    assert got["tau"] == pytest.approx(4.0)
    stop = want[5]
    cut = speculative_generate(target, consumer, prompt, [0, 1, 3], max_new_tokens=13, eos_token_id=stop)
    assert cut["tokens"] == want[: want.index(stop) + 1]


# -- cached passes and batched generation -------------------------------------------------------------------------------
def test_cached_passes_equal_prefill_and_rejected_rows_are_overwritten():
    target = _target()
    ids = [torch.randint(0, 500, (n,), generator=torch.Generator().manual_seed(n)) for n in (9, 5)]
    full = [target.prefill(t, [len(t)], [0, 2], want_logits=True) for t in ids]
    cache = target.new_decode_cache(2, 16)
    a = target.extend(cache, [ids[0][:6], ids[1][:2]], [0, 2])
    cache.accept(0, 6)
    cache.accept(1, 2)
    target.extend(cache, [torch.tensor([7, 8, 9]), torch.empty(0, dtype=torch.long)])      # a rejected trial of sequence 0
    b = target.extend(cache, [ids[0][6:], ids[1][2:]], [0, 2])
    torch.testing.assert_close(torch.cat([a["logits"][:6], b["logits"][:3]]), full[0]["logits"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(torch.cat([a["logits"][6:], b["logits"][3:]]), full[1]["logits"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(torch.cat([a["hidden_states"][:6], b["hidden_states"][:3]]), full[0]["hidden_states"], rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError, match="exceed the cache"):
        target.extend(cache, [torch.zeros(11, dtype=torch.long), torch.empty(0, dtype=torch.long)])


@pytest.mark.parametrize("kind", [None, "dspark", "dflash"])
def test_batched_generation_is_the_targets_text_with_or_without_a_draft(kind):
    from aspec_b200.inference.speculative_decode import batched_generate
    target = _target()
    consumer = _consumer(kind) if kind else None
    prompts = [torch.randint(0, 500, (n,), generator=torch.Generator().manual_seed(n)) for n in (11, 4, 7)]
    budgets = [9, 12, 0]
    got = batched_generate(target, prompts, max_new_tokens=budgets, temperature=0.0, consumer=consumer,
                           layer_ids=LAYERS.get(kind, ()))
    for p, g, n in zip(prompts, got, budgets):
        assert g["tokens"] == (greedy_generate(target, p, n) if n else [])
        if n and consumer is not None:
            assert g["target_passes"] == len(g["accepted_per_round"]) + 1 <= n
            assert 1 + sum(a + 1 for a in g["accepted_per_round"]) >= n
    # sampled text belongs to the sequence and its seed, not to the batch it ran in
    kw = dict(temperature=0.8, top_k=40, top_p=0.9, consumer=consumer, layer_ids=LAYERS.get(kind, ()))
    both = batched_generate(target, prompts[:2], max_new_tokens=[8, 8], seeds=[21, 22], **kw)
    alone = batched_generate(target, prompts[1:2], max_new_tokens=[8], seeds=[22], **kw)
    assert both[1]["tokens"] == alone[0]["tokens"] and len(both[0]["tokens"]) == 8
    # ... nor to the Draft that proposed (or to having one at all): the noise of a draw is keyed by seed and position
    no_draft = batched_generate(target, prompts[:2], max_new_tokens=[8, 8], seeds=[21, 22], **{**kw, "consumer": None, "layer_ids": ()})
    assert [g["tokens"] for g in no_draft] == [g["tokens"] for g in both]
    assert both[0]["tokens"] != batched_generate(target, prompts[:1], max_new_tokens=[8], seeds=[23], **kw)[0]["tokens"]


def test_stop_tokens_wait_for_the_minimum_length_and_filters_keep_the_head_of_the_distribution():
    from aspec_b200.inference.speculative_decode import batched_generate, filter_logits
    target = _target()
    prompt = torch.randint(0, 500, (9,), generator=torch.Generator().manual_seed(4))
    want = greedy_generate(target, prompt, 10)
    stop = want[2]
    cut = batched_generate(target, [prompt], max_new_tokens=[10], temperature=0.0, stop_token_ids=[stop])[0]
    assert cut["tokens"] == want[:3] and cut["stopped"] == "stop_token"
    held = batched_generate(target, [prompt], max_new_tokens=[10], temperature=0.0, stop_token_ids=[stop], min_new_tokens=5)[0]
    assert len(held["tokens"]) >= 5 and stop not in held["tokens"][:5]
    x = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    assert filter_logits(x, 1.0, 2, 1.0).isinf().tolist() == [[False, False, True, True]]
    assert filter_logits(x, 1.0, -1, 0.7).isinf().tolist() == [[False, False, True, True]]
    assert filter_logits(x, 1.0, -1, 0.1).isinf().tolist() == [[False, True, True, True]]
    torch.testing.assert_close(filter_logits(x, 0.5, -1, 1.0), x * 2)


def test_sequences_get_query_tiles_of_their_own_without_changing_the_result():
    """The padding that keeps one sequence per attention tile (needed by the kernels, exercised here on the CPU path):
    same logits and features as without it, for a pass with ragged new-token counts and an idle sequence."""
    from aspec_b200.models.target.dense import tile_padding
    gather, keep = tile_padding([3, 0, 5, 4], 4, "cpu")
    assert gather.tolist() == [0, 1, 2, 2, 3, 4, 5, 6, 7, 7, 7, 7, 8, 9, 10, 11]
    assert keep.tolist() == [0, 1, 2, 4, 5, 6, 7, 8, 12, 13, 14, 15]
    assert gather[keep].tolist() == list(range(12))                     # the kept rows are the real rows, in order
    target = _target()
    ids = [torch.randint(0, 500, (n,), generator=torch.Generator().manual_seed(n)) for n in (9, 6, 7)]
    plain, padded = target.new_decode_cache(3, 16), target.new_decode_cache(3, 16)
    padded.tile_positions = 4
    for step in ([ids[0][:5], ids[1][:2], ids[2][:7]], [ids[0][5:], torch.empty(0, dtype=torch.long), ids[2][:0]], [ids[0][:0], ids[1][2:], ids[2][:0]]):
        if sum(t.numel() for t in step) == 0:
            continue
        a, b = target.extend(plain, step, [0, 2]), target.extend(padded, step, [0, 2])
        torch.testing.assert_close(a["logits"], b["logits"], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(a["hidden_states"], b["hidden_states"], rtol=1e-5, atol=1e-6)
        for r, t in enumerate(step):
            plain.accept(r, t.numel())
            padded.accept(r, t.numel())
    from aspec_b200.ops.attention_sm100 import positions_per_tile
    assert positions_per_tile(32, 8) == 32 and positions_per_tile(8, 8) == 128 and positions_per_tile(40, 8) is None


def test_the_decode_benchmark_runs_on_a_toy_shape(capsys):
    from tools.performance import bench_decode
    res = bench_decode.main(["--small", "--device", "cpu"])
    capsys.readouterr()
    assert res["generated_tokens"] == res["sequences"] * res["new_tokens"] and res["target_passes"] == res["new_tokens"]
    assert res["generated_tokens_per_s"] > 0 and res["tokens_per_pass_per_sequence"] == 1.0


def test_keyed_noise_is_uniform_and_a_function_of_seed_position_and_column():
    from aspec_b200.inference.speculative_decode import keyed_uniform
    u = keyed_uniform(7, torch.arange(32), 40000)
    assert 0.0 < float(u.min()) and float(u.max()) < 1.0
    assert abs(float(u.mean()) - 0.5) < 2e-3 and abs(float(u.var()) - 1 / 12) < 1e-3
    share = torch.histc(u.flatten(), bins=16, min=0, max=1) / u.numel()
    assert float(share.min()) > 0.06 and float(share.max()) < 0.065
    assert abs(float(torch.corrcoef(torch.stack([u[0], u[1]]))[0, 1])) < 0.02            # neighbouring positions
    assert abs(float(torch.corrcoef(torch.stack([u[0, :-1], u[0, 1:]]))[0, 1])) < 0.02    # neighbouring columns
    assert abs(float(torch.corrcoef(torch.stack([u[3], keyed_uniform(8, torch.tensor([3]), 40000)[0]]))[0, 1])) < 0.02
    assert torch.equal(keyed_uniform(7, torch.tensor([3, 9]), 100), u[[3, 9], :100])      # any subset, any order of asking
