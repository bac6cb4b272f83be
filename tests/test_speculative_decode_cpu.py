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
