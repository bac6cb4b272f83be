"""Data pipeline, offline feature store, feature contract, topology study, trackers and small runtime modules on CPU
(reference: tests/test_data_*.py, tests/test_offline_dataset.py, tests/test_feature_contract.py, tests/test_topology.py)."""
import json
import os
import signal

import pytest
import torch

from aspec_b200.data.dataset import load_training_samples
from aspec_b200.data.loss_mask import compute_assistant_loss_mask
from aspec_b200.data.parse import create_parser
from aspec_b200.data.preprocessing import generate_vocab_mapping
from aspec_b200.data.template import TEMPLATE_REGISTRY
from aspec_b200.data.utils import unpack_loss_mask
from aspec_b200.feature_contract import (FeatureContractError, FeatureContractRuntime, build_target_feature_contract,
                                         shared_feature_union, validate_feature_contract)
from aspec_b200.offline.dataset import OfflineFeatureStore
from aspec_b200.offline.generate import materialize, target_binding


class Tok:
    """Special tokens are single ids; every other character is one id."""
    specials = ["<|im_start|>", "<|im_end|>", "<think>", "</think>"]
    eos_token_id = 1001

    def encode(self, text, add_special_tokens=False):
        out, i = [], 0
        while i < len(text):
            for k, s in enumerate(self.specials):
                if text.startswith(s, i):
                    out.append(1000 + k)
                    i += len(s)
                    break
            else:
                out.append(ord(text[i]) % 1000)
                i += 1
        return out

    def get_vocab(self):
        return {s: 1000 + k for k, s in enumerate(self.specials)}

    def apply_chat_template(self, messages, tools=None, tokenize=True, add_generation_prompt=False, **kw):
        text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        if add_generation_prompt:
            text += "<|im_start|>assistant\n"
        return self.encode(text)


CONV = [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "<think>hm</think>\n\nhello"},
        {"role": "user", "content": "more"}, {"role": "assistant", "content": "sure", "reasoning_content": "think2"}]


def test_thinking_parser_drops_history_reasoning_and_masks_the_last_turn():
    parser = create_parser(Tok(), TEMPLATE_REGISTRY.get("qwen3-thinking"))
    text = parser.format(CONV, last_turn_only=True)
    assert "hm" not in text and "<think>\nthink2\n</think>\n\nsure" in text
    ids, mask = parser.parse(CONV, 512, last_turn_only=True)
    supervised = "<think>\nthink2\n</think>\n\nsure<|im_end|>\n"
    assert int(mask.sum()) == len(Tok().encode(supervised)) and len(ids) == len(mask)
    assert int(mask[: len(ids) - int(mask.sum())].sum()) == 0              # everything before the last reply is unsupervised


def test_dataset_loader_cache_renderer_and_vocab_mapping(tmp_path):
    path = tmp_path / "c.jsonl"
    path.write_text("\n".join(json.dumps({"conversations": CONV}) for _ in range(3)))
    args = {"max_seq_length": 512, "chat_template": "qwen", "cache_dir": str(tmp_path)}
    rep = {}
    samples = load_training_samples(str(path), args, tokenizer=Tok(), report=rep)
    assert len(samples) == 3 and rep["cache"] == "miss" and rep["last_turn_only"] == 3
    rep2 = {}
    again = load_training_samples(str(path), args, tokenizer=Tok(), report=rep2)
    assert rep2["cache"] == "hit" and torch.equal(again[0]["input_ids"], samples[0]["input_ids"])
    rendered = load_training_samples(str(path), {"max_seq_length": 512, "renderer": "kimi_k3"}, tokenizer=Tok())
    mask = unpack_loss_mask(rendered[0]["packed_loss_mask"], rendered[0]["input_ids"].numel())
    assert int(mask.sum()) == 12 + 5                                        # both replies, each with its end-of-turn token
    d2t, t2d = generate_vocab_mapping(samples, 2000, 16)
    assert d2t.shape == (16,) and int(t2d.sum()) == 16
    pre = tmp_path / "pre.jsonl"
    pre.write_text(json.dumps({"input_ids": [1, 2, 3, 4], "loss_mask": [0, 0, 1, 1]}) + "\n")
    assert load_training_samples(str(pre), {"max_seq_length": 8})[0]["packed_loss_mask"] == "2,2"
    # every document has an identity (ledgers, feature stores and seeds key on it): its own id, else its place in the file
    assert [s["data_id"] for s in samples] == ["0", "1", "2"] and [s["data_id"] for s in again] == ["0", "1", "2"]
    assert [s["data_id"] for s in rendered] == ["0", "1", "2"]
    named = tmp_path / "named.jsonl"
    named.write_text("\n".join([json.dumps({"id": "a7", "conversations": CONV}), json.dumps({"conversations": CONV[:1]}),
                                json.dumps({"data_id": 12, "conversations": CONV})]))
    assert [s["data_id"] for s in load_training_samples(str(named), args, tokenizer=Tok())] == ["a7", "12"]   # row 1 has no reply
    pre.write_text("\n".join(json.dumps({"id": i, "input_ids": [1, 2, 3], "loss_mask": [0, 1, 1]}) for i in ("x", "y")))
    assert [s["data_id"] for s in load_training_samples(str(pre), {"max_seq_length": 8})] == ["x", "y"]
    pre.write_text("\n".join(json.dumps({"id": i, "input_ids": [1, 2, 3], "loss_mask": [0, 1, 1]}) for i in ("x", "y", "x")))
    with pytest.raises(ValueError, match="share one id"):
        load_training_samples(str(pre), {"max_seq_length": 8})
    dup = tmp_path / "dup.jsonl"
    dup.write_text("\n".join(json.dumps({"id": "same", "conversations": CONV}) for _ in range(2)))
    with pytest.raises(ValueError, match="share one id"):
        load_training_samples(str(dup), {"max_seq_length": 512, "chat_template": "qwen"}, tokenizer=Tok())


def test_native_assistant_span_scan():
    mask, last = compute_assistant_loss_mask(torch.tensor([5, 1, 2, 7, 7, 9, 1, 2, 8, 8]), [1, 2], [9])
    assert mask.tolist() == [0, 0, 0, 1, 1, 0, 0, 0, 1, 1] and last == 8
    only_last, _ = compute_assistant_loss_mask(torch.tensor([5, 1, 2, 7, 7, 9, 1, 2, 8, 8]), [1, 2], [9], last_turn_only=True)
    assert only_last.tolist() == [0] * 8 + [1, 1]


def test_feature_contract_identity_validation_and_union():
    kw = dict(drafter_family="dspark", target_hidden_size=32, target_num_hidden_layers=8, store_last_hidden_states=True)
    a = build_target_feature_contract(aux_hidden_state_layers=[1, 3, 5], **kw)
    validate_feature_contract(a)
    tampered = dict(a, target_hidden_size=64)
    with pytest.raises(FeatureContractError, match="identity mismatch"):
        validate_feature_contract(tampered)
    with pytest.raises(FeatureContractError):
        build_target_feature_contract(aux_hidden_state_layers=[1, 9], **kw)
    rt = FeatureContractRuntime(a, role="consumer", participant="t")
    good = {"input_ids": torch.zeros(7, dtype=torch.long), "hidden_states": torch.zeros(7, 96, dtype=torch.bfloat16),
            "last_hidden_states": torch.zeros(7, 32, dtype=torch.bfloat16)}
    rt.validate_payload(good)
    with pytest.raises(FeatureContractError, match="width"):
        rt.validate_payload({**good, "hidden_states": torch.zeros(7, 64, dtype=torch.bfloat16)})
    b = build_target_feature_contract(aux_hidden_state_layers=[3, 7], **{**kw, "store_last_hidden_states": False})
    union = shared_feature_union([a, b])
    assert union["contract"]["aux_hidden_state_layers"] == [1, 3, 5, 7]
    assert union["views"][1]["layer_columns"] == [1, 3] and not union["views"][1]["last_hidden_states"]


def test_offline_store_round_trip_hash_check_and_resume(tmp_path):
    dc = dict(target_hidden_size=32, target_num_hidden_layers=8, target_layer_ids=[1, 3, 5])
    binding = target_binding({"model": "toy"}, dc, "dspark", True)
    docs = [{"data_id": i, "input_ids": torch.randint(0, 50, (10 + i,)), "loss_mask": torch.ones(10 + i)} for i in range(3)]
    feats = lambda ids: (torch.randn(len(ids), 96), torch.randn(len(ids), 32))
    out = str(tmp_path / "off")
    materialize(out, docs[:2], feats, binding)
    store = OfflineFeatureStore(out)
    assert len(store) == 2 and store.load("1")["hidden_states"].shape == (11, 96)
    assert next(store.samples())["packed_loss_mask"] == "0,10"
    materialize(out, docs, feats, binding, resume=True)                     # appends only the missing document
    assert len(OfflineFeatureStore(out)) == 3
    with pytest.raises(FeatureContractError):
        OfflineFeatureStore(out).validate_consumer("sha-of-another-contract")
    victim = os.path.join(out, store.rows()[0]["file"])
    with open(victim, "ab") as f:
        f.write(b"x")
    with pytest.raises(ValueError, match="manifest hash"):
        OfflineFeatureStore(out).load("0")
    with pytest.raises(FileExistsError):
        OfflineFeatureStore(out, create=True, binding=binding)


def test_topology_prediction_and_legal_splits():
    from aspec_b200.topology import legal_splits, predict
    assert legal_splits(8, cp=2) == [(2, 6), (4, 4), (6, 2)]
    assert predict(48000, 90000, 5, 3) == (240000, "target")
    assert predict(48000, 90000, 6, 2)[1] == "draft"


def test_trackers_locality_identity_and_termination(tmp_path):
    from aspec_b200.locality import apportion
    from aspec_b200.runtime_control import TerminationRequested, deferred_termination, install_termination_handlers, restore_handlers
    from aspec_b200.runtime_identity import runtime_identity, verify_runtime_identity
    from aspec_b200.utils.env import forwarded_environment, recorded_environment
    from aspec_b200.utils.logging import Trackers
    t = Trackers(str(tmp_path), "wandb,nosuch")
    t.log({"train/avg_loss": 1.5, "note": "x"}, 3)
    t.close()
    tracking = json.load(open(tmp_path / "tracking.json"))
    assert tracking["active"][0] == "jsonl" and "nosuch" in tracking["unavailable"]
    assert json.loads(open(tmp_path / "runs" / "metrics.jsonl").read())["train/avg_loss"] == 1.5
    assert apportion(10, {"a": 3, "b": 1, "c": 0}) == {"a": 7, "b": 3, "c": 0}
    ident = runtime_identity()
    verify_runtime_identity(ident)
    with pytest.raises(ValueError):
        verify_runtime_identity({**ident, "sha256": "0" * 64})
    env = forwarded_environment({"ASPEC_X": "1", "CUDA_VISIBLE_DEVICES": "3", "RANDOM": "z", "NCCL_DEBUG": "INFO"})
    assert env == {"ASPEC_X": "1", "NCCL_DEBUG": "INFO"}
    assert recorded_environment({"ASPEC_API_TOKEN": "secret"})["ASPEC_API_TOKEN"] == "***"
    prev = install_termination_handlers((signal.SIGUSR1,))
    try:
        with pytest.raises(TerminationRequested):
            with deferred_termination():
                os.kill(os.getpid(), signal.SIGUSR1)
                reached = True                                              # delivery is deferred to the end of the block
            raise AssertionError("termination was swallowed")
        assert reached
    finally:
        restore_handlers(prev)


def test_workload_builders_are_deterministic_and_load_as_training_samples(tmp_path):
    import json
    from aspec_b200.commands.build_workload import build_fixed, build_mixed
    from aspec_b200.data.dataset import load_training_samples
    a = build_fixed(str(tmp_path / "a.jsonl"), sequence_length=64, rows=5, seed=3, min_token_id=10, max_token_id=500, prompt_tokens=16)
    b = build_fixed(str(tmp_path / "b.jsonl"), sequence_length=64, rows=5, seed=3, min_token_id=10, max_token_id=500, prompt_tokens=16)
    assert a["sha256"] == b["sha256"] and a["rows"] == 5
    rows = [json.loads(l) for l in open(tmp_path / "a.jsonl")]
    assert all(len(r["input_ids"]) == 64 and r["loss_tokens"] == 48 and 10 <= min(r["input_ids"]) and max(r["input_ids"]) < 500 for r in rows)
    m = build_mixed(str(tmp_path / "a.jsonl"), str(tmp_path / "m.jsonl"), lengths=[16, 40, 64], repetitions=2)
    assert m["rows"] == 6
    mixed = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert [r["seq_len"] for r in mixed] == [16, 40, 64, 16, 40, 64]
    assert mixed[1]["input_ids"] == rows[1]["input_ids"][:40] and mixed[1]["loss_tokens"] == 24 and mixed[0]["loss_tokens"] == 0
    samples = load_training_samples(str(tmp_path / "m.jsonl"), {"max_seq_length": 64})
    assert len(samples) >= 4                                            # rows without supervised tokens may be dropped


def test_kimi_and_minimax_dialects_format_history_tools_and_images():
    from aspec_b200.data.parse import create_parser
    from aspec_b200.data.template import TEMPLATE_REGISTRY
    tok = Tok()
    convo = [
        {"role": "user", "content": [{"type": "text", "text": "look "}, {"type": "image"}]},
        {"role": "assistant", "content": "<think>old thought</think>first", "tool_calls": [
            {"id": "call_1", "function": {"name": "add", "arguments": "{\"a\": 1, \"b\": [2]}"}}]},
        {"role": "tool", "content": "3", "tool_call_id": "call_1"},
        {"role": "tool", "content": "4"},
        {"role": "user", "content": "and now?"},
        {"role": "assistant", "content": "answer", "reasoning_content": "new thought"},
    ]
    kimi = create_parser(tok, TEMPLATE_REGISTRY.get("kimi-k25-vlm"))
    text = kimi.format(convo)
    assert text.startswith("<|im_user|>user<|im_middle|>look <|media_begin|>image<|media_content|><|media_pad|><|media_end|>\n<|im_end|>")
    # history turn: reasoning dropped, an empty block in its place, the call section after the text
    assert ("<|im_assistant|>assistant<|im_middle|><think></think>first<|tool_calls_section_begin|><|tool_call_begin|>call_1"
            "<|tool_call_argument_begin|>{\"a\": 1, \"b\": [2]}<|tool_call_end|><|tool_calls_section_end|><|im_end|>") in text
    assert "<|im_system|>tool<|im_middle|>## Return of call_1\n3<|im_end|><|im_system|>tool<|im_middle|>4<|im_end|>" in text
    assert text.endswith("<|im_assistant|>assistant<|im_middle|><think>new thought</think>answer<|im_end|>")
    assert "old thought" not in text
    assert kimi.format(convo[:1], add_generation_prompt=True).endswith("<|im_assistant|>assistant<|im_middle|><think>")
    assert "<|image|>" in kimi.format(convo[:1], expand_media_tokens=False)
    ids, mask = kimi.parse(convo, 4096)
    assert ids.shape == mask.shape and 0 < int(mask.sum()) < len(ids)
    _, last = kimi.parse(convo, 4096, last_turn_only=True)
    assert 0 < int(last.sum()) < int(mask.sum())
    supervised = "".join(chr(int(t)) for t, m in zip(ids, last) if m and t < 1000)
    assert supervised.startswith("new thought") or "answer" in supervised

    mm = create_parser(tok, TEMPLATE_REGISTRY.get("minimax-m2"))
    text = mm.format(convo)
    assert text.startswith("]~!b[]~b]system\nYou are a helpful assistant. Your name is MiniMax-M2.5")
    assert "]~b]user\nlook ]<]start of image[>[]<]vision pad[>[]<]end of image[>[\n[e~[\n" in text
    assert ("]~b]ai\nfirst\n<minimax:tool_call>\n<invoke name=\"add\">\n<parameter name=\"a\">1</parameter>\n"
            "<parameter name=\"b\">[2]</parameter>\n</invoke>\n</minimax:tool_call>[e~[\n") in text
    assert "]~b]tool\n<response>3</response>\n<response>4</response>[e~[\n" in text          # one tool turn for both results
    assert text.endswith("]~b]ai\n<think>\nnew thought\n</think>\n\nanswer[e~[\n") and "old thought" not in text
    own_system = mm.format([{"role": "system", "content": "be brief"}] + convo[4:])
    assert own_system.startswith("]~!b[]~b]system\nbe brief[e~[\n]~b]user\nand now?[e~[\n")
    ids, mask = mm.parse(convo, 4096)
    assert 0 < int(mask.sum()) < len(ids)
    assert mm.format(convo[:1], add_generation_prompt=True).endswith("]~b]ai\n<think>\n")
