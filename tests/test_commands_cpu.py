"""Command-line entry points end to end on the CPU: environment check, the bounded quick start (plan, train, resume,
report, export), acceptance evaluation of the exported asset with live and with stored Target features, and the
corpus preparation commands."""
import json
import os

import pytest
import torch


def _pretokenized(path, n=6, length=48, vocab=500, seed=0):
    g = torch.Generator().manual_seed(seed)
    with open(path, "w") as f:
        for i in range(n):
            ids = torch.randint(0, vocab, (length + i,), generator=g).tolist()
            f.write(json.dumps({"data_id": f"doc-{i}", "input_ids": ids,
                                "loss_mask": [0] * 8 + [1] * (len(ids) - 8)}) + "\n")
    return str(path)


def test_doctor_reports_every_check(capsys):
    from aspec_b200.commands import doctor
    rc = doctor.main(["--json"])
    report = json.loads(capsys.readouterr().out)
    names = {c["name"] for c in report["checks"]}
    assert {"torch", "nvcc"} <= names and report["gpu_requested"] is False
    assert rc in (0, 1) and all(isinstance(c["ok"], bool) for c in report["checks"])


@pytest.fixture(scope="module")
def quickstart_run(tmp_path_factory):
    from aspec_b200.commands import quickstart
    out = tmp_path_factory.mktemp("quickstart") / "run"
    assert quickstart.main(["tiny", "--output", str(out), "--steps", "2"]) == 0
    return out


def test_quickstart_trains_resumes_and_exports(quickstart_run):
    acceptance = json.loads((quickstart_run / "acceptance.json").read_text())
    assert acceptance["status"] == "passed"
    stages = {s["stage"]: s for s in acceptance["stages"]}
    assert stages["train first half"]["rc"] == 0 and stages["resume second half"]["rc"] == 0
    assert stages["report"]["valid"] is True
    asset = quickstart_run / "stage-2" / "asset"
    assert (asset / "model.safetensors").exists() and (asset / "export_manifest.json").exists()


def test_quickstart_plan_only_starts_nothing(tmp_path, capsys):
    from aspec_b200.commands import quickstart
    out = tmp_path / "planned"
    assert quickstart.main(["tiny", "--output", str(out), "--plan"]) == 0
    assert "plan" in capsys.readouterr().out.lower()
    assert not (out / "stage-1" / "checkpoints").exists()


def test_report_on_quickstart_stage(quickstart_run, capsys):
    from aspec_b200 import train_entry
    rc = train_entry.main(["--report", str(quickstart_run / "stage-2"), "--report-format", "json"])
    report = json.loads(capsys.readouterr().out)
    assert rc == 0 and isinstance(report, dict) and report


def test_evaluate_exported_asset_with_live_target(quickstart_run, tmp_path, capsys):
    from aspec_b200.commands import evaluate_draft
    data = _pretokenized(tmp_path / "held.jsonl")
    out = tmp_path / "eval.json"
    rc = evaluate_draft.main(["--asset-dir", str(quickstart_run / "stage-2" / "asset"), "--data", data,
                              "--block-size", "4", "--anchors-per-doc", "3", "--device", "cpu", "--output", str(out)])
    capsys.readouterr()
    result = json.loads(out.read_text())
    assert rc == 0 and result["proposals"] == 18 and result["documents"] == 6
    assert len(result["accept_rate_at"]) == 3 and 1.0 <= result["tau"] <= 4.0
    rates = result["accept_rate_at"]
    assert all(0.0 <= r <= 1.0 for r in rates) and rates == sorted(rates, reverse=True)
    # the decode loop: greedy speculative generation from every document's prompt with the live Target
    rc = evaluate_draft.main(["--asset-dir", str(quickstart_run / "stage-2" / "asset"), "--data", data, "--block-size", "4",
                              "--anchors-per-doc", "1", "--device", "cpu", "--output", str(out), "--generate", "6",
                              "--generate-docs", "3"])
    capsys.readouterr()
    gen = json.loads(out.read_text())["generation"]
    assert rc == 0 and gen["new_tokens"] == 18 and gen["target_passes"] >= 3
    assert 1.0 <= gen["tokens_per_target_pass"] <= 4.0 and 0.0 <= gen["mean_accepted_draft_tokens"] <= 3.0


def test_prepare_target_data_then_evaluate_from_store(quickstart_run, tmp_path, capsys):
    from aspec_b200.commands import evaluate_draft, prepare_target_dataset
    from aspec_b200.offline.dataset import OfflineFeatureStore
    asset = quickstart_run / "stage-2" / "asset"
    data = _pretokenized(tmp_path / "held.jsonl", n=4)
    store_dir = tmp_path / "features"
    rc = prepare_target_dataset.main(["--input", data, "--output-dir", str(store_dir), "--draft-config",
                                      str(asset / "config.json"), "--device", "cpu"])
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and summary["samples"] == 4
    store = OfflineFeatureStore(str(store_dir))
    one = store.load("doc-0")
    assert one["hidden_states"].shape[0] == 48
    # a second call with --resume adds nothing and keeps the contract
    rc = prepare_target_dataset.main(["--input", data, "--output-dir", str(store_dir), "--draft-config",
                                      str(asset / "config.json"), "--device", "cpu", "--resume"])
    again = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and again["samples"] == 4 and again["contract_id"] == summary["contract_id"]
    # the stored features and output head give the statistics that the live Target gives
    results = []
    for extra in (["--features", str(store_dir)], []):
        out = tmp_path / f"eval{len(extra)}.json"
        assert evaluate_draft.main(["--asset-dir", str(asset), "--data", data, "--block-size", "4", "--anchors-per-doc", "2",
                                    "--device", "cpu", "--output", str(out), *extra]) == 0
        capsys.readouterr()
        results.append(json.loads(out.read_text()))
    assert results[0]["proposals"] == results[1]["proposals"] == 8
    assert results[0]["accept_rate_at"] == pytest.approx(results[1]["accept_rate_at"], abs=0.26)


def test_prepare_data_split_is_stable_and_deduplicated(tmp_path, capsys):
    from aspec_b200.commands import prepare_quality_dataset
    rows = [{"conversations": [{"role": "user", "content": f"question {i}"}, {"role": "assistant", "content": f"answer {i}"}]}
            for i in range(200)]
    rows += rows[:10]                                                            # duplicates
    rows.append({"conversations": [{"role": "user", "content": "no answer"}]})   # too short
    src = tmp_path / "corpus.jsonl"
    src.write_text("".join(json.dumps(r) + "\n" for r in rows))
    for name in ("a", "b"):
        assert prepare_quality_dataset.main(["--input", str(src), "--output-dir", str(tmp_path / name),
                                             "--eval-fraction", "0.1", "--seed", "3"]) == 0
    capsys.readouterr()
    a, b = (json.loads((tmp_path / n / "manifest.json").read_text()) for n in ("a", "b"))
    assert a["duplicates"] == 10 and a["too_short"] == 1 and a["train"]["rows"] + a["eval"]["rows"] == 200
    assert 5 <= a["eval"]["rows"] <= 40
    assert a["train"]["sha256"] == b["train"]["sha256"] and a["eval"]["sha256"] == b["eval"]["sha256"]
    # growing the corpus never moves an old row to the other side
    grown = tmp_path / "grown.jsonl"
    grown.write_text(src.read_text() + json.dumps({"conversations": [{"role": "user", "content": "new"},
                                                                     {"role": "assistant", "content": "row"}]}) + "\n")
    assert prepare_quality_dataset.main(["--input", str(grown), "--output-dir", str(tmp_path / "c"),
                                         "--eval-fraction", "0.1", "--seed", "3"]) == 0
    capsys.readouterr()
    old_eval = set((tmp_path / "a" / "eval.jsonl").read_text().splitlines())
    new_eval = set((tmp_path / "c" / "eval.jsonl").read_text().splitlines())
    assert old_eval <= new_eval and len(new_eval - old_eval) <= 1


def test_select_answers_rules(tmp_path, capsys):
    from aspec_b200.commands import prepare_selected_answers
    rows = [{"id": 1, "prompt": [{"role": "user", "content": "q"}],
             "candidates": [{"content": "long answer text", "score": 0.9}, {"content": "short", "score": 0.4}]},
            {"id": 2, "prompt": [{"role": "user", "content": "q2"}], "candidates": [{"content": "weak", "score": 0.1}]},
            {"id": 3, "prompt": [{"role": "user", "content": "q3"}], "candidates": []}]
    src = tmp_path / "cands.jsonl"
    src.write_text("".join(json.dumps(r) + "\n" for r in rows))

    def run(*extra):
        out = tmp_path / "out.jsonl"
        assert prepare_selected_answers.main(["--input", str(src), "--output", str(out), *extra]) == 0
        stats = json.loads(capsys.readouterr().out)
        return stats, [json.loads(line) for line in out.read_text().splitlines()]

    stats, kept = run()
    assert stats == {"output": str(tmp_path / "out.jsonl"), "kept": 2, "dropped": 1, "rule": "best_score"}
    assert kept[0]["conversations"][-1] == {"role": "assistant", "content": "long answer text"}
    stats, kept = run("--rule", "shortest")
    assert kept[0]["conversations"][-1]["content"] == "short"
    stats, kept = run("--min-score", "0.5")
    assert stats["kept"] == 1 and stats["dropped"] == 2 and kept[0]["id"] == 1


def test_convert_data_packs_loss_masks(tmp_path, capsys):
    from aspec_b200.commands import convert_pretokenized_jsonl
    from aspec_b200.data.dataset import load_training_samples
    src = _pretokenized(tmp_path / "raw.jsonl", n=3, length=20)
    out = tmp_path / "packed.jsonl"
    rc = convert_pretokenized_jsonl.main(["--input", src, "--output", str(out), "--tokenizer", "unused",
                                          "--max-seq-length", "21"])
    stats = json.loads(capsys.readouterr().out)
    rows = [json.loads(line) for line in out.read_text().splitlines()]
    assert rc == 0 and stats["samples"] == 3 and stats["pretokenized"] is True
    assert [r["data_id"] for r in rows] == ["doc-0", "doc-1", "doc-2"]
    assert [len(r["input_ids"]) for r in rows] == [20, 21, 21]               # the third row is cut at the length limit
    assert rows[0]["packed_loss_mask"] == "8,12" and "loss_mask" not in rows[0]
    again = load_training_samples(str(out), {"max_seq_length": 64})
    assert [s["packed_loss_mask"] for s in again] == [r["packed_loss_mask"] for r in rows]


def test_stitch_native_mtp_into_target_directory(tmp_path, capsys):
    from safetensors.torch import load_file, save_file
    from aspec_b200.commands import stitch_native_mtp
    asset, target, out = tmp_path / "asset", tmp_path / "target", tmp_path / "stitched"
    asset.mkdir(), target.mkdir()
    trained = {"mtp.layers.0.self_attn.q_proj.weight": torch.randn(8, 8), "mtp.fc.weight": torch.randn(8, 16),
               "embed_tokens.weight": torch.randn(4, 8)}                      # only mtp.* tensors are stitched
    save_file(trained, str(asset / "model.safetensors"))
    (asset / "export_manifest.json").write_text(json.dumps({"algorithm": "mtp"}))
    save_file({"model.layers.0.w": torch.zeros(2), "mtp.fc.weight": torch.zeros(8, 16)}, str(target / "model-00001.safetensors"))
    (target / "config.json").write_text("{}")
    (target / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": {
        "model.layers.0.w": "model-00001.safetensors", "mtp.fc.weight": "model-00001.safetensors"}}))
    rc = stitch_native_mtp.main(["--asset-dir", str(asset), "--target-dir", str(target), "--output-dir", str(out)])
    report = json.loads(capsys.readouterr().out)
    assert rc == 0 and report["tensors"] == 2 and report["replaced_existing"] == 1
    index = json.loads((out / "model.safetensors.index.json").read_text())["weight_map"]
    assert index["mtp.fc.weight"] == report["shard"] and index["model.layers.0.w"] == "model-00001.safetensors"
    assert (out / "config.json").is_symlink() and (out / "model-00001.safetensors").is_symlink()
    stitched = load_file(str(out / report["shard"]))
    assert set(stitched) == {"mtp.layers.0.self_attn.q_proj.weight", "mtp.fc.weight"}
    assert torch.equal(stitched["mtp.fc.weight"], trained["mtp.fc.weight"])
    # the Target directory itself is never modified, and other algorithms are refused
    assert json.loads((target / "model.safetensors.index.json").read_text())["weight_map"]["mtp.fc.weight"] == "model-00001.safetensors"
    with pytest.raises(ValueError, match="in place"):
        stitch_native_mtp.stitch(str(asset), str(target), str(target))
    (asset / "export_manifest.json").write_text(json.dumps({"algorithm": "dflash"}))
    with pytest.raises(ValueError, match="native MTP"):
        stitch_native_mtp.stitch(str(asset), str(target), str(tmp_path / "other"))


@pytest.mark.timeout(600)
def test_offline_training_from_prepared_features(tmp_path, capsys):
    """prepare-target-data -> training with the offline replay engine: the stored head is the one trained against, and
    a store made for other Target layers is refused before any step runs."""
    from aspec_b200 import train_entry
    from aspec_b200.commands import prepare_target_dataset
    data = _pretokenized(tmp_path / "docs.jsonl", n=16, length=40)
    feats = tmp_path / "feats"
    assert prepare_target_dataset.main(["--input", data, "--output-dir", str(feats), "--draft-config", "dspark_tiny.json",
                                        "--device", "cpu"]) == 0
    assert (feats / "lm_head.pt").exists()
    recipe = tmp_path / "recipe.yaml"
    recipe.write_text(f"""
model:
  draft_model_config: dspark_tiny.json
dataset:
  train_data_path: {data}
inference:
  inference_engine_type: offline
  offline:
    feature_dir: {feats}
training:
  training_num_gpus_per_node: 1
  micro_batch_size: 1
  draft_accumulation_steps: 2
  max_seq_length: 128
  num_train_steps: 2
  learning_rate: 1e-3
  dspark_block_size: 4
  dspark_num_anchors: 16
output_dir: {tmp_path / 'run'}
""")
    capsys.readouterr()
    assert train_entry.main(["--config", str(recipe)]) == 0
    evidence = json.loads((tmp_path / "run" / "evidence.json").read_text())
    assert evidence["state"] == "completed" and evidence["training_summary"]["completed_steps"] == 2
    assert evidence["training_summary"]["ledger"]["validated"]
    assert (feats / "embed_tokens.pt").exists()
    # the same recipe with the live Target (same seed, hence the same model) trains the same trajectory: the stored
    # features, output head and embedding are the ones the live run uses
    def losses(run_dir):
        return [json.loads(l)["train/avg_loss"] for l in open(run_dir / "runs" / "metrics.jsonl") if "train/avg_loss" in l]
    common = ["training.deterministic_anchor_sampling=true", "training.save_final_checkpoint=false"]
    assert train_entry.main(["--config", str(recipe), *common, f"output_dir={tmp_path / 'stored'}"]) == 0
    assert train_entry.main(["--config", str(recipe), *common, "inference.inference_engine_type=native",
                             "inference.inference_num_gpus=1", f"output_dir={tmp_path / 'live'}"]) == 0
    capsys.readouterr()
    stored, live = losses(tmp_path / "stored"), losses(tmp_path / "live")
    assert len(stored) == len(live) == 2 and stored == pytest.approx(live, rel=2e-3)
    with pytest.raises(ValueError, match="offline features hold layers"):
        train_entry.main(["--config", str(recipe), "model.draft_model_config=dflash_tiny.json",
                          f"output_dir={tmp_path / 'other'}"])


@pytest.mark.timeout(600)
def test_debug_instruments_and_observed_capabilities(tmp_path, capsys):
    """A run with the profiler window, step dumps and the timeline switched on writes all three under the run
    directory, and the evidence names the implementations that really ran."""
    from aspec_b200 import train_entry
    run = tmp_path / "run"
    overrides = ["output_dir=" + str(run), "training.num_train_steps=3", "debug.use_pytorch_profiler=true",
                 "debug.profile_step_start=1", "debug.profile_step_end=2", "debug.save_debug_train_data=true",
                 "debug.max_dump_steps=2", "debug.timeline_enabled=true"]
    from aspec_b200.assets import find_asset
    assert train_entry.main(["--config", find_asset("quickstart_tiny.yaml"), *overrides]) == 0
    capsys.readouterr()
    evidence = json.loads((run / "evidence.json").read_text())
    assert evidence["state"] == "completed"
    observed = evidence["capabilities_observed"]
    assert set(observed["attention"]) == {"reference_fp32_cpu"} and observed["attention"]["reference_fp32_cpu"] > 0
    assert set(observed["gemm"]) == {"torch"}
    assert [p.name for p in (run / "traces").glob("trace-*.json")] == ["trace-steps1-2-rank0.json"]
    assert sorted(p.name for p in (run / "dumps").iterdir()) == ["step-0-rank0.pt", "step-1-rank0.pt"]
    dump = torch.load(run / "dumps" / "step-1-rank0.pt", weights_only=False)
    assert "input_ids" in dump["batch"] and dump["grad_norms"] and "loss" in " ".join(dump["outputs"])
    metrics = [json.loads(line) for line in (run / "runs" / "metrics.jsonl").read_text().splitlines()]
    assert [m["step"] for m in metrics] == [0, 1, 2] and all("train/avg_loss" in m for m in metrics)
    assert json.loads((run / "tracking.json").read_text())["active"] == ["jsonl"]
    rows = [json.loads(line) for f in (run / "timeline").glob("timeline-trainer-0-*.jsonl") for line in f.read_text().splitlines()]
    updates = [r for r in rows if r["name"] == "train_update"]
    assert [r["step"] for r in updates] == [0, 1, 2] and all(r["duration_ns"] > 0 for r in updates)
    assert any(r["name"] == "batch_ready" for r in rows)
    driver = [json.loads(line) for f in (run / "timeline").glob("timeline-driver-0-*.jsonl") for line in f.read_text().splitlines()]
    assert [r["step"] for r in driver if r["name"] == "optimizer_step"] == [0, 1, 2]


@pytest.mark.timeout(600)
def test_initial_weights_from_an_exported_asset_and_wsd_schedule(quickstart_run, tmp_path, capsys):
    """A run that starts from the quick start's exported Draft holds exactly that Draft's weights (checked with a zero
    learning rate), a warm-up / stable / decay schedule reports the expected rates, and an asset of another
    architecture is refused."""
    from pathlib import Path
    from safetensors.torch import load_file
    from aspec_b200 import train_entry
    from aspec_b200.assets import find_asset
    from aspec_b200.commands.convert_to_hf import convert_checkpoint
    asset = quickstart_run / "stage-2" / "asset"
    recipe = find_asset("quickstart_tiny.yaml")
    frozen = tmp_path / "frozen"
    assert train_entry.main(["--config", recipe, f"output_dir={frozen}", "training.num_train_steps=1", "training.learning_rate=0.0",
                             "training.min_lr=0.0", "training.save_final_checkpoint=true",
                             f"model.initial_draft_model_path={asset}"]) == 0
    convert_checkpoint(input_dir=Path(frozen / "checkpoints" / "iter_0000001"), output_dir=Path(tmp_path / "again"),
                       artifact_format="aspec")
    before, after = load_file(str(asset / "model.safetensors")), load_file(str(tmp_path / "again" / "model.safetensors"))
    assert set(before) == set(after) and all(torch.equal(before[k], after[k]) for k in before)
    capsys.readouterr()
    assert train_entry.main(["--config", recipe, f"output_dir={tmp_path / 'wsd'}", "training.num_train_steps=4",
                             "training.lr_decay_style=WSD", "training.lr_wsd_decay_ratio=0.5", "training.lr_wsd_decay_style=linear",
                             "training.warmup_ratio=0.25", "training.learning_rate=1e-3", "training.min_lr=0.0"]) == 0
    summary = json.loads((tmp_path / "wsd" / "evidence.json").read_text())["training_summary"]
    assert summary["completed_steps"] == 4
    with pytest.raises(Exception, match="does not fit this Draft configuration"):
        train_entry.main(["--config", recipe, f"output_dir={tmp_path / 'bad'}", "model.draft_model_config=dflash_tiny.json",
                          f"model.initial_draft_model_path={asset}"])


@pytest.mark.timeout(600)
def test_required_throughput_measurement(tmp_path, capsys):
    from aspec_b200 import train_entry
    from aspec_b200.assets import find_asset
    recipe = find_asset("quickstart_tiny.yaml")
    with pytest.raises(ValueError, match="no valid steady throughput window"):
        train_entry.main(["--config", recipe, f"output_dir={tmp_path / 'short'}", "training.num_train_steps=2",
                          "debug.performance_measurement_required=true", "debug.performance_warmup_steps=2"])
    assert json.loads((tmp_path / "short" / "evidence.json").read_text())["state"] == "completed"
    assert train_entry.main(["--config", recipe, f"output_dir={tmp_path / 'long'}", "training.num_train_steps=4",
                             "debug.performance_measurement_required=true", "debug.performance_warmup_steps=1",
                             "debug.performance_drain_steps=1"]) == 0
    window = json.loads((tmp_path / "long" / "evidence.json").read_text())["training_summary"]["window"]
    assert window["valid"] and window["steps"] == 2 and window["tokens_per_second"] > 0
    capsys.readouterr()


def _tiny_tokenizer(path):
    """A byte-level tokenizer with the chat template's special tokens, saved where ``AutoTokenizer`` finds it offline."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    specials = ["<|im_start|>", "<|im_end|>", "<|endoftext|>", "<think>", "</think>"]
    vocab = {s: i for i, s in enumerate(specials)}
    for ch in sorted(pre_tokenizers.ByteLevel.alphabet()):
        vocab[ch] = len(vocab)
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens(specials)
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|im_end|>", pad_token="<|endoftext|>").save_pretrained(str(path))
    return str(path)


@pytest.mark.timeout(600)
def test_training_from_the_bundled_conversation_file(tmp_path, capsys):
    """Conversations -> chat template -> tokens and assistant masks -> rows -> updates, through the command line; every
    document is named after its row's ``id`` in the ledger."""
    from aspec_b200 import assets, train_entry
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    data = os.path.join(root, "examples", "data", "sample_conversations.jsonl")
    common = ["--config", assets.find_asset("quickstart_tiny.yaml"), f"dataset.train_data_path={data}",
              f"dataset.tokenizer_path={_tiny_tokenizer(tmp_path / 'tok')}", "dataset.chat_template=qwen", "training.max_seq_length=700",
              "training.num_train_steps=2", "training.save_final_checkpoint=false", f"cache_dir={tmp_path / 'cache'}"]
    assert train_entry.main([*common, f"output_dir={tmp_path / 'run'}"]) == 0
    evidence = json.loads((tmp_path / "run" / "evidence.json").read_text())
    adm = evidence["sections"]["dataset_admission"]
    assert evidence["state"] == "completed" and adm["admitted"] == adm["source_rows"] > 0 and not adm["rejected"]
    assert evidence["training_summary"]["ledger"]["validated"]
    # the same file, but the Target writes the final replies itself (stops at the end-of-turn token)
    assert train_entry.main([*common, "inference.inference_engine_type=native", "inference.inference_num_gpus=1",
                             "training.train_with_decode=true", "decode.max_new_tokens=12", "decode.stop_token_ids=[1]",
                             f"output_dir={tmp_path / 'decode'}"]) == 0
    capsys.readouterr()
    rows = [json.loads(l) for l in open(tmp_path / "decode" / "runs" / "metrics.jsonl")]
    assert all(0 < r["decode/generated_tokens"] <= 4 * 12 for r in rows if "decode/generated_tokens" in r)
