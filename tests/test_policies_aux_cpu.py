"""Configuration policies (EAGLE4, MTP conditioning), analytical acceptance statistics, run reports, the timeline,
step dumps, profiling windows and the recipe catalogue command, all on the CPU."""
import json
import os

import pytest
import torch


# -- EAGLE4 configuration policy ---------------------------------------------------------------------------------------
def _eagle4(**extra):
    raw = {"vocab_size": 1000, "hidden_size": 64, "num_hidden_layers": 1,
           "efficient_lm_head_config": {"type": "low_rank", "rank": 16, "num_candidates": 32}}
    raw.update(extra)
    return raw


def test_eagle4_policy_defaults_and_bounds():
    from aspec_b200.config.eagle4 import eagle4_policy, eagle4_training_policy
    policy = eagle4_policy(_eagle4())
    assert policy["stage"] == "draft" and policy["rank"] == 16 and policy["num_candidates"] == 32
    assert policy["teacher_top_k"] == 32 and policy["loss_chunk_size"] == 128
    assert "loss_chunk_size" not in eagle4_training_policy(_eagle4(candidate_loss_chunk_size=64))
    assert eagle4_policy(_eagle4(eagle4_training_stage="candidate_head", candidate_teacher_top_k=50))["teacher_top_k"] == 50
    for bad in (dict(num_hidden_layers=2), dict(eagle4_training_stage="both"), dict(draft_vocab_size=500),
                dict(lm_head_rank_divisor=4), dict(efficient_lm_head_config={"type": "dense"}), dict(fc_norm="yes"),
                dict(attention_bias=True), dict(rope_is_neox_style=False),
                dict(efficient_lm_head_config={"type": "low_rank", "rank": 65, "num_candidates": 32}),
                dict(efficient_lm_head_config={"type": "low_rank", "rank": 16, "num_candidates": 1001}),
                dict(efficient_lm_head_config={"type": "low_rank", "rank": True, "num_candidates": 32}),
                dict(candidate_loss_chunk_size=0)):
        with pytest.raises(ValueError, match="EAGLE4"):
            eagle4_policy(_eagle4(**bad))


def test_eagle4_structure_routing_geometry():
    from aspec_b200.config.eagle4 import eagle4_structure
    assert eagle4_structure(_eagle4()) == {"ffn_type": "dense"}
    with pytest.raises(ValueError, match="enable_moe is false"):
        eagle4_structure(_eagle4(n_routed_experts=8))
    moe = dict(enable_moe=True, n_routed_experts=16, num_experts_per_tok=4, moe_intermediate_size=32, n_group=4, topk_group=2)
    s = eagle4_structure(_eagle4(**moe))
    assert s["ffn_type"] == "eagle4_moe" and s["n_group"] == 4 and s["topk_group"] == 2 and s["expert_bias_update_rate"] == 1e-3
    assert s["routed_scaling_factor"] == 1.0 and "moe_latent_size" not in s
    latent = eagle4_structure(_eagle4(**moe, moe_architecture="nemotron_latent_relu2", hidden_act="relu2",
                                      moe_latent_size=24, moe_shared_expert_intermediate_size=48, n_shared_experts=1))
    assert latent["moe_latent_size"] == 24 and latent["n_shared_experts"] == 1
    for bad in (dict(num_experts_per_tok=17), dict(n_group=3), dict(topk_group=5), dict(n_group=16),
                dict(n_group=4, topk_group=1, num_experts_per_tok=5), dict(hidden_act="relu2"),
                dict(moe_architecture="dense_moe"), dict(scoring_func="softmax"), dict(aux_loss_alpha=0.01),
                dict(routed_scaling_factor=float("nan")), dict(n_shared_experts=-1), dict(norm_topk_prob=1)):
        with pytest.raises(ValueError, match="EAGLE4"):
            eagle4_structure(_eagle4(**{**moe, **bad}))


def test_eagle4_asset_metadata_matches_stage():
    from aspec_b200.config.eagle4 import eagle4_asset_metadata
    draft = eagle4_asset_metadata(_eagle4(), 0)
    assert draft["scope"] == "draft_initialization" and draft["candidate_head_trained"] is False
    trained = eagle4_asset_metadata(_eagle4(eagle4_training_stage="candidate_head"), 120)
    assert trained["scope"] == "trained_candidate" and trained["candidate_optimizer_steps"] == 120
    with pytest.raises(ValueError):
        eagle4_asset_metadata(_eagle4(), 5)
    with pytest.raises(ValueError):
        eagle4_asset_metadata(_eagle4(eagle4_training_stage="candidate_head"), 0)


# -- MTP conditioning --------------------------------------------------------------------------------------------------
def _conditioned(mode="hidden", **extra):
    native = {"hidden_size": 64, "vocab_size": 512, "num_hidden_layers": 4, "num_attention_heads": 4,
              "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "layer_types": ["full_attention"]}
    raw = {"architectures": ["DSparkDraftModel"], "hidden_size": 64, "target_hidden_size": 64, "vocab_size": 512,
           "target_num_hidden_layers": 4, "layer_types": ["full_attention"],
           "mtp_conditioning": {"mode": mode, "native_config": native}}
    raw.update(extra)
    return raw


def test_mtp_conditioning_resolution_and_refusals():
    from aspec_b200.config.mtp_conditioning import mtp_conditioning_semantics, resolve_mtp_conditioning
    assert resolve_mtp_conditioning({"hidden_size": 64}) is None and mtp_conditioning_semantics({}) is None
    hidden = mtp_conditioning_semantics(_conditioned("hidden"))
    assert hidden["mode"] == "hidden" and hidden["fusion"] == "zero_initialized_embedding_residual"
    assert hidden["native_config"]["hidden_size"] == 64 and "native_mtp" in hidden["frozen"]
    assert mtp_conditioning_semantics(_conditioned("token"))["fusion"] is None
    bad_specs = [dict(mtp_conditioning={"mode": "hidden"}), dict(mtp_conditioning={"mode": "both", "native_config": {}}),
                 dict(mtp_conditioning={"mode": "token", "native_config": "path"}), dict(ffn_type="moe"),
                 dict(is_causal=True), dict(attention_mode="mla"), dict(layer_types=["sliding_attention"]),
                 dict(architectures=["LlamaForCausalLMEagle3"]), dict(model_type="dflash2"), dict(vocab_size=1024),
                 dict(target_num_hidden_layers=8), dict(hidden_size=32)]
    for bad in bad_specs:
        with pytest.raises(ValueError):
            resolve_mtp_conditioning(_conditioned(**bad))
    resolved = resolve_mtp_conditioning(_conditioned())
    resolved["native_config"]["hidden_size"] = 1          # a copy: the caller's dictionary is never aliased
    assert _conditioned()["mtp_conditioning"]["native_config"]["hidden_size"] == 64


# -- acceptance statistics ---------------------------------------------------------------------------------------------
def test_acceptance_statistics_against_direct_sums():
    from aspec_b200.ops.acceptance import acceptance_components, acceptance_statistics
    alpha = torch.tensor([[0.5, 0.5, 0.5], [1.0, 0.0, 1.0], [0.9, 0.9, 0.9]])
    mask = torch.tensor([[1, 1, 1], [1, 1, 0], [0, 0, 0]])
    stats = acceptance_statistics(alpha, mask)
    assert stats.shape == (2, 4)
    assert torch.allclose(stats[0, :3], torch.tensor([1.5, 0.5, 0.5])) and torch.equal(stats[1, :3], torch.tensor([2., 2., 1.]))
    # tau: 1 + .5 + .25 + .125 and 1 + 1 + 0 + 0; the fully masked block counts in neither row
    assert stats[0, 3].item() == pytest.approx(1.875 + 2.0) and stats[1, 3].item() == 2.0
    parts = acceptance_components(stats)
    assert list(parts) == ["accept_rate@0", "accept_rate@1", "accept_rate@2", "tau_probabilistic"]
    with pytest.raises(ValueError):
        acceptance_statistics(alpha, mask[:, :2])


# -- run report --------------------------------------------------------------------------------------------------------
def test_run_report_flags_every_inconsistency(tmp_path):
    from aspec_b200.reporting import build_run_report, render_report
    run = tmp_path / "run"
    run.mkdir()
    empty = build_run_report(str(run))
    assert not empty["valid"] and set(empty["problems"]) == {"missing plan.json", "missing evidence.json"}
    plan = {"plan_id": "sha256:aa", "workload": {"algorithm": "dspark"}, "policy": "strict", "capabilities": []}
    good = {"plan_id": "sha256:aa", "state": "completed", "accelerators": {"cuda": False},
            "training_summary": {"completed_steps": 4, "ledger": {"validated": True, "committed_work_ids": list(range(8))},
                                 "window": {"valid": True, "tokens_per_second": 1234.5, "steps": 3}}}
    (run / "plan.json").write_text(json.dumps(plan))
    (run / "evidence.json").write_text(json.dumps(good))
    (run / "checkpoints").mkdir()
    (run / "checkpoints" / "latest_checkpointed_iteration.txt").write_text("4")
    report = build_run_report(str(run))
    assert report["valid"] and report["committed_work"] == 8 and report["latest_checkpoint"] == 4
    text = render_report(report)
    assert "1234.5 input tokens/s over 3 steady updates" in text and "PROBLEM" not in text
    for change, needle in (({"plan_id": "sha256:bb"}, "different plan"), ({"state": "failed"}, "run state is 'failed'")):
        (run / "evidence.json").write_text(json.dumps({**good, **change}))
        bad = build_run_report(str(run))
        assert not bad["valid"] and any(needle in p for p in bad["problems"]) and "PROBLEM" in render_report(bad)
    # a GPU run whose dispatcher launched another implementation than the plan chose is flagged; a CPU run is not
    planned = {**plan, "capabilities": [{"subsystem": "attention", "choice": "tcgen05_interval_flash", "reason": ""}]}
    (run / "plan.json").write_text(json.dumps(planned))
    fallback = {**good, "capabilities_observed": {"attention": {"dense_mask_fp32": 12}}}
    (run / "evidence.json").write_text(json.dumps(fallback))
    assert build_run_report(str(run))["valid"]
    (run / "evidence.json").write_text(json.dumps({**fallback, "accelerators": {"cuda": True}}))
    flagged = build_run_report(str(run))
    assert not flagged["valid"] and "the run launched ['dense_mask_fp32']" in flagged["problems"][0]
    (run / "evidence.json").write_text(json.dumps({**fallback, "accelerators": {"cuda": True}, "capabilities_observed": {
        "attention": {"tcgen05_interval_flash": 40, "dense_mask_fp32": 2}}}))
    assert build_run_report(str(run))["valid"]
    (run / "plan.json").write_text(json.dumps(plan))
    unvalidated = json.loads(json.dumps(good))
    unvalidated["training_summary"]["ledger"]["validated"] = False
    (run / "evidence.json").write_text(json.dumps(unvalidated))
    assert any("ledger" in p for p in build_run_report(str(run))["problems"])


def test_evidence_recorder_lifecycle(tmp_path):
    from types import SimpleNamespace
    from aspec_b200.evidence import SCHEMA, RunEvidenceRecorder, package_hash
    plan = SimpleNamespace(plan_id="sha256:cc", capabilities=[SimpleNamespace(subsystem="attention", planned="tcgen05")])
    rec = RunEvidenceRecorder(plan, str(tmp_path))
    doc = json.loads((tmp_path / "evidence.json").read_text())
    assert doc["schema_version"] == SCHEMA and doc["state"] == "running" and doc["package_sha256"] == package_hash()
    assert doc["capabilities_planned"] == [{"subsystem": "attention", "planned": "tcgen05"}]
    rec.record("dataset", {"admitted": 10})
    rec.observe_capability("attention", "reference")
    try:
        raise RuntimeError("lost a rank")
    except RuntimeError as exc:
        rec.fail(exc)
    doc = json.loads((tmp_path / "evidence.json").read_text())
    assert doc["state"] == "failed" and doc["failure"]["type"] == "RuntimeError" and "lost a rank" in doc["failure"]["traceback"]
    assert doc["sections"]["dataset"] == {"admitted": 10} and doc["capabilities_observed"] == {"attention": "reference"}
    rec.complete({"completed_steps": 2})
    doc = json.loads((tmp_path / "evidence.json").read_text())
    assert doc["state"] == "completed" and doc["training_summary"] == {"completed_steps": 2}
    assert not os.path.exists(str(tmp_path / "evidence.json.tmp"))


def test_preflight_without_gpus():
    from aspec_b200.preflight import run_cluster_preflight
    out = run_cluster_preflight({"world_size": 2, "inference_num_gpus": 2, "inference_engine_type": "native"})
    assert out["required_gpus"] == 4 and out["mode"] == "single_node"
    if not torch.cuda.is_available():
        assert out["visible_gpus"] == 0 and out["ok"] is True
    assert run_cluster_preflight({"world_size": 2, "inference_num_gpus": 2, "inference_engine_type": "synthetic"})["required_gpus"] == 2
    # colocated roles share GPUs: the larger role sets the requirement
    assert run_cluster_preflight({"world_size": 8, "inference_num_gpus": 2, "inference_engine_type": "native",
                                  "colocate": True})["required_gpus"] == 8


# -- timeline, dumps, profiling windows --------------------------------------------------------------------------------
def test_timeline_events_spans_and_env(tmp_path, monkeypatch):
    from aspec_b200.utils.timeline import Timeline, timeline_from_env
    off = Timeline(None)
    off.event("ignored")
    with off.span("ignored"):
        pass
    off.close()
    t = Timeline(str(tmp_path), role="trainer", rank=3, run_id="r1", flush_every=2)
    t.event("step", index=1)
    assert (tmp_path / f"timeline-trainer-3-{os.getpid()}.jsonl").read_text() == ""        # still buffered
    with t.span("backward", micro=0):
        pass
    t.event("tail")
    t.close()
    rows = [json.loads(line) for line in (tmp_path / f"timeline-trainer-3-{os.getpid()}.jsonl").read_text().splitlines()]
    assert [r["name"] for r in rows] == ["step", "backward", "tail"]
    assert rows[1]["duration_ns"] >= 0 and rows[1]["micro"] == 0 and rows[0]["rank"] == 3 and rows[0]["run_id"] == "r1"
    assert rows[0]["t_ns"] <= rows[1]["t_ns"] <= rows[2]["t_ns"]
    monkeypatch.delenv("ASPEC_TIMELINE_DIR", raising=False)
    assert timeline_from_env("driver").enabled is False
    monkeypatch.setenv("ASPEC_TIMELINE_DIR", str(tmp_path / "env"))
    monkeypatch.setenv("ASPEC_TIMELINE_RUN_ID", "r2")
    live = timeline_from_env("driver", 1)
    assert live.enabled and live.run_id == "r2"
    live.close()


def test_dump_step_records_batch_outputs_and_norms(tmp_path):
    from aspec_b200.utils.train_dump import dump_step
    model = torch.nn.Linear(4, 2)
    model(torch.ones(3, 4)).sum().backward()
    big = torch.ones(64)
    path = dump_step(str(tmp_path), 7, 1, batch={"input_ids": torch.arange(5), "features": big, "note": "x"},
                     outputs={"loss": torch.tensor(1.5), "terms": [torch.tensor(2.0)]}, model=model, max_tensor_elems=16)
    assert path.endswith(os.path.join("dumps", "step-7-rank1.pt"))
    record = torch.load(path, weights_only=False)
    assert torch.equal(record["batch"]["input_ids"], torch.arange(5)) and record["batch"]["note"] == "x"
    assert record["batch"]["features"] == {"shape": (64,), "dtype": "torch.float32", "norm": 8.0}
    assert record["outputs"]["loss"].item() == 1.5 and record["outputs"]["terms"][0].item() == 2.0
    assert record["grad_norms"]["bias"] == pytest.approx(float(model.bias.grad.norm()))
    assert set(record["param_norms"]) == {"weight", "bias"}


def test_step_profiler_window_writes_one_trace(tmp_path):
    from aspec_b200.utils.profiling import StepProfiler
    idle = StepProfiler(str(tmp_path / "none"))
    for i in range(3):
        idle.step(i)
    idle.close()
    assert idle.written == [] and not (tmp_path / "none").exists()
    prof = StepProfiler(str(tmp_path / "traces"), start_step=1, end_step=3, rank=2)
    for i in range(5):
        prof.step(i)
        assert prof.active == (1 <= i < 3)
        torch.ones(8).sum()
    prof.close()
    assert [os.path.basename(p) for p in prof.written] == ["trace-steps1-3-rank2.json"]
    assert "traceEvents" in json.loads(open(prof.written[0]).read())
    late = StepProfiler(str(tmp_path / "late"), start_step=0, end_step=10)
    late.step(0)
    late.close()                                                  # a run that ends inside the window still writes it
    assert len(late.written) == 1 and not late.active


# -- recipe catalogue command ------------------------------------------------------------------------------------------
def test_recipes_command_list_show_plan(capsys):
    from aspec_b200.commands import recipes
    names = sorted(recipes.catalog())
    assert "quickstart_tiny" in names and len(names) >= 19
    assert recipes.main(["list"]) == 0
    listed = capsys.readouterr().out
    assert all(name in listed for name in names)
    assert recipes.main(["show", "quickstart_tiny"]) == 0
    assert "dspark_tiny" in capsys.readouterr().out
    assert recipes.main(["plan", "quickstart_tiny"]) == 0
    assert "sha256:" in capsys.readouterr().out


def test_typed_evidence_sections_are_checked_against_the_plan(tmp_path):
    from types import SimpleNamespace
    import pytest
    from aspec_b200.evidence import EvidenceError, RunEvidenceRecorder
    caps = [SimpleNamespace(subsystem="attention", choice="tcgen05_interval_flash", reason=""),
            SimpleNamespace(subsystem="feature_transport", choice="peer_memory", reason=""),
            SimpleNamespace(subsystem="data_parallel", choice="REPLICATE", reason="")]
    plan = SimpleNamespace(plan_id="sha256:aa", capabilities=caps, policy={"draft_gpus": 2, "target_gpus": 1})
    rec = RunEvidenceRecorder(plan, str(tmp_path))
    with pytest.raises(EvidenceError):       # 10 source rows cannot be 7 admitted + 2 rejected
        rec.record_dataset_admission(dataset_size=7, admission={"source_rows": 10, "admitted": 7, "rejected": {"too_long": 2}})
    rec.record_dataset_admission(dataset_size=7, admission={"source_rows": 10, "admitted": 7, "rejected": {"too_long": 3}, "fingerprint": "f"})
    with pytest.raises(EvidenceError):       # the plan has two Draft trainers
        rec.record_actor_initialization(training_actors=[{"name": "t0", "device": "cuda:1"}], inference_engines=[{"name": "e0", "device": "cuda:0"}])
    with pytest.raises(EvidenceError):       # two processes on one GPU
        rec.record_actor_initialization(training_actors=[{"name": "t0", "device": "cuda:1"}, {"name": "t1", "device": "cuda:1"}],
                                        inference_engines=[{"name": "e0", "device": "cuda:0"}])
    rec.record_actor_initialization(training_actors=[{"name": "t0", "device": "cuda:1"}, {"name": "t1", "device": "cuda:2"}],
                                    inference_engines=[{"name": "e0", "device": "cuda:0"}])
    with pytest.raises(EvidenceError):
        rec.record_cluster_preflight({"state": "failed", "problems": ["peer_access"]})
    with pytest.raises(EvidenceError):
        rec.record_cluster_preflight({"state": "validated", "gpu_count": 2})
    rec.record_cluster_preflight({"state": "validated", "gpu_count": 8})
    with pytest.raises(EvidenceError):       # committed work without a validated ledger is not evidence
        rec.record_training({"completed_steps": 3, "ledger": {"validated": False}})
    rec.observe_capability("attention", {"tcgen05_interval_flash": 12, "dense_mask_fp32": 1})
    rec.record_training({"completed_steps": 3, "ledger": {"validated": True, "committed": 48}})
    with pytest.raises(EvidenceError):
        rec.record_cleanup({"order": ["trainers", "engines"]})
    rec.record_cleanup({"order": ["manager", "engines", "trainers"], "engines_observed_dead": True})
    rec.complete({"completed_steps": 3})
    doc = json.loads((tmp_path / "evidence.json").read_text())
    assert doc["phase"] == "completed" and doc["sections"]["dataset_admission"]["rejected"] == {"too_long": 3}
    act = doc["capabilities_activated"]
    assert act["attention"]["launches"] == 12 and act["feature_transport"]["optimizer_steps_observed"] == 3
    assert act["data_parallel"]["draft_gpus"] == 2 and act["work_ledger"]["committed"] == 48
    assert doc["sections"]["actor_initialization"]["training_actor_count"] == 2
