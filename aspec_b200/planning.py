"""Config -> immutable, hashed ``ExecutionPlan``.

The plan is what the run is held to: workload contract (what is trained on what), execution policy (how
many ranks in which role, which parallelism), capability decisions (which kernel / transport path each
subsystem takes and why), and the resolved draft config.  ``plan_id`` is the SHA-256 of its canonical
JSON; ``to_runtime_args`` flattens it for the processes (reference: aspec/planning.py:99-196, 1822-2314).
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List

from aspec_b200 import __version__
from aspec_b200.config.draft_attention import (context_shard_alignment, resolve_attention_policy, thd_contract)
from aspec_b200.config.draft_config import (AutoDraftModelConfig, draft_model_semantics, resolve_draft_algorithm)
from aspec_b200.config.draft_structure import resolve_ffn_policy
from aspec_b200.config.train_config import Config, config_to_flat_args

HBM_BYTES = 180 * 1024 ** 3


@dataclass(frozen=True)
class CapabilityDecision:
    subsystem: str
    choice: str
    reason: str


@dataclass
class ExecutionPlan:
    workload: Dict[str, Any]
    policy: Dict[str, Any]
    capabilities: List[CapabilityDecision]
    draft_config: Dict[str, Any]
    runtime_args: Dict[str, Any]
    memory: Dict[str, Any] = field(default_factory=dict)
    schema_version: str = "aspec.execution-plan/v1"

    def _body(self) -> dict:
        return {"schema_version": self.schema_version, "framework_version": __version__, "workload": self.workload,
                "policy": self.policy, "capabilities": [dataclasses.asdict(c) for c in self.capabilities],
                "draft_config": self.draft_config, "memory": self.memory}

    @property
    def plan_id(self) -> str:
        return "sha256:" + hashlib.sha256(json.dumps(self._body(), sort_keys=True, default=str).encode()).hexdigest()

    def to_json(self) -> str:
        return json.dumps({"plan_id": self.plan_id, **self._body(), "runtime_args": self.runtime_args}, indent=2,
                          sort_keys=True, default=str)

    def to_runtime_args(self) -> Dict[str, Any]:
        return {**self.runtime_args, "plan_id": self.plan_id}


def _load_draft(flat: Dict[str, Any]) -> dict:
    path = flat.get("draft_model_config")
    if not path:
        raise ValueError("model.draft_model_config is required")
    from aspec_b200.assets import load_draft_config
    raw = dict(load_draft_config(path))
    raw.update(flat.get("draft_overrides") or {})          # model.draft_overrides: fields laid over the file
    return AutoDraftModelConfig.from_dict(raw).to_dict()


def resolve_batch_size(flat: Dict[str, Any], dp: int) -> dict:
    """Documents per optimizer update and the derived global quantities."""
    mbs, acc = int(flat["micro_batch_size"]), int(flat["draft_accumulation_steps"])
    per_update = dp * mbs * acc
    return {"dp_size": dp, "micro_batch_size": mbs, "accumulation": acc, "documents_per_update": per_update,
            "max_tokens_per_update": per_update * int(flat["max_seq_length"])}


def estimate_memory(draft: dict, flat: Dict[str, Any], algorithm: str, shard: int, strategy: str = "REPLICATE") -> dict:
    """Resident bytes per Draft GPU: bf16 weights, fp32 gradient, master and moments (what of them the strategy shards
    over ``shard`` ranks), frozen head and embedding, ring slots and the largest vocabulary-sized activations.
    REPLICATE keeps all 18 bytes per parameter; SHARD_OPTIMIZER keeps weights and gradients (6) and shards masters and
    moments (12); FULL_SHARD shards all 18 and adds two whole layers of working copies (weights + gradients)."""
    D, V, L = draft["hidden_size"], draft["vocab_size"], draft["num_hidden_layers"]
    I = draft.get("intermediate_size", 4 * D)
    hq, hk = draft["num_attention_heads"], draft["num_key_value_heads"]
    d = draft.get("head_dim") or D // hq
    per_layer = D * (hq * d) * 2 + D * (hk * d) * 2 + 3 * D * I
    n_tl = draft.get("num_target_layers") or draft.get("num_aux_hidden_states") or 3
    Dt = draft.get("target_hidden_size") or D
    trainable = L * per_layer + n_tl * Dt * D
    if algorithm == "dspark":
        trainable += 2 * V * int(draft.get("markov_rank", 0))
    if algorithm in ("eagle3", "eagle4"):
        trainable += (draft.get("draft_vocab_size") or V) * D
    frozen = 2 * V * D
    rows = int(flat.get("dspark_num_anchors", 512)) * int(flat.get("dspark_block_size", 7))
    logits = 2 * rows * V * 2
    row_tokens = int(flat["max_seq_length"]) * (1 if flat.get("dflash_packing") else max(int(flat.get("micro_batch_size", 1)), 1))
    slot = row_tokens * (n_tl + 1) * Dt * 2 + row_tokens * 8
    ring = slot * int(flat.get("transport_destination_ring_slots", 1))
    shard = max(shard, 1)
    strategy = str(strategy).upper()
    if strategy == "FULL_SHARD" and shard > 1:
        root = trainable - L * per_layer
        weights = trainable * 2 // shard + (2 * per_layer + root) * 2
        state = trainable * 16 // shard + (2 * per_layer + root) * 4
    elif strategy == "SHARD_OPTIMIZER" and shard > 1:
        weights, state = trainable * 2, trainable * 4 + trainable * 12 // shard
    else:
        weights, state = trainable * 2, trainable * 16
    total = weights + state + frozen * 2 + logits + ring
    return {"trainable_parameters": trainable, "frozen_parameters": frozen, "weights_bf16": weights,
            "optimizer_fp32": state, "frozen_bf16": frozen * 2, "vocab_activations": logits,
            "ring_bytes": ring, "estimated_total": total, "hbm_bytes": HBM_BYTES, "fits": total < 0.9 * HBM_BYTES}


def estimate_target_memory(target: dict, tp: int = 1, max_tokens: int = 0) -> dict:
    """Resident bf16 bytes per GPU of one in-framework Target replica spread over ``tp`` GPUs: attention and feed-forward
    (or expert) weights divide by ``tp``; embedding, output head and norms do not; plus the activations of one pass over
    ``max_tokens`` tokens (residual stream, q/k/v, one feed-forward intermediate)."""
    D, V, L = int(target["hidden_size"]), int(target["vocab_size"]), int(target["num_hidden_layers"])
    hq, hk = int(target["num_attention_heads"]), int(target["num_key_value_heads"])
    d = int(target.get("head_dim") or D // hq)
    I = int(target.get("intermediate_size") or 4 * D)
    E = int(target.get("num_experts") or 0)
    dense_first = int(target.get("first_k_dense_replace") or 0) if E else L
    attn = D * (hq + 2 * hk) * d + hq * d * D
    dense_ffn = 3 * D * I
    Im = int(target.get("moe_intermediate_size") or 0)
    shared = int(target.get("num_shared_experts") or 0) * int(target.get("moe_shared_expert_intermediate_size") or Im)
    moe_ffn = E * 3 * D * Im + 3 * D * shared
    sharded = L * attn + dense_first * dense_ffn + (L - dense_first) * moe_ffn
    whole = 2 * V * D + (L - dense_first) * E * D
    tp = max(int(tp), 1)
    width = max(I, Im * max(int(target.get("num_experts_per_tok") or 1), 1)) // tp
    act = int(max_tokens) * (4 * D + (hq + 2 * hk) * d // tp + 3 * width) * 2
    total = (sharded // tp + whole) * 2 + act
    return {"parameters": sharded + whole, "weights_bf16_per_gpu": (sharded // tp + whole) * 2, "activations": act,
            "estimated_total": total, "tp_size": tp, "fits": total < 0.9 * HBM_BYTES}


GPUS_PER_NODE = 8


def validate_scope(flat: Dict[str, Any], draft: dict, algorithm: str, policy: dict, ffn: dict) -> List[str]:
    """What this framework can run, checked before anything starts; returns notes for decisions it made on the way.

    The rules are the ones a recipe can violate here (reference: aspec/planning.py:797-1238, whose checks about Ray
    placement, the serving engine's parallelism and the store's transports have no counterpart in this process model):
    GPU budget of one node, divisibility of every parallel degree, which attention variants each sequence-parallel
    scheme covers, engine / dataset prerequisites, and schedule arithmetic."""
    notes: List[str] = []
    g = flat.get
    world = int(flat["world_size"])
    engine = g("inference_engine_type")
    if engine not in ("native", "offline", "synthetic"):
        raise ValueError(f"inference.inference_engine_type {engine!r} is not available: use native (in-framework Target), "
                         "offline (stored features) or synthetic")
    targets = int(g("inference_num_gpus") or 0) if engine == "native" else 0
    if int(g("training_num_nodes", 1) or 1) != 1:
        raise ValueError("training.training_num_nodes must be 1: processes are started on this node only")
    if world < 1:
        raise ValueError("at least one Draft GPU is needed")
    if engine == "native" and targets < 1:
        raise ValueError("the in-framework Target needs inference.inference_num_gpus >= 1")
    shared = bool(g("colocate"))                     # both roles on the same GPUs
    if (max(world, targets) if shared else world + targets) > GPUS_PER_NODE:
        raise ValueError(f"{targets} Target + {world} Draft GPUs exceed the {GPUS_PER_NODE} GPUs of one node"
                         + ("" if shared else " (training.colocate shares GPUs between the roles)"))
    if engine == "offline" and not g("offline_feature_dir"):
        raise ValueError("inference_engine_type=offline needs inference.offline.feature_dir")
    per_engine = int(g("inference_num_gpus_per_engine", 1) or 1)
    if engine == "native" and targets % per_engine:
        raise ValueError(f"inference_num_gpus ({targets}) must be a multiple of inference_num_gpus_per_engine ({per_engine})")
    tp = int(g("target_tp_size", 1) or 1)
    if engine == "native":
        from aspec_b200.inference.factory import target_config_from_args
        tcfg = target_config_from_args(flat, draft)
        if tp > 1:
            if targets % tp:
                raise ValueError(f"inference_num_gpus ({targets}) must be a multiple of inference.target.tp_size ({tp})")
            for key in ("num_attention_heads", "num_key_value_heads"):
                if int(tcfg[key]) % tp:
                    raise ValueError(f"inference.target.tp_size ({tp}) must divide the Target's {key} ({tcfg[key]})")
            notes.append(f"Target engines are tensor parallel over {tp} GPUs each: {targets // tp} engine(s)")
        need = estimate_target_memory(tcfg, tp, int(g("inference_batch_tokens") or 0) or int(flat["max_seq_length"]))
        if not need["fits"]:
            raise ValueError(f"one Target replica needs about {need['estimated_total'] / 2**30:.0f} GiB per GPU with "
                             f"inference.target.tp_size={tp}, more than a GPU's 180 GB: raise inference.target.tp_size")
    if int(g("target_pp_size", 1) or 1) != 1:
        raise ValueError("inference.target.pp_size must be 1: the in-framework Target shards by tensor parallelism only")
    if g("eval_data_path") and int(g("eval_interval") or 0) <= 0:
        notes.append("dataset.eval_data_path is set but eval_interval is 0: evaluation never runs")
    if int(g("micro_batch_size", 1)) < 1 or int(g("draft_accumulation_steps", 1)) < 1:
        raise ValueError("micro_batch_size and draft_accumulation_steps must be positive")
    # -- sequence / context parallel schemes ---------------------------------------------------------------
    u, r = int(g("sp_ulysses_size", 1) or 1), int(g("sp_ring_size", 1) or 1)
    cp = int(g("draft_context_parallel_size", 1) or 1)
    eagle = algorithm in ("eagle3", "eagle4")
    if u * r > 1:
        if eagle:
            heads, kv = int(draft["num_attention_heads"]), int(draft["num_key_value_heads"])
            if heads % u or kv % u:
                raise ValueError(f"sp_ulysses_size ({u}) must divide the attention head counts ({heads}, {kv})")
        elif algorithm == "mtp":
            raise ValueError("native-MTP training is not sharded over sequences: set sp_ulysses_size = sp_ring_size = 1")
        else:
            notes.append(f"block-drafting algorithms shard the context by ownership (direct context parallelism): "
                         f"sp_ulysses_size x sp_ring_size = {u * r} is taken as draft_context_parallel_size")
    if cp > 1 and not eagle:
        kinds = set(policy.get("layer_types") or [])
        unsupported = kinds - {"full_attention", "sliding_attention", "deepseek_sparse_attention"}
        if unsupported:
            raise ValueError(f"context parallelism covers dense, sliding-window and DSA layers, not {sorted(unsupported)}")
        if "deepseek_sparse_attention" in kinds and draft.get("dsa_training_stage") == "indexer_warmup":
            raise ValueError("the DSA indexer warm-up stage runs with draft_context_parallel_size=1")
    if draft.get("mtp_conditioning") and cp != 1:
        raise ValueError("MTP conditioning requires draft_context_parallel_size=1")
    # -- head shapes the attention kernels cover ---------------------------------------------------------------
    max_pos = draft.get("max_position_embeddings")
    if max_pos and int(flat["max_seq_length"]) > int(max_pos) and not (draft.get("rope_scaling") or draft.get("rope_parameters")):
        notes.append(f"max_seq_length {flat['max_seq_length']} exceeds the Draft's max_position_embeddings {max_pos} "
                     "without a RoPE scaling rule")
    # -- train with decode: the Target engines write the responses themselves ------------------------------------
    if g("train_with_decode"):
        if engine != "native":
            raise ValueError("training.train_with_decode needs the in-framework Target (inference_engine_type=native): stored or "
                             "synthetic features cannot be continued")
        if int(g("decode_max_new_tokens", 512)) < max(int(g("decode_min_new_tokens", 2)), 1):
            raise ValueError("decode.max_new_tokens must be at least decode.min_new_tokens and positive")
        if float(g("decode_temperature", 1.0)) < 0 or not 0.0 < float(g("decode_top_p", 1.0)) <= 1.0:
            raise ValueError("decode.temperature must not be negative and decode.top_p must lie in (0, 1]")
        speculative = g("decode_weight_sync_enabled") or g("decode_speculative_draft_model_path")
        if speculative and (algorithm not in ("dspark", "dflash") or draft.get("mtp_conditioning")):
            raise ValueError("a decoding Target proposes with DSpark / DFlash block Drafts only (no MTP conditioning): "
                             "turn decode.weight_sync_enabled and decode.speculative_draft_model_path off to decode with the "
                             "Target alone")
        if g("decode_weight_sync_enabled") and int(g("decode_weight_sync_interval", 500) or 0) < 1:
            raise ValueError("decode.weight_sync_interval must be positive")
        if g("experiments"):
            raise ValueError("training.train_with_decode is a single-Draft mode: a shared-Target run prefills recorded responses")
        notes.append("train_with_decode: documents give the prompt (everything before their last supervised span); responses "
                     f"of up to {int(g('decode_max_new_tokens', 512))} tokens are drawn from the Target and supervised whole")
    # -- keys that would change what is trained and have no implementation (the reference refuses these too) -----
    if int(g("eagle3_num_anchors") or 0):
        raise ValueError("anchored EAGLE3 (training.eagle3_num_anchors) is not part of the training path: EAGLE3 / EAGLE4 "
                         "train on every supervised position")
    if g("compile_model"):
        notes.append("training.compile_model has no effect: there is no tracing compiler on this path")
    # -- schedule ---------------------------------------------------------------------------------------------
    steps = g("num_train_steps")
    if steps is not None and int(steps) < 0:
        raise ValueError("training.num_train_steps must not be negative")
    warm, drain = int(g("performance_warmup_steps") or 0), int(g("performance_drain_steps") or 0)
    if g("performance_measurement_required") and steps and int(steps) <= warm + drain:
        notes.append(f"debug.performance_measurement_required needs more than {warm + drain} optimizer steps "
                     f"(performance_warmup_steps + performance_drain_steps), the run has {steps}: it will end without a "
                     "valid steady window and fail after writing its evidence")
    save, keep = int(g("save_interval") or 0), g("max_checkpoints")
    if keep is not None and int(keep) < 0:
        raise ValueError("training.max_checkpoints must not be negative")
    if g("continual_training") and not g("load_path"):
        notes.append("training.continual_training is set without training.load_path: the run starts from random weights "
                     "unless --load-path is given on the command line")
    if save and steps and int(steps) and save > int(steps) and g("save_final_checkpoint") is False:
        notes.append(f"save_interval {save} is larger than the run ({steps} steps) and the final checkpoint is off: "
                     "nothing will be saved")
    return notes


def compile_execution_plan(config: Config) -> ExecutionPlan:
    flat = vars(config_to_flat_args(config)).copy()
    draft = _load_draft(flat)
    algorithm = resolve_draft_algorithm(draft)
    world = int(flat["world_size"])
    cp = int(flat["draft_context_parallel_size"])
    u, r = int(flat["sp_ulysses_size"]), int(flat["sp_ring_size"])
    if u * r > 1 and cp == 1:
        cp = u * r
        flat["draft_context_parallel_size"] = cp
    ep, vp = int(flat["expert_parallel_size"]), int(flat["vocab_parallel_size"])
    if world % cp:
        raise ValueError(f"world size {world} is not divisible by context parallel size {cp}")
    dp = world // cp
    caps: List[CapabilityDecision] = []
    policy = resolve_attention_policy(draft) if algorithm != "mtp" else {"layer_types": ["full_attention"]}
    ffn = resolve_ffn_policy(draft) if algorithm != "mtp" else {"ffn_type": "dense"}
    # ---- scope validation ----------------------------------------------------------------------
    if flat["dflash_packing"] and algorithm not in ("dflash", "dspark", "dflash2", "eagle3", "eagle4", "mtp"):
        raise ValueError("packing is not defined for this algorithm")
    if algorithm in ("dflash", "dspark", "dflash2"):
        n_anchor = int(flat["dspark_num_anchors"] if algorithm == "dspark" else flat["dflash_num_anchors"])
        if cp > 1 and n_anchor % cp:
            raise ValueError(f"num_anchors ({n_anchor}) must be divisible by the context-parallel size ({cp})")
        want_layers = int(flat["dspark_num_target_layers"] if algorithm == "dspark" else flat["dflash_num_target_layers"])
        if draft.get("num_target_layers") not in (None, want_layers) and flat.get("strict_target_layers", False):
            raise ValueError("training.*_num_target_layers disagrees with the draft config")
    if draft.get("mtp_conditioning") and (cp != 1 or flat["anchor_sampling_scope"] != "row"):
        raise ValueError("MTP conditioning currently requires CP1 row anchors")
    if ffn["ffn_type"] == "dense" and ep > 1:
        raise ValueError("expert_parallel_size > 1 requires a MoE draft")
    if ep > 1 and ffn.get("num_experts", 0) % ep:
        raise ValueError("num_experts must be divisible by expert_parallel_size")
    if ep > 1 and str(flat["fsdp_strategy"]).upper() == "FULL_SHARD":
        raise ValueError("expert parallelism shards the experts itself: use training.fsdp_strategy=REPLICATE with it")
    if vp > 1 and draft["vocab_size"] % vp:
        raise ValueError("vocab_size must be divisible by vocab_parallel_size")
    if ep > 1 and world % ep or vp > 1 and world % vp:
        raise ValueError("expert / vocab parallel sizes must divide the Draft world size")
    align = context_shard_alignment(policy) if algorithm != "mtp" else 1
    if cp > 1 and int(flat["max_seq_length"]) // max(align, 1) < cp:
        raise ValueError("sequence too short to give every context-parallel rank an aligned shard")
    for note in validate_scope(flat, draft, algorithm, policy, ffn):
        caps.append(CapabilityDecision("scope", "note", note))
    # ---- capability decisions ------------------------------------------------------------------
    head_dim = draft.get("head_dim") or draft["hidden_size"] // draft["num_attention_heads"]
    mla = draft.get("attention_mode") == "mla" or draft.get("model_type") in ("k3_dspark", "deepseek_v3")
    caps.append(CapabilityDecision("gemm", "tcgen05_tma_persistent", "bf16 weights, sm_100a"))
    if mla:
        qk_dim = int(draft.get("qk_nope_head_dim") or 0) + int(draft.get("qk_rope_head_dim") or 0)
        v_dim = int(draft.get("v_head_dim") or 0)
    else:
        qk_dim = v_dim = int(head_dim)
    kernel_heads = v_dim == 128 and qk_dim in (128, 192)
    caps.append(CapabilityDecision(
        "attention", "tcgen05_interval_flash" if kernel_heads else "dense_mask_fp32",
        f"query/key head dim {qk_dim}, value head dim {v_dim}: the TMEM flash kernels cover (128, 128) and the "
        f"materialised-MLA shape (192, 128)" if kernel_heads else
        f"head dims ({qk_dim}, {v_dim}) have no kernel: fp32 dense-mask statement, refused above a bounded score size"))
    caps.append(CapabilityDecision("vocab_head", "fused_rowstats_gemm+streaming_loss", "logits stay bf16; no fp32 [rows, V]"))
    # a trainer holds the slots of all micro-batches of an update until its optimizer step commits, and the next
    # update's rows are dispatched meanwhile: fewer slots than that deadlock the producer against the consumer
    ahead = max(int(flat.get("dispatch_ahead_updates", 1) or 1), 1)
    need_slots = int(flat["draft_accumulation_steps"]) * int(flat["micro_batch_size"]) * (1 if ahead == 1 else ahead) + 1
    if int(flat.get("transport_destination_ring_slots", 1) or 1) < need_slots:
        caps.append(CapabilityDecision("feature_ring", f"destination_ring_slots raised to {need_slots}",
                                       f"configured {flat.get('transport_destination_ring_slots')}: one update keeps "
                                       f"{need_slots - 1} slots leased until its optimizer step commits"))
        flat["transport_destination_ring_slots"] = need_slots
    caps.append(CapabilityDecision("feature_transport", flat["transport_data_plane"],
                                   "Target epilogues store into the Draft ranks' ring slots over NVLink"))
    caps.append(CapabilityDecision("data_parallel", flat["fsdp_strategy"], {
        "REPLICATE": "whole replicas; flat fp32 gradient buffer, one SUM reduction per update",
        "SHARD_OPTIMIZER": "whole bf16 replicas and gradient buffers; fp32 masters and moments sharded; reduce + AdamW + "
                           "parameter scatter over peer memory once per update",
        "FULL_SHARD": "parameters, gradients, masters and moments sharded per decoder layer; layers gathered by peer loads one "
                      "ahead of compute; each layer's gradient reduce-scattered under the backward of the layers below",
    }[str(flat["fsdp_strategy"]).upper()]))
    if cp > 1:
        caps.append(CapabilityDecision("context_parallel", f"ulysses{u}xring{r}" if u * r > 1 else f"direct_cp{cp}",
                                       f"context sharded contiguously per document, alignment {align}"))
    if ep > 1:
        caps.append(CapabilityDecision("expert_parallel", f"ep{ep}",
                                       "each rank of a group keeps E / ep experts of every MoE layer; dispatch / combine run "
                                       "inside the grouped expert GEMMs over peer memory; expert gradients are reduced over "
                                       "replicas only; checkpoints hold whole banks"))
    if vp > 1:
        caps.append(CapabilityDecision("vocab_parallel", f"vp{vp}", "head rows sharded; log-sum-exp merged over peer memory"))
    thd = thd_contract(policy) if algorithm != "mtp" else {}
    workload = {"algorithm": algorithm, "draft_model_semantics": draft_model_semantics(draft),
                "attention_policy": {k: policy.get(k) for k in ("layer_types", "window_semantics", "draft_block_attention")},
                "ffn_policy": ffn, "thd_contract": thd, "max_seq_length": flat["max_seq_length"],
                "packing": bool(flat["dflash_packing"]), "dataset": flat.get("train_data_path"),
                "target": flat.get("target_model_path") or flat.get("target_model_config") or "shape-bound random init",
                "engine": flat["inference_engine_type"], "context_shard_alignment": align}
    pol = {"world_size": world, "target_gpus": int(flat["inference_num_gpus"]) if flat["inference_engine_type"] == "native" else 0,
           "draft_gpus": world, "context_parallel": cp, "ulysses": u, "ring": r, "expert_parallel": ep,
           "vocab_parallel": vp, "fsdp_strategy": flat["fsdp_strategy"], "colocate": bool(flat.get("colocate")), **resolve_batch_size(flat, dp),
           "num_train_steps": flat.get("num_train_steps"), "seed": flat["seed"]}
    memory = estimate_memory(draft, flat, algorithm, dp, flat["fsdp_strategy"])
    if not memory["fits"]:
        raise ValueError(f"estimated {memory['estimated_total'] / 2**30:.1f} GiB per Draft GPU exceeds 180 GB HBM3e; "
                         "use FULL_SHARD, fewer anchors or a smaller ring")
    flat["draft_algorithm"] = algorithm
    return ExecutionPlan(workload, pol, caps, draft, flat, memory)
