"""Run configuration: typed schema + YAML + ``section.key=value`` overrides -> validated ``Config``.

Sections and field names are those of the reference's recipes (aspec/config/train_config.py:42-300):
``model dataset training inference transport|mooncake logging debug decode cluster experiments[]
output_dir cache_dir``.  Loading = schema defaults (+) optional base file (+) YAML (+) dotlist, with
``${oc.env:VAR,default}`` interpolation resolved once, in the submitting process; unknown keys are
errors (fail closed).  ``config_to_flat_args`` flattens to the namespace the runtime consumes, with the
same section prefixes (``cluster_ decode_ transport_ offline_ target_``) and derived fields
(``world_size checkpoint_dir dynamic_loss_mask``).

Differences that follow from the B200-native design: the Target runs in-framework
(``inference.inference_engine_type: native | offline | synthetic``) and features move through
symmetric-memory rings (``transport`` section; a ``mooncake`` section in an old recipe is accepted and
mapped), and there are ``training.expert_parallel_size`` / ``training.vocab_parallel_size``.
"""
from __future__ import annotations

import argparse
import copy
import dataclasses
import os
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import yaml


@dataclass
class DatasetConfig:
    chat_template: Optional[str] = "llama3"
    defer_tokenization: bool = False
    eval_data_path: Optional[str] = None
    eval_interval: int = 50
    eval_cache_idle_timeout_seconds: float = 300.0
    eval_decode_anchors_per_doc: int = 0          # > 0: block proposals of the live Draft on the held-out rows (tau) at every evaluation
    eval_num_documents: int = 32                  # rows of the synthetic held-out split
    eval_micro_batch_size: Optional[int] = None
    eval_prompt_key: Optional[str] = None
    last_turn_loss_only: Any = "auto"
    tokenizer_path: Optional[str] = None          # directory of a Hugging Face tokenizer; default: model.target_model_path
    length_group_size: int = 32
    min_loss_tokens: int = 0
    prompt_key: str = "conversations"
    renderer: Optional[str] = None
    shuffle_dataset: bool = True
    dataset_seed: Optional[int] = None
    train_data_path: Optional[str] = ""
    # synthetic source (train_data_path: "synthetic")
    synthetic_num_documents: int = 4096
    synthetic_vocab_size: Optional[int] = None      # default: the draft's vocabulary minus its reserved tail
    synthetic_min_length: int = 256
    synthetic_max_length: int = 4096
    synthetic_length_distribution: str = "log_uniform"
    synthetic_loss_tail_fraction: float = 0.6


@dataclass
class DebugConfig:
    enable_perf_metrics: bool = True
    max_dump_steps: int = 5
    memory_recorder: str = "torch"
    memory_snapshot_dir: str = "."
    memory_snapshot_num_steps: Optional[int] = None
    memory_snapshot_path: str = ""
    profile_dir_name: Optional[str] = "/tmp/aspec_profiles"
    profile_step_end: int = 0
    profile_step_start: int = 0
    profile_target: list = field(default_factory=lambda: ["train_overall"])
    performance_drain_steps: int = 0
    performance_measurement_required: bool = False
    performance_warmup_steps: int = 0
    topology_producer_profile_samples: int = 0
    topology_producer_profile_warmup_samples: int = 0
    record_memory_history: bool = False
    save_debug_train_data: Optional[str] = None
    timeline_enabled: bool = False
    timeline_flush_every: int = 128
    timeline_output_dir: str = ""
    timeline_run_id: str = ""
    use_pytorch_profiler: bool = False
    # host-side fault injection for validation runs (never on by default; nothing here touches a GPU):
    # {"kind": "raise" | "sleep", "step": k, "rank": r, "seconds": s} makes trainer r raise / stall at update k
    fault_injection: Optional[dict] = None
    producer_fail_after: Optional[int] = None      # the Target engine raises after this many rows
    producer_delay_seconds: float = 0.0            # synthetic engine: sleep per row (a slow producer)


@dataclass
class LoggingConfig:
    report_to: str = "none"
    use_tensorboard: bool = False
    use_wandb: bool = False
    wandb_dir: Optional[str] = None
    wandb_group: Optional[str] = None
    wandb_host: Optional[str] = None
    wandb_key: Optional[str] = None
    wandb_mode: Optional[str] = None
    wandb_project: Optional[str] = None
    wandb_random_suffix: bool = True
    wandb_run_id: Optional[str] = None
    wandb_team: Optional[str] = None


@dataclass
class ClusterConfig:
    mode: str = "single_node"
    nodes: Optional[List[dict]] = None          # [{name, gpus}]: the machines of a static cluster; default: this machine
    node_name: Optional[str] = None             # which entry of ``nodes`` this process runs on
    shared_root: Optional[str] = None
    storage_mode: str = "shared"
    file_transfer_timeout_seconds: float = 600.0
    require_homogeneous_gpus: bool = True
    preflight_timeout_seconds: float = 120.0


@dataclass
class ModelConfig:
    draft_model_config: Optional[str] = None
    initial_draft_model_path: Optional[str] = None
    native_context_length: Optional[int] = None
    keep_initial_vocab_mapping: bool = False
    embedding_key: str = "model.embed_tokens.weight"
    freeze_lm_head: bool = False
    lm_head_key: str = "lm_head.weight"
    norm_key: str = "model.norm.weight"
    target_model_backend: str = "native"
    target_model_path: str = ""
    target_model_config: Optional[str] = None      # JSON of a Target architecture for random-init runs
    # fields laid over the Draft configuration file (``model.draft_overrides.dsa_training_stage=sparse``): a training
    # stage or a budget can change between phases without a second JSON file
    draft_overrides: Dict[str, Any] = field(default_factory=dict)
    mtp_source_path: Optional[str] = None          # checkpoint directory with the native ``mtp.*`` tensors (default: target_model_path)
    trust_remote_code: bool = False


@dataclass
class TrainingConfig:
    attention_backend: str = "sm100_flash"
    draft_context_parallel_size: int = 1
    colocate: bool = False
    continual_training: bool = False
    continue_source_cursor: bool = False
    distributed_backend: str = "nccl"
    distributed_timeout_minutes: int = 10
    draft_accumulation_steps: int = 1
    mtp_steps: int = 3
    mtp_step_weight_beta: float = 0.6
    eagle3_num_anchors: int = 0
    eagle3_anchor_max_gap: Optional[int] = None
    fsdp_reduce_dtype: str = "float32"
    fsdp_strategy: str = "REPLICATE"
    placement_strategy: str = "training_first"
    training_node_ips: Optional[List[str]] = None
    training_node_selectors: Optional[List[dict]] = None
    compile_model: bool = False
    sp_ring_size: int = 1
    sp_ulysses_size: int = 1
    expert_parallel_size: int = 1
    vocab_parallel_size: int = 1
    gradient_checkpointing: bool = False
    eagle3_loss_gradient_checkpointing: Optional[bool] = None
    learning_rate: float = 1e-4
    lk_eta: float = 3.0
    load_path: Optional[str] = None
    loss_type: str = "forward_kl"
    eagle3_target_cache: str = "lazy"
    lr_decay_style: str = "cosine"
    lr_wsd_decay_ratio: float = 0.2
    lr_wsd_decay_style: str = "cosine"
    lr_total_steps: Optional[int] = None
    max_concurrent_batches: int = 1
    max_grad_norm: float = 0.5
    max_seq_length: int = 8192
    min_lr: float = 0.0
    weight_decay: float = 0.0
    num_epochs: int = 10
    num_train_steps: Optional[int] = None
    source_work_budget: Optional[int] = None
    micro_batch_size: int = 2
    optimizer_step_timeout_seconds: float = 1800.0
    streaming_dispatch_with_training: bool = False
    pipeline_dispatch_with_training: bool = False
    prefetch_depth: int = 2
    dispatch_ahead_updates: int = 1      # updates whose rows are at the Target engines beyond the one in training
    save_interval: int = 5000
    save_per_epoch: bool = False
    save_final_checkpoint: bool = True
    max_checkpoints: int = 0
    seed: int = 0
    deterministic_anchor_sampling: bool = False
    anchor_sampling_scope: str = "row"
    train_backend: str = "fsdp"
    train_env_vars: str = "{}"
    train_with_decode: bool = False
    training_num_gpus_per_node: int = 1
    training_num_nodes: int = 1
    ttt_length: int = 7
    ploss_weights: Optional[List[float]] = None
    warmup_ratio: float = 0.015
    wsd_decay_ratio: Optional[float] = None
    wsd_decay_style: Optional[str] = None
    dflash_block_size: int = 16
    dflash_dpace_alpha: float = 0.5
    dflash_loss_decay_gamma: float = 7.0
    dflash_loss_objective: str = "decay"
    dflash_ce_loss_alpha: float = 1.0
    dflash_l1_loss_alpha: float = 0.0
    dflash_num_anchors: int = 512
    dflash_num_target_layers: int = 5
    dflash_packing: bool = False
    packing_min_samples_per_dispatch: int = 0
    dflash2_selector_loss_alpha: float = 1.0
    dspark_block_size: int = 7
    dspark_num_anchors: int = 512
    dspark_num_target_layers: int = 5
    dspark_loss_decay_gamma: float = 4.0
    dspark_ce_loss_alpha: float = 0.1
    dspark_l1_loss_alpha: float = 0.9
    dspark_l1_target_temperature: float = 1.0
    dspark_l1_target_top_p: float = 1.0
    dspark_l1_target_top_k: int = -1
    dspark_l1_draft_temperature: float = 1.0
    dspark_l1_draft_top_p: float = 1.0
    dspark_l1_draft_top_k: int = -1
    dspark_confidence_head_alpha: float = 1.0


@dataclass
class DecodeConfig:
    cuda_graph_max_bs: Optional[int] = None
    max_new_tokens: int = 512
    min_new_tokens: int = 2
    stop_token_ids: Optional[List[int]] = None
    max_running_requests: Optional[int] = None
    speculative_algorithm: Optional[str] = None
    speculative_draft_model_path: Optional[str] = None
    speculative_eagle_topk: Optional[int] = None
    speculative_num_draft_tokens: Optional[int] = None
    speculative_num_steps: Optional[int] = None
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    weight_sync_enabled: bool = False
    weight_sync_interval: int = 500


@dataclass
class TargetEngineConfig:
    """In-framework Target prefill engine (replaces the reference's SGLang engine section)."""
    tp_size: int = 1
    pp_size: int = 1
    nnodes: int = 1
    mem_fraction_static: float = 0.8
    max_prefill_tokens: int = 16384
    init_timeout: int = 300
    extra_args: Dict[str, Any] = field(default_factory=dict)


@dataclass
class OfflineTrainingConfig:
    feature_dir: Optional[str] = None
    require_complete: bool = True
    replay_workers: int = 1


@dataclass
class InferenceConfig:
    inference_engine_type: str = "native"     # native | offline | synthetic
    inference_num_gpus: int = 1
    inference_num_gpus_per_engine: int = 1
    inference_num_gpus_per_node: int = 8
    inference_batch_size: int = 8               # rows per Target call (upper bound when inference_batch_tokens is set)
    inference_batch_tokens: int = 0             # > 0: send a batch once it holds this many tokens
    inference_buffer_threshold: int = 32
    inference_node_ips: Optional[List[str]] = None
    max_sample_pool_size: int = 64
    store_last_hidden_states: bool = True
    last_hidden_states_prenorm: Optional[bool] = None
    aux_hidden_states_layers: Optional[List[int]] = None
    target: TargetEngineConfig = field(default_factory=TargetEngineConfig)
    offline: OfflineTrainingConfig = field(default_factory=OfflineTrainingConfig)


@dataclass
class TransportConfig:
    """Symmetric-memory feature rings between Target and Draft ranks."""
    data_plane: str = "nvlink_p2p"            # nvlink_p2p | nvls_multicast | host_staged
    source_ring_slots: int = 16
    destination_ring_slots: int = 1
    slot_bytes: int = 512 * 1024 * 1024
    acquire_timeout_seconds: float = 120.0
    read_timeout_seconds: float = 120.0
    device_wait_limit_ms: float = 2000.0
    release_history_per_slot: int = 32


@dataclass
class Config:
    experiments: List[Dict[str, Any]] = field(default_factory=list)
    cluster: ClusterConfig = field(default_factory=ClusterConfig)
    dataset: DatasetConfig = field(default_factory=DatasetConfig)
    debug: DebugConfig = field(default_factory=DebugConfig)
    decode: DecodeConfig = field(default_factory=DecodeConfig)
    inference: InferenceConfig = field(default_factory=InferenceConfig)
    logging: LoggingConfig = field(default_factory=LoggingConfig)
    model: ModelConfig = field(default_factory=ModelConfig)
    transport: TransportConfig = field(default_factory=TransportConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    cache_dir: str = "./cache"
    cache_key: Optional[str] = None
    model_download_dir: Optional[str] = None
    output_dir: str = ""

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)


# ------------------------------------------------------------------ loading -------------------
_ENV = re.compile(r"\$\{oc\.env:([A-Za-z_][A-Za-z0-9_]*)(?:,([^}]*))?\}")
_PATH_KEYS = {("model", "draft_model_config"), ("model", "target_model_config"), ("dataset", "train_data_path"), ("dataset", "tokenizer_path"), ("model", "mtp_source_path"),
              ("dataset", "eval_data_path"), ("training", "load_path"), ("model", "initial_draft_model_path")}
# `mooncake:` keys of reference recipes that have a transport meaning here
_MOONCAKE_ALIASES = {"p2p_source_slots": "source_ring_slots", "p2p_destination_slots": "destination_ring_slots",
                     "p2p_slot_size": "slot_bytes", "source_ring_slots": "source_ring_slots",
                     "destination_ring_slots": "destination_ring_slots", "slot_bytes": "slot_bytes"}


def _interpolate(value):
    if isinstance(value, str):
        def sub(m):
            env = os.environ.get(m.group(1))
            if env is not None:
                return env
            if m.group(2) is None:
                raise ValueError(f"environment variable {m.group(1)} is not set and has no default")
            return m.group(2)
        new = _ENV.sub(sub, value)
        if new != value and _ENV.fullmatch(value):
            return yaml.safe_load(new) if new != "" else new
        return new
    if isinstance(value, dict):
        return {k: _interpolate(v) for k, v in value.items()}
    if isinstance(value, list):
        return [_interpolate(v) for v in value]
    return value


def _apply(obj, data: dict, path: str) -> None:
    names = {f.name: f for f in dataclasses.fields(obj)}
    for key, value in data.items():
        if key not in names:
            raise ValueError(f"Unknown config key '{path}{key}'")
        current = getattr(obj, key)
        if dataclasses.is_dataclass(current):
            if not isinstance(value, dict):
                raise ValueError(f"Config section '{path}{key}' must be a mapping")
            _apply(current, value, f"{path}{key}.")
        else:
            setattr(obj, key, _coerce(copy.deepcopy(value), names[key], f"{path}{key}"))


def _coerce(value, fld, where):
    """YAML 1.1 reads ``6e-4`` as a string; numbers for numeric fields are accepted in that form."""
    kind = str(fld.type)
    if isinstance(value, str) and ("float" in kind or "int" in kind) and "str" not in kind and "Any" not in kind:
        try:
            number = float(value)
        except ValueError:
            raise ValueError(f"Config key '{where}' expects a number, got {value!r}") from None
        return int(number) if "float" not in kind and number == int(number) else number
    return value


def _set_dotted(tree: dict, dotted: str, value) -> None:
    parts = dotted.split(".")
    node = tree
    for p in parts[:-1]:
        node = node.setdefault(p, {})
        if not isinstance(node, dict):
            raise ValueError(f"Override '{dotted}' descends into a non-mapping")
    node[parts[-1]] = value


def parse_dotlist(items) -> dict:
    tree: dict = {}
    for item in items or []:
        if "=" not in item:
            raise ValueError(f"Override '{item}' is not of the form section.key=value")
        key, raw = item.split("=", 1)
        _set_dotted(tree, key.strip(), yaml.safe_load(raw) if raw != "" else "")
    return tree


def _merge(base: dict, extra: dict) -> dict:
    out = copy.deepcopy(base)
    for k, v in extra.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = _merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


def _resolve_paths(tree: dict, base_dir: Path) -> None:
    for section, key in _PATH_KEYS:
        value = tree.get(section, {}).get(key) if isinstance(tree.get(section), dict) else None
        if isinstance(value, str) and value and value != "synthetic" and not os.path.isabs(value) \
                and not value.startswith(("hf://", "s3://")):
            cand = (base_dir / value)
            if cand.exists():
                tree[section][key] = str(cand.resolve())


def load_config(path: Optional[str] = None, cli_args=None, base_path: Optional[str] = None) -> Config:
    tree: dict = {}
    for p in (base_path, path):
        if p:
            with open(p) as f:
                data = yaml.safe_load(f) or {}
            if not isinstance(data, dict):
                raise ValueError(f"{p} must contain a mapping")
            _resolve_paths(data, Path(p).resolve().parent)
            tree = _merge(tree, data)
    tree = _merge(tree, parse_dotlist(cli_args))
    tree = _interpolate(tree)
    if "mooncake" in tree:
        legacy = tree.pop("mooncake") or {}
        transport = tree.setdefault("transport", {})
        for k, v in legacy.items():
            if k in _MOONCAKE_ALIASES:
                transport.setdefault(_MOONCAKE_ALIASES[k], v)
    if isinstance(tree.get("inference"), dict) and "sglang" in tree["inference"]:
        legacy = tree["inference"].pop("sglang") or {}
        tgt = tree["inference"].setdefault("target", {})
        for k in ("tp_size", "pp_size", "nnodes", "mem_fraction_static", "init_timeout", "extra_args"):
            if k in legacy:
                tgt.setdefault(k, legacy[k])
    if isinstance(tree.get("inference"), dict) and tree["inference"].get("inference_engine_type") == "sgl":
        tree["inference"]["inference_engine_type"] = "native"
    config = Config()
    _apply(config, tree, "")
    validate_config(config)
    return config


# ---------------------------------------------------------------- validation ------------------
def _positive(value, name):
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ValueError(f"{name} must be a positive integer")


def validate_config(c: Config) -> None:
    t, inf, tr = c.training, c.inference, c.transport
    if inf.inference_engine_type not in ("native", "offline", "synthetic"):
        raise ValueError("inference.inference_engine_type must be native, offline or synthetic "
                         f"(got {inf.inference_engine_type!r})")
    if c.cluster.mode not in ("single_node", "static_multi_node"):
        raise ValueError("cluster.mode must be single_node or static_multi_node")
    if c.cluster.mode == "static_multi_node":
        if c.cluster.storage_mode not in ("shared", "node_local"):
            raise ValueError("cluster.storage_mode must be shared or node_local")
        if c.cluster.storage_mode == "shared" and not c.cluster.shared_root:
            raise ValueError("static_multi_node with shared storage requires cluster.shared_root")
        if not t.training_node_ips or len(t.training_node_ips) != t.training_num_nodes:
            raise ValueError("static_multi_node requires one training_node_ips entry per training node")
    elif t.training_num_nodes != 1:
        raise ValueError("single_node cluster mode requires training.training_num_nodes=1")
    if inf.inference_engine_type == "offline" and not inf.offline.feature_dir:
        raise ValueError("offline training requires inference.offline.feature_dir")
    for name in ("micro_batch_size", "draft_accumulation_steps", "max_seq_length", "training_num_gpus_per_node",
                 "training_num_nodes", "draft_context_parallel_size", "sp_ring_size", "sp_ulysses_size",
                 "expert_parallel_size", "vocab_parallel_size"):
        _positive(getattr(t, name), f"training.{name}")
    if t.num_train_steps is not None:
        _positive(t.num_train_steps, "training.num_train_steps")
    for name, lo in (("learning_rate", 0.0), ("min_lr", 0.0), ("weight_decay", 0.0), ("max_grad_norm", 0.0),
                     ("warmup_ratio", 0.0), ("optimizer_step_timeout_seconds", 0.0)):
        v = getattr(t, name)
        if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v or v < lo:
            raise ValueError(f"training.{name} must be a finite number >= {lo}")
    if t.min_lr > t.learning_rate:
        raise ValueError("training.min_lr must not exceed training.learning_rate")
    if not 0.0 <= t.warmup_ratio < 1.0:
        raise ValueError("training.warmup_ratio must be in [0, 1)")
    if t.fsdp_strategy not in ("REPLICATE", "SHARD_OPTIMIZER", "FULL_SHARD"):
        raise ValueError("training.fsdp_strategy must be REPLICATE, SHARD_OPTIMIZER or FULL_SHARD")
    if t.fsdp_reduce_dtype not in ("float32", "bfloat16"):
        raise ValueError("training.fsdp_reduce_dtype must be float32 or bfloat16")
    if t.lr_decay_style not in ("constant", "linear", "cosine", "inverse-square-root", "WSD"):
        raise ValueError(f"Unknown training.lr_decay_style {t.lr_decay_style!r}")
    if t.loss_type not in ("forward_kl", "lk_alpha", "lk_lambda"):
        raise ValueError("training.loss_type must be forward_kl, lk_alpha or lk_lambda")
    if t.anchor_sampling_scope not in ("row", "sample"):
        raise ValueError("training.anchor_sampling_scope must be row or sample")
    if t.dflash_loss_objective not in ("decay", "dpace"):
        raise ValueError("training.dflash_loss_objective must be decay or dpace")
    world = t.training_num_nodes * t.training_num_gpus_per_node
    cp = t.draft_context_parallel_size
    usp = t.sp_ring_size * t.sp_ulysses_size
    if cp > 1 and usp > 1 and cp != usp:
        raise ValueError("draft_context_parallel_size must equal sp_ulysses_size * sp_ring_size when both are set")
    sp = max(cp, usp)
    if world % sp:
        raise ValueError(f"training world size {world} is not divisible by the context-parallel degree {sp}")
    if t.dflash_packing and t.micro_batch_size != 1:
        raise ValueError("training.dflash_packing packs documents into one THD row: micro_batch_size must be 1")
    if t.continue_source_cursor and not (t.continual_training and t.load_path):
        raise ValueError("training.continue_source_cursor requires continual_training=true and training.load_path")
    for name in ("source_ring_slots", "destination_ring_slots", "slot_bytes"):
        _positive(getattr(tr, name), f"transport.{name}")
    if tr.data_plane not in ("nvlink_p2p", "nvls_multicast", "host_staged"):
        raise ValueError("transport.data_plane must be nvlink_p2p, nvls_multicast or host_staged")
    # ring capacity: one in-flight sample per slot; the ready pool plus one engine batch must fit
    if inf.inference_engine_type == "native":
        need = min(inf.max_sample_pool_size, tr.source_ring_slots * max(inf.inference_num_gpus // max(inf.inference_num_gpus_per_engine, 1), 1))
        if need < t.micro_batch_size:
            raise ValueError("transport.source_ring_slots cannot hold one micro-batch of samples")
    if c.experiments:
        names = [e.get("name") for e in c.experiments]
        if any(not isinstance(n, str) or not n for n in names) or len(set(names)) != len(names):
            raise ValueError("experiments[] entries need unique non-empty names")


# ---------------------------------------------------------------- flattening ------------------
_PREFIXED = {"cluster": "cluster_", "decode": "decode_", "transport": "transport_", "offline": "offline_",
             "target": "target_"}


def config_to_flat_args(config: Config) -> argparse.Namespace:
    flat: Dict[str, Any] = {}

    def add(key, val, origin):
        if key in flat:
            raise ValueError(f"Duplicate config key '{key}' (from '{origin}')")
        flat[key] = copy.deepcopy(val)

    for f in dataclasses.fields(config):
        section = getattr(config, f.name)
        if not dataclasses.is_dataclass(section):
            add(f.name, section, f.name)
            continue
        prefix = _PREFIXED.get(f.name, "")
        for g in dataclasses.fields(section):
            val = getattr(section, g.name)
            if dataclasses.is_dataclass(val) and g.name in _PREFIXED:
                for h in dataclasses.fields(val):
                    add(f"{_PREFIXED[g.name]}{h.name}", getattr(val, h.name), f"{f.name}.{g.name}.{h.name}")
            else:
                add(f"{prefix}{g.name}", val, f"{f.name}.{g.name}")
    for key in ("wsd_decay_ratio", "wsd_decay_style"):
        flat[key] = flat[key] if flat.get(key) is not None else flat[f"lr_{key}"]
    flat["world_size"] = flat["training_num_nodes"] * flat["training_num_gpus_per_node"]
    flat["rank"] = 0
    if flat["inference_engine_type"] in ("offline", "synthetic"):
        flat["defer_tokenization"] = False
    flat["dynamic_loss_mask"] = (flat["inference_engine_type"] == "native"
                                 and (flat["defer_tokenization"] or bool(flat.get("renderer")))
                                 and not flat["train_with_decode"])
    flat["use_wandb"] = flat.get("use_wandb", False) or flat.get("report_to") == "wandb"
    flat["use_tensorboard"] = flat.get("use_tensorboard", False) or flat.get("report_to") == "tensorboard"
    flat["checkpoint_dir"] = str(Path(flat["output_dir"]) / "checkpoints") if flat.get("output_dir") else None
    if flat.get("last_hidden_states_prenorm") is None:
        flat["last_hidden_states_prenorm"] = False
    return argparse.Namespace(**flat)


def save_config(config: Config, path: str) -> None:
    with open(path, "w") as f:
        yaml.safe_dump(config.to_dict(), f, sort_keys=True)
