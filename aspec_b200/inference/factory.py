"""Creates the engine actors for the configured backend and returns the frozen Target tensors the
trainers borrow (output head, embedding).  (reference: aspec/inference/factory.py:44-722)"""
from __future__ import annotations

import json
from typing import Dict, List


from aspec_b200.runtime.actor import ProcessActor


def target_config_from_args(flat: Dict, draft_config: dict) -> dict:
    path = flat.get("target_model_config")
    if path:
        raw = json.load(open(path)) if isinstance(path, str) else dict(path)
        return raw.get("text_config", raw)
    # default: a Target shaped like the Draft's binding
    return {"hidden_size": draft_config.get("target_hidden_size", draft_config["hidden_size"]),
            "intermediate_size": draft_config.get("intermediate_size", 4 * draft_config["hidden_size"]),
            "num_hidden_layers": draft_config.get("target_num_hidden_layers", 36),
            "num_attention_heads": draft_config["num_attention_heads"],
            "num_key_value_heads": draft_config["num_key_value_heads"], "head_dim": draft_config.get("head_dim"),
            "vocab_size": draft_config["vocab_size"], "rms_norm_eps": draft_config.get("rms_norm_eps", 1e-6),
            "rope_theta": draft_config.get("rope_theta", 1e6)}


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def create_engines(flat: Dict, draft_config: dict, layer_ids: List[int], target_devices: List[str],
                   ring_handles: Dict[int, dict]):
    kind = flat["inference_engine_type"]
    hidden = int(draft_config.get("target_hidden_size", draft_config["hidden_size"]))
    fault = flat.get("producer_fail_after")
    if kind == "native":
        from aspec_b200.inference.engine import NativeTargetEngine
        tcfg = target_config_from_args(flat, draft_config)
        tp = max(int(flat.get("target_tp_size", 1) or 1), 1)
        if len(target_devices) % tp:
            raise ValueError(f"{len(target_devices)} Target GPUs cannot form engines of target_tp_size={tp}")

        def rank_actor(i, dev, tp_rank=0, address=None):
            label = f"target{i}" if tp == 1 else f"target{i}.{tp_rank}"
            return ProcessActor(NativeTargetEngine, tcfg, layer_ids, dev, "bfloat16" if dev.startswith("cuda") else "float32",
                                int(flat.get("seed", 0)), f"target{i}", bool(flat.get("device_flags", False)),
                                flat.get("target_weights_path"), fault, float(flat.get("producer_delay_seconds", 0.0) or 0.0),
                                tp_rank, tp, address, name=label)
        if tp == 1:
            engines = [rank_actor(i, dev) for i, dev in enumerate(target_devices)]
        else:
            # one engine = ``tp`` processes, one per GPU, that meet on a port of their own and act as one actor
            from aspec_b200.runtime.actor import ActorGroup
            engines = []
            for i in range(len(target_devices) // tp):
                address = f"tcp://127.0.0.1:{_free_port()}"
                engines.append(ActorGroup([rank_actor(i, target_devices[i * tp + r], r, address) for r in range(tp)],
                                          name=f"target{i}"))
        for i, e in enumerate(engines):
            e.wait_ready()
            e.call("attach_rings", {c: hs[i] for c, hs in ring_handles.items()}, timeout=300)
        n_trainers = len(ring_handles)
        head = engines[0].call("lm_head", n_trainers, timeout=300)
        embedding = engines[0].call("embedding", n_trainers, timeout=300)
        return engines, head, embedding
    if kind == "synthetic":
        from aspec_b200.inference.engine import SyntheticEngine
        eng = SyntheticEngine(layer_ids, hidden, "cpu", seed=int(flat.get("seed", 0)),
                              delay_s=float(flat.get("producer_delay_seconds", 0.0)), fail_after=fault)
        eng.attach_rings({c: hs[0] for c, hs in ring_handles.items()})
        return [eng], None, None
    if kind == "offline":
        from aspec_b200.inference.engine import OfflineReplayEngine
        import os
        eng = OfflineReplayEngine(flat["offline_feature_dir"], require_complete=bool(flat.get("offline_require_complete", True)))
        stored = eng.store.binding["feature_contract"]
        if list(stored["aux_hidden_state_layers"]) != [int(i) for i in layer_ids] or int(stored["target_hidden_size"]) != hidden:
            raise ValueError(f"offline features hold layers {stored['aux_hidden_state_layers']} of width {stored['target_hidden_size']}; "
                             f"this Draft needs layers {list(layer_ids)} of width {hidden}")
        eng.attach_rings({c: hs[0] for c, hs in ring_handles.items()})
        head_file = os.path.join(flat["offline_feature_dir"], "lm_head.pt")      # written by prepare-target-data
        embed_file = os.path.join(flat["offline_feature_dir"], "embed_tokens.pt")
        return ([eng], ({"file": head_file} if os.path.isfile(head_file) else None),
                ({"file": embed_file} if os.path.isfile(embed_file) else None))
    raise ValueError(f"unknown inference engine type {kind!r}")
