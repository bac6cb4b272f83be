"""Target feature engines.

``InferenceEngine`` is the contract the scheduler drives (reference: aspec/inference/engine/base.py:29-91):
``init``, ``generate``, ``health_check``, ``shutdown``, ``get_status``.  Implementations:

* ``NativeTargetEngine`` - runs the in-framework Target (``models.target.dense``) prefill-only on its GPU
  and lets the captured-layer epilogues write into the consumers' ring slots (replaces the SGLang engine,
  aspec/inference/engine/sgl_engine.py:155-1062, and its direct sink, aspec/inference/target_prefill.py);
* ``SyntheticEngine`` - random features of the right shape (Draft-only runs, CPU tests);
* ``OfflineReplayEngine`` - replays materialised features from an offline store
  (aspec/inference/engine/offline_replay_engine.py:45-240).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch

from aspec_b200.transport.feature_ring import RemoteRing, RingFeatureSink, feature_bytes
from aspec_b200.utils.types import InferenceOutput, RowRequest


class InferenceEngine:
    name = "engine"

    def init(self) -> None:
        raise NotImplementedError

    def attach_rings(self, handles: Dict[int, dict]) -> None:
        if getattr(self, "tp_rank", 0) > 0:
            return                      # only the first rank of a tensor-parallel engine stores features
        self._attach(handles)

    def _attach(self, handles: Dict[int, dict]) -> None:
        """``handles[c]`` maps consumer ``c``'s ring; an optional ``"layer_ids"`` entry names the subset of this
        engine's captured layers that the consumer wants (several Drafts sharing one Target)."""
        self.rings = {int(c): RemoteRing(h) for c, h in handles.items()}
        self.consumer_layers = {int(c): tuple(h["layer_ids"]) for c, h in handles.items() if h.get("layer_ids")}

    def _layers_of(self, consumer: int):
        return getattr(self, "consumer_layers", {}).get(consumer, tuple(self.layer_ids))

    def _copy_features(self, req: RowRequest, views, hidden_states, last_hidden_states, row_slice=slice(None)) -> None:
        """Copy union-layout features ``[n, K * D]`` into every reader's slot, selecting its layer columns."""
        D = hidden_states.shape[-1] // len(self.layer_ids)
        for (consumer, _s, _g), v in zip(req.leases, views):
            layers = self._layers_of(consumer)
            src = hidden_states
            if tuple(layers) != tuple(self.layer_ids):
                cols = torch.cat([torch.arange(self.layer_ids.index(l) * D, (self.layer_ids.index(l) + 1) * D) for l in layers])
                src = hidden_states[:, cols]
            v["hidden_states"][row_slice].copy_(src.to(v["hidden_states"].dtype))
            if "last_hidden_states" in v and last_hidden_states is not None:
                v["last_hidden_states"][row_slice].copy_(last_hidden_states.to(v["last_hidden_states"].dtype))

    def generate(self, requests: Sequence[RowRequest]) -> List[InferenceOutput]:
        raise NotImplementedError

    def health_check(self) -> bool:
        return True

    def get_status(self) -> dict:
        return {"name": self.name, "rows": getattr(self, "rows_done", 0), "tokens": getattr(self, "tokens_done", 0),
                "busy_seconds": getattr(self, "busy_seconds", 0.0)}

    def shutdown(self) -> None:
        pass

    close = shutdown

    # -- shared helpers ---------------------------------------------------------------------------
    def _slot_views(self, req: RowRequest):
        n = int(req.input_ids.shape[0])
        views = []
        for consumer, slot, _gen in req.leases:
            views.append(self.rings[consumer].views(slot, n))
        return views

    def _finish(self, req: RowRequest, views, layer_ids, device_flags: bool) -> InferenceOutput:
        n = int(req.input_ids.shape[0])
        keys = []
        for (consumer, slot, gen), v in zip(req.leases, views):
            ring = self.rings[consumer]
            v["input_ids"].copy_(req.input_ids, non_blocking=True)
            if device_flags:
                ring.publish(slot, gen)
            keys.append(ring.descriptor(slot, gen, n, self._layers_of(consumer)).to_key())
        lay = self.rings[req.leases[0][0]].layout
        self.rows_done = getattr(self, "rows_done", 0) + 1
        self.tokens_done = getattr(self, "tokens_done", 0) + n
        return InferenceOutput(req.row_id, list(req.data_ids), keys,
                               {"input_ids": (n,), "hidden_states": (n, lay.num_layers * lay.hidden),
                                "last_hidden_states": (n, lay.hidden)},
                               tuple(req.document_lengths), list(req.packed_loss_masks), list(req.metadata),
                               feature_bytes(n, lay.num_layers, lay.hidden, lay.elem, lay.store_last_hidden), self.name)


class NativeTargetEngine(InferenceEngine):
    def __init__(self, target_config: dict, layer_ids: Sequence[int], device: str = "cuda:0", dtype: str = "bfloat16",
                 seed: int = 0, name: str = "target0", device_flags: bool = False, weights_path: Optional[str] = None,
                 fail_after: Optional[int] = None, delay_s: float = 0.0, tp_rank: int = 0, tp_size: int = 1,
                 tp_address: Optional[str] = None):
        """``tp_size > 1``: this process is rank ``tp_rank`` of a tensor-parallel engine whose ranks meet at ``tp_address``
        (``tcp://host:port``).  All ranks run every call; rank 0 owns the rings and the answers."""
        from aspec_b200.models.target.dense import DenseTarget, TargetConfig
        self.tp_rank, self.tp_size = int(tp_rank), int(tp_size)
        self.name = name
        self.delay_s = float(delay_s or 0.0)    # a slow producer for pipeline experiments (host sleep per call)
        self.device = torch.device(device)
        self.layer_ids = tuple(layer_ids)
        self.device_flags = device_flags
        self.fail_after = fail_after            # fault injection on the host: raise after N rows
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if self.tp_size > 1:
            import datetime
            import torch.distributed as dist
            dist.init_process_group("nccl" if self.device.type == "cuda" else "gloo", init_method=tp_address,
                                    rank=self.tp_rank, world_size=self.tp_size, timeout=datetime.timedelta(minutes=30),
                                    device_id=self.device if self.device.type == "cuda" else None)
        torch.manual_seed(seed)
        prev = torch.get_default_dtype()
        torch.set_default_dtype(getattr(torch, dtype))
        try:
            with torch.device(self.device):      # 8B+ parameters are created directly in device memory
                self.model = DenseTarget(TargetConfig(**target_config), self.tp_rank, self.tp_size)
        finally:
            torch.set_default_dtype(prev)
        if weights_path and self.tp_size > 1:
            self.model.load_whole_state_dict(torch.load(weights_path, map_location="cpu", mmap=True))
        elif weights_path:
            self.model.load_state_dict(torch.load(weights_path, map_location=self.device), strict=True)
        else:
            self.model.init_random(seed)
        self.model.eval()
        self.rings: Dict[int, RemoteRing] = {}
        self.busy_seconds = 0.0

    def init(self) -> None:
        pass

    def lm_head(self, copies: int = 1) -> list:
        """Relayable handles (one per trainer) of the frozen output head."""
        from aspec_b200.transport.feature_ring import export_tensor
        return [export_tensor(self.model.lm_head.detach()) for _ in range(copies)]

    def embedding(self, copies: int = 1) -> list:
        from aspec_b200.transport.feature_ring import export_tensor
        return [export_tensor(self.model.embed_tokens.weight.detach()) for _ in range(copies)]

    # -- train-with-decode: the engine continues the prompts itself -----------------------------------------------------
    def load_draft(self, asset_dir: str) -> dict:
        """Load (first call) or hot-reload (later calls) the Draft that proposes blocks while this engine decodes.  The
        text does not depend on it - every kept token is the Target's own draw - only the tokens per Target pass do
        (reference: speculative decode with weight sync, aspec/inference/engine/sgl_engine_decode.py:39-424)."""
        from aspec_b200.draft_artifact import BlockDraftConsumer, load_native_draft
        if getattr(self, "draft", None) is None:
            model, manifest = load_native_draft(asset_dir, device=self.device, dtype=self.model.lm_head.dtype)
            block = int(manifest.get("training_contract", {}).get("block_size") or getattr(model.config, "block_size", 0) or 0)
            self.draft = BlockDraftConsumer(model, block_size=block)
            self.draft_layers = tuple(int(l) for l in model.config.target_layer_ids)
        else:
            manifest = self.draft.update_weights_from_disk(asset_dir)
        self.draft_loads = getattr(self, "draft_loads", 0) + 1
        return {"algorithm": manifest["algorithm"], "loads": self.draft_loads}

    @torch.no_grad()
    def _decode(self, requests: Sequence[RowRequest]) -> List[RowRequest]:
        """Continue every document of every request; returns requests over prompt + response with the response as the
        supervised span.  A response never outgrows what the planner reserved for its document."""
        import dataclasses
        from aspec_b200.data.utils import pack_loss_mask
        from aspec_b200.inference.speculative_decode import batched_generate
        prompts, budgets, seeds = [], [], []
        for req in requests:
            off = 0
            for j, n in enumerate(req.document_lengths):
                prompts.append(req.input_ids[off:off + n])
                budgets.append(int(req.decode["max_new_tokens"][j]))
                seeds.append(int(req.decode["seeds"][j]))
                off += n
        d = requests[0].decode
        consumer = getattr(self, "draft", None)
        # documents decoded together share every Target pass but each holds its keys and values for its whole reserved
        # length: ``decode.max_running_requests`` and a byte budget for the cache bound how many run at once (a document's
        # text does not depend on which others it ran with)
        cfg = self.model.config
        row_bytes = 2 * cfg.num_hidden_layers * self.model.layers[0].hk * cfg.head_dim * self.model.lm_head.element_size()
        longest = max(int(p.numel()) + b for p, b in zip(prompts, budgets)) + 16
        fit = max(int(float(d.get("cache_budget_bytes") or 24 * 2 ** 30) // max(row_bytes * longest, 1)), 1)
        wave = max(min(fit, int(d.get("max_running_requests") or len(prompts)), len(prompts)), 1)
        res = []
        for lo in range(0, len(prompts), wave):
            res += batched_generate(self.model, prompts[lo:lo + wave], max_new_tokens=budgets[lo:lo + wave],
                                    min_new_tokens=int(d.get("min_new_tokens", 0)), stop_token_ids=d.get("stop_token_ids") or (),
                                    temperature=float(d.get("temperature", 1.0)), top_k=int(d.get("top_k", -1)),
                                    top_p=float(d.get("top_p", 1.0)), seeds=seeds[lo:lo + wave], consumer=consumer,
                                    layer_ids=getattr(self, "draft_layers", ()))
        self.decode_waves = getattr(self, "decode_waves", 0) + -(-len(prompts) // wave)
        out, i = [], 0
        for req in requests:
            ids, lengths, masks = [], [], []
            stats = {"generated_tokens": 0, "target_passes": 0, "accepted_draft_tokens": 0, "verify_rounds": 0}
            off = 0
            for n in req.document_lengths:
                new = res[i]["tokens"]
                ids += [req.input_ids[off:off + n].reshape(-1), torch.tensor(new, dtype=torch.long)]
                lengths.append(n + len(new))
                masks.append(pack_loss_mask([0] * n + [1] * len(new)))
                stats["generated_tokens"] += len(new)
                stats["target_passes"] += res[i]["target_passes"]
                stats["accepted_draft_tokens"] += sum(res[i]["accepted_per_round"])
                stats["verify_rounds"] += len(res[i]["accepted_per_round"])
                off += n
                i += 1
            done = dataclasses.replace(req, input_ids=torch.cat(ids), document_lengths=tuple(lengths), packed_loss_masks=masks,
                                       decode=None)
            done.decode_stats = stats
            out.append(done)
        for k in ("generated_tokens", "target_passes", "accepted_draft_tokens", "verify_rounds"):
            setattr(self, "decode_" + k, getattr(self, "decode_" + k, 0) + sum(r.decode_stats[k] for r in out))
        return out

    def get_status(self) -> dict:
        st = super().get_status()
        if getattr(self, "decode_generated_tokens", 0):
            st["decode"] = {k: getattr(self, "decode_" + k, 0) for k in
                            ("generated_tokens", "target_passes", "accepted_draft_tokens", "verify_rounds")}
            st["decode"]["draft_loads"] = getattr(self, "draft_loads", 0)
            st["decode"]["waves"] = getattr(self, "decode_waves", 0)
        return st

    @torch.no_grad()
    def generate(self, requests: Sequence[RowRequest]) -> List[InferenceOutput]:
        t0 = time.perf_counter()
        outs = []
        if any(req.decode for req in requests):
            if not all(req.decode for req in requests):
                raise ValueError("one call holds either prompts to continue or rows to prefill, not both")
            requests = self._decode(requests)
        if self.fail_after is not None and getattr(self, "rows_done", 0) + len(requests) > self.fail_after:
            raise RuntimeError(f"{self.name}: injected producer failure")
        if self.delay_s:
            time.sleep(self.delay_s)
        if self.tp_rank > 0:
            # a tensor-parallel helper: same pass, same collectives, nothing to store and nothing to report
            ids = torch.cat([req.input_ids.reshape(-1) for req in requests]).to(self.device, non_blocking=True)
            self.model.prefill(ids, [n for req in requests for n in req.document_lengths], ())
            self.busy_seconds += time.perf_counter() - t0
            return []
        # all requests of the call run as ONE packed prefill (bigger GEMMs); each request's rows go to its own slots
        all_views, segments, off = [], [], 0
        for req in requests:
            views = self._slot_views(req)
            n = int(req.input_ids.shape[0])
            segments.append((off, off + n, RingFeatureSink(views, self.layer_ids, self.model.config.hidden_size,
                                                           [self._layers_of(c) for c, _s, _g in req.leases])))
            all_views.append(views)
            off += n
        ids = torch.cat([req.input_ids.reshape(-1) for req in requests]).to(self.device, non_blocking=True)
        lengths = [n for req in requests for n in req.document_lengths]
        self.model.prefill(ids, lengths, self.layer_ids, sink=segments if len(requests) > 1 else segments[0][2])
        for req, views in zip(requests, all_views):
            outs.append(self._finish(req, views, self.layer_ids, self.device_flags))
            outs[-1].stats = dict(getattr(req, "decode_stats", {}))
        if self.device.type == "cuda" and not self.device_flags:
            torch.cuda.current_stream(self.device).synchronize()     # host-ordered readiness
        self.busy_seconds += time.perf_counter() - t0
        return outs


class SyntheticEngine(InferenceEngine):
    """Random features; deterministic per document so that runs and resumes agree."""

    def __init__(self, layer_ids: Sequence[int], hidden: int, device: str = "cpu", dtype: str = "float32",
                 name: str = "synthetic0", seed: int = 0, delay_s: float = 0.0, fail_after: Optional[int] = None):
        self.name, self.layer_ids, self.hidden = name, tuple(layer_ids), hidden
        self.device, self.dtype, self.seed = torch.device(device), getattr(torch, dtype), seed
        self.delay_s, self.fail_after = delay_s, fail_after
        self.rings = {}

    def init(self) -> None:
        pass

    def generate(self, requests):
        outs = []
        for req in requests:
            if self.fail_after is not None and getattr(self, "rows_done", 0) >= self.fail_after:
                raise RuntimeError(f"{self.name}: injected producer failure")
            if self.delay_s:
                time.sleep(self.delay_s)
            views = self._slot_views(req)
            n = int(req.input_ids.shape[0])
            # one stream per (document, layer): a layer's features do not depend on which other layers are captured, so
            # a Draft sees the same features alone and as one reader of a shared stream
            doc = self.seed * 7919 + int(req.input_ids.sum()) % (2 ** 31)
            parts = []
            for layer in (*self.layer_ids, -1):
                g = torch.Generator().manual_seed((doc * 1000003 + int(layer) + 1) % (2 ** 63 - 1))
                parts.append(torch.randn(n, self.hidden, generator=g))
            hs, last = torch.cat(parts[:-1], -1), parts[-1]
            self._copy_features(req, views, hs, last)
            outs.append(self._finish(req, views, self.layer_ids, device_flags=True))
        return outs


class OfflineReplayEngine(InferenceEngine):
    """Replays ``samples/*.pt`` of an offline feature store into ring slots."""

    def __init__(self, feature_dir: str, name: str = "offline0", require_complete: bool = True):
        from aspec_b200.offline.dataset import OfflineFeatureStore
        self.name = name
        self.store = OfflineFeatureStore(feature_dir, allow_incomplete=not require_complete)
        self.layer_ids = tuple(self.store.binding["feature_contract"]["aux_hidden_state_layers"])
        self.rings = {}

    def init(self) -> None:
        pass

    def generate(self, requests):
        outs = []
        for req in requests:
            views = self._slot_views(req)
            off = 0
            for data_id, n in zip(req.data_ids, req.document_lengths):
                try:
                    rec = self.store.load(data_id)
                except KeyError:
                    raise KeyError(f"document {data_id!r} of the training data has no stored features in {self.store.root}: the "
                                   "store was made from other documents (or from the same file before its documents had "
                                   "ids); prepare it again from this training file") from None
                if int(rec["input_ids"].numel()) != int(n):
                    raise ValueError(f"document {data_id!r}: the store holds {int(rec['input_ids'].numel())} tokens, the training "
                                     f"data {int(n)} (another max_seq_length or tokenizer?)")
                last = rec.get("last_hidden_states")
                self._copy_features(req, views, rec["hidden_states"].reshape(n, -1),
                                    None if last is None else last.reshape(n, -1), slice(off, off + n))
                off += n
            outs.append(self._finish(req, views, self.layer_ids, device_flags=True))
        return outs
