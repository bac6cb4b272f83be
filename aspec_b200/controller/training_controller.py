"""Driver-side scheduler state: dataset, row planning, and the work ledger.

Role of the reference's ``AsyncTrainingController`` (aspec/controller/training_controller.py:355-1921),
re-shaped for push transport: because a Target rank stores features directly into the consuming Draft
rank's memory, the consumer of every row is decided *before* the row is produced.  Document lengths and
loss masks are known up front, so the same policies apply ahead of time:

* unpacked: ``dp * micro_batch_size`` samples per micro-step, length-sorted and dealt so every rank gets
  neighbours in length (aspec/controller/training_controller.py:1535-1611);
* packed (``dflash_packing``): ``pack_work_aware_rows`` over a look-ahead pool - rows seeded with the oldest
  samples, then best-fit by useful-anchor density (aspec/controller/packing.py:87-167);
* finite tails: an update that cannot be completed is dropped and reported (aspec/controller/loop.py:1537-1583).

Every produced row is registered in the ledger, marked dispatched with the number of consumers, released
by its trainers and committed with the optimizer step.
"""
from __future__ import annotations

import random
import zlib
from typing import Any, Dict, List, Optional, Sequence

import torch

from aspec_b200.controller.packing import (count_eagle_supervised_positions, count_eligible_anchor_starts,
                                           pack_work_aware_rows)
from aspec_b200.data.synthetic import SyntheticSpec, make_document
from aspec_b200.utils.types import InferenceOutput, RowRequest
from aspec_b200.work_lifecycle import WorkLifecycleLedger, build_work_identity


def draft_vocabulary_from_samples(samples, draft_config: dict, args: dict):
    """``(d2t, t2d)`` for a Draft whose head covers ``draft_vocab_size < vocab_size`` tokens: the most frequent
    supervised tokens of the admitted dataset (reference: aspec/data/preprocessing.py ``generate_vocab_mapping_file``).
    ``None`` when the head is not pruned, or when ``model.keep_initial_vocab_mapping`` keeps the mapping that came with
    the initial Draft asset."""
    vocab = int(draft_config.get("vocab_size") or 0)
    small = int(draft_config.get("draft_vocab_size") or vocab)
    if not vocab or small >= vocab or args.get("keep_initial_vocab_mapping"):
        return None
    from aspec_b200.data.preprocessing import generate_vocab_mapping
    return generate_vocab_mapping(samples, vocab, small)


def prompt_of(sample: dict) -> torch.Tensor:
    """The tokens before the LAST supervised span of a document: earlier turns stay as context, the final response is
    what a decoding Target writes anew (reference: the dataset is rendered with a generation prompt when training with
    decode, aspec/data/dataset.py:285-360)."""
    ids = sample["input_ids"].reshape(-1)
    runs = [int(v) for v in str(sample["packed_loss_mask"]).split(",") if v != ""]
    # runs alternate unsupervised, supervised, ...; find where the last non-empty supervised run starts
    start, last = 0, None
    for i, n in enumerate(runs):
        if i % 2 == 1 and n > 0:
            last = start
        start += n
    return ids[: last if last is not None else ids.numel()].clone()


class TrainingController:
    def __init__(self, args: Dict[str, Any], dp_size: int, consumers_per_row: int = 1, algorithm: str = "dspark"):
        self.args = dict(args)
        self.dp_size = int(dp_size)
        self.consumers_per_row = int(consumers_per_row)
        self.algorithm = algorithm
        self.ledger = WorkLifecycleLedger()
        self.samples: List[dict] = []
        self.epoch = 0
        self.cursor = 0
        self.order: List[int] = []
        self.committed_ids: set = set()          # work ids committed in earlier attempts (resume)
        self.dropped_tail = 0
        self.rows_planned = 0
        self.inference_error: Optional[str] = None
        self.block_size = int(args.get("dspark_block_size", 7) if algorithm == "dspark" else args.get("dflash_block_size", 16))

    # -- dataset ----------------------------------------------------------------------------------
    def load_dataset(self, samples: Optional[Sequence[dict]] = None) -> int:
        a = self.args
        if samples is None:
            path = a.get("train_data_path") or "synthetic"
            if path == "synthetic":
                spec = SyntheticSpec(vocab_size=int(a.get("synthetic_vocab_size") or 32000),
                                     min_len=int(a.get("synthetic_min_length", 256)),
                                     max_len=min(int(a.get("synthetic_max_length", 4096)), int(a["max_seq_length"])),
                                     length_distribution=a.get("synthetic_length_distribution", "log_uniform"),
                                     loss_tail_fraction=float(a.get("synthetic_loss_tail_fraction", 0.6)),
                                     seed=int(a.get("dataset_seed") if a.get("dataset_seed") is not None else a.get("seed", 0)))
                samples = [make_document(spec, i) for i in range(int(a.get("synthetic_num_documents", 4096)))]
            else:
                from aspec_b200.data.dataset import load_training_samples
                samples = load_training_samples(path, a)
        max_len = int(a["max_seq_length"])
        min_loss = int(a.get("min_loss_tokens", 0))
        self.samples = []
        rejected = {"longer_than_max_seq_length": 0, "no_supervised_position": 0, "fewer_loss_tokens_than_min_loss_tokens": 0}
        source_rows = 0
        decode = bool(a.get("train_with_decode"))
        if decode:
            rejected.update(no_prompt=0, no_room_for_a_response=0)
        for s in samples:
            source_rows += 1
            if decode:
                # the document gives the prompt only (everything before its last supervised span); the Target engine
                # writes the response, for which the row keeps room up to ``decode_max_new_tokens``
                prompt = prompt_of(s)
                room = min(int(a.get("decode_max_new_tokens", 512)), max_len - int(prompt.numel()))
                if prompt.numel() < 1:
                    rejected["no_prompt"] += 1
                elif room < max(int(a.get("decode_min_new_tokens", 2)), self.block_size, 1):
                    rejected["no_room_for_a_response"] += 1
                else:
                    self.samples.append({**s, "input_ids": prompt, "packed_loss_mask": str(int(prompt.numel())),
                                         "length": int(prompt.numel()) + room, "useful": room, "max_new_tokens": room})
                continue
            n = int(s["input_ids"].shape[-1])
            if n > max_len:
                rejected["longer_than_max_seq_length"] += 1
                continue
            if self.algorithm in ("eagle3", "eagle4", "mtp"):
                useful = count_eagle_supervised_positions(s["packed_loss_mask"], n, int(a.get("ttt_length", 7)))
            else:
                useful = count_eligible_anchor_starts(s["packed_loss_mask"], n, self.block_size)
            if useful <= 0:
                rejected["no_supervised_position"] += 1
                continue
            if sum(int(v) for v in s["packed_loss_mask"].split(",")[1::2]) < min_loss:
                rejected["fewer_loss_tokens_than_min_loss_tokens"] += 1
                continue
            self.samples.append({**s, "length": n, "useful": useful})
        # source-to-runtime accounting for the run's evidence: every source row is admitted or rejected for a reason
        self.admission = {"source_rows": source_rows, "rejected": {k: v for k, v in rejected.items() if v}}
        self._start_epoch()
        return len(self.samples)

    def _start_epoch(self) -> None:
        self.order = list(range(len(self.samples)))
        if self.args.get("shuffle_dataset", True):
            seed = int(self.args.get("dataset_seed") if self.args.get("dataset_seed") is not None else self.args.get("seed", 0))
            random.Random(seed * 1000003 + self.epoch).shuffle(self.order)
            group = int(self.args.get("length_group_size", 32))
            if group > 1:      # length-grouped ordering: neighbours in the stream have similar lengths
                chunks = [self.order[i:i + group * self.dp_size] for i in range(0, len(self.order), group * self.dp_size)]
                self.order = [i for ch in chunks for i in sorted(ch, key=lambda j: -self.samples[j]["length"])]
        self.cursor = 0

    def dataset_fingerprint(self) -> str:
        import hashlib
        h = hashlib.sha256()
        for s in self.samples:
            h.update(f"{s['data_id']}:{s['length']};".encode())
        return h.hexdigest()

    def _identity(self, sample: dict) -> dict:
        return build_work_identity(split="train", epoch=self.epoch, source_id=sample["data_id"])

    # -- planning ---------------------------------------------------------------------------------
    def _take(self, n: int) -> Optional[List[int]]:
        out = []
        while len(out) < n and self.cursor < len(self.order):
            idx = self.order[self.cursor]
            self.cursor += 1
            if self._identity(self.samples[idx])["work_id"] in self.committed_ids:
                continue       # already trained on before the checkpoint this run resumed from
            out.append(idx)
        return out if len(out) == n else None

    def plan_update(self, accumulation: int) -> Optional[List[List[List[int]]]]:
        """Rows for one optimizer update: ``[microstep][dp_rank] -> sample indices``.  ``None`` = epoch tail."""
        a = self.args
        mbs = int(a.get("micro_batch_size", 1))
        plan = []
        start_cursor = self.cursor
        for _ in range(accumulation):
            if a.get("dflash_packing"):
                pool_n = max(int(a.get("packing_min_samples_per_dispatch", 0)), self.dp_size,
                             min(int(a.get("max_sample_pool_size", 64)), len(self.order) - self.cursor))
                pool = self._take(min(pool_n, max(len(self.order) - self.cursor, 0))) or []
                if len(pool) < self.dp_size:
                    plan = None
                    break
                res = pack_work_aware_rows([self.samples[i]["length"] for i in pool],
                                           [self.samples[i]["useful"] for i in pool], dp_size=self.dp_size,
                                           max_seq_length=int(a["max_seq_length"]))
                rows = [[pool[j] for j in row] for row in res.rank_rows]
                used = set(res.selected_indices)
                leftovers = [pool[j] for j in range(len(pool)) if j not in used]
                # samples that did not fit go back to the front of the stream
                for idx in reversed(leftovers):
                    self.cursor -= 1
                    self.order[self.cursor] = idx
                plan.append(rows)
            else:
                got = self._take(self.dp_size * mbs)
                if got is None:
                    plan = None
                    break
                got.sort(key=lambda i: -self.samples[i]["length"])
                rows = [[] for _ in range(self.dp_size)]
                # serpentine deal: every rank receives samples of neighbouring lengths and similar totals
                for j, idx in enumerate(got):
                    r = j % self.dp_size
                    if (j // self.dp_size) % 2:
                        r = self.dp_size - 1 - r
                    rows[r].append(idx)
                plan.append(rows)
        if plan is None:
            self.dropped_tail += len(self.order) - start_cursor
            return None
        return plan

    def next_epoch(self) -> None:
        self.epoch += 1
        self._start_epoch()

    def row_request(self, sample_indices: Sequence[int], layer_ids) -> RowRequest:
        docs = [self.samples[i] for i in sample_indices]
        self.rows_planned += 1
        decode = None
        if self.args.get("train_with_decode"):
            a = self.args
            seed = int(a.get("seed", 0))
            decode = {"max_new_tokens": [int(d["max_new_tokens"]) for d in docs],
                      # a document's noise depends on the document, the epoch and the run's seed - not on its row or engine
                      "seeds": [zlib.crc32(f"{d['data_id']}|{self.epoch}".encode()) ^ seed for d in docs],
                      "min_new_tokens": int(a.get("decode_min_new_tokens", 2)), "stop_token_ids": list(a.get("decode_stop_token_ids") or ()),
                      "max_running_requests": a.get("decode_max_running_requests"),
                      "temperature": float(a.get("decode_temperature", 1.0)), "top_k": int(a.get("decode_top_k", -1)),
                      "top_p": float(a.get("decode_top_p", 1.0))}
        return RowRequest(row_id=f"row-{self.epoch}-{self.rows_planned}", data_ids=[d["data_id"] for d in docs],
                          input_ids=torch.cat([d["input_ids"].reshape(-1) for d in docs]),
                          document_lengths=tuple(int(d["input_ids"].numel()) for d in docs),
                          packed_loss_masks=[d["packed_loss_mask"] for d in docs],
                          metadata=[self._identity(d) for d in docs], layer_ids=tuple(layer_ids), decode=decode)

    # -- ledger ------------------------------------------------------------------------------------
    def register_result(self, out: InferenceOutput) -> None:
        per_doc = max(out.size_bytes // max(len(out.data_ids), 1), 0)
        self.ledger.register_outputs([{"data_id": d, "feature_key": f"{out.feature_keys[0]}#{i}", "metadata": m,
                                       "size_bytes": per_doc}
                                      for i, (d, m) in enumerate(zip(out.data_ids, out.metadata))])
        for m in out.metadata:
            self.ledger.mark_dispatched(m, expected_consumers=self.consumers_per_row)

    def release_result(self, out: InferenceOutput, participant: str, outcome: str = "consumed") -> None:
        for i, (d, m) in enumerate(zip(out.data_ids, out.metadata)):
            self.ledger.release_output(execution_id=m["execution_id"], data_id=d,
                                       feature_key=f"{out.feature_keys[0]}#{i}", participant=participant, outcome=outcome)

    def commit_optimizer_step(self, optimizer_step: int, execution_ids: Sequence[str]) -> None:
        unique = len(set(execution_ids))
        self.ledger.commit_optimizer_step(optimizer_step=optimizer_step, execution_ids=list(execution_ids),
                                          expected_unique=unique, expected_occurrences=self.consumers_per_row)

    def work_state(self) -> dict:
        st = self.ledger.status()
        return {"dataset_epoch": self.epoch, "dataset_size": len(self.samples), "dataset_cursor": self.cursor,
                "dataset_fingerprint": self.dataset_fingerprint(),
                "committed_work_ids": sorted(set(st["committed_work_ids"]) | self.committed_ids),
                "dropped_tail_samples": self.dropped_tail}

    def restore(self, work_state: dict) -> None:
        if work_state.get("dataset_fingerprint") not in (None, self.dataset_fingerprint()):
            raise ValueError("checkpoint was written for a different dataset (fingerprint mismatch)")
        self.epoch = int(work_state.get("dataset_epoch", 0))
        self.committed_ids = set(work_state.get("committed_work_ids", []))
        self.dropped_tail = int(work_state.get("dropped_tail_samples", 0))      # the count runs over the whole run
        self._start_epoch()
