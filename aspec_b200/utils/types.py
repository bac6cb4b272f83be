"""Control-plane messages.  Only descriptors travel between processes; tensors never do
(reference: aspec/utils/types.py:27-52, aspec/training/data_fetcher.py:98-108)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Tuple


@dataclass
class RowRequest:
    """One training row to produce: one document (MBS1) or several packed documents."""
    row_id: str
    data_ids: List[str]
    input_ids: Any                          # CPU int64 tensor [T] (documents concatenated)
    document_lengths: Tuple[int, ...]
    packed_loss_masks: List[str]
    metadata: List[Dict[str, Any]]          # work identity per document
    leases: List[Tuple[int, int, int]] = field(default_factory=list)   # (consumer, slot, generation)
    layer_ids: Tuple[int, ...] = ()
    # train-with-decode: the documents are prompts and the engine writes the responses itself.  Keys: ``max_new_tokens``
    # and ``seeds`` (one per document), ``min_new_tokens``, ``stop_token_ids``, ``temperature``, ``top_k``, ``top_p``
    decode: Any = None


@dataclass
class InferenceOutput:
    row_id: str
    data_ids: List[str]
    feature_keys: List[str]                 # one per consumer lease
    tensor_shapes: Dict[str, tuple]
    document_lengths: Tuple[int, ...]
    packed_loss_masks: List[str]
    metadata: List[Dict[str, Any]]
    size_bytes: int
    engine: str = ""
    stats: Dict[str, Any] = field(default_factory=dict)      # decode: generated tokens, Target passes, accepted Draft tokens


@dataclass
class TrainSample:
    feature_key: str
    tensor_shapes: Dict[str, tuple]
    document_lengths: Tuple[int, ...]
    packed_loss_masks: List[str]
    metadata: List[Dict[str, Any]]
    data_ids: List[str]
    row_id: str
    last_in_row: bool = True
    last_turn_loss_only: bool = False
