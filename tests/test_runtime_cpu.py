"""Host runtime: slot ring leases, work ledger state machine, packer, feature ring descriptors."""
import threading
import time

import pytest
import torch

from aspec_b200.controller.packing import (count_eagle_supervised_positions, count_eligible_anchor_starts,
                                           pack_work_aware_rows)
from aspec_b200.parallel.context import context_shard_bounds, packed_shard_positions
from aspec_b200.transport.feature_ring import FeatureDescriptor, FeatureRing, RemoteRing, SlotLayout
from aspec_b200.transport.slot_ring import GenerationSlotRing, RingLease
from aspec_b200.work_lifecycle import WorkLifecycleError, WorkLifecycleLedger, build_work_identity


def test_ring_generations_and_stale_release():
    ring = GenerationSlotRing(2)
    a = ring.acquire("p0")
    b = ring.acquire("p1")
    assert {a.slot_id, b.slot_id} == {0, 1} and a.generation == 1
    with pytest.raises(TimeoutError):
        ring.acquire("p2", timeout=0.05)
    ring.release(a.slot_id, a.generation, "p0")
    with pytest.raises(RuntimeError):
        ring.release(a.slot_id, a.generation, "p0")            # duplicate
    c = ring.acquire("p2")
    assert c.slot_id == a.slot_id and c.generation == 2
    with pytest.raises(RuntimeError):
        ring.release(c.slot_id, 1, "p2")                        # stale generation
    with pytest.raises(RuntimeError):
        ring.release(c.slot_id, c.generation, "someone-else")   # wrong owner
    assert ring.in_use == 2


def test_ring_readers_and_idempotent_ack():
    ring = GenerationSlotRing(1)
    lease = ring.acquire("src")
    assert ring.register_readers(lease, ["d0", "d1"])
    with pytest.raises(RuntimeError):
        ring.register_readers(lease, ["d2"])                    # audience is frozen
    with pytest.raises(RuntimeError):
        ring.release(lease.slot_id, lease.generation, "src")    # readers pending
    with pytest.raises(RuntimeError):
        ring.release_reader(lease, "intruder")
    assert ring.reader_pending(lease, "d0")
    assert ring.release_reader(lease, "d0") is False
    assert ring.release_reader(lease, "d1") is True and ring.in_use == 0
    # a retried acknowledgement of the old lease must not free the next generation
    newer = ring.acquire("src")
    assert ring.release_acknowledged(lease.slot_id, lease.generation, "src") is False
    assert ring.in_use == 1
    assert ring.release_acknowledged(newer.slot_id, newer.generation, "src") is True
    with pytest.raises(RuntimeError):
        ring.release_acknowledged(0, 99, "src")


def test_ring_acquire_blocks_until_release():
    ring = GenerationSlotRing(1)
    first = ring.acquire("a")
    got = {}

    def waiter():
        got["lease"] = ring.acquire("b", timeout=5.0)

    t = threading.Thread(target=waiter)
    t.start()
    time.sleep(0.1)
    ring.release(first.slot_id, first.generation, "a")
    t.join(5.0)
    assert got["lease"].generation == 2 and ring.wait_until_empty(0.01) is False


def _meta(i, epoch=0):
    return build_work_identity(split="train", epoch=epoch, source_id=f"doc{i}")


def test_ledger_happy_path_and_validation():
    L = WorkLifecycleLedger()
    metas = [_meta(i) for i in range(3)]
    L.register_outputs([{"data_id": f"doc{i}", "feature_key": f"k{i}", "metadata": m, "size_bytes": 100}
                        for i, m in enumerate(metas)])
    assert L.resident_outputs == 3 and L.resident_bytes == 300
    for m in metas[:2]:
        L.mark_dispatched(m, expected_consumers=2)
    for i, m in enumerate(metas[:2]):
        for p in ("t0", "t1"):
            L.release_output(execution_id=m["execution_id"], data_id=f"doc{i}", feature_key=f"k{i}", participant=p,
                             outcome="consumed")
    assert L.state_of(metas[0]["execution_id"]) == "released"
    L.commit_optimizer_step(optimizer_step=0, execution_ids=[m["execution_id"] for m in metas[:2]] * 2,
                            expected_unique=2, expected_occurrences=2)
    L.begin_discard(metas[2])
    L.confirm_discarded([metas[2]])
    st = L.status()
    assert st["validated"] and st["resident_outputs"] == 0 and len(st["committed_work_ids"]) == 2
    assert st["peak_resident_outputs"] == 3


def test_ledger_rejects_protocol_violations():
    L = WorkLifecycleLedger()
    m = _meta(0)
    L.register_output(data_id="doc0", feature_key="k0", metadata=m, size_bytes=1)
    with pytest.raises(WorkLifecycleError):
        L.register_output(data_id="doc0", feature_key="k9", metadata=m, size_bytes=1)       # duplicate execution
    with pytest.raises(WorkLifecycleError):
        L.register_outputs([{"data_id": "a", "feature_key": "k0", "metadata": _meta(5), "size_bytes": 1}])  # duplicate key
    with pytest.raises(WorkLifecycleError):
        L.commit_optimizer_step(optimizer_step=0, execution_ids=[m["execution_id"]], expected_unique=1)  # not released
    L.mark_dispatched(m, expected_consumers=1)
    with pytest.raises(WorkLifecycleError):
        L.mark_dispatched(m, expected_consumers=1)
    with pytest.raises(WorkLifecycleError):
        L.release_output(execution_id=m["execution_id"], data_id="WRONG", feature_key="k0", participant="t", outcome="consumed")
    L.release_output(execution_id=m["execution_id"], data_id="doc0", feature_key="k0", participant="t", outcome="consumed")
    L.commit_optimizer_step(optimizer_step=3, execution_ids=[m["execution_id"]], expected_unique=1)
    with pytest.raises(WorkLifecycleError):
        L.commit_optimizer_step(optimizer_step=3, execution_ids=[], expected_unique=0)       # repeated step
    assert not L.status()["validated"]                     # errors were recorded
    # a batch with one bad entry registers nothing
    L2 = WorkLifecycleLedger()
    with pytest.raises(WorkLifecycleError):
        L2.register_outputs([{"data_id": "a", "feature_key": "x", "metadata": _meta(1), "size_bytes": 1},
                             {"data_id": "b", "feature_key": "x", "metadata": _meta(2), "size_bytes": 1}])
    assert L2.resident_outputs == 0


def test_ledger_failure_and_owner_fence():
    L = WorkLifecycleLedger()
    metas = [_meta(i) for i in range(3)]
    L.register_outputs([{"data_id": f"doc{i}", "feature_key": f"k{i}", "metadata": m, "size_bytes": 10}
                        for i, m in enumerate(metas)])
    L.mark_dispatched(metas[0], expected_consumers=1)
    L.release_output(execution_id=metas[0]["execution_id"], data_id="doc0", feature_key="k0", participant="t",
                     outcome="discarded_after_error")
    assert L.state_of(metas[0]["execution_id"]) == "failed"
    L.mark_dispatched(metas[1], expected_consumers=1)
    assert L.discard_after_owner_fence([metas[1]["execution_id"]]) == 1
    assert L.discard_all_after_owner_fence() == 1 and L.resident_outputs == 0


def test_packer_matches_policy():
    res = pack_work_aware_rows([100, 200, 50, 60, 300, 10], [10, 20, 40, 5, 100, 9], dp_size=2, max_seq_length=400)
    assert res.rank_rows[0] == [0, 4] and set(res.rank_rows[1]) == {1, 5, 2, 3}
    assert res.packed_tokens == 720 and res.fill_ratio == pytest.approx(0.9)
    assert pack_work_aware_rows([10], [1], dp_size=2, max_seq_length=64) is None
    with pytest.raises(ValueError):
        pack_work_aware_rows([100], [1], dp_size=1, max_seq_length=64)
    capped = pack_work_aware_rows([10] * 8, [5] * 8, dp_size=2, max_seq_length=100, max_selected=3)
    assert len(capped.selected_indices) == 3
    assert count_eligible_anchor_starts("2,3,2,2,1", 10, 2) == 5
    assert count_eligible_anchor_starts([0, 10], 10, 4) == 7
    assert count_eagle_supervised_positions("1,9", 10, 3) == 8 + 8 + 7


def test_context_shard_bounds():
    T, w = 103, 4
    spans = [context_shard_bounds(T, r, w, alignment=4) for r in range(w)]
    assert spans[0][0] == 0 and spans[-1][1] == T
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert all(s % 4 == 0 for s, _ in spans)
    assert context_shard_bounds(3, 0, 4) == (0, 0) and context_shard_bounds(3, 3, 4) == (2, 3)
    pos = packed_shard_positions([10, 6], 1, 2)
    assert pos == [5, 6, 7, 8, 9, 13, 14, 15]


def test_feature_ring_descriptor_and_stale_rejection():
    lay = SlotLayout(64, 3, 16, dtype="float32")
    assert all(v % 256 == 0 for v in lay.offsets.values())
    ring = FeatureRing(2, lay, "cpu", run_id="r1", attempt_id="0", consumer=3)
    remote = RemoteRing(ring.export())
    v = remote.views(1, 10)
    v["hidden_states"].fill_(2.0)
    v["input_ids"].copy_(torch.arange(10))
    d = remote.descriptor(1, 5, 10, [2, 18, 33])
    assert FeatureDescriptor.from_key(d.to_key()) == d
    with pytest.raises(TimeoutError):
        ring.read(d.to_key(), device_flags=True)            # never published
    remote.publish(1, 5)
    got = ring.read(d.to_key(), device_flags=True)
    assert got["hidden_states"].shape == (10, 48) and got["input_ids"][-1] == 9
    stale = FeatureDescriptor("r0", "0", 3, 1, 5, 10, (2, 18, 33), 16, "float32")
    with pytest.raises(RuntimeError):
        ring.read(stale.to_key())
    wrong = FeatureDescriptor("r1", "0", 4, 1, 5, 10, (2, 18, 33), 16, "float32")
    with pytest.raises(RuntimeError):
        ring.read(wrong.to_key())


def test_inference_manager_cuts_batches_by_tokens():
    """With a token budget, short rows are grouped until the budget is reached; long rows go out alone; the row cap
    still bounds a batch."""
    import time
    import torch
    from aspec_b200.controller.inference_manager import InferenceManager
    from aspec_b200.transport.slot_ring import GenerationSlotRing
    from aspec_b200.utils.types import InferenceOutput, RowRequest

    class Engine:
        def __init__(self):
            self.batches = []

        def generate(self, requests):
            self.batches.append([sum(r.document_lengths) for r in requests])
            return [InferenceOutput(r.row_id, r.data_ids, [f"k{r.row_id}"], {}, r.document_lengths, r.packed_loss_masks, r.metadata, 0)
                    for r in requests]

    eng = Engine()
    done = []
    mgr = InferenceManager([eng], {0: GenerationSlotRing(64)}, on_result=lambda out, req: done.append(out.row_id),
                           batch_size=6, batch_tokens=1000)
    lengths = [300, 300, 300, 300, 2000, 100, 100, 100, 100, 100, 100, 100]
    for i, n in enumerate(lengths):                       # queued before the worker starts, so batching is deterministic
        mgr.submit(RowRequest(str(i), [str(i)], torch.zeros(n, dtype=torch.int64), (n,), [str(n)], [{}]), [0])
    mgr.start()
    deadline = time.monotonic() + 20
    while len(done) < len(lengths) and time.monotonic() < deadline:
        time.sleep(0.01)
    mgr.stop()
    mgr.raise_if_failed()
    assert len(done) == len(lengths)
    assert eng.batches[0] == [300, 300, 300, 300]          # 1200 >= 1000 tokens
    assert eng.batches[1] == [2000]                        # a long row alone
    assert eng.batches[2] == [100] * 6                     # the row cap
    assert sum(len(b) for b in eng.batches) == len(lengths)
