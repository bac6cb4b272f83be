"""Checkpoint exchange between node-local run directories (temp directories stand in for the nodes' disks)."""
import os

import pytest

from aspec_b200 import node_local_files as nlf


def _write(path, data: bytes):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "wb") as f:
        f.write(data)


def _stores(tmp_path, names=("a", "b", "c")):
    return {n: nlf.NodeStore(tmp_path / n / "run", "run-1") for n in names}


def test_send_tree_pushes_verified_copies_to_every_node(tmp_path, monkeypatch):
    monkeypatch.setattr(nlf, "CHUNK_BYTES", 1000)                       # several chunks per file
    src = tmp_path / "ckpt"
    _write(src / "model" / "shard0.bin", os.urandom(3500))
    _write(src / "meta.json", b"{}")
    _write(src / "empty", b"")
    stores = _stores(tmp_path)
    sent = nlf.send_tree(stores, src, "resume-input/iter_0000002", skip=["a"])
    assert sent == 2 * 3502
    want = nlf.manifest(src)
    for n in ("b", "c"):
        assert stores[n].inventory("resume-input/iter_0000002") == want
    assert stores["a"].inventory("resume-input/iter_0000002") == {}
    assert not list((tmp_path / "b").rglob("*" + nlf.NodeStore.PARTIAL))


def test_publish_refuses_corrupted_or_conflicting_bytes_and_escaping_paths(tmp_path):
    store = nlf.NodeStore(tmp_path / "n")
    store.append("x.bin", 0, b"hello")
    with pytest.raises(ValueError):
        store.publish("x.bin", {"size": 5, "sha256": "0" * 64})
    assert not (tmp_path / "n" / "x.bin").exists()
    with pytest.raises(ValueError):
        store.append("y.bin", 7, b"late chunk first")
    with pytest.raises(ValueError):
        store.append("../outside.bin", 0, b"no")
    _write(tmp_path / "n" / "z.bin", b"old")
    store.append("z.bin", 0, b"new")
    import hashlib
    with pytest.raises(ValueError):
        store.publish("z.bin", {"size": 3, "sha256": hashlib.sha256(b"new").hexdigest()})
    os.symlink(tmp_path / "n" / "z.bin", tmp_path / "n" / "link")
    with pytest.raises(ValueError):
        nlf.manifest(tmp_path / "n")


def test_collect_merges_shards_detects_conflicts_and_clears_staging(tmp_path, monkeypatch):
    monkeypatch.setattr(nlf, "CHUNK_BYTES", 512)
    stores = _stores(tmp_path, ("a", "b"))
    rel = nlf.staging_dir(4)
    assert rel == "checkpoints/.iter_0000005.incomplete"
    _write(tmp_path / "a" / "run" / rel / "rank0.bin", os.urandom(1300))
    _write(tmp_path / "b" / "run" / rel / "rank1.bin", os.urandom(700))
    common = os.urandom(100)
    for n in ("a", "b"):
        _write(tmp_path / n / "run" / rel / "meta.json", common)
    out = tmp_path / "a" / "run"                                         # node a is the coordinator
    merged = nlf.collect_checkpoint(stores, ["a", "b"], out, completed_step=4)
    assert sorted(merged) == ["meta.json", "rank0.bin", "rank1.bin"]
    assert nlf.manifest(out / rel) == merged
    # a second node staging different bytes under an existing name is refused
    _write(tmp_path / "b" / "run" / rel / "rank0.bin", os.urandom(1300))
    with pytest.raises(ValueError):
        nlf.collect_checkpoint(stores, ["a", "b"], out, completed_step=4)
    os.rename(out / rel, out / "checkpoints" / "iter_0000005")            # publication on the coordinator
    nlf.clear_staging(stores, ["a", "b"], completed_step=4)
    assert not (tmp_path / "b" / "run" / rel).exists()
    with pytest.raises(ValueError):
        stores["b"].remove_staging("checkpoints/iter_0000005")            # only unpublished staging may be removed


def test_prepare_resume_and_switch(tmp_path):
    stores = _stores(tmp_path, ("a", "b"))
    ck = tmp_path / "old-run" / "checkpoints" / "iter_0000003"
    _write(ck / "model.bin", b"weights")
    path = nlf.prepare_resume(stores, ck, tmp_path / "a" / "run", coordinator="a")
    assert path.endswith("resume-input/iter_0000003") and os.path.exists(os.path.join(path, "model.bin"))
    assert stores["b"].inventory("resume-input/iter_0000003").keys() == {"model.bin"}
    assert nlf.enabled({"cluster_mode": "static_multi_node", "cluster_storage_mode": "node_local"})
    assert not nlf.enabled({"cluster_mode": "single_node"})
