"""Checkpoint exchange between nodes whose run directories are NOT on a shared filesystem.

With node-local storage every trainer writes its checkpoint shards under its own node's copy of the run directory.
Before a checkpoint is published the coordinator pulls every training node's staged shards into its own staging
directory, and before a resume it pushes the checkpoint to every node.  Transfers are chunked (bounded memory),
every file is verified against its SHA-256 before it becomes visible under its final name, symlinks and paths that
leave the store are refused, and two nodes that stage different bytes under one name are a hard error.

The reference does this with one Ray actor per node (aspec/ray/node_local_files.py:60-245).  Here a node's files
are served by a ``NodeStore``; ``stores`` maps node names to objects with the same methods - in-process stores for a
single machine and for tests, proxies of ``runtime.actor.ProcessActor`` (``ActorStore``) when a store runs in
another process.  A network transport between machines is not part of this single-node runtime.
"""
from __future__ import annotations

import hashlib
import os
import shutil
from pathlib import Path
from typing import Dict, Iterable, Mapping

CHUNK_BYTES = 8 * 1024 * 1024


def file_digest(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            block = f.read(CHUNK_BYTES)
            if not block:
                break
            h.update(block)
    return h.hexdigest()


def manifest(root) -> Dict[str, dict]:
    """``{relative posix path: {"size", "sha256"}}`` of every regular file under ``root``; symlinks are refused."""
    root = Path(root)
    if not root.is_dir():
        raise FileNotFoundError(str(root))
    out: Dict[str, dict] = {}
    for p in sorted(root.rglob("*")):
        if p.is_symlink():
            raise ValueError(f"checkpoint exchange refuses symlinks: {p}")
        if p.is_file():
            out[p.relative_to(root).as_posix()] = {"size": p.stat().st_size, "sha256": file_digest(p)}
    return out


class NodeStore:
    """The run directory of one node.  All paths are relative to it and may not leave it."""

    PARTIAL = ".exchange-partial"

    def __init__(self, root, run_id: str = ""):
        self.root = Path(root)
        self.run_id = str(run_id)
        self.root.mkdir(parents=True, exist_ok=True)

    def _path(self, relative: str) -> Path:
        p = (self.root / relative).resolve()
        base = self.root.resolve()
        if base != p and base not in p.parents:
            raise ValueError(f"path leaves the node store: {relative}")
        return p

    def append(self, relative: str, offset: int, data: bytes) -> int:
        """Write ``data`` at ``offset`` of the file's partial copy; offsets must arrive in order."""
        target = self._path(relative)
        part = target.with_name(target.name + self.PARTIAL)
        part.parent.mkdir(parents=True, exist_ok=True)
        have = part.stat().st_size if part.exists() else 0
        if offset == 0 and have:
            part.unlink()
            have = 0
        if offset != have:
            raise ValueError(f"out-of-order chunk for {relative}: offset {offset}, have {have}")
        with open(part, "ab") as f:
            f.write(data)
        return have + len(data)

    def publish(self, relative: str, info: Mapping) -> None:
        """Verify the partial copy against ``info`` and move it to its final name (atomic rename)."""
        target = self._path(relative)
        part = target.with_name(target.name + self.PARTIAL)
        if not part.exists():
            if info["size"] == 0:
                part.parent.mkdir(parents=True, exist_ok=True)
                part.touch()
            else:
                raise FileNotFoundError(f"nothing was sent for {relative}")
        if part.stat().st_size != info["size"] or file_digest(part) != info["sha256"]:
            part.unlink()
            raise ValueError(f"checksum mismatch for {relative}")
        if target.exists() and file_digest(target) != info["sha256"]:
            raise ValueError(f"{relative} already exists on this node with different bytes")
        os.replace(part, target)

    def inventory(self, relative: str = ".") -> Dict[str, dict]:
        root = self._path(relative)
        return manifest(root) if root.is_dir() else {}

    def read(self, relative: str, offset: int, size: int = CHUNK_BYTES) -> bytes:
        with open(self._path(relative), "rb") as f:
            f.seek(offset)
            return f.read(size)

    def remove_staging(self, relative: str) -> None:
        p = self._path(relative)
        if not p.name.startswith(".") or not p.name.endswith(".incomplete"):
            raise ValueError("only unpublished staging directories may be removed")
        if not p.exists():
            raise FileNotFoundError(str(p))
        shutil.rmtree(p)


class ActorStore:
    """A ``NodeStore`` that lives in another process behind a ``runtime.actor.ProcessActor``."""

    def __init__(self, actor, timeout: float = 600.0):
        self._actor, self._timeout = actor, timeout

    def __getattr__(self, name):
        return lambda *a, **k: self._actor.call(name, *a, timeout=self._timeout, **k)


def enabled(args) -> bool:
    get = args.get if isinstance(args, dict) else lambda k, d=None: getattr(args, k, d)
    return get("cluster_mode", "single_node") == "static_multi_node" and get("cluster_storage_mode", "shared") == "node_local"


def staging_dir(completed_step: int) -> str:
    return f"checkpoints/.iter_{completed_step + 1:07d}.incomplete"


def send_tree(stores: Mapping[str, NodeStore], source, relative: str, skip: Iterable[str] = ()) -> int:
    """Push every file under ``source`` to ``relative/`` on every node (except ``skip``).  Returns bytes sent."""
    files = manifest(source)
    sent = 0
    for node, store in stores.items():
        if node in set(skip):
            continue
        for name, info in files.items():
            dest = f"{relative}/{name}"
            with open(Path(source) / name, "rb") as f:
                offset = 0
                while True:
                    block = f.read(CHUNK_BYTES)
                    if not block:
                        break
                    store.append(dest, offset, block)
                    offset += len(block)
                    sent += len(block)
            store.publish(dest, info)
    return sent


def collect_checkpoint(stores: Mapping[str, NodeStore], training_nodes: Iterable[str], output_dir, completed_step: int) -> Dict[str, dict]:
    """Pull the shards every training node staged for the checkpoint after ``completed_step`` into the coordinator's
    staging directory.  Returns the merged manifest.  The same name with different bytes on two nodes is an error."""
    relative = staging_dir(completed_step)
    destination = Path(output_dir) / relative
    destination.mkdir(parents=True, exist_ok=True)
    merged: Dict[str, dict] = {}
    for node in training_nodes:
        store = stores[node]
        for name, info in store.inventory(relative).items():
            target = destination / name
            if target.exists():
                if target.stat().st_size != info["size"] or file_digest(target) != info["sha256"]:
                    raise ValueError(f"conflicting checkpoint shard {name} from node {node}")
                merged[name] = info
                continue
            target.parent.mkdir(parents=True, exist_ok=True)
            partial = target.with_name(target.name + ".collect-partial")
            with open(partial, "wb") as out:
                for offset in range(0, info["size"], CHUNK_BYTES):
                    block = store.read(f"{relative}/{name}", offset, CHUNK_BYTES)
                    if len(block) != min(CHUNK_BYTES, info["size"] - offset):
                        partial.unlink(missing_ok=True)
                        raise ValueError(f"truncated transfer of {name} from node {node}")
                    out.write(block)
            if file_digest(partial) != info["sha256"]:
                partial.unlink(missing_ok=True)
                raise ValueError(f"checksum mismatch collecting {name} from node {node}")
            os.replace(partial, target)
            merged[name] = info
    return merged


def clear_staging(stores: Mapping[str, NodeStore], training_nodes: Iterable[str], completed_step: int) -> None:
    """After publication: the coordinator's staging was renamed into place; every other node's copy is disposable."""
    relative = staging_dir(completed_step)
    for node in training_nodes:
        try:
            stores[node].remove_staging(relative)
        except FileNotFoundError:
            pass


def prepare_resume(stores: Mapping[str, NodeStore], checkpoint_dir, output_dir, coordinator: str) -> str:
    """Copy ``checkpoint_dir`` under ``output_dir/resume-input/`` and push it to every other node; returns the new
    load path (the same relative location on every node)."""
    source = Path(checkpoint_dir)
    relative = f"resume-input/{source.name}"
    local = Path(output_dir) / relative
    if not local.exists():
        shutil.copytree(source, local)
    send_tree(stores, source, relative, skip=[coordinator])
    return str(local)
