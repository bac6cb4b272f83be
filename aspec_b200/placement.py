"""Deterministic placement of Target (inference) and Draft (training) roles on the GPUs of a cluster.

The reference asks Ray for placement groups (PACK, or per-role node constraints) and then sorts the bundles it got by
node address and GPU index, so that the role of every GPU is the same on every restart
(aspec/ray/placement_group.py:235-330, 544-640).  Here the cluster is described explicitly - a list of nodes with the
GPU indices they offer - and the same policies are a pure function of that description:

* ``training_first`` / ``inference_first``: one packed list of all GPUs (nodes in address order, GPUs in index order);
  the first role takes the head of the list, the other the tail;
* ``colocate``: both roles share the same GPUs;
* ``custom``: every role names the nodes it may use (``training_nodes`` / ``inference_nodes``), each packed in order;
  a node may not serve both roles unless ``colocate`` is set.

A single role can be placed alone (``roles={"training"}``), but custom constraints need both, as in the reference.
The result is what the launcher needs: per role the ordered ``(node, gpu)`` pairs, plus this node's device strings.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Sequence, Set, Tuple


@dataclass(frozen=True)
class Node:
    name: str                      # address or host name; the sort key of the packed order
    gpus: Tuple[int, ...]

    @classmethod
    def of(cls, name: str, gpus) -> "Node":
        ids = tuple(range(gpus)) if isinstance(gpus, int) else tuple(int(g) for g in gpus)
        if len(set(ids)) != len(ids) or any(g < 0 for g in ids):
            raise ValueError(f"node {name}: GPU indices must be distinct and non-negative")
        return cls(str(name), tuple(sorted(ids)))


@dataclass
class Placement:
    training: List[Tuple[str, int]] = field(default_factory=list)
    inference: List[Tuple[str, int]] = field(default_factory=list)
    strategy: str = "training_first"

    def devices_on(self, node: str, role: str) -> List[str]:
        return [f"cuda:{g}" for n, g in getattr(self, role) if n == node]

    def nodes_of(self, role: str) -> List[str]:
        seen: List[str] = []
        for n, _ in getattr(self, role):
            if n not in seen:
                seen.append(n)
        return seen

    def to_dict(self) -> dict:
        return {"strategy": self.strategy, "training": [list(p) for p in self.training],
                "inference": [list(p) for p in self.inference]}


def _node_key(name: str):
    """Addresses sort numerically by octet, other names lexicographically after them."""
    parts = name.split(".")
    if len(parts) == 4 and all(p.isdigit() for p in parts):
        return (0, tuple(int(p) for p in parts), "")
    return (1, (), name)


def _packed(nodes: Iterable[Node]) -> List[Tuple[str, int]]:
    return [(n.name, g) for n in sorted(nodes, key=lambda n: _node_key(n.name)) for g in n.gpus]


def _as_list(value, what: str) -> List[str]:
    if value is None:
        return []
    if isinstance(value, str):
        return [v.strip() for v in value.split(",") if v.strip()]
    if isinstance(value, (list, tuple)):
        return [str(v) for v in value]
    raise ValueError(f"{what} must be a list of node names or a comma-separated string")


def _get(args, key: str, default=None):
    return args.get(key, default) if isinstance(args, dict) else getattr(args, key, default)


def _role_nodes(args, role: str) -> List[str]:
    """``training_nodes`` / ``inference_nodes``, or the reference's spelling ``training_node_ips`` / ``inference_node_ips``."""
    return _as_list(_get(args, f"{role}_nodes") or _get(args, f"{role}_node_ips"), f"{role}_nodes")


def has_custom_fields(args) -> bool:
    return bool(_role_nodes(args, "training") or _role_nodes(args, "inference"))


def create_placement(args, nodes: Sequence[Node], roles: Optional[Set[str]] = None) -> Placement:
    """``args``: mapping or namespace with ``training_num_nodes``, ``training_num_gpus_per_node``, ``inference_num_gpus``,
    ``placement_strategy`` (``training_first`` | ``inference_first`` | ``custom``), ``colocate`` and, for ``custom``,
    ``training_nodes`` / ``inference_nodes``."""
    roles = {"training", "inference"} if roles is None else set(roles)
    if not roles or roles - {"training", "inference"}:
        raise ValueError(f"Invalid placement roles: {sorted(roles)}")
    names = [n.name for n in nodes]
    if len(set(names)) != len(names):
        raise ValueError("node names must be distinct")
    strategy = _get(args, "placement_strategy", "training_first") or "training_first"
    if strategy not in ("training_first", "inference_first", "custom"):
        raise ValueError(f"unknown placement_strategy {strategy!r}")
    n_train = int(_get(args, "training_num_nodes", 1) or 0) * int(_get(args, "training_num_gpus_per_node", 0) or 0)
    n_inf = int(_get(args, "inference_num_gpus", 0) or 0)
    colocate = bool(_get(args, "colocate", False))
    if strategy != "custom" and has_custom_fields(args):
        raise ValueError("training_nodes / inference_nodes are only honoured with placement_strategy=custom")

    if len(roles) == 1:
        if strategy == "custom":
            raise ValueError("Custom placement is only supported when training and inference roles are created together")
        role = next(iter(roles))
        count = n_train if role == "training" else n_inf
        if count <= 0:
            raise ValueError(f"{role.capitalize()} placement requires a positive GPU count")
        packed = _packed(nodes)
        if count > len(packed):
            raise ValueError(f"{role} needs {count} GPUs, the cluster offers {len(packed)}")
        out = Placement(strategy=strategy)
        setattr(out, role, packed[:count])
        return out

    if n_train <= 0:
        raise ValueError("Training placement requires a positive GPU count")
    if colocate:
        pool = _packed(_select(nodes, _role_nodes(args, "training"))) if strategy == "custom" else _packed(nodes)
        if n_train > len(pool):
            raise ValueError(f"colocated roles need {n_train} GPUs, {len(pool)} offered")
        return Placement(training=pool[:n_train], inference=pool[:n_train], strategy=strategy)

    if strategy == "custom":
        t_names, i_names = _role_nodes(args, "training"), _role_nodes(args, "inference")
        if not t_names or (n_inf > 0 and not i_names):
            raise ValueError("custom placement needs training_nodes and inference_nodes")
        both = set(t_names) & set(i_names)
        if both:
            raise ValueError(f"nodes {sorted(both)} are named for both roles; set colocate to share GPUs")
        t_pool, i_pool = _packed(_select(nodes, t_names)), _packed(_select(nodes, i_names))
        if n_train > len(t_pool) or n_inf > len(i_pool):
            raise ValueError(f"custom placement: training needs {n_train} of {len(t_pool)} GPUs, inference {n_inf} of {len(i_pool)}")
        return Placement(training=t_pool[:n_train], inference=i_pool[:n_inf], strategy=strategy)

    packed = _packed(nodes)
    if n_train + n_inf > len(packed):
        raise ValueError(f"plan needs {n_inf} Target + {n_train} Draft GPUs, the cluster offers {len(packed)}")
    if strategy == "training_first":
        return Placement(training=packed[:n_train], inference=packed[n_train:n_train + n_inf], strategy=strategy)
    return Placement(inference=packed[:n_inf], training=packed[n_inf:n_inf + n_train], strategy=strategy)


def _select(nodes: Sequence[Node], names: Sequence[str]) -> List[Node]:
    by_name = {n.name: n for n in nodes}
    missing = [n for n in names if n not in by_name]
    if missing:
        raise ValueError(f"placement names unknown nodes: {missing}")
    return [by_name[n] for n in names]


def local_cluster(gpu_count: int, name: str = "127.0.0.1") -> List[Node]:
    return [Node.of(name, gpu_count)]


def cluster_from_args(args, visible_gpus: int) -> List[Node]:
    """``cluster_nodes: [{name, gpus}]`` when the recipe lists them, else this machine with its visible GPUs."""
    spec = _get(args, "cluster_nodes")
    if spec:
        return [Node.of(s["name"], s["gpus"]) for s in spec]
    return local_cluster(visible_gpus)
