"""Deterministic role placement over an explicit cluster description."""
import pytest

from aspec_b200.placement import Node, cluster_from_args, create_placement, local_cluster

TWO_NODES = [Node.of("10.0.0.12", 8), Node.of("10.0.0.3", 8)]          # listed out of address order on purpose


def _args(**kw):
    base = dict(training_num_nodes=1, training_num_gpus_per_node=6, inference_num_gpus=2, placement_strategy="training_first")
    base.update(kw)
    return base


def test_packed_order_is_by_address_then_gpu_index_and_is_stable():
    p = create_placement(_args(training_num_gpus_per_node=8, inference_num_gpus=8), TWO_NODES)
    assert p.training == [("10.0.0.3", g) for g in range(8)]              # 10.0.0.3 sorts before 10.0.0.12 numerically
    assert p.inference == [("10.0.0.12", g) for g in range(8)]
    again = create_placement(_args(training_num_gpus_per_node=8, inference_num_gpus=8), list(reversed(TWO_NODES)))
    assert again.to_dict() == p.to_dict()


def test_training_first_and_inference_first_split_one_packed_list():
    one = local_cluster(8)
    t = create_placement(_args(), one)
    assert [g for _, g in t.training] == [0, 1, 2, 3, 4, 5] and [g for _, g in t.inference] == [6, 7]
    i = create_placement(_args(placement_strategy="inference_first"), one)
    assert [g for _, g in i.inference] == [0, 1] and [g for _, g in i.training] == [2, 3, 4, 5, 6, 7]
    assert i.devices_on("127.0.0.1", "inference") == ["cuda:0", "cuda:1"]
    with pytest.raises(ValueError):
        create_placement(_args(inference_num_gpus=3), one)                  # 6 + 3 > 8


def test_colocate_shares_the_gpus():
    p = create_placement(_args(training_num_gpus_per_node=4, colocate=True), local_cluster(4))
    assert p.training == p.inference and len(p.training) == 4


def test_custom_constraints_pin_roles_to_named_nodes():
    args = _args(placement_strategy="custom", training_num_nodes=1, training_num_gpus_per_node=8, inference_num_gpus=4,
                 training_nodes=["10.0.0.12"], inference_nodes="10.0.0.3")
    p = create_placement(args, TWO_NODES)
    assert p.nodes_of("training") == ["10.0.0.12"] and p.nodes_of("inference") == ["10.0.0.3"]
    assert [g for _, g in p.inference] == [0, 1, 2, 3]
    with pytest.raises(ValueError):                                          # a node for both roles without colocate
        create_placement(dict(args, inference_nodes=["10.0.0.12"]), TWO_NODES)
    with pytest.raises(ValueError):                                          # unknown node
        create_placement(dict(args, inference_nodes=["10.0.0.99"]), TWO_NODES)
    with pytest.raises(ValueError):                                          # constraints without the custom strategy
        create_placement(dict(args, placement_strategy="training_first"), TWO_NODES)
    with pytest.raises(ValueError):                                          # custom needs both roles
        create_placement(args, TWO_NODES, roles={"training"})


def test_single_role_and_cluster_description():
    p = create_placement(_args(), local_cluster(8), roles={"inference"})
    assert p.training == [] and [g for _, g in p.inference] == [0, 1]
    with pytest.raises(ValueError):
        create_placement(_args(inference_num_gpus=0), local_cluster(8), roles={"inference"})
    nodes = cluster_from_args({"cluster_nodes": [{"name": "a", "gpus": [1, 3]}, {"name": "b", "gpus": 2}]}, visible_gpus=8)
    assert [n.gpus for n in nodes] == [(1, 3), (0, 1)]
    assert cluster_from_args({}, visible_gpus=4)[0].gpus == (0, 1, 2, 3)
