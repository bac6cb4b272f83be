"""Import-only stand-in (see the package docstring)."""


class _Unavailable:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("ray is not installed; only the import is satisfied")


class Queue(_Unavailable):
    pass


class Empty(Exception):
    pass


class Full(Exception):
    pass


class PlacementGroup(_Unavailable):
    pass


class PlacementGroupSchedulingStrategy(_Unavailable):
    pass


class NodeAffinitySchedulingStrategy(_Unavailable):
    pass


def placement_group(*args, **kwargs):
    raise RuntimeError("ray is not installed; only the import is satisfied")


remove_placement_group = get_current_placement_group = placement_group_table = placement_group
