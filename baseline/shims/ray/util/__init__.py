"""See the package docstring: import-only stand-ins."""


def _unavailable(*args, **kwargs):
    raise RuntimeError("ray is not installed; only the import is satisfied")


get_node_ip_address = _unavailable


class _Namespace:
    def __getattr__(self, name):
        return _unavailable
